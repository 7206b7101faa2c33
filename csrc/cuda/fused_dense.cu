// Fused CaSync kernels for the dense (quantising) algorithms: onebit, TBQ and
// TernGrad.  One persistent launch synchronises a whole bucket of tensors:
//
//   ring : N hops of  wait -> decode incoming partial sum -> merge with the local
//          chunk and its residual -> re-encode -> store the payload straight into
//          the successor GPU's inbox over NVLink -> release a flag; the last hop
//          stores the fully reduced payload into every rank's inbox, and every
//          rank decodes all N chunks into the gradient (averaged).
//   PS   : encode each of the N chunks and store chunk j into owner j's inbox;
//          the owner decodes and sums the N payloads in rank order, re-encodes
//          with its server residual and stores the result into every inbox;
//          every rank decodes all N chunks.
//
// There is no NCCL call and no separate encode or decode launch.  Payload and
// flag traffic is plain st.global / st.release.sys to peer-mapped memory; the
// receiver always reads its own memory.  CTA b of one rank only ever waits for
// CTA b of other ranks, so no CTA waits on another CTA of its own GPU.  Every
// wait is bounded: on expiry the CTA records a status word, stops waiting and
// still runs to completion inside its own buffers.
//
// Reference parity: CaSync-Ring and CaSync-PS of mark14wu/hipress are selected
// with --topo Ring|PS (README.md:45,51); their cost shape (N encodes, N decodes,
// 2(N-1) sends for ring; gather + broadcast for PS) is in
// src/SeCoPa/SeCoPa.py:75-103.  The runtime source itself is not published.
#include <cuda_runtime.h>

#include "dense_tile.cuh"
#include "hipress/capi.h"
#include "sync.cuh"

namespace hipress {

struct SegDev {
  const float* g;
  float* r;
  float* out;
  float* sr;
  uint32_t n;
  uint32_t chunk;        // elements per chunk, multiple of kTile
  uint32_t tiles;        // tiles per chunk
  uint32_t tile_prefix;  // tiles of the segments before this one
  uint32_t pay_off;      // byte offset of this segment's chunk payload inside a slot
  uint32_t id;
};

struct BucketDev {
  SegDev seg[HP_MAX_SEGS];
  int nseg;
  uint32_t tiles_total;  // tiles of one chunk summed over segments
  uint64_t slot_bytes;
};

struct FusedParams {
  DenseParams P;
  float inv_n;
};

__device__ __forceinline__ int find_seg(const BucketDev& bk, uint32_t tt) {
  int i = bk.nseg - 1;
  while (i > 0 && tt < bk.seg[i].tile_prefix) --i;
  return i;
}

// decode tile t of the payload at `base` and add it to x (or assign when !add)
template <int ALG, int B>
__device__ __forceinline__ void decode_into(const uint8_t* base, uint32_t chunk, uint32_t t, int m,
                                            float tau, bool add, float (&x)[kIter][4]) {
  PayloadView v = payload_view(const_cast<uint8_t*>(base), ALG, chunk);
  float meta[2];
  load_meta<ALG>(v.meta, t, meta);
  const uint8_t* tc = v.codes + (size_t)t * (kTile * B / 8);
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    float d[4];
    decode_frag<ALG, B>(load_frag<B>(tc, j, m), meta, tau, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) x[j][e] = add ? x[j][e] + d[e] : d[e];
  }
}

// store staged codes + metadata (+ header for tile 0) of tile t into a payload
template <int ALG, int B>
__device__ __forceinline__ void store_payload_tile(uint8_t* base, uint32_t chunk, uint32_t t, int m,
                                                   uint32_t n_valid, const float (&meta)[2],
                                                   float tau, const TileSmem& s) {
  PayloadView v = payload_view(base, ALG, chunk);
  copy_codes(v.codes + (size_t)t * (kTile * B / 8), s.codes, tile_code_bytes(m, B));
  if (threadIdx.x == 0) {
    if (ALG == kOnebit) v.meta[t] = meta[0];
    if (ALG == kTernGrad) {
      v.meta[2 * t] = meta[0];
      v.meta[2 * t + 1] = meta[1];
    }
    if (t == 0) write_header(base, n_valid, ALG, B, tau);
  }
}

__device__ __forceinline__ uint32_t chunk_valid(uint32_t n, uint32_t chunk, int c) {
  const uint64_t start = (uint64_t)c * chunk;
  if (start >= n) return 0;
  const uint64_t rest = n - start;
  return (uint32_t)(rest < chunk ? rest : chunk);
}

// ------------------------------------------------------------------------ ring
template <int ALG, int B>
__global__ void __launch_bounds__(kThreads)
ring_dense_kernel(const BucketDev bk, const HpComm cm, const FusedParams fp) {
  __shared__ TileSmem s;
  __shared__ WaitState ws;
  const int N = cm.nranks;
  const int R = cm.emulate ? (int)blockIdx.y : cm.rank;
  const int E = cm.emulate ? (int)blockIdx.y : 0;
  const int G = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  uint8_t* my_inbox = reinterpret_cast<uint8_t*>(cm.inbox[R]);
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(cm.flags[R]);
  wait_init(ws);

  for (int hop = 0; hop < N; ++hop) {
    const int c = (R - hop + N) % N;
    const bool last = hop == N - 1;
    if (hop > 0)
      wait_flag(my_flags + (size_t)(hop - 1) * G + b, cm.epoch, cm.timeout_ns, status,
                HP_STATUS_TIMEOUT | (1u << 16) | ((uint32_t)(hop - 1) << 8) | (b & 255), ws);
    const uint8_t* in_slot = my_inbox + (size_t)(hop > 0 ? hop - 1 : 0) * bk.slot_bytes;
    const int succ = (R + 1) % N;
    for (uint32_t tt = b; tt < bk.tiles_total; tt += G) {
      const SegDev& sg = bk.seg[find_seg(bk, tt)];
      const uint32_t t = tt - sg.tile_prefix;
      const uint32_t nv = chunk_valid(sg.n, sg.chunk, c);
      const int64_t left = (int64_t)nv - (int64_t)t * kTile;
      if (left <= 0) continue;
      const int m = (int)(left < kTile ? left : kTile);
      const size_t off = (size_t)c * sg.chunk + (size_t)t * kTile;
      float x[kIter][4];
      load_tile(sg.g + E * cm.emu_stride_g + off, m, x);
      if (hop > 0) decode_into<ALG, B>(in_slot + sg.pay_off, sg.chunk, t, m, fp.P.tau, true, x);
      float* rp = sg.r ? sg.r + E * cm.emu_stride_r + off : nullptr;
      if (rp) {
        float rr[kIter][4];
        load_tile(rp, m, rr);
#pragma unroll
        for (int j = 0; j < kIter; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[j][e] = rr[j][e] + x[j][e];
      }
      float meta[2];
      uint32_t frag[kIter];
      encode_tile<ALG, B>(x, m, fp.P, sg.id, off, fp.P.salt + (uint32_t)(R * 256 + hop), s, meta,
                          frag);
      if (rp) store_tile(rp, m, x);
      stage_frags<B>(s.codes, frag);
      __syncthreads();
      if (!last) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[succ]) + (size_t)hop * bk.slot_bytes +
                       sg.pay_off;
        store_payload_tile<ALG, B>(dst, sg.chunk, t, m, nv, meta, fp.P.tau, s);
      } else {
        for (int q = 0; q < N; ++q) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) +
                         (size_t)(N - 1 + R) * bk.slot_bytes + sg.pay_off;
          store_payload_tile<ALG, B>(dst, sg.chunk, t, m, nv, meta, fp.P.tau, s);
        }
      }
      __syncthreads();
    }
    // publish: everything this CTA stored for this hop is complete
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      if (!last) {
        st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[succ]) + (size_t)hop * G + b, cm.epoch);
      } else {
        for (int q = 0; q < N; ++q)
          st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) +
                             (size_t)(N - 1 + R) * G + b,
                         cm.epoch);
      }
    }
  }

  // gather: decode the N reduced chunks (rank src finalised chunk src+1)
  for (int qq = 0; qq < N; ++qq) {
    const int src = (R + qq) % N;
    const int c = (src + 1) % N;
    wait_flag(my_flags + (size_t)(N - 1 + src) * G + b, cm.epoch, cm.timeout_ns, status,
              HP_STATUS_TIMEOUT | (2u << 16) | ((uint32_t)src << 8) | (b & 255), ws);
    const uint8_t* slot = my_inbox + (size_t)(N - 1 + src) * bk.slot_bytes;
    for (uint32_t tt = b; tt < bk.tiles_total; tt += G) {
      const SegDev& sg = bk.seg[find_seg(bk, tt)];
      const uint32_t t = tt - sg.tile_prefix;
      const uint32_t nv = chunk_valid(sg.n, sg.chunk, c);
      const int64_t left = (int64_t)nv - (int64_t)t * kTile;
      if (left <= 0) continue;
      const int m = (int)(left < kTile ? left : kTile);
      const size_t off = (size_t)c * sg.chunk + (size_t)t * kTile;
      float x[kIter][4];
      decode_into<ALG, B>(slot + sg.pay_off, sg.chunk, t, m, fp.P.tau, false, x);
#pragma unroll
      for (int j = 0; j < kIter; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) x[j][e] = x[j][e] * fp.inv_n;
      store_tile(sg.out + E * cm.emu_stride_out + off, m, x);
    }
  }
}

// -------------------------------------------------------------------------- PS
template <int ALG, int B>
__global__ void __launch_bounds__(kThreads)
ps_dense_kernel(const BucketDev bk, const HpComm cm, const FusedParams fp) {
  __shared__ TileSmem s;
  __shared__ WaitState ws;
  const int N = cm.nranks;
  const int R = cm.emulate ? (int)blockIdx.y : cm.rank;
  const int E = cm.emulate ? (int)blockIdx.y : 0;
  const int G = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  uint8_t* my_inbox = reinterpret_cast<uint8_t*>(cm.inbox[R]);
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(cm.flags[R]);
  wait_init(ws);

  // phase 1: push.  Remote owners first, own chunk last.
  for (int i = 0; i < N; ++i) {
    const int j = (R + 1 + i) % N;
    uint8_t* dslot = reinterpret_cast<uint8_t*>(cm.inbox[j]) + (size_t)R * bk.slot_bytes;
    for (uint32_t tt = b; tt < bk.tiles_total; tt += G) {
      const SegDev& sg = bk.seg[find_seg(bk, tt)];
      const uint32_t t = tt - sg.tile_prefix;
      const uint32_t nv = chunk_valid(sg.n, sg.chunk, j);
      const int64_t left = (int64_t)nv - (int64_t)t * kTile;
      if (left <= 0) continue;
      const int m = (int)(left < kTile ? left : kTile);
      const size_t off = (size_t)j * sg.chunk + (size_t)t * kTile;
      float x[kIter][4];
      load_tile(sg.g + E * cm.emu_stride_g + off, m, x);
      float* rp = sg.r ? sg.r + E * cm.emu_stride_r + off : nullptr;
      if (rp) {
        float rr[kIter][4];
        load_tile(rp, m, rr);
#pragma unroll
        for (int jj = 0; jj < kIter; ++jj)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[jj][e] = rr[jj][e] + x[jj][e];
      }
      float meta[2];
      uint32_t frag[kIter];
      encode_tile<ALG, B>(x, m, fp.P, sg.id, off, fp.P.salt + (uint32_t)(R * 256), s, meta, frag);
      if (rp) store_tile(rp, m, x);
      stage_frags<B>(s.codes, frag);
      __syncthreads();
      store_payload_tile<ALG, B>(dslot + sg.pay_off, sg.chunk, t, m, nv, meta, fp.P.tau, s);
      __syncthreads();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[j]) + (size_t)R * G + b, cm.epoch);
    }
  }

  // phase 2: server for chunk R: sum the N payloads in rank order, re-encode, broadcast
  for (int q = 0; q < N; ++q)
    wait_flag(my_flags + (size_t)q * G + b, cm.epoch, cm.timeout_ns, status,
              HP_STATUS_TIMEOUT | (1u << 16) | ((uint32_t)q << 8) | (b & 255), ws);
  for (uint32_t tt = b; tt < bk.tiles_total; tt += G) {
    const SegDev& sg = bk.seg[find_seg(bk, tt)];
    const uint32_t t = tt - sg.tile_prefix;
    const uint32_t nv = chunk_valid(sg.n, sg.chunk, R);
    const int64_t left = (int64_t)nv - (int64_t)t * kTile;
    if (left <= 0) continue;
    const int m = (int)(left < kTile ? left : kTile);
    const size_t coff = (size_t)t * kTile;  // offset inside the owned chunk
    float x[kIter][4];
    for (int q = 0; q < N; ++q)
      decode_into<ALG, B>(my_inbox + (size_t)q * bk.slot_bytes + sg.pay_off, sg.chunk, t, m,
                          fp.P.tau, q > 0, x);
    float* rp = sg.sr ? sg.sr + E * cm.emu_stride_sr + coff : nullptr;
    if (rp) {
      float rr[kIter][4];
      load_tile(rp, m, rr);
#pragma unroll
      for (int jj = 0; jj < kIter; ++jj)
#pragma unroll
        for (int e = 0; e < 4; ++e) x[jj][e] = rr[jj][e] + x[jj][e];
    }
    float meta[2];
    uint32_t frag[kIter];
    encode_tile<ALG, B>(x, m, fp.P, sg.id, (size_t)R * sg.chunk + coff,
                        fp.P.salt + (uint32_t)(R * 256 + 1), s, meta, frag);
    if (rp) store_tile(rp, m, x);
    stage_frags<B>(s.codes, frag);
    __syncthreads();
    for (int q = 0; q < N; ++q) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) +
                     (size_t)(N + R) * bk.slot_bytes + sg.pay_off;
      store_payload_tile<ALG, B>(dst, sg.chunk, t, m, nv, meta, fp.P.tau, s);
    }
    __syncthreads();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int q = 0; q < N; ++q)
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) + (size_t)(N + R) * G + b,
                     cm.epoch);
  }

  // phase 3: pull: decode every owner's reduced chunk
  for (int i = 0; i < N; ++i) {
    const int j = (R + i) % N;
    wait_flag(my_flags + (size_t)(N + j) * G + b, cm.epoch, cm.timeout_ns, status,
              HP_STATUS_TIMEOUT | (2u << 16) | ((uint32_t)j << 8) | (b & 255), ws);
    const uint8_t* slot = my_inbox + (size_t)(N + j) * bk.slot_bytes;
    for (uint32_t tt = b; tt < bk.tiles_total; tt += G) {
      const SegDev& sg = bk.seg[find_seg(bk, tt)];
      const uint32_t t = tt - sg.tile_prefix;
      const uint32_t nv = chunk_valid(sg.n, sg.chunk, j);
      const int64_t left = (int64_t)nv - (int64_t)t * kTile;
      if (left <= 0) continue;
      const int m = (int)(left < kTile ? left : kTile);
      const size_t off = (size_t)j * sg.chunk + (size_t)t * kTile;
      float x[kIter][4];
      decode_into<ALG, B>(slot + sg.pay_off, sg.chunk, t, m, fp.P.tau, false, x);
#pragma unroll
      for (int jj = 0; jj < kIter; ++jj)
#pragma unroll
        for (int e = 0; e < 4; ++e) x[jj][e] = x[jj][e] * fp.inv_n;
      store_tile(sg.out + E * cm.emu_stride_out + off, m, x);
    }
  }
}

// ------------------------------------------------------------------ host side
static int build_bucket(int alg, int bits, const HpSeg* segs, int nseg, int nranks,
                        BucketDev& bk) {
  if (nseg < 1 || nseg > HP_MAX_SEGS || nranks < 1 || nranks > HP_MAX_RANKS) return HP_ERR_BAD_ARG;
  uint64_t pay = 0, tiles = 0;
  for (int i = 0; i < nseg; ++i) {
    const uint64_t n = segs[i].n;
    if (n == 0 || n > 0xFFFFF000ull) return HP_ERR_BAD_ARG;
    const uint64_t per = (n + nranks - 1) / nranks;
    const uint64_t chunk = align_up(per, kTile);
    SegDev& d = bk.seg[i];
    d.g = static_cast<const float*>(segs[i].g);
    d.r = static_cast<float*>(segs[i].r);
    d.out = static_cast<float*>(segs[i].out);
    d.sr = static_cast<float*>(segs[i].sr);
    d.n = (uint32_t)n;
    d.chunk = (uint32_t)chunk;
    d.tiles = (uint32_t)(chunk / kTile);
    d.tile_prefix = (uint32_t)tiles;
    d.pay_off = (uint32_t)pay;
    d.id = segs[i].id;
    tiles += d.tiles;
    pay += align_up(dense_payload_bytes(alg, bits, chunk), 128);
    if (pay > 0xFFFFFFFFull || tiles > 0x7FFFFFFFull) return HP_ERR_TOO_LARGE;
  }
  bk.nseg = nseg;
  bk.tiles_total = (uint32_t)tiles;
  bk.slot_bytes = pay;
  return 0;
}

static int num_slots(int topo, int nranks) {
  return topo == HP_TOPO_RING ? 2 * nranks - 1 : 2 * nranks;
}

template <int ALG, int B>
static int launch_fused(int topo, const BucketDev& bk, const HpComm& cm, const FusedParams& fp,
                        int ctas, cudaStream_t st) {
  void (*kern)(const BucketDev, const HpComm, const FusedParams) =
      topo == HP_TOPO_RING ? ring_dense_kernel<ALG, B> : ps_dense_kernel<ALG, B>;
  if (cm.emulate) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, 0);
    if (e != cudaSuccess) return (int)e;
    if ((long long)ctas * cm.nranks > (long long)per_sm * sms) return HP_ERR_RESIDENCY;
    void* args[] = {(void*)&bk, (void*)&cm, (void*)&fp};
    e = cudaLaunchCooperativeKernel((const void*)kern, dim3(ctas, cm.nranks), dim3(kThreads),
                                    args, 0, st);
    return (int)e;
  }
  kern<<<dim3(ctas, 1), kThreads, 0, st>>>(bk, cm, fp);
  return (int)cudaGetLastError();
}

}  // namespace hipress

using namespace hipress;

extern "C" {

// bytes of one rank's inbox for a bucket of tensors with the given sizes
int hp_fused_dense_layout(int topo, int alg, int bits, const uint64_t* ns, int nseg, int nranks,
                          uint64_t* inbox_bytes, uint64_t* slot_bytes, uint32_t* tiles_total) {
  if (nseg < 1 || nseg > HP_MAX_SEGS) return HP_ERR_BAD_ARG;
  HpSeg segs[HP_MAX_SEGS] = {};
  for (int i = 0; i < nseg; ++i) segs[i].n = ns[i];
  BucketDev bk;
  int rc = build_bucket(alg, bits, segs, nseg, nranks, bk);
  if (rc) return rc;
  if (inbox_bytes) *inbox_bytes = bk.slot_bytes * (uint64_t)num_slots(topo, nranks);
  if (slot_bytes) *slot_bytes = bk.slot_bytes;
  if (tiles_total) *tiles_total = bk.tiles_total;
  return 0;
}

// uint32 flag words one rank needs for `ctas` CTAs
uint64_t hp_fused_flag_words(int topo, int nranks, int ctas) {
  return (uint64_t)num_slots(topo, nranks) * (uint64_t)ctas;
}

// elements of the server residual a PS owner keeps for a tensor of n elements
uint64_t hp_fused_chunk_elems(uint64_t n, int nranks) {
  return align_up((n + nranks - 1) / nranks, kTile);
}

int hp_cuda_fused_dense(int topo, int alg, int bits, const HpSeg* segs, int nseg,
                        const HpComm* comm, float tau, uint64_t seed, uint32_t step, uint32_t salt,
                        int ctas, void* stream) {
  if (topo != HP_TOPO_RING && topo != HP_TOPO_PS) return HP_ERR_BAD_ARG;
  if (!comm || ctas < 1 || ctas > 65535) return HP_ERR_BAD_ARG;
  BucketDev bk;
  int rc = build_bucket(alg, bits, segs, nseg, comm->nranks, bk);
  if (rc) return rc;
  if ((uint32_t)ctas > bk.tiles_total) ctas = (int)bk.tiles_total;
  FusedParams fp;
  fp.P = DenseParams{tau, step, salt, (uint32_t)seed, (uint32_t)(seed >> 32)};
  fp.inv_n = 1.0f / (float)comm->nranks;
  cudaStream_t st = (cudaStream_t)stream;
#define CALL(A, B) return launch_fused<A, B>(topo, bk, *comm, fp, ctas, st)
  if (alg == kOnebit && bits == 1) { CALL(kOnebit, 1); }
  else if (alg == kTbq && bits == 2) { CALL(kTbq, 2); }
  else if (alg == kTernGrad && bits == 1) { CALL(kTernGrad, 1); }
  else if (alg == kTernGrad && bits == 2) { CALL(kTernGrad, 2); }
  else if (alg == kTernGrad && bits == 4) { CALL(kTernGrad, 4); }
  else if (alg == kTernGrad && bits == 8) { CALL(kTernGrad, 8); }
#undef CALL
  return HP_ERR_BAD_ARG;
}

}  // extern "C"
