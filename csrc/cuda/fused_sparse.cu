// Fused CaSync-PS for the top-k algorithms (DGC, GradDrop): a short, fixed
// sequence of launches per bucket with no NCCL call and no host round trip.
//
//   push   : per (tensor, owner) unit: state update + radix select (3 histogram
//            passes) + compaction whose (index, value) pairs are stored straight
//            into the owner GPU's inbox; the CTA that finishes a unit releases
//            the owner's flag.
//   server : the owner waits (bounded) for the N flags of a tensor, adds the N
//            sparse payloads into its accumulator (= server-side residual),
//            re-selects the top-k of the sum and stores the result into every
//            rank's inbox, releasing their flags.
//   pull   : every rank zero-fills the gradient, waits for each owner's flag and
//            scatters value / N.
//
// All units of a bucket are batched in each launch (gridDim.y = units), which is
// the "bulk synchronisation" of many small tensors.  Waiting only happens across
// GPUs: the launches of one GPU are ordered by the stream.
//
// Reference parity: DGC through the PS topology is the reference's ResNet-50
// style configuration (--comp_alg dgc, README.md:180; CaSync-PS cost shape
// src/SeCoPa/SeCoPa.py:75-89 of mark14wu/hipress).
#include <cuda_runtime.h>

#include "hipress/capi.h"
#include "sparse_core.cuh"
#include "sync.cuh"

namespace hipress {

struct SpSeg {
  const float* g;
  float* a;    // accumulator: DGC v / GradDrop residual
  float* u;    // DGC momentum or null
  float* out;  // averaged gradient (may alias g)
  float* sr;   // server accumulator for the owned chunk [chunk]
  uint32_t n, chunk, kmax, pay_off;
  uint32_t cap;         // candidate pairs per (tensor, chunk) unit
  uint64_t cand_push;   // first push unit's candidate list, in pairs from the region start
  uint64_t cand_srv;    // the server unit's candidate list
};

struct SpBucket {
  SpSeg seg[HP_MAX_SEGS];
  int nseg;
  int alg;
  float ratio, momentum, inv_n;
  uint64_t slot_bytes;
  uint64_t cand_pairs;  // candidate pairs of all units of one rank
};

__device__ __forceinline__ uint32_t sp_chunk_valid(uint32_t n, uint32_t chunk, int c) {
  const uint64_t start = (uint64_t)c * chunk;
  if (start >= n) return 0;
  const uint64_t rest = n - start;
  return (uint32_t)(rest < chunk ? rest : chunk);
}

__device__ __forceinline__ void write_empty_header(uint8_t* out, int alg) {
  WireHeader h;
  h.n = 0; h.alg = (uint8_t)alg; h.bitwidth = 0; h.flags = 0; h.a = 0.0f; h.b = 0;
  *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(&h);
}

// ---------------------------------------------------------------- push
// unit y = seg * N + owner
// STAGE 0: update + hist0   1: split (certain elements go to the owner at once)
//       2,3: digit passes on the candidate list   4: candidate compaction + flag
//       5,6,7: full-array passes and compaction, only after a candidate overflow
template <int STAGE>
__global__ void __launch_bounds__(kSpThreads)
sp_push_kernel(const SpBucket bk, const HpComm cm, int R, int E, uint32_t* ws_all,
               uint8_t* cand_all) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  const int N = cm.nranks;
  const int si = blockIdx.y / N, c = blockIdx.y % N;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* ws = ws_all + (size_t)blockIdx.y * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cand_all + (sg.cand_push + (uint64_t)c * sg.cap) * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  const size_t off = (size_t)c * sg.chunk;
  const float* g = sg.g + E * cm.emu_stride_g + off;
  float* a = sg.a + E * cm.emu_stride_r + off;
  float* u = sg.u ? sg.u + E * cm.emu_stride_r + off : nullptr;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[c]) + (size_t)R * bk.slot_bytes + sg.pay_off;
  EmitDst d;
  d.n = 1;
  d.out[0] = dst;
  bool last = false;
  if (STAGE == 0) {
    if (len == 0) return;
    if (bk.alg == kDgc) pass0_body<2>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
    else pass0_body<1>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    __shared__ SplitSmem sp;
    split_body(a, u, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, fs, sp, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 2 || STAGE == 3) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 2) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 4) {
    if (len == 0) {
      last = blockIdx.x == 0 && threadIdx.x == 0;
      if (last) write_empty_header(dst, bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, u, ws[kWsCandCount], k, sg.kmax, d, ws, fs, es, blockIdx.x,
                       gridDim.x, cand_idx, a, len);
    }
  } else if (STAGE == 5 || STAGE == 6) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 5) pass_body<1>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, a, u, len, k, sg.kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
  }
  if (last) {  // thread 0 of the CTA that completed the unit
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[c]) + (size_t)R * bk.nseg + si, cm.epoch);
  }
}

// -------------------------------------------------------------- server
// unit y = seg; the owned chunk is chunk R
// STAGE 0: wait + scatter-add   1: hist0   2: split (to every rank)   3,4: candidate
//       digit passes   5: candidate compaction + flags   6,7,8: overflow path
template <int STAGE>
__global__ void __launch_bounds__(kSpThreads)
sp_server_kernel(const SpBucket bk, const HpComm cm, int R, int E, uint32_t* ws_all,
                 uint8_t* cand_all) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  __shared__ WaitState wst;
  const int N = cm.nranks;
  const int si = blockIdx.y;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, R);
  uint32_t* ws = ws_all + (size_t)blockIdx.y * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cand_all + sg.cand_srv * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  float* acc = sg.sr + E * cm.emu_stride_sr;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  EmitDst d;
  d.n = N;
  for (int q = 0; q < N; ++q)
    d.out[q] = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) + (size_t)(N + R) * bk.slot_bytes +
               sg.pay_off;
  bool last = false;
  if (STAGE == 0) {
    wait_init(wst);
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(cm.flags[R]);
    for (int q = 0; q < N; ++q)
      wait_flag(my_flags + (size_t)q * bk.nseg + si, cm.epoch, cm.timeout_ns, status,
                HP_STATUS_TIMEOUT | (4u << 16) | ((uint32_t)q << 8) | (si & 255), wst);
    if (len == 0) return;
    const uint8_t* inbox = reinterpret_cast<const uint8_t*>(cm.inbox[R]);
    for (int q = 0; q < N; ++q)
      scatter_body(inbox + (size_t)q * bk.slot_bytes + sg.pay_off, acc, len, sg.kmax, 1.0f, 2,
                   blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    pass0_body<0>(nullptr, acc, nullptr, len, 0.0f, ws, sh, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 2) {
    if (len == 0) return;
    __shared__ SplitSmem sp;
    split_body(acc, nullptr, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, fs, sp, blockIdx.x,
               gridDim.x);
    return;
  } else if (STAGE == 3 || STAGE == 4) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 3) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 5) {
    if (len == 0) {
      last = blockIdx.x == 0 && threadIdx.x == 0;
      if (last)
        for (int q = 0; q < N; ++q) write_empty_header(d.out[q], bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, nullptr, ws[kWsCandCount], k, sg.kmax, d, ws, fs, es,
                       blockIdx.x, gridDim.x, cand_idx, acc, len);
    }
  } else if (STAGE == 6 || STAGE == 7) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 6) pass_body<1>(acc, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(acc, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, acc, nullptr, len, k, sg.kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
  }
  if (last) {
    __threadfence_system();
    for (int q = 0; q < N; ++q)
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) +
                         (size_t)(N + R) * bk.nseg + si,
                     cm.epoch);
  }
}

// ---------------------------------------------------------------- pull
// STAGE 0: zero-fill (unit y = seg); STAGE 1: wait + scatter (unit y = seg * N + owner)
template <int STAGE>
__global__ void __launch_bounds__(kSpThreads)
sp_pull_kernel(const SpBucket bk, const HpComm cm, int R, int E) {
  __shared__ WaitState wst;
  const int N = cm.nranks;
  if (STAGE == 0) {
    const SpSeg& sg = bk.seg[blockIdx.y];
    float* out = sg.out + E * cm.emu_stride_out;
    const bool vec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    const uint64_t stride = (uint64_t)gridDim.x * kSpThreads * 4;
    for (uint64_t i = ((uint64_t)blockIdx.x * kSpThreads + threadIdx.x) * 4; i < sg.n; i += stride)
      st4(out, i, sg.n, vec, make_float4(0.f, 0.f, 0.f, 0.f));
    return;
  }
  const int si = blockIdx.y / N, j = blockIdx.y % N;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, j);
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  wait_init(wst);
  wait_flag(reinterpret_cast<const uint32_t*>(cm.flags[R]) + (size_t)(N + j) * bk.nseg + si, cm.epoch,
            cm.timeout_ns, status, HP_STATUS_TIMEOUT | (5u << 16) | ((uint32_t)j << 8) | (si & 255),
            wst);
  if (len == 0) return;
  const uint8_t* p = reinterpret_cast<const uint8_t*>(cm.inbox[R]) + (size_t)(N + j) * bk.slot_bytes +
                     sg.pay_off;
  scatter_body(p, sg.out + E * cm.emu_stride_out + (size_t)j * sg.chunk, len, sg.kmax, bk.inv_n, 0,
               blockIdx.x, gridDim.x);
}

// ---------------------------------------------------------------- ring
// One hop of the sparse ring for every tensor of the bucket (unit y = seg).  At hop
// h rank R works on chunk (R - h) mod N: the predecessor's pairs are added into the
// local accumulator, then the state update, the exact top-k selection and the
// compaction run, and the pairs go into the successor's inbox -- or, at the last
// hop, into every rank's inbox.
// STAGE 0: wait + add incoming   1: update + hist0   2: split   3,4: candidate digit
//       passes   5: candidate compaction + flag(s)   6,7,8: overflow path
template <int STAGE>
__global__ void __launch_bounds__(kSpThreads)
sp_ring_kernel(const SpBucket bk, const HpComm cm, int R, int E, int hop, uint32_t* ws_all,
               uint8_t* cand_all) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  __shared__ WaitState wst;
  const int N = cm.nranks;
  const int si = blockIdx.y;
  const int c = (R - hop + N) % N;
  const bool last_hop = hop == N - 1;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* ws = ws_all + ((size_t)hop * bk.nseg + si) * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cand_all + (sg.cand_push + (uint64_t)c * sg.cap) * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  const size_t off = (size_t)c * sg.chunk;
  const float* g = sg.g + E * cm.emu_stride_g + off;
  float* a = sg.a + E * cm.emu_stride_r + off;
  float* u = sg.u ? sg.u + E * cm.emu_stride_r + off : nullptr;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  EmitDst d;
  if (!last_hop) {
    d.n = 1;
    d.out[0] = reinterpret_cast<uint8_t*>(cm.inbox[(R + 1) % N]) + (size_t)hop * bk.slot_bytes + sg.pay_off;
  } else {
    d.n = N;
    for (int q = 0; q < N; ++q)
      d.out[q] = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) +
                 (size_t)(N - 1 + R) * bk.slot_bytes + sg.pay_off;
  }
  bool last = false;
  if (STAGE == 0) {
    if (hop == 0) return;
    wait_init(wst);
    wait_flag(reinterpret_cast<const uint32_t*>(cm.flags[R]) + (size_t)(hop - 1) * bk.nseg + si,
              cm.epoch, cm.timeout_ns, status,
              HP_STATUS_TIMEOUT | (6u << 16) | ((uint32_t)(hop - 1) << 8) | (si & 255), wst);
    if (len == 0) return;
    scatter_body(reinterpret_cast<const uint8_t*>(cm.inbox[R]) + (size_t)(hop - 1) * bk.slot_bytes +
                     sg.pay_off,
                 a, len, sg.kmax, 1.0f, 1, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    if (bk.alg == kDgc) pass0_body<2>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
    else pass0_body<1>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 2) {
    if (len == 0) return;
    __shared__ SplitSmem sp;
    split_body(a, u, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, fs, sp, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 3 || STAGE == 4) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 3) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else if (STAGE == 5) {
    if (len == 0) {
      last = blockIdx.x == 0 && threadIdx.x == 0;
      if (last)
        for (int q = 0; q < d.n; ++q) write_empty_header(d.out[q], bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, u, ws[kWsCandCount], k, sg.kmax, d, ws, fs, es, blockIdx.x,
                       gridDim.x, cand_idx, a, len);
    }
  } else if (STAGE == 6 || STAGE == 7) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 6) pass_body<1>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    else pass_body<2>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, a, u, len, k, sg.kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
  }
  if (last) {
    __threadfence_system();
    if (!last_hop) {
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + 1) % N]) + (size_t)hop * bk.nseg + si,
                     cm.epoch);
    } else {
      for (int q = 0; q < N; ++q)
        st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) +
                           (size_t)(N - 1 + R) * bk.nseg + si,
                       cm.epoch);
    }
  }
}

// gather of the ring: unit y = seg * N + src; rank src finalised chunk src + 1
__global__ void __launch_bounds__(kSpThreads)
sp_ring_gather_kernel(const SpBucket bk, const HpComm cm, int R, int E) {
  __shared__ WaitState wst;
  const int N = cm.nranks;
  const int si = blockIdx.y / N, src = blockIdx.y % N;
  const int c = (src + 1) % N;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  wait_init(wst);
  wait_flag(reinterpret_cast<const uint32_t*>(cm.flags[R]) + (size_t)(N - 1 + src) * bk.nseg + si,
            cm.epoch, cm.timeout_ns, status,
            HP_STATUS_TIMEOUT | (7u << 16) | ((uint32_t)src << 8) | (si & 255), wst);
  if (len == 0) return;
  const uint8_t* p = reinterpret_cast<const uint8_t*>(cm.inbox[R]) +
                     (size_t)(N - 1 + src) * bk.slot_bytes + sg.pay_off;
  scatter_body(p, sg.out + E * cm.emu_stride_out + (size_t)c * sg.chunk, len, sg.kmax, bk.inv_n, 0,
               blockIdx.x, gridDim.x);
}

static int build_sp_bucket(int alg, float ratio, float momentum, const HpSeg* segs,
                           void* const* accs, void* const* us, int nseg, int nranks, SpBucket& bk) {
  if (nseg < 1 || nseg > HP_MAX_SEGS || nranks < 1 || nranks > HP_MAX_RANKS) return HP_ERR_BAD_ARG;
  if (alg != kDgc && alg != kGradDrop) return HP_ERR_BAD_ARG;
  uint64_t pay = 0, cand = 0;
  for (int i = 0; i < nseg; ++i) {
    const uint64_t n = segs[i].n;
    if (n == 0 || n > 0xFFFFF000ull) return HP_ERR_BAD_ARG;
    const uint64_t chunk = align_up((n + nranks - 1) / nranks, kTile);
    SpSeg& d = bk.seg[i];
    d.g = static_cast<const float*>(segs[i].g);
    d.a = accs ? static_cast<float*>(accs[i]) : static_cast<float*>(segs[i].r);
    d.u = us ? static_cast<float*>(us[i]) : nullptr;
    d.out = static_cast<float*>(segs[i].out);
    d.sr = static_cast<float*>(segs[i].sr);
    d.n = (uint32_t)n;
    d.chunk = (uint32_t)chunk;
    d.kmax = (uint32_t)sparse_k(chunk, ratio);
    d.pay_off = (uint32_t)pay;
    d.cap = (uint32_t)align_up(8ull * d.kmax + 4096, 32);
    d.cand_push = cand;
    cand += (uint64_t)d.cap * nranks;
    d.cand_srv = cand;
    cand += d.cap;
    pay += align_up(sparse_payload_bytes(d.kmax), 128);
    if (pay > 0xFFFFFFFFull) return HP_ERR_TOO_LARGE;
  }
  bk.nseg = nseg;
  bk.alg = alg;
  bk.ratio = ratio;
  bk.momentum = momentum;
  bk.inv_n = 1.0f / (float)nranks;
  bk.slot_bytes = pay;
  bk.cand_pairs = cand;
  return 0;
}

}  // namespace hipress

using namespace hipress;

extern "C" {

// sizes a caller needs to reserve for a bucket of tensors with the given sizes
int hp_fused_sparse_layout(float ratio, const uint64_t* ns, int nseg, int nranks,
                           uint64_t* inbox_bytes, uint64_t* flag_words, uint64_t* ws_bytes) {
  if (nseg < 1 || nseg > HP_MAX_SEGS) return HP_ERR_BAD_ARG;
  HpSeg segs[HP_MAX_SEGS] = {};
  for (int i = 0; i < nseg; ++i) segs[i].n = ns[i];
  SpBucket bk;
  int rc = build_sp_bucket(kDgc, ratio, 0.f, segs, nullptr, nullptr, nseg, nranks, bk);
  if (rc) return rc;
  if (inbox_bytes) *inbox_bytes = bk.slot_bytes * 2ull * nranks;
  if (flag_words) *flag_words = 2ull * nranks * nseg;
  // push units (nseg * nranks) + server units (nseg), per emulated rank
  if (ws_bytes)
    *ws_bytes = align_up((uint64_t)(nseg * nranks + nseg) * kWsWords * 4, 256) + bk.cand_pairs * 8;
  return 0;
}

// One synchronisation of a bucket through the PS topology.  segs[i].r is the
// accumulator (DGC v / GradDrop residual), us[i] the DGC momentum (or NULL),
// segs[i].sr the server accumulator of the owned chunk.  ws: zero-initialised
// scratch of hp_fused_sparse_layout().ws_bytes per rank played by this call.
int hp_cuda_fused_sparse_ps(int alg, float ratio, float momentum, const HpSeg* segs,
                            void* const* us, int nseg, const HpComm* comm, void* ws, int ctas,
                            void* stream) {
  if (!comm || ctas > 1024) return HP_ERR_BAD_ARG;
  SpBucket bk;
  const int N = comm->nranks;
  int rc = build_sp_bucket(alg, ratio, momentum, segs, nullptr, us, nseg, N, bk);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int ranks_here = comm->emulate ? N : 1;
  const size_t hist_words = (size_t)(nseg * N + nseg) * kWsWords;
  const size_t hist_bytes = align_up(hist_words * 4, 256);
  const size_t ws_rank_bytes = hist_bytes + bk.cand_pairs * 8;
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  for (int r = 0; r < ranks_here; ++r) {  // only the histogram blocks need clearing
    cudaError_t e = cudaMemsetAsync(wsb + (size_t)r * ws_rank_bytes, 0, hist_words * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  // ctas <= 0: size the grids so that every launch fills the GPU about four
  // CTAs per SM, whatever the number of (tensor, owner) units
  auto per_unit = [&](int units) {
    if (ctas > 0) return ctas;
    int c = (148 * 4 + units - 1) / units;
    return c < 4 ? 4 : (c > 592 ? 592 : c);
  };
  const dim3 gpush(per_unit(nseg * N), nseg * N), gsrv(per_unit(nseg), nseg);
  const dim3 cpush(gpush.x < 32 ? gpush.x : 32, nseg * N), csrv(gsrv.x < 32 ? gsrv.x : 32, nseg);
  const dim3 gpull(per_unit(nseg * N) < 16 ? per_unit(nseg * N) : 16, nseg * N);
  // With emulated ranks every phase is issued for all ranks before the next one,
  // so a wait never targets a launch that is still queued behind it.
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    uint32_t* w = reinterpret_cast<uint32_t*>(wsb + (size_t)r * ws_rank_bytes);
    uint8_t* cd = wsb + (size_t)r * ws_rank_bytes + hist_bytes;
    sp_push_kernel<0><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<1><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<2><<<cpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<3><<<cpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<4><<<cpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<5><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<6><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_push_kernel<7><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
  }
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    uint32_t* w = reinterpret_cast<uint32_t*>(wsb + (size_t)r * ws_rank_bytes) +
                  (size_t)nseg * N * kWsWords;
    uint8_t* cd = wsb + (size_t)r * ws_rank_bytes + hist_bytes;
    sp_server_kernel<0><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<1><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<2><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<3><<<csrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<4><<<csrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<5><<<csrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<6><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<7><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
    sp_server_kernel<8><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w, cd);
  }
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    sp_pull_kernel<0><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E);
    sp_pull_kernel<1><<<gpull, kSpThreads, 0, st>>>(bk, *comm, R, E);
  }
  return (int)cudaGetLastError();
}

// One synchronisation of a bucket through the ring topology: N hops, each a fixed
// sequence of launches over all tensors of the bucket, then the gather.  Same
// arguments as hp_cuda_fused_sparse_ps (segs[i].sr is not used).
int hp_cuda_fused_sparse_ring(int alg, float ratio, float momentum, const HpSeg* segs,
                              void* const* us, int nseg, const HpComm* comm, void* ws, int ctas,
                              void* stream) {
  if (!comm || ctas > 1024) return HP_ERR_BAD_ARG;
  SpBucket bk;
  const int N = comm->nranks;
  int rc = build_sp_bucket(alg, ratio, momentum, segs, nullptr, us, nseg, N, bk);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int ranks_here = comm->emulate ? N : 1;
  const size_t hist_words = (size_t)(nseg * N + nseg) * kWsWords;  // ring uses nseg * N of them
  const size_t hist_bytes = align_up(hist_words * 4, 256);
  const size_t ws_rank_bytes = hist_bytes + bk.cand_pairs * 8;
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  for (int r = 0; r < ranks_here; ++r) {
    cudaError_t e = cudaMemsetAsync(wsb + (size_t)r * ws_rank_bytes, 0, hist_words * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  auto per_unit = [&](int units) {
    if (ctas > 0) return ctas;
    int c = (148 * 4 + units - 1) / units;
    return c < 4 ? 4 : (c > 592 ? 592 : c);
  };
  const dim3 gh(per_unit(nseg), nseg), ch(gh.x < 32 ? gh.x : 32, nseg);
  const dim3 gpull(per_unit(nseg * N) < 16 ? per_unit(nseg * N) : 16, nseg * N);
  // hop-major order: with emulated ranks the producer of a hop's input has
  // always been issued before its consumer
  for (int hop = 0; hop < N; ++hop) {
    for (int r = 0; r < ranks_here; ++r) {
      const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
      uint32_t* w = reinterpret_cast<uint32_t*>(wsb + (size_t)r * ws_rank_bytes);
      uint8_t* cd = wsb + (size_t)r * ws_rank_bytes + hist_bytes;
      if (hop > 0) sp_ring_kernel<0><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<1><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<2><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<3><<<ch, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<4><<<ch, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<5><<<ch, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<6><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<7><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
      sp_ring_kernel<8><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E, hop, w, cd);
    }
  }
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    sp_pull_kernel<0><<<gh, kSpThreads, 0, st>>>(bk, *comm, R, E);
    sp_ring_gather_kernel<<<gpull, kSpThreads, 0, st>>>(bk, *comm, R, E);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
