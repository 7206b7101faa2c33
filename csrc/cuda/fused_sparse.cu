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
};

struct SpBucket {
  SpSeg seg[HP_MAX_SEGS];
  int nseg;
  int alg;
  float ratio, momentum, inv_n;
  uint64_t slot_bytes;
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
template <int STAGE>  // 0: update + hist0, 1: hist1, 2: hist2, 3: emit + flag
__global__ void __launch_bounds__(kSpThreads)
sp_push_kernel(const SpBucket bk, const HpComm cm, int R, int E, uint32_t* ws_all) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  const int N = cm.nranks;
  const int si = blockIdx.y / N, c = blockIdx.y % N;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* ws = ws_all + (size_t)blockIdx.y * kWsWords;
  const size_t off = (size_t)c * sg.chunk;
  const float* g = sg.g + E * cm.emu_stride_g + off;
  float* a = sg.a + E * cm.emu_stride_r + off;
  float* u = sg.u ? sg.u + E * cm.emu_stride_r + off : nullptr;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  if (STAGE == 0) {
    if (len == 0) return;
    if (bk.alg == kDgc) pass0_body<2>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
    else pass0_body<1>(g, a, u, len, bk.momentum, ws, sh, blockIdx.x, gridDim.x);
  } else if (STAGE == 1) {
    if (len == 0) return;
    pass_body<1>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
  } else if (STAGE == 2) {
    if (len == 0) return;
    pass_body<2>(a, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
  } else {
    uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[c]) + (size_t)R * bk.slot_bytes + sg.pay_off;
    bool last;
    if (len == 0) {
      last = blockIdx.x == 0 && threadIdx.x == 0;
      if (last) write_empty_header(dst, bk.alg);
    } else {
      EmitDst d;
      d.n = 1;
      d.out[0] = dst;
      last = emit_body(bk.alg, a, u, len, k, sg.kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
    }
    if (last) {  // thread 0 of the CTA that completed the unit
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[c]) + (size_t)R * bk.nseg + si, cm.epoch);
    }
  }
}

// -------------------------------------------------------------- server
// unit y = seg; the owned chunk is chunk R
template <int STAGE>  // 0: wait + scatter-add, 1..3: hist passes, 4: emit to all + flags
__global__ void __launch_bounds__(kSpThreads)
sp_server_kernel(const SpBucket bk, const HpComm cm, int R, int E, uint32_t* ws_all) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  __shared__ WaitState wst;
  const int N = cm.nranks;
  const int si = blockIdx.y;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, R);
  uint32_t* ws = ws_all + (size_t)blockIdx.y * kWsWords;
  float* acc = sg.sr + E * cm.emu_stride_sr;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
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
  } else if (STAGE == 1) {
    if (len == 0) return;
    pass0_body<0>(nullptr, acc, nullptr, len, 0.0f, ws, sh, blockIdx.x, gridDim.x);
  } else if (STAGE == 2) {
    if (len == 0) return;
    pass_body<1>(acc, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
  } else if (STAGE == 3) {
    if (len == 0) return;
    pass_body<2>(acc, len, k, ws, sh, fs, blockIdx.x, gridDim.x);
  } else {
    EmitDst d;
    d.n = N;
    for (int q = 0; q < N; ++q)
      d.out[q] = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) + (size_t)(N + R) * bk.slot_bytes +
                 sg.pay_off;
    bool last;
    if (len == 0) {
      last = blockIdx.x == 0 && threadIdx.x == 0;
      if (last)
        for (int q = 0; q < N; ++q) write_empty_header(d.out[q], bk.alg);
    } else {
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

static int build_sp_bucket(int alg, float ratio, float momentum, const HpSeg* segs,
                           void* const* accs, void* const* us, int nseg, int nranks, SpBucket& bk) {
  if (nseg < 1 || nseg > HP_MAX_SEGS || nranks < 1 || nranks > HP_MAX_RANKS) return HP_ERR_BAD_ARG;
  if (alg != kDgc && alg != kGradDrop) return HP_ERR_BAD_ARG;
  uint64_t pay = 0;
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
    pay += align_up(sparse_payload_bytes(d.kmax), 128);
    if (pay > 0xFFFFFFFFull) return HP_ERR_TOO_LARGE;
  }
  bk.nseg = nseg;
  bk.alg = alg;
  bk.ratio = ratio;
  bk.momentum = momentum;
  bk.inv_n = 1.0f / (float)nranks;
  bk.slot_bytes = pay;
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
  if (ws_bytes) *ws_bytes = (uint64_t)(nseg * nranks + nseg) * kWsWords * 4;
  return 0;
}

// One synchronisation of a bucket through the PS topology.  segs[i].r is the
// accumulator (DGC v / GradDrop residual), us[i] the DGC momentum (or NULL),
// segs[i].sr the server accumulator of the owned chunk.  ws: zero-initialised
// scratch of hp_fused_sparse_layout().ws_bytes per rank played by this call.
int hp_cuda_fused_sparse_ps(int alg, float ratio, float momentum, const HpSeg* segs,
                            void* const* us, int nseg, const HpComm* comm, void* ws, int ctas,
                            void* stream) {
  if (!comm || ctas < 1 || ctas > 1024) return HP_ERR_BAD_ARG;
  SpBucket bk;
  const int N = comm->nranks;
  int rc = build_sp_bucket(alg, ratio, momentum, segs, nullptr, us, nseg, N, bk);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int ranks_here = comm->emulate ? N : 1;
  const size_t ws_rank_words = (size_t)(nseg * N + nseg) * kWsWords;
  cudaError_t e = cudaMemsetAsync(ws, 0, ws_rank_words * 4 * ranks_here, st);
  if (e != cudaSuccess) return (int)e;
  uint32_t* wsw = static_cast<uint32_t*>(ws);
  const dim3 gpush(ctas, nseg * N), gsrv(ctas, nseg);
  // With emulated ranks every phase is issued for all ranks before the next one,
  // so a wait never targets a launch that is still queued behind it.
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    uint32_t* w = wsw + (size_t)r * ws_rank_words;
    sp_push_kernel<0><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_push_kernel<1><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_push_kernel<2><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_push_kernel<3><<<gpush, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
  }
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    uint32_t* w = wsw + (size_t)r * ws_rank_words + (size_t)nseg * N * kWsWords;
    sp_server_kernel<0><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_server_kernel<1><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_server_kernel<2><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_server_kernel<3><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
    sp_server_kernel<4><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E, w);
  }
  for (int r = 0; r < ranks_here; ++r) {
    const int R = comm->emulate ? r : comm->rank, E = comm->emulate ? r : 0;
    sp_pull_kernel<0><<<gsrv, kSpThreads, 0, st>>>(bk, *comm, R, E);
    sp_pull_kernel<1><<<dim3(4, nseg * N), kSpThreads, 0, st>>>(bk, *comm, R, E);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
