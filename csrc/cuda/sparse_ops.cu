// Sparse (top-k) compression for DGC and GradDrop on sm_100a.
//
//   pass 0   state update fused with the first radix histogram
//              DGC      : u = m*u + g ; v += u        (momentum correction)
//              GradDrop : r += g
//            and a 4096-bin shared-memory histogram of bits 30..19 of |v|
//   pass 1,2 histograms of bits 18..8 and 7..0 among elements matching the
//            prefix chosen so far (every CTA re-derives the prefix from the global
//            histograms, so no tiny "scan" launches sit between the passes)
//   emit     exact threshold known: block-aggregated compaction of (index,value)
//            pairs straight into the payload (which may live on a peer GPU), sent
//            entries of v (and u) zeroed, header written by the last CTA.
//
// The selection is exact: every |v_i| above the k-th largest magnitude is sent,
// plus entries equal to it until k are sent (which of several equal entries is
// unspecified on the GPU; the CPU oracle takes the lowest indices).  Zeros are
// never sent.  Pair order inside the payload is unspecified.
//
// Reference parity: DGC and GradDrop are two of the five built-in algorithms of
// mark14wu/hipress (README.md:9; --comp_alg dgc README.md:180); CompLL planned
// sort/copy_if for them (src/CompLL/GCGen/unit.py:24-29) but has no translation
// rule, so there is no reference kernel to compare with.
#include "sparse_core.cuh"
#include "hipress/noalloc.h"

namespace hipress {

template <int MODE>
__global__ void __launch_bounds__(kSpThreads)
sparse_pass0_kernel(const float* __restrict__ g, float* __restrict__ a, float* __restrict__ u,
                    uint64_t n, float momentum, uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  pass0_body<MODE>(g, a, u, n, momentum, ws, sh, blockIdx.x, gridDim.x);
}

template <int PASS>
__global__ void __launch_bounds__(kSpThreads)
sparse_pass_kernel(const float* __restrict__ a, uint64_t n, uint32_t k,
                   uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  pass_body<PASS>(a, n, k, ws, sh, fs, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(kSpThreads)
sparse_emit_kernel(int alg, float* __restrict__ a, float* __restrict__ u, uint64_t n, uint32_t k,
                   uint32_t kmax, uint8_t* __restrict__ out, uint32_t* __restrict__ ws) {
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  EmitDst d;
  d.n = 1;
  d.out[0] = out;
  emit_body(alg, a, u, n, k, kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
}

// ---- candidate path: split pass, then digit passes and compaction on the list
__global__ void __launch_bounds__(kSpThreads)
sparse_split_kernel(float* __restrict__ a, float* __restrict__ u, uint64_t n, uint32_t k,
                    uint32_t kmax, uint8_t* __restrict__ out, uint32_t* __restrict__ ws,
                    float* __restrict__ cand_val, uint32_t* __restrict__ cand_idx, uint32_t cap) {
  __shared__ FindSmem fs;
  __shared__ SplitSmem sp;
  EmitDst d;
  d.n = 1;
  d.out[0] = out;
  split_body(a, u, n, k, kmax, d, ws, cand_val, cand_idx, cap, fs, sp, blockIdx.x, gridDim.x);
}

template <int PASS>
__global__ void __launch_bounds__(kSpThreads)
sparse_cand_pass_kernel(const float* __restrict__ cand_val, uint32_t k, uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  if (ws[kWsOverflow]) return;
  pass_body<PASS>(cand_val, ws[kWsCandCount], k, ws, sh, fs, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(kSpThreads)
sparse_cand_emit_kernel(int alg, float* __restrict__ cand_val, const uint32_t* __restrict__ cand_idx,
                        float* __restrict__ a, float* __restrict__ u, uint32_t k, uint32_t kmax,
                        uint8_t* __restrict__ out, uint32_t* __restrict__ ws, uint64_t n) {
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  if (ws[kWsOverflow]) return;
  EmitDst d;
  d.n = 1;
  d.out[0] = out;
  emit_body(alg, cand_val, u, ws[kWsCandCount], k, kmax, d, ws, fs, es, blockIdx.x, gridDim.x,
            cand_idx, a, (uint32_t)n);
}

// ---- the full-array passes, run only when the candidate list overflowed
template <int PASS>
__global__ void __launch_bounds__(kSpThreads)
sparse_fallback_pass_kernel(const float* __restrict__ a, uint64_t n, uint32_t k,
                            uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  if (!ws[kWsOverflow]) return;
  pass_body<PASS>(a, n, k, ws, sh, fs, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(kSpThreads)
sparse_fallback_emit_kernel(int alg, float* __restrict__ a, float* __restrict__ u, uint64_t n,
                            uint32_t k, uint32_t kmax, uint8_t* __restrict__ out,
                            uint32_t* __restrict__ ws) {
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  if (!ws[kWsOverflow]) return;
  EmitDst d;
  d.n = 1;
  d.out[0] = out;
  emit_body(alg, a, u, n, k, kmax, d, ws, fs, es, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(kSpThreads)
sparse_scatter_kernel(const uint8_t* __restrict__ payload, float* __restrict__ out, uint64_t n,
                      uint32_t kmax, float scale, int accumulate) {
  scatter_body(payload, out, n, kmax, scale, accumulate, blockIdx.x, gridDim.x);
}

}  // namespace hipress

using namespace hipress;

extern "C" {

// minimum scratch (histograms + counters); with room for a candidate list of
// about 8 * kmax pairs on top, the encoder reads the array once instead of three
// times after the state update
uint64_t hp_sparse_workspace_bytes() { return (uint64_t)kWsWords * 4; }
uint64_t hp_sparse_workspace_bytes_for(uint64_t kmax) {
  return (uint64_t)kWsWords * 4 + (8 * kmax + 4096) * 8;
}

// ws_bytes beyond the histogram block is used as the candidate list; when there
// is none (the allocation-free entry point) the three full-array passes run.
static int sparse_encode_impl(int alg, const float* g, float* a, float* u, uint64_t n, uint64_t k,
                              uint64_t kmax, float momentum, int update, uint8_t* out,
                              uint32_t* ws, uint64_t ws_bytes, int max_ctas, cudaStream_t st) {
  if (n == 0 || n > 0xFFFFF000ull || k < 1 || k > n || k > kmax || kmax > 0xFFFFFFFFull)
    return HP_ERR_BAD_ARG;
  if (alg != kDgc && alg != kGradDrop) return HP_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(out) & 15) return HP_ERR_BAD_ARG;
  if (update && !g) return HP_ERR_BAD_ARG;
  if (update && alg == kDgc && !u) return HP_ERR_BAD_ARG;
  if (max_ctas <= 0) max_ctas = 148 * 4;
  const uint64_t tiles = (n + 4095) / 4096;
  const int grid = (int)(tiles < (uint64_t)max_ctas ? tiles : (uint64_t)max_ctas);
  cudaError_t e = cudaMemsetAsync(ws, 0, (size_t)kWsWords * 4, st);
  if (e != cudaSuccess) return (int)e;
  if (!update) sparse_pass0_kernel<0><<<grid, kSpThreads, 0, st>>>(g, a, u, n, momentum, ws);
  else if (alg == kGradDrop) sparse_pass0_kernel<1><<<grid, kSpThreads, 0, st>>>(g, a, u, n, momentum, ws);
  else sparse_pass0_kernel<2><<<grid, kSpThreads, 0, st>>>(g, a, u, n, momentum, ws);
  float* uu = alg == kDgc ? u : nullptr;
  const uint64_t head = (uint64_t)kWsWords * 4;
  const uint64_t cap = ws_bytes > head ? (ws_bytes - head) / 8 : 0;
  if (cap >= 1024) {
    float* cand_val = reinterpret_cast<float*>(ws + kWsWords);
    uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + cap);
    const int cgrid = grid < 64 ? grid : 64;
    sparse_split_kernel<<<grid, kSpThreads, 0, st>>>(a, uu, n, (uint32_t)k, (uint32_t)kmax, out, ws,
                                                      cand_val, cand_idx, (uint32_t)cap);
    sparse_cand_pass_kernel<1><<<cgrid, kSpThreads, 0, st>>>(cand_val, (uint32_t)k, ws);
    sparse_cand_pass_kernel<2><<<cgrid, kSpThreads, 0, st>>>(cand_val, (uint32_t)k, ws);
    sparse_cand_emit_kernel<<<cgrid, kSpThreads, 0, st>>>(alg, cand_val, cand_idx, a, uu, (uint32_t)k,
                                                          (uint32_t)kmax, out, ws, n);
    sparse_fallback_pass_kernel<1><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
    sparse_fallback_pass_kernel<2><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
    sparse_fallback_emit_kernel<<<grid, kSpThreads, 0, st>>>(alg, a, uu, n, (uint32_t)k,
                                                              (uint32_t)kmax, out, ws);
  } else {
    sparse_pass_kernel<1><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
    sparse_pass_kernel<2><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
    sparse_emit_kernel<<<grid, kSpThreads, 0, st>>>(alg, a, uu, n, (uint32_t)k, (uint32_t)kmax, out,
                                                     ws);
  }
  return (int)cudaGetLastError();
}

// a: accumulator (DGC v / GradDrop residual).  update=1 applies the state update
// with g first; update=0 selects from a as it is (server / ring re-selection).
int hp_cuda_sparse_encode(int alg, const float* g, float* a, float* u, uint64_t n, uint64_t k,
                          uint64_t kmax, float momentum, int update, uint8_t* out, void* workspace,
                          uint64_t workspace_bytes, int max_ctas, void* stream) {
  if (workspace_bytes < (uint64_t)kWsWords * 4) return HP_ERR_BAD_ARG;
  return sparse_encode_impl(alg, g, a, u, n, k, kmax, momentum, update, out,
                            static_cast<uint32_t*>(workspace), workspace_bytes, max_ctas,
                            (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Allocation-free variant (see hipress/noalloc.h): the scratch lives in this
// file-scope device array.  In host code the name below is only a handle for
// the runtime, never a device address; the address each GPU gave the array is
// fetched once per device with cudaGetSymbolAddress and passed to the kernels.
static __device__ __align__(256) uint32_t g_noalloc_scratch[kWsWords];

static uint32_t* g_noalloc_ptr[64];  // per device, filled on the first call there

uint64_t hp_cuda_noalloc_scratch_bytes(void) { return (uint64_t)kWsWords * 4; }

int hp_cuda_sparse_encode_noalloc(int alg, const float* g, float* a, float* u, uint64_t n,
                                  uint64_t k, uint64_t kmax, float momentum, int update,
                                  uint8_t* out, int max_ctas, void* stream) {
  if (n > HP_NOALLOC_MAX_ELEMS) return HP_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return HP_ERR_BAD_ARG;
  if (!g_noalloc_ptr[dev]) {  // set-up: once per device, with that device current
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!p) return HP_ERR_BAD_ARG;
    g_noalloc_ptr[dev] = static_cast<uint32_t*>(p);
  }
  return sparse_encode_impl(alg, g, a, u, n, k, kmax, momentum, update, out, g_noalloc_ptr[dev],
                            (uint64_t)kWsWords * 4, max_ctas, (cudaStream_t)stream);
}

// accumulate=0: out is zero-filled first.  accumulate=1: out[idx] += val*scale.
int hp_cuda_sparse_decode(const uint8_t* payload, float* out, uint64_t n, uint64_t kmax,
                          float scale, int accumulate, void* stream) {
  if (n == 0) return 0;
  if (reinterpret_cast<uintptr_t>(payload) & 15) return HP_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (!accumulate) {
    cudaError_t e = cudaMemsetAsync(out, 0, n * sizeof(float), st);
    if (e != cudaSuccess) return (int)e;
  }
  if (kmax == 0) return 0;
  int grid = (int)((kmax + kSpThreads - 1) / kSpThreads);
  if (grid > 148 * 8) grid = 148 * 8;
  sparse_scatter_kernel<<<grid, kSpThreads, 0, st>>>(payload, out, n, (uint32_t)kmax, scale,
                                                      accumulate);
  return (int)cudaGetLastError();
}

}  // extern "C"
