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
#include <cuda_runtime.h>
#include <stdint.h>

#include "hipress/capi.h"
#include "hipress/common.h"
#include "hipress/noalloc.h"

namespace hipress {

constexpr int kSpThreads = 256;
constexpr int kBins = 4096;
// workspace words: 3 histograms, then counters
constexpr int kWsOutCount = 3 * kBins + 0;
constexpr int kWsTieCount = 3 * kBins + 1;
constexpr int kWsDone = 3 * kBins + 2;
constexpr int kWsWords = 3 * kBins + 16;

__device__ __forceinline__ uint32_t digit_of(uint32_t key, int pass) {
  return pass == 0 ? (key >> 19) : (pass == 1 ? ((key >> 8) & 0x7FFu) : (key & 0xFFu));
}

struct FindSmem {
  uint32_t sums[kSpThreads];
  uint32_t res[2];
};

// Largest bin whose suffix count reaches k.  krem = how many of the k fall in
// that bin or below the bins above it, i.e. k - count(bins > bin).
__device__ __forceinline__ void find_bin(const uint32_t* __restrict__ hist, uint32_t k,
                                         FindSmem& fs, uint32_t& bin, uint32_t& krem) {
  constexpr int per = kBins / kSpThreads;  // 16
  uint32_t c[per];
  uint32_t sum = 0;
#pragma unroll
  for (int i = 0; i < per; ++i) {
    c[i] = hist[threadIdx.x * per + i];
    sum += c[i];
  }
  fs.sums[threadIdx.x] = sum;
  if (threadIdx.x == 0) {
    fs.res[0] = 0;
    fs.res[1] = 0;
  }
  __syncthreads();
  uint32_t above = 0;
  for (int t = (int)threadIdx.x + 1; t < kSpThreads; ++t) above += fs.sums[t];
  if (above < k && k <= above + sum) {
    uint32_t acc = above;
#pragma unroll
    for (int i = per - 1; i >= 0; --i) {
      if (acc < k && k <= acc + c[i]) {
        fs.res[0] = threadIdx.x * per + i;
        fs.res[1] = k - acc;
      }
      acc += c[i];
    }
  }
  __syncthreads();
  bin = fs.res[0];
  krem = fs.res[1];
  __syncthreads();
}

__device__ __forceinline__ void flush_hist(const uint32_t* sh, uint32_t* __restrict__ gh) {
  for (int i = threadIdx.x; i < kBins; i += kSpThreads) {
    const uint32_t c = sh[i];
    if (c) atomicAdd(gh + i, c);
  }
}

__device__ __forceinline__ float4 ld4(const float* p, uint64_t i, uint64_t n, bool vec) {
  if (vec && i + 3 < n) return *reinterpret_cast<const float4*>(p + i);
  float4 v;
  v.x = i < n ? p[i] : 0.0f;
  v.y = i + 1 < n ? p[i + 1] : 0.0f;
  v.z = i + 2 < n ? p[i + 2] : 0.0f;
  v.w = i + 3 < n ? p[i + 3] : 0.0f;
  return v;
}
__device__ __forceinline__ void st4(float* p, uint64_t i, uint64_t n, bool vec, float4 v) {
  if (vec && i + 3 < n) {
    *reinterpret_cast<float4*>(p + i) = v;
    return;
  }
  if (i < n) p[i] = v.x;
  if (i + 1 < n) p[i + 1] = v.y;
  if (i + 2 < n) p[i + 2] = v.z;
  if (i + 3 < n) p[i + 3] = v.w;
}

// MODE 0: select only (a already holds the accumulator)
// MODE 1: GradDrop  a += g
// MODE 2: DGC       u = m*u + g ; a += u
template <int MODE>
__global__ void __launch_bounds__(kSpThreads)
sparse_pass0_kernel(const float* __restrict__ g, float* __restrict__ a, float* __restrict__ u,
                    uint64_t n, float momentum, uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  for (int i = threadIdx.x; i < kBins; i += kSpThreads) sh[i] = 0;
  __syncthreads();
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g) |
                     reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  const uint64_t stride = (uint64_t)gridDim.x * kSpThreads * 4;
  for (uint64_t i = ((uint64_t)blockIdx.x * kSpThreads + threadIdx.x) * 4; i < n; i += stride) {
    float4 av = ld4(a, i, n, vec);
    if (MODE == 1) {
      const float4 gv = ld4(g, i, n, vec);
      av.x = av.x + gv.x; av.y = av.y + gv.y; av.z = av.z + gv.z; av.w = av.w + gv.w;
      st4(a, i, n, vec, av);
    } else if (MODE == 2) {
      const float4 gv = ld4(g, i, n, vec);
      float4 uv = ld4(u, i, n, vec);
      uv.x = __fmaf_rn(momentum, uv.x, gv.x);
      uv.y = __fmaf_rn(momentum, uv.y, gv.y);
      uv.z = __fmaf_rn(momentum, uv.z, gv.z);
      uv.w = __fmaf_rn(momentum, uv.w, gv.w);
      av.x = av.x + uv.x; av.y = av.y + uv.y; av.z = av.z + uv.z; av.w = av.w + uv.w;
      st4(u, i, n, vec, uv);
      st4(a, i, n, vec, av);
    }
    const float e[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (i + q < n) atomicAdd(&sh[abs_key(e[q]) >> 19], 1u);
  }
  __syncthreads();
  flush_hist(sh, ws);
}

template <int PASS>
__global__ void __launch_bounds__(kSpThreads)
sparse_pass_kernel(const float* __restrict__ a, uint64_t n, uint32_t k,
                   uint32_t* __restrict__ ws) {
  __shared__ uint32_t sh[kBins];
  __shared__ FindSmem fs;
  for (int i = threadIdx.x; i < kBins; i += kSpThreads) sh[i] = 0;
  uint32_t bin0, k1, bin1 = 0, k2;
  find_bin(ws, k, fs, bin0, k1);
  if (PASS == 2) find_bin(ws + kBins, k1, fs, bin1, k2);
  const uint32_t prefix = PASS == 1 ? bin0 : ((bin0 << 11) | bin1);
  const int shift = PASS == 1 ? 19 : 8;
  const bool vec = (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  const uint64_t stride = (uint64_t)gridDim.x * kSpThreads * 4;
  for (uint64_t i = ((uint64_t)blockIdx.x * kSpThreads + threadIdx.x) * 4; i < n; i += stride) {
    const float4 av = ld4(a, i, n, vec);
    const float e[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t key = abs_key(e[q]);
      if (i + q < n && (key >> shift) == prefix) atomicAdd(&sh[digit_of(key, PASS)], 1u);
    }
  }
  __syncthreads();
  flush_hist(sh, ws + PASS * kBins);
}

struct EmitSmem {
  uint32_t warp_tot[kSpThreads / 32];
  uint32_t base_gt;
  uint32_t base_eq;
  uint32_t tot;
};

// Compaction.  Tile = 4096 elements per CTA iteration, 16 per thread.
__global__ void __launch_bounds__(kSpThreads)
sparse_emit_kernel(int alg, float* __restrict__ a, float* __restrict__ u, uint64_t n, uint32_t k,
                   uint32_t kmax, uint8_t* __restrict__ out, uint32_t* __restrict__ ws) {
  __shared__ FindSmem fs;
  __shared__ EmitSmem es;
  uint32_t bin0, k1, bin1, k2, bin2, need_eq;
  find_bin(ws, k, fs, bin0, k1);
  find_bin(ws + kBins, k1, fs, bin1, k2);
  find_bin(ws + 2 * kBins, k2, fs, bin2, need_eq);
  const uint32_t thr = (bin0 << 19) | (bin1 << 8) | bin2;
  if (thr == 0) need_eq = 0;  // zeros are never sent
  uint32_t* idx_out = reinterpret_cast<uint32_t*>(out + 16);
  float* val_out = reinterpret_cast<float*>(out + 16 + align_up(4ull * kmax, 16));
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const uint64_t tiles = (n + 4095) / 4096;
  for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    float e[16];
    uint32_t flag = 0;  // 2 bits per element: bit0 greater, bit1 equal
    uint32_t cnt = 0;   // low 16: greater, high 16: equal
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
      const float4 av = ld4(a, i, n, vec);
      e[4 * j] = av.x; e[4 * j + 1] = av.y; e[4 * j + 2] = av.z; e[4 * j + 3] = av.w;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t key = abs_key(e[4 * j + q]);
        if (i + q < n) {
          if (key > thr) { flag |= 1u << (2 * (4 * j + q)); cnt += 1u; }
          else if (key == thr && need_eq) { flag |= 2u << (2 * (4 * j + q)); cnt += 1u << 16; }
        }
      }
    }
    // block exclusive scan of the packed counts
    uint32_t inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += y;
    }
    if (lane == 31) es.warp_tot[warp] = inc;
    __syncthreads();
    uint32_t wbase = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kSpThreads / 32; ++w) {
      const uint32_t wt = es.warp_tot[w];
      if (w < warp) wbase += wt;
      tot += wt;
    }
    const uint32_t excl = wbase + inc - cnt;
    if (tot == 0) {       // uniform across the CTA
      __syncthreads();
      continue;
    }
    const uint32_t tot_gt = tot & 0xFFFFu, tot_eq = tot >> 16;
    if (threadIdx.x == 0) {
      uint32_t acc_eq = 0, beq = 0;
      if (tot_eq) {
        beq = atomicAdd(ws + kWsTieCount, tot_eq);
        acc_eq = beq >= need_eq ? 0u : min(tot_eq, need_eq - beq);
      }
      es.base_eq = acc_eq;  // number of ties this tile may send
      es.base_gt = (tot_gt + acc_eq) ? atomicAdd(ws + kWsOutCount, tot_gt + acc_eq) : 0u;
    }
    __syncthreads();
    const uint32_t base = es.base_gt, acc_eq = es.base_eq;
    uint32_t pg = base + (excl & 0xFFFFu);             // next slot for a "greater" element
    uint32_t rank_eq = excl >> 16;                     // tie rank inside this tile
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t f = (flag >> (2 * (4 * j + q))) & 3u;
        uint32_t pos = 0xFFFFFFFFu;
        if (f & 1u) pos = pg++;
        else if (f & 2u) {
          if (rank_eq < acc_eq) pos = base + tot_gt + rank_eq;
          ++rank_eq;
        }
        if (pos < kmax) {
          idx_out[pos] = (uint32_t)(i + q);
          val_out[pos] = e[4 * j + q];
          a[i + q] = 0.0f;
          if (u) u[i + q] = 0.0f;
        }
      }
    }
    __syncthreads();
  }
  // last CTA writes the header
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(ws + kWsDone, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      const uint32_t sent = atomicAdd(ws + kWsOutCount, 0u);
      WireHeader h;
      h.n = (uint32_t)n;
      h.alg = (uint8_t)alg;
      h.bitwidth = 0;
      h.flags = 0;
      h.a = __uint_as_float(thr);
      h.b = sent < kmax ? sent : kmax;
      *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(&h);
    }
  }
}

// out[idx] (+)= val * scale ; indices come from another rank: bounds-checked
__global__ void __launch_bounds__(kSpThreads)
sparse_scatter_kernel(const uint8_t* __restrict__ payload, float* __restrict__ out, uint64_t n,
                      uint32_t kmax, float scale, int accumulate) {
  const WireHeader* h = reinterpret_cast<const WireHeader*>(payload);
  uint32_t k = h->b;
  if (k > kmax) k = kmax;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 16);
  const float* val = reinterpret_cast<const float*>(payload + 16 + align_up(4ull * kmax, 16));
  for (uint32_t j = blockIdx.x * kSpThreads + threadIdx.x; j < k; j += gridDim.x * kSpThreads) {
    const uint32_t i = __ldcg(idx + j);
    const float d = __ldcg(val + j) * scale;
    if (i < n) out[i] = accumulate ? out[i] + d : d;
  }
}

}  // namespace hipress

using namespace hipress;

extern "C" {

uint64_t hp_sparse_workspace_bytes() { return (uint64_t)kWsWords * 4; }

static int sparse_encode_impl(int alg, const float* g, float* a, float* u, uint64_t n, uint64_t k,
                              uint64_t kmax, float momentum, int update, uint8_t* out,
                              uint32_t* ws, int max_ctas, cudaStream_t st) {
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
  sparse_pass_kernel<1><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
  sparse_pass_kernel<2><<<grid, kSpThreads, 0, st>>>(a, n, (uint32_t)k, ws);
  sparse_emit_kernel<<<grid, kSpThreads, 0, st>>>(alg, a, alg == kDgc ? u : nullptr, n,
                                                   (uint32_t)k, (uint32_t)kmax, out, ws);
  return (int)cudaGetLastError();
}

// a: accumulator (DGC v / GradDrop residual).  update=1 applies the state update
// with g first; update=0 selects from a as it is (server / ring re-selection).
int hp_cuda_sparse_encode(int alg, const float* g, float* a, float* u, uint64_t n, uint64_t k,
                          uint64_t kmax, float momentum, int update, uint8_t* out, void* workspace,
                          int max_ctas, void* stream) {
  return sparse_encode_impl(alg, g, a, u, n, k, kmax, momentum, update, out,
                            static_cast<uint32_t*>(workspace), max_ctas, (cudaStream_t)stream);
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
                            max_ctas, (cudaStream_t)stream);
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
