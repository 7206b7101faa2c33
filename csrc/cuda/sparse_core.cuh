// Device code of the top-k (DGC / GradDrop) compressor, shared by the
// stand-alone kernels (sparse_ops.cu) and the fused parameter-server kernels
// (fused_sparse.cu): radix-histogram passes, threshold search, block-aggregated
// compaction and scatter.  `cta` / `nctas` say which share of the work the calling
// CTA takes, so one launch can serve many (tensor, chunk) units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "hipress/capi.h"
#include "hipress/common.h"

namespace hipress {

constexpr int kSpThreads = 256;
constexpr int kBins = 4096;
// workspace words: 3 histograms, then counters
constexpr int kWsOutCount = 3 * kBins + 0;
constexpr int kWsTieCount = 3 * kBins + 1;
constexpr int kWsDone = 3 * kBins + 2;
constexpr int kWsCandCount = 3 * kBins + 3;  // candidates appended by the split pass
constexpr int kWsOverflow = 3 * kBins + 4;   // candidate list did not fit: use the full passes
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
static __device__ __noinline__ void find_bin(const uint32_t* __restrict__ hist, uint32_t k,
                                         FindSmem& fs, uint32_t& bin, uint32_t& krem) {
  constexpr int per = kBins / kSpThreads;  // 16
  uint32_t c[per];
  uint32_t sum = 0;
#pragma unroll
  for (int i = 0; i < per; ++i) {
    c[i] = __ldcg(hist + threadIdx.x * per + i);  // written by other CTAs' atomics: read at L2
    sum += c[i];
  }
  // above = how many elements sit in the bins of higher threads: suffix sum by warp
  // shuffles plus the warps' totals (a serial walk over the 256 partial sums cost
  // several microseconds per call, and a selection makes six calls)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t v = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t y = __shfl_down_sync(0xffffffffu, v, o);
    if (lane + o < 32) v += y;
  }
  if (lane == 0) fs.sums[warp] = v;
  if (threadIdx.x == 0) {
    fs.res[0] = 0;
    fs.res[1] = 0;
  }
  __syncthreads();
  uint32_t above = v - sum;
#pragma unroll
  for (int w = 0; w < kSpThreads / 32; ++w)
    if (w > warp) above += fs.sums[w];
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
static __device__ __noinline__ void pass0_body(const float* __restrict__ g, float* __restrict__ a,
                                           float* __restrict__ u, uint64_t n, float momentum,
                                           uint32_t* __restrict__ ws, uint32_t* sh, uint32_t cta,
                                           uint32_t nctas) {
  for (int i = threadIdx.x; i < kBins; i += kSpThreads) sh[i] = 0;
  __syncthreads();
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g) |
                     reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  const uint64_t stride = (uint64_t)nctas * kSpThreads * 4;
  for (uint64_t i = ((uint64_t)cta * kSpThreads + threadIdx.x) * 4; i < n; i += stride) {
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

// One copy of the code for both digit passes (PASS is a run-time value) and one per
// body below: the persistent kernels call every body from several phases, and inlined
// copies made them so large that cold instruction fetches showed in the phase times.
static __device__ __noinline__ void pass_body_rt(int PASS, const float* __restrict__ a, uint64_t n,
                                          uint32_t k, uint32_t* __restrict__ ws, uint32_t* sh,
                                          FindSmem& fs, uint32_t cta, uint32_t nctas) {
  for (int i = threadIdx.x; i < kBins; i += kSpThreads) sh[i] = 0;
  uint32_t bin0, k1, bin1 = 0, k2;
  find_bin(ws, k, fs, bin0, k1);
  if (PASS == 2) find_bin(ws + kBins, k1, fs, bin1, k2);
  const uint32_t prefix = PASS == 1 ? bin0 : ((bin0 << 11) | bin1);
  const int shift = PASS == 1 ? 19 : 8;
  const bool vec = (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  // 4096-element tiles, four independent 16-byte loads per thread in flight
  const uint64_t tiles = (n + 4095) / 4096;
  for (uint64_t t = cta; t < tiles; t += nctas) {
    float4 av[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      av[j] = ld4(a, t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4, n, vec);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
      const float e[4] = {av[j].x, av[j].y, av[j].z, av[j].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t key = abs_key(e[q]);
        if (i + q < n && (key >> shift) == prefix) atomicAdd(&sh[digit_of(key, PASS)], 1u);
      }
    }
  }
  __syncthreads();
  flush_hist(sh, ws + PASS * kBins);
}
template <int PASS>
__device__ __forceinline__ void pass_body(const float* __restrict__ a, uint64_t n, uint32_t k,
                                          uint32_t* __restrict__ ws, uint32_t* sh, FindSmem& fs,
                                          uint32_t cta, uint32_t nctas) {
  pass_body_rt(PASS, a, n, k, ws, sh, fs, cta, nctas);
}

struct EmitSmem {
  uint32_t warp_tot[kSpThreads / 32];
  uint32_t base_gt;
  uint32_t base_eq;
  uint32_t tot;
};

// where the pairs go: one payload per destination (several for a broadcast);
// destinations may be peer GPUs' memory
struct EmitDst {
  uint8_t* out[HP_MAX_RANKS];
  int n;
};

// Compaction.  Tile = 4096 elements per CTA iteration, 16 per thread.  Returns
// true in thread 0 of the CTA that finished last, after it wrote the headers.
// With `remap` the scanned array `a` is a compacted candidate list: element i stands
// for element remap[i] of the accumulator a_orig (and of u), which is what gets
// reported and zeroed.
static __device__ __noinline__ bool emit_body(int alg, float* __restrict__ a, float* __restrict__ u,
                                          uint64_t n, uint32_t k, uint32_t kmax, const EmitDst& dst,
                                          uint32_t* __restrict__ ws, FindSmem& fs, EmitSmem& es,
                                          uint32_t cta, uint32_t nctas,
                                          const uint32_t* __restrict__ remap = nullptr,
                                          float* __restrict__ a_orig = nullptr,
                                          uint32_t n_orig = 0) {
  uint32_t bin0, k1, bin1, k2, bin2, need_eq;
  find_bin(ws, k, fs, bin0, k1);
  find_bin(ws + kBins, k1, fs, bin1, k2);
  find_bin(ws + 2 * kBins, k2, fs, bin2, need_eq);
  const uint32_t thr = (bin0 << 19) | (bin1 << 8) | bin2;
  if (thr == 0) need_eq = 0;  // zeros are never sent
  const size_t val_off = 16 + align_up(4ull * kmax, 16);
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const uint64_t tiles = (n + 4095) / 4096;
  for (uint64_t t = cta; t < tiles; t += nctas) {
    // The loops over a thread's 16 elements stay rolled (and the second one loads the
    // values again, from cache) on purpose: this body runs once or a few times per
    // launch, so its time is instruction fetch, not arithmetic -- fully unrolled it
    // took 13 us per tile, most of it waiting for code.
    uint32_t flag = 0;  // 2 bits per element: bit0 greater, bit1 equal
    uint32_t cnt = 0;   // low 16: greater, high 16: equal
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
      const float4 av = ld4(a, i, n, vec);
      const float e4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t key = abs_key(e4[q]);
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
    const bool rvec = (reinterpret_cast<uintptr_t>(remap) & 15) == 0;
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const uint32_t fj = (flag >> (8 * j)) & 255u;
      if (fj == 0) continue;
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
      const float4 av = ld4(a, i, n, vec);
      const float e4[4] = {av.x, av.y, av.z, av.w};
      uint32_t r4[4] = {0u, 0u, 0u, 0u};
      if (remap) {  // original indices of a candidate list, fetched four at a time
        const float4 rv = ld4(reinterpret_cast<const float*>(remap), i, n, rvec);
        r4[0] = __float_as_uint(rv.x); r4[1] = __float_as_uint(rv.y);
        r4[2] = __float_as_uint(rv.z); r4[3] = __float_as_uint(rv.w);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t f = (fj >> (2 * q)) & 3u;
        uint32_t pos = 0xFFFFFFFFu;
        if (f & 1u) pos = pg++;
        else if (f & 2u) {
          if (rank_eq < acc_eq) pos = base + tot_gt + rank_eq;
          ++rank_eq;
        }
        if (pos < kmax) {
          uint32_t where = remap ? r4[q] : (uint32_t)(i + q);
          if (remap && where >= n_orig) where = 0;  // never index outside the accumulator
          for (int d = 0; d < dst.n; ++d) {
            reinterpret_cast<uint32_t*>(dst.out[d] + 16)[pos] = where;
            reinterpret_cast<float*>(dst.out[d] + val_off)[pos] = e4[q];
          }
          if (remap) a_orig[where] = 0.0f;
          else a[i + q] = 0.0f;
          if (u) u[where] = 0.0f;
        }
      }
    }
    __syncthreads();
  }
  // last CTA writes the header
  __syncthreads();
  if (threadIdx.x == 0) {
    // device scope is enough here: the one thread that finds itself last publishes
    // the unit (header, then a system-scope release of the flag by the caller), and
    // release is cumulative over what it has observed through this counter
    __threadfence();
    const uint32_t ticket = atomicAdd(ws + kWsDone, 1u);
    if (ticket == nctas - 1) {
      __threadfence();
      const uint32_t sent = atomicAdd(ws + kWsOutCount, 0u);
      WireHeader h;
      h.n = remap ? n_orig : (uint32_t)n;  // always the length of the accumulator
      h.alg = (uint8_t)alg;
      h.bitwidth = 0;
      h.flags = 0;
      h.a = __uint_as_float(thr);
      h.b = sent < kmax ? sent : kmax;
      for (int d = 0; d < dst.n; ++d)
        *reinterpret_cast<uint4*>(dst.out[d]) = *reinterpret_cast<const uint4*>(&h);
      return true;
    }
  }
  return false;
}

// Split pass (after pass 0): everything above the threshold's 12-bit bin is
// certainly among the k largest and is sent and zeroed at once; the elements of
// that bin go to a compact candidate list (value + original index) on which the
// remaining two digit passes and the final compaction run.  One pass over the
// array instead of three.  A candidate list that does not fit raises the
// overflow word and the full-array passes take over.
constexpr int kSplitBuf = 1024;  // pairs a CTA collects in shared memory per list

struct SplitSmem {
  float sel_val[kSplitBuf];
  uint32_t sel_idx[kSplitBuf];
  float cnd_val[kSplitBuf];
  uint32_t cnd_idx[kSplitBuf];
  uint32_t nsel, ncnd, base_sel, base_cnd;
};

// Selected elements are rare (about 0.1 % of the array), so a CTA collects its
// finds in shared memory with plain shared atomics -- no block scan, no barrier
// per tile -- and reserves its slice of the global lists once at the end.  Finds
// beyond the shared buffer go to the global lists one by one.
static __device__ __noinline__ void split_body(float* __restrict__ a, float* __restrict__ u, uint64_t n,
                                           uint32_t k, uint32_t kmax, const EmitDst& dst,
                                           uint32_t* __restrict__ ws, float* __restrict__ cand_val,
                                           uint32_t* __restrict__ cand_idx, uint32_t cand_cap,
                                           FindSmem& fs, SplitSmem& sp, uint32_t cta, uint32_t nctas) {
  uint32_t bin0, k1;
  if (threadIdx.x == 0) {
    sp.nsel = 0;
    sp.ncnd = 0;
  }
  find_bin(ws, k, fs, bin0, k1);  // contains the barriers that publish nsel / ncnd
  const size_t val_off = 16 + align_up(4ull * kmax, 16);
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  const uint64_t tiles = (n + 4095) / 4096;
  for (uint64_t t = cta; t < tiles; t += nctas) {
    float4 av[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      av[j] = ld4(a, t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4, n, vec);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t i = t * 4096 + (uint64_t)(j * kSpThreads + threadIdx.x) * 4;
      const float e[4] = {av[j].x, av[j].y, av[j].z, av[j].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t bin = abs_key(e[q]) >> 19;
        if (i + q >= n || bin < bin0) continue;
        if (bin > bin0) {  // certainly among the k largest: send and zero now
          const uint32_t p = atomicAdd(&sp.nsel, 1u);
          if (p < (uint32_t)kSplitBuf) {
            sp.sel_val[p] = e[q];
            sp.sel_idx[p] = (uint32_t)(i + q);
          } else {
            const uint32_t pos = atomicAdd(ws + kWsOutCount, 1u);
            if (pos < kmax)
              for (int d = 0; d < dst.n; ++d) {
                reinterpret_cast<uint32_t*>(dst.out[d] + 16)[pos] = (uint32_t)(i + q);
                reinterpret_cast<float*>(dst.out[d] + val_off)[pos] = e[q];
              }
          }
          a[i + q] = 0.0f;
          if (u) u[i + q] = 0.0f;
        } else {           // inside the threshold bin: decided on the candidate list
          const uint32_t p = atomicAdd(&sp.ncnd, 1u);
          if (p < (uint32_t)kSplitBuf) {
            sp.cnd_val[p] = e[q];
            sp.cnd_idx[p] = (uint32_t)(i + q);
          } else {
            const uint32_t pos = atomicAdd(ws + kWsCandCount, 1u);
            if (pos < cand_cap) {
              cand_val[pos] = e[q];
              cand_idx[pos] = (uint32_t)(i + q);
            } else {
              ws[kWsOverflow] = 1u;
            }
          }
        }
      }
    }
  }
  __syncthreads();
  const uint32_t nsel = min(sp.nsel, (uint32_t)kSplitBuf), ncnd = min(sp.ncnd, (uint32_t)kSplitBuf);
  if (threadIdx.x == 0) {
    sp.base_sel = nsel ? atomicAdd(ws + kWsOutCount, nsel) : 0u;
    sp.base_cnd = ncnd ? atomicAdd(ws + kWsCandCount, ncnd) : 0u;
    if (ncnd && sp.base_cnd + ncnd > cand_cap) ws[kWsOverflow] = 1u;
  }
  __syncthreads();
  for (uint32_t p = threadIdx.x; p < nsel; p += kSpThreads) {
    const uint32_t pos = sp.base_sel + p;
    if (pos < kmax)
      for (int d = 0; d < dst.n; ++d) {
        reinterpret_cast<uint32_t*>(dst.out[d] + 16)[pos] = sp.sel_idx[p];
        reinterpret_cast<float*>(dst.out[d] + val_off)[pos] = sp.sel_val[p];
      }
  }
  for (uint32_t p = threadIdx.x; p < ncnd; p += kSpThreads) {
    const uint32_t pos = sp.base_cnd + p;
    if (pos < cand_cap) {
      cand_val[pos] = sp.cnd_val[p];
      cand_idx[pos] = sp.cnd_idx[p];
    }
  }
}

// out[idx] (+)= val * scale ; indices come from another rank: bounds-checked
static __device__ __noinline__ void scatter_body(const uint8_t* __restrict__ payload,
                                             float* __restrict__ out, uint64_t n, uint32_t kmax,
                                             float scale, int accumulate, uint32_t cta,
                                             uint32_t nctas) {
  const WireHeader* h = reinterpret_cast<const WireHeader*>(payload);
  uint32_t k = __ldcg(&h->b);
  if (k > kmax) k = kmax;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 16);
  const float* val = reinterpret_cast<const float*>(payload + 16 + align_up(4ull * kmax, 16));
  for (uint32_t j = cta * kSpThreads + threadIdx.x; j < k; j += nctas * kSpThreads) {
    const uint32_t i = __ldcg(idx + j);
    const float d = __ldcg(val + j) * scale;
    if (i < n) {
      if (accumulate == 2) atomicAdd(out + i, d);  // several payloads may hit one index
      else out[i] = accumulate ? out[i] + d : d;
    }
  }
}

}  // namespace hipress
