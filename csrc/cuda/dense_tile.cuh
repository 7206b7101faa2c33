// Tile-level device code shared by the stand-alone encode/decode kernels and by
// the fused ring / parameter-server kernels.
//
// A tile is kTile (4096) consecutive fp32 elements handled by one 256-thread
// CTA: every thread keeps 16 elements in registers (four float4 at float4-index
// j*256+tid), so the residual add, the per-tile scale or min/max reduction, the
// quantisation and the residual write-back all happen on one pass over HBM
// (12 B/element with error feedback, 4 B/element without).  The reference does
// this with two synchronising thrust::reduce calls, a thrust::transform with
// one thread per output byte and four host memcpys per tensor
// (src/CompLL/GCGen/output/TernGradEncode/TernGradEncode_body.h:115-123).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "hipress/common.h"

namespace hipress {

constexpr int kThreads = 256;
constexpr int kIter = kTile / (kThreads * 4);  // float4 per thread per tile
static_assert(kIter * kThreads * 4 == kTile, "tile must split evenly");

struct TileSmem {
  alignas(16) uint8_t codes[kTile];  // staged code bytes, up to 8 bits/element
  double red_d[kThreads / 32];
  float red_a[kThreads / 32];
  float red_b[kThreads / 32];
};

// ------------------------------------------------------------------ memory ops
__device__ __forceinline__ void load_tile(const float* __restrict__ p, int m,
                                          float (&x)[kIter][4]) {
  const bool vec = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    const int i0 = 4 * (j * kThreads + (int)threadIdx.x);
    if (vec && i0 + 3 < m) {
      const float4 v = *reinterpret_cast<const float4*>(p + i0);
      x[j][0] = v.x; x[j][1] = v.y; x[j][2] = v.z; x[j][3] = v.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) x[j][e] = (i0 + e < m) ? p[i0 + e] : 0.0f;
    }
  }
}

__device__ __forceinline__ void store_tile(float* __restrict__ p, int m,
                                           const float (&x)[kIter][4]) {
  const bool vec = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    const int i0 = 4 * (j * kThreads + (int)threadIdx.x);
    if (vec && i0 + 3 < m) {
      *reinterpret_cast<float4*>(p + i0) = make_float4(x[j][0], x[j][1], x[j][2], x[j][3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i0 + e < m) p[i0 + e] = x[j][e];
    }
  }
}

// a full tile at a 16-byte aligned address: no per-element checks
__device__ __forceinline__ void store_tile_full(float* __restrict__ p, const float (&x)[kIter][4]) {
#pragma unroll
  for (int j = 0; j < kIter; ++j)
    reinterpret_cast<float4*>(p)[j * kThreads + (int)threadIdx.x] =
        make_float4(x[j][0], x[j][1], x[j][2], x[j][3]);
}
__device__ __forceinline__ bool tile_is_full_aligned(const float* p, int m) {
  return m == kTile && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// Code fragment = the 4*B bits of the four elements of one float4.
// Payload bytes that another GPU wrote are read with ld.global.cg (L2 only).
template <int B>
__device__ __forceinline__ uint32_t load_frag(const uint8_t* __restrict__ codes, int j, int m) {
  const int f = j * kThreads + (int)threadIdx.x;
  if (4 * f >= m) return 0u;
  if (B == 1) {
    const uint32_t b = __ldcg(codes + (f >> 1));
    return (f & 1) ? (b >> 4) : (b & 15u);
  } else if (B == 2) {
    return __ldcg(codes + f);
  } else if (B == 4) {
    return __ldcg(reinterpret_cast<const unsigned short*>(codes) + f);
  } else {
    return __ldcg(reinterpret_cast<const unsigned int*>(codes) + f);
  }
}

template <int B>
__device__ __forceinline__ void stage_frags(uint8_t* sc, const uint32_t (&frag)[kIter]) {
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    const int f = j * kThreads + (int)threadIdx.x;
    if (B == 1) {
      const uint32_t hi = __shfl_down_sync(0xffffffffu, frag[j], 1);
      if (!(threadIdx.x & 1)) sc[f >> 1] = (uint8_t)(frag[j] | (hi << 4));
    } else if (B == 2) {
      sc[f] = (uint8_t)frag[j];
    } else if (B == 4) {
      reinterpret_cast<uint16_t*>(sc)[f] = (uint16_t)frag[j];
    } else {
      reinterpret_cast<uint32_t*>(sc)[f] = frag[j];
    }
  }
}

__device__ __forceinline__ int tile_code_bytes(int m, int bits) {
  return (int)align_up(((uint64_t)m * bits + 7) / 8, 16);
}

// 16-byte stores; dst may be a peer GPU's memory (plain st.global over NVLink).
__device__ __forceinline__ void copy_codes(uint8_t* __restrict__ dst, const uint8_t* sc,
                                           int nbytes) {
  for (int o = (int)threadIdx.x * 16; o < nbytes; o += kThreads * 16)
    *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(sc + o);
}

// ------------------------------------------------------------- block reductions
// All 256 threads must call; every thread returns the same value.
__device__ __forceinline__ double block_sum(double v, TileSmem& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) s.red_d[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) t += s.red_d[w];
  __syncthreads();
  return t;
}

// Warp level: one redux.sync.{min,max}.f32 each (the fp32 forms of the warp
// reduction are sm_100a instructions) instead of five shuffle + compare rounds.
__device__ __forceinline__ void block_minmax(float& mn, float& mx, TileSmem& s) {
  asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(mn) : "f"(mn));
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(mx) : "f"(mx));
  if ((threadIdx.x & 31) == 0) {
    s.red_a[threadIdx.x >> 5] = mn;
    s.red_b[threadIdx.x >> 5] = mx;
  }
  __syncthreads();
  mn = s.red_a[0];
  mx = s.red_b[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) {
    mn = fminf(mn, s.red_a[w]);
    mx = fmaxf(mx, s.red_b[w]);
  }
  __syncthreads();
}

// ------------------------------------------------------------------ algorithms
// decode the four elements of fragment j into d[0..3]
template <int ALG, int B>
__device__ __forceinline__ void decode_frag(uint32_t frag, const float (&meta)[2], float tau,
                                            float (&d)[4]) {
  constexpr uint32_t mask = (1u << B) - 1u;
  float gap = 0.0f;
  if (ALG == kTernGrad) gap = tern_gap(meta[0], meta[1], B);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (ALG == kTbq) {
      // tbq_value of the 2-bit code at bits 2e, 2e+1 by testing the bits in place
      // (bit 1: non-zero level, bit 0: positive)
      const bool nz = (frag & (2u << (e * B))) != 0u, pos = (frag & (1u << (e * B))) != 0u;
      d[e] = nz ? (pos ? tau : -tau) : 0.0f;
    } else {
      const uint32_t c = (frag >> (e * B)) & mask;
      if (ALG == kOnebit) d[e] = onebit_value(c, meta[0]);
      else d[e] = tern_value(c, meta[0], gap);
    }
  }
}

// Quantise the register tile x (m valid elements).  On return frag[] holds the
// code fragments (zero for elements past m), meta[] the tile metadata, and x the
// quantisation error x - decode(code) of every valid element (left untouched by
// TernGrad when the caller keeps no residual: want_err = false).
template <int ALG, int B, bool FULL, bool ERR>
__device__ __forceinline__ void encode_tile_impl(float (&x)[kIter][4], int m, const DenseParams& P,
                                                 uint32_t tensor_id, uint64_t elem0, uint32_t salt,
                                                 TileSmem& s, float (&meta)[2],
                                                 uint32_t (&frag)[kIter]) {
  meta[0] = 0.0f;
  meta[1] = 0.0f;
  if (ALG == kOnebit) {
    double part = 0.0;
#pragma unroll
    for (int j = 0; j < kIter; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (FULL || 4 * (j * kThreads + (int)threadIdx.x) + e < m) part += (double)fabsf(x[j][e]);
    const double tot = block_sum(part, s);
    meta[0] = (float)(tot / (double)m);
  } else if (ALG == kTernGrad) {
    float mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kIter; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (FULL || 4 * (j * kThreads + (int)threadIdx.x) + e < m) {
          mn = fminf(mn, x[j][e]);
          mx = fmaxf(mx, x[j][e]);
        }
    block_minmax(mn, mx, s);
    meta[0] = mn;
    meta[1] = mx;
  }
  float gap = 0.0f, scale16 = 0.0f;
  if (ALG == kTernGrad) {
    gap = tern_gap(meta[0], meta[1], B);
    scale16 = tern_scale16(gap);
  }
  // TernGrad: one Philox call per pair of rows (see rnd16_counter); a tile that does
  // not start on a 2048-element boundary of its tensor cannot share calls
  const bool paired = ALG != kTernGrad || (elem0 & 2047u) == 0;
  Philox4 rnd;
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    const int i0 = 4 * (j * kThreads + (int)threadIdx.x);
    uint32_t half = 0u;
    if (ALG == kTernGrad) {
      const uint64_t ge = elem0 + (uint64_t)i0;
      half = paired ? (uint32_t)(j & 1) : rnd16_half(ge);
      if (!paired || !(j & 1))
        rnd = philox4x32(rnd16_counter(ge), tensor_id, P.step, salt, P.seed_lo, P.seed_hi);
    }
    uint32_t f = 0u;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (FULL || i0 + e < m) {
        uint32_t c;
        float d;
        if (ALG == kOnebit) {
          c = onebit_code(x[j][e]);
          d = onebit_value(c, meta[0]);
        } else if (ALG == kTbq) {
          // tbq_code and tbq_value of it from one pair of compares
          const bool pos = x[j][e] >= P.tau, neg = x[j][e] <= -P.tau;
          c = pos ? 3u : (neg ? 2u : 0u);
          d = pos ? P.tau : (neg ? -P.tau : 0.0f);
        } else {
          c = tern_code(x[j][e], meta[0], scale16, rnd16(rnd.v[e], half), B);
          d = ERR ? tern_value(c, meta[0], gap) : 0.0f;
        }
        f |= c << (e * B);
        if (ERR) x[j][e] = x[j][e] - d;
      }
    }
    frag[j] = f;
  }
}

template <int ALG, int B>
__device__ __forceinline__ void encode_tile(float (&x)[kIter][4], int m, const DenseParams& P,
                                            uint32_t tensor_id, uint64_t elem0, uint32_t salt,
                                            TileSmem& s, float (&meta)[2],
                                            uint32_t (&frag)[kIter], bool want_err = true) {
  if (ALG == kTernGrad && !want_err) {
    if (m == kTile) encode_tile_impl<ALG, B, true, false>(x, m, P, tensor_id, elem0, salt, s, meta, frag);
    else encode_tile_impl<ALG, B, false, false>(x, m, P, tensor_id, elem0, salt, s, meta, frag);
  } else {
    if (m == kTile) encode_tile_impl<ALG, B, true, true>(x, m, P, tensor_id, elem0, salt, s, meta, frag);
    else encode_tile_impl<ALG, B, false, true>(x, m, P, tensor_id, elem0, salt, s, meta, frag);
  }
}

// Byte layout of one dense payload of `n_layout` elements (n_layout fixes where
// the code region starts; fewer elements may actually be valid).
struct PayloadView {
  uint8_t* base;
  float* meta;
  uint8_t* codes;
};
__device__ __forceinline__ PayloadView payload_view(uint8_t* base, int alg, uint64_t n_layout) {
  PayloadView v;
  v.base = base;
  v.meta = reinterpret_cast<float*>(base + 16);
  v.codes = base + 16 + dense_meta_bytes(alg, n_layout);
  return v;
}

__device__ __forceinline__ void write_header(uint8_t* base, uint32_t n, int alg, int bits,
                                             float tau) {
  WireHeader h;
  h.n = n;
  h.alg = (uint8_t)alg;
  h.bitwidth = (uint8_t)bits;
  h.flags = dense_meta_floats(alg) ? 1 : 0;
  h.a = alg == kTbq ? tau : 0.0f;
  h.b = kTile;
  *reinterpret_cast<uint4*>(base) = *reinterpret_cast<const uint4*>(&h);
}

// read tile metadata that may have been written by a peer
template <int ALG>
__device__ __forceinline__ void load_meta(const float* meta, uint32_t t, float (&m)[2]) {
  m[0] = 0.0f;
  m[1] = 0.0f;
  if (ALG == kOnebit) m[0] = __ldcg(meta + t);
  if (ALG == kTernGrad) {
    m[0] = __ldcg(meta + 2 * t);
    m[1] = __ldcg(meta + 2 * t + 1);
  }
}

}  // namespace hipress
