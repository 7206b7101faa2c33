// Stand-alone dense (quantising) compression ops for onebit, TBQ and TernGrad:
// one encode kernel (optionally merging an incoming payload, the ring "recv ->
// decode -> merge -> encode" chain of CaSync) and one decode / decode-accumulate
// kernel.  They are the building blocks of the unfused baseline and the public
// per-tensor API; the fused ring / PS kernels reuse the same tile code.
//
// Reference parity: op pair Encode(gradient, compressed, params) /
// Decode(compressed, gradient), in place, caller-allocated buffers
// (src/CompLL/GCGen/output/TernGradEncode/TernGradEncode.cc:10-24).
#include "dense_tile.cuh"
#include "hipress/capi.h"

namespace hipress {

template <int ALG, int B>
__global__ void __launch_bounds__(kThreads, 4)
dense_encode_kernel(const float* __restrict__ g, float* __restrict__ r,
                    const uint8_t* __restrict__ in_payload, uint8_t* __restrict__ out,
                    uint32_t n, DenseParams P, uint32_t tensor_id, uint64_t elem_offset) {
  __shared__ TileSmem s;
  const uint32_t tiles = (uint32_t)num_tiles(n);
  PayloadView ov = payload_view(out, ALG, n);
  PayloadView iv = payload_view(const_cast<uint8_t*>(in_payload), ALG, n);
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) write_header(out, n, ALG, B, P.tau);
    // zero the padding behind the tile metadata so payload bytes are deterministic
    const uint32_t used = tiles * dense_meta_floats(ALG);
    const uint32_t padded = (uint32_t)(dense_meta_bytes(ALG, n) / 4);
    for (uint32_t i = used + threadIdx.x; i < padded; i += kThreads) ov.meta[i] = 0.0f;
  }
  for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const uint32_t start = t * kTile;
    const int m = (int)min((uint32_t)kTile, n - start);
    float x[kIter][4];
    load_tile(g + start, m, x);
    if (in_payload) {
      float im[2];
      load_meta<ALG>(iv.meta, t, im);
      const uint8_t* ic = iv.codes + (size_t)t * (kTile * B / 8);
#pragma unroll
      for (int j = 0; j < kIter; ++j) {
        float d[4];
        decode_frag<ALG, B>(load_frag<B>(ic, j, m), im, P.tau, d);
#pragma unroll
        for (int e = 0; e < 4; ++e) x[j][e] = x[j][e] + d[e];
      }
    }
    if (r) {
      float rr[kIter][4];
      load_tile(r + start, m, rr);
#pragma unroll
      for (int j = 0; j < kIter; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) x[j][e] = rr[j][e] + x[j][e];
    }
    float meta[2];
    uint32_t frag[kIter];
    encode_tile<ALG, B>(x, m, P, tensor_id, elem_offset + start, P.salt, s, meta, frag, r != nullptr);
    if (r) store_tile(r + start, m, x);
    stage_frags<B>(s.codes, frag);
    __syncthreads();
    copy_codes(ov.codes + (size_t)t * (kTile * B / 8), s.codes, tile_code_bytes(m, B));
    if (threadIdx.x == 0) {
      if (ALG == kOnebit) ov.meta[t] = meta[0];
      if (ALG == kTernGrad) {
        ov.meta[2 * t] = meta[0];
        ov.meta[2 * t + 1] = meta[1];
      }
    }
    __syncthreads();
  }
}

// Decode is write bound (4 B/element out, bits in).  Each CTA iteration handles
// kDecBatch tiles and issues all their payload loads before the first store, so
// one L2 round trip is exposed per batch instead of per tile.
constexpr int kDecBatch = 4;

template <int ALG, int B>
__global__ void __launch_bounds__(kThreads)
dense_decode_kernel(const uint8_t* __restrict__ payload, float* __restrict__ out, uint32_t n,
                    float tau, float scale, int accumulate) {
  const uint32_t tiles = (uint32_t)num_tiles(n);
  PayloadView pv = payload_view(const_cast<uint8_t*>(payload), ALG, n);
  for (uint32_t t0 = blockIdx.x * kDecBatch; t0 < tiles; t0 += gridDim.x * kDecBatch) {
    uint32_t fr[kDecBatch][kIter];
    float mt[kDecBatch][2];
#pragma unroll
    for (int u = 0; u < kDecBatch; ++u) {
      const uint32_t t = t0 + u;
      if (t < tiles) {
        const int m = (int)min((uint32_t)kTile, n - t * kTile);
        load_meta<ALG>(pv.meta, t, mt[u]);
        const uint8_t* tc = pv.codes + (size_t)t * (kTile * B / 8);
#pragma unroll
        for (int j = 0; j < kIter; ++j) fr[u][j] = load_frag<B>(tc, j, m);
      }
    }
#pragma unroll
    for (int u = 0; u < kDecBatch; ++u) {
      const uint32_t t = t0 + u;
      if (t < tiles) {
        const uint32_t start = t * kTile;
        const int m = (int)min((uint32_t)kTile, n - start);
        float x[kIter][4];
        if (accumulate) load_tile(out + start, m, x);
#pragma unroll
        for (int j = 0; j < kIter; ++j) {
          float d[4];
          decode_frag<ALG, B>(fr[u][j], mt[u], tau, d);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            x[j][e] = accumulate ? x[j][e] + d[e] * scale : d[e] * scale;
        }
        store_tile(out + start, m, x);
      }
    }
  }
}

template <int ALG, int B>
static int launch_encode(const float* g, float* r, const uint8_t* in, uint8_t* out, uint64_t n,
                         const DenseParams& P, uint32_t tensor_id, uint64_t elem_offset,
                         int max_ctas, cudaStream_t st) {
  const uint64_t tiles = num_tiles(n);
  int grid = (int)(tiles < (uint64_t)max_ctas ? tiles : (uint64_t)max_ctas);
  if (grid < 1) grid = 1;
  dense_encode_kernel<ALG, B><<<grid, kThreads, 0, st>>>(g, r, in, out, (uint32_t)n, P,
                                                          tensor_id, elem_offset);
  return (int)cudaGetLastError();
}

template <int ALG, int B>
static int launch_decode(const uint8_t* p, float* out, uint64_t n, float tau, float scale,
                         int acc, int max_ctas, cudaStream_t st) {
  const uint64_t tiles = (num_tiles(n) + kDecBatch - 1) / kDecBatch;
  int grid = (int)(tiles < (uint64_t)max_ctas ? tiles : (uint64_t)max_ctas);
  if (grid < 1) grid = 1;
  dense_decode_kernel<ALG, B><<<grid, kThreads, 0, st>>>(p, out, (uint32_t)n, tau, scale, acc);
  return (int)cudaGetLastError();
}

}  // namespace hipress

using namespace hipress;

#define HP_DISPATCH_DENSE(alg, bits, CALL)                         \
  do {                                                             \
    if (alg == kOnebit && bits == 1) { CALL(kOnebit, 1); }         \
    else if (alg == kTbq && bits == 2) { CALL(kTbq, 2); }          \
    else if (alg == kTernGrad && bits == 1) { CALL(kTernGrad, 1); }\
    else if (alg == kTernGrad && bits == 2) { CALL(kTernGrad, 2); }\
    else if (alg == kTernGrad && bits == 4) { CALL(kTernGrad, 4); }\
    else if (alg == kTernGrad && bits == 8) { CALL(kTernGrad, 8); }\
    else return HP_ERR_BAD_ARG;                                    \
  } while (0)

extern "C" {

int hp_cuda_dense_encode(int alg, int bits, const float* g, float* r, const uint8_t* in_payload,
                         uint8_t* out, uint64_t n, float tau, uint64_t seed, uint32_t step,
                         uint32_t salt, uint32_t tensor_id, uint64_t elem_offset, int max_ctas,
                         void* stream) {
  if (n == 0) return 0;
  if (n > 0xFFFFF000ull || (elem_offset & 3)) return HP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(in_payload) & 15))
    return HP_ERR_BAD_ARG;
  DenseParams P{tau, step, salt, (uint32_t)seed, (uint32_t)(seed >> 32)};
  cudaStream_t st = (cudaStream_t)stream;
  if (max_ctas <= 0) max_ctas = 148 * 8;
#define CALL(A, B) return launch_encode<A, B>(g, r, in_payload, out, n, P, tensor_id, elem_offset, max_ctas, st)
  HP_DISPATCH_DENSE(alg, bits, CALL);
#undef CALL
  return 0;
}

int hp_cuda_dense_decode(int alg, int bits, const uint8_t* payload, float* out, uint64_t n,
                         float tau, float scale, int accumulate, int max_ctas, void* stream) {
  if (n == 0) return 0;
  if (n > 0xFFFFF000ull || (reinterpret_cast<uintptr_t>(payload) & 15)) return HP_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (max_ctas <= 0) max_ctas = 148 * 8;
#define CALL(A, B) return launch_decode<A, B>(payload, out, n, tau, scale, accumulate, max_ctas, st)
  HP_DISPATCH_DENSE(alg, bits, CALL);
#undef CALL
  return 0;
}

}  // extern "C"
