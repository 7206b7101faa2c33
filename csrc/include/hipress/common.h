// Shared host/device definitions: wire formats, per-element compression math and
// the counter-based random generator.  Everything in this header compiles both
// as plain C++ (the CPU oracle) and as CUDA device code, so the two
// implementations quantise identically bit for bit.
//
// Parity notes against the reference (mark14wu/hipress):
//   * the reference's only algorithm source is TernGrad
//     (src/CompLL/GCGen/pse/TernGradEncode.pse, TernGradDecode.pse); its 10-byte
//     unaligned header (output/TernGradEncode/TernGradEncode_body.h:114-123) is
//     replaced by an aligned 16-byte header so payloads can be moved with
//     128-bit loads and stores;
//   * its linear-congruential generator seeded identically in every thread
//     (output/naive_random.hpp:25-67) is replaced by Philox4x32-7 keyed by
//     (seed, element index, tensor id, step, salt).
#pragma once
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define HP_HD __host__ __device__ __forceinline__
#else
#define HP_HD inline
#endif

namespace hipress {

// ---------------------------------------------------------------------------
// Wire format
// ---------------------------------------------------------------------------
constexpr int kTile = 4096;  // elements that share one scale / min-max record

enum Alg : int {
  kOnebit = 1,
  kTbq = 2,
  kTernGrad = 3,
  kDgc = 4,
  kGradDrop = 5,
};

// 16-byte little-endian header in front of every payload.
struct alignas(16) WireHeader {
  uint32_t n;        // number of fp32 elements the payload describes
  uint8_t alg;       // Alg
  uint8_t bitwidth;  // bits per element (dense) or 0 (sparse)
  uint16_t flags;    // bit 0: payload carries per-tile metadata
  float a;           // tbq: threshold; sparse: selection threshold |v|
  uint32_t b;        // sparse: k (number of pairs); dense: tile size
};
static_assert(sizeof(WireHeader) == 16, "header must be 16 bytes");

HP_HD uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
HP_HD uint64_t num_tiles(uint64_t n) { return (n + kTile - 1) / kTile; }

// floats of per-tile metadata
HP_HD int dense_meta_floats(int alg) {
  return alg == kOnebit ? 1 : (alg == kTernGrad ? 2 : 0);
}
HP_HD uint64_t dense_meta_bytes(int alg, uint64_t n) {
  return align_up(num_tiles(n) * dense_meta_floats(alg) * 4, 16);
}
HP_HD uint64_t dense_code_bytes(int bits, uint64_t n) {
  return align_up((n * (uint64_t)bits + 7) / 8, 16);
}
// [header 16][tile metadata][codes]; tile t's codes start at t*kTile*bits/8.
HP_HD uint64_t dense_payload_bytes(int alg, int bits, uint64_t n) {
  return 16 + dense_meta_bytes(alg, n) + dense_code_bytes(bits, n);
}
// sparse payload: [header 16][k x u32 index][k x f32 value], capacity kmax pairs,
// the value array starts at 16 + align16(4*kmax).
HP_HD uint64_t sparse_payload_bytes(uint64_t kmax) {
  return 16 + 2 * align_up(4 * kmax, 16);
}
HP_HD uint64_t sparse_k(uint64_t n, float ratio) {
  if (n == 0) return 0;
  double kd = ceil((double)ratio * (double)n);
  uint64_t k = (uint64_t)kd;
  if (k < 1) k = 1;
  if (k > n) k = n;
  return k;
}

// ---------------------------------------------------------------------------
// Philox4x32 (Salmon et al.), counter based: one call yields four words.  Seven
// rounds (the smaller of the two standard round counts, Crush-resistant per the
// Random123 paper) are enough for stochastic rounding and keep the TernGrad
// encoder closer to the memory roofline than ten.
// ---------------------------------------------------------------------------
struct Philox4 {
  uint32_t v[4];
};

HP_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  uint64_t p = (uint64_t)a * (uint64_t)b;
  hi = (uint32_t)(p >> 32);
  lo = (uint32_t)p;
}

constexpr int kPhiloxRounds = 7;

HP_HD Philox4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                         uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < kPhiloxRounds; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c2, hi1, lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// uniform in [0,1) with 24 bits, exact in fp32 on host and device
HP_HD float u01(uint32_t r) { return (float)(r >> 8) * (1.0f / 16777216.0f); }

// Stochastic rounding draws (TernGrad): 16-bit uniforms, so one Philox call serves
// eight elements -- the four elements of float4 number q = elem >> 2 and of float4
// q + 256, which are two consecutive rows of one thread of a 4096-element tile.  The
// call is keyed by q with bit 8 cleared; float4 q takes the low halves of the four
// words when its bit 8 is clear and the high halves when it is set.  A pure function
// of the element index, so the CPU oracle and every kernel layout draw the same
// numbers.
HP_HD uint32_t rnd16_counter(uint64_t elem) { return (uint32_t)(elem >> 2) & ~256u; }
HP_HD uint32_t rnd16_half(uint64_t elem) { return (uint32_t)(elem >> 10) & 1u; }
HP_HD uint32_t rnd16(uint32_t word, uint32_t half) { return half ? (word >> 16) : (word & 0xFFFFu); }

// ---------------------------------------------------------------------------
// Parameters shared by every dense (quantising) algorithm
// ---------------------------------------------------------------------------
struct DenseParams {
  float tau;       // tbq threshold
  uint32_t step;   // training step, feeds the random counter
  uint32_t salt;   // rank / hop salt, feeds the random counter
  uint32_t seed_lo;
  uint32_t seed_hi;
};

// ---------------------------------------------------------------------------
// Per-element math.  No implicit fused multiply-add: both compilers are run
// with contraction off and fmaf is written out where one rounding is wanted.
// ---------------------------------------------------------------------------

// TBQ / "2bit": 11 -> +tau, 10 -> -tau, 00 -> 0
HP_HD uint32_t tbq_code(float x, float tau) {
  return x >= tau ? 3u : (x <= -tau ? 2u : 0u);
}
HP_HD float tbq_value(uint32_t code, float tau) {
  return code == 3u ? tau : (code == 2u ? -tau : 0.0f);
}

// onebit: bit set when x < 0; decoded as -s / +s
HP_HD uint32_t onebit_code(float x) { return x < 0.0f ? 1u : 0u; }
HP_HD float onebit_value(uint32_t code, float s) { return code ? -s : s; }

// TernGrad generalised to 2^bits levels
HP_HD float tern_gap(float mn, float mx, int bits) {
  return (mx - mn) / (float)((1u << bits) - 1u);
}
// Stochastic rounding in fixed point.  scale16 = 65536 / gap is computed once per
// tile; per element t = floor((x - min) * scale16) is the position in units of
// 2^-16 of a quantisation step, and q = (t + u16) >> 16 with a 16-bit uniform u16
// rounds up with probability frac(t / 65536): unbiased to 2^-16 of a step.  Integer
// adds and shifts replace a floor, two compares and a float conversion per element;
// t < 2^24 for every supported bit width, so the float product is exact enough to
// keep level placement within one step.  The conversion saturates and maps NaN to 0
// on both implementations.
HP_HD float tern_scale16(float gap) { return gap > 0.0f ? 65536.0f / gap : 0.0f; }
HP_HD int32_t f2i_floor_sat(float t) {
#if defined(__CUDA_ARCH__)
  return __float2int_rd(t);
#else
  if (!(t == t)) return 0;
  if (t >= 2147483648.0f) return 2147483647;
  if (t <= -2147483648.0f) return (int32_t)(-2147483647 - 1);
  return (int32_t)floorf(t);
#endif
}
HP_HD uint32_t tern_code(float x, float mn, float scale16, uint32_t u16, int bits) {
  // scale16 == 0 (a constant tile) needs no test of its own: the product is 0 or NaN,
  // both convert to 0, and (0 + u16) >> 16 == 0
  const uint32_t t = (uint32_t)f2i_floor_sat((x - mn) * scale16);
  const uint32_t q = (t + u16) >> 16;
  const uint32_t qmax = (1u << bits) - 1u;
  return q > qmax ? qmax : q;
}
HP_HD float tern_value(uint32_t q, float mn, float gap) {
  return fmaf((float)q, gap, mn);
}

// Order-preserving map of |x| to an unsigned key (bigger magnitude, bigger key).
HP_HD uint32_t abs_key(float x) {
  union { float f; uint32_t u; } c;
  c.f = x;
  return c.u & 0x7FFFFFFFu;
}

}  // namespace hipress
