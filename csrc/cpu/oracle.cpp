// CPU restatement of the five compression algorithms and their wire formats.
// It is the numerical oracle for the CUDA kernels (same header, same math via
// hipress/common.h) and the compressor used by the host (gloo) transport.
//
// Reference parity: the only CPU compression code in mark14wu/hipress is the
// thrust::host instantiation of the generated TernGrad pair
// (src/CompLL/GCGen/output/TernGradEncode/TernGradEncode.cc:26-28).  That code
// reduces min/max in int, reads the wrong element index and packs MSB-first
// while unpacking LSB-first; this oracle implements the algorithm the DSL
// source describes (pse/TernGradEncode.pse) rather than those defects.
#include <algorithm>
#include <cstring>
#include <vector>

#include "hipress/common.h"

using namespace hipress;

namespace {

inline uint32_t get_code(const uint8_t* codes, uint64_t i, int bits) {
  uint64_t bit = i * (uint64_t)bits;
  return (codes[bit >> 3] >> (bit & 7)) & ((1u << bits) - 1u);
}
inline void put_code(uint8_t* codes, uint64_t i, int bits, uint32_t c) {
  uint64_t bit = i * (uint64_t)bits;
  codes[bit >> 3] |= (uint8_t)(c << (bit & 7));
}

struct DenseView {
  const WireHeader* hdr;
  const float* meta;
  const uint8_t* codes;
};

inline DenseView view(const uint8_t* p, int alg, uint64_t n) {
  DenseView v;
  v.hdr = reinterpret_cast<const WireHeader*>(p);
  v.meta = reinterpret_cast<const float*>(p + 16);
  v.codes = p + 16 + dense_meta_bytes(alg, n);
  return v;
}

// decoded value of element i of a dense payload
inline float dense_value(const DenseView& v, int alg, int bits, uint64_t i, float tau) {
  uint64_t t = i / kTile;
  uint32_t c = get_code(v.codes, i, bits);
  switch (alg) {
    case kOnebit: return onebit_value(c, v.meta[t]);
    case kTbq: return tbq_value(c, tau);
    case kTernGrad: {
      float mn = v.meta[2 * t], mx = v.meta[2 * t + 1];
      return tern_value(c, mn, tern_gap(mn, mx, bits));
    }
  }
  return 0.0f;
}

bool dense_args_ok(int alg, int bits) {
  if (alg == kOnebit) return bits == 1;
  if (alg == kTbq) return bits == 2;
  if (alg == kTernGrad) return bits == 1 || bits == 2 || bits == 4 || bits == 8;
  return false;
}

}  // namespace

extern "C" {

uint64_t hp_dense_payload_bytes(int alg, int bits, uint64_t n) {
  return dense_payload_bytes(alg, bits, n);
}
uint64_t hp_sparse_payload_bytes(uint64_t kmax) { return sparse_payload_bytes(kmax); }
uint64_t hp_sparse_k(uint64_t n, float ratio) { return sparse_k(n, ratio); }
int hp_tile_elems() { return kTile; }

// Integrity check of a received payload before it is decoded.  Dense: pass the
// element count n the receiver expects and kmax = 0; sparse: bits = 0 and the
// capacity kmax the buffer was laid out for.  Returns 0 or the first mismatch:
//   1 buffer shorter than the format needs   2 algorithm id   3 bit width
//   4 element count   5 tile size / flags    6 pair count above capacity or n
//   7 pair index out of range
int hp_payload_check(const uint8_t* payload, uint64_t payload_bytes, int alg, int bits, uint64_t n,
                     uint64_t kmax) {
  if (payload_bytes < 16) return 1;
  const WireHeader* h = reinterpret_cast<const WireHeader*>(payload);
  const bool sparse = alg == kDgc || alg == kGradDrop;
  if (h->alg != (uint8_t)alg) return 2;
  if (h->bitwidth != (uint8_t)(sparse ? 0 : bits)) return 3;
  if (h->n != (uint32_t)n) return 4;
  if (sparse) {
    if (payload_bytes < sparse_payload_bytes(kmax)) return 1;
    if (h->b > kmax || h->b > n) return 6;
    const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 16);
    for (uint32_t j = 0; j < h->b; ++j)
      if (idx[j] >= n) return 7;
    return 0;
  }
  if (!dense_args_ok(alg, bits)) return 3;
  if (payload_bytes < dense_payload_bytes(alg, bits, n)) return 1;
  if (h->b != (uint32_t)kTile || h->flags != (dense_meta_floats(alg) ? 1 : 0)) return 5;
  return 0;
}

// x = g (+ decode(in_payload)) (+ r);  payload = Q(x);  r = x - decode(payload)
int hp_cpu_dense_encode(int alg, int bits, const float* g, float* r,
                        const uint8_t* in_payload, uint8_t* out, uint64_t n, float tau,
                        uint64_t seed, uint32_t step, uint32_t salt, uint32_t tensor_id,
                        uint64_t elem_offset) {
  if (!dense_args_ok(alg, bits)) return 1;
  const uint64_t total = dense_payload_bytes(alg, bits, n);
  std::memset(out, 0, total);
  WireHeader* h = reinterpret_cast<WireHeader*>(out);
  h->n = (uint32_t)n;
  h->alg = (uint8_t)alg;
  h->bitwidth = (uint8_t)bits;
  h->flags = dense_meta_floats(alg) ? 1 : 0;
  h->a = alg == kTbq ? tau : 0.0f;
  h->b = kTile;
  float* meta = reinterpret_cast<float*>(out + 16);
  uint8_t* codes = out + 16 + dense_meta_bytes(alg, n);
  DenseView in{};
  if (in_payload) in = view(in_payload, alg, n);

  std::vector<float> x(kTile);
  for (uint64_t t0 = 0, t = 0; t0 < n; t0 += kTile, ++t) {
    const uint64_t m = std::min<uint64_t>(kTile, n - t0);
    for (uint64_t i = 0; i < m; ++i) {
      float v = g[t0 + i];
      if (in_payload) v = v + dense_value(in, alg, bits, t0 + i, tau);
      if (r) v = r[t0 + i] + v;
      x[i] = v;
    }
    if (alg == kTbq) {
      for (uint64_t i = 0; i < m; ++i) {
        uint32_t c = tbq_code(x[i], tau);
        put_code(codes, t0 + i, bits, c);
        if (r) r[t0 + i] = x[i] - tbq_value(c, tau);
      }
    } else if (alg == kOnebit) {
      double s = 0.0;
      for (uint64_t i = 0; i < m; ++i) s += (double)fabsf(x[i]);
      float sc = (float)(s / (double)m);
      meta[t] = sc;
      for (uint64_t i = 0; i < m; ++i) {
        uint32_t c = onebit_code(x[i]);
        put_code(codes, t0 + i, bits, c);
        if (r) r[t0 + i] = x[i] - onebit_value(c, sc);
      }
    } else {  // TernGrad
      float mn = x[0], mx = x[0];
      for (uint64_t i = 1; i < m; ++i) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
      }
      meta[2 * t] = mn;
      meta[2 * t + 1] = mx;
      const float gap = tern_gap(mn, mx, bits);
      const float scale16 = tern_scale16(gap);
      for (uint64_t i = 0; i < m; ++i) {
        const uint64_t ge = elem_offset + t0 + i;
        Philox4 rnd = philox4x32(rnd16_counter(ge), tensor_id, step, salt,
                                    (uint32_t)seed, (uint32_t)(seed >> 32));
        uint32_t c = tern_code(x[i], mn, scale16, rnd16(rnd.v[ge & 3], rnd16_half(ge)), bits);
        put_code(codes, t0 + i, bits, c);
        if (r) r[t0 + i] = x[i] - tern_value(c, mn, gap);
      }
    }
  }
  return 0;
}

// out = (accumulate ? out : 0) + decode(payload) * scale
int hp_cpu_dense_decode(int alg, int bits, const uint8_t* payload, float* out, uint64_t n,
                        float tau, float scale, int accumulate) {
  if (!dense_args_ok(alg, bits)) return 1;
  DenseView v = view(payload, alg, n);
  for (uint64_t i = 0; i < n; ++i) {
    float d = dense_value(v, alg, bits, i, tau) * scale;
    out[i] = accumulate ? out[i] + d : d;
  }
  return 0;
}

// DGC momentum correction: u = m*u + g ; v += u
int hp_cpu_dgc_update(const float* g, float* u, float* v, uint64_t n, float momentum) {
  for (uint64_t i = 0; i < n; ++i) {
    float un = fmaf(momentum, u[i], g[i]);
    u[i] = un;
    v[i] = v[i] + un;
  }
  return 0;
}

// GradDrop residual accumulation: r += g
int hp_cpu_acc_update(const float* g, float* r, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) r[i] = r[i] + g[i];
  return 0;
}

// Exact top-k of |v|: sends every |v_i| above the k-th largest magnitude plus the
// lowest-index entries equal to it until exactly k are sent (zeros are never
// sent, so fewer than k pairs leave when v has fewer than k non-zeros).  Sent entries of v
// (and of u when given) are zeroed.  Indices ascend in the payload.
int hp_cpu_sparse_select(int alg, float* v, float* u, uint64_t n, uint64_t k, uint8_t* out,
                         uint64_t kmax) {
  if (k > kmax || k > n) return 1;
  std::memset(out, 0, sparse_payload_bytes(kmax));
  WireHeader* h = reinterpret_cast<WireHeader*>(out);
  h->n = (uint32_t)n;
  h->alg = (uint8_t)alg;
  h->bitwidth = 0;
  h->flags = 0;
  h->b = (uint32_t)k;
  uint32_t* idx = reinterpret_cast<uint32_t*>(out + 16);
  float* val = reinterpret_cast<float*>(out + 16 + align_up(4 * kmax, 16));
  if (k == 0) return 0;
  std::vector<uint32_t> keys(n);
  for (uint64_t i = 0; i < n; ++i) keys[i] = abs_key(v[i]);
  std::vector<uint32_t> tmp(keys);
  std::nth_element(tmp.begin(), tmp.begin() + (k - 1), tmp.end(), std::greater<uint32_t>());
  const uint32_t thr = tmp[k - 1];
  uint64_t gt = 0;
  for (uint64_t i = 0; i < n; ++i) gt += keys[i] > thr;
  uint64_t need_eq = thr == 0 ? 0 : k - gt, w = 0;  // zeros are never sent
  for (uint64_t i = 0; i < n; ++i) {
    bool take = keys[i] > thr;
    if (!take && keys[i] == thr && need_eq > 0) {
      take = true;
      --need_eq;
    }
    if (take) {
      idx[w] = (uint32_t)i;
      val[w] = v[i];
      ++w;
      v[i] = 0.0f;
      if (u) u[i] = 0.0f;
    }
  }
  union { uint32_t u; float f; } c;
  c.u = thr;
  h->a = c.f;
  h->b = (uint32_t)w;
  return 0;
}

// accumulate == 0: out = 0 everywhere, then out[idx] = val*scale
// accumulate == 1: out[idx] += val*scale
int hp_cpu_sparse_decode(const uint8_t* payload, float* out, uint64_t n, uint64_t kmax,
                         float scale, int accumulate) {
  const WireHeader* h = reinterpret_cast<const WireHeader*>(payload);
  const uint64_t k = h->b;
  if (k > kmax) return 1;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 16);
  const float* val = reinterpret_cast<const float*>(payload + 16 + align_up(4 * kmax, 16));
  if (!accumulate) std::memset(out, 0, n * sizeof(float));
  for (uint64_t j = 0; j < k; ++j) {
    if (idx[j] >= n) return 2;
    float d = val[j] * scale;
    out[idx[j]] = accumulate ? out[idx[j]] + d : d;
  }
  return 0;
}

}  // extern "C"
