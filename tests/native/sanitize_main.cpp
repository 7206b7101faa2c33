// Driver run under AddressSanitizer + UBSan: exercises the CPU oracle and the
// bucket planner on awkward sizes so that any out-of-bounds access in the host
// code aborts the test.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <vector>

extern "C" {
uint64_t hp_dense_payload_bytes(int alg, int bits, uint64_t n);
uint64_t hp_sparse_payload_bytes(uint64_t kmax);
uint64_t hp_sparse_k(uint64_t n, float ratio);
int hp_cpu_dense_encode(int alg, int bits, const float* g, float* r, const uint8_t* in, uint8_t* out,
                        uint64_t n, float tau, uint64_t seed, uint32_t step, uint32_t salt,
                        uint32_t tensor_id, uint64_t elem_offset);
int hp_cpu_dense_decode(int alg, int bits, const uint8_t* p, float* out, uint64_t n, float tau,
                        float scale, int accumulate);
int hp_cpu_dgc_update(const float* g, float* u, float* v, uint64_t n, float momentum);
int hp_cpu_sparse_select(int alg, float* v, float* u, uint64_t n, uint64_t k, uint8_t* out, uint64_t kmax);
int hp_cpu_sparse_decode(const uint8_t* p, float* out, uint64_t n, uint64_t kmax, float scale, int acc);
int hp_plan_buckets(int n, const uint64_t* numel, const int32_t* compress, const int32_t* partitions,
                    uint64_t bucket_bytes, uint64_t plain_bucket_bytes, int32_t* bucket_of,
                    int32_t* bucket_fused, int seg_cap, int32_t* seg_bucket, int32_t* seg_entry,
                    int32_t* seg_part, uint64_t* seg_lo, uint64_t* seg_hi, int32_t* nseg_out);
}

int main() {
  const uint64_t sizes[] = {1, 2, 3, 7, 8, 9, 4095, 4096, 4097, 8191, 12289};
  const int algs[][2] = {{1, 1}, {2, 2}, {3, 1}, {3, 2}, {3, 4}, {3, 8}};
  int checks = 0;
  for (uint64_t n : sizes) {
    std::vector<float> g(n), r(n, 0.f), out(n);
    for (uint64_t i = 0; i < n; ++i) g[i] = std::sin(0.37f * (float)i) * 0.05f;
    for (auto& a : algs) {
      std::vector<uint8_t> p(hp_dense_payload_bytes(a[0], a[1], n)), q(p.size());
      if (hp_cpu_dense_encode(a[0], a[1], g.data(), a[0] == 3 ? nullptr : r.data(), nullptr, p.data(), n,
                              0.01f, 1, 2, 3, 4, 0)) return 1;
      if (hp_cpu_dense_encode(a[0], a[1], g.data(), nullptr, p.data(), q.data(), n, 0.01f, 1, 2, 3, 4, 4096)) return 2;
      if (hp_cpu_dense_decode(a[0], a[1], q.data(), out.data(), n, 0.01f, 0.5f, 0)) return 3;
      if (hp_cpu_dense_decode(a[0], a[1], q.data(), out.data(), n, 0.01f, 0.5f, 1)) return 4;
      ++checks;
    }
    std::vector<float> u(n, 0.f), v(n, 0.f);
    hp_cpu_dgc_update(g.data(), u.data(), v.data(), n, 0.9f);
    const uint64_t k = hp_sparse_k(n, 0.1f);
    std::vector<uint8_t> sp(hp_sparse_payload_bytes(k));
    if (hp_cpu_sparse_select(4, v.data(), u.data(), n, k, sp.data(), k)) return 5;
    if (hp_cpu_sparse_decode(sp.data(), out.data(), n, k, 1.0f, 0)) return 6;
    if (hp_cpu_sparse_decode(sp.data(), out.data(), n, k, 1.0f, 1)) return 7;
    ++checks;
  }
  // planner: many gradients, odd partition counts, tiny buckets
  const int n = 57;
  std::vector<uint64_t> numel(n);
  std::vector<int32_t> comp(n), parts(n), bof(n), bfused(n);
  for (int i = 0; i < n; ++i) {
    numel[i] = 1 + (uint64_t)i * 7919 % 300000;
    comp[i] = numel[i] > 5000;
    parts[i] = 1 + i % 9;
  }
  const int cap = 1024;
  std::vector<int32_t> sb(cap), se(cap), spp(cap);
  std::vector<uint64_t> lo(cap), hi(cap);
  int32_t nseg = 0;
  const int nb = hp_plan_buckets(n, numel.data(), comp.data(), parts.data(), 1 << 20, 1 << 16, bof.data(),
                                 bfused.data(), cap, sb.data(), se.data(), spp.data(), lo.data(), hi.data(), &nseg);
  if (nb < 1) return 8;
  uint64_t covered = 0;
  for (int s = 0; s < nseg; ++s) covered += hi[s] - lo[s];
  uint64_t want = 0;
  for (int i = 0; i < n; ++i) want += comp[i] ? numel[i] : 0;
  if (covered != want) return 9;
  std::printf("sanitize ok: %d checks, %d buckets, %d segments\n", checks, nb, nseg);
  return 0;
}
