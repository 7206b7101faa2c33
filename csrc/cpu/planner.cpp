// Native bucket planner of the CaSync runtime: turns the per-gradient plan
// (compress or not, partitions K) into launch buckets.  Gradients are visited in
// reverse registration order (the order backward produces them); compressed ones
// are cut into K tile-aligned segments and packed into fused buckets of at most
// HP_MAX_SEGS segments / bucket_bytes, the others into plain all-reduce buckets.
// Buckets are then ordered by completion: a bucket is complete once its
// lowest-index gradient exists, and every rank must launch in that same order.
//
// Reference parity: Horovod's tensor-fusion / response-cache logic is what the
// reference's modified Horovod core provides for this purpose (the fork itself is
// not published; README.md:106-108 of mark14wu/hipress only names its install
// script).  Here the order is static, so no per-step negotiation is needed.
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "hipress/capi.h"
#include "hipress/common.h"

using namespace hipress;

namespace {
struct B {
  int fused;
  std::vector<int> entries;
  std::vector<int> seg_entry, seg_part;
  std::vector<uint64_t> seg_lo, seg_hi;
  uint64_t bytes = 0;
  int min_index = 1 << 30;
};

void split(uint64_t n, int k, std::vector<uint64_t>& lo, std::vector<uint64_t>& hi) {
  const uint64_t tiles = (n + kTile - 1) / kTile;
  if (k < 1) k = 1;
  if ((uint64_t)k > tiles) k = (int)tiles;
  const uint64_t per = align_up((n + k - 1) / k, kTile);
  for (uint64_t a = 0; a < n; a += per) {
    lo.push_back(a);
    hi.push_back(std::min(n, a + per));
  }
}
}  // namespace

extern "C" {

// Inputs: numel[i], compress[i] (0/1), partitions[i] for n gradients in registration
// order.  Outputs (caller-allocated, capacity >= n for *_of arrays, seg_cap for
// segment arrays): bucket_of[i] = bucket index of gradient i in LAUNCH order,
// bucket_fused[b]; segments listed bucket by bucket: seg_bucket, seg_entry,
// seg_part, seg_lo, seg_hi.  Returns the number of buckets, or a negative error.
int hp_plan_buckets(int n, const uint64_t* numel, const int32_t* compress,
                    const int32_t* partitions, uint64_t bucket_bytes, uint64_t plain_bucket_bytes,
                    int32_t* bucket_of, int32_t* bucket_fused, int seg_cap, int32_t* seg_bucket,
                    int32_t* seg_entry, int32_t* seg_part, uint64_t* seg_lo, uint64_t* seg_hi,
                    int32_t* nseg_out) {
  if (n < 1) return HP_ERR_BAD_ARG;
  std::vector<B> done;
  B curf, curp;
  curf.fused = 1;
  curp.fused = 0;
  auto close = [&](B& b, int fused) {
    if (!b.entries.empty()) done.push_back(b);
    b = B();
    b.fused = fused;
  };
  for (int i = n - 1; i >= 0; --i) {
    if (compress[i]) {
      std::vector<uint64_t> lo, hi;
      int k = partitions[i];
      split(numel[i], k, lo, hi);
      while ((int)lo.size() > HP_MAX_SEGS) {  // a tensor alone in its bucket: fewer, larger parts
        lo.clear();
        hi.clear();
        k = std::max(1, k / 2);
        split(numel[i], k, lo, hi);
      }
      if (!curf.entries.empty() &&
          ((int)(curf.seg_lo.size() + lo.size()) > HP_MAX_SEGS || curf.bytes + 4 * numel[i] > bucket_bytes))
        close(curf, 1);
      curf.entries.push_back(i);
      for (size_t s = 0; s < lo.size(); ++s) {
        curf.seg_entry.push_back(i);
        curf.seg_part.push_back((int)s);
        curf.seg_lo.push_back(lo[s]);
        curf.seg_hi.push_back(hi[s]);
      }
      curf.bytes += 4 * numel[i];
      curf.min_index = std::min(curf.min_index, i);
    } else {
      if (!curp.entries.empty() && curp.bytes + 4 * numel[i] > plain_bucket_bytes) close(curp, 0);
      curp.entries.push_back(i);
      curp.bytes += 4 * numel[i];
      curp.min_index = std::min(curp.min_index, i);
    }
  }
  close(curf, 1);
  close(curp, 0);
  std::stable_sort(done.begin(), done.end(),
                   [](const B& a, const B& b) { return a.min_index > b.min_index; });
  int ns = 0;
  for (size_t b = 0; b < done.size(); ++b) {
    bucket_fused[b] = done[b].fused;
    for (int e : done[b].entries) bucket_of[e] = (int)b;
    for (size_t s = 0; s < done[b].seg_lo.size(); ++s) {
      if (ns >= seg_cap) return HP_ERR_TOO_LARGE;
      seg_bucket[ns] = (int)b;
      seg_entry[ns] = done[b].seg_entry[s];
      seg_part[ns] = done[b].seg_part[s];
      seg_lo[ns] = done[b].seg_lo[s];
      seg_hi[ns] = done[b].seg_hi[s];
      ++ns;
    }
  }
  *nseg_out = ns;
  return (int)done.size();
}

}  // extern "C"
