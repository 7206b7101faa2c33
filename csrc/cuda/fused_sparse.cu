// Fused CaSync-PS and CaSync-Ring for the top-k algorithms (DGC, GradDrop): ONE
// persistent cooperative launch per bucket, no NCCL call, no host round trip.  The
// stages below run as grid-synchronised phases of that launch (a bounded barrier
// over the launch's own CTAs between phases that depend on one another); waiting
// across GPUs happens on release / acquire flags, as in the dense kernels.
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
// All units of a bucket are batched in every phase (the CTAs share out the units'
// slices), which is the "bulk synchronisation" of many small tensors.  An earlier
// version ran every stage as a launch of its own: 19 launches per bucket for PS and
// 9 per ring hop, with a floor of about 0.2 ms per bucket from launch latency alone.
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
  uint32_t cap;         // candidate pairs per (tensor, chunk) unit
  uint64_t cand_push;   // first push unit's candidate list, in pairs from the region start
  uint64_t cand_srv;    // the server unit's candidate list
};

struct SpBucket {
  SpSeg seg[HP_MAX_SEGS];
  int nseg;
  int alg;
  float ratio, momentum, inv_n;
  uint64_t slot_bytes;
  uint64_t cand_pairs;  // candidate pairs of all units of one rank
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

// ------------------------------------------------------ persistent-kernel plumbing
struct SpSmem {
  uint32_t sh[kBins];
  FindSmem fs;
  EmitSmem es;
  SplitSmem sp;
  WaitState wst;
  uint32_t any;
};

// control words of one rank played by a launch, behind its histogram blocks; zero
// when the kernel starts (cleared with the histograms)
constexpr int kCtlBarrier = 0;
constexpr int kCtlStamps = 8;    // low 32 bits of %globaltimer: kernel start, then after every barrier
constexpr int kCtlWords = 128;

struct SpCtx {
  int N, R, E;
  uint32_t G;            // CTAs that play this rank
  uint32_t* ws;          // histogram / counter blocks of this rank, kWsWords per unit
  uint8_t* cand;         // candidate lists of this rank
  uint32_t* ctl;         // control words of this rank
  uint32_t* status;
  uint32_t gen;          // barriers passed so far
};

// the flag value a CTA releases: its epoch, marked when it had given up on a wait
__device__ __forceinline__ uint32_t flag_value(const HpComm& cm, const SpSmem& sm) {
  return cm.epoch | (*(volatile const int*)&sm.wst.poisoned ? kGaveUp : 0u);
}

__device__ __forceinline__ void sp_barrier(const HpComm& cm, SpCtx& cx, SpSmem& sm) {
  // a peer may be late by up to one wait bound before a CTA reaches the barrier
  grid_barrier(cx.ctl + kCtlBarrier, cx.gen, cx.G, 2 * cm.timeout_ns + 1000000000ull, cx.status,
               HP_STATUS_TIMEOUT | (8u << 16) | (cx.gen & 255u), sm.wst);
  if (blockIdx.x == 0 && threadIdx.x == 0 && kCtlStamps + cx.gen < (uint32_t)kCtlWords)
    cx.ctl[kCtlStamps + cx.gen] = (uint32_t)global_timer_ns();
}

// extra stamps of CTA 0 inside a phase (profile words 64..)
__device__ __forceinline__ void sp_mark(const SpCtx& cx, int id) {
  if (blockIdx.x == 0 && threadIdx.x == 0 && 64 + id < kCtlWords)
    cx.ctl[64 + id] = (uint32_t)global_timer_ns();
}

// between two stages that one CTA runs back to back on the same unit
__device__ __forceinline__ void cta_fence_sync() {
  __threadfence();
  __syncthreads();
}

// Phase driver: `units` work units, each cut into `per` slices; slice v of the phase
// goes to CTA v % G.  f(unit, slice, per) is what one CTA of the old one-launch-per-
// stage grid did.
template <typename F>
__device__ __forceinline__ void run_units(const SpCtx& cx, uint32_t units, uint32_t per, F f) {
  const uint32_t total = units * per;
  for (uint32_t v = blockIdx.x; v < total; v += cx.G) {
    f((int)(v / per), v % per, per);
    __syncthreads();  // shared memory is reused by the next slice
  }
}

// did any of `units` units (histogram blocks from `ws`) overflow its candidate list?
// Read after a barrier that follows every writer, so all CTAs agree.
__device__ __forceinline__ bool any_overflow(const uint32_t* ws, uint32_t units, SpSmem& sm) {
  if (threadIdx.x == 0) sm.any = 0;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < units; i += kSpThreads)
    if (__ldcg(ws + (size_t)i * kWsWords + kWsOverflow)) sm.any = 1;
  __syncthreads();
  const bool r = sm.any != 0;
  __syncthreads();
  return r;
}

// longest candidate list among `units` units; same conditions as any_overflow
__device__ __forceinline__ uint32_t max_candidates(const uint32_t* ws, uint32_t units, SpSmem& sm) {
  if (threadIdx.x == 0) sm.any = 0;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < units; i += kSpThreads)
    atomicMax(&sm.any, __ldcg(ws + (size_t)i * kWsWords + kWsCandCount));
  __syncthreads();
  const uint32_t r = sm.any;
  __syncthreads();
  return r;
}
// A unit whose candidate list has at most this many pairs goes through both digit
// passes and the compaction on ONE CTA with no barrier in between; longer lists
// (a steady-state accumulator is dense just below its threshold) are shared out
// over several CTAs again, with a barrier after each pass.
constexpr uint32_t kSmallCand = 8192;

__device__ __forceinline__ uint32_t slices_heavy(const SpCtx& cx, uint32_t units) {
  const uint32_t p = cx.G / (units ? units : 1);
  return p < 1 ? 1 : (p > 592 ? 592 : p);
}
__device__ __forceinline__ uint32_t slices_cap(const SpCtx& cx, uint32_t units, uint32_t cap) {
  const uint32_t p = slices_heavy(cx, units);
  return p > cap ? cap : p;
}

// ---------------------------------------------------------------- push
// unit y = seg * N + owner
// STAGE 0: update + hist0   1: split (certain elements go to the owner at once)
//       2,3: digit passes on the candidate list   4: candidate compaction + flag
//       5,6,7: full-array passes and compaction, only after a candidate overflow
template <int STAGE>
__device__ __forceinline__ void push_stage(const SpBucket& bk, const HpComm& cm, const SpCtx& cx,
                                           SpSmem& sm, int y, uint32_t x, uint32_t nx) {
  const int N = cx.N, R = cx.R, E = cx.E;
  const int si = y / N, c = y % N;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* ws = cx.ws + (size_t)y * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cx.cand + (sg.cand_push + (uint64_t)c * sg.cap) * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  const size_t off = (size_t)c * sg.chunk;
  const float* g = sg.g + E * cm.emu_stride_g + off;
  float* a = sg.a + E * cm.emu_stride_r + off;
  float* u = sg.u ? sg.u + E * cm.emu_stride_r + off : nullptr;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[c]) + (size_t)R * bk.slot_bytes + sg.pay_off;
  EmitDst d;
  d.n = 1;
  d.out[0] = dst;
  bool last = false;
  if (STAGE == 0) {
    if (len == 0) return;
    if (bk.alg == kDgc) pass0_body<2>(g, a, u, len, bk.momentum, ws, sm.sh, x, nx);
    else pass0_body<1>(g, a, u, len, bk.momentum, ws, sm.sh, x, nx);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    split_body(a, u, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, sm.fs, sm.sp, x, nx);
    return;
  } else if (STAGE == 2 || STAGE == 3) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 2) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else if (STAGE == 4) {
    if (len == 0) {
      last = x == 0 && threadIdx.x == 0;
      if (last) write_empty_header(dst, bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, u, ws[kWsCandCount], k, sg.kmax, d, ws, sm.fs, sm.es, x, nx,
                       cand_idx, a, len);
    }
  } else if (STAGE == 5 || STAGE == 6) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 5) pass_body<1>(a, len, k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(a, len, k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, a, u, len, k, sg.kmax, d, ws, sm.fs, sm.es, x, nx);
  }
  if (last) {  // thread 0 of the slice that completed the unit
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[c]) + (size_t)R * bk.nseg + si,
                   flag_value(cm, sm));
  }
}

// -------------------------------------------------------------- server
// unit y = seg; the owned chunk is chunk R
// STAGE 0: wait + scatter-add   1: hist0   2: split (to every rank)   3,4: candidate
//       digit passes   5: candidate compaction + flags   6,7,8: overflow path
template <int STAGE>
__device__ __forceinline__ void server_stage(const SpBucket& bk, const HpComm& cm, const SpCtx& cx,
                                             SpSmem& sm, int y, uint32_t x, uint32_t nx) {
  const int N = cx.N, R = cx.R, E = cx.E;
  const int si = y;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, R);
  uint32_t* ws = cx.ws + ((size_t)bk.nseg * N + y) * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cx.cand + sg.cand_srv * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  float* acc = sg.sr + E * cm.emu_stride_sr;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  EmitDst d;
  d.n = N;
  for (int q = 0; q < N; ++q)
    d.out[q] = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) + (size_t)(N + R) * bk.slot_bytes +
               sg.pay_off;
  bool last = false;
  if (STAGE == 0) {
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(cm.flags[R]);
    for (int q = 0; q < N; ++q)
      wait_flag(my_flags + (size_t)q * bk.nseg + si, cm.epoch, cm.timeout_ns, cx.status,
                HP_STATUS_TIMEOUT | (4u << 16) | ((uint32_t)q << 8) | (si & 255), sm.wst);
    if (len == 0) return;
    const uint8_t* inbox = reinterpret_cast<const uint8_t*>(cm.inbox[R]);
    for (int q = 0; q < N; ++q)
      scatter_body(inbox + (size_t)q * bk.slot_bytes + sg.pay_off, acc, len, sg.kmax, 1.0f, 2, x, nx);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    pass0_body<0>(nullptr, acc, nullptr, len, 0.0f, ws, sm.sh, x, nx);
    return;
  } else if (STAGE == 2) {
    if (len == 0) return;
    split_body(acc, nullptr, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, sm.fs, sm.sp, x, nx);
    return;
  } else if (STAGE == 3 || STAGE == 4) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 3) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else if (STAGE == 5) {
    if (len == 0) {
      last = x == 0 && threadIdx.x == 0;
      if (last)
        for (int q = 0; q < N; ++q) write_empty_header(d.out[q], bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, nullptr, ws[kWsCandCount], k, sg.kmax, d, ws, sm.fs, sm.es, x,
                       nx, cand_idx, acc, len);
    }
  } else if (STAGE == 6 || STAGE == 7) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 6) pass_body<1>(acc, len, k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(acc, len, k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, acc, nullptr, len, k, sg.kmax, d, ws, sm.fs, sm.es, x, nx);
  }
  if (last) {
    __threadfence_system();
    const uint32_t fv = flag_value(cm, sm);
    for (int q = 0; q < N; ++q)
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) +
                         (size_t)(N + R) * bk.nseg + si,
                     fv);
  }
}

// ---------------------------------------------------------------- pull
// zero-fill of the result (unit y = seg).  It runs one phase after the update pass has
// read the gradient (which may be the same buffer): clearing each element right behind
// its load in that pass made the pass five times slower when the buffers were the same
// (a store to a line whose fill is still in flight).
__device__ __forceinline__ void zero_stage(const SpBucket& bk, const HpComm& cm, const SpCtx& cx,
                                           int y, uint32_t x, uint32_t nx) {
  const SpSeg& sg = bk.seg[y];
  float* out = sg.out + cx.E * cm.emu_stride_out;
  const bool vec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const uint64_t stride = (uint64_t)nx * kSpThreads * 4;
  for (uint64_t i = ((uint64_t)x * kSpThreads + threadIdx.x) * 4; i < sg.n; i += stride)
    st4(out, i, sg.n, vec, make_float4(0.f, 0.f, 0.f, 0.f));
}

// wait for the reduced chunk c that arrives in inbox slot `slot` and scatter value / N
// into the (zero-filled) result; unit y = seg * N + j.  A CTA that has given up leaves
// the result alone.
__device__ __forceinline__ void gather_stage(const SpBucket& bk, const HpComm& cm, const SpCtx& cx,
                                             SpSmem& sm, int si, int slot, int c, uint32_t phase,
                                             uint32_t x, uint32_t nx) {
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  wait_flag(reinterpret_cast<const uint32_t*>(cm.flags[cx.R]) + (size_t)slot * bk.nseg + si, cm.epoch,
            cm.timeout_ns, cx.status,
            HP_STATUS_TIMEOUT | (phase << 16) | ((uint32_t)(slot & 255) << 8) | (si & 255), sm.wst);
  if (len == 0 || *(volatile int*)&sm.wst.poisoned) return;
  const uint8_t* p = reinterpret_cast<const uint8_t*>(cm.inbox[cx.R]) + (size_t)slot * bk.slot_bytes +
                     sg.pay_off;
  scatter_body(p, sg.out + cx.E * cm.emu_stride_out + (size_t)c * sg.chunk, len, sg.kmax, bk.inv_n, 0,
               x, nx);
}

// ---------------------------------------------------------------- ring
// One hop of the sparse ring for every tensor of the bucket (unit y = seg).  At hop
// h rank R works on chunk (R - h) mod N: the predecessor's pairs are added into the
// local accumulator, then the state update, the exact top-k selection and the
// compaction run, and the pairs go into the successor's inbox -- or, at the last
// hop, into every rank's inbox.
// STAGE 0: wait + add incoming   1: update + hist0   2: split   3,4: candidate digit
//       passes   5: candidate compaction + flag(s)   6,7,8: overflow path
template <int STAGE>
__device__ __forceinline__ void ring_stage(const SpBucket& bk, const HpComm& cm, const SpCtx& cx,
                                           SpSmem& sm, int hop, int y, uint32_t x, uint32_t nx) {
  const int N = cx.N, R = cx.R, E = cx.E;
  const int si = y;
  const int c = (R - hop + N) % N;
  const bool last_hop = hop == N - 1;
  const SpSeg& sg = bk.seg[si];
  const uint32_t len = sp_chunk_valid(sg.n, sg.chunk, c);
  uint32_t* ws = cx.ws + ((size_t)hop * bk.nseg + si) * kWsWords;
  float* cand_val = reinterpret_cast<float*>(cx.cand + (sg.cand_push + (uint64_t)c * sg.cap) * 8);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + sg.cap);
  const size_t off = (size_t)c * sg.chunk;
  const float* g = sg.g + E * cm.emu_stride_g + off;
  float* a = sg.a + E * cm.emu_stride_r + off;
  float* u = sg.u ? sg.u + E * cm.emu_stride_r + off : nullptr;
  const uint32_t k = (uint32_t)sparse_k(len, bk.ratio);
  EmitDst d;
  if (!last_hop) {
    d.n = 1;
    d.out[0] = reinterpret_cast<uint8_t*>(cm.inbox[(R + 1) % N]) + (size_t)hop * bk.slot_bytes + sg.pay_off;
  } else {
    d.n = N;
    for (int q = 0; q < N; ++q)
      d.out[q] = reinterpret_cast<uint8_t*>(cm.inbox[(R + q) % N]) +
                 (size_t)(N - 1 + R) * bk.slot_bytes + sg.pay_off;
  }
  bool last = false;
  if (STAGE == 0) {
    if (hop == 0) return;
    wait_flag(reinterpret_cast<const uint32_t*>(cm.flags[R]) + (size_t)(hop - 1) * bk.nseg + si,
              cm.epoch, cm.timeout_ns, cx.status,
              HP_STATUS_TIMEOUT | (6u << 16) | ((uint32_t)(hop - 1) << 8) | (si & 255), sm.wst);
    if (len == 0) return;
    scatter_body(reinterpret_cast<const uint8_t*>(cm.inbox[R]) + (size_t)(hop - 1) * bk.slot_bytes +
                     sg.pay_off,
                 a, len, sg.kmax, 1.0f, 1, x, nx);
    return;
  } else if (STAGE == 1) {
    if (len == 0) return;
    if (bk.alg == kDgc) pass0_body<2>(g, a, u, len, bk.momentum, ws, sm.sh, x, nx);
    else pass0_body<1>(g, a, u, len, bk.momentum, ws, sm.sh, x, nx);
    return;
  } else if (STAGE == 2) {
    if (len == 0) return;
    split_body(a, u, len, k, sg.kmax, d, ws, cand_val, cand_idx, sg.cap, sm.fs, sm.sp, x, nx);
    return;
  } else if (STAGE == 3 || STAGE == 4) {
    if (len == 0 || ws[kWsOverflow]) return;
    if (STAGE == 3) pass_body<1>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(cand_val, ws[kWsCandCount], k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else if (STAGE == 5) {
    if (len == 0) {
      last = x == 0 && threadIdx.x == 0;
      if (last)
        for (int q = 0; q < d.n; ++q) write_empty_header(d.out[q], bk.alg);
    } else {
      if (ws[kWsOverflow]) return;
      last = emit_body(bk.alg, cand_val, u, ws[kWsCandCount], k, sg.kmax, d, ws, sm.fs, sm.es, x, nx,
                       cand_idx, a, len);
    }
  } else if (STAGE == 6 || STAGE == 7) {
    if (len == 0 || !ws[kWsOverflow]) return;
    if (STAGE == 6) pass_body<1>(a, len, k, ws, sm.sh, sm.fs, x, nx);
    else pass_body<2>(a, len, k, ws, sm.sh, sm.fs, x, nx);
    return;
  } else {
    if (len == 0 || !ws[kWsOverflow]) return;
    last = emit_body(bk.alg, a, u, len, k, sg.kmax, d, ws, sm.fs, sm.es, x, nx);
  }
  if (last) {
    __threadfence_system();
    const uint32_t fv = flag_value(cm, sm);
    if (!last_hop) {
      st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + 1) % N]) + (size_t)hop * bk.nseg + si, fv);
    } else {
      for (int q = 0; q < N; ++q)
        st_release_sys(reinterpret_cast<uint32_t*>(cm.flags[(R + q) % N]) +
                           (size_t)(N - 1 + R) * bk.nseg + si,
                       fv);
    }
  }
}

// ------------------------------------------------------------- the two kernels
struct SpLaunch {
  uint8_t* ws;            // scratch of all ranks played by the launch
  uint64_t ws_rank_bytes; // per rank: histogram blocks, control words, candidate lists
  uint64_t hist_words;    // histogram words per rank (the control words follow)
  uint64_t hist_bytes;    // offset of the candidate lists inside a rank's scratch
};

__device__ __forceinline__ void sp_prologue(const HpComm& cm, const SpLaunch& L, SpCtx& cx,
                                            SpSmem& sm) {
  cx.N = cm.nranks;
  cx.R = cm.emulate ? (int)blockIdx.y : cm.rank;
  cx.E = cm.emulate ? (int)blockIdx.y : 0;
  cx.G = gridDim.x;
  uint8_t* base = L.ws + (size_t)cx.E * L.ws_rank_bytes;
  cx.ws = reinterpret_cast<uint32_t*>(base);
  cx.ctl = cx.ws + L.hist_words;
  cx.cand = base + L.hist_bytes;
  cx.status = reinterpret_cast<uint32_t*>(cm.status) + 4 * cx.E;
  cx.gen = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) cx.ctl[kCtlStamps] = (uint32_t)global_timer_ns();
  wait_init(sm.wst);
}

// CTA 0's last stamp and the number of barriers it passed (the other CTAs may still
// be scattering: the stamps are a profile of the phases, not a completion signal)
__device__ __forceinline__ void sp_epilogue(const SpCtx& cx) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (kCtlStamps + cx.gen + 1 < (uint32_t)kCtlWords)
      cx.ctl[kCtlStamps + cx.gen + 1] = (uint32_t)global_timer_ns();
    cx.ctl[1] = cx.gen;
  }
}

// PS: push (every rank selects per owner and stores the pairs into the owner's
// inbox), server (the owner adds the N payloads, re-selects, stores the result into
// every inbox), pull (every rank scatters value / N).  Five barriers when the
// candidate lists are short, nine otherwise (more only after an overflow).
__global__ void __launch_bounds__(kSpThreads, 3)
sp_ps_kernel(const SpBucket bk, const HpComm cm, const SpLaunch L) {
  __shared__ SpSmem sm;
  SpCtx cx;
  sp_prologue(cm, L, cx, sm);
  const uint32_t nseg = (uint32_t)bk.nseg, units = nseg * (uint32_t)cx.N;
  const uint32_t ph = slices_heavy(cx, units), pc = slices_cap(cx, units, 32);
  const uint32_t sh = slices_heavy(cx, nseg), sc = slices_cap(cx, nseg, 32);
#define PUSH(S, P) run_units(cx, units, P, [&](int y, uint32_t x, uint32_t nx) { push_stage<S>(bk, cm, cx, sm, y, x, nx); })
#define SRV(S, P) run_units(cx, nseg, P, [&](int y, uint32_t x, uint32_t nx) { server_stage<S>(bk, cm, cx, sm, y, x, nx); })
  PUSH(0, ph);
  sp_barrier(cm, cx, sm);
  PUSH(1, ph);
  sp_barrier(cm, cx, sm);
  const bool ovf = any_overflow(cx.ws, units, sm);
  // the candidate list of a unit is short (about as many pairs as are sent): one CTA
  // takes a unit through both digit passes and the compaction, no barrier in between
  if (max_candidates(cx.ws, units, sm) <= kSmallCand) {
    run_units(cx, units, 1, [&](int y, uint32_t x, uint32_t nx) {
      push_stage<2>(bk, cm, cx, sm, y, x, nx);
      cta_fence_sync();
      push_stage<3>(bk, cm, cx, sm, y, x, nx);
      cta_fence_sync();
      push_stage<4>(bk, cm, cx, sm, y, x, nx);
    });
  } else {
    PUSH(2, pc);
    sp_barrier(cm, cx, sm);
    PUSH(3, pc);
    sp_barrier(cm, cx, sm);
    PUSH(4, pc);
  }
  if (ovf) {
    PUSH(5, ph);
    sp_barrier(cm, cx, sm);
    PUSH(6, ph);
    sp_barrier(cm, cx, sm);
    PUSH(7, ph);
  }
  // The gradient was read two barriers ago (it may be the result buffer): clear the
  // result here, where the CTAs would otherwise only wait for the peers' pushes.
  run_units(cx, nseg, sh, [&](int y, uint32_t x, uint32_t nx) { zero_stage(bk, cm, cx, y, x, nx); });
  SRV(0, sh);
  sp_barrier(cm, cx, sm);
  SRV(1, sh);
  sp_barrier(cm, cx, sm);
  SRV(2, sh);
  sp_barrier(cm, cx, sm);
  const bool ovf2 = any_overflow(cx.ws + (size_t)units * kWsWords, nseg, sm);
  if (max_candidates(cx.ws + (size_t)units * kWsWords, nseg, sm) <= kSmallCand) {
    run_units(cx, nseg, 1, [&](int y, uint32_t x, uint32_t nx) {
      server_stage<3>(bk, cm, cx, sm, y, x, nx);
      cta_fence_sync();
      server_stage<4>(bk, cm, cx, sm, y, x, nx);
      cta_fence_sync();
      server_stage<5>(bk, cm, cx, sm, y, x, nx);
    });
  } else {
    SRV(3, sc);
    sp_barrier(cm, cx, sm);
    SRV(4, sc);
    sp_barrier(cm, cx, sm);
    SRV(5, sc);
  }
  if (ovf2) {
    SRV(6, sh);
    sp_barrier(cm, cx, sm);
    SRV(7, sh);
    sp_barrier(cm, cx, sm);
    SRV(8, sh);
  }
  const int N = cx.N;
  run_units(cx, units, slices_cap(cx, units, 16), [&](int y, uint32_t x, uint32_t nx) {
    const int j = y % N;
    gather_stage(bk, cm, cx, sm, y / N, N + j, j, 5u, x, nx);
  });
#undef PUSH
#undef SRV
  sp_epilogue(cx);
}

// Ring: N hops of (add the predecessor's pairs, update, select, store into the
// successor's inbox), the last hop storing into every inbox; then every rank scatters
// the N reduced chunks.  Three barriers per hop when the candidate lists are short,
// five otherwise.
__global__ void __launch_bounds__(kSpThreads, 3)
sp_ring_kernel(const SpBucket bk, const HpComm cm, const SpLaunch L) {
  __shared__ SpSmem sm;
  SpCtx cx;
  sp_prologue(cm, L, cx, sm);
  const int N = cx.N;
  const uint32_t nseg = (uint32_t)bk.nseg;
  const uint32_t sh = slices_heavy(cx, nseg), sc = slices_cap(cx, nseg, 32);
#define HOP(S, P) run_units(cx, nseg, P, [&](int y, uint32_t x, uint32_t nx) { ring_stage<S>(bk, cm, cx, sm, hop, y, x, nx); })
  for (int hop = 0; hop < N; ++hop) {
    if (hop > 0) {
      HOP(0, sc);
      sp_barrier(cm, cx, sm);
    }
    HOP(1, sh);
    sp_barrier(cm, cx, sm);
    HOP(2, sh);
    if (hop == N - 1)  // every chunk of the gradient has been read: clear the result
      run_units(cx, nseg, sh, [&](int y, uint32_t x, uint32_t nx) { zero_stage(bk, cm, cx, y, x, nx); });
    sp_barrier(cm, cx, sm);
    const bool ovf = any_overflow(cx.ws + (size_t)hop * nseg * kWsWords, nseg, sm);
    if (max_candidates(cx.ws + (size_t)hop * nseg * kWsWords, nseg, sm) <= kSmallCand) {
      sp_mark(cx, 0);
      run_units(cx, nseg, 1, [&](int y, uint32_t x, uint32_t nx) {
        ring_stage<3>(bk, cm, cx, sm, hop, y, x, nx);
        cta_fence_sync();
        sp_mark(cx, 1);
        ring_stage<4>(bk, cm, cx, sm, hop, y, x, nx);
        cta_fence_sync();
        sp_mark(cx, 2);
        ring_stage<5>(bk, cm, cx, sm, hop, y, x, nx);
        sp_mark(cx, 3);
      });
    } else {
      HOP(3, sc);
      sp_barrier(cm, cx, sm);
      HOP(4, sc);
      sp_barrier(cm, cx, sm);
      sp_mark(cx, 2);
      HOP(5, sc);
      sp_mark(cx, 3);
    }
    if (ovf) {
      HOP(6, sh);
      sp_barrier(cm, cx, sm);
      HOP(7, sh);
      sp_barrier(cm, cx, sm);
      HOP(8, sh);
    }
  }
#undef HOP
  // gather: rank src finalised chunk src + 1
  sp_mark(cx, 4);
  const uint32_t units = nseg * (uint32_t)N;
  run_units(cx, units, slices_cap(cx, units, 16), [&](int y, uint32_t x, uint32_t nx) {
    const int src = y % N;
    gather_stage(bk, cm, cx, sm, y / N, N - 1 + src, (src + 1) % N, 7u, x, nx);
  });
  sp_epilogue(cx);
}

static int build_sp_bucket(int alg, float ratio, float momentum, const HpSeg* segs,
                           void* const* accs, void* const* us, int nseg, int nranks, SpBucket& bk) {
  if (nseg < 1 || nseg > HP_MAX_SEGS || nranks < 1 || nranks > HP_MAX_RANKS) return HP_ERR_BAD_ARG;
  if (alg != kDgc && alg != kGradDrop) return HP_ERR_BAD_ARG;
  uint64_t pay = 0, cand = 0;
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
    d.cap = (uint32_t)align_up(8ull * d.kmax + 4096, 32);
    d.cand_push = cand;
    cand += (uint64_t)d.cap * nranks;
    d.cand_srv = cand;
    cand += d.cap;
    pay += align_up(sparse_payload_bytes(d.kmax), 128);
    if (pay > 0xFFFFFFFFull) return HP_ERR_TOO_LARGE;
  }
  bk.nseg = nseg;
  bk.alg = alg;
  bk.ratio = ratio;
  bk.momentum = momentum;
  bk.inv_n = 1.0f / (float)nranks;
  bk.slot_bytes = pay;
  bk.cand_pairs = cand;
  return 0;
}

// ------------------------------------------------------------------ host side
static uint64_t sp_hist_words(int nseg, int nranks) {
  return (uint64_t)(nseg * nranks + nseg) * kWsWords;   // the ring uses nseg * nranks of them
}

static int launch_sparse(int topo, const SpBucket& bk, const HpComm& cm, void* ws, int ctas,
                         cudaStream_t st) {
  const void* kern = topo == HP_TOPO_RING ? (const void*)sp_ring_kernel : (const void*)sp_ps_kernel;
  const int N = cm.nranks, nseg = bk.nseg;
  static int resident[2][64] = {};   // CTAs the GPU holds at once, per (topology, device)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  int cap = (dev >= 0 && dev < 64) ? resident[topo][dev] : 0;
  if (cap == 0) {
    int sms = 0, per_sm = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kSpThreads, 0);
    if (e != cudaSuccess) return (int)e;
    cap = per_sm * sms;
    if (cap < 1) return HP_ERR_RESIDENCY;
    if (dev >= 0 && dev < 64) resident[topo][dev] = cap;
  }
  const int ranks_here = cm.emulate ? N : 1;
  int G = ctas;
  if (G <= 0) {   // a quarter of the bucket's tiles, at least 32, at most what the GPU holds
    uint64_t tiles = 0;
    for (int i = 0; i < nseg; ++i) tiles += (bk.seg[i].n + kTile - 1) / kTile;
    G = (int)(tiles / 4 < 32 ? 32 : (tiles / 4 > 592 ? 592 : tiles / 4));
    if (G > cap / ranks_here) G = cap / ranks_here;
  }
  if (G < 1 || (long long)G * ranks_here > (long long)cap) return HP_ERR_RESIDENCY;
  SpLaunch L;
  L.ws = static_cast<uint8_t*>(ws);
  L.hist_words = sp_hist_words(nseg, N);
  L.hist_bytes = align_up((L.hist_words + kCtlWords) * 4, 256);
  L.ws_rank_bytes = L.hist_bytes + bk.cand_pairs * 8;
  for (int r = 0; r < ranks_here; ++r) {  // histograms, counters and control words start at zero
    e = cudaMemsetAsync(L.ws + (size_t)r * L.ws_rank_bytes, 0, (L.hist_words + kCtlWords) * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  void* args[] = {(void*)&bk, (void*)&cm, (void*)&L};
  // cooperative: the CTAs of a launch wait for one another at the phase barriers
  e = cudaLaunchCooperativeKernel(kern, dim3(G, ranks_here), dim3(kSpThreads), args, 0, st);
  return (int)e;
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
  // per rank played by a launch: histogram blocks of the push (nseg * nranks) and
  // server (nseg) units, control words, candidate lists
  if (ws_bytes)
    *ws_bytes = align_up((sp_hist_words(nseg, nranks) + kCtlWords) * 4, 256) + bk.cand_pairs * 8;
  return 0;
}

// One synchronisation of a bucket through the PS topology: one cooperative launch.
// segs[i].r is the accumulator (DGC v / GradDrop residual), us[i] the DGC momentum
// (or NULL), segs[i].sr the server accumulator of the owned chunk.  ws: scratch of
// hp_fused_sparse_layout().ws_bytes per rank played by this call.  ctas <= 0: the
// grid is sized from the bucket.
int hp_cuda_fused_sparse_ps(int alg, float ratio, float momentum, const HpSeg* segs,
                            void* const* us, int nseg, const HpComm* comm, void* ws, int ctas,
                            void* stream) {
  if (!comm || ctas > 1024) return HP_ERR_BAD_ARG;
  SpBucket bk;
  int rc = build_sp_bucket(alg, ratio, momentum, segs, nullptr, us, nseg, comm->nranks, bk);
  if (rc) return rc;
  return launch_sparse(HP_TOPO_PS, bk, *comm, ws, ctas, (cudaStream_t)stream);
}

// One synchronisation of a bucket through the ring topology: one cooperative launch.
// Same arguments as hp_cuda_fused_sparse_ps (segs[i].sr is not used).
int hp_cuda_fused_sparse_ring(int alg, float ratio, float momentum, const HpSeg* segs,
                              void* const* us, int nseg, const HpComm* comm, void* ws, int ctas,
                              void* stream) {
  if (!comm || ctas > 1024) return HP_ERR_BAD_ARG;
  SpBucket bk;
  int rc = build_sp_bucket(alg, ratio, momentum, segs, nullptr, us, nseg, comm->nranks, bk);
  if (rc) return rc;
  return launch_sparse(HP_TOPO_RING, bk, *comm, ws, ctas, (cudaStream_t)stream);
}

}  // extern "C"
