// Fused CaSync kernels for the dense (quantising) algorithms: onebit, TBQ and
// TernGrad.  One persistent launch synchronises a whole bucket of tensors:
//
//   ring : N hops of  poll incoming partial sum -> decode -> merge with the local
//          chunk and its residual -> re-encode -> store the payload straight into
//          the successor GPU's inbox over NVLink; the last hop stores the fully
//          reduced payload into every rank's inbox, and every rank decodes all N
//          chunks into the gradient (averaged).
//   PS   : encode each of the N chunks and store chunk j into owner j's inbox;
//          the owner decodes and sums the N payloads in rank order, re-encodes
//          with its server residual and stores the result into every inbox;
//          every rank decodes all N chunks.
//
// There is no NCCL call and no separate encode or decode launch.  Payloads are
// plain 8-byte stores {codes, epoch} to peer-mapped memory; the receiver polls its
// own memory until the epoch of this launch shows up (see "transport" below).  A
// CTA only ever waits for data produced by other GPUs, never for another CTA of
// its own GPU.  Every wait is bounded: on expiry the thread records a status
// word, the CTA stops waiting and still runs to completion inside its own
// buffers.  g and r tiles are prefetched with bulk copies (pipeline.cuh).
//
// Reference parity: CaSync-Ring and CaSync-PS of mark14wu/hipress are selected
// with --topo Ring|PS (README.md:45,51); their cost shape (N encodes, N decodes,
// 2(N-1) sends for ring; gather + broadcast for PS) is in
// src/SeCoPa/SeCoPa.py:75-103.  The runtime source itself is not published.
#include <cuda_runtime.h>

#include "dense_tile.cuh"
#include "hipress/capi.h"
#include "pipeline.cuh"
#include "sync.cuh"

namespace hipress {

struct SegDev {
  const float* g;
  float* r;
  float* out;
  float* sr;
  uint32_t n;
  uint32_t chunk;        // elements per chunk, multiple of kTile
  uint32_t tiles;        // tiles per chunk
  uint32_t tile_prefix;  // tiles of one chunk of the segments before this one
  uint32_t pay_off;      // byte offset of this segment's chunk payload inside a slot
  uint32_t id;
};

struct BucketDev {
  SegDev seg[HP_MAX_SEGS];
  int nseg;
  uint32_t tiles_total;  // tiles of one chunk summed over segments = work items of a phase
  uint64_t slot_bytes;
  uint64_t inbox_bytes;  // slot_bytes * slots of the topology: what a rank's inbox holds
  uint64_t dbg_limit;    // debug build: pretend the inbox ends here (0: at inbox_bytes)
};

// The decode phases take their tiles in groups of kGroup: the payload loads of a
// whole group go out before the first one is waited for.
constexpr int kGroup = 4;

struct FusedParams {
  DenseParams P;
  float inv_n;
};

// ------------------------------------------------------------------ transport
// Payloads travel in 8-byte slots {32 bits of codes, 32-bit epoch}: one aligned
// 8-byte store is delivered whole, so the receiver polls the slot itself until
// the epoch of this launch shows up.  No separate flag, no system-scope fence and
// no CTA barrier per hop; the cost is 2x on payload bytes that are 16-32x smaller
// than the gradient to begin with.  Slots are never reused inside a launch and the
// epoch grows with every launch, so stale contents can never match.
//
// Per tile: [META slots (scale / min,max as raw bits)] [W * 256 code slots], where
// thread t owns code slots w*256 + t and W = 32-bit words of codes per thread.
template <int B>
struct LL {
  static constexpr int W = B <= 2 ? 1 : B / 2;
};
template <int ALG>
struct MetaOf {
  static constexpr int N = ALG == kOnebit ? 1 : (ALG == kTernGrad ? 2 : 0);
};
template <int ALG, int B>
__device__ __forceinline__ constexpr int tile_slots() {
  return MetaOf<ALG>::N + LL<B>::W * kThreads;
}

__device__ __forceinline__ void ll_store(uint2* slot, uint32_t data, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(slot), "r"(data), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ uint2 ll_load(const uint2* slot) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(slot)
               : "memory");
  return v;
}

// Spin (bounded) until the slot carries this launch's epoch.  `v` holds a first
// load issued earlier so that several slots can be in flight before any spinning.
// The top bit of the epoch word is the sender's "I gave up" mark: a CTA whose own
// wait expired keeps sending (so nobody downstream has to wait out a timeout of
// its own) but marks what it sends, and a receiver that sees the mark gives up at
// once as well.  A CTA that has given up ("poisoned") touches neither the error
// feedback state nor the gradient any more.  (kGaveUp: sync.cuh)

__device__ __forceinline__ uint32_t ll_finish(const uint2* slot, uint2 v, const HpComm& cm,
                                              uint32_t* status, uint32_t code, WaitState& ws) {
  if (v.y == cm.epoch) return v.x;
  volatile int* poisoned = &ws.poisoned;
  if (*poisoned) return v.x;
  if ((v.y & ~kGaveUp) != cm.epoch) {
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (true) {
      v = ll_load(slot);
      if ((v.y & ~kGaveUp) == cm.epoch) break;
      // back off: thousands of threads polling L2 would slow the GEMMs of backward
      // that run next to this kernel while a peer is late
      if (polls > 4) __nanosleep(polls > 64 ? 400 : 100);
      if ((++polls & 63u) == 0 && (*poisoned || global_timer_ns() - t0 > cm.timeout_ns)) {
        atomicCAS(status, 0u, code);
        *poisoned = 1;
        break;
      }
    }
    if (cm.trace && threadIdx.x == 0) ws.spin_ns += global_timer_ns() - t0;
  }
  if (v.y == (cm.epoch | kGaveUp) && !*poisoned) {
    atomicCAS(status, 0u, code | HP_STATUS_UPSTREAM);
    *poisoned = 1;
  }
  return v.x;
}

template <int B>
__device__ __forceinline__ void pack_words(const uint32_t (&f)[kIter], uint32_t (&w)[LL<B>::W]) {
  if (B == 1) w[0] = f[0] | (f[1] << 4) | (f[2] << 8) | (f[3] << 12);
  else if (B == 2) w[0] = f[0] | (f[1] << 8) | (f[2] << 16) | (f[3] << 24);
  else if (B == 4) { w[0] = f[0] | (f[1] << 16); w[LL<B>::W - 1] = f[2] | (f[3] << 16); }
  else {
#pragma unroll
    for (int j = 0; j < kIter; ++j) w[j % LL<B>::W] = f[j];
  }
}
template <int B>
__device__ __forceinline__ void unpack_words(const uint32_t (&w)[LL<B>::W], uint32_t (&f)[kIter]) {
  if (B == 1) { f[0] = w[0] & 15u; f[1] = (w[0] >> 4) & 15u; f[2] = (w[0] >> 8) & 15u; f[3] = (w[0] >> 12) & 15u; }
  else if (B == 2) { f[0] = w[0] & 255u; f[1] = (w[0] >> 8) & 255u; f[2] = (w[0] >> 16) & 255u; f[3] = w[0] >> 24; }
  else if (B == 4) { f[0] = w[0] & 0xFFFFu; f[1] = w[0] >> 16; f[2] = w[LL<B>::W - 1] & 0xFFFFu; f[3] = w[LL<B>::W - 1] >> 16; }
  else {
#pragma unroll
    for (int j = 0; j < kIter; ++j) f[j] = w[j % LL<B>::W];
  }
}

// slots of tile t inside the payload that starts at `base`
template <int ALG, int B>
__device__ __forceinline__ uint2* tile_base(uint8_t* base, uint32_t t) {
  return reinterpret_cast<uint2*>(base) + (size_t)t * tile_slots<ALG, B>();
}

// Debug build (-DHIPRESS_DEBUG): every tile of payload slots a kernel is about to
// store into or poll is checked against the inbox it belongs to.  A tile outside it
// is recorded in the status word (HP_STATUS_BOUNDS | what) and skipped -- never
// touched.  In the normal build the check folds to `true`.
template <int ALG, int B>
__device__ __forceinline__ bool dbg_tile_ok(const BucketDev& bk, const void* inbox,
                                            const uint8_t* payload, uint32_t t, uint32_t* status,
                                            uint32_t what) {
#ifdef HIPRESS_DEBUG
  const uint8_t* lo = static_cast<const uint8_t*>(inbox);
  const uint64_t limit = bk.dbg_limit ? bk.dbg_limit : bk.inbox_bytes;
  const uint64_t end = (uint64_t)(payload - lo) + (uint64_t)(t + 1) * tile_slots<ALG, B>() * 8ull;
  if (payload < lo || end > limit) {
    atomicCAS(status, 0u, HP_STATUS_BOUNDS | what);
    return false;
  }
#endif
  return true;
}

// send one encoded tile: this thread's code words, and (thread 0) the metadata
template <int ALG, int B>
__device__ __forceinline__ void send_tile(uint8_t* base, uint32_t t, const uint32_t (&w)[LL<B>::W],
                                          const float (&meta)[2], uint32_t epoch) {
  uint2* tb = tile_base<ALG, B>(base, t);
  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < MetaOf<ALG>::N; ++k) ll_store(tb + k, __float_as_uint(meta[k]), epoch);
  }
#pragma unroll
  for (int k = 0; k < LL<B>::W; ++k)
    ll_store(tb + MetaOf<ALG>::N + k * kThreads + threadIdx.x, w[k], epoch);
}

// first (non-blocking) loads of a tile's slots
template <int ALG, int B>
struct TileRx {
  uint2 w[LL<B>::W];
  uint2 m[MetaOf<ALG>::N > 0 ? MetaOf<ALG>::N : 1];
};
template <int ALG, int B>
__device__ __forceinline__ void recv_issue(const uint8_t* base, uint32_t t, TileRx<ALG, B>& rx) {
  const uint2* tb = tile_base<ALG, B>(const_cast<uint8_t*>(base), t);
#pragma unroll
  for (int k = 0; k < MetaOf<ALG>::N; ++k) rx.m[k] = ll_load(tb + k);
#pragma unroll
  for (int k = 0; k < LL<B>::W; ++k) rx.w[k] = ll_load(tb + MetaOf<ALG>::N + k * kThreads + threadIdx.x);
}
// wait for whatever was not there yet, then decode into d[j][e]
template <int ALG, int B>
__device__ __forceinline__ void recv_finish(const uint8_t* base, uint32_t t, TileRx<ALG, B>& rx,
                                            const HpComm& cm, uint32_t* status, uint32_t code,
                                            WaitState& ws, float tau, float (&d)[kIter][4],
                                            float meta_scale = 1.0f) {
  const uint2* tb = tile_base<ALG, B>(const_cast<uint8_t*>(base), t);
  float meta[2] = {0.0f, 0.0f};
#pragma unroll
  for (int k = 0; k < MetaOf<ALG>::N; ++k)
    meta[k] = __uint_as_float(ll_finish(tb + k, rx.m[k], cm, status, code, ws));
  if (ALG == kOnebit) meta[0] = meta[0] * meta_scale;  // see decode_phase
  uint32_t w[LL<B>::W], f[kIter];
#pragma unroll
  for (int k = 0; k < LL<B>::W; ++k)
    w[k] = ll_finish(tb + MetaOf<ALG>::N + k * kThreads + threadIdx.x, rx.w[k], cm, status, code, ws);
  unpack_words<B>(w, f);
#pragma unroll
  for (int j = 0; j < kIter; ++j) decode_frag<ALG, B>(f[j], meta, tau, d[j]);
}

__device__ __forceinline__ uint32_t chunk_valid(uint32_t n, uint32_t chunk, int c) {
  const uint64_t start = (uint64_t)c * chunk;
  if (start >= n) return 0;
  const uint64_t rest = n - start;
  return (uint32_t)(rest < chunk ? rest : chunk);
}

// ------------------------------------------------------------ shared memory
constexpr int kStages = 2;  // tiles of g (+ r) in flight per CTA

struct FusedSmem {
  alignas(128) float g[kStages][kTile];
  alignas(128) float r[kStages][kTile];
  TileSmem tile;
  alignas(8) uint64_t full[kStages];
  WaitState ws;
};

// ------------------------------------------------ encode phases (ring hops / PS push)
// What one phase of the encode sequence does, as a function of topology.
struct PhaseSpec {
  int chunk;      // chunk of every tensor handled in this phase
  int in_slot;    // inbox slot to wait for and merge, or -1
  int ndst;       // payload goes to ranks (dst0 + q) % N, q < ndst
  int dst0;
  int dst_slot;   // slot index inside the destination inbox
  uint32_t salt;
};

template <int TOPO>
__device__ __forceinline__ PhaseSpec phase_spec(int ph, int N, int R) {
  PhaseSpec p;
  if (TOPO == HP_TOPO_RING) {
    p.chunk = (R - ph + N) % N;
    p.in_slot = ph > 0 ? ph - 1 : -1;
    if (ph < N - 1) {
      p.ndst = 1; p.dst0 = (R + 1) % N; p.dst_slot = ph;
    } else {
      p.ndst = N; p.dst0 = R; p.dst_slot = N - 1 + R;
    }
    p.salt = (uint32_t)(R * 256 + ph);
  } else {  // PS push: remote owners first, own chunk last
    p.chunk = (R + 1 + ph) % N;
    p.in_slot = -1;
    p.ndst = 1; p.dst0 = p.chunk; p.dst_slot = R;
    p.salt = (uint32_t)(R * 256);
  }
  return p;
}

struct TileRef {
  int seg;
  uint32_t t;   // tile of (seg, chunk)
  int m;        // valid elements in the tile
  size_t off;   // element offset of the tile inside the tensor
};

// Work distribution.  A launch is a sequence of phases (ring: N hops then N
// gathers; PS: N pushes, the server pass, N pulls); every phase visits the
// T = tiles_total tiles of one chunk of every tensor.  Tile i of phase ph is
// work item ph * T + i, and item w belongs to CTA w % G: the assignment keeps
// rotating across phases, so a bucket whose chunk has fewer tiles than there are
// CTAs still spreads its phases over the whole grid (the CTAs of later hops wait
// for their input while the earlier hops run elsewhere), and a chunk that is not
// a multiple of G tiles leaves no CTA idle for a whole phase.  Every CTA takes its
// items in increasing order, and an item only ever depends on a lower-numbered
// item of another GPU, so the lowest unfinished item can always run: the grid must
// fit the GPU (the launcher clamps it), nothing else is needed for progress.
struct Cursor {
  int phase, seg, chunk;
  uint32_t rot;          // (phase * T) % G
  uint32_t t, nvt, nv;   // next tile, valid tiles and valid elements of (seg, chunk)
};

__device__ __forceinline__ void cursor_enter_seg(const BucketDev& bk, int G, int b, Cursor& c) {
  if (c.seg >= bk.nseg) return;
  const SegDev& sg = bk.seg[c.seg];
  c.nv = chunk_valid(sg.n, sg.chunk, c.chunk);
  c.nvt = (c.nv + kTile - 1) / kTile;
  const uint32_t p = (c.rot + sg.tile_prefix) % (uint32_t)G;
  c.t = ((uint32_t)b + (uint32_t)G - p) % (uint32_t)G;
}

__device__ __forceinline__ void cursor_begin(const BucketDev& bk, int G, int b, int phase,
                                             int chunk, Cursor& c) {
  c.phase = phase;
  c.chunk = chunk;
  c.seg = 0;
  c.rot = (uint32_t)(((uint64_t)phase * bk.tiles_total) % (uint64_t)G);
  cursor_enter_seg(bk, G, b, c);
}

// next tile of the cursor's phase that belongs to this CTA; false when the phase is exhausted
__device__ __forceinline__ bool cursor_next(const BucketDev& bk, int G, int b, Cursor& c,
                                            TileRef& out) {
  while (c.seg < bk.nseg) {
    if (c.t < c.nvt) {
      const SegDev& sg = bk.seg[c.seg];
      const uint32_t left = c.nv - c.t * kTile;
      out.seg = c.seg;
      out.t = c.t;
      out.m = (int)(left < (uint32_t)kTile ? left : (uint32_t)kTile);
      out.off = (size_t)c.chunk * sg.chunk + (size_t)c.t * kTile;
      c.t += (uint32_t)G;
      return true;
    }
    ++c.seg;
    cursor_enter_seg(bk, G, b, c);
  }
  return false;
}

// a tile can be prefetched with a bulk copy when it is full and 16-byte aligned
__device__ __forceinline__ bool bulk_ok(const float* g, const float* r, int m) {
  return m == kTile && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(r)) & 15) == 0;
}

__device__ __forceinline__ void load_tile_smem(const float* sp, float (&x)[kIter][4]) {
#pragma unroll
  for (int j = 0; j < kIter; ++j) {
    const float4 v = *reinterpret_cast<const float4*>(sp + 4 * (j * kThreads + (int)threadIdx.x));
    x[j][0] = v.x; x[j][1] = v.y; x[j][2] = v.z; x[j][3] = v.w;
  }
}

// device-side timestamps (see HpComm.trace): word 0 first CTA start (min), 1 end of
// the last encode phase (max), 2 kernel end (max), 3 epoch, 4+ph end of phase ph
// (max over CTAs), 4+HP_TRACE_PHASES+ph nanoseconds thread 0 of every CTA spent
// polling for input in phase ph (sum over CTAs)
__device__ __forceinline__ void trace_mark(const HpComm& cm, int E, int which) {
  if (cm.trace && threadIdx.x == 0) {
    unsigned long long* t = reinterpret_cast<unsigned long long*>(cm.trace) + HP_TRACE_WORDS * E;
    const unsigned long long now = global_timer_ns();
    if (which == 0) atomicMin(t, now);
    else atomicMax(t + which, now);
    if (which == 2) t[3] = cm.epoch;
  }
}
__device__ __forceinline__ void trace_phase(const HpComm& cm, int E, int ph, WaitState& ws) {
  if (cm.trace && threadIdx.x == 0 && ph < HP_TRACE_PHASES) {
    unsigned long long* t = reinterpret_cast<unsigned long long*>(cm.trace) + HP_TRACE_WORDS * E;
    atomicMax(t + 4 + ph, (unsigned long long)global_timer_ns());
    atomicAdd(t + 4 + HP_TRACE_PHASES + ph, (unsigned long long)ws.spin_ns);
    ws.spin_ns = 0;
  }
}

template <int ALG, int B, int TOPO>
__device__ __forceinline__ void encode_phases(const BucketDev& bk, const HpComm& cm,
                                              const FusedParams& fp, FusedSmem& sm, int R, int E,
                                              uint32_t* status) {
  const int N = cm.nranks;
  const int G = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  uint8_t* my_inbox = reinterpret_cast<uint8_t*>(cm.inbox[R]);
  // prefetcher state: runs ahead of the consumer over the same tile sequence
  Cursor prod;
  cursor_begin(bk, G, b, 0, phase_spec<TOPO>(0, N, R).chunk, prod);
  bool prod_more = true;
  uint32_t issued = 0, consumed = 0;  // tiles prefetched / used through the bulk pipeline

  for (int ph = 0; ph < N; ++ph) {
    const PhaseSpec ps = phase_spec<TOPO>(ph, N, R);
    Cursor cons;
    cursor_begin(bk, G, b, ph, ps.chunk, cons);
    const size_t dst_off = (size_t)ps.dst_slot * bk.slot_bytes;
    const uint8_t* in_base =
        ps.in_slot >= 0 ? my_inbox + (size_t)ps.in_slot * bk.slot_bytes : nullptr;
    TileRef tr;
    while (cursor_next(bk, G, b, cons, tr)) {
      const SegDev& sg = bk.seg[tr.seg];
      // top up the prefetch pipeline (stages of finished tiles are free: the
      // previous tile ended with a CTA barrier)
      while (prod_more && issued - consumed < kStages) {
        TileRef pr;
        bool got = cursor_next(bk, G, b, prod, pr);
        while (!got && prod.phase + 1 < N) {  // run ahead across phases
          cursor_begin(bk, G, b, prod.phase + 1, phase_spec<TOPO>(prod.phase + 1, N, R).chunk,
                       prod);
          got = cursor_next(bk, G, b, prod, pr);
        }
        if (!got) {
          prod_more = false;
          break;
        }
        const SegDev& psg = bk.seg[pr.seg];
        const float* pg = psg.g + E * cm.emu_stride_g + pr.off;
        const float* prr = psg.r ? psg.r + E * cm.emu_stride_r + pr.off : nullptr;
        if (bulk_ok(pg, prr, pr.m)) {
          if (threadIdx.x == 0) {
            const int st = issued % kStages;
            mbar_expect_tx(&sm.full[st], (prr ? 2u : 1u) * kTile * 4u);
            bulk_load(sm.g[st], pg, kTile * 4u, &sm.full[st]);
            if (prr) bulk_load(sm.r[st], prr, kTile * 4u, &sm.full[st]);
          }
          ++issued;
        }
      }
      const int m = tr.m;
      const uint32_t t = tr.t;
      const float* gp = sg.g + E * cm.emu_stride_g + tr.off;
      float* rp = sg.r ? sg.r + E * cm.emu_stride_r + tr.off : nullptr;
      float x[kIter][4];
      // first loads of the incoming payload go out before anything waits
      TileRx<ALG, B> rx;
      const bool has_in = in_base && dbg_tile_ok<ALG, B>(bk, my_inbox, in_base + sg.pay_off, t, status, 1u);
      if (in_base && !has_in) sm.ws.poisoned = 1;
      if (has_in) recv_issue<ALG, B>(in_base + sg.pay_off, t, rx);
      const bool bulk = bulk_ok(gp, rp, m);
      int st = 0;
      if (bulk) {
        st = consumed % kStages;
        if (!sm.ws.poisoned &&
            !mbar_wait_bounded(&sm.full[st], (consumed / kStages) & 1, cm.timeout_ns, status,
                               HP_STATUS_TIMEOUT | (3u << 16) | (b & 255)))
          sm.ws.poisoned = 1;
        ++consumed;
        load_tile_smem(sm.g[st], x);
      } else {
        load_tile(gp, m, x);
      }
      if (has_in) {
        float d[kIter][4];
        recv_finish<ALG, B>(in_base + sg.pay_off, t, rx, cm, status,
                            HP_STATUS_TIMEOUT | (1u << 16) | ((uint32_t)ps.in_slot << 8) | (b & 255),
                            sm.ws, fp.P.tau, d);
#pragma unroll
        for (int j = 0; j < kIter; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[j][e] = x[j][e] + d[j][e];
      }
      if (rp) {
        float rr[kIter][4];
        if (bulk) load_tile_smem(sm.r[st], rr);
        else load_tile(rp, m, rr);
#pragma unroll
        for (int j = 0; j < kIter; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[j][e] = rr[j][e] + x[j][e];
      }
      float meta[2];
      uint32_t frag[kIter];
      encode_tile<ALG, B>(x, m, fp.P, sg.id, tr.off, fp.P.salt + ps.salt, sm.tile, meta, frag,
                          rp != nullptr);
      // after an expired wait the merged input is not a real partial sum: the error
      // feedback state keeps its last good contents
      const bool bad = *(volatile int*)&sm.ws.poisoned != 0;
      if (rp && !bad) {
        if (bulk) store_tile_full(rp, x);
        else store_tile(rp, m, x);
      }
      uint32_t words[LL<B>::W];
      pack_words<B>(frag, words);
      const uint32_t ep = cm.epoch | (bad ? kGaveUp : 0u);
      // one destination on a hop, every rank on the last one (a rolled loop: the
      // broadcast is one phase in N)
#pragma unroll 1
      for (int q = 0; q < ps.ndst; ++q) {
        int d = ps.dst0 + q;
        if (d >= N) d -= N;
        uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[d]) + dst_off + sg.pay_off;
        if (dbg_tile_ok<ALG, B>(bk, cm.inbox[d], dst, t, status, 2u))
          send_tile<ALG, B>(dst, t, words, meta, ep);
      }
      __syncthreads();  // the prefetch stage of this tile may be refilled from here on
    }
    trace_phase(cm, E, ph, sm.ws);
  }
}

// decode the reduced chunk `c` that arrives in inbox slot `slot` into the gradient;
// `phase` continues the work-item numbering of the encode phases
template <int ALG, int B>
__device__ __forceinline__ void decode_phase(const BucketDev& bk, const HpComm& cm,
                                             const FusedParams& fp, FusedSmem& sm, int R, int E,
                                             int phase, int slot, int c, uint32_t* status) {
  const int G = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  const uint8_t* sp = reinterpret_cast<const uint8_t*>(cm.inbox[R]) + (size_t)slot * bk.slot_bytes;
  const uint32_t code = HP_STATUS_TIMEOUT | (2u << 16) | ((uint32_t)slot << 8) | (b & 255);
  Cursor cur;
  cursor_begin(bk, G, b, phase, c, cur);
  bool more = true;
  while (more) {
    // first loads of a whole group of tiles go out before anything spins
    TileRef tr[kGroup];
    TileRx<ALG, B> rx[kGroup];
    int cnt = 0;
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      if (more) {
        more = cursor_next(bk, G, b, cur, tr[u]);
        if (more) {
          if (dbg_tile_ok<ALG, B>(bk, cm.inbox[R], sp + bk.seg[tr[u].seg].pay_off, tr[u].t, status, 3u)) {
            recv_issue<ALG, B>(sp + bk.seg[tr[u].seg].pay_off, tr[u].t, rx[u]);
          } else {
            sm.ws.poisoned = 1;   // ll_finish returns at once, nothing is stored
            rx[u] = TileRx<ALG, B>();
          }
          cnt = u + 1;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      if (u < cnt) {
        const SegDev& sg = bk.seg[tr[u].seg];
        float x[kIter][4];
        // onebit and TBQ decode to +-level or 0, so level * (1/N) is the same float
        // whether the level or the element is scaled; TernGrad's min + q * gap is not
        constexpr bool kFold = ALG != kTernGrad;
        recv_finish<ALG, B>(sp + sg.pay_off, tr[u].t, rx[u], cm, status, code, sm.ws,
                            kFold ? fp.P.tau * fp.inv_n : fp.P.tau, x, kFold ? fp.inv_n : 1.0f);
        if (!kFold) {
#pragma unroll
          for (int j = 0; j < kIter; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) x[j][e] = x[j][e] * fp.inv_n;
        }
        // a tile whose payload never arrived is left as it was (the local gradient)
        if (!*(volatile int*)&sm.ws.poisoned) {
          float* op = sg.out + E * cm.emu_stride_out + tr[u].off;
          if (tile_is_full_aligned(op, tr[u].m)) store_tile_full(op, x);
          else store_tile(op, tr[u].m, x);
        }
      }
    }
  }
}

__device__ __forceinline__ void fused_prologue(FusedSmem& sm) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&sm.full[i], 1);
    mbar_init_fence();
    sm.ws.poisoned = 0;
    sm.ws.spin_ns = 0;
  }
  __syncthreads();
}

// ------------------------------------------------------------------------ ring
template <int ALG, int B>
__global__ void __launch_bounds__(kThreads, 3)
ring_dense_kernel(const BucketDev bk, const HpComm cm, const FusedParams fp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
  const int N = cm.nranks;
  const int R = cm.emulate ? (int)blockIdx.y : cm.rank;
  const int E = cm.emulate ? (int)blockIdx.y : 0;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  fused_prologue(sm);
  trace_mark(cm, E, 0);
  encode_phases<ALG, B, HP_TOPO_RING>(bk, cm, fp, sm, R, E, status);
  trace_mark(cm, E, 1);
  // gather: rank src finalised chunk src+1
  for (int qq = 0; qq < N; ++qq) {
    const int src = (R + qq) % N;
    decode_phase<ALG, B>(bk, cm, fp, sm, R, E, N + qq, N - 1 + src, (src + 1) % N, status);
    trace_phase(cm, E, N + qq, sm.ws);
  }
  trace_mark(cm, E, 2);
}

// -------------------------------------------------------------------------- PS
template <int ALG, int B>
__global__ void __launch_bounds__(kThreads, 3)
ps_dense_kernel(const BucketDev bk, const HpComm cm, const FusedParams fp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
  TileSmem& s = sm.tile;
  const int N = cm.nranks;
  const int R = cm.emulate ? (int)blockIdx.y : cm.rank;
  const int E = cm.emulate ? (int)blockIdx.y : 0;
  const int G = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  uint32_t* status = reinterpret_cast<uint32_t*>(cm.status) + 4 * E;
  uint8_t* my_inbox = reinterpret_cast<uint8_t*>(cm.inbox[R]);
  fused_prologue(sm);
  trace_mark(cm, E, 0);

  // phases 0 .. N-1: push
  encode_phases<ALG, B, HP_TOPO_PS>(bk, cm, fp, sm, R, E, status);
  trace_mark(cm, E, 1);

  // phase N: server for chunk R: sum the N payloads in rank order, re-encode, broadcast
  {
    Cursor cur;
    cursor_begin(bk, G, b, N, R, cur);
    TileRef tr;
    const size_t dst_off = (size_t)(N + R) * bk.slot_bytes;
    while (cursor_next(bk, G, b, cur, tr)) {
      const SegDev& sg = bk.seg[tr.seg];
      const int m = tr.m;
      const uint32_t t = tr.t;
      const size_t coff = (size_t)t * kTile;  // offset inside the owned chunk
      float x[kIter][4];
      // the N pushes are polled two at a time: loads of the next source are in
      // flight while the current one is decoded
      TileRx<ALG, B> rx[2];
      if (!dbg_tile_ok<ALG, B>(bk, my_inbox, my_inbox + (size_t)(N - 1) * bk.slot_bytes + sg.pay_off, t,
                               status, 4u)) {
        sm.ws.poisoned = 1;
        continue;
      }
      recv_issue<ALG, B>(my_inbox + sg.pay_off, t, rx[0]);
      for (int q = 0; q < N; ++q) {
        if (q + 1 < N)
          recv_issue<ALG, B>(my_inbox + (size_t)(q + 1) * bk.slot_bytes + sg.pay_off, t,
                             rx[(q + 1) & 1]);
        float d[kIter][4];
        recv_finish<ALG, B>(my_inbox + (size_t)q * bk.slot_bytes + sg.pay_off, t, rx[q & 1], cm,
                            status, HP_STATUS_TIMEOUT | (1u << 16) | ((uint32_t)q << 8) | (b & 255),
                            sm.ws, fp.P.tau, d);
#pragma unroll
        for (int j = 0; j < kIter; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[j][e] = q > 0 ? x[j][e] + d[j][e] : d[j][e];
      }
      float* rp = sg.sr ? sg.sr + E * cm.emu_stride_sr + coff : nullptr;
      if (rp) {
        float rr[kIter][4];
        load_tile(rp, m, rr);
#pragma unroll
        for (int jj = 0; jj < kIter; ++jj)
#pragma unroll
          for (int e = 0; e < 4; ++e) x[jj][e] = rr[jj][e] + x[jj][e];
      }
      float meta[2];
      uint32_t frag[kIter];
      encode_tile<ALG, B>(x, m, fp.P, sg.id, (size_t)R * sg.chunk + coff,
                          fp.P.salt + (uint32_t)(R * 256 + 1), s, meta, frag, rp != nullptr);
      const bool bad = *(volatile int*)&sm.ws.poisoned != 0;
      if (rp && !bad) {
        if (tile_is_full_aligned(rp, m)) store_tile_full(rp, x);
        else store_tile(rp, m, x);
      }
      uint32_t words[LL<B>::W];
      pack_words<B>(frag, words);
      const uint32_t ep = cm.epoch | (bad ? kGaveUp : 0u);
#pragma unroll 1
      for (int q = 0; q < N; ++q) {
        int d = R + q;
        if (d >= N) d -= N;
        uint8_t* dst = reinterpret_cast<uint8_t*>(cm.inbox[d]) + dst_off + sg.pay_off;
        if (dbg_tile_ok<ALG, B>(bk, cm.inbox[d], dst, t, status, 5u))
          send_tile<ALG, B>(dst, t, words, meta, ep);
      }
    }
    trace_phase(cm, E, N, sm.ws);
  }

  // phases N+1 .. 2N: pull: decode every owner's reduced chunk
  for (int i = 0; i < N; ++i) {
    const int j = (R + i) % N;
    decode_phase<ALG, B>(bk, cm, fp, sm, R, E, N + 1 + i, N + j, j, status);
    trace_phase(cm, E, N + 1 + i, sm.ws);
  }
  trace_mark(cm, E, 2);
}

// ------------------------------------------------------------------ host side
static int build_bucket(int alg, int bits, const HpSeg* segs, int nseg, int nranks,
                        BucketDev& bk) {
  if (nseg < 1 || nseg > HP_MAX_SEGS || nranks < 1 || nranks > HP_MAX_RANKS) return HP_ERR_BAD_ARG;
  uint64_t pay = 0, tiles = 0;
  for (int i = 0; i < nseg; ++i) {
    const uint64_t n = segs[i].n;
    if (n == 0 || n > 0xFFFFF000ull) return HP_ERR_BAD_ARG;
    const uint64_t per = (n + nranks - 1) / nranks;
    const uint64_t chunk = align_up(per, kTile);
    SegDev& d = bk.seg[i];
    d.g = static_cast<const float*>(segs[i].g);
    d.r = static_cast<float*>(segs[i].r);
    d.out = static_cast<float*>(segs[i].out);
    d.sr = static_cast<float*>(segs[i].sr);
    d.n = (uint32_t)n;
    d.chunk = (uint32_t)chunk;
    d.tiles = (uint32_t)(chunk / kTile);
    d.tile_prefix = (uint32_t)tiles;
    d.pay_off = (uint32_t)pay;
    d.id = segs[i].id;
    tiles += d.tiles;
    {
      const uint64_t words = bits <= 2 ? 1 : bits / 2;
      const uint64_t slots = dense_meta_floats(alg) + words * kThreads;  // per tile
      pay += align_up((chunk / kTile) * slots * 8, 128);
    }
    if (pay > 0xFFFFFFFFull || tiles > 0x7FFFFFFFull) return HP_ERR_TOO_LARGE;
  }
  bk.nseg = nseg;
  bk.tiles_total = (uint32_t)tiles;
  bk.slot_bytes = pay;
  bk.inbox_bytes = 0;
  bk.dbg_limit = 0;
  return 0;
}

static int num_slots(int topo, int nranks) {
  return topo == HP_TOPO_RING ? 2 * nranks - 1 : 2 * nranks;
}
// phases of one launch (see Cursor)
static int num_phases(int topo, int nranks) {
  return topo == HP_TOPO_RING ? 2 * nranks : 2 * nranks + 1;
}

template <int ALG, int B>
static int launch_fused(int topo, const BucketDev& bk, const HpComm& cm, const FusedParams& fp,
                        int ctas, cudaStream_t st) {
  void (*kern)(const BucketDev, const HpComm, const FusedParams) =
      topo == HP_TOPO_RING ? ring_dense_kernel<ALG, B> : ps_dense_kernel<ALG, B>;
  const size_t smem = sizeof(FusedSmem);
  // per (topology, device): the shared-memory attribute is sticky, and the number of
  // CTAs the GPU can hold at once does not change
  static int resident[2][64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  int cap = (dev >= 0 && dev < 64) ? resident[topo][dev] : 0;
  if (cap == 0) {
    e = cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    int sms = 0, per_sm = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
    if (e != cudaSuccess) return (int)e;
    cap = per_sm * sms;
    if (cap < 1) return HP_ERR_RESIDENCY;
    if (dev >= 0 && dev < 64) resident[topo][dev] = cap;
  }
  if (cm.emulate) {
    if ((long long)ctas * cm.nranks > (long long)cap) return HP_ERR_RESIDENCY;
    void* args[] = {(void*)&bk, (void*)&cm, (void*)&fp};
    e = cudaLaunchCooperativeKernel((const void*)kern, dim3(ctas, cm.nranks), dim3(kThreads),
                                    args, smem, st);
    return (int)e;
  }
  // a CTA may wait for a peer's CTA of any index (the work items rotate over the
  // grid), so the whole grid has to fit the GPU once nothing else runs on it
  if (ctas > cap) ctas = cap;
  kern<<<dim3(ctas, 1), kThreads, smem, st>>>(bk, cm, fp);
  return (int)cudaGetLastError();
}

}  // namespace hipress

using namespace hipress;

// debug build: see hp_cuda_debug_set_inbox_limit
static uint64_t g_dbg_inbox_limit = 0;

extern "C" {

// 1 when the library was built with -DHIPRESS_DEBUG (per-access bounds checks on)
int hp_cuda_debug_build(void) {
#ifdef HIPRESS_DEBUG
  return 1;
#else
  return 0;
#endif
}

// Debug build only: make the kernels' bounds checks treat every inbox as `bytes`
// long (0: its real size), so a test can make the checks fire without any access
// actually leaving the allocation.  Returns HP_ERR_BAD_ARG in the normal build.
int hp_cuda_debug_set_inbox_limit(uint64_t bytes) {
#ifdef HIPRESS_DEBUG
  g_dbg_inbox_limit = bytes;
  return 0;
#else
  (void)bytes;
  return HP_ERR_BAD_ARG;
#endif
}

// bytes of one rank's inbox for a bucket of tensors with the given sizes
int hp_fused_dense_layout(int topo, int alg, int bits, const uint64_t* ns, int nseg, int nranks,
                          uint64_t* inbox_bytes, uint64_t* slot_bytes, uint32_t* tiles_total) {
  if (nseg < 1 || nseg > HP_MAX_SEGS) return HP_ERR_BAD_ARG;
  HpSeg segs[HP_MAX_SEGS] = {};
  for (int i = 0; i < nseg; ++i) segs[i].n = ns[i];
  BucketDev bk;
  int rc = build_bucket(alg, bits, segs, nseg, nranks, bk);
  if (rc) return rc;
  if (inbox_bytes) *inbox_bytes = bk.slot_bytes * (uint64_t)num_slots(topo, nranks);
  if (slot_bytes) *slot_bytes = bk.slot_bytes;
  if (tiles_total) *tiles_total = bk.tiles_total;
  return 0;
}

// elements of the server residual a PS owner keeps for a tensor of n elements
uint64_t hp_fused_chunk_elems(uint64_t n, int nranks) {
  return align_up((n + nranks - 1) / nranks, kTile);
}

int hp_cuda_fused_dense(int topo, int alg, int bits, const HpSeg* segs, int nseg,
                        const HpComm* comm, float tau, uint64_t seed, uint32_t step, uint32_t salt,
                        int ctas, void* stream) {
  if (topo != HP_TOPO_RING && topo != HP_TOPO_PS) return HP_ERR_BAD_ARG;
  if (!comm || ctas < 1 || ctas > 65535) return HP_ERR_BAD_ARG;
  BucketDev bk;
  int rc = build_bucket(alg, bits, segs, nseg, comm->nranks, bk);
  if (rc) return rc;
  bk.inbox_bytes = bk.slot_bytes * (uint64_t)num_slots(topo, comm->nranks);
  bk.dbg_limit = g_dbg_inbox_limit;
  {  // never more CTAs than work items
    const uint64_t items = (uint64_t)bk.tiles_total * (uint64_t)num_phases(topo, comm->nranks);
    if ((uint64_t)ctas > items) ctas = (int)items;
  }
  FusedParams fp;
  fp.P = DenseParams{tau, step, salt, (uint32_t)seed, (uint32_t)(seed >> 32)};
  fp.inv_n = 1.0f / (float)comm->nranks;
  cudaStream_t st = (cudaStream_t)stream;
#define CALL(A, B) return launch_fused<A, B>(topo, bk, *comm, fp, ctas, st)
  if (alg == kOnebit && bits == 1) { CALL(kOnebit, 1); }
  else if (alg == kTbq && bits == 2) { CALL(kTbq, 2); }
  else if (alg == kTernGrad && bits == 1) { CALL(kTernGrad, 1); }
  else if (alg == kTernGrad && bits == 2) { CALL(kTernGrad, 2); }
  else if (alg == kTernGrad && bits == 4) { CALL(kTernGrad, 4); }
  else if (alg == kTernGrad && bits == 8) { CALL(kTernGrad, 8); }
#undef CALL
  return HP_ERR_BAD_ARG;
}

}  // extern "C"
