// C ABI of the native libraries (loaded from Python with ctypes).
//   libhipress_cpu.so   hp_cpu_*  : CPU oracle / host-transport compressor
//   libhipress_cuda.so  hp_cuda_* : sm_100a kernels and the fused CaSync runtime
// Every hp_cuda_* function returns 0 on success, a cudaError_t value (> 0) when
// the CUDA runtime reported one, or one of the negative HP_ERR_* codes below.
#pragma once
#include <stdint.h>

#define HP_ERR_BAD_ARG (-1)
#define HP_ERR_TOO_LARGE (-2)
#define HP_ERR_RESIDENCY (-3)  // emulated ranks would not all be co-resident

#define HP_MAX_RANKS 8
#define HP_MAX_SEGS 40

// topology ids
#define HP_TOPO_RING 0
#define HP_TOPO_PS 1

// device-side trace of the fused dense kernels (HpComm.trace): uint64 words per rank
#define HP_TRACE_PHASES 20
#define HP_TRACE_WORDS (4 + 2 * HP_TRACE_PHASES)

// status words written by a kernel whose bounded wait expired
#define HP_STATUS_OK 0u
#define HP_STATUS_TIMEOUT 0x80000000u  // | (phase << 16) | (slot << 8) | cta
#define HP_STATUS_BOUNDS 0x20000000u    // debug build: an index left its buffer (recorded, skipped) | site
#define HP_STATUS_UPSTREAM 0x40000000u  // or-ed in: the sender of this input had given up first

#ifdef __cplusplus
extern "C" {
#endif

// One tensor of a bucket.  Pointers are device pointers of the calling rank.
typedef struct {
  void* g;      // fp32 gradient [n]
  void* r;      // fp32 residual [n] or NULL (no error feedback)
  void* out;    // fp32 averaged result [n]; may alias g
  void* sr;     // PS topology: server residual for the owned chunk [chunk] or NULL
  uint64_t n;
  uint32_t id;  // tensor id (random stream selector)
  uint32_t pad;
} HpSeg;

// Symmetric-memory view of the job as seen from the calling rank.
typedef struct {
  int32_t nranks;
  int32_t rank;
  int32_t emulate;      // 1: one launch plays all ranks on this GPU (gridDim.y = nranks)
  uint32_t epoch;       // strictly increasing per launch on one (inbox, flags) pair
  uint64_t timeout_ns;  // bound of every flag wait
  void* inbox[HP_MAX_RANKS];   // rank q's inbox, mapped into this process
  void* flags[HP_MAX_RANKS];   // rank q's flag words (uint32), mapped into this process
  void* status;                // this rank's status words (emulate: nranks * 4 words)
  // emulation only: element strides between consecutive ranks' copies of g / r / out / sr
  int64_t emu_stride_g, emu_stride_r, emu_stride_out, emu_stride_sr;
  // optional device-side timing of the fused dense kernels: HP_TRACE_WORDS uint64 per rank
  // played by the launch {first CTA start (min), last encode phase end (max), last CTA end
  // (max), epoch, end of phase p (max over CTAs) x HP_TRACE_PHASES, time spent polling for
  // input in phase p (thread 0, summed over CTAs) x HP_TRACE_PHASES}, %globaltimer
  // nanoseconds; the host presets {UINT64_MAX, 0, 0, ...}.  NULL = off.
  void* trace;
} HpComm;

#ifdef __cplusplus
}
#endif
