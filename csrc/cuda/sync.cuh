// Cross-GPU signalling primitives: system-scope release/acquire flag words and a
// wait that can never hang the GPU.  A wait that expires records a status word
// for the host, marks the CTA as "poisoned" (later waits return at once) and
// lets the kernel run to completion inside its own buffers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hipress {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct WaitState {
  int poisoned;
  unsigned long long spin_ns;  // time thread 0 spent polling (only kept when tracing)
};

__device__ __forceinline__ void wait_init(WaitState& ws) {
  if (threadIdx.x == 0) {
    ws.poisoned = 0;
    ws.spin_ns = 0;
  }
  __syncthreads();
}

// The top bit of a flag (and of the epoch word of a payload slot) is the sender's
// "I gave up" mark: a kernel whose own wait expired still releases its flags, so
// nobody downstream has to wait out a timeout of its own, but marks them; a waiter
// that sees the mark records HP_STATUS_UPSTREAM and gives up at once as well.
// Epochs therefore use 31 bits.
constexpr uint32_t kGaveUp = 0x80000000u;

// Thread 0 polls until *flag == epoch (mark ignored), at most timeout_ns (and at
// most a fixed number of polls); all threads of the CTA leave together.
__device__ __forceinline__ void wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                                          uint32_t* status, uint32_t code, WaitState& ws) {
  if (threadIdx.x == 0 && !ws.poisoned) {
    uint32_t v = ld_acquire_sys(flag);
    if ((v & ~kGaveUp) != epoch) {
      const uint64_t t0 = global_timer_ns();
      const uint64_t max_polls = timeout_ns / 8 + 4096;
      uint64_t polls = 0;
      while (((v = ld_acquire_sys(flag)) & ~kGaveUp) != epoch) {
        ++polls;
        if ((polls & 63) == 0 &&
            (global_timer_ns() - t0 > timeout_ns || polls > max_polls)) {
          atomicCAS(status, 0u, code);
          ws.poisoned = 1;
          break;
        }
        __nanosleep(32);
      }
    }
    if (v == (epoch | kGaveUp) && !ws.poisoned) {
      atomicCAS(status, 0u, code | 0x40000000u);  // HP_STATUS_UPSTREAM
      ws.poisoned = 1;
    }
  }
  __syncthreads();
}

// Barrier over the CTAs of one cooperative launch that play one rank: `count` is a
// word that was zero when the kernel started, `gen` the caller's running barrier
// number (same in every CTA), `ctas` how many CTAs take part.  Bounded like every
// other wait: on expiry the status word is set and the CTA goes on (its later
// barriers return at once), so a kernel can never hang on a barrier.  All CTAs are
// co-resident (cooperative launch), which is what makes waiting for one another
// legitimate.
__device__ __forceinline__ void grid_barrier(uint32_t* count, uint32_t& gen, uint32_t ctas,
                                             uint64_t timeout_ns, uint32_t* status, uint32_t code,
                                             WaitState& ws) {
  __syncthreads();
  ++gen;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(count, 1u);   // a CTA that gave up still arrives, it just does not wait
    const uint32_t target = gen * ctas;
    volatile uint32_t* vc = count;
    if (!ws.poisoned && *vc < target) {
      const uint64_t t0 = global_timer_ns();
      uint64_t polls = 0;
      while (*vc < target) {
        if ((++polls & 255) == 0 && global_timer_ns() - t0 > timeout_ns) {
          atomicCAS(status, 0u, code);
          ws.poisoned = 1;
          break;
        }
      }
    }
    __threadfence();
  }
  __syncthreads();
}

}  // namespace hipress
