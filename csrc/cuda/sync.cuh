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

// Thread 0 polls until *flag == epoch, at most timeout_ns (and at most a fixed
// number of polls); all threads of the CTA leave together.
__device__ __forceinline__ void wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                                          uint32_t* status, uint32_t code, WaitState& ws) {
  if (threadIdx.x == 0 && !ws.poisoned) {
    if (ld_acquire_sys(flag) != epoch) {
      const uint64_t t0 = global_timer_ns();
      const uint64_t max_polls = timeout_ns / 8 + 4096;
      uint64_t polls = 0;
      while (ld_acquire_sys(flag) != epoch) {
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
  }
  __syncthreads();
}

}  // namespace hipress
