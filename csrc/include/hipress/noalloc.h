// Allocation-free entry point for the top-k (DGC / GradDrop) encoder.
//
// hp_cuda_sparse_encode() needs about 48 KB of scratch (three radix histograms
// and a few counters) that its caller has to allocate on the device.  Some
// callers are not in a position to allocate: code that runs while a memory pool
// is frozen, inside a framework callback that forbids allocator re-entry, or in a
// process whose device memory has been handed out in full to another allocator,
// where a cudaMalloc would fail or stall the device.  For them this variant keeps
// the scratch in a fixed array inside the library's device image instead.
//
// What a caller has to know:
//   * Inputs and outputs are still the caller's; only the scratch is internal.
//     The function calls no cudaMalloc / cudaFree and no allocating library
//     routine.
//   * The scratch array exists once per GPU that loads the library, from load
//     until the process exits (hp_cuda_noalloc_scratch_bytes() bytes).
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current).  Make that first call
//     before any stream capture begins, from one thread.
//   * All calls on a device share the one array, and it keeps whatever the last
//     call left in it; the function clears the words that must start at zero
//     itself, on the given stream.  Two calls that overlap on the GPU (different
//     streams, no ordering between them) would corrupt each other's histograms:
//     order them.
//   * At most HP_NOALLOC_MAX_ELEMS elements per call; larger inputs are refused
//     with HP_ERR_TOO_LARGE before anything is launched.
//
// The reference (mark14wu/hipress) has no counterpart of this function.
#pragma once
#include <stdint.h>

#define HP_NOALLOC_MAX_ELEMS (1ull << 28)  // 1 GiB of fp32 gradient

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as hp_cuda_sparse_encode(), minus the workspace.
int hp_cuda_sparse_encode_noalloc(int alg, const float* g, float* a, float* u, uint64_t n,
                                  uint64_t k, uint64_t kmax, float momentum, int update,
                                  uint8_t* out, int max_ctas, void* stream);

// bytes of device memory the internal scratch array occupies per GPU
uint64_t hp_cuda_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
