// Symmetric-memory plumbing for the fused kernels: a device arena per rank that
// every other rank of the box maps through CUDA IPC, plus small device utilities
// (peer-store bandwidth probe, bounded-wait self test).
//
// Reference parity: the reference moves compressed payloads with MPI/NCCL/PS-Lite
// between hosts (README.md:58,153); on one NVSwitch box the transport is peer
// memory written from inside the kernels, and this file only sets the mappings up.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "hipress/capi.h"
#include "sync.cuh"

namespace hipress {

__global__ void peer_store_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                  uint64_t n16) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride)
    dst[i] = src[i];
}

// Waits on a flag nobody sets; used to show that an expired wait reports a
// status word and returns instead of hanging.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                                  uint32_t* status) {
  __shared__ WaitState ws;
  wait_init(ws);
  wait_flag(flag, epoch, timeout_ns, status, HP_STATUS_TIMEOUT | (7u << 16), ws);
  // a second wait after a timeout must return immediately
  wait_flag(flag, epoch, timeout_ns, status, HP_STATUS_TIMEOUT | (8u << 16), ws);
}

__global__ void set_flag_kernel(uint32_t* flag, uint32_t v) {
  __threadfence_system();
  st_release_sys(flag, v);
}

}  // namespace hipress

using namespace hipress;

extern "C" {

int hp_cuda_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

const char* hp_cuda_error_string(int code) {
  if (code == HP_ERR_BAD_ARG) return "hipress: bad argument";
  if (code == HP_ERR_TOO_LARGE)
    return "hipress: input larger than this entry point supports (bucket or element limit)";
  if (code == HP_ERR_RESIDENCY) return "hipress: emulated ranks would not be co-resident";
  return cudaGetErrorString((cudaError_t)code);
}

// Arena allocated with cudaMalloc so that it can be exported through CUDA IPC
// (memory from a framework's caching allocator is not always exportable).
int hp_cuda_arena_alloc(uint64_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  // the zeroes must be in place before any peer can learn the address
  return (int)cudaDeviceSynchronize();
}
int hp_cuda_arena_free(void* ptr) { return (int)cudaFree(ptr); }

int hp_cuda_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }
int hp_cuda_ipc_export(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int hp_cuda_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int hp_cuda_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

// same-process peers (one process driving several GPUs, used by tests)
int hp_cuda_enable_peer(int dev, int peer) {
  int cur = 0;
  cudaGetDevice(&cur);
  cudaError_t e = cudaSetDevice(dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaDeviceEnablePeerAccess(peer, 0);
  cudaSetDevice(cur);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

int hp_cuda_peer_store(const void* src, void* dst, uint64_t bytes, int ctas, void* stream) {
  if (bytes % 16) return HP_ERR_BAD_ARG;
  if (ctas <= 0) ctas = 148 * 4;
  peer_store_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes / 16);
  return (int)cudaGetLastError();
}

int hp_cuda_wait_probe(const void* flag, uint32_t epoch, uint64_t timeout_ns, void* status,
                       void* stream) {
  wait_probe_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(static_cast<const uint32_t*>(flag), epoch,
                                                        timeout_ns, static_cast<uint32_t*>(status));
  return (int)cudaGetLastError();
}

int hp_cuda_set_flag(void* flag, uint32_t v, void* stream) {
  set_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(static_cast<uint32_t*>(flag), v);
  return (int)cudaGetLastError();
}

}  // extern "C"
