// SM partitioning for communication kernels: a CUDA green context that owns a
// small group of SMs and a stream bound to it.  Fused synchronisation kernels
// launched on that stream stay on those SMs (several CTAs per SM, enough to pull
// a large share of HBM bandwidth), so they overlap backward's GEMMs instead of
// taking one CTA slot on every SM of the chip.  The driver entry points are
// resolved at run time; when green contexts are unavailable the caller falls
// back to an ordinary high-priority stream.
//
// No counterpart in the reference: Horovod-era runtimes overlap by running NCCL
// on a separate stream and let the hardware arbitrate.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hipress/capi.h"

namespace {

template <typename F>
bool resolve(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

}  // namespace

extern "C" {

// Creates a stream restricted to >= min_sms SMs.  Returns 0 and fills stream_out /
// sms_out on success; HP_ERR_BAD_ARG when the driver lacks the feature or refuses.
int hp_cuda_partition_stream_create(int device, int min_sms, int priority, void** stream_out,
                                    int* sms_out, void** green_ctx_out) {
  typedef CUresult (*GetDevResource_t)(CUdevice, CUdevResource*, CUdevResourceType);
  typedef CUresult (*SplitByCount_t)(CUdevResource*, unsigned int*, const CUdevResource*,
                                     CUdevResource*, unsigned int, unsigned int);
  typedef CUresult (*GenerateDesc_t)(CUdevResourceDesc*, CUdevResource*, unsigned int);
  typedef CUresult (*GreenCtxCreate_t)(CUgreenCtx*, CUdevResourceDesc, CUdevice, unsigned int);
  typedef CUresult (*GreenCtxStreamCreate_t)(CUstream*, CUgreenCtx, unsigned int, int);
  typedef CUresult (*DeviceGet_t)(CUdevice*, int);
  GetDevResource_t getRes;
  SplitByCount_t split;
  GenerateDesc_t genDesc;
  GreenCtxCreate_t gcreate;
  GreenCtxStreamCreate_t gstream;
  DeviceGet_t devGet;
  if (!resolve("cuDeviceGetDevResource", getRes) || !resolve("cuDevSmResourceSplitByCount", split) ||
      !resolve("cuDevResourceGenerateDesc", genDesc) || !resolve("cuGreenCtxCreate", gcreate) ||
      !resolve("cuGreenCtxStreamCreate", gstream) || !resolve("cuDeviceGet", devGet))
    return HP_ERR_BAD_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return HP_ERR_BAD_ARG;
  cudaFree(0);  // make sure the primary context exists
  CUdevice dev;
  if (devGet(&dev, device) != CUDA_SUCCESS) return HP_ERR_BAD_ARG;
  CUdevResource all, group, rest;
  if (getRes(dev, &all, CU_DEV_RESOURCE_TYPE_SM) != CUDA_SUCCESS) return HP_ERR_BAD_ARG;
  unsigned int ngroups = 1;
  if (split(&group, &ngroups, &all, &rest, 0, (unsigned int)min_sms) != CUDA_SUCCESS || ngroups < 1)
    return HP_ERR_BAD_ARG;
  CUdevResourceDesc desc;
  if (genDesc(&desc, &group, 1) != CUDA_SUCCESS) return HP_ERR_BAD_ARG;
  CUgreenCtx g;
  if (gcreate(&g, desc, dev, CU_GREEN_CTX_DEFAULT_STREAM) != CUDA_SUCCESS) return HP_ERR_BAD_ARG;
  CUstream s;
  if (gstream(&s, g, CU_STREAM_NON_BLOCKING, priority) != CUDA_SUCCESS) return HP_ERR_BAD_ARG;
  *stream_out = (void*)s;
  if (sms_out) *sms_out = (int)group.sm.smCount;
  if (green_ctx_out) *green_ctx_out = (void*)g;
  return 0;
}

int hp_cuda_partition_stream_destroy(void* stream, void* green_ctx) {
  typedef CUresult (*GreenCtxDestroy_t)(CUgreenCtx);
  if (stream) cudaStreamDestroy((cudaStream_t)stream);
  GreenCtxDestroy_t gdestroy;
  if (green_ctx && resolve("cuGreenCtxDestroy", gdestroy)) gdestroy((CUgreenCtx)green_ctx);
  return 0;
}

}  // extern "C"
