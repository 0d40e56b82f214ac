// Small CUDA runtime helpers used by host-only translation units (kept here so those files need no CUDA headers).
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include "../common/log.h"
#include "hccl/hccl_types.h"

namespace hccl {

HcclResult CudaSetDeviceChecked(int dev)
{
    cudaError_t e = cudaSetDevice(dev);
    if (e != cudaSuccess) { HCCL_ERROR("cudaSetDevice(%d): %s", dev, cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

HcclResult CudaStreamSync(cudaStream_t s) { return cudaStreamSynchronize(s) == cudaSuccess ? HCCL_SUCCESS : HCCL_E_RUNTIME; }

bool CudaStreamIsCapturing(cudaStream_t s)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    return st != cudaStreamCaptureStatusNone;
}

HcclResult CudaMemcpyAsyncD2D(void *dst, const void *src, uint64_t bytes, cudaStream_t s)
{
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) { HCCL_ERROR("cudaMemcpyAsync: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

HcclResult CudaMemsetDevice(void *dst, int v, uint64_t bytes)
{
    cudaError_t e = cudaMemset(dst, v, bytes);
    if (e != cudaSuccess) { HCCL_ERROR("cudaMemset: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

void NvtxPush(const char *name) { nvtxRangePushA(name); }
void NvtxPop() { nvtxRangePop(); }

}  // namespace hccl
