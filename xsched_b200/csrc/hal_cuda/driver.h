// The real CUDA driver, opened by path with dlopen so that the HAL keeps working when the interposing
// shim is what the process sees as libcuda.so.1.  Only the entry points the preemption path needs are
// resolved (the reference resolves all of cuda.h through generated wrappers,
// platforms/cuda/hal/include/xsched/cuda/hal/common/driver.h:16-30).
#pragma once
#include <cuda.h>
#include <string>

namespace xsched::cuda {

struct DriverApi {
    void *handle = nullptr;
    std::string path;
#define XSCHED_DRV(name) decltype(&::name) name = nullptr;
    XSCHED_DRV(cuInit)
    XSCHED_DRV(cuGetErrorString)
    XSCHED_DRV(cuCtxGetCurrent)
    XSCHED_DRV(cuCtxSetCurrent)
    XSCHED_DRV(cuCtxPushCurrent)
    XSCHED_DRV(cuCtxPopCurrent)
    XSCHED_DRV(cuCtxGetDevice)
    XSCHED_DRV(cuCtxGetStreamPriorityRange)
    XSCHED_DRV(cuCtxSynchronize)
    XSCHED_DRV(cuDeviceGetAttribute)
    XSCHED_DRV(cuStreamGetCtx)
    XSCHED_DRV(cuStreamGetFlags)
    XSCHED_DRV(cuStreamSynchronize)
    XSCHED_DRV(cuStreamQuery)
    XSCHED_DRV(cuStreamCreateWithPriority)
    XSCHED_DRV(cuStreamDestroy)
    XSCHED_DRV(cuStreamWaitEvent)
    XSCHED_DRV(cuStreamWriteValue32)
    XSCHED_DRV(cuStreamWriteValue64)
    XSCHED_DRV(cuMemHostAlloc)
    XSCHED_DRV(cuMemHostGetDevicePointer)
    XSCHED_DRV(cuMemFreeHost)
    XSCHED_DRV(cuMemAlloc)
    XSCHED_DRV(cuMemFree)
    XSCHED_DRV(cuMemsetD32)
    XSCHED_DRV(cuMemsetD8Async)
    XSCHED_DRV(cuMemsetD32Async)
    XSCHED_DRV(cuMemcpyAsync)
    XSCHED_DRV(cuMemcpyHtoDAsync)
    XSCHED_DRV(cuMemcpyDtoHAsync)
    XSCHED_DRV(cuMemcpyDtoDAsync)
    XSCHED_DRV(cuLaunchKernel)
    XSCHED_DRV(cuLaunchKernelEx)
    XSCHED_DRV(cuLaunchHostFunc)
    XSCHED_DRV(cuFuncGetParamInfo)
    XSCHED_DRV(cuPointerGetAttribute)
    XSCHED_DRV(cuEventCreate)
    XSCHED_DRV(cuEventDestroy)
    XSCHED_DRV(cuEventRecord)
    XSCHED_DRV(cuEventQuery)
    XSCHED_DRV(cuEventSynchronize)
    XSCHED_DRV(cuGetProcAddress)
#undef XSCHED_DRV
    /// Raw symbol lookup in the real library (nullptr if absent).
    void *Sym(const char *name) const;
};

/// Loads on first use; ends the process with a clear message when no real driver can be found
/// (there is no CPU fallback for the CUDA path).
const DriverApi &Driver();
/// Path resolution only (for tests): XSCHED_CUDA_LIB, then the usual system directories, skipping
/// any file that is this interposer itself.  Empty when nothing is found.
std::string FindRealDriver();

const char *ErrorString(CUresult r);

} // namespace xsched::cuda

#define CUDA_ASSERT(call)                                                                       \
    do {                                                                                        \
        const CUresult r_ = (call);                                                             \
        if (UNLIKELY(r_ != CUDA_SUCCESS)) XERRO("CUDA driver call failed: %s -> %d (%s)", #call, (int)r_, ::xsched::cuda::ErrorString(r_)); \
    } while (0)
