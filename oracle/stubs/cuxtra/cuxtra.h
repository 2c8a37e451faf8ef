// Stand-in for the reference's un-vendored `cuxtra` dependency (3rdparty/cuxtra is an empty submodule).
// TEST / BASELINE INFRASTRUCTURE: exists only so that the reference's own level-1 CUDA HAL and shim compile
// into oracle/_ref/ (libhalcuda_ref.so, libshimcuda_ref.so).
//
// Only the four argument-introspection calls used by platforms/cuda/hal/src/common/cuda_command.cpp:57-113
// are provided, over the public driver API (cuFuncGetParamInfo, CUDA >= 12.4).  The driver-internal hooks
// that the reference's level 2 / level 3 need (instrumentation memory, trap handlers, timeslices) cannot be
// reproduced; those sources are not part of this build.
#pragma once
#include <cstddef>
#include "xsched/cuda/hal/common/cuda.h"
#include "xsched/cuda/hal/common/driver.h"

// The handle the runtime passes to cuLaunchKernel is accepted as is by cuFuncGetParamInfo.
inline CUfunction cuXtraKernelGetFunction(CUkernel kernel) { return (CUfunction)kernel; }

inline size_t cuXtraGetParamCount(CUfunction func) {
    size_t n = 0, off = 0, size = 0;
    while (xsched::cuda::Driver::FuncGetParamInfo(func, n, &off, &size) == CUDA_SUCCESS) ++n;
    return n;
}

inline void cuXtraGetParamInfo(CUfunction func, size_t index, size_t *offset, size_t *size, void *) {
    size_t off = 0, sz = 0;
    xsched::cuda::Driver::FuncGetParamInfo(func, index, &off, &sz);
    if (offset) *offset = off;
    if (size) *size = sz;
}

inline void cuXtraGetExtraBuffer(void **extra, void **buffer, size_t *size) {
    *buffer = nullptr;
    *size = 0;
    if (extra == nullptr) return;
    for (int i = 0; extra[i] != CU_LAUNCH_PARAM_END && i < 16; i += 2) {
        if (extra[i] == CU_LAUNCH_PARAM_BUFFER_POINTER) *buffer = extra[i + 1];
        else if (extra[i] == CU_LAUNCH_PARAM_BUFFER_SIZE) *size = *(size_t *)extra[i + 1];
    }
}
