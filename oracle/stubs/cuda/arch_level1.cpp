// Queue factory for the reference's CUDA HAL restricted to level 1 — BASELINE INFRASTRUCTURE.
// Replaces platforms/cuda/hal/src/arch/arch.cpp in the oracle/_ref build: that file also instantiates the
// level-2/3 queues (SASS guardians for sm35/70/86, trap handlers), which need the un-vendored `cuxtra`
// library.  For compute capability 10.0 the reference's own dispatch ends in its default branch,
// CudaQueueLv1 (arch.cpp:81-82, :111-112), which is exactly what this file returns.
#include "xsched/cuda/hal/common/levels.h"
#include "xsched/cuda/hal/level1/cuda_queue.h"

namespace xsched::cuda {

std::shared_ptr<preempt::HwQueue> CudaQueueCreate(CUstream stream) { return std::make_shared<CudaQueueLv1>(stream); }

CUresult DirectLaunch(std::shared_ptr<CudaKernelCommand> kernel, CUstream stream) { return CudaQueueLv1::DirectLaunch(kernel, stream); }

} // namespace xsched::cuda
