/*
 * CUDA hardware-abstraction layer, exported by libhalcuda.so.
 *
 * CudaQueueCreate / CudaQueueGet replace the reference's entry points of the same name
 * (platforms/cuda/hal/include/xsched/cuda/hal.h:11-13, platforms/cuda/hal/src/arch/arch.cpp:54-116):
 * the HwQueue handle is the stream pointer itself, creation is idempotent, the NULL stream is
 * refused with kXSchedErrorNotSupported.
 *
 * The CudaXpk* entry points have no counterpart in the reference.  They turn a task of the
 * preemptible-kernel library (xsched_b200/pk.h) into a deactivatable HwCommand, which is what lets a
 * level-2 XQueue stop a running kernel at a tile boundary and resume it from its cursor.
 */
#pragma once
#include "xsched/xsched.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *CUstream;

XResult CudaQueueCreate(HwQueueHandle *hwq, CUstream stream);
XResult CudaQueueGet(HwQueueHandle *hwq, CUstream stream);

/* Device address of the preempt flag owned by the CUDA HwQueue: pass it as `flag_dev` when creating
 * xpk tasks that will be submitted to this queue, so that Deactivate() stops them. */
XResult CudaQueueGetPreemptFlag(HwQueueHandle hwq, uint32_t **flag_dev);

/* Wrap an xpk task (xpkTask_t, passed as void*) into a HwCommand.  Each launch of the command runs
 * the task from tile 0 to completion (`rewind` != 0) or continues a partially done task
 * (`rewind` == 0).  The command is deactivatable: HwQueue::Deactivate stops it at the next tile
 * boundary and HwQueue::Reactivate relaunches it from its cursor.  The task must outlive the
 * command's completion; it is not destroyed by the command. */
XResult CudaXpkCommandCreate(HwCommandHandle *hw_cmd, void *xpk_task, int rewind);

/* An asynchronous copy as a HwCommand of the CUDA backend (what the interposer makes of cuMemcpy*Async): kind 0 =
 * host to device, 1 = device to host, 2 = device to device.  Host-to-device and device-to-host copies carry the
 * transfer-only property (xsched/preempt/xqueue/xcommand.h), which the XQueue uses under
 * XSCHED_TRANSFER_AWARE_READY=ON; host memory should be pinned.  No counterpart among the reference's C entry
 * points (its copies exist only inside the shim, platforms/cuda/hal/include/xsched/cuda/hal/common/cuda_command.h:167-199). */
XResult CudaMemcpyCommandCreate(HwCommandHandle *hw_cmd, void *dst, const void *src, size_t bytes, int kind);

/* Per-queue counters for observability: commands launched, window stalls, deactivations,
 * and the last measured Deactivate-to-idle latency in nanoseconds. */
typedef struct {
    uint64_t launched, completed, window_stalls, deactivations, relaunches, last_preempt_ns;
} CudaQueueStats;
XResult CudaQueueGetStats(HwQueueHandle hwq, CudaQueueStats *stats);

#ifdef __cplusplus
}
#endif
