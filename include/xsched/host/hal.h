/*
 * Host-only hardware-abstraction layer ("single-lane XPU"), exported by libhalhost.so.
 *
 * A lane is one executor thread that runs commands strictly one at a time, in the order they were
 * launched on any HwQueue of that lane — a stand-in for an accelerator with one hardware FIFO, so
 * that a high-priority command really waits behind low-priority commands already in flight.  A
 * command busy-spins for a given number of microseconds.  It fills the role the reference's template
 * platform plays for porting and smoke tests (platforms/example/hal/src/opencl_queue.cpp:7-52, which
 * needs an OpenCL device), but runs on plain CPU cores.
 *
 * Levels: 1 (Launch/Synchronize) and 2 (Deactivate pulls the queue's not-yet-started commands out
 * of the lane; Reactivate pushes the unfinished ones back in order).
 */
#pragma once
#include "xsched/types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Create a HwQueue on lane `lane_id` (the lane and its executor thread are created on first use). */
XResult HostLaneQueueCreate(HwQueueHandle *hwq, uint32_t lane_id);
/* A command that occupies the lane for `spin_us` microseconds.  Submit it with XQueueSubmit. */
XResult HostLaneCommandCreate(HwCommandHandle *hw_cmd, int64_t spin_us);
/* Monotonic timestamps (ns, CLOCK_MONOTONIC) of the command's last start and finish on the lane;
 * 0 while not started / not finished.  The handle stays queryable until HostLaneCommandRelease. */
XResult HostLaneCommandTimes(HwCommandHandle hw_cmd, int64_t *start_ns, int64_t *finish_ns);
/* Timestamp of the command's (last) HwQueue::Launch, i.e. when it entered the lane; 0 if never. */
XResult HostLaneCommandLaunchTime(HwCommandHandle hw_cmd, int64_t *launch_ns);
XResult HostLaneCommandRelease(HwCommandHandle hw_cmd);
/* Commands executed by the lane so far, and how many were pulled back by Deactivate. */
XResult HostLaneStats(uint32_t lane_id, uint64_t *executed, uint64_t *flushed);
/* Pin the lane's executor thread to a CPU core (-1 = unpinned). */
XResult HostLaneSetAffinity(uint32_t lane_id, int cpu);

#ifdef __cplusplus
}
#endif
