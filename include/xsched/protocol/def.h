// Configuration surface of the preemption path: defaults and environment-variable names.  The names
// and defaults are the reference's (protocol/include/xsched/protocol/def.h:3-70) because they are part
// of what a user of the reference sets in the environment; XSCHED_POLICY_SCOPE and XSCHED_CUDA_* below
// the marked line are additions of this implementation.
#pragma once

#define XSCHED_DEFAULT_PREEMPT_LEVEL       kPreemptLevelBlock
#define XSCHED_DEFAULT_COMMAND_THRESHOLD   16     // commands allowed in flight on the hardware queue
#define XSCHED_DEFAULT_COMMAND_BATCH_SIZE  8      // every n-th command is made individually waitable

// XSCHED_AUTO_XQUEUE=ON makes the shim create an XQueue for every stream, configured by the rest.
#define XSCHED_AUTO_XQUEUE_ENV_NAME              "XSCHED_AUTO_XQUEUE"
#define XSCHED_AUTO_XQUEUE_LEVEL_ENV_NAME        "XSCHED_AUTO_XQUEUE_LEVEL"
#define XSCHED_AUTO_XQUEUE_THRESHOLD_ENV_NAME    "XSCHED_AUTO_XQUEUE_THRESHOLD"
#define XSCHED_AUTO_XQUEUE_BATCH_SIZE_ENV_NAME   "XSCHED_AUTO_XQUEUE_BATCH_SIZE"
#define XSCHED_AUTO_XQUEUE_PRIORITY_ENV_NAME     "XSCHED_AUTO_XQUEUE_PRIORITY"
#define XSCHED_AUTO_XQUEUE_UTILIZATION_ENV_NAME  "XSCHED_AUTO_XQUEUE_UTILIZATION"
#define XSCHED_AUTO_XQUEUE_TIMESLICE_ENV_NAME    "XSCHED_AUTO_XQUEUE_TIMESLICE"
#define XSCHED_AUTO_XQUEUE_DEADLINE_ENV_NAME     "XSCHED_AUTO_XQUEUE_DEADLINE"
#define XSCHED_AUTO_XQUEUE_KDEADLINE_ENV_NAME    "XSCHED_AUTO_XQUEUE_KDEADLINE"
#define XSCHED_AUTO_XQUEUE_LAXITY_ENV_NAME       "XSCHED_AUTO_XQUEUE_LAXITY"

#define XSCHED_CUDA_LIB_ENV_NAME                 "XSCHED_CUDA_LIB"   // path of the real libcuda.so.1
#define XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS_ENV_NAME "XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS"
// (addition) ON: an XQueue announces itself ready when its first compute command is about to be launched and idle
// again once only transfers remain, so that lower priorities keep the compute units while a request copies its data.
#define XSCHED_TRANSFER_AWARE_READY_ENV_NAME "XSCHED_TRANSFER_AWARE_READY"

// Scheduler selection.  XSCHED_POLICY=<name> implies the in-process (LCL) scheduler.
#define XSCHED_SCHEDULER_ENV_NAME  "XSCHED_SCHEDULER"
#define XSCHED_SCHEDULER_NAME_APP  "APP"
#define XSCHED_SCHEDULER_NAME_LCL  "LCL"
#define XSCHED_SCHEDULER_NAME_GLB  "GLB"
#define XSCHED_POLICY_ENV_NAME     "XSCHED_POLICY"
#define XSCHED_POLICY_NAME_HPF     "HPF"
#define XSCHED_POLICY_NAME_HHPF    "HHPF"
#define XSCHED_POLICY_NAME_CHPF    "CHPF"
#define XSCHED_POLICY_NAME_UP      "UP"
#define XSCHED_POLICY_NAME_PUP     "PUP"
#define XSCHED_POLICY_NAME_SPUP    "SPUP"
#define XSCHED_POLICY_NAME_KEDF    "KEDF"
#define XSCHED_POLICY_NAME_LAX     "LAX"
#define XSCHED_POLICY_NAME_AWF     "AWF"
#define XSCHED_POLICY_NAME_CFS     "CFS"
#define XSCHED_POLICY_NAME_MLFQ    "MLFQ"
#define XSCHED_UNKNOWN_NAME        "Unknown"

// What XQueue::Suspend does when the scheduler (not the application) asks for it.
#define XSCHED_SCHEDULER_SUSPEND_SYNC_HWQ_ENV_NAME   "XSCHED_SCHEDULER_SUSPEND_SYNC_HWQ"
#define XSCHED_SCHEDULER_SUSPEND_WAIT_ALL_ENV_NAME   "XSCHED_SCHEDULER_SUSPEND_WAIT_ALL"
#define XSCHED_SCHEDULER_SUSPEND_WAIT_IDLE_ENV_NAME  "XSCHED_SCHEDULER_SUSPEND_WAIT_IDLE"

// Server rendezvous: the server listens on channel key 1, a client on its pid.
#define XSCHED_SERVER_CHANNEL_KEY   1
#define XSCHED_SERVER_DEFAULT_PORT  50000

// ---- additions of this implementation -------------------------------------------------------------
// LAX decides over all devices at once in the reference (one global maximum).  DEVICE makes it decide
// per XDevice, which is what a box with several independent GPUs needs.  Default: GLOBAL (reference).
#define XSCHED_POLICY_SCOPE_ENV_NAME      "XSCHED_POLICY_SCOPE"     // GLOBAL | DEVICE
// Namespace prefix of the rendezvous sockets, so that several servers can share one host.
#define XSCHED_IPC_NAMESPACE_ENV_NAME     "XSCHED_IPC_NAMESPACE"
// ON: the receivers of the agent <-> server channel poll instead of sleeping (one busy core per receiver,
// a few microseconds per hop instead of a thread wake-up).  Default OFF.
#define XSCHED_IPC_SPIN_ENV_NAME          "XSCHED_IPC_SPIN"
