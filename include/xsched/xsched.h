/*
 * xsched.h — the public C ABI of the preemption path: XQueue, HwQueue/HwCommand handles and
 * scheduling hints.  Exported by libpreempt.so.
 *
 * Every declaration keeps the name, argument order, argument meaning and error behaviour of
 * the XSched interface it replaces, so that code written against XSched links unchanged:
 *   - types and enumerators ......... include/xsched/types.h:10-149   (reference)
 *   - XQueue / HwQueue / HwCommand ... include/xsched/xqueue.h:16-112  (reference)
 *   - XHint* ........................ include/xsched/hint.h:13-56     (reference)
 * types.h, xqueue.h and hint.h of this tree forward to this header.
 */
#ifndef XSCHED_B200_PUBLIC_API_H
#define XSCHED_B200_PUBLIC_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ handles ---------- */
/* reference: include/xsched/types.h:10-14.  An XDevice packs (device type << 32 | device id);
 * for CUDA the id is the PCI address domain<<16 | bus<<8 | dev<<3. */
typedef uint64_t XDevice;
typedef uint32_t XDeviceId;
typedef uint64_t XQueueHandle;
typedef uint64_t HwQueueHandle;
typedef uint64_t HwCommandHandle;

/* ------------------------------------------------------------------ enumerations ------ */
/* reference: include/xsched/types.h:16-25 */
typedef enum {
    kXSchedSuccess = 0, kXSchedErrorHardware = 1, kXSchedErrorInvalidValue = 2, kXSchedErrorNotFound = 3,
    kXSchedErrorNotAllowed = 4, kXSchedErrorNotSupported = 5, kXSchedErrorBadResponse = 6,
    kXSchedErrorUnknown = 999,
} XResult;

/* reference: include/xsched/types.h:27-36 */
typedef enum {
    kPlatformUnknown = 0, kPlatformVPI = 1, kPlatformCUDA = 2, kPlatformCUDLA = 3, kPlatformHIP = 4,
    kPlatformAscend = 5, kPlatformOpenCL = 6, kPlatformLevelZero = 7,
} XPlatform;

/* reference: include/xsched/types.h:38-46 */
typedef enum {
    kDeviceTypeUnknown = 0, kDeviceTypeCPU = 1, kDeviceTypeGPU = 2, kDeviceTypeNPU = 3, kDeviceTypeFPGA = 4,
    kDeviceTypeASIC = 5, kDeviceTypeMCA = 6,
} XDeviceType;

/* reference: include/xsched/types.h:48-54.  Level 1 = progressive-launch window, level 2 =
 * deactivate/reactivate (cooperative tile-cursor preemption here), level 3 = interrupt. */
typedef enum {
    kPreemptLevelUnknown = 0, kPreemptLevelBlock = 1, kPreemptLevelDeactivate = 2, kPreemptLevelInterrupt = 3,
    kPreemptLevelMax,
} XPreemptLevel;

/* reference: include/xsched/types.h:56-60 */
typedef enum { kQueueStateUnknown = 0, kQueueStateIdle = 1, kQueueStateReady = 2 } XQueueState;

/* reference: include/xsched/types.h:62-71 */
typedef enum {
    kQueueFeatureNone = 0x0000, kQueueFeatureAsyncSubmit = 0x0001, kQueueFeatureDynamicLevel = 0x0002,
    kQueueFeatureDynamicThreshold = 0x0004, kQueueFeatureDynamicBatchSize = 0x0008,
    kQueueFeatureSyncSuspend = 0x0010, kQueueFeatureResumeDropCommands = 0x0020, kQueueFeatureMaskAll = -1,
} XQueueFeature;

/* reference: include/xsched/types.h:73-90 */
typedef enum { kQueueCreateFlagNone = 0x0000, kQueueCreateFlagBlockingSubmit = 0x0001, kQueueCreateFlagMaskAll = -1 } XQueueCreateFlag;
typedef enum {
    kQueueSuspendFlagNone = 0x0000, kQueueSuspendFlagSyncHwQueue = 0x0001, kQueueSuspendFlagWaitAll = 0x0002,
    kQueueSuspendFlagWaitIdle = 0x0004, kQueueSuspendFlagMaskAll = -1,
} XQueueSuspendFlag;
typedef enum { kQueueResumeFlagNone = 0x0000, kQueueResumeFlagDropCommands = 0x0001, kQueueResumeFlagMaskAll = -1 } XQueueResumeFlag;

/* reference: include/xsched/types.h:92-98 */
typedef enum {
    kSchedulerUnknown = 0, kSchedulerAppManaged = 1, kSchedulerLocal = 2, kSchedulerGlobal = 3, kSchedulerMax,
} XSchedulerType;

/* reference: include/xsched/types.h:101-118.  Every policy the reference can create is provided;
 * kPolicyStrictProcessUtilizationPartition is declared there but has no implementation, nor here. */
typedef enum {
    kPolicyUnknown = 0, kPolicyHighestPriorityFirst = 1, kPolicyHeterogeneousHighestPriorityFirst = 2,
    kPolicyCPUHighestPriorityFirst = 3, kPolicyUtilizationPartition = 4, kPolicyProcessUtilizationPartition = 5,
    kPolicyStrictProcessUtilizationPartition = 6, kPolicyKEarliestDeadlineFirst = 7, kPolicyLaxity = 8,
    kPolicyActiveWindowFirst = 9, kPolicyCompletelyFairScheduler = 10, kPolicyMultiLevelFeedbackQueue = 11,
    kPolicyMax,
} XPolicyType;

/* reference: include/xsched/types.h:120 */
typedef XResult (*LaunchCallback)(HwQueueHandle, void *);

/* reference: include/xsched/types.h:122-149 — hint value types and their ranges */
typedef int32_t Priority;      /* larger = more important */
#define PRIORITY_NO_EXECUTE (-256)
#define PRIORITY_MIN        (-255)
#define PRIORITY_DEFAULT    0
#define PRIORITY_MAX        255
typedef int32_t Utilization;   /* percent */
#define UTILIZATION_MIN     0
#define UTILIZATION_DEFAULT 100
#define UTILIZATION_MAX     100
typedef int64_t Timeslice;     /* microseconds */
#define TIMESLICE_MIN       100
#define TIMESLICE_DEFAULT   5000
#define TIMESLICE_MAX       10000000
#define TIMESLICE_UNLIMITED UINT64_MAX
typedef int64_t Laxity;        /* microseconds the queue may be delayed after becoming ready */
#define NO_LAXITY           (-1)
typedef int64_t Deadline;      /* microseconds after becoming ready */
#define NO_DEADLINE         (-1)

/* ------------------------------------------------------------------ XQueue -----------
 * reference: include/xsched/xqueue.h:16-86, implementation preempt/src/xqueue/xqueue.cpp:255-402.
 * Errors: InvalidValue for a null out-pointer or a level outside [1,3]; NotFound for an unknown
 * handle; NotSupported for kQueueCreateFlagBlockingSubmit and for a level change on a HwQueue
 * without dynamic levels.  XQueueCreate on a HwQueue that already has an XQueue returns that
 * XQueue.  XQueueSubmit consumes the HwCommand handle.  Suspend/Resume are re-entrant. */
XResult XQueueCreate(XQueueHandle *xq, HwQueueHandle hwq, int64_t level, int64_t flags);
XResult XQueueDestroy(XQueueHandle xq);
XResult XQueueGet(XQueueHandle *xq, HwQueueHandle hwq);
XResult XQueueSetPreemptLevel(XQueueHandle xq, XPreemptLevel level);
XResult XQueueSetLaunchConfig(XQueueHandle xq, int64_t threshold, int64_t batch_size);
XResult XQueueSubmit(XQueueHandle xq, HwCommandHandle hw_cmd);
XResult XQueueWait(XQueueHandle xq, HwCommandHandle hw_cmd);
XResult XQueueWaitAll(XQueueHandle xq);
XResult XQueueQuery(XQueueHandle xq, XQueueState *state);
XResult XQueueSuspend(XQueueHandle xq, int64_t flags);
XResult XQueueResume(XQueueHandle xq, int64_t flags);
XResult XQueueProfileHwCommandCount(XQueueHandle xq, int64_t *count);

/* ------------------------------------------------------------------ HwQueue / HwCommand
 * reference: include/xsched/xqueue.h:88-112, implementation preempt/src/hal/hw_queue.cpp:66-101,
 * preempt/src/hal/hw_command.cpp:82-99.  HwQueueDestroy answers NotAllowed while an XQueue is
 * attached.  HwQueueLaunch consumes the command handle and launches it directly, bypassing any
 * XQueue. */
XResult HwQueueDestroy(HwQueueHandle hwq);
XResult HwQueueLaunch(HwQueueHandle hwq, HwCommandHandle hw_cmd);
XResult HwQueueSynchronize(HwQueueHandle hwq);
XResult HwCommandCreateCallback(HwCommandHandle *hw_cmd, LaunchCallback launch, void *data);
XResult HwCommandDestroy(HwCommandHandle hw_cmd);

/* ------------------------------------------------------------------ hints ------------
 * reference: include/xsched/hint.h:13-56, implementation preempt/src/sched/hint.cpp:12-71. */
XResult XHintSetScheduler(XSchedulerType scheduler, XPolicyType policy);
XResult XHintPriority(XQueueHandle xq, Priority prio);
XResult XHintUtilization(XQueueHandle xq, Utilization util);
XResult XHintTimeslice(Timeslice ts_us);
XResult XHintLaxity(XQueueHandle xq, Laxity lax_us, Priority lax_prio, Priority crit_prio);
XResult XHintDeadline(XQueueHandle xq, Deadline ddl_us);
XResult XHintKDeadline(size_t k);

#ifdef __cplusplus
}
#endif
#endif /* XSCHED_B200_PUBLIC_API_H */
