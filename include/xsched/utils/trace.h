// Stage stamps for latency break-downs: with XSCHED_TRACE_FILE=<path> every process of a run (applications,
// xserver) appends {monotonic ns, stage, two words} records to an in-memory ring and writes them to
// <path>.<pid> when it exits; without the variable a stamp is one predictable branch.  The monotonic clock
// is system-wide, so the files of several processes merge into one timeline.  (The reference has timers and
// percentile helpers for its own experiments, utils/include/xsched/utils/timing.h:19-86, but no cross-process
// timeline; this is the per-stage view of the path "ready event -> policy -> Suspend -> first high-priority CTA".)
#pragma once
#include <cstdint>

namespace xsched::utils {

enum TraceStage : uint32_t {
    kTraceReadySent = 1,      // agent: XQueue ready event handed to the scheduler             a = xqueue handle
    kTraceIdleSent,           // agent: XQueue idle event                                       a = xqueue handle
    kTraceEventRecv,          // scheduler: event taken off the wire / queue                   a = event type, b = pid
    kTraceDecision,           // scheduler: policy has run                                      a = operations to send
    kTraceOpSent,             // scheduler: operation handed to a process                       a = pid
    kTraceOpRecv,             // agent: operation arrived                                       a = operation id
    kTraceSuspendBegin,       // XQueue::Suspend entered                                        a = xqueue handle
    kTraceSuspendEnd,         //                 returned                                       a = xqueue handle
    kTraceResumeBegin,        // XQueue::Resume entered                                         a = xqueue handle
    kTraceResumeEnd,          //                returned                                        a = xqueue handle
    kTraceDeactivateIssued,   // CUDA queue: preempt flag write handed to the driver           a = hwqueue handle
    kTraceHwqSynced,          // CUDA queue: Synchronize after a Deactivate returned            a = hwqueue handle
    kTraceTaskGpuTimes,       // CUDA queue, at Reactivate: a flushed task's device stamps      a = first-CTA start, b = last-CTA exit (GPU ns)
    kTraceGpuClockOffset,     // application: host monotonic ns - GPU globaltimer ns            a = offset (two's complement), b = uncertainty ns
    kTraceAppSubmit,          // application: request submitted                                 a = request index
    kTraceAppDone,            // application: request completed                                 a = request index
    kTraceAppGpuTimes,        // application: the request kernel's device stamps                a = first-CTA start, b = last-CTA exit (GPU ns)
    kTraceStageMax
};

const char *TraceStageName(uint32_t stage);
bool TraceEnabled();
void TraceStamp(uint32_t stage, uint64_t a = 0, uint64_t b = 0);
/// Writes what the ring holds (called at process exit; callable earlier, e.g. before _exit).
void TraceFlush();

} // namespace xsched::utils

extern "C" {
/// C entry points for programs that only link the C ABI (the benchmark workers).
int XTraceEnabled(void);
void XTraceStamp(uint32_t stage, uint64_t a, uint64_t b);
void XTraceFlush(void);
}

#define XTRACE(stage, ...)                                                                          \
    do {                                                                                            \
        if (__builtin_expect(::xsched::utils::TraceEnabled(), 0)) ::xsched::utils::TraceStamp(stage __VA_OPT__(,) __VA_ARGS__); \
    } while (0)
