// The per-process scheduling agent: owns the scheduler chosen for this process (APP / LCL / GLB),
// forwards XQueue events and hints to it and executes the operations it returns on local XQueues.
// Same role as the reference's SchedAgent + SchedExecutor (preempt/src/sched/agent.cpp:21-140,
// preempt/src/sched/executor.cpp:26-102).
#pragma once
#include <memory>
#include "xsched/types.h"
#include "xsched/sched/scheduler.h"
#include "xsched/sched/wire.h"

namespace xsched::preempt {

class SchedAgent {
public:
    /// Deliver an event to the current scheduler (dropped with a warning before initialisation).
    static void SendEvent(const sched::Event &event);
    static void SendHint(const void *hint, size_t size);
    /// XHintSetScheduler: swap scheduler and/or policy at run time.
    static XResult ReplaceScheduler(XSchedulerType scheduler, XPolicyType policy);
    /// The scheduler currently in use (for tests and the server).
    static std::shared_ptr<sched::Scheduler> Current();
    /// Execute one operation against this process's XQueues and acknowledge it.
    static void Execute(const sched::Operation &op);
};

} // namespace xsched::preempt
