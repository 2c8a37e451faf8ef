// Scheduling agent of this process + the XHint* C entry points
// (reference: preempt/src/sched/agent.cpp:21-140, executor.cpp:26-102, hint.cpp:12-71).
//
// The scheduler is chosen at load time from XSCHED_POLICY (=> in-process scheduler with that policy)
// or XSCHED_SCHEDULER (APP | LCL | GLB); XHintSetScheduler can replace it later.  Operations coming
// back from the scheduler are executed here: queues to run are resumed first, then queues to stop are
// suspended with the flags selected by XSCHED_SCHEDULER_SUSPEND_{SYNC_HWQ,WAIT_ALL,WAIT_IDLE}.
#include "xsched/preempt/sched/agent.h"

#include <atomic>
#include <fstream>
#include <mutex>
#include "xsched/xsched.h"
#include "xsched/preempt/xqueue/xqueue.h"
#include "xsched/protocol/def.h"
#include "xsched/protocol/names.h"
#include "xsched/utils/trace.h"
#include "xsched/utils/xassert.h"

namespace xsched::preempt {

using namespace xsched::sched;

namespace {

std::mutex g_mtx;                                   // guards g_scheduler replacement
std::atomic<std::shared_ptr<Scheduler>> g_scheduler;   // read lock-free from scheduler threads
std::atomic<bool> g_executing{false};

std::string Cmdline() {
    std::string out;
    std::ifstream f("/proc/self/cmdline", std::ios::binary);
    std::string arg;
    while (f.good() && std::getline(f, arg, '\0') && !arg.empty()) out += arg + " ";
    if (out.size() > 255) out.resize(255);
    return out;
}

bool PolicyAvailable(XPolicyType p) { return p > kPolicyUnknown && p < kPolicyMax && p != kPolicyStrictProcessUtilizationPartition; }

void Start(XSchedulerType scheduler, XPolicyType policy) {
    if (policy > kPolicyUnknown && policy < kPolicyMax && !PolicyAvailable(policy)) {
        XWARN("policy %s is not provided by this build; falling back to the application-managed scheduler",
              protocol::GetPolicyTypeName(policy));
        policy = kPolicyUnknown;
        scheduler = kSchedulerAppManaged;
    }
    auto s = CreateScheduler(scheduler, policy);
    s->SetExecutor(&SchedAgent::Execute);
    s->Run();
    s->RecvEvent(Event::ProcessCreate(Cmdline()));
    g_scheduler.store(std::move(s));
}

void Finish() {
    auto s = g_scheduler.exchange(nullptr);
    if (!s) return;
    s->RecvEvent(Event::ProcessDestroy((int32_t)GetProcessId()));
    s->Stop();
}

struct Bootstrap {
    Bootstrap() {
        std::lock_guard<std::mutex> lk(g_mtx);
        XSchedulerType st = kSchedulerUnknown;
        XPolicyType pt = kPolicyUnknown;
        const std::string s = GetEnv(XSCHED_SCHEDULER_ENV_NAME), p = GetEnv(XSCHED_POLICY_ENV_NAME);
        if (!s.empty()) st = protocol::GetSchedulerType(s);
        if (!p.empty()) pt = protocol::GetPolicyType(p);
        g_executing.store(true);
        Start(st, pt);
    }
    ~Bootstrap() {
        g_executing.store(false);
        std::lock_guard<std::mutex> lk(g_mtx);
        Finish();
    }
};
Bootstrap g_bootstrap;

int64_t SchedulerSuspendFlags() {
    static const int64_t flags =
        (GetEnvOption(XSCHED_SCHEDULER_SUSPEND_SYNC_HWQ_ENV_NAME, false) ? kQueueSuspendFlagSyncHwQueue : 0) |
        (GetEnvOption(XSCHED_SCHEDULER_SUSPEND_WAIT_ALL_ENV_NAME, false) ? kQueueSuspendFlagWaitAll : 0) |
        (GetEnvOption(XSCHED_SCHEDULER_SUSPEND_WAIT_IDLE_ENV_NAME, false) ? kQueueSuspendFlagWaitIdle : 0);
    return flags;
}

} // namespace

std::shared_ptr<Scheduler> SchedAgent::Current() {
    return g_scheduler.load();
}

void SchedAgent::SendEvent(const Event &event) {
    std::shared_ptr<Scheduler> s = g_scheduler.load();
    if (!s) { XDEBG("no scheduler yet: event %d dropped", event.Type()); return; }
    s->RecvEvent(event);
}

void SchedAgent::SendHint(const void *hint, size_t size) { SendEvent(Event::Hint(hint, size)); }

XResult SchedAgent::ReplaceScheduler(XSchedulerType scheduler, XPolicyType policy) {
    if (scheduler <= kSchedulerUnknown || scheduler >= kSchedulerMax) return kXSchedErrorInvalidValue;
    std::lock_guard<std::mutex> lk(g_mtx);
    auto cur = g_scheduler.load();
    if (!cur) return kXSchedErrorUnknown;
    const bool policy_valid = policy > kPolicyUnknown && policy < kPolicyMax;
    if (policy_valid && !PolicyAvailable(policy)) return kXSchedErrorNotSupported;
    if (cur->GetType() == scheduler) {
        if (scheduler != kSchedulerLocal) return kXSchedSuccess;
        if (!policy_valid) return kXSchedErrorInvalidValue;
        static_cast<LocalScheduler *>(cur.get())->SetPolicy(policy);
        return kXSchedSuccess;
    }
    // Switching scheduler type.  As in the reference, asking for the local scheduler without a valid
    // policy is not an error: the process ends up application-managed.
    Finish();
    Start(scheduler, policy_valid ? policy : kPolicyUnknown);
    return kXSchedSuccess;
}

void SchedAgent::Execute(const Operation &op) {
    const OperationMeta &m = op.Meta();
    XASSERT(m.pid == (int32_t)GetProcessId(), "operation " FMT_64U " for process %d delivered to process %d", m.id, m.pid, GetProcessId());
    XTRACE(utils::kTraceOpRecv, m.id, (uint64_t)m.type);
    if (g_executing.load()) {
        if (m.type == kOperationSched) {
            const OpSchedHeader &h = *reinterpret_cast<const OpSchedHeader *>(op.bytes.data());
            const uint64_t *handles = reinterpret_cast<const uint64_t *>(op.bytes.data() + sizeof(OpSchedHeader));
            // The XQueue may be gone by now: operations are asynchronous.
            for (uint64_t i = 0; i < h.running_cnt; ++i)
                if (auto xq = XQueueManager::Get(handles[i])) xq->Resume(kQueueResumeFlagNone);
            for (uint64_t i = 0; i < h.suspended_cnt; ++i)
                if (auto xq = XQueueManager::Get(handles[h.running_cnt + i])) xq->Suspend(SchedulerSuspendFlags());
        } else if (m.type == kOperationConfig) {
            const OpConfig &c = *reinterpret_cast<const OpConfig *>(op.bytes.data());
            if (c.level > kPreemptLevelUnknown) {
                const XResult r = XQueueSetPreemptLevel(c.handle, (XPreemptLevel)c.level);
                if (r != kXSchedSuccess) XWARN("config operation: level %d refused for XQueue 0x" FMT_64X " (%d)", c.level, c.handle, (int)r);
            }
            if (c.threshold > 0 || c.batch_size > 0) {
                const XResult r = XQueueSetLaunchConfig(c.handle, c.threshold, c.batch_size);
                if (r != kXSchedSuccess) XWARN("config operation: launch config refused for XQueue 0x" FMT_64X " (%d)", c.handle, (int)r);
            }
        } else if (m.type != kOperationNone) {
            XERRO("unsupported operation type %d", m.type);
        }
    }
    // Acknowledge.  Called on the scheduler's own thread, so talk to the scheduler object directly.
    std::shared_ptr<Scheduler> s = g_scheduler.load();
    if (s) s->RecvEvent(Event::OperationComplete(m.id));
}

} // namespace xsched::preempt

using namespace xsched::preempt;
using namespace xsched::sched;

#define REQUIRE_XQUEUE(xq)                                                     \
    do {                                                                       \
        const XResult r_ = XQueueManager::Exists(xq);                          \
        if (r_ != kXSchedSuccess) {                                            \
            XWARN("XQueue 0x" FMT_64X " does not exist", (uint64_t)(xq));      \
            return r_;                                                         \
        }                                                                      \
    } while (0)

EXPORT_C_FUNC XResult XHintSetScheduler(XSchedulerType scheduler, XPolicyType policy) {
    return SchedAgent::ReplaceScheduler(scheduler, policy);
}

EXPORT_C_FUNC XResult XHintPriority(XQueueHandle xq, Priority prio) {
    REQUIRE_XQUEUE(xq);
    HintPriority h{kHintTypePriority, 0, xq, prio, 0};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XHintUtilization(XQueueHandle xq, Utilization util) {
    REQUIRE_XQUEUE(xq);
    HintUtilization h{kHintTypeUtilization, (int32_t)GetProcessId(), xq, util, 0};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XHintTimeslice(Timeslice ts_us) {
    HintTimeslice h{kHintTypeTimeslice, 0, ts_us};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XHintLaxity(XQueueHandle xq, Laxity lax_us, Priority lax_prio, Priority crit_prio) {
    REQUIRE_XQUEUE(xq);
    HintLaxity h{kHintTypeLaxity, 0, xq, lax_us, lax_prio, crit_prio};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XHintDeadline(XQueueHandle xq, Deadline ddl_us) {
    REQUIRE_XQUEUE(xq);
    HintDeadline h{kHintTypeDeadline, 0, xq, ddl_us};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XHintKDeadline(size_t k) {
    HintKDeadline h{kHintTypeKDeadline, 0, (uint64_t)k};
    SchedAgent::SendHint(&h, sizeof(h));
    return kXSchedSuccess;
}
