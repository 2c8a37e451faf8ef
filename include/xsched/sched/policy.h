// Scheduling policies.  A policy looks at the status of every XQueue the scheduler knows and says, for
// each, whether it should run or be suspended; it may also ask to be called again at a given time.
// The decision rules of HPF and LAX are the reference's (sched/src/policy/hpf.cpp:8-68,
// sched/src/policy/lax.cpp:8-72); the plumbing (a Decision object instead of bound callbacks) is not.
#pragma once
#include <cstdint>
#include <limits>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>
#include "xsched/types.h"
#include "xsched/utils/common.h"
#include "xsched/sched/wire.h"

namespace xsched::sched {

struct XQueueStatus {
    XQueueHandle handle = 0;
    XDevice device = 0;
    int32_t level = 0;
    PID pid = 0;
    int64_t threshold = 0;
    int64_t batch_size = 0;
    bool ready = false;
    bool suspended = false;
    int64_t ready_time_us = 0;       // microseconds since the epoch
};

struct ProcessStatus {
    PID pid = 0;
    std::string cmdline;
    std::set<XQueueHandle> running;
    std::set<XQueueHandle> suspended;
};

struct Status {
    std::map<XQueueHandle, XQueueStatus> xqueues;      // ordered: policies iterate deterministically
    std::map<PID, ProcessStatus> processes;
};

/// What a policy wants after one Sched() round.
struct Decision {
    std::vector<XQueueHandle> suspend;
    std::vector<XQueueHandle> resume;
    /// Verdicts whose order matters (a policy may suspend a queue and pick it again in the same round):
    /// applied after `suspend` and `resume`, in sequence; true = suspend.
    std::vector<std::pair<XQueueHandle, bool>> ordered;
    std::vector<int64_t> timers_us;                    // absolute times (epoch us) to re-run Sched()
    void Suspend(XQueueHandle h) { ordered.emplace_back(h, true); }
    void Resume(XQueueHandle h) { ordered.emplace_back(h, false); }
    void Clear() { suspend.clear(); resume.clear(); ordered.clear(); timers_us.clear(); }
};

enum class PolicyScope { kGlobal, kDevice };

class Policy {
public:
    explicit Policy(XPolicyType type) : kType(type) {}
    virtual ~Policy() = default;
    /// `now_us` is passed in (not read from a clock) so that decisions are reproducible.
    virtual void Sched(const Status &status, int64_t now_us, Decision &out) = 0;
    /// `hint` points at one of the Hint* records of wire.h.
    virtual void RecvHint(const void *hint, size_t size) = 0;
    const XPolicyType kType;
};

/// Highest priority first, decided per device: a queue is suspended iff a READY queue with a strictly
/// higher priority exists on the same device.  Unknown priority = 0; hints are clamped to [-255, 255].
///
/// Resume hysteresis (an addition, off unless XSCHED_HPF_RESUME_HYSTERESIS_US > 0 in the scheduler's process): a
/// queue that has just gone idle still counts as ready for that many microseconds, so that lower priorities are
/// not resumed into the short gaps of a high-priority task that submits, waits and submits again (a decode loop
/// reads one token back per step) only to be preempted again at once; a timer re-runs the decision when the
/// window ends.  With 0 the decisions are exactly the reference's.
class HighestPriorityFirstPolicy final : public Policy {
public:
    HighestPriorityFirstPolicy();
    explicit HighestPriorityFirstPolicy(int64_t resume_hysteresis_us) : Policy(kPolicyHighestPriorityFirst), hysteresis_us_(resume_hysteresis_us) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
    Priority GetPriority(XQueueHandle h) const;
private:
    std::unordered_map<XQueueHandle, Priority> prio_;
    int64_t hysteresis_us_ = 0;
    std::unordered_map<XQueueHandle, int64_t> idle_since_;      // queues seen ready before and idle now -> when that was noticed
    std::unordered_map<XQueueHandle, bool> was_ready_;
};

/// Laxity ("LLF"): a ready queue runs at lax_prio until ready_time + laxity has passed and at crit_prio
/// afterwards; queues without a hint run at priority 0; not-ready queues count at lax_prio.  The
/// highest effective priority among READY queues wins and everything below it is suspended; a timer
/// is requested at the earliest pending flip.  Scope kGlobal takes one maximum over all devices (the
/// reference's behaviour), kDevice one per XDevice.
class LaxityPolicy final : public Policy {
public:
    explicit LaxityPolicy(PolicyScope scope = PolicyScope::kGlobal) : Policy(kPolicyLaxity), scope_(scope) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    struct Info { Laxity lax; Priority lax_prio; Priority crit_prio; };
    PolicyScope scope_;
    std::unordered_map<XQueueHandle, Info> info_;
};

/// Priority hints clamped to [PRIORITY_MIN, PRIORITY_MAX]; unknown queue = PRIORITY_DEFAULT.
class PriorityTable {
public:
    /// True when `hint` was a priority hint (and was recorded).
    bool Recv(const void *hint, size_t size);
    Priority Get(XQueueHandle h) const;
private:
    std::unordered_map<XQueueHandle, Priority> prio_;
};

/// HPF with ONE maximum over all devices ("heterogeneous": a ready high-priority queue on any device
/// holds back lower priorities everywhere).  Reference: sched/src/policy/hhpf.cpp:8-56.
class HeterogeneousHpfPolicy final : public Policy {
public:
    HeterogeneousHpfPolicy() : Policy(kPolicyHeterogeneousHighestPriorityFirst) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override { prio_.Recv(hint, size); }
private:
    PriorityTable prio_;
};

/// HPF per device where a queue's priority is its process's Linux scheduling priority, read from
/// /proc/<pid>/sched at every round (value v of the "prio" line; v >= 100 counts as -v, so a nicer
/// process ranks lower and a real-time one ranks above every normal one).  Hints are ignored.
/// Reference: sched/src/policy/chpf.cpp:10-72.
class CpuHpfPolicy final : public Policy {
public:
    CpuHpfPolicy() : Policy(kPolicyCPUHighestPriorityFirst) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *, size_t) override {}
    static Priority LinuxPriority(PID pid);            // 0 when it cannot be read
};

/// Utilization partition: hinted XQueues take turns, one at a time over ALL devices, each for
/// timeslice * util / sum(util); queues without a utilization hint are suspended whenever a turn is
/// handed out.  Reference: sched/src/policy/up.cpp:6-164.
class UtilizationPartitionPolicy final : public Policy {
public:
    UtilizationPartitionPolicy() : Policy(kPolicyUtilizationPartition) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    int64_t Budget(Utilization util) const;
    void HandOutAny(const Status &status, int64_t now_us, Decision &out);
    void HandOutTo(XQueueHandle h, Utilization util, const Status &status, int64_t now_us, Decision &out);
    XQueueHandle current_ = 0;
    int64_t current_end_us_ = 0;
    std::map<XQueueHandle, Utilization> utils_;
    int64_t timeslice_us_ = TIMESLICE_DEFAULT;
};

/// Utilization partition between PROCESSES: a run queue of processes that own XQueues; the head runs
/// (all its queues resumed, everybody else's suspended) for its budget, unused time is carried over with a
/// 10 % decay of whatever exceeds one fresh budget.  Reference: sched/src/policy/pup.cpp:7-200.
class ProcessUtilizationPartitionPolicy final : public Policy {
public:
    ProcessUtilizationPartitionPolicy() : Policy(kPolicyProcessUtilizationPartition) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    struct Entry { PID pid; bool ready; bool running; int64_t budget_us; };
    int64_t FreshBudget(PID pid) const;
    static bool ProcessReady(const ProcessStatus &p, const Status &status);
    void SwitchTo(PID pid, const Status &status, Decision &out);
    std::vector<Entry> queue_;                         // front = index 0
    std::map<PID, Utilization> utils_;
    std::set<PID> queued_;
    int64_t slice_end_us_ = std::numeric_limits<int64_t>::min();
    int64_t timeslice_us_ = TIMESLICE_DEFAULT;
};

/// K earliest deadlines first: the k queues whose (ready time + hinted deadline) is smallest run, the
/// rest are suspended; idle or un-hinted queues count as "never".  Reference: sched/src/policy/kedf.cpp:11-78.
class KEarliestDeadlineFirstPolicy final : public Policy {
public:
    KEarliestDeadlineFirstPolicy() : Policy(kPolicyKEarliestDeadlineFirst) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    size_t k_ = 1;
    std::unordered_map<XQueueHandle, Deadline> deadlines_;
};

/// Active window first: while a process that owns the active window of some display has a ready queue,
/// only such processes run.  Reference: sched/src/policy/awf.cpp:6-51.
class ActiveWindowFirstPolicy final : public Policy {
public:
    ActiveWindowFirstPolicy() : Policy(kPolicyActiveWindowFirst) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    std::set<PID> active_;
    std::map<uint64_t, PID> by_display_;
};

/// Completely fair: per device the ready queue with the smallest weighted virtual runtime runs for a
/// 1 ms slice; weight = 1024 * 1.2^priority.  Reference: sched/src/policy/cfs.cpp:10-124.
class CompletelyFairPolicy final : public Policy {
public:
    CompletelyFairPolicy() : Policy(kPolicyCompletelyFairScheduler) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
private:
    struct Node { double weight = 1024.0; double vruntime = 0.0; int64_t last_resume_us = 0; bool running = false; };
    std::unordered_map<XQueueHandle, Node> nodes_;
};

/// Multi-level feedback queue, per device: four levels (0 = best) with slices of 10/20/40/80 ms; a queue
/// that uses up its slice drops a level, one that has waited rises; evaluated every 5 ms.
/// Reference: sched/src/policy/mlfq.cpp:7-173, sched/include/xsched/sched/policy/mlfq.h:11-53.
class MultiLevelFeedbackPolicy final : public Policy {
public:
    MultiLevelFeedbackPolicy() : Policy(kPolicyMultiLevelFeedbackQueue) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *, size_t) override {}
private:
    struct Node {
        int level = 0;
        bool running = false, was_ready = false;
        int64_t level_since_us = 0, pending_us = 0, pending_from_us = 0, slice_used_us = 0, resumed_at_us = 0;
    };
    std::map<XQueueHandle, Node> nodes_;
};

/// nullptr for a policy type this implementation does not provide.
std::unique_ptr<Policy> CreatePolicy(XPolicyType type);
PolicyScope PolicyScopeFromEnv();

} // namespace xsched::sched
