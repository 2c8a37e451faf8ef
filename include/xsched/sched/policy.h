// Scheduling policies.  A policy looks at the status of every XQueue the scheduler knows and says, for
// each, whether it should run or be suspended; it may also ask to be called again at a given time.
// The decision rules of HPF and LAX are the reference's (sched/src/policy/hpf.cpp:8-68,
// sched/src/policy/lax.cpp:8-72); the plumbing (a Decision object instead of bound callbacks) is not.
#pragma once
#include <cstdint>
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
    std::vector<int64_t> timers_us;                    // absolute times (epoch us) to re-run Sched()
    void Clear() { suspend.clear(); resume.clear(); timers_us.clear(); }
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
class HighestPriorityFirstPolicy final : public Policy {
public:
    HighestPriorityFirstPolicy() : Policy(kPolicyHighestPriorityFirst) {}
    void Sched(const Status &status, int64_t now_us, Decision &out) override;
    void RecvHint(const void *hint, size_t size) override;
    Priority GetPriority(XQueueHandle h) const;
private:
    std::unordered_map<XQueueHandle, Priority> prio_;
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

/// nullptr for a policy type this implementation does not provide.
std::unique_ptr<Policy> CreatePolicy(XPolicyType type);
PolicyScope PolicyScopeFromEnv();

} // namespace xsched::sched
