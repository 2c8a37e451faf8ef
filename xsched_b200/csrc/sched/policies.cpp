// HPF and LAX decision rules.  Same outcomes as the reference's policies on the same status
// (sched/src/policy/hpf.cpp:8-68, sched/src/policy/lax.cpp:8-72); every queue in the status gets
// exactly one verdict per round, in handle order.
#include "xsched/sched/policy.h"

#include <algorithm>
#include <limits>
#include "xsched/protocol/def.h"
#include "xsched/utils/env.h"
#include "xsched/utils/log.h"

namespace xsched::sched {

// ------------------------------------------------------------------------------------------- HPF
Priority HighestPriorityFirstPolicy::GetPriority(XQueueHandle h) const {
    auto it = prio_.find(h);
    return it == prio_.end() ? PRIORITY_DEFAULT : it->second;
}

HighestPriorityFirstPolicy::HighestPriorityFirstPolicy() : Policy(kPolicyHighestPriorityFirst) {
    const std::string v = GetEnv("XSCHED_HPF_RESUME_HYSTERESIS_US");
    if (!v.empty()) hysteresis_us_ = std::max<int64_t>(0, std::atoll(v.c_str()));
}

void HighestPriorityFirstPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    // With a resume hysteresis, a queue that went idle less than that long ago still counts as ready.
    std::unordered_map<XQueueHandle, bool> lingering;
    if (hysteresis_us_ > 0) {
        for (const auto &[h, q] : status.xqueues) {
            bool &was = was_ready_[h];
            if (q.ready) { idle_since_.erase(h); was = true; continue; }
            if (was) { idle_since_[h] = now_us; was = false; }
            auto it = idle_since_.find(h);
            if (it == idle_since_.end()) continue;
            if (now_us - it->second < hysteresis_us_) { lingering[h] = true; out.timers_us.push_back(it->second + hysteresis_us_); }
            else idle_since_.erase(it);
        }
        for (auto it = was_ready_.begin(); it != was_ready_.end();)        // forget queues that are gone
            it = status.xqueues.count(it->first) ? std::next(it) : (idle_since_.erase(it->first), was_ready_.erase(it));
    }
    // Highest priority among the READY queues of each device.
    std::map<XDevice, Priority> top;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready && !lingering.count(h)) continue;
        const Priority p = GetPriority(h);
        auto [it, fresh] = top.try_emplace(q.device, p);
        if (!fresh && p > it->second) it->second = p;
    }
    for (const auto &[h, q] : status.xqueues) {
        auto it = top.find(q.device);
        const Priority bar = it == top.end() ? PRIORITY_MIN : it->second;
        (GetPriority(h) < bar ? out.suspend : out.resume).push_back(h);
    }
}

void HighestPriorityFirstPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(HintPriority)) return;
    const HintPriority &h = *reinterpret_cast<const HintPriority *>(hint);
    if (h.type != kHintTypePriority) return;
    const Priority p = std::clamp<Priority>(h.prio, PRIORITY_MIN, PRIORITY_MAX);
    if (p != h.prio) XWARN("priority %d outside [%d, %d]; XQueue 0x" FMT_64X " gets %d", h.prio, PRIORITY_MIN, PRIORITY_MAX, h.handle, p);
    prio_[h.handle] = p;
}

// ------------------------------------------------------------------------------------------- LAX
void LaxityPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    struct Top { Priority prio = PRIORITY_MIN; };
    std::map<XDevice, Top> top;                      // one entry (key 0) when the scope is global
    auto key = [this](const XQueueStatus &q) -> XDevice { return scope_ == PolicyScope::kDevice ? q.device : 0; };

    bool has_timer = false;
    int64_t earliest = std::numeric_limits<int64_t>::max();
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        Top &t = top[key(q)];
        auto it = info_.find(h);
        if (it == info_.end()) {                      // no hint: plain priority 0
            t.prio = std::max<Priority>(t.prio, PRIORITY_DEFAULT);
            continue;
        }
        const int64_t flip = q.ready_time_us + it->second.lax;
        const bool relaxed = now_us < flip;
        t.prio = std::max(t.prio, relaxed ? it->second.lax_prio : it->second.crit_prio);
        if (relaxed && flip < earliest) { earliest = flip; has_timer = true; }
    }
    for (const auto &[h, q] : status.xqueues) {
        Priority p = PRIORITY_DEFAULT;
        auto it = info_.find(h);
        if (it != info_.end()) {
            const int64_t flip = q.ready_time_us + it->second.lax;
            p = (!q.ready || now_us < flip) ? it->second.lax_prio : it->second.crit_prio;
        }
        auto tt = top.find(key(q));
        const Priority bar = tt == top.end() ? PRIORITY_MIN : tt->second.prio;
        (p < bar ? out.suspend : out.resume).push_back(h);
    }
    if (has_timer) out.timers_us.push_back(earliest);
}

void LaxityPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(HintLaxity)) return;
    const HintLaxity &h = *reinterpret_cast<const HintLaxity *>(hint);
    if (h.type != kHintTypeLaxity) return;
    info_[h.handle] = Info{h.lax_us < 0 ? (Laxity)NO_LAXITY : h.lax_us, h.lax_prio, h.crit_prio};
}

PolicyScope PolicyScopeFromEnv() {
    const std::string v = GetEnv(XSCHED_POLICY_SCOPE_ENV_NAME);
    return (v == "DEVICE" || v == "device") ? PolicyScope::kDevice : PolicyScope::kGlobal;
}

std::unique_ptr<Policy> CreatePolicy(XPolicyType type) {
    switch (type) {
    case kPolicyHighestPriorityFirst: return std::make_unique<HighestPriorityFirstPolicy>();
    case kPolicyLaxity: return std::make_unique<LaxityPolicy>(PolicyScopeFromEnv());
    case kPolicyHeterogeneousHighestPriorityFirst: return std::make_unique<HeterogeneousHpfPolicy>();
    case kPolicyCPUHighestPriorityFirst: return std::make_unique<CpuHpfPolicy>();
    case kPolicyUtilizationPartition: return std::make_unique<UtilizationPartitionPolicy>();
    case kPolicyProcessUtilizationPartition: return std::make_unique<ProcessUtilizationPartitionPolicy>();
    case kPolicyKEarliestDeadlineFirst: return std::make_unique<KEarliestDeadlineFirstPolicy>();
    case kPolicyActiveWindowFirst: return std::make_unique<ActiveWindowFirstPolicy>();
    case kPolicyCompletelyFairScheduler: return std::make_unique<CompletelyFairPolicy>();
    case kPolicyMultiLevelFeedbackQueue: return std::make_unique<MultiLevelFeedbackPolicy>();
    default: return nullptr;       // kPolicyStrictProcessUtilizationPartition: declared by the reference, implemented nowhere
    }
}

} // namespace xsched::sched
