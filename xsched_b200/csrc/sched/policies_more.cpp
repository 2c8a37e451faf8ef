// The reference's remaining policies, restated against this scheduler's Policy interface: the clock is a
// parameter (decisions are reproducible) and verdicts go into a Decision instead of bound callbacks.
// A verdict that a round does not give leaves the queue as it is, as in the reference.
//   HHPF sched/src/policy/hhpf.cpp   CHPF chpf.cpp   UP up.cpp   PUP pup.cpp
//   KEDF kedf.cpp   AWF awf.cpp   CFS cfs.cpp   MLFQ mlfq.cpp
#include "xsched/sched/policy.h"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <sstream>
#include "xsched/utils/log.h"

namespace xsched::sched {

// ------------------------------------------------------------------------------ priority hints
bool PriorityTable::Recv(const void *hint, size_t size) {
    if (size < sizeof(HintPriority)) return false;
    const HintPriority &h = *reinterpret_cast<const HintPriority *>(hint);
    if (h.type != kHintTypePriority) return false;
    const Priority p = std::clamp<Priority>(h.prio, PRIORITY_MIN, PRIORITY_MAX);
    if (p != h.prio) XWARN("priority %d outside [%d, %d]; XQueue 0x" FMT_64X " gets %d", h.prio, PRIORITY_MIN, PRIORITY_MAX, h.handle, p);
    prio_[h.handle] = p;
    return true;
}

Priority PriorityTable::Get(XQueueHandle h) const {
    auto it = prio_.find(h);
    return it == prio_.end() ? PRIORITY_DEFAULT : it->second;
}

// ------------------------------------------------------------------------------------------- HHPF
void HeterogeneousHpfPolicy::Sched(const Status &status, int64_t, Decision &out) {
    Priority top = PRIORITY_MIN;
    for (const auto &[h, q] : status.xqueues)
        if (q.ready) top = std::max(top, prio_.Get(h));
    for (const auto &[h, q] : status.xqueues) (prio_.Get(h) < top ? out.suspend : out.resume).push_back(h);
}

// ------------------------------------------------------------------------------------------- CHPF
Priority CpuHpfPolicy::LinuxPriority(PID pid) {
    std::ifstream f("/proc/" + std::to_string(pid) + "/sched");
    std::string line;
    while (std::getline(f, line)) {
        if (line.find("prio") == std::string::npos) continue;
        std::istringstream is(line);
        std::string name, colon;
        Priority v = 0;
        is >> name >> colon >> v;
        // kernel scale: 0-99 real-time (larger = more urgent), 100-139 normal (larger = nicer)
        return v >= 100 ? -v : v;
    }
    return 0;
}

void CpuHpfPolicy::Sched(const Status &status, int64_t, Decision &out) {
    std::map<PID, Priority> by_pid;
    for (const auto &[pid, p] : status.processes) by_pid[pid] = LinuxPriority(pid);
    auto prio_of = [&](PID pid) { auto it = by_pid.find(pid); return it == by_pid.end() ? 0 : it->second; };
    std::map<XDevice, Priority> top;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        const Priority p = prio_of(q.pid);
        auto [it, fresh] = top.try_emplace(q.device, p);
        if (!fresh && p > it->second) it->second = p;
    }
    for (const auto &[h, q] : status.xqueues) {
        auto it = top.find(q.device);
        const Priority bar = it == top.end() ? PRIORITY_MIN : it->second;
        (prio_of(q.pid) < bar ? out.suspend : out.resume).push_back(h);
    }
}

// --------------------------------------------------------------------------------------------- UP
int64_t UtilizationPartitionPolicy::Budget(Utilization util) const {
    int64_t total = 0;
    for (const auto &[h, u] : utils_) total += u;
    return total == 0 ? TIMESLICE_DEFAULT : timeslice_us_ * util / total;
}

// Nothing holds the turn: the first ready queue that has a share gets it, every other queue stops.
void UtilizationPartitionPolicy::HandOutAny(const Status &status, int64_t now_us, Decision &out) {
    current_ = 0;
    for (const auto &[h, q] : status.xqueues) {
        auto share = utils_.find(h);
        if (current_ != 0 || !q.ready || share == utils_.end()) { out.Suspend(h); continue; }
        out.Resume(h);
        current_ = h;
        current_end_us_ = now_us + Budget(share->second);
        out.timers_us.push_back(current_end_us_);
    }
}

void UtilizationPartitionPolicy::HandOutTo(XQueueHandle h, Utilization util, const Status &status, int64_t now_us, Decision &out) {
    for (const auto &[other, q] : status.xqueues)
        if (other != h) out.Suspend(other);
    out.Resume(h);
    current_ = h;
    current_end_us_ = now_us + Budget(util);
    out.timers_us.push_back(current_end_us_);
}

void UtilizationPartitionPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    auto alive = [&](XQueueHandle h) { return status.xqueues.find(h) != status.xqueues.end(); };
    for (auto it = utils_.begin(); it != utils_.end();) it = alive(it->first) ? std::next(it) : utils_.erase(it);
    if (current_ != 0 && !alive(current_)) current_ = 0;
    if (utils_.empty()) return;
    if (current_ == 0) { HandOutAny(status, now_us, out); return; }

    const XQueueStatus &cur = status.xqueues.at(current_);
    if (now_us < current_end_us_ && cur.ready) return;        // its turn is not over

    // Turn over (time is up, or the holder went idle): next ready share holder in handle order, wrapping
    // around, the holder itself excluded.
    auto self = utils_.find(current_);
    if (self == utils_.end()) { HandOutAny(status, now_us, out); return; }   // the holder never had a share
    auto ready = [&](XQueueHandle h) { return status.xqueues.at(h).ready; };
    for (auto it = std::next(self); it != utils_.end(); ++it)
        if (ready(it->first)) { HandOutTo(it->first, it->second, status, now_us, out); return; }
    for (auto it = utils_.begin(); it != self; ++it)
        if (ready(it->first)) { HandOutTo(it->first, it->second, status, now_us, out); return; }
    current_ = 0;                                              // nobody else wants it
}

void UtilizationPartitionPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(int32_t)) return;
    switch (*reinterpret_cast<const int32_t *>(hint)) {
    case kHintTypeUtilization: {
        if (size < sizeof(HintUtilization)) return;
        const HintUtilization &h = *reinterpret_cast<const HintUtilization *>(hint);
        if (h.util < UTILIZATION_MIN || h.util > UTILIZATION_MAX) { XWARN("invalid utilization %d", h.util); return; }
        utils_[h.handle] = h.util;
        return;
    }
    case kHintTypeTimeslice:
        if (size >= sizeof(HintTimeslice)) timeslice_us_ = reinterpret_cast<const HintTimeslice *>(hint)->ts_us;
        return;
    default:
        return;
    }
}

// -------------------------------------------------------------------------------------------- PUP
int64_t ProcessUtilizationPartitionPolicy::FreshBudget(PID pid) const {
    auto util_of = [this](PID p) -> int64_t { auto it = utils_.find(p); return it == utils_.end() ? UTILIZATION_DEFAULT : it->second; };
    int64_t total = 0;
    for (const Entry &e : queue_) total += util_of(e.pid);
    if (total == 0) return 0;
    return timeslice_us_ * (int64_t)queue_.size() * util_of(pid) / total;
}

bool ProcessUtilizationPartitionPolicy::ProcessReady(const ProcessStatus &p, const Status &status) {
    auto any_ready = [&](const std::set<XQueueHandle> &set) {
        for (XQueueHandle h : set) {
            auto it = status.xqueues.find(h);
            if (it != status.xqueues.end() && it->second.ready) return true;
        }
        return false;
    };
    return any_ready(p.running) || any_ready(p.suspended);
}

void ProcessUtilizationPartitionPolicy::SwitchTo(PID pid, const Status &status, Decision &out) {
    for (Entry &e : queue_) {
        auto it = status.processes.find(e.pid);
        if (it == status.processes.end()) continue;
        if (e.pid == pid) for (XQueueHandle h : it->second.suspended) out.Resume(h);
        else for (XQueueHandle h : it->second.running) out.Suspend(h);
        e.running = e.pid == pid;
    }
}

void ProcessUtilizationPartitionPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    for (auto it = utils_.begin(); it != utils_.end();)
        it = status.processes.count(it->first) ? std::next(it) : utils_.erase(it);

    auto owns_queues = [](const ProcessStatus &p) { return !p.running.empty() || !p.suspended.empty(); };
    bool any_ready = false;
    for (auto it = queue_.begin(); it != queue_.end();) {
        auto ps = status.processes.find(it->pid);
        if (ps == status.processes.end() || !owns_queues(ps->second)) {
            queued_.erase(it->pid);
            it = queue_.erase(it);
            continue;
        }
        it->ready = ProcessReady(ps->second, status);
        any_ready = any_ready || it->ready;
        ++it;
    }
    for (const auto &[pid, ps] : status.processes) {
        if (!owns_queues(ps) || queued_.count(pid)) continue;
        const bool ready = ProcessReady(ps, status);
        any_ready = any_ready || ready;
        queue_.push_back(Entry{pid, ready, false, 0});
        queued_.insert(pid);
    }
    if (queue_.empty() || !any_ready) return;

    auto rotate = [this](int64_t budget) {          // head goes to the tail, not running, with `budget` saved
        Entry e = queue_.front();
        queue_.erase(queue_.begin());
        e.running = false;
        e.budget_us = budget;
        queue_.push_back(e);
    };
    // Budget of a turn: what was saved, its excess over one fresh budget decayed by 10 %, plus a fresh one.
    auto turn_budget = [this](const Entry &e) {
        const int64_t fresh = FreshBudget(e.pid);
        int64_t b = e.budget_us;
        if (b > fresh) b = (int64_t)((double)fresh + (double)(b - fresh) * 0.9);
        return b + fresh;
    };

    if (queue_.front().running) {
        const bool time_left = slice_end_us_ > now_us;
        if (time_left && queue_.front().ready) return;
        rotate(time_left ? slice_end_us_ - now_us : 0);
    }
    while (!queue_.front().ready) {                 // an idle process keeps (and grows) its budget at the tail
        const int64_t b = turn_budget(queue_.front());
        rotate(b);
    }
    slice_end_us_ = now_us + turn_budget(queue_.front());
    out.timers_us.push_back(slice_end_us_);
    SwitchTo(queue_.front().pid, status, out);
}

void ProcessUtilizationPartitionPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(int32_t)) return;
    switch (*reinterpret_cast<const int32_t *>(hint)) {
    case kHintTypeUtilization: {
        if (size < sizeof(HintUtilization)) return;
        const HintUtilization &h = *reinterpret_cast<const HintUtilization *>(hint);
        if (h.pid == 0) return;
        if (h.util < UTILIZATION_MIN || h.util > UTILIZATION_MAX) { XWARN("invalid utilization %d", h.util); return; }
        utils_[h.pid] = h.util;
        return;
    }
    case kHintTypeTimeslice: {
        if (size < sizeof(HintTimeslice)) return;
        const int64_t ts = reinterpret_cast<const HintTimeslice *>(hint)->ts_us;
        if (ts < TIMESLICE_MIN || ts > TIMESLICE_MAX) { XWARN("invalid timeslice " FMT_64D, ts); return; }
        timeslice_us_ = ts;
        return;
    }
    default:
        return;
    }
}

// ------------------------------------------------------------------------------------------- KEDF
void KEarliestDeadlineFirstPolicy::Sched(const Status &status, int64_t, Decision &out) {
    constexpr int64_t kNever = std::numeric_limits<int64_t>::max();
    std::vector<std::pair<int64_t, XQueueHandle>> order;
    order.reserve(status.xqueues.size());
    for (const auto &[h, q] : status.xqueues) {
        auto it = deadlines_.find(h);
        order.emplace_back(q.ready && it != deadlines_.end() ? q.ready_time_us + it->second : kNever, h);
    }
    std::stable_sort(order.begin(), order.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
    for (size_t i = 0; i < order.size(); ++i) (i < k_ ? out.resume : out.suspend).push_back(order[i].second);
}

void KEarliestDeadlineFirstPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(int32_t)) return;
    switch (*reinterpret_cast<const int32_t *>(hint)) {
    case kHintTypeDeadline:
        if (size >= sizeof(HintDeadline)) {
            const HintDeadline &h = *reinterpret_cast<const HintDeadline *>(hint);
            deadlines_[h.handle] = h.ddl_us;
        }
        return;
    case kHintTypeKDeadline:
        if (size >= sizeof(HintKDeadline)) {
            const uint64_t k = reinterpret_cast<const HintKDeadline *>(hint)->k;
            if (k < 1) XWARN("invalid k " FMT_64U, k);
            else k_ = (size_t)k;
        }
        return;
    default:
        return;
    }
}

// -------------------------------------------------------------------------------------------- AWF
void ActiveWindowFirstPolicy::Sched(const Status &status, int64_t, Decision &out) {
    bool active_wants_gpu = false;
    for (const auto &[h, q] : status.xqueues)
        if (q.ready && active_.count(q.pid)) { active_wants_gpu = true; break; }
    for (const auto &[h, q] : status.xqueues)
        (active_wants_gpu && !active_.count(q.pid) ? out.suspend : out.resume).push_back(h);
}

void ActiveWindowFirstPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(HintWindowActive)) return;
    const HintWindowActive &h = *reinterpret_cast<const HintWindowActive *>(hint);
    if (h.type != kHintTypeWindowActive || h.pid == 0) return;
    auto it = by_display_.find(h.display);
    if (it != by_display_.end()) active_.erase(it->second);     // one active window per display
    active_.insert(h.pid);
    by_display_[h.display] = h.pid;
}

// -------------------------------------------------------------------------------------------- CFS
void CompletelyFairPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    constexpr int64_t kSliceUs = 1000;
    // charge the time since the last round to whoever was running
    for (const auto &[h, q] : status.xqueues) {
        auto it = nodes_.find(h);
        if (it != nodes_.end() && it->second.running)
            it->second.vruntime += (double)(now_us - it->second.last_resume_us) * (1024.0 / it->second.weight);
    }
    // smallest virtual runtime among the ready queues already known, per device
    std::map<XDevice, double> floor;
    bool any_ready = false;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        any_ready = true;
        auto it = nodes_.find(h);
        if (it == nodes_.end()) continue;
        auto [f, fresh] = floor.try_emplace(q.device, it->second.vruntime);
        if (!fresh && it->second.vruntime < f->second) f->second = it->second.vruntime;
    }
    // newcomers start at their device's floor (no starvation of the old ones); pick the minimum
    std::map<XDevice, XQueueHandle> pick;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        auto it = nodes_.find(h);
        if (it == nodes_.end()) {
            Node n;
            n.last_resume_us = now_us;
            auto f = floor.find(q.device);
            n.vruntime = f != floor.end() ? f->second : 0.0;
            if (f == floor.end()) floor[q.device] = n.vruntime;
            it = nodes_.emplace(h, n).first;
        }
        auto p = pick.find(q.device);
        if (p == pick.end() || it->second.vruntime < nodes_[p->second].vruntime) pick[q.device] = h;
    }
    for (const auto &[h, q] : status.xqueues) {
        Node &n = nodes_[h];
        if (!q.ready) { n.running = false; continue; }
        if (pick[q.device] == h) {
            if (!n.running) out.Resume(h);
            n.running = true;
            n.last_resume_us = now_us;
        } else {
            out.Suspend(h);
            n.running = false;
        }
    }
    if (any_ready) out.timers_us.push_back(now_us + kSliceUs);
}

void CompletelyFairPolicy::RecvHint(const void *hint, size_t size) {
    if (size < sizeof(HintPriority)) return;
    const HintPriority &h = *reinterpret_cast<const HintPriority *>(hint);
    if (h.type != kHintTypePriority) return;
    nodes_[h.handle].weight = 1024.0 * std::pow(1.2, h.prio);      // +20 % share per priority step
}

// ------------------------------------------------------------------------------------------- MLFQ
void MultiLevelFeedbackPolicy::Sched(const Status &status, int64_t now_us, Decision &out) {
    constexpr int kLowestLevel = 3;
    constexpr int64_t kRiseAfterUs = 100000, kTickUs = 5000;
    auto slice_of = [](int level) { return (int64_t)10000 << level; };

    for (const auto &[h, q] : status.xqueues) {
        auto [it, fresh] = nodes_.try_emplace(h);
        Node &n = it->second;
        if (fresh) n.level_since_us = n.pending_from_us = n.resumed_at_us = now_us;
        if (q.ready && !n.was_ready) n.pending_from_us = now_us;          // a new request starts waiting now
        n.was_ready = q.ready;
    }
    std::map<XDevice, std::map<int, int>> ready_at_level;
    for (const auto &[h, q] : status.xqueues)
        if (q.ready) ready_at_level[q.device][nodes_[h].level]++;

    bool any_ready = false;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        any_ready = true;
        Node &n = nodes_[h];
        if (!n.running) { n.pending_us += now_us - n.pending_from_us; n.pending_from_us = now_us; }
        else { n.slice_used_us += now_us - n.resumed_at_us; n.resumed_at_us = now_us; }

        // rise: time at this level, minus a share (0.9/N among N peers) of the time spent waiting
        const int peers = ready_at_level[q.device][n.level];
        const double discount = peers > 1 ? 0.9 / peers : 1.0;
        const double effective = (double)(now_us - n.level_since_us) - (double)n.pending_us * discount;
        if (effective > (double)kRiseAfterUs) {
            if (n.level > 0) n.level--;
            n.level_since_us = now_us;
            n.pending_us = 0;
            n.slice_used_us = 0;
        }
        // drop: slice used up; the queue yields at once
        if (n.running && n.slice_used_us >= slice_of(n.level)) {
            if (n.level < kLowestLevel) n.level++;
            n.level_since_us = now_us;
            n.slice_used_us = 0;
            n.pending_us = 0;
            n.running = false;
            out.Suspend(h);
            n.pending_from_us = now_us;
        }
    }
    // best level per device; among equals the one that has waited longest
    std::map<XDevice, XQueueHandle> pick;
    for (const auto &[h, q] : status.xqueues) {
        if (!q.ready) continue;
        const Node &n = nodes_[h];
        auto p = pick.find(q.device);
        if (p == pick.end()) { pick[q.device] = h; continue; }
        const Node &best = nodes_[p->second];
        if (n.level < best.level || (n.level == best.level && n.pending_us > best.pending_us)) p->second = h;
    }
    for (const auto &[h, q] : status.xqueues) {
        Node &n = nodes_[h];
        if (!q.ready) { n.running = false; continue; }
        if (pick[q.device] == h) {
            if (!n.running) {
                out.Resume(h);
                n.running = true;
                n.pending_from_us = now_us;
            }
            n.resumed_at_us = now_us;
        } else if (n.running) {          // a queue that was never picked is left as it is
            out.Suspend(h);
            n.running = false;
            n.pending_from_us = now_us;
        }
    }
    if (any_ready) out.timers_us.push_back(now_us + kTickUs);
}

} // namespace xsched::sched
