// LocalScheduler: event queue -> status -> policy -> operations.  Behaviour follows the reference's
// sched/src/scheduler/local.cpp:12-446 (event semantics in UpdateStatus :237-407, one policy round per
// batch of events :142-196, full running/suspended sets per operation :198-206); an operation is sent
// to a process only when its sets changed, since re-sending identical sets is a no-op on the client.
#include "xsched/sched/scheduler.h"

#include <algorithm>
#include <chrono>
#include "xsched/protocol/names.h"
#include "xsched/utils/trace.h"
#include "xsched/utils/xassert.h"

namespace xsched::sched {

LocalScheduler::LocalScheduler(XPolicyType type) : Scheduler(kSchedulerLocal), policy_type_(type) { InstallPolicy(type); }

LocalScheduler::~LocalScheduler() { Stop(); }

void LocalScheduler::InstallPolicy(XPolicyType type) {
    policy_ = CreatePolicy(type);
    XASSERT(policy_ != nullptr, "policy %s (%d) is not available in this build", protocol::GetPolicyTypeName(type), (int)type);
    policy_type_ = type;
}

void LocalScheduler::Run() {
    if (thread_.joinable()) return;
    { std::lock_guard<std::mutex> lk(mtx_); stop_ = false; }
    thread_ = std::thread(&LocalScheduler::Worker, this);
}

void LocalScheduler::Stop() {
    if (!thread_.joinable()) return;
    { std::lock_guard<std::mutex> lk(mtx_); queue_.push_back(Event::Terminate()); }
    cv_.notify_all();
    thread_.join();
    timers_.clear();
}

void LocalScheduler::RecvEvent(const Event &event) {
    // Acknowledgements are recorded on the receiving thread: the worker may be blocked in
    // WaitAllOperations() waiting for exactly these.
    switch (event.Type()) {
    case kEventProcessCreate: {
        { std::lock_guard<std::mutex> lk(op_mtx_); ops_.try_emplace(event.Pid()); }
        op_cv_.notify_all();
        break;
    }
    case kEventProcessDestroy: {
        { std::lock_guard<std::mutex> lk(op_mtx_); ops_.erase(event.Pid()); }
        op_cv_.notify_all();
        break;
    }
    case kEventOperationComplete: {
        const uint64_t id = event.As<EvOpComplete>().op_id;
        {
            std::lock_guard<std::mutex> lk(op_mtx_);
            auto it = ops_.find(event.Pid());
            if (it == ops_.end()) { XWARN("operation " FMT_64U " acknowledged by unknown process %d", id, event.Pid()); return; }
            it->second.completed = std::max(it->second.completed, id);
        }
        op_cv_.notify_all();
        return;
    }
    default: break;
    }
    { std::lock_guard<std::mutex> lk(mtx_); queue_.push_back(event); }
    cv_.notify_all();
}

void LocalScheduler::SetPolicy(XPolicyType type) {
    if (type == policy_type_) return;
    const char *old_name = protocol::GetPolicyTypeName(policy_type_);
    const bool was_running = thread_.joinable();
    Stop();
    InstallPolicy(type);
    {
        std::lock_guard<std::mutex> lk(status_mtx_);
        for (auto &[h, q] : status_.xqueues) {
            if (!q.suspended) continue;
            q.suspended = false;
            auto pit = status_.processes.find(q.pid);
            if (pit == status_.processes.end()) continue;
            pit->second.suspended.erase(h);
            pit->second.running.insert(h);
            dirty_.insert(q.pid);
        }
    }
    if (was_running) Run();
    XINFO("policy changed from %s to %s", old_name, protocol::GetPolicyTypeName(type));
}

Status LocalScheduler::Snapshot() {
    std::lock_guard<std::mutex> lk(status_mtx_);
    return status_;
}

void LocalScheduler::WaitAllOperations() {
    std::unique_lock<std::mutex> lk(op_mtx_);
    op_cv_.wait(lk, [this] {
        for (const auto &[pid, ids] : ops_) if (ids.completed < ids.issued) return false;
        return true;
    });
}

void LocalScheduler::Worker() {
    std::deque<Event> batch;
    std::unique_lock<std::mutex> lk(mtx_);
    while (true) {
        // Sleep until an event arrives or the earliest timer is due.
        while (queue_.empty()) {
            if (timers_.empty()) { cv_.wait(lk); continue; }
            const int64_t now = NowEpochUs();
            if (now < timers_.front()) {
                cv_.wait_for(lk, std::chrono::microseconds(timers_.front() - now));
                continue;
            }
            timers_.erase(timers_.begin(), std::upper_bound(timers_.begin(), timers_.end(), now));
            break;
        }
        batch.swap(queue_);
        lk.unlock();

        bool terminate = false;
        {
            std::lock_guard<std::mutex> sl(status_mtx_);
            for (const Event &e : batch) {
                if (e.Type() == kEventSchedulerTerminate) { terminate = true; continue; }
                Apply(e);
            }
            Decide();
        }
        batch.clear();
        rounds_.fetch_add(1);
        if (terminate) return;
        lk.lock();
    }
}

void LocalScheduler::StepInline(const Event *events, size_t n) {
    std::lock_guard<std::mutex> sl(status_mtx_);
    const int64_t now = Now();
    timers_.erase(timers_.begin(), std::upper_bound(timers_.begin(), timers_.end(), now));
    for (size_t i = 0; i < n; ++i) {
        const Event &e = events[i];
        switch (e.Type()) {       // same bookkeeping RecvEvent does on the receiving thread
        case kEventProcessCreate: { std::lock_guard<std::mutex> lk(op_mtx_); ops_.try_emplace(e.Pid()); break; }
        case kEventProcessDestroy: { std::lock_guard<std::mutex> lk(op_mtx_); ops_.erase(e.Pid()); break; }
        case kEventOperationComplete: {
            std::lock_guard<std::mutex> lk(op_mtx_);
            auto it = ops_.find(e.Pid());
            if (it != ops_.end()) it->second.completed = std::max(it->second.completed, e.As<EvOpComplete>().op_id);
            continue;
        }
        case kEventSchedulerTerminate: continue;
        default: break;
        }
        Apply(e);
    }
    Decide();
    rounds_.fetch_add(1);
}

uint64_t LocalScheduler::NextOperationId(PID pid) {
    std::lock_guard<std::mutex> lk(op_mtx_);
    auto it = ops_.find(pid);
    return it == ops_.end() ? 0 : ++it->second.issued;
}

int64_t LocalScheduler::NextTimerUs() const {
    return timers_.empty() ? INT64_MAX : timers_.front();
}

XQueueStatus &LocalScheduler::Ensure(XQueueHandle h, PID pid) {
    auto it = status_.xqueues.find(h);
    if (it != status_.xqueues.end()) return it->second;
    XQueueStatus q;
    q.handle = h;
    q.pid = pid;
    q.ready_time_us = Now();
    ProcessStatus &p = status_.processes[pid];
    p.pid = pid;
    p.running.insert(h);
    dirty_.insert(pid);
    return status_.xqueues.emplace(h, q).first->second;
}

void LocalScheduler::Apply(const Event &e) {
    switch (e.Type()) {
    case kEventHint: {
        const EvHint &d = e.As<EvHint>();
        policy_->RecvHint(d.hint, (size_t)d.size - offsetof(EvHint, hint));
        break;
    }
    case kEventProcessCreate: {
        ProcessStatus &p = status_.processes[e.Pid()];
        p.pid = e.Pid();
        p.cmdline = e.As<EvProcessCreate>().cmdline;
        break;
    }
    case kEventProcessDestroy: {
        auto pit = status_.processes.find(e.Pid());
        if (pit == status_.processes.end()) break;
        for (XQueueHandle h : pit->second.running) status_.xqueues.erase(h);
        for (XQueueHandle h : pit->second.suspended) status_.xqueues.erase(h);
        status_.processes.erase(pit);
        dirty_.erase(e.Pid());
        break;
    }
    case kEventXQueueCreate:
    case kEventXQueueConfigUpdate: {
        const EvXQueueConfig &d = e.As<EvXQueueConfig>();
        XQueueStatus &q = Ensure(d.handle, e.Pid());
        q.device = d.device; q.level = d.level; q.threshold = d.threshold; q.batch_size = d.batch_size;
        break;
    }
    case kEventXQueueDestroy: {
        const uint64_t h = e.As<EvXQueueHandle>().handle;
        auto qit = status_.xqueues.find(h);
        if (qit == status_.xqueues.end()) break;
        auto pit = status_.processes.find(qit->second.pid);
        if (pit != status_.processes.end()) {
            pit->second.running.erase(h);
            pit->second.suspended.erase(h);
            dirty_.insert(qit->second.pid);
        }
        status_.xqueues.erase(qit);
        break;
    }
    case kEventXQueueReady: {
        const EvXQueueReady &d = e.As<EvXQueueReady>();
        XQueueStatus &q = Ensure(d.handle, e.Pid());
        q.ready = true;
        q.ready_time_us = d.ready_time_us;
        break;
    }
    case kEventXQueueIdle: {
        Ensure(e.As<EvXQueueHandle>().handle, e.Pid()).ready = false;
        break;
    }
    default: break;
    }
}

void LocalScheduler::Decide() {
    decision_.Clear();
    policy_->Sched(status_, Now(), decision_);
    XTRACE(utils::kTraceDecision, decision_.suspend.size() + decision_.resume.size() + decision_.ordered.size());

    auto move = [this](XQueueHandle h, bool to_suspended) {
        auto qit = status_.xqueues.find(h);
        if (qit == status_.xqueues.end() || qit->second.suspended == to_suspended) return;
        qit->second.suspended = to_suspended;
        auto pit = status_.processes.find(qit->second.pid);
        if (pit == status_.processes.end()) return;
        (to_suspended ? pit->second.running : pit->second.suspended).erase(h);
        (to_suspended ? pit->second.suspended : pit->second.running).insert(h);
        dirty_.insert(qit->second.pid);
    };
    for (XQueueHandle h : decision_.suspend) move(h, true);
    for (XQueueHandle h : decision_.resume) move(h, false);
    for (const auto &[h, suspend] : decision_.ordered) move(h, suspend);

    for (PID pid : dirty_) {
        auto pit = status_.processes.find(pid);
        if (pit == status_.processes.end()) continue;
        const ProcessStatus &p = pit->second;
        if (p.running.empty() && p.suspended.empty()) continue;
        uint64_t id = 0;
        {
            std::lock_guard<std::mutex> lk(op_mtx_);
            auto it = ops_.find(pid);
            if (it != ops_.end()) id = ++it->second.issued;
        }
        Execute(Operation::Sched(id, pid, std::vector<uint64_t>(p.running.begin(), p.running.end()),
                                 std::vector<uint64_t>(p.suspended.begin(), p.suspended.end())));
        XTRACE(utils::kTraceOpSent, (uint64_t)pid, id);
    }
    dirty_.clear();

    for (int64_t t : decision_.timers_us) timers_.push_back(t);
    std::sort(timers_.begin(), timers_.end());
}

} // namespace xsched::sched
