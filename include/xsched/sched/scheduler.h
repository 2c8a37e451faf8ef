// Schedulers: where events go and where operations come from.
//   AppManaged  swallows events (the application calls XQueueSuspend/Resume itself);
//   Local       runs a policy inside this process (also the engine inside the server);
//   Global      forwards events to the server and executes the operations it sends back.
// Roles as in the reference (sched/src/scheduler/scheduler.cpp:19-34, local.cpp:12-446,
// global.cpp:7-69).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <thread>
#include <vector>
#include "xsched/types.h"
#include "xsched/sched/policy.h"
#include "xsched/sched/wire.h"

namespace xsched::sched {

using Executor = std::function<void(const Operation &)>;

class Scheduler {
public:
    explicit Scheduler(XSchedulerType type) : kType(type) {}
    virtual ~Scheduler() = default;
    virtual void Run() = 0;
    virtual void Stop() = 0;
    virtual void RecvEvent(const Event &event) = 0;
    XSchedulerType GetType() const { return kType; }
    void SetExecutor(Executor e) { executor_ = std::move(e); }
protected:
    void Execute(const Operation &op) { if (executor_) executor_(op); }
private:
    const XSchedulerType kType;
    Executor executor_;
};

class AppManagedScheduler final : public Scheduler {
public:
    AppManagedScheduler() : Scheduler(kSchedulerAppManaged) {}
    void Run() override {}
    void Stop() override {}
    void RecvEvent(const Event &) override {}
};

/// One worker thread: drain all queued events into the status, run the policy once, send one Sched
/// operation (the full running + suspended sets) to every process that owns an XQueue.  Operations
/// are therefore idempotent and may be coalesced.  Timers requested by the policy wake the worker.
class LocalScheduler final : public Scheduler {
public:
    explicit LocalScheduler(XPolicyType type);
    ~LocalScheduler() override;
    void Run() override;
    void Stop() override;
    void RecvEvent(const Event &event) override;

    void SetPolicy(XPolicyType type);            // hot swap: everything is resumed first
    XPolicyType GetPolicy() const { return policy_type_; }
    /// Copy of the current status (taken on the worker between rounds).
    Status Snapshot();
    /// Block until every operation issued so far was acknowledged (OperationComplete).
    void WaitAllOperations();
    uint64_t Rounds() const { return rounds_.load(); }
    /// Id for an operation that is sent to `pid` from outside the policy loop (a configuration change asked for
    /// over the control interface); 0 when the process is unknown.
    uint64_t NextOperationId(PID pid);

    /// Threadless operation (used by the server's polling loop instead of Run()): apply `n` events and
    /// run one policy round on the calling thread.  With n == 0 only due timers are served.
    void StepInline(const Event *events, size_t n);
    /// Earliest pending policy timer (epoch us), or INT64_MAX.
    int64_t NextTimerUs() const;
    /// Replace the wall clock the inline mode reads (tests step a virtual clock through StepInline).
    void SetClock(std::function<int64_t()> clock) { clock_ = std::move(clock); }

private:
    int64_t Now() const { return clock_ ? clock_() : NowEpochUs(); }
    std::function<int64_t()> clock_;
    void Worker();
    void Apply(const Event &e);
    void Decide();
    XQueueStatus &Ensure(XQueueHandle h, PID pid);
    void InstallPolicy(XPolicyType type);
    std::set<PID> dirty_;                        // processes whose running/suspended sets changed

    XPolicyType policy_type_;
    std::unique_ptr<Policy> policy_;
    Status status_;
    Decision decision_;
    std::vector<int64_t> timers_;                // sorted ascending

    std::mutex mtx_;
    std::condition_variable cv_;
    std::deque<Event> queue_;
    bool stop_ = false;
    std::mutex status_mtx_;                      // status_ is written by the worker, read by Snapshot()
    std::thread thread_;
    std::atomic<uint64_t> rounds_{0};

    struct OpIds { uint64_t issued = 0, completed = 0; };
    std::mutex op_mtx_;
    std::condition_variable op_cv_;
    std::map<PID, OpIds> ops_;
};

class GlobalScheduler final : public Scheduler {
public:
    GlobalScheduler();
    ~GlobalScheduler() override;
    void Run() override;
    void Stop() override;
    void RecvEvent(const Event &event) override;
private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

std::shared_ptr<Scheduler> CreateScheduler(XSchedulerType scheduler, XPolicyType policy);

} // namespace xsched::sched
