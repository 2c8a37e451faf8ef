#include "preempt/windowed_xqueue.h"

#include <sys/prctl.h>

#include "xsched/preempt/sched/agent.h"
#include "xsched/protocol/def.h"
#include "xsched/sched/wire.h"
#include "xsched/utils/env.h"
#include "xsched/utils/trace.h"
#include "xsched/utils/xassert.h"

namespace xsched::preempt {

using sched::Event;

WindowedXQueue::WindowedXQueue(std::shared_ptr<HwQueue> hwq, XPreemptLevel level, int64_t threshold, int64_t batch_size)
    : XQueue(kXQueueImplTypeAsync,
             kQueueFeatureAsyncSubmit | (hwq->SupportDynamicLevel() ? kQueueFeatureDynamicLevel : 0) |
                 kQueueFeatureDynamicThreshold | kQueueFeatureDynamicBatchSize | kQueueFeatureSyncSuspend |
                 kQueueFeatureResumeDropCommands,
             hwq),
      level_(level), transfer_aware_(GetEnvOption(XSCHED_TRANSFER_AWARE_READY_ENV_NAME, false)), threshold_(threshold), batch_size_(batch_size) {
    XASSERT(level_ > kPreemptLevelUnknown && level_ < kPreemptLevelMax, "invalid preempt level %d", (int)level_);
    XASSERT(threshold_ >= batch_size_, "the in-flight threshold must not be smaller than the batch size");
    tail_marker_ = std::make_shared<XQueueWaitAllCommand>();
    tail_marker_->SetState(kCommandStateCompleted);
    worker_ = std::thread([this] {
        prctl(PR_SET_TIMERSLACK, 1000UL, 0, 0, 0);   // 1 us timer slack: short sleeps in waits stay short
        kHwQueue->OnXQueueCreate();        // on the launching thread: a CUDA queue binds its context here
        WorkerMain();
    });
    kHwQueue->OnPreemptLevelChange(level_);
    SchedAgent::SendEvent(Event::XQueueCreate(kHandle, kDevice, level_, threshold_, batch_size_));
}

WindowedXQueue::~WindowedXQueue() {
    terminated_.store(true);               // a terminated queue is never suspended again
    Resume(kQueueResumeFlagDropCommands);
    auto bye = std::make_shared<XQueueDestroyCommand>();
    Enqueue(bye);
    bye->Wait();
    if (worker_.joinable()) worker_.join();
    SchedAgent::SendEvent(Event::XQueueDestroy(kHandle));
}

// ------------------------------------------------------------------------------- pending side
void WindowedXQueue::Enqueue(std::shared_ptr<XCommand> cmd) {
    const int64_t ready_us = sched::NowEpochUs();
    cmd->SetState(kCommandStatePending);
    bool became_ready = false;
    {
        std::lock_guard<std::mutex> lk(q_mu_);
        if (cmd->GetType() == kCommandTypeHardware && state_ == kQueueStateIdle) {
            state_ = kQueueStateReady;
            // A transfer by itself is not announced (transfer-aware mode): the worker announces the queue when a
            // compute command is about to be launched.
            became_ready = !(transfer_aware_ && cmd->GetProps(kCommandPropertyTransferOnly));
            if (became_ready) announced_ = true;
        }
        tail_is_marker_ = false;
        pending_.push_back(std::move(cmd));
    }
    q_cv_.notify_all();
    if (became_ready) { SchedAgent::SendEvent(Event::XQueueReady(kHandle, ready_us)); XTRACE(utils::kTraceReadySent, kHandle); }
}

void WindowedXQueue::Announce(bool ready) {
    {
        std::lock_guard<std::mutex> lk(q_mu_);
        if (announced_ == ready) return;
        announced_ = ready;
    }
    if (ready) { SchedAgent::SendEvent(Event::XQueueReady(kHandle, sched::NowEpochUs())); XTRACE(utils::kTraceReadySent, kHandle); }
    else { SchedAgent::SendEvent(Event::XQueueIdle(kHandle)); XTRACE(utils::kTraceIdleSent, kHandle); }
}

// Next pending command.  With nothing pending: returns nullptr when `block_when_empty` is false;
// otherwise declares the queue idle (everything submitted has completed) and sleeps.
std::shared_ptr<XCommand> WindowedXQueue::TakeOrIdle(bool block_when_empty) {
    std::unique_lock<std::mutex> lk(q_mu_);
    if (pending_.empty()) {
        if (!block_when_empty) return nullptr;
        bool became_idle = false, tell = false;
        if (state_ == kQueueStateReady) {
            state_ = kQueueStateIdle;
            ++idle_epochs_;
            became_idle = true;
            tell = announced_;                     // a queue that only ever held transfers was never announced
            announced_ = false;
        }
        if (became_idle) {
            lk.unlock();
            idle_cv_.notify_all();
            if (tell) {
                SchedAgent::SendEvent(Event::XQueueIdle(kHandle));
                XTRACE(utils::kTraceIdleSent, kHandle);
            }
            lk.lock();
        }
        q_cv_.wait(lk, [this] { return !pending_.empty(); });
    }
    auto cmd = std::move(pending_.front());
    pending_.pop_front();
    return cmd;
}

void WindowedXQueue::WaitForNextIdle() {
    std::unique_lock<std::mutex> lk(q_mu_);
    if (state_ == kQueueStateIdle) return;
    const uint64_t epoch = idle_epochs_;
    idle_cv_.wait(lk, [&] { return idle_epochs_ != epoch; });
}

void WindowedXQueue::DropPending() {
    std::deque<std::shared_ptr<XCommand>> dropped;
    {
        std::lock_guard<std::mutex> lk(q_mu_);
        dropped.swap(pending_);
    }
    for (auto &c : dropped) c->SetState(kCommandStateCompleted);
}

XQueueState WindowedXQueue::Query() {
    std::lock_guard<std::mutex> lk(q_mu_);
    return state_;
}

void WindowedXQueue::Submit(std::shared_ptr<HwCommand> hw_cmd) {
    hw_cmd->OnSubmit(shared_from_this());
    hw_cmd->SetIdx(next_idx_.fetch_add(1));
    kHwQueue->OnHwCommandSubmit(hw_cmd);
    const bool blocking = hw_cmd->GetProps(kCommandPropertyBlockingSubmit) != 0;
    Enqueue(hw_cmd);
    if (blocking) hw_cmd->WaitUntil(kCommandStateInFlight);
}

std::shared_ptr<XQueueWaitAllCommand> WindowedXQueue::SubmitWaitAll() {
    std::shared_ptr<XQueueWaitAllCommand> marker;
    {
        std::lock_guard<std::mutex> lk(q_mu_);
        // Idle queue, or a marker is already the newest entry: reuse it (an idle queue's marker is
        // complete, so waiting on it returns at once).
        if (state_ == kQueueStateIdle && pending_.empty() && tail_is_marker_) return tail_marker_;
        if (tail_is_marker_ && tail_marker_->GetState() < kCommandStateCompleted) return tail_marker_;
        marker = std::make_shared<XQueueWaitAllCommand>();
        marker->SetState(kCommandStatePending);
        tail_marker_ = marker;
        tail_is_marker_ = true;
        pending_.push_back(marker);
    }
    q_cv_.notify_all();
    return marker;
}

void WindowedXQueue::WaitAll() { SubmitWaitAll()->Wait(); }

void WindowedXQueue::Wait(std::shared_ptr<HwCommand> hw_cmd) {
    if (!hw_cmd->Synchronizable()) {       // only its state can tell
        hw_cmd->WaitUntil(kCommandStateCompleted);
        return;
    }
    if (hw_cmd->GetState() >= kCommandStateCompleted) return;
    hw_cmd->WaitUntil(kCommandStateInFlight);
    std::unique_lock<std::mutex> lk(w_mu_);
    SyncCmdLocked(lk, hw_cmd);
}

// ------------------------------------------------------------------------------- worker side
void WindowedXQueue::WorkerMain() {
    while (true) {
        bool have_inflight;
        {
            std::lock_guard<std::mutex> lk(w_mu_);
            have_inflight = !inflight_.empty();
        }
        // With work still in flight do not sleep on the pending list: retire the oldest waitable
        // command instead, so completion (and the idle edge) is noticed without new submissions.
        std::shared_ptr<XCommand> cmd = TakeOrIdle(/*block_when_empty=*/!have_inflight);
        if (cmd == nullptr) {
            std::unique_lock<std::mutex> lk(w_mu_);
            if (inflight_.empty()) continue;
            if (!sync_points_.empty()) SyncCmdLocked(lk, sync_points_.front());
            else SyncAllLocked(lk);
            if (worker_done_) return;
            continue;
        }
        switch (cmd->GetType()) {
        case kCommandTypeHardware:
            LaunchOne(std::static_pointer_cast<HwCommand>(cmd));
            break;
        case kCommandTypeHostFunction: {
            cmd->SetState(kCommandStateInFlight);
            {
                std::unique_lock<std::mutex> lk(w_mu_);
                SyncAllLocked(lk);
                static_cast<HostFunctionCommand *>(cmd.get())->Execute();
            }
            cmd->SetState(kCommandStateCompleted);
            break;
        }
        case kCommandTypeXQueueWaitAll:
        case kCommandTypeBatchSynchronize: {
            cmd->SetState(kCommandStateInFlight);
            {
                std::unique_lock<std::mutex> lk(w_mu_);
                SyncAllLocked(lk);
            }
            cmd->SetState(kCommandStateCompleted);
            break;
        }
        case kCommandTypeXQueueDestroy: {
            cmd->SetState(kCommandStateInFlight);
            {
                std::unique_lock<std::mutex> lk(w_mu_);
                SyncAllLocked(lk);
                worker_done_ = true;
            }
            w_cv_.notify_all();
            cmd->SetState(kCommandStateCompleted);
            return;
        }
        default:
            XASSERT(false, "unknown command type %d", (int)cmd->GetType());
        }
    }
}

void WindowedXQueue::WaitWhilePaused(std::unique_lock<std::mutex> &lk) {
    w_cv_.wait(lk, [this] { return !paused_ || worker_done_; });
}

void WindowedXQueue::RetireThrough(int64_t idx) {
    while (!sync_points_.empty() && sync_points_.front()->GetIdx() <= idx) sync_points_.pop_front();
    while (!inflight_.empty() && inflight_.front()->GetIdx() <= idx) {
        inflight_.front()->SetState(kCommandStateCompleted);
        inflight_.pop_front();
    }
}

void WindowedXQueue::RetireAll() {
    sync_points_.clear();
    for (auto &c : inflight_) c->SetState(kCommandStateCompleted);
    inflight_.clear();
}

// Wait until the hardware queue has drained, then retire everything in flight.  A Synchronize that
// overlapped a pause proves nothing (a deactivated queue returns early), so it is repeated after the
// pause is lifted.
void WindowedXQueue::SyncAllLocked(std::unique_lock<std::mutex> &lk) {
    while (true) {
        WaitWhilePaused(lk);
        if (worker_done_) return;
        if (inflight_.empty()) return;
        const int64_t seen = pause_count_;
        lk.unlock();
        kHwQueue->Synchronize();
        lk.lock();
        if (seen == pause_count_) break;
    }
    RetireAll();
}

// Wait for one waitable command, then retire it and everything launched before it.  Callable from
// the worker and from application threads (XQueueWait).  The command is taken by value: callers pass
// elements of sync_points_, which another thread may pop while this one waits unlocked.
void WindowedXQueue::SyncCmdLocked(std::unique_lock<std::mutex> &lk, std::shared_ptr<HwCommand> cmd) {
    XASSERT(cmd->Synchronizable(), "SyncCmd needs a synchronizable command");
    while (true) {
        // Another thread may retire the command while this one sleeps on the pause.
        while (paused_ && !worker_done_) {
            if (cmd->GetState() >= kCommandStateCompleted) return;
            w_cv_.wait(lk);
        }
        if (cmd->GetState() >= kCommandStateCompleted || worker_done_) return;
        XASSERT(cmd->GetState() >= kCommandStateInFlight, "waiting for a command that was not launched");
        const int64_t seen = pause_count_;
        lk.unlock();
        cmd->Synchronize();
        lk.lock();
        if (seen == pause_count_) break;
    }
    RetireThrough(cmd->GetIdx());
}

void WindowedXQueue::LaunchOne(std::shared_ptr<HwCommand> cmd) {
    // Under level >= 2 a command that can neither be deactivated nor harmlessly re-executed must not
    // overtake deactivatable work: were the queue deactivated, the earlier kernels would be flushed
    // and this command would run on stale data.
    const bool fence_deactivatable = level_ >= kPreemptLevelDeactivate &&
        cmd->GetProps(kCommandPropertyDeactivatable | kCommandPropertyIdempotent) == kCommandPropertyNone;

    cmd->BeforeLaunch();
    std::unique_lock<std::mutex> lk(w_mu_);

    if (transfer_aware_) {
        const bool transfer = cmd->GetProps(kCommandPropertyTransferOnly) != 0;
        bool announced, compute_pending = false;
        {
            std::lock_guard<std::mutex> ql(q_mu_);
            announced = announced_;
            if (transfer && announced)
                for (const auto &p : pending_)
                    if (p->GetType() == kCommandTypeHardware && !p->GetProps(kCommandPropertyTransferOnly)) { compute_pending = true; break; }
        }
        if (!transfer && !announced) {
            // First compute command after transfers: it cannot start before they are done, so neither does the
            // queue need the compute units before then.  Wait for them, then tell the scheduler.
            SyncAllLocked(lk);
            lk.unlock();
            Announce(true);
            lk.lock();
        } else if (transfer && announced && !compute_pending) {
            // A transfer behind the last compute command: once that one has finished the queue holds no compute
            // work any more; say so before the transfer is handed over.
            SyncAllLocked(lk);
            lk.unlock();
            Announce(false);
            lk.lock();
        }
    }

    if (fence_deactivatable) {
        bool found = false;
        std::shared_ptr<HwCommand> sync_on;
        for (auto it = inflight_.rbegin(); it != inflight_.rend(); ++it) {
            if ((*it)->Synchronizable()) sync_on = *it;     // oldest waitable one at/after the newest deactivatable
            if ((*it)->GetProps(kCommandPropertyDeactivatable)) { found = true; break; }
        }
        if (found) {
            if (sync_on) SyncCmdLocked(lk, sync_on);
            else SyncAllLocked(lk);
        }
    }

    // Launch only while not paused and with room in the window.  A wait below releases the lock, so
    // both conditions are re-checked afterwards.
    while (true) {
        WaitWhilePaused(lk);
        if ((int64_t)inflight_.size() < threshold_) break;
        // Window full: wait for the first waitable command at or after the oldest in-flight one.
        std::shared_ptr<HwCommand> sync_on;
        const int64_t front_idx = inflight_.front()->GetIdx();
        for (auto &c : sync_points_) if (c->GetIdx() >= front_idx) { sync_on = c; break; }
        if (sync_on) SyncCmdLocked(lk, sync_on);
        else SyncAllLocked(lk);
        if (worker_done_) break;
    }

    if (cmd->GetIdx() <= drop_through_) {
        lk.unlock();
        cmd->SetState(kCommandStateCompleted);
        return;
    }
    if (cmd->GetIdx() - last_sync_idx_ >= batch_size_) cmd->EnableSynchronization();

    if (auto cb = std::dynamic_pointer_cast<HwCallbackCommand>(cmd)) {
        XASSERT(cb->Launch(kHwQueue->GetHandle()) == kXSchedSuccess, "launch callback of HwCommand %p failed", (void *)cb.get());
    } else {
        kHwQueue->Launch(cmd);
    }
    cmd->SetState(kCommandStateInFlight);
    inflight_.push_back(cmd);
    if ((int64_t)inflight_.size() > max_inflight_.load(std::memory_order_relaxed)) max_inflight_.store((int64_t)inflight_.size());
    if (cmd->Synchronizable()) {
        sync_points_.push_back(cmd);
        last_sync_idx_ = cmd->GetIdx();
    }
}

// ------------------------------------------------------------------------------- suspend / resume
// Suspend and Resume may come from different threads at the same time: the application calls them, and so
// does the scheduling agent when an operation arrives (its first operation for a new XQueue lists the queue
// as running, which is a Resume).  They are serialised: a Resume that ran between this function's "pause"
// and "Deactivate" steps would re-issue nothing, un-pause the worker, and leave the commands that Deactivate
// then pulls back out of the hardware queue stranded for good.
void WindowedXQueue::Suspend(int64_t flags) {
    if (terminated_.load()) return;
    std::lock_guard<std::mutex> serial(suspend_mu_);
    bool expected = false;
    if (!suspended_.compare_exchange_strong(expected, true)) return;     // re-entrant
    XTRACE(utils::kTraceSuspendBegin, kHandle);

    if (flags & kQueueSuspendFlagWaitIdle) WaitForNextIdle();
    else if (flags & kQueueSuspendFlagWaitAll) WaitAll();

    {
        std::lock_guard<std::mutex> lk(w_mu_);
        paused_ = true;
        ++pause_count_;
    }
    if (level_ >= kPreemptLevelDeactivate) kHwQueue->Deactivate();
    if (level_ >= kPreemptLevelInterrupt) kHwQueue->Interrupt();
    if (flags & kQueueSuspendFlagSyncHwQueue) kHwQueue->Synchronize();
    XTRACE(utils::kTraceSuspendEnd, kHandle);
}

void WindowedXQueue::Resume(int64_t flags) {
    std::lock_guard<std::mutex> serial(suspend_mu_);
    bool expected = true;
    if (!suspended_.compare_exchange_strong(expected, false)) return;
    XTRACE(utils::kTraceResumeBegin, kHandle);

    auto unpause = [this] {
        { std::lock_guard<std::mutex> lk(w_mu_); paused_ = false; }
        w_cv_.notify_all();
        XTRACE(utils::kTraceResumeEnd, kHandle);
    };

    if (level_ == kPreemptLevelBlock) {
        // Commands launched before the suspension may still be running: keep the in-flight log.
        unpause();
        return;
    }

    if (!(flags & kQueueResumeFlagDropCommands)) {
        CommandLog log;
        { std::lock_guard<std::mutex> lk(w_mu_); log = inflight_; }
        if (level_ >= kPreemptLevelInterrupt) kHwQueue->Restore(log);
        if (level_ >= kPreemptLevelDeactivate) kHwQueue->Reactivate(log);
        unpause();
        return;
    }

    // Drop: bring the hardware queue back with nothing to replay, then forget every command
    // submitted so far, launched or not.
    const CommandLog none;
    if (level_ >= kPreemptLevelInterrupt) kHwQueue->Restore(none);
    if (level_ >= kPreemptLevelDeactivate) kHwQueue->Reactivate(none);
    DropPending();
    {
        std::lock_guard<std::mutex> lk(w_mu_);
        RetireAll();
        drop_through_ = next_idx_.load() - 1;
        paused_ = false;
    }
    w_cv_.notify_all();
}

// ------------------------------------------------------------------------------- configuration
void WindowedXQueue::SetPreemptLevel(XPreemptLevel level) {
    XASSERT(level > kPreemptLevelUnknown && level < kPreemptLevelMax, "invalid preempt level %d", (int)level);
    if (!GetFeatures(kQueueFeatureDynamicLevel)) {
        XASSERT(level == level_, "this XQueue's HwQueue does not support changing the preempt level");
        return;
    }
    if (level > kHwQueue->GetMaxSupportedLevel()) {
        XWARN("preempt level %d is above what the HwQueue supports (%d); unchanged", (int)level, (int)kHwQueue->GetMaxSupportedLevel());
        return;
    }
    WaitAll();
    kHwQueue->OnPreemptLevelChange(level);
    int64_t th, bs;
    {
        std::lock_guard<std::mutex> lk(w_mu_);
        level_ = level;
        th = threshold_; bs = batch_size_;
    }
    SchedAgent::SendEvent(Event::XQueueConfigUpdate(kHandle, kDevice, level, th, bs));
}

void WindowedXQueue::SetLaunchConfig(int64_t threshold, int64_t batch_size) {
    if (threshold <= 0 && batch_size <= 0) return;
    int64_t th, bs;
    {
        std::lock_guard<std::mutex> lk(w_mu_);
        th = threshold > 0 ? threshold : threshold_;
        bs = batch_size > 0 ? batch_size : batch_size_;
    }
    XASSERT(th >= bs, "command threshold (" FMT_64D ") must not be smaller than the batch size (" FMT_64D ")", th, bs);
    WaitAll();
    {
        std::lock_guard<std::mutex> lk(w_mu_);
        threshold_ = th; batch_size_ = bs;
    }
    SchedAgent::SendEvent(Event::XQueueConfigUpdate(kHandle, kDevice, level_, th, bs));
}

} // namespace xsched::preempt
