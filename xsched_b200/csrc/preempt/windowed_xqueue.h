// WindowedXQueue: the asynchronous XQueue.  Submissions go to a pending list; one worker thread
// launches them on the HwQueue while keeping at most `threshold` commands in flight (the
// progressive-launch window) and makes every `batch_size`-th command individually waitable, so that
// suspending the queue leaves only a bounded amount of already-launched work to drain.
//
// Behaviour is that of the reference's AsyncXQueue + CommandBuffer + LaunchWorker
// (preempt/src/xqueue/async_xqueue.cpp:10-207, command_buffer.cpp:8-155, launch_worker.cpp:7-368):
// same idle/ready edges and events, same window and batch rules, same pause / deactivate / drop
// semantics.  The structure is different: a single class, two locks (pending list / in-flight log),
// and a drain step that retires in-flight work directly instead of synthesising marker commands.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <list>
#include <mutex>
#include <thread>
#include "xsched/protocol/def.h"
#include "xsched/preempt/xqueue/xqueue.h"

namespace xsched::preempt {

class WindowedXQueue final : public XQueue {
public:
    WindowedXQueue(std::shared_ptr<HwQueue> hwq, XPreemptLevel level,
                   int64_t threshold = XSCHED_DEFAULT_COMMAND_THRESHOLD,
                   int64_t batch_size = XSCHED_DEFAULT_COMMAND_BATCH_SIZE);
    ~WindowedXQueue() override;

    void Submit(std::shared_ptr<HwCommand> hw_cmd) override;
    std::shared_ptr<XQueueWaitAllCommand> SubmitWaitAll() override;
    void WaitAll() override;
    void Wait(std::shared_ptr<HwCommand> hw_cmd) override;
    XQueueState Query() override;
    int64_t GetHwCommandCount() override { return next_idx_.load() - 1; }

    void Suspend(int64_t flags) override;
    void Resume(int64_t flags) override;
    void SetPreemptLevel(XPreemptLevel level) override;
    void SetLaunchConfig(int64_t threshold, int64_t batch_size) override;

    /// Largest number of commands that were in flight at once (for tests of the window bound).
    int64_t MaxInFlightObserved() const { return max_inflight_.load(); }

private:
    // ---- pending side (guarded by q_mu_) ----
    void Enqueue(std::shared_ptr<XCommand> cmd);
    std::shared_ptr<XCommand> TakeOrIdle(bool block_when_empty);
    void WaitForNextIdle();
    void DropPending();

    // ---- worker side (guarded by w_mu_) ----
    void WorkerMain();
    void LaunchOne(std::shared_ptr<HwCommand> cmd);
    void SyncAllLocked(std::unique_lock<std::mutex> &lk);
    void SyncCmdLocked(std::unique_lock<std::mutex> &lk, std::shared_ptr<HwCommand> cmd);
    void RetireThrough(int64_t idx);
    void RetireAll();
    void WaitWhilePaused(std::unique_lock<std::mutex> &lk);

    XPreemptLevel level_;
    std::atomic<bool> suspended_{false};
    std::mutex suspend_mu_;          // Suspend() and Resume() run one at a time (see Suspend)
    std::atomic<bool> terminated_{false};
    std::atomic<int64_t> next_idx_{1};            // HwCommand indices start at 1

    std::mutex q_mu_;
    std::condition_variable q_cv_;                // pending list became non-empty
    std::condition_variable idle_cv_;             // ready -> idle edge
    std::deque<std::shared_ptr<XCommand>> pending_;
    std::shared_ptr<XQueueWaitAllCommand> tail_marker_;   // newest wait-all marker (done when idle)
    bool tail_is_marker_ = true;
    XQueueState state_ = kQueueStateIdle;
    uint64_t idle_epochs_ = 0;
    // What the scheduler has been told.  Without XSCHED_TRANSFER_AWARE_READY it is the same as state_; with it, a
    // queue holding only transfer commands stays unannounced, the ready event is sent by the worker when it is about
    // to launch a compute command (after the transfers before it have finished), and the idle event when a transfer
    // follows the last compute command (after that one has finished).
    const bool transfer_aware_;
    bool announced_ = false;                      // guarded by q_mu_
    void Announce(bool ready);                    // sends the event if the announced state changes

    std::mutex w_mu_;
    std::condition_variable w_cv_;                // pause lifted / terminated
    int64_t threshold_;
    int64_t batch_size_;
    CommandLog inflight_;                         // launched, completion not yet observed
    CommandLog sync_points_;                      // the synchronizable subset of inflight_
    int64_t last_sync_idx_ = -1;
    int64_t drop_through_ = -1;
    int64_t pause_count_ = 0;
    bool paused_ = false;
    bool worker_done_ = false;
    std::atomic<int64_t> max_inflight_{0};

    std::thread worker_;
};

} // namespace xsched::preempt
