// Host-only HAL: single-lane executor (see include/xsched/host/hal.h).  This file uses only the HAL
// contract (HwQueue / HwCommand / the two managers), so the very same source also compiles against
// the reference's headers — that build is how the reference core is driven as the CPU checker.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <pthread.h>
#include <sched.h>

#include "xsched/types.h"
#include "xsched/preempt/hal/hw_command.h"
#include "xsched/preempt/hal/hw_queue.h"

#if __has_include("xsched/host/hal.h")
#include "xsched/host/hal.h"
#endif

#define LANE_EXPORT extern "C" __attribute__((visibility("default")))

using namespace xsched::preempt;

namespace {

int64_t MonoNs() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

class LaneCommand final : public HwCommand {
public:
    explicit LaneCommand(int64_t spin_us) : HwCommand(kCommandPropertyDeactivatable), spin_us_(spin_us) {}
    void Synchronize() override {
        // Returns when the command ran, or when it was pulled out of the lane by Deactivate.
        int32_t s = stage_.load(std::memory_order_acquire);
        while (s == kQueued || s == kRunning) {
            stage_.wait(s, std::memory_order_acquire);
            s = stage_.load(std::memory_order_acquire);
        }
    }
    bool Synchronizable() override { return waitable_; }
    bool EnableSynchronization() override { waitable_ = true; return true; }

    enum Stage : int32_t { kNew = 0, kQueued = 1, kRunning = 2, kDone = 3, kFlushed = 4 };
    void SetStage(int32_t s) { stage_.store(s, std::memory_order_release); stage_.notify_all(); }
    int32_t GetStage() const { return stage_.load(std::memory_order_acquire); }
    bool TryStart() { int32_t e = kQueued; return stage_.compare_exchange_strong(e, kRunning); }
    bool TryFlush() { int32_t e = kQueued; if (!stage_.compare_exchange_strong(e, kFlushed)) return false; stage_.notify_all(); return true; }

    const int64_t spin_us_;
    std::atomic<int64_t> launch_ns_{0}, start_ns_{0}, finish_ns_{0};
private:
    std::atomic<int32_t> stage_{kNew};
    std::atomic<bool> waitable_{false};
};

class Lane {
public:
    explicit Lane(uint32_t id) : id_(id), thread_([this] { Run(); }) {}
    void Push(std::shared_ptr<LaneCommand> c) {
        c->SetStage(LaneCommand::kQueued);
        { std::lock_guard<std::mutex> lk(mu_); fifo_.push_back(std::move(c)); }
        cv_.notify_one();
    }
    void SetAffinity(int cpu) {
        cpu_set_t set;
        CPU_ZERO(&set);
        if (cpu >= 0) CPU_SET(cpu, &set);
        else for (int i = 0; i < CPU_SETSIZE; ++i) CPU_SET(i, &set);
        pthread_setaffinity_np(thread_.native_handle(), sizeof(set), &set);
    }
    std::atomic<uint64_t> executed{0}, flushed{0};
private:
    void Run() {
        while (true) {
            std::shared_ptr<LaneCommand> c;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [this] { return !fifo_.empty(); });
                c = std::move(fifo_.front());
                fifo_.pop_front();
            }
            if (!c->TryStart()) continue;                 // pulled back by Deactivate
            const int64_t t0 = MonoNs();
            c->start_ns_.store(t0);
            const int64_t until = t0 + c->spin_us_ * 1000;
            while (MonoNs() < until) { /* occupy the lane */ }
            c->finish_ns_.store(MonoNs());
            executed.fetch_add(1);
            c->SetStage(LaneCommand::kDone);
        }
    }
    const uint32_t id_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<std::shared_ptr<LaneCommand>> fifo_;
    std::thread thread_;
};

std::mutex g_mu;
std::map<uint32_t, Lane *> &Lanes() { static auto *m = new std::map<uint32_t, Lane *>(); return *m; }
Lane *GetLane(uint32_t id) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = Lanes().find(id);
    if (it != Lanes().end()) return it->second;
    Lane *l = new Lane(id);                               // lives until process exit
    Lanes()[id] = l;
    return l;
}
std::unordered_map<HwCommandHandle, std::shared_ptr<LaneCommand>> &Kept() {
    static auto *m = new std::unordered_map<HwCommandHandle, std::shared_ptr<LaneCommand>>();
    return *m;
}

class LaneQueue final : public HwQueue {
public:
    LaneQueue(uint32_t lane_id, HwQueueHandle handle) : lane_id_(lane_id), handle_(handle), lane_(GetLane(lane_id)) {}

    void Launch(std::shared_ptr<HwCommand> hw_cmd) override {
        auto c = std::dynamic_pointer_cast<LaneCommand>(hw_cmd);
        if (!c) return;
        c->launch_ns_.store(MonoNs());
        { std::lock_guard<std::mutex> lk(mu_); launched_.push_back(c); Trim(); }
        lane_->Push(std::move(c));
    }
    void Synchronize() override {
        // Wait for everything launched on this queue that is still in the lane.
        while (true) {
            std::shared_ptr<LaneCommand> c;
            {
                std::lock_guard<std::mutex> lk(mu_);
                Trim();
                for (auto &x : launched_) {
                    const int32_t s = x->GetStage();
                    if (s == LaneCommand::kQueued || s == LaneCommand::kRunning) { c = x; break; }
                }
            }
            if (!c) return;
            c->Synchronize();
        }
    }
    void Deactivate() override {
        std::lock_guard<std::mutex> lk(mu_);
        for (auto &x : launched_) if (x->TryFlush()) lane_->flushed.fetch_add(1);
    }
    void Reactivate(const CommandLog &log) override {
        // Re-issue, in order, what was pulled out.  The command that was running kept running.
        for (auto &hc : log) {
            auto c = std::dynamic_pointer_cast<LaneCommand>(hc);
            if (c && c->GetStage() == LaneCommand::kFlushed) lane_->Push(c);
        }
    }
    XDevice GetDevice() override { return ((uint64_t)kDeviceTypeCPU << 32) | lane_id_; }
    HwQueueHandle GetHandle() override { return handle_; }
    bool SupportDynamicLevel() override { return true; }
    XPreemptLevel GetMaxSupportedLevel() override { return kPreemptLevelDeactivate; }

private:
    void Trim() {
        while (!launched_.empty() && launched_.front()->GetStage() == LaneCommand::kDone) launched_.pop_front();
    }
    const uint32_t lane_id_;
    const HwQueueHandle handle_;
    Lane *const lane_;
    std::mutex mu_;
    std::deque<std::shared_ptr<LaneCommand>> launched_;
};

std::atomic<uint64_t> g_next_queue{1};

} // namespace

LANE_EXPORT XResult HostLaneQueueCreate(HwQueueHandle *hwq, uint32_t lane_id) {
    if (hwq == nullptr) return kXSchedErrorInvalidValue;
    const HwQueueHandle h = 0x4C414E4500000000ull | ((uint64_t)(lane_id & 0xFFFF) << 16) | (g_next_queue.fetch_add(1) & 0xFFFF);
    const XResult r = HwQueueManager::Add(h, [&]() -> std::shared_ptr<HwQueue> { return std::make_shared<LaneQueue>(lane_id, h); });
    if (r == kXSchedSuccess) *hwq = h;
    return r;
}

LANE_EXPORT XResult HostLaneCommandCreate(HwCommandHandle *hw_cmd, int64_t spin_us) {
    if (hw_cmd == nullptr || spin_us < 0) return kXSchedErrorInvalidValue;
    auto c = std::make_shared<LaneCommand>(spin_us);
    const HwCommandHandle h = HwCommandManager::Add(c);
    { std::lock_guard<std::mutex> lk(g_mu); Kept()[h] = c; }
    *hw_cmd = h;
    return kXSchedSuccess;
}

LANE_EXPORT XResult HostLaneCommandLaunchTime(HwCommandHandle hw_cmd, int64_t *launch_ns) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = Kept().find(hw_cmd);
    if (it == Kept().end() || launch_ns == nullptr) return kXSchedErrorNotFound;
    *launch_ns = it->second->launch_ns_.load();
    return kXSchedSuccess;
}

LANE_EXPORT XResult HostLaneCommandTimes(HwCommandHandle hw_cmd, int64_t *start_ns, int64_t *finish_ns) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = Kept().find(hw_cmd);
    if (it == Kept().end()) return kXSchedErrorNotFound;
    if (start_ns) *start_ns = it->second->start_ns_.load();
    if (finish_ns) *finish_ns = it->second->finish_ns_.load();
    return kXSchedSuccess;
}

LANE_EXPORT XResult HostLaneCommandRelease(HwCommandHandle hw_cmd) {
    std::lock_guard<std::mutex> lk(g_mu);
    return Kept().erase(hw_cmd) ? kXSchedSuccess : kXSchedErrorNotFound;
}

LANE_EXPORT XResult HostLaneStats(uint32_t lane_id, uint64_t *executed, uint64_t *flushed) {
    Lane *l = GetLane(lane_id);
    if (executed) *executed = l->executed.load();
    if (flushed) *flushed = l->flushed.load();
    return kXSchedSuccess;
}

LANE_EXPORT XResult HostLaneSetAffinity(uint32_t lane_id, int cpu) {
    GetLane(lane_id)->SetAffinity(cpu);
    return kXSchedSuccess;
}
