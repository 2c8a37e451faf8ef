// XCommand state machine: Created -> Pending -> InFlight -> Completed, monotone
// (reference: preempt/src/xqueue/xcommand.cpp:6-33).  Waiters sleep on the state word itself
// (std::atomic wait/notify, a futex on Linux).
#include "xsched/preempt/xqueue/xcommand.h"
#include "xsched/utils/xassert.h"

namespace xsched::preempt {

void XCommand::SetState(XCommandState state) {
    XASSERT(state >= kCommandStateCreated && state <= kCommandStateCompleted, "invalid command state %d", (int)state);
    int32_t old = state_.load(std::memory_order_acquire);
    while (true) {
        XASSERT((int32_t)state >= old, "command state must not go back (%d -> %d)", old, (int)state);
        if ((int32_t)state == old) return;
        if (state_.compare_exchange_weak(old, (int32_t)state, std::memory_order_acq_rel)) break;
    }
    state_.notify_all();
    std::vector<std::function<void(XCommandState)>> ls;
    {
        std::lock_guard<std::mutex> lk(mtx_);
        ls = listeners_;
    }
    for (int32_t s = old + 1; s <= (int32_t)state; ++s)
        for (auto &l : ls) l((XCommandState)s);
}

void XCommand::WaitUntil(XCommandState state) {
    // Short spin first: most waits end within tens of microseconds and a futex sleep + wake costs that much.
    for (int i = 0; i < 2000; ++i) {
        if (state_.load(std::memory_order_acquire) >= (int32_t)state) return;
        __builtin_ia32_pause();
    }
    int32_t cur = state_.load(std::memory_order_acquire);
    while (cur < (int32_t)state) {
        state_.wait(cur, std::memory_order_acquire);
        cur = state_.load(std::memory_order_acquire);
    }
}

void XCommand::AddStateListener(std::function<void(XCommandState)> listener) {
    std::lock_guard<std::mutex> lk(mtx_);
    listeners_.push_back(std::move(listener));
}

} // namespace xsched::preempt
