// XCommand: anything an XQueue's worker consumes.  Contract (names, enumerators, semantics) as in the
// reference's preempt/include/xsched/preempt/xqueue/xcommand.h:14-137; the state word here is a
// futex-backed atomic instead of a mutex + condition variable, so a state query never takes a lock
// and a waiter is woken by the one store that changes the state.
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <vector>
#include "xsched/types.h"

namespace xsched::preempt {

enum XCommandType {
    kCommandTypeHardware         = 0,   // a HwCommand, launched on the HwQueue
    kCommandTypeHostFunction     = 1,   // runs on the worker after everything before it completed
    kCommandTypeXQueueWaitAll    = 2,   // completes when everything before it completed
    kCommandTypeBatchSynchronize = 3,   // worker-internal: wait for the oldest synchronizable command
    kCommandTypeXQueueDestroy    = 4,   // ends the worker
};

typedef int64_t XCommandProperties;
enum XCommandProperty {
    kCommandPropertyNone           = 0x0000,  // neither deactivatable nor idempotent: under level >= 2 it is
                                              // launched only after every in-flight deactivatable command
                                              // has completed (it could not be stopped with them)
    kCommandPropertyDeactivatable  = 0x0001,  // HwQueue::Deactivate stops it; Reactivate re-executes it safely
    kCommandPropertyIdempotent     = 0x0002,  // may be re-executed freely (writes no memory)
    kCommandPropertyBlockingSubmit = 0x0004,  // Submit() returns only once it is in flight
    kCommandPropertyTransferOnly   = 0x0008,  // (addition) moves data over the host link and occupies no compute unit;
                                              // with XSCHED_TRANSFER_AWARE_READY=ON such commands alone do not make
                                              // their XQueue "ready" in the scheduler's eyes
    kCommandPropertyMaskAll        = -1,
};

enum XCommandState {
    kCommandStateCreated = 0, kCommandStatePending = 1, kCommandStateInFlight = 2, kCommandStateCompleted = 3,
    kCommandStateMax = 4,
};

class XCommand : public std::enable_shared_from_this<XCommand> {
public:
    explicit XCommand(XCommandType type, XCommandProperties props = kCommandPropertyNone) : kCommandType(type), props_(props) {}
    virtual ~XCommand() = default;

    virtual void Wait() { WaitUntil(kCommandStateCompleted); }

    XCommandState GetState() const { return (XCommandState)state_.load(std::memory_order_acquire); }
    /// Monotone: moving backwards is a fatal error, repeating the current state is a no-op.  Listeners
    /// are called once for every state crossed, in order.
    void SetState(XCommandState state);
    void WaitUntil(XCommandState state);
    void AddStateListener(std::function<void(XCommandState)> listener);
    /// Lock for short critical sections on fields derived classes attach to the command.
    std::unique_lock<std::mutex> GetLock() { return std::unique_lock<std::mutex>(mtx_); }

    XCommandType GetType() const { return kCommandType; }
    void SetProps(XCommandProperties props) { props_ |= props; }
    XCommandProperties GetProps(XCommandProperties mask = kCommandPropertyMaskAll) const { return props_ & mask; }

private:
    const XCommandType kCommandType;
    XCommandProperties props_;
    std::atomic<int32_t> state_{kCommandStateCreated};
    std::mutex mtx_;
    std::vector<std::function<void(XCommandState)>> listeners_;
};

class HostFunctionCommand final : public XCommand {
public:
    explicit HostFunctionCommand(std::function<void()> f) : XCommand(kCommandTypeHostFunction), func_(std::move(f)) {}
    void Execute() { func_(); }
private:
    std::function<void()> func_;
};

class XQueueWaitAllCommand final : public XCommand {
public:
    XQueueWaitAllCommand() : XCommand(kCommandTypeXQueueWaitAll) {}
};
class BatchSynchronizeCommand final : public XCommand {
public:
    BatchSynchronizeCommand() : XCommand(kCommandTypeBatchSynchronize) {}
};
class XQueueDestroyCommand final : public XCommand {
public:
    XQueueDestroyCommand() : XCommand(kCommandTypeXQueueDestroy) {}
};

} // namespace xsched::preempt
