// HwCommand: one unit of work for a hardware queue.  This is the half of the HAL contract a backend
// implements per command; it keeps the reference's interface
// (preempt/include/xsched/preempt/hal/hw_command.h:16-94) method for method.
#pragma once
#include <memory>
#include <mutex>
#include <unordered_map>
#include "xsched/types.h"
#include "xsched/utils/common.h"
#include "xsched/preempt/xqueue/xcommand.h"

namespace xsched::preempt {

class XQueue;

class HwCommand : public XCommand {
public:
    explicit HwCommand(XCommandProperties props = kCommandPropertyNone);
    virtual ~HwCommand() = default;

    /// Block until the hardware finished this command.  May also return once the command was flushed
    /// by HwQueue::Deactivate or killed by HwQueue::Interrupt.  Only valid after
    /// EnableSynchronization() returned true and the command was launched.
    virtual void Synchronize() = 0;
    /// Whether Synchronize() may be called.
    virtual bool Synchronizable() = 0;
    /// Ask the backend to make this command individually waitable (an event, a fence, a completion
    /// counter written after it).  Returns false if the backend cannot.
    virtual bool EnableSynchronization() = 0;
    /// Called on the worker thread right before Launch, without the worker lock held; may block
    /// (e.g. a stream-wait-event command waits here until the event's record command completed).
    virtual void BeforeLaunch() {}

    /// Process-unique handle (object address xor pid << 48).
    virtual HwCommandHandle GetHandle() { return (uint64_t)this ^ ((uint64_t)GetProcessId() << 48); }

    /// 1-based submission index inside its XQueue; valid after Submit.
    int64_t GetIdx() const { return idx_; }
    void SetIdx(int64_t idx) { idx_ = idx; }
    /// 0 until the command is submitted to an XQueue.
    XQueueHandle GetXQueueHandle() const { return xqueue_handle_; }

    /// Wait for real completion: through the owning XQueue when submitted, else Synchronize().
    virtual void Wait() final override;
    void OnSubmit(std::shared_ptr<XQueue> xqueue);

private:
    int64_t idx_ = -1;
    XQueueHandle xqueue_handle_ = 0;
    std::shared_ptr<XQueue> xqueue_ = nullptr;     // dropped when the command completes
};

/// A command whose launch is an application callback (HwCommandCreateCallback).
class HwCallbackCommand final : public HwCommand {
public:
    HwCallbackCommand(LaunchCallback launch, void *data) : HwCommand(kCommandPropertyNone), launch_(launch), data_(data) {}
    void Synchronize() override {}
    bool Synchronizable() override { return false; }
    bool EnableSynchronization() override { return false; }
    XResult Launch(HwQueueHandle hwq) { return launch_(hwq, data_); }
private:
    LaunchCallback launch_;
    void *data_;
};

/// Registry behind HwCommandHandle values handed to C callers.
class HwCommandManager {
public:
    STATIC_CLASS(HwCommandManager);
    static HwCommandHandle Add(std::shared_ptr<HwCommand> hw_cmd);
    static std::shared_ptr<HwCommand> Del(HwCommandHandle hw_cmd_h);    // removes and returns
    static std::shared_ptr<HwCommand> Get(HwCommandHandle hw_cmd_h);
};

} // namespace xsched::preempt
