// HwQueue: the hardware-queue half of the HAL contract — Launch / Synchronize (level 1),
// Deactivate / Reactivate (level 2), Interrupt / Restore (level 3) plus life-cycle hooks.  Interface
// as in the reference's preempt/include/xsched/preempt/hal/hw_queue.h:19-93.
//
// Threading rules the XQueue core guarantees to a backend:
//   * Launch runs on the XQueue's worker thread with the worker lock held: it must not block.
//   * Synchronize runs without the worker lock and may be blocked while Deactivate is called from
//     another thread; it may return early once the queue was flushed.
//   * Deactivate/Interrupt run on the thread that called XQueue::Suspend (the scheduler executor);
//     Restore/Reactivate run on the thread that called XQueue::Resume, before the worker is released.
#pragma once
#include <functional>
#include <list>
#include <memory>
#include "xsched/types.h"
#include "xsched/utils/common.h"
#include "xsched/preempt/hal/hw_command.h"

namespace xsched::preempt {

class XQueue;
/// Commands launched on the HwQueue and not yet known to be complete, oldest first.
using CommandLog = std::list<std::shared_ptr<HwCommand>>;

class HwQueue {
public:
    HwQueue() = default;
    virtual ~HwQueue() = default;

    virtual void Launch(std::shared_ptr<HwCommand> hw_cmd) = 0;
    virtual void Synchronize() = 0;

    virtual void Deactivate() {}
    virtual void Reactivate(const CommandLog &log) { UNUSED(log); }
    virtual void Interrupt() {}
    virtual void Restore(const CommandLog &log) { UNUSED(log); }

    virtual XDevice GetDevice() = 0;
    virtual HwQueueHandle GetHandle() = 0;
    virtual bool SupportDynamicLevel() = 0;
    virtual XPreemptLevel GetMaxSupportedLevel() = 0;

    virtual void OnPreemptLevelChange(XPreemptLevel level) { UNUSED(level); }
    /// Runs once on the freshly created worker thread (a CUDA backend binds its context here).
    virtual void OnXQueueCreate() {}
    /// Runs in XQueue::Submit, on the submitting thread, before the command is queued.
    virtual void OnHwCommandSubmit(std::shared_ptr<HwCommand> hw_cmd) { UNUSED(hw_cmd); }

    std::shared_ptr<XQueue> GetXQueue() { return xq_; }
    void SetXQueue(std::shared_ptr<XQueue> xq) { xq_ = std::move(xq); }

private:
    std::shared_ptr<XQueue> xq_ = nullptr;
};

/// Registry behind HwQueueHandle values.  A backend registers a queue with Add(handle, factory); the
/// factory runs only if the handle is new (creation is idempotent).
class HwQueueManager {
public:
    STATIC_CLASS(HwQueueManager);
    static XResult Add(HwQueueHandle hwq_h, std::function<std::shared_ptr<HwQueue>()> create);
    static XResult Del(HwQueueHandle hwq_h);             // NotAllowed while an XQueue is attached
    static std::shared_ptr<HwQueue> Get(HwQueueHandle hwq_h);
    static std::shared_ptr<XQueue> GetXQueue(HwQueueHandle hwq_h);
};

} // namespace xsched::preempt
