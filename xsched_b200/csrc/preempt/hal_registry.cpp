// HwCommand base behaviour, the HwQueue / HwCommand handle registries and the C entry points
// HwQueueDestroy / HwQueueLaunch / HwQueueSynchronize / HwCommandCreateCallback / HwCommandDestroy
// (reference: preempt/src/hal/hw_command.cpp:9-99, preempt/src/hal/hw_queue.cpp:10-101).
#include <mutex>
#include <unordered_map>
#include "xsched/xsched.h"
#include "xsched/preempt/hal/hw_command.h"
#include "xsched/preempt/hal/hw_queue.h"
#include "xsched/preempt/xqueue/xqueue.h"
#include "xsched/utils/xassert.h"

namespace xsched::preempt {

// ---------------------------------------------------------------------------------- HwCommand
HwCommand::HwCommand(XCommandProperties props) : XCommand(kCommandTypeHardware, props) {
    // The command keeps its XQueue alive while it is queued; let go once it is complete.
    AddStateListener([this](XCommandState s) {
        if (s < kCommandStateCompleted) return;
        std::shared_ptr<XQueue> drop;
        auto lk = GetLock();
        drop.swap(xqueue_);
        lk.unlock();
    });
}

void HwCommand::Wait() {
    std::shared_ptr<XQueue> xq;
    XQueueHandle xq_h;
    {
        auto lk = GetLock();
        xq = xqueue_;
        xq_h = xqueue_handle_;
    }
    if (xq_h == 0) {      // never submitted to an XQueue: wait on the hardware directly
        XASSERT(Synchronizable(), "a HwCommand that is waited on must be synchronizable or submitted to an XQueue");
        Synchronize();
        return;
    }
    if (xq == nullptr) {  // the XQueue reference is dropped only at completion
        XASSERT(GetState() >= kCommandStateCompleted, "HwCommand lost its XQueue before completing");
        return;
    }
    xq->Wait(std::static_pointer_cast<HwCommand>(shared_from_this()));
}

void HwCommand::OnSubmit(std::shared_ptr<XQueue> xqueue) {
    XASSERT(xqueue != nullptr, "OnSubmit without an XQueue");
    auto lk = GetLock();
    xqueue_handle_ = xqueue->GetHandle();
    xqueue_ = std::move(xqueue);
}

// ---------------------------------------------------------------------------------- registries
namespace {
std::mutex g_cmd_mtx;
std::unordered_map<HwCommandHandle, std::shared_ptr<HwCommand>> &Cmds() {
    static auto *m = new std::unordered_map<HwCommandHandle, std::shared_ptr<HwCommand>>();
    return *m;
}
std::mutex g_hwq_mtx;
std::unordered_map<HwQueueHandle, std::shared_ptr<HwQueue>> &Hwqs() {
    static auto *m = new std::unordered_map<HwQueueHandle, std::shared_ptr<HwQueue>>();
    return *m;
}
} // namespace

HwCommandHandle HwCommandManager::Add(std::shared_ptr<HwCommand> hw_cmd) {
    const HwCommandHandle h = hw_cmd->GetHandle();
    std::lock_guard<std::mutex> lk(g_cmd_mtx);
    Cmds()[h] = std::move(hw_cmd);
    return h;
}

std::shared_ptr<HwCommand> HwCommandManager::Del(HwCommandHandle h) {
    std::lock_guard<std::mutex> lk(g_cmd_mtx);
    auto it = Cmds().find(h);
    if (it == Cmds().end()) return nullptr;
    auto cmd = std::move(it->second);
    Cmds().erase(it);
    return cmd;
}

std::shared_ptr<HwCommand> HwCommandManager::Get(HwCommandHandle h) {
    std::lock_guard<std::mutex> lk(g_cmd_mtx);
    auto it = Cmds().find(h);
    return it == Cmds().end() ? nullptr : it->second;
}

XResult HwQueueManager::Add(HwQueueHandle h, std::function<std::shared_ptr<HwQueue>()> create) {
    std::lock_guard<std::mutex> lk(g_hwq_mtx);
    if (Hwqs().count(h)) {
        XDEBG("HwQueue 0x" FMT_64X " already registered", h);
        return kXSchedSuccess;
    }
    auto hwq = create();
    if (hwq == nullptr) {
        XWARN("could not create HwQueue 0x" FMT_64X, h);
        return kXSchedErrorUnknown;
    }
    XASSERT(hwq->GetHandle() == h, "HwQueue handle mismatch");
    Hwqs()[h] = std::move(hwq);
    return kXSchedSuccess;
}

XResult HwQueueManager::Del(HwQueueHandle h) {
    std::lock_guard<std::mutex> lk(g_hwq_mtx);
    auto it = Hwqs().find(h);
    if (it == Hwqs().end()) {
        XWARN("HwQueue 0x" FMT_64X " does not exist", h);
        return kXSchedErrorNotFound;
    }
    if (auto xq = it->second->GetXQueue()) {
        XWARN("HwQueue 0x" FMT_64X " still has XQueue 0x" FMT_64X " attached; destroy the XQueue first", h, xq->GetHandle());
        return kXSchedErrorNotAllowed;
    }
    Hwqs().erase(it);
    return kXSchedSuccess;
}

std::shared_ptr<HwQueue> HwQueueManager::Get(HwQueueHandle h) {
    std::lock_guard<std::mutex> lk(g_hwq_mtx);
    auto it = Hwqs().find(h);
    return it == Hwqs().end() ? nullptr : it->second;
}

std::shared_ptr<XQueue> HwQueueManager::GetXQueue(HwQueueHandle h) {
    auto hwq = Get(h);
    return hwq ? hwq->GetXQueue() : nullptr;
}

} // namespace xsched::preempt

using namespace xsched::preempt;

EXPORT_C_FUNC XResult HwQueueDestroy(HwQueueHandle hwq) { return HwQueueManager::Del(hwq); }

EXPORT_C_FUNC XResult HwQueueLaunch(HwQueueHandle hwq, HwCommandHandle hw_cmd) {
    auto q = HwQueueManager::Get(hwq);
    if (!q) { XWARN("HwQueue 0x" FMT_64X " does not exist", hwq); return kXSchedErrorNotFound; }
    auto cmd = HwCommandManager::Del(hw_cmd);      // the handle is consumed
    if (!cmd) { XWARN("HwCommand 0x" FMT_64X " does not exist", hw_cmd); return kXSchedErrorNotFound; }
    if (auto cb = std::dynamic_pointer_cast<HwCallbackCommand>(cmd)) return cb->Launch(hwq);
    q->Launch(cmd);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult HwQueueSynchronize(HwQueueHandle hwq) {
    auto q = HwQueueManager::Get(hwq);
    if (!q) { XWARN("HwQueue 0x" FMT_64X " does not exist", hwq); return kXSchedErrorNotFound; }
    q->Synchronize();
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult HwCommandCreateCallback(HwCommandHandle *hw_cmd, LaunchCallback launch, void *data) {
    if (hw_cmd == nullptr) return kXSchedErrorInvalidValue;
    *hw_cmd = HwCommandManager::Add(std::make_shared<HwCallbackCommand>(launch, data));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult HwCommandDestroy(HwCommandHandle hw_cmd) {
    if (!HwCommandManager::Del(hw_cmd)) {
        XWARN("HwCommand 0x" FMT_64X " does not exist", hw_cmd);
        return kXSchedErrorNotFound;
    }
    return kXSchedSuccess;
}
