// XQueue registry and the XQueue* C entry points (reference: preempt/src/xqueue/xqueue.cpp:12-402).
#include <list>
#include <mutex>
#include <unordered_map>
#include "preempt/windowed_xqueue.h"
#include "xsched/xsched.h"
#include "xsched/protocol/def.h"
#include "xsched/utils/xassert.h"

namespace xsched::preempt {

namespace {
std::mutex g_xq_mtx;
std::unordered_map<XQueueHandle, std::shared_ptr<XQueue>> &Xqs() {
    static auto *m = new std::unordered_map<XQueueHandle, std::shared_ptr<XQueue>>();
    return *m;
}
} // namespace

XResult XQueueManager::Add(XQueueHandle *xq_hp, HwQueueHandle hwq_h, int64_t level, int64_t flags) {
    if (xq_hp == nullptr) return kXSchedErrorInvalidValue;
    if (level <= kPreemptLevelUnknown || level >= kPreemptLevelMax) return kXSchedErrorInvalidValue;
    if (flags & kQueueCreateFlagBlockingSubmit) return kXSchedErrorNotSupported;     // no blocking XQueue

    std::lock_guard<std::mutex> lk(g_xq_mtx);
    auto hwq = HwQueueManager::Get(hwq_h);
    if (!hwq) {
        XWARN("HwQueue 0x" FMT_64X " does not exist or is not registered", hwq_h);
        return kXSchedErrorNotFound;
    }
    if (auto existing = hwq->GetXQueue()) {          // one XQueue per HwQueue: hand the existing one back
        XASSERT(Xqs().count(existing->GetHandle()), "XQueue 0x" FMT_64X " is attached but not registered", existing->GetHandle());
        *xq_hp = existing->GetHandle();
        return kXSchedSuccess;
    }
    auto xq = std::make_shared<WindowedXQueue>(hwq, (XPreemptLevel)level);
    hwq->SetXQueue(xq);                              // reference cycle, broken in Del()
    Xqs()[xq->GetHandle()] = xq;
    *xq_hp = xq->GetHandle();
    return kXSchedSuccess;
}

XResult XQueueManager::Del(XQueueHandle xq_h) {
    std::shared_ptr<XQueue> xq;
    {
        std::lock_guard<std::mutex> lk(g_xq_mtx);
        auto it = Xqs().find(xq_h);
        if (it == Xqs().end()) {
            XWARN("XQueue 0x" FMT_64X " does not exist", xq_h);
            return kXSchedErrorNotFound;
        }
        xq = it->second;
        if (auto hwq = xq->GetHwQueue()) hwq->SetXQueue(nullptr);
        Xqs().erase(it);
    }
    // Let everything submitted finish so the worker never touches the HwQueue after this returns.
    xq->Resume(kQueueResumeFlagNone);
    xq->WaitAll();
    return kXSchedSuccess;
}

XResult XQueueManager::Exists(XQueueHandle xq_h) {
    std::lock_guard<std::mutex> lk(g_xq_mtx);
    return Xqs().count(xq_h) ? kXSchedSuccess : kXSchedErrorNotFound;
}

std::shared_ptr<XQueue> XQueueManager::Get(XQueueHandle xq_h) {
    std::lock_guard<std::mutex> lk(g_xq_mtx);
    auto it = Xqs().find(xq_h);
    return it == Xqs().end() ? nullptr : it->second;
}

XResult XQueueManager::ForEachWaitAll() {
    std::list<std::shared_ptr<XQueueWaitAllCommand>> markers;
    {
        std::lock_guard<std::mutex> lk(g_xq_mtx);
        for (auto &[h, xq] : Xqs()) {
            auto m = xq->SubmitWaitAll();
            if (!m) return kXSchedErrorUnknown;
            markers.push_back(std::move(m));
        }
    }
    for (auto &m : markers) m->Wait();
    return kXSchedSuccess;
}

XResult XQueueManager::ForEach(std::function<XResult(std::shared_ptr<XQueue>)> func) {
    std::lock_guard<std::mutex> lk(g_xq_mtx);
    for (auto &[h, xq] : Xqs()) {
        const XResult r = func(xq);
        if (r != kXSchedSuccess) return r;
    }
    return kXSchedSuccess;
}

XResult XQueueManager::AutoCreate(std::function<XResult(HwQueueHandle *)> create_hwq) {
    if (!GetEnvOption(XSCHED_AUTO_XQUEUE_ENV_NAME, false)) return kXSchedSuccess;
    HwQueueHandle hwq = 0;
    XResult res = create_hwq(&hwq);
    if (res != kXSchedSuccess) { XWARN("auto-create: HwQueue creation failed (%d)", (int)res); return res; }

    int64_t v = 0;
    int64_t level = XSCHED_DEFAULT_PREEMPT_LEVEL;
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_LEVEL_ENV_NAME, v)) level = v;
    XQueueHandle xq = 0;
    res = XQueueCreate(&xq, hwq, level, kQueueCreateFlagNone);
    if (res != kXSchedSuccess) {
        XWARN("auto-create: XQueue (level " FMT_64D ") for HwQueue 0x" FMT_64X " failed (%d)", level, hwq, (int)res);
        return res;
    }

    int64_t threshold = -1, batch = -1;
    const bool set_th = GetEnvInt64(XSCHED_AUTO_XQUEUE_THRESHOLD_ENV_NAME, threshold);
    const bool set_bs = GetEnvInt64(XSCHED_AUTO_XQUEUE_BATCH_SIZE_ENV_NAME, batch);
    if (set_th || set_bs) {
        res = XQueueSetLaunchConfig(xq, threshold, batch);
        if (res != kXSchedSuccess) XWARN("auto-create: launch config [" FMT_64D ", " FMT_64D "] refused (%d)", threshold, batch, (int)res);
    }
    int64_t prio = PRIORITY_DEFAULT;
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_PRIORITY_ENV_NAME, prio)) {
        res = XHintPriority(xq, (Priority)prio);
        if (res != kXSchedSuccess) XWARN("auto-create: priority hint refused (%d)", (int)res);
    }
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_UTILIZATION_ENV_NAME, v)) res = XHintUtilization(xq, (Utilization)v);
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_TIMESLICE_ENV_NAME, v)) res = XHintTimeslice(v);
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_DEADLINE_ENV_NAME, v)) res = XHintDeadline(xq, v);
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_KDEADLINE_ENV_NAME, v)) res = XHintKDeadline((size_t)v);
    // Laxity: relaxed priority 0, critical priority = the configured priority.
    if (GetEnvInt64(XSCHED_AUTO_XQUEUE_LAXITY_ENV_NAME, v)) res = XHintLaxity(xq, v, PRIORITY_DEFAULT, (Priority)prio);
    return res;
}

XResult XQueueManager::AutoDestroy(HwQueueHandle hwq_h) {
    if (!GetEnvOption(XSCHED_AUTO_XQUEUE_ENV_NAME, false)) return kXSchedSuccess;
    auto xq = HwQueueManager::GetXQueue(hwq_h);
    if (!xq) return kXSchedErrorNotFound;
    XResult res = XQueueDestroy(xq->GetHandle());
    if (res != kXSchedSuccess) return res;
    return HwQueueDestroy(hwq_h);
}

} // namespace xsched::preempt

using namespace xsched::preempt;

#define XQ_OR_RETURN(var, handle)                                              \
    std::shared_ptr<XQueue> var = XQueueManager::Get(handle);                  \
    if (var == nullptr) {                                                      \
        XWARN("XQueue 0x" FMT_64X " does not exist", (uint64_t)(handle));      \
        return kXSchedErrorNotFound;                                           \
    }

EXPORT_C_FUNC XResult XQueueCreate(XQueueHandle *xq, HwQueueHandle hwq, int64_t level, int64_t flags) {
    return XQueueManager::Add(xq, hwq, level, flags);
}

EXPORT_C_FUNC XResult XQueueDestroy(XQueueHandle xq) { return XQueueManager::Del(xq); }

EXPORT_C_FUNC XResult XQueueGet(XQueueHandle *xq, HwQueueHandle hwq) {
    if (xq == nullptr) return kXSchedErrorInvalidValue;
    auto q = HwQueueManager::GetXQueue(hwq);
    if (!q) return kXSchedErrorNotFound;
    *xq = q->GetHandle();
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueSetPreemptLevel(XQueueHandle xq, XPreemptLevel level) {
    if (level <= kPreemptLevelUnknown || level >= kPreemptLevelMax) return kXSchedErrorInvalidValue;
    XQ_OR_RETURN(q, xq);
    if (!q->GetFeatures(kQueueFeatureDynamicLevel)) return kXSchedErrorNotSupported;
    q->SetPreemptLevel(level);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueSetLaunchConfig(XQueueHandle xq, int64_t threshold, int64_t batch_size) {
    XQ_OR_RETURN(q, xq);
    if (threshold <= 0 && batch_size <= 0) return kXSchedSuccess;
    if (threshold > 0 && !q->GetFeatures(kQueueFeatureDynamicThreshold)) return kXSchedErrorNotSupported;
    if (batch_size > 0 && !q->GetFeatures(kQueueFeatureDynamicBatchSize)) return kXSchedErrorNotSupported;
    q->SetLaunchConfig(threshold, batch_size);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueSubmit(XQueueHandle xq, HwCommandHandle hw_cmd) {
    XQ_OR_RETURN(q, xq);
    auto cmd = HwCommandManager::Del(hw_cmd);        // ownership moves to the XQueue
    if (!cmd) { XWARN("HwCommand 0x" FMT_64X " does not exist", hw_cmd); return kXSchedErrorNotFound; }
    q->Submit(cmd);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueWait(XQueueHandle xq, HwCommandHandle hw_cmd) {
    XQ_OR_RETURN(q, xq);
    auto cmd = HwCommandManager::Get(hw_cmd);
    if (!cmd) { XWARN("HwCommand 0x" FMT_64X " does not exist", hw_cmd); return kXSchedErrorNotFound; }
    q->Wait(cmd);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueWaitAll(XQueueHandle xq) {
    XQ_OR_RETURN(q, xq);
    q->WaitAll();
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueQuery(XQueueHandle xq, XQueueState *state) {
    if (state == nullptr) return kXSchedErrorInvalidValue;
    XQ_OR_RETURN(q, xq);
    *state = q->Query();
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueSuspend(XQueueHandle xq, int64_t flags) {
    XQ_OR_RETURN(q, xq);
    q->Suspend(flags);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueResume(XQueueHandle xq, int64_t flags) {
    XQ_OR_RETURN(q, xq);
    q->Resume(flags);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult XQueueProfileHwCommandCount(XQueueHandle xq, int64_t *count) {
    if (count == nullptr) return kXSchedErrorInvalidValue;
    XQ_OR_RETURN(q, xq);
    *count = q->GetHwCommandCount();
    return kXSchedSuccess;
}
