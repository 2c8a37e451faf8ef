// CUDA HwQueue.
//   Level 1  Launch = enqueue on the stream (+ completion-counter write when waitable);
//            Synchronize = take a ticket, write it behind everything, wait for it on the host word.
//   Level 2  Deactivate = raise the queue's preempt flag (one 32-bit stream memory write on a separate
//            high-priority stream): running xpk kernels stop at their next tile boundary, xpk kernels
//            queued behind them start, see the flag and return at once.  Reactivate = wait for the
//            stream to drain, lower the flag, relaunch from the first unfinished xpk command on; each
//            xpk task continues from its tile cursor.
// Contract: preempt/include/xsched/preempt/hal/hw_queue.h:19-77 (reference); the level-1 behaviour
// corresponds to platforms/cuda/hal/src/level1/cuda_queue.cpp:15-98 and the level-2 flush/replay to
// platforms/cuda/hal/src/level2/cuda_queue.cpp:8-72 + instrument.cpp:181-222.
#include <chrono>
#include <mutex>
#include "hal_cuda/cuda_command.h"
#include "hal_cuda/driver.h"
#include "xsched/cuda/hal.h"
#include "xsched/preempt/hal/hw_queue.h"
#include "xsched/preempt/xqueue/xqueue.h"
#include "xsched/protocol/names.h"
#include "xsched/utils/trace.h"
#include "xsched_b200/pk.h"
#include "xsched/utils/xassert.h"

namespace xsched::cuda {

using namespace xsched::preempt;

static int64_t NowNs() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Makes a queue's CUDA context current for the duration of a call.  HAL entry points are called from
// several threads (the XQueue worker, the scheduler's executor thread, application threads); a thread
// that never bound a context would otherwise run runtime-API launches on device 0's primary context,
// whatever device the queue belongs to.
class ContextScope {
public:
    explicit ContextScope(CUcontext ctx) { CUDA_ASSERT(Driver().cuCtxPushCurrent(ctx)); }
    ~ContextScope() { CUcontext old; Driver().cuCtxPopCurrent(&old); }
    ContextScope(const ContextScope &) = delete;
    ContextScope &operator=(const ContextScope &) = delete;
};

class CudaQueue final : public HwQueue {
public:
    explicit CudaQueue(CUstream stream) : stream_(stream) {
        const DriverApi &d = Driver();
        CUcontext cur = nullptr, sctx = nullptr;
        CUDA_ASSERT(d.cuCtxGetCurrent(&cur));
        CUDA_ASSERT(d.cuStreamGetCtx(stream, &sctx));
        XASSERT(cur == sctx, "CudaQueueCreate: the current context (%p) is not the stream's context (%p)", (void *)cur, (void *)sctx);
        ctx_ = sctx;
        CUdevice dev;
        CUDA_ASSERT(d.cuCtxGetDevice(&dev));
        int dom = 0, bus = 0, devid = 0;
        CUDA_ASSERT(d.cuDeviceGetAttribute(&dom, CU_DEVICE_ATTRIBUTE_PCI_DOMAIN_ID, dev));
        CUDA_ASSERT(d.cuDeviceGetAttribute(&bus, CU_DEVICE_ATTRIBUTE_PCI_BUS_ID, dev));
        CUDA_ASSERT(d.cuDeviceGetAttribute(&devid, CU_DEVICE_ATTRIBUTE_PCI_DEVICE_ID, dev));
        xdevice_ = protocol::MakeDevice(kDeviceTypeGPU, protocol::MakePciId((uint32_t)dom, (uint32_t)bus, (uint32_t)devid, 0));

        counter_ = std::make_shared<CompletionCounter>();
        void *host = nullptr;
        CUDA_ASSERT(d.cuMemHostAlloc(&host, 64, CU_MEMHOSTALLOC_DEVICEMAP | CU_MEMHOSTALLOC_PORTABLE));
        *(volatile uint64_t *)host = 0;
        counter_->host = (volatile uint64_t *)host;
        counter_->stream = stream_;
        counter_->ctx = ctx_;
        CUDA_ASSERT(d.cuMemHostGetDevicePointer(&counter_->dev, host, 0));

        CUDA_ASSERT(d.cuMemAlloc(&flag_, 256));
        CUDA_ASSERT(d.cuMemsetD32(flag_, 0, 64));
        // Early-warning word of the flag in mapped host memory (kernels with a relay see a raise ~2 us after the
        // store in Deactivate, instead of the 6-14 us the stream write takes): its device address goes into bytes
        // [8,16) of the flag block (layout: include/xsched_b200/pk.h, xpkFlagAttachRelay).  Driver calls only: the
        // interposer must not start a CUDA runtime inside a program that has none.
        void *relay_host = nullptr;
        CUdeviceptr relay_dev = 0;
        if (d.cuMemHostAlloc(&relay_host, 64, CU_MEMHOSTALLOC_DEVICEMAP | CU_MEMHOSTALLOC_PORTABLE) == CUDA_SUCCESS) {
            *(volatile uint32_t *)relay_host = 0;
            if (d.cuMemHostGetDevicePointer(&relay_dev, relay_host, 0) == CUDA_SUCCESS &&
                d.cuMemsetD32(flag_ + 8, (unsigned)(relay_dev & 0xFFFFFFFFu), 1) == CUDA_SUCCESS &&
                d.cuMemsetD32(flag_ + 12, (unsigned)(relay_dev >> 32), 1) == CUDA_SUCCESS)
                relay_ = (volatile uint32_t *)relay_host;
            else
                d.cuMemFreeHost(relay_host);
        }
        int lo = 0, hi = 0;
        CUDA_ASSERT(d.cuCtxGetStreamPriorityRange(&lo, &hi));
        CUDA_ASSERT(d.cuStreamCreateWithPriority(&ctrl_, CU_STREAM_NON_BLOCKING, hi));
        CUDA_ASSERT(d.cuStreamSynchronize(stream_));     // nothing may be running on the stream yet
    }
    ~CudaQueue() override {
        ContextScope scope(ctx_);
        const DriverApi &d = Driver();
        d.cuStreamDestroy(ctrl_);
        d.cuMemFree(flag_);
        if (relay_) d.cuMemFreeHost((void *)relay_);
        d.cuMemFreeHost((void *)counter_->host);
    }

    void Launch(std::shared_ptr<HwCommand> hw_cmd) override {
        ContextScope scope(ctx_);
        auto c = std::dynamic_pointer_cast<CudaCommand>(hw_cmd);
        XASSERT(c != nullptr, "a command that is not a CudaCommand was submitted to a CUDA queue");
        LaunchAndNote(c);
        stats_.launched.fetch_add(1, std::memory_order_relaxed);
    }

    void OnHwCommandSubmit(std::shared_ptr<HwCommand> hw_cmd) override {
        // A callback command enqueues on the stream by itself: from then on the newest completion write
        // is not known to be the last thing on the stream.
        if (std::dynamic_pointer_cast<CudaCommand>(hw_cmd) == nullptr) foreign_.store(true, std::memory_order_relaxed);
    }

    void Synchronize() override {
        // When the newest thing on the stream is already a completion write, wait for that one: no driver
        // call, and the write retires the moment the work before it ends.  This is the common case while
        // preempting (every command of a small window carries a write).
        uint64_t t = 0;
        {
            std::lock_guard<std::mutex> lk(tail_mu_);
            if (!foreign_.load(std::memory_order_relaxed)) t = tail_ticket_;
            if (t == 0) {
                ContextScope scope(ctx_);
                CUresult r = CUDA_SUCCESS;
                t = counter_->Issue(stream_, &r);
                CUDA_ASSERT(r);
                tail_ticket_ = t;
            }
        }
        counter_->Wait(t);
        const int64_t t0 = deactivate_ns_.exchange(0);
        if (t0) { stats_.last_preempt_ns.store((uint64_t)(NowNs() - t0)); XTRACE(utils::kTraceHwqSynced, GetHandle()); }
    }

    void Deactivate() override {
        ContextScope scope(ctx_);
        deactivate_ns_.store(NowNs());
        if (relay_) __atomic_store_n(relay_, 1u, __ATOMIC_SEQ_CST);
        CUDA_ASSERT(Driver().cuStreamWriteValue32(ctrl_, flag_, 1, CU_STREAM_WRITE_VALUE_DEFAULT));
        XTRACE(utils::kTraceDeactivateIssued, GetHandle());
        stats_.deactivations.fetch_add(1, std::memory_order_relaxed);
    }

    void Reactivate(const CommandLog &log) override {
        ContextScope scope(ctx_);
        const DriverApi &d = Driver();
        CUDA_ASSERT(d.cuStreamSynchronize(stream_));      // flushed kernels have published their cursors (and no relay is running)
        if (relay_) __atomic_store_n(relay_, 0u, __ATOMIC_SEQ_CST);
        CUDA_ASSERT(d.cuStreamWriteValue32(ctrl_, flag_, 0, CU_STREAM_WRITE_VALUE_DEFAULT));
        CUDA_ASSERT(d.cuStreamSynchronize(ctrl_));        // the flag is down before anything relaunches
        bool replay = false;
        for (const auto &hc : log) {
            auto c = std::dynamic_pointer_cast<CudaCommand>(hc);
            if (!c) continue;
            auto x = std::dynamic_pointer_cast<CudaXpkCommand>(c);
            if (!replay) {
                if (!x || x->TaskCompleted()) continue;   // finished before the flush
                replay = true;                            // first unfinished preemptible command
            } else if (x && x->TaskCompleted()) {
                continue;
            }
            if (x && utils::TraceEnabled()) {
                uint64_t start_ns = 0, exit_ns = 0;         // device stamps of the launch that was flushed
                if (xpkTaskTimes((xpkTask_t)x->Task(), &start_ns, &exit_ns) == XPK_SUCCESS) XTRACE(utils::kTraceTaskGpuTimes, start_ns, exit_ns);
            }
            LaunchAndNote(c);
            stats_.relaunches.fetch_add(1, std::memory_order_relaxed);
        }
    }

    XDevice GetDevice() override { return xdevice_; }
    HwQueueHandle GetHandle() override { return (HwQueueHandle)(uintptr_t)stream_; }
    bool SupportDynamicLevel() override { return true; }
    XPreemptLevel GetMaxSupportedLevel() override { return kPreemptLevelDeactivate; }
    void OnXQueueCreate() override { CUDA_ASSERT(Driver().cuCtxSetCurrent(ctx_)); }

    CUdeviceptr Flag() const { return flag_; }
    CUstream Stream() const { return stream_; }
    void FillStats(CudaQueueStats *s) const {
        s->launched = stats_.launched.load(); s->completed = counter_->Load(); s->window_stalls = 0;
        s->deactivations = stats_.deactivations.load(); s->relaunches = stats_.relaunches.load();
        s->last_preempt_ns = stats_.last_preempt_ns.load();
    }

private:
    void LaunchAndNote(const std::shared_ptr<CudaCommand> &c) {
        std::lock_guard<std::mutex> lk(tail_mu_);      // the stream's tail changes only under this lock
        const CUresult r = c->LaunchOn(stream_, counter_);
        // A refused command ends the process here (XERRO does not return), as a failed launch does under the
        // reference's CUDA_ASSERT: no command is ever registered as waitable without its completion write.
        if (UNLIKELY(r != CUDA_SUCCESS)) XERRO("the CUDA driver refused a queued command: %d (%s): %s", (int)r, ErrorString(r), c->Describe().c_str());
        tail_ticket_ = c->Synchronizable() ? c->Ticket() : 0;
    }

    CUstream stream_;
    CUcontext ctx_ = nullptr;
    std::mutex tail_mu_;
    uint64_t tail_ticket_ = 0;             // ticket of the completion write that ends the stream, 0 = unknown
    std::atomic<bool> foreign_{false};
    XDevice xdevice_ = 0;
    std::shared_ptr<CompletionCounter> counter_;
    CUdeviceptr flag_ = 0;
    volatile uint32_t *relay_ = nullptr;       // mapped host word announcing a raise of flag_ early
    CUstream ctrl_ = nullptr;
    std::atomic<int64_t> deactivate_ns_{0};
    struct { std::atomic<uint64_t> launched{0}, deactivations{0}, relaunches{0}, last_preempt_ns{0}; } stats_;
};

} // namespace xsched::cuda

using namespace xsched::cuda;
using namespace xsched::preempt;

static inline HwQueueHandle HandleOf(CUstream s) { return (HwQueueHandle)(uintptr_t)s; }

EXPORT_C_FUNC XResult CudaQueueCreate(HwQueueHandle *hwq, CUstream stream) {
    if (hwq == nullptr) return kXSchedErrorInvalidValue;
    if (stream == nullptr) { XWARN("CudaQueueCreate: the default stream is not supported"); return kXSchedErrorNotSupported; }
    const XResult r = HwQueueManager::Add(HandleOf(stream), [&]() -> std::shared_ptr<HwQueue> { return std::make_shared<CudaQueue>(stream); });
    if (r == kXSchedSuccess) *hwq = HandleOf(stream);
    return r;
}

EXPORT_C_FUNC XResult CudaQueueGet(HwQueueHandle *hwq, CUstream stream) {
    if (hwq == nullptr) return kXSchedErrorInvalidValue;
    if (stream == nullptr) return kXSchedErrorNotSupported;
    if (HwQueueManager::Get(HandleOf(stream)) == nullptr) return kXSchedErrorNotFound;
    *hwq = HandleOf(stream);
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult CudaQueueGetPreemptFlag(HwQueueHandle hwq, uint32_t **flag_dev) {
    if (flag_dev == nullptr) return kXSchedErrorInvalidValue;
    auto q = std::dynamic_pointer_cast<CudaQueue>(HwQueueManager::Get(hwq));
    if (!q) return kXSchedErrorNotFound;
    *flag_dev = (uint32_t *)(uintptr_t)q->Flag();
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult CudaXpkCommandCreate(HwCommandHandle *hw_cmd, void *xpk_task, int rewind) {
    if (hw_cmd == nullptr || xpk_task == nullptr) return kXSchedErrorInvalidValue;
    *hw_cmd = HwCommandManager::Add(std::make_shared<CudaXpkCommand>(xpk_task, rewind != 0));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult CudaMemcpyCommandCreate(HwCommandHandle *hw_cmd, void *dst, const void *src, size_t bytes, int kind) {
    if (hw_cmd == nullptr || dst == nullptr || src == nullptr || kind < 0 || kind > 2) return kXSchedErrorInvalidValue;
    const CopyKind k = kind == 0 ? CopyKind::kHtoD : (kind == 1 ? CopyKind::kDtoH : CopyKind::kDtoD);
    *hw_cmd = HwCommandManager::Add(std::make_shared<CudaMemcpyCommand>(k, (CUdeviceptr)(uintptr_t)dst, (CUdeviceptr)(uintptr_t)src, bytes));
    return kXSchedSuccess;
}

EXPORT_C_FUNC XResult CudaQueueGetStats(HwQueueHandle hwq, CudaQueueStats *stats) {
    if (stats == nullptr) return kXSchedErrorInvalidValue;
    auto q = std::dynamic_pointer_cast<CudaQueue>(HwQueueManager::Get(hwq));
    if (!q) return kXSchedErrorNotFound;
    q->FillStats(stats);
    return kXSchedSuccess;
}
