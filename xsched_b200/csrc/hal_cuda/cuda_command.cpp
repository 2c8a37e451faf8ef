#include "hal_cuda/cuda_command.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>
#include <unordered_map>
#include <immintrin.h>
#include "hal_cuda/driver.h"
#include "xsched/utils/xassert.h"
#include "xsched_b200/pk.h"

namespace xsched::cuda {

void CompletionCounter::Wait(uint64_t ticket, int64_t expected_remaining_us) const {
    if (Load() >= ticket) return;
    // Phase 0: the work is known to need a while longer: sleep through half of it, looking in between.
    if (expected_remaining_us > 400) {
        int64_t budget = std::min<int64_t>(expected_remaining_us / 2, 5000);
        while (budget > 0 && Load() < ticket) {
            const int64_t slice = std::min<int64_t>(budget, 500);
            std::this_thread::sleep_for(std::chrono::microseconds(slice));
            budget -= slice;
        }
        if (Load() >= ticket) return;
    }
    // Phase 1: spin with pause for ~100 us (a completion is usually that close); phase 2: yield the core
    // between looks for up to ~1 ms; phase 3: sleep in 20 us slices so a long kernel does not burn a core.
    const auto t0 = std::chrono::steady_clock::now();
    auto elapsed_us = [&] { return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count(); };
    while (true) {
        for (int i = 0; i < 64; ++i) {
            if (Load() >= ticket) return;
            _mm_pause();
        }
        if (elapsed_us() > 100) break;
    }
    while (elapsed_us() < 1000) {
        if (Load() >= ticket) return;
        std::this_thread::yield();
    }
    // Phase 3 also looks at the stream itself every ~4 ms.
    int idle_looks = 0;
    for (uint32_t n = 1; Load() < ticket; ++n) {
        std::this_thread::sleep_for(std::chrono::microseconds(20));
        if ((n % 64u) != 0 || stream == nullptr) continue;
        const CUresult r = QueryStream();
        if (r == CUDA_ERROR_NOT_READY) { idle_looks = 0; continue; }
        if (Load() >= ticket) return;
        if (r != CUDA_SUCCESS)
            XERRO("waiting for completion ticket %llu: the stream's context reports error %d (%s)", (unsigned long long)ticket, (int)r, ErrorString(r));
        if (++idle_looks >= 3)
            XERRO("waiting for completion ticket %llu: the stream is idle but its counter stands at %llu (the write never ran)",
                  (unsigned long long)ticket, (unsigned long long)Load());
    }
}

CUresult CompletionCounter::QueryStream() const {
    const DriverApi &d = Driver();
    if (ctx && d.cuCtxPushCurrent(ctx) != CUDA_SUCCESS) return CUDA_ERROR_INVALID_CONTEXT;
    const CUresult r = d.cuStreamQuery(stream);
    CUcontext old;
    if (ctx) d.cuCtxPopCurrent(&old);
    return r;
}

uint64_t CompletionCounter::Issue(CUstream stream, CUresult *res) {
    std::lock_guard<std::mutex> lk(issue_mu);
    const uint64_t t = next_ticket.load(std::memory_order_relaxed) + 1;
    const CUresult r = Driver().cuStreamWriteValue64(stream, dev, t, CU_STREAM_WRITE_VALUE_DEFAULT);
    if (res) *res = r;
    if (r != CUDA_SUCCESS) return 0;
    next_ticket.store(t, std::memory_order_relaxed);
    return t;
}

void CudaCommand::Synchronize() {
    XASSERT(counter_ != nullptr && ticket_.load() != 0, "Synchronize() on a command that was not launched as waitable");
    counter_->Wait(ticket_.load(std::memory_order_acquire), ExpectedRemainingUs());
    OnWaited();
}

CUresult CudaCommand::LaunchOn(CUstream stream, const std::shared_ptr<CompletionCounter> &counter) {
    CUresult r = Enqueue(stream);
    if (r != CUDA_SUCCESS) return r;
    if (want_sync_.load(std::memory_order_acquire)) {
        // A relaunch after a flush takes a fresh ticket: the old write already executed behind the
        // flushed kernel and proves nothing.
        // (assigned once: a relaunch from the scheduler's thread may overlap a waiter reading it)
        if (counter_ == nullptr) counter_ = counter;
        const uint64_t t = counter->Issue(stream, &r);
        if (t) ticket_.store(t, std::memory_order_release);
    }
    return r;
}

// ------------------------------------------------------------------------------------ kernel launch
CudaKernelLaunchCommand::CudaKernelLaunchCommand(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                                                 unsigned bz, unsigned shmem, void **params, void **extra)
    : CudaCommand(preempt::kCommandPropertyNone), f_(f), g_{gx, gy, gz}, b_{bx, by, bz}, shmem_(shmem) {
    CopyArgs(params, extra);
}

CudaKernelLaunchCommand::CudaKernelLaunchCommand(const CUlaunchConfig *c, CUfunction f, void **params, void **extra)
    : CudaCommand(preempt::kCommandPropertyNone), f_(f), g_{c->gridDimX, c->gridDimY, c->gridDimZ},
      b_{c->blockDimX, c->blockDimY, c->blockDimZ}, shmem_(c->sharedMemBytes), use_ex_(true) {
    if (c->attrs && c->numAttrs) attrs_.assign(c->attrs, c->attrs + c->numAttrs);
    CopyArgs(params, extra);
}

// Offset and size of parameter i of a kernel, from whichever query understands the handle: the CUDA
// runtime and the math libraries launch library kernels (CUkernel handles passed where a CUfunction
// is expected), which the function-level query refuses.
static CUresult ParamInfo(CUfunction f, size_t i, size_t *off, size_t *sz, bool *as_kernel) {
    using KernelInfoFn = CUresult (*)(CUkernel, size_t, size_t *, size_t *);
    static const KernelInfoFn kernel_info = (KernelInfoFn)Driver().Sym("cuKernelGetParamInfo");
    if (!*as_kernel) {
        const CUresult r = Driver().cuFuncGetParamInfo(f, i, off, sz);
        if (r == CUDA_SUCCESS || r == CUDA_ERROR_INVALID_VALUE || i != 0 || !kernel_info) return r;
        *as_kernel = true;                  // first query refused the handle itself: try it as a CUkernel
    }
    return kernel_info((CUkernel)f, i, off, sz);
}

void CudaKernelLaunchCommand::CopyArgs(void **params, void **extra) {
    auto borrow = [&] {
        borrowed_ = true;
        caller_params_ = params;
        caller_extra_ = extra;
        SetProps(preempt::kCommandPropertyBlockingSubmit);
    };
    if (params != nullptr) {
        // Argument layout comes from the driver: offset and size of parameter i until it says "no more".
        std::vector<std::pair<size_t, size_t>> layout;
        size_t total = 0;
        bool as_kernel = false;
        for (size_t i = 0;; ++i) {
            size_t off = 0, sz = 0;
            const CUresult r = ParamInfo(f_, i, &off, &sz, &as_kernel);
            if (r != CUDA_SUCCESS) {
                // "Invalid value" ends the list; anything else means the layout cannot be asked for.
                if (r != CUDA_ERROR_INVALID_VALUE) { borrow(); return; }
                break;
            }
            layout.emplace_back(off, sz);
            total = std::max(total, off + sz);
        }
        arg_bytes_.resize(total);
        arg_ptrs_.resize(layout.size());
        for (size_t i = 0; i < layout.size(); ++i) {
            std::memcpy(arg_bytes_.data() + layout[i].first, params[i], layout[i].second);
            arg_ptrs_[i] = arg_bytes_.data() + layout[i].first;
        }
    } else if (extra != nullptr) {
        // CU_LAUNCH_PARAM_BUFFER_POINTER / _SIZE / _END list.
        void *buf = nullptr;
        size_t size = 0;
        for (int i = 0; extra[i] != CU_LAUNCH_PARAM_END && i < 16; i += 2) {
            if (extra[i] == CU_LAUNCH_PARAM_BUFFER_POINTER) buf = extra[i + 1];
            else if (extra[i] == CU_LAUNCH_PARAM_BUFFER_SIZE) size = *(size_t *)extra[i + 1];
        }
        if (buf == nullptr) { borrow(); return; }
        extra_bytes_.assign((unsigned char *)buf, (unsigned char *)buf + size);
        use_extra_ = true;
    }
}

CUresult CudaKernelLaunchCommand::Enqueue(CUstream stream) {
    void **params = arg_ptrs_.empty() ? nullptr : arg_ptrs_.data();
    void **extra = nullptr;
    size_t size = extra_bytes_.size();
    if (borrowed_) {
        params = caller_params_;
        extra = caller_extra_;
    } else if (use_extra_) {
        extra_[0] = CU_LAUNCH_PARAM_BUFFER_POINTER; extra_[1] = extra_bytes_.data();
        extra_[2] = CU_LAUNCH_PARAM_BUFFER_SIZE;    extra_[3] = &size;
        extra_[4] = CU_LAUNCH_PARAM_END;
        extra = extra_;
        params = nullptr;
    }
    if (use_ex_) {
        CUlaunchConfig c{};
        c.gridDimX = g_[0]; c.gridDimY = g_[1]; c.gridDimZ = g_[2];
        c.blockDimX = b_[0]; c.blockDimY = b_[1]; c.blockDimZ = b_[2];
        c.sharedMemBytes = shmem_;
        c.hStream = stream;
        c.attrs = attrs_.empty() ? nullptr : attrs_.data();
        c.numAttrs = (unsigned)attrs_.size();
        return Driver().cuLaunchKernelEx(&c, f_, params, extra);
    }
    return Driver().cuLaunchKernel(f_, g_[0], g_[1], g_[2], b_[0], b_[1], b_[2], shmem_, stream, params, extra);
}

std::string CudaKernelLaunchCommand::Describe() const {
    const char *name = nullptr;
    using GetNameFn = CUresult (*)(const char **, CUfunction);
    static const GetNameFn get_name = (GetNameFn)Driver().Sym("cuFuncGetName");
    if (get_name) get_name(&name, f_);
    char buf[512];
    snprintf(buf, sizeof(buf), "kernel %s grid (%u,%u,%u) block (%u,%u,%u) shmem %u, %zu params / %zu bytes%s%s, %zu attrs",
             name ? name : "?", g_[0], g_[1], g_[2], b_[0], b_[1], b_[2], shmem_, arg_ptrs_.size(), arg_bytes_.size(),
             use_extra_ ? ", extra buffer" : (borrowed_ ? ", borrowed arguments" : ""), use_ex_ ? ", cuLaunchKernelEx" : "", attrs_.size());
    return buf;
}

// ------------------------------------------------------------------------------------ copies, sets
bool IsPageableHost(const void *p) {
    unsigned type = 0;
    const CUresult r = Driver().cuPointerGetAttribute(&type, CU_POINTER_ATTRIBUTE_MEMORY_TYPE, (CUdeviceptr)(uintptr_t)p);
    return r != CUDA_SUCCESS || type == 0;
}

CudaMemcpyCommand::CudaMemcpyCommand(CopyKind kind, CUdeviceptr dst, CUdeviceptr src, size_t bytes, bool stage_source)
    : CudaCommand(kind == CopyKind::kHtoD || kind == CopyKind::kDtoH ? preempt::kCommandPropertyTransferOnly : preempt::kCommandPropertyNone),
      kind_(kind), dst_(dst), src_(src), bytes_(bytes) {
    if (stage_source && bytes) {
        const unsigned char *p = (const unsigned char *)(uintptr_t)src;
        staged_.assign(p, p + bytes);
        src_ = (CUdeviceptr)(uintptr_t)staged_.data();
    }
}

std::string CudaMemcpyCommand::Describe() const {
    char buf[160];
    snprintf(buf, sizeof(buf), "copy kind %d dst %#llx src %#llx bytes %zu%s", (int)kind_, (unsigned long long)dst_,
             (unsigned long long)src_, bytes_, staged_.empty() ? "" : " (staged source)");
    return buf;
}

CUresult CudaMemcpyCommand::Enqueue(CUstream stream) {
    const DriverApi &d = Driver();
    switch (kind_) {
    case CopyKind::kHtoD: return d.cuMemcpyHtoDAsync(dst_, (const void *)src_, bytes_, stream);
    case CopyKind::kDtoH: return d.cuMemcpyDtoHAsync((void *)dst_, src_, bytes_, stream);
    case CopyKind::kDtoD: return d.cuMemcpyDtoDAsync(dst_, src_, bytes_, stream);
    default: return d.cuMemcpyAsync(dst_, src_, bytes_, stream);
    }
}

CUresult CudaMemsetCommand::Enqueue(CUstream stream) {
    if (width_ == 1) return Driver().cuMemsetD8Async(dst_, (unsigned char)value_, count_, stream);
    return Driver().cuMemsetD32Async(dst_, value_, count_, stream);
}

CUresult CudaEventRecordCommand::Enqueue(CUstream stream) {
    if (!with_flags_) return Driver().cuEventRecord(ev_, stream);
    using Fn = CUresult (*)(CUevent, CUstream, unsigned);
    static const Fn record_with_flags = (Fn)Driver().Sym("cuEventRecordWithFlags");
    return record_with_flags ? record_with_flags(ev_, stream, flags_) : CUDA_ERROR_NOT_SUPPORTED;
}

void CudaEventWaitCommand::BeforeLaunch() {
    if (record_) record_->WaitUntil(preempt::kCommandStateInFlight);
}
CUresult CudaEventWaitCommand::Enqueue(CUstream stream) { return Driver().cuStreamWaitEvent(stream, ev_, flags_); }

CUresult CudaHostFuncCommand::Enqueue(CUstream stream) { return Driver().cuLaunchHostFunc(stream, fn_, data_); }

// ------------------------------------------------------------------------------------ xpk task
bool CudaXpkCommand::TaskCompleted() const {
    xpkTaskInfo info;
    if (xpkTaskQuery((xpkTask_t)task_, &info) != XPK_SUCCESS) return false;
    return info.status == XPK_STATUS_COMPLETED;
}

// Duration (launch -> wait returned) each task showed last time, so that the next wait for the same task
// can sleep through most of it.  Tasks are re-submitted in loops; a preempted run only makes the figure larger
// once, and the sleep is capped.
namespace {
std::mutex g_dur_mu;
std::unordered_map<void *, int64_t> g_last_duration_us;
int64_t SteadyNs() { return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
}

int64_t CudaXpkCommand::ExpectedRemainingUs() const {
    int64_t last = 0;
    {
        std::lock_guard<std::mutex> lk(g_dur_mu);
        auto it = g_last_duration_us.find(task_);
        if (it != g_last_duration_us.end()) last = it->second;
    }
    const int64_t at = launched_at_ns_.load(std::memory_order_relaxed);
    if (last == 0 || at == 0) return 0;
    return std::max<int64_t>(0, last - (SteadyNs() - at) / 1000);
}

void CudaXpkCommand::OnWaited() {
    const int64_t at = launched_at_ns_.load(std::memory_order_relaxed);
    if (at == 0) return;
    const int64_t us = (SteadyNs() - at) / 1000;
    std::lock_guard<std::mutex> lk(g_dur_mu);
    if (g_last_duration_us.size() > 4096) g_last_duration_us.clear();      // tasks come and go; keep the table small
    g_last_duration_us[task_] = us;
}

CUresult CudaXpkCommand::Enqueue(CUstream stream) {
    xpkTask_t t = (xpkTask_t)task_;
    launched_at_ns_.store(SteadyNs(), std::memory_order_relaxed);
    if (!launched_once_ && rewind_) {
        if (xpkTaskReset(t, stream) != XPK_SUCCESS) return CUDA_ERROR_LAUNCH_FAILED;
    }
    launched_once_ = true;
    return xpkTaskLaunch(t, stream, 0) == XPK_SUCCESS ? CUDA_SUCCESS : CUDA_ERROR_LAUNCH_FAILED;
}

} // namespace xsched::cuda
