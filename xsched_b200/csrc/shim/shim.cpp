// libshimcuda.so — transparent interposer for the CUDA driver library.  Installed under the names
// libcuda.so.1 / libcuda.so in a directory that is put first on LD_LIBRARY_PATH, it is what the CUDA
// runtime (and therefore any framework) loads as "the driver".  Calls that enqueue work on a stream that
// has an XQueue — cuLaunchKernel, cuMemcpy*Async, cuMemset*Async, cuEventRecord, cuStreamWaitEvent,
// cuLaunchHostFunc — become HwCommands submitted to that XQueue and return CUDA_SUCCESS at once;
// cuStreamSynchronize / cuEventSynchronize / cuEventQuery / cuStreamQuery / cuCtxSynchronize / cuMemFree
// wait on (or ask) the XQueue; cuStreamCreate* / cuStreamDestroy create and destroy XQueues when
// XSCHED_AUTO_XQUEUE=ON.  Every other driver entry point is forwarded untouched by a one-instruction
// trampoline generated from the function list of cuda.h (shim_exports.inc).
//
// Behaviour follows the reference's shim (platforms/cuda/shim/src/shim.cpp:25-567, shim.h:20-105,
// cuGetProcAddress override intercept.cpp:1108-1166): legacy-stream calls first drain XQueues of blocking
// streams and then go straight to the driver; while a stream capture is open everything goes straight to
// the driver.  Unlike the reference, the generic cuMemcpyAsync is routed too.  x86-64 only (trampolines).
//
// Per-thread default stream (programs built with --default-stream per-thread, or that pass CU_STREAM_PER_THREAD):
// every routed entry point has a `_ptsz` twin, and lookups with CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM get
// the twin.  CU_STREAM_PER_THREAD — and, in a twin, the NULL stream — is replaced by a private non-blocking stream
// of the calling thread (one per context), which gets its own XQueue like any created stream (reference:
// platforms/cuda/shim/src/shim.cpp:25-41, shim.h:20-62).  XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS=ON makes every
// cuStreamCreate* hand out one shared, reference-counted stream (reference: shim.cpp:472-567).
#include <atomic>
#include <cstdio>
#include <cstring>
#include <list>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <cuda.h>

#include "hal_cuda/cuda_command.h"
#include "hal_cuda/driver.h"
#include "xsched/cuda/hal.h"
#include "xsched/preempt/hal/hw_queue.h"
#include "xsched/preempt/xqueue/xqueue.h"
#include "xsched/protocol/def.h"
#include "xsched/utils/xassert.h"

using namespace xsched::cuda;
using namespace xsched::preempt;

// Marker looked for by the HAL's driver loader: a library exporting it is not the real driver.
extern "C" {
__attribute__((visibility("default"))) int XSchedShimMarker = 1;
}

namespace {

// ---- statistics (dumped as JSON to $XSCHED_SHIM_STATS_FILE at exit) ----
struct Stats {
    std::atomic<uint64_t> launches_queued{0}, launches_direct{0}, copies_queued{0}, copies_direct{0}, events_queued{0},
        syncs_via_xqueue{0}, streams_with_xqueue{0}, getproc_hooked{0}, copies_waited{0}, launches_blocking{0}, calls_queued{0}, graphs_queued{0},
        thread_streams{0}, getproc_hooked_ptsz{0}, single_stream_refs{0};
} g_stats;

void DumpStats() {
    const std::string path = GetEnv("XSCHED_SHIM_STATS_FILE");
    if (path.empty()) return;
    if (FILE *f = std::fopen(path.c_str(), "w")) {
        std::fprintf(f, "{\"launches_queued\": %llu, \"launches_direct\": %llu, \"copies_queued\": %llu, \"copies_direct\": %llu, "
                        "\"events_queued\": %llu, \"syncs_via_xqueue\": %llu, \"streams_with_xqueue\": %llu, \"getproc_hooked\": %llu, \"copies_waited\": %llu, \"launches_blocking\": %llu, \"calls_queued\": %llu, \"graphs_queued\": %llu, "
                        "\"thread_streams\": %llu, \"getproc_hooked_ptsz\": %llu, \"single_stream_refs\": %llu}\n",
                     (unsigned long long)g_stats.launches_queued, (unsigned long long)g_stats.launches_direct,
                     (unsigned long long)g_stats.copies_queued, (unsigned long long)g_stats.copies_direct,
                     (unsigned long long)g_stats.events_queued, (unsigned long long)g_stats.syncs_via_xqueue,
                     (unsigned long long)g_stats.streams_with_xqueue, (unsigned long long)g_stats.getproc_hooked,
                     (unsigned long long)g_stats.copies_waited, (unsigned long long)g_stats.launches_blocking,
                     (unsigned long long)g_stats.calls_queued, (unsigned long long)g_stats.graphs_queued,
                     (unsigned long long)g_stats.thread_streams, (unsigned long long)g_stats.getproc_hooked_ptsz,
                     (unsigned long long)g_stats.single_stream_refs);
        std::fclose(f);
    }
}

// ---- real entry points used by the handlers ----
template <class F> F Real(const char *name) {
    void *p = Driver().Sym(name);
    XASSERT(p != nullptr, "the CUDA driver lacks %s", name);
    return reinterpret_cast<F>(p);
}
#define REAL(fn, sym) static const auto real = Real<decltype(&fn)>(sym)

std::atomic<int64_t> g_capturing{0};

bool IsLegacy(CUstream s) { return s == nullptr || s == CU_STREAM_LEGACY; }

void AutoCreate(CUstream s);

// Set while a `_ptsz` twin runs on this thread: there the NULL stream means the per-thread default stream.
thread_local bool t_ptsz = false;
struct PtszScope {
    bool prev;
    PtszScope() : prev(t_ptsz) { t_ptsz = true; }
    ~PtszScope() { t_ptsz = prev; }
};

// The calling thread's private stand-in for the per-thread default stream in the current context.  Created on
// first use, non-blocking, with an XQueue when XSCHED_AUTO_XQUEUE is on.  Like the reference it lives until the
// process ends (a stream cannot be destroyed safely from a thread-exit hook once its context may be gone).
CUstream ThreadStream() {
    struct Entry { CUcontext ctx; CUstream stream; };
    thread_local std::vector<Entry> mine;
    CUcontext ctx = nullptr;
    if (Driver().cuCtxGetCurrent(&ctx) != CUDA_SUCCESS || ctx == nullptr) return CU_STREAM_PER_THREAD;    // let the driver report it
    for (const Entry &e : mine) if (e.ctx == ctx) return e.stream;
    CUstream st = nullptr;
    if (Driver().cuStreamCreateWithPriority(&st, CU_STREAM_NON_BLOCKING, 0) != CUDA_SUCCESS) return CU_STREAM_PER_THREAD;
    AutoCreate(st);
    mine.push_back(Entry{ctx, st});
    g_stats.thread_streams++;
    return st;
}

// Stream handle as the rest of a handler sees it: CU_STREAM_PER_THREAD (and NULL inside a _ptsz twin) becomes
// the thread's private stream; NULL elsewhere stays the legacy default stream.
CUstream Normalize(CUstream s) {
    if (s == CU_STREAM_PER_THREAD || (s == nullptr && t_ptsz)) return ThreadStream();
    return s;
}

// Work on the legacy default stream is ordered after everything on blocking streams: drain their XQueues.
void DrainBlockingStreams() {
    std::list<std::shared_ptr<XQueueWaitAllCommand>> markers;
    XQueueManager::ForEach([&](std::shared_ptr<XQueue> xq) -> XResult {
        unsigned flags = 0;
        CUstream s = (CUstream)(uintptr_t)xq->GetHwQueue()->GetHandle();
        if (Driver().cuStreamGetFlags(s, &flags) == CUDA_SUCCESS && (flags & CU_STREAM_NON_BLOCKING)) return kXSchedSuccess;
        if (auto m = xq->SubmitWaitAll()) markers.push_back(std::move(m));
        return kXSchedSuccess;
    });
    for (auto &m : markers) m->Wait();
}

// The XQueue to submit to, or nullptr when the call must go straight to the driver.
std::shared_ptr<XQueue> Route(CUstream s) {
    if (g_capturing.load(std::memory_order_relaxed) > 0) return nullptr;
    if (IsLegacy(s)) { DrainBlockingStreams(); return nullptr; }
    if (s == CU_STREAM_PER_THREAD) return nullptr;        // only when no private stream could be made
    return HwQueueManager::GetXQueue((HwQueueHandle)(uintptr_t)s);
}

std::mutex g_ev_mu;
std::unordered_map<CUevent, std::shared_ptr<CudaEventRecordCommand>> g_events;   // event -> its newest record command

std::shared_ptr<CudaEventRecordCommand> FindRecord(CUevent ev) {
    std::lock_guard<std::mutex> lk(g_ev_mu);
    auto it = g_events.find(ev);
    return it == g_events.end() ? nullptr : it->second;
}

void AutoCreate(CUstream s) {
    const XResult r = XQueueManager::AutoCreate([&](HwQueueHandle *hwq) { return CudaQueueCreate(hwq, s); });
    if (r == kXSchedSuccess && HwQueueManager::GetXQueue((HwQueueHandle)(uintptr_t)s)) g_stats.streams_with_xqueue++;
}

CUresult Unsupported() { return CUDA_ERROR_NOT_SUPPORTED; }

} // namespace

// ======================================================================================= handlers
extern "C" {
#define SHIM_API __attribute__((visibility("default")))

SHIM_API CUresult CUDAAPI cuLaunchKernel(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                                         unsigned shmem, CUstream s, void **params, void **extra) {
    s = Normalize(s);
    REAL(cuLaunchKernel, "cuLaunchKernel");
    auto xq = Route(s);
    if (xq) {
        auto cmd = std::make_shared<CudaKernelLaunchCommand>(f, gx, gy, gz, bx, by, bz, shmem, params, extra);
        xq->Submit(cmd);     // returns after the launch when the arguments had to be borrowed
        if (cmd->ParamsCopied()) g_stats.launches_queued++; else g_stats.launches_blocking++;
        return CUDA_SUCCESS;
    }
    g_stats.launches_direct++;
    return real(f, gx, gy, gz, bx, by, bz, shmem, s, params, extra);
}

SHIM_API CUresult CUDAAPI cuLaunchKernelEx(const CUlaunchConfig *config, CUfunction f, void **params, void **extra) {
    if (config == nullptr) return CUDA_ERROR_INVALID_VALUE;
    CUlaunchConfig normalized = *config;
    normalized.hStream = Normalize(config->hStream);
    config = &normalized;
    auto xq = Route(config->hStream);
    if (xq) {
        auto cmd = std::make_shared<CudaKernelLaunchCommand>(config, f, params, extra);
        xq->Submit(cmd);
        if (cmd->ParamsCopied()) g_stats.launches_queued++; else g_stats.launches_blocking++;
        return CUDA_SUCCESS;
    }
    g_stats.launches_direct++;
    return Driver().cuLaunchKernelEx(config, f, params, extra);
}

// The remaining stream-ordered entry points become closure commands.  `blocking` = the call returns only
// after the worker handed it to the driver (arguments borrowed from the caller, or a result the caller reads).
extern "C++" {
template <class F>
static bool SubmitCall(CUstream s, const char *what, F &&call, bool blocking = false) {
    auto xq = Route(s);
    if (!xq) return false;
    xq->Submit(std::make_shared<CudaCallCommand>(what, std::function<CUresult(CUstream)>(std::forward<F>(call)),
                                                 blocking ? kCommandPropertyBlockingSubmit : kCommandPropertyNone));
    g_stats.calls_queued++;
    return true;
}
} // extern "C++"

SHIM_API CUresult CUDAAPI cuLaunchCooperativeKernel(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                                                    unsigned shmem, CUstream s, void **params) {
    s = Normalize(s);
    REAL(cuLaunchCooperativeKernel, "cuLaunchCooperativeKernel");
    if (SubmitCall(s, "cooperative launch", [=](CUstream st) { return real(f, gx, gy, gz, bx, by, bz, shmem, st, params); }, /*blocking=*/true))
        return CUDA_SUCCESS;
    return real(f, gx, gy, gz, bx, by, bz, shmem, s, params);
}
SHIM_API CUresult CUDAAPI cuMemAllocAsync(CUdeviceptr *p, size_t n, CUstream s) {
    s = Normalize(s);
    REAL(cuMemAllocAsync, "cuMemAllocAsync");
    // Blocking: the address is read by the caller as soon as the call returns.
    auto res = std::make_shared<CUresult>(CUDA_SUCCESS);
    if (SubmitCall(s, "cuMemAllocAsync", [=](CUstream st) { *res = real(p, n, st); return CUDA_SUCCESS; }, /*blocking=*/true)) return *res;
    return real(p, n, s);
}
SHIM_API CUresult CUDAAPI cuMemFreeAsync(CUdeviceptr p, CUstream s) {
    s = Normalize(s);
    REAL(cuMemFreeAsync, "cuMemFreeAsync");
    if (SubmitCall(s, "cuMemFreeAsync", [=](CUstream st) { return real(p, st); })) return CUDA_SUCCESS;
    return real(p, s);
}
static bool PageableSide(CUmemorytype type, const void *host) {
    return type == CU_MEMORYTYPE_HOST && host != nullptr && IsPageableHost(host);
}
SHIM_API CUresult CUDAAPI cuMemcpy2DAsync(const CUDA_MEMCPY2D *c, CUstream s) {
    s = Normalize(s);
    REAL(cuMemcpy2DAsync, "cuMemcpy2DAsync_v2");
    if (c == nullptr) return CUDA_ERROR_INVALID_VALUE;
    auto xq = Route(s);
    if (!xq) return real(c, s);
    if (PageableSide(c->srcMemoryType, c->srcHost) || PageableSide(c->dstMemoryType, c->dstHost)) {
        xq->WaitAll();                       // pageable host memory: the call is synchronous for its caller anyway
        const CUresult r = real(c, s);
        return r != CUDA_SUCCESS ? r : Driver().cuStreamSynchronize(s);
    }
    const CUDA_MEMCPY2D copy = *c;
    SubmitCall(s, "cuMemcpy2DAsync", [=](CUstream st) { return real(&copy, st); });
    return CUDA_SUCCESS;
}
SHIM_API CUresult CUDAAPI cuMemcpy3DAsync(const CUDA_MEMCPY3D *c, CUstream s) {
    s = Normalize(s);
    REAL(cuMemcpy3DAsync, "cuMemcpy3DAsync_v2");
    if (c == nullptr) return CUDA_ERROR_INVALID_VALUE;
    auto xq = Route(s);
    if (!xq) return real(c, s);
    if (PageableSide(c->srcMemoryType, c->srcHost) || PageableSide(c->dstMemoryType, c->dstHost)) {
        xq->WaitAll();
        const CUresult r = real(c, s);
        return r != CUDA_SUCCESS ? r : Driver().cuStreamSynchronize(s);
    }
    const CUDA_MEMCPY3D copy = *c;
    SubmitCall(s, "cuMemcpy3DAsync", [=](CUstream st) { return real(&copy, st); });
    return CUDA_SUCCESS;
}
SHIM_API CUresult CUDAAPI cuMemcpyPeerAsync(CUdeviceptr d, CUcontext dc, CUdeviceptr sp, CUcontext sc, size_t n, CUstream s) {
    s = Normalize(s);
    REAL(cuMemcpyPeerAsync, "cuMemcpyPeerAsync");
    if (SubmitCall(s, "cuMemcpyPeerAsync", [=](CUstream st) { return real(d, dc, sp, sc, n, st); })) return CUDA_SUCCESS;
    return real(d, dc, sp, sc, n, s);
}
SHIM_API CUresult CUDAAPI cuMemsetD16Async(CUdeviceptr d, unsigned short v, size_t n, CUstream s) {
    s = Normalize(s);
    REAL(cuMemsetD16Async, "cuMemsetD16Async");
    if (SubmitCall(s, "cuMemsetD16Async", [=](CUstream st) { return real(d, v, n, st); })) return CUDA_SUCCESS;
    return real(d, v, n, s);
}
SHIM_API CUresult CUDAAPI cuMemsetD2D8Async(CUdeviceptr d, size_t pitch, unsigned char v, size_t w, size_t h, CUstream s) {
    s = Normalize(s);
    REAL(cuMemsetD2D8Async, "cuMemsetD2D8Async");
    if (SubmitCall(s, "cuMemsetD2D8Async", [=](CUstream st) { return real(d, pitch, v, w, h, st); })) return CUDA_SUCCESS;
    return real(d, pitch, v, w, h, s);
}
SHIM_API CUresult CUDAAPI cuMemsetD2D16Async(CUdeviceptr d, size_t pitch, unsigned short v, size_t w, size_t h, CUstream s) {
    s = Normalize(s);
    REAL(cuMemsetD2D16Async, "cuMemsetD2D16Async");
    if (SubmitCall(s, "cuMemsetD2D16Async", [=](CUstream st) { return real(d, pitch, v, w, h, st); })) return CUDA_SUCCESS;
    return real(d, pitch, v, w, h, s);
}
SHIM_API CUresult CUDAAPI cuMemsetD2D32Async(CUdeviceptr d, size_t pitch, unsigned v, size_t w, size_t h, CUstream s) {
    s = Normalize(s);
    REAL(cuMemsetD2D32Async, "cuMemsetD2D32Async");
    if (SubmitCall(s, "cuMemsetD2D32Async", [=](CUstream st) { return real(d, pitch, v, w, h, st); })) return CUDA_SUCCESS;
    return real(d, pitch, v, w, h, s);
}
// A graph launch is one command of the stream's XQueue: it takes part in the window, and the scheduler
// sees the queue as busy while the graph runs.
SHIM_API CUresult CUDAAPI cuGraphLaunch(CUgraphExec g, CUstream s) {
    s = Normalize(s);
    REAL(cuGraphLaunch, "cuGraphLaunch");
    if (SubmitCall(s, "cuGraphLaunch", [=](CUstream st) { return real(g, st); })) { g_stats.graphs_queued++; return CUDA_SUCCESS; }
    return real(g, s);
}
SHIM_API CUresult CUDAAPI cuGraphUpload(CUgraphExec g, CUstream s) {
    s = Normalize(s);
    REAL(cuGraphUpload, "cuGraphUpload");
    if (SubmitCall(s, "cuGraphUpload", [=](CUstream st) { return real(g, st); })) return CUDA_SUCCESS;
    return real(g, s);
}
SHIM_API CUresult CUDAAPI cuStreamAddCallback(CUstream s, CUstreamCallback cb, void *data, unsigned flags) {
    s = Normalize(s);
    REAL(cuStreamAddCallback, "cuStreamAddCallback");
    if (SubmitCall(s, "cuStreamAddCallback", [=](CUstream st) { return real(st, cb, data, flags); })) return CUDA_SUCCESS;
    return real(s, cb, data, flags);
}
// Synchronous copies imply the legacy stream: everything queued on blocking streams goes first.
SHIM_API CUresult CUDAAPI cuMemcpy(CUdeviceptr d, CUdeviceptr sp, size_t n) {
    REAL(cuMemcpy, "cuMemcpy");
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    return real(d, sp, n);
}
SHIM_API CUresult CUDAAPI cuMemcpyDtoH(void *d, CUdeviceptr sp, size_t n) {
    REAL(cuMemcpyDtoH, "cuMemcpyDtoH_v2");
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    return real(d, sp, n);
}
SHIM_API CUresult CUDAAPI cuMemcpyHtoD(CUdeviceptr d, const void *sp, size_t n) {
    REAL(cuMemcpyHtoD, "cuMemcpyHtoD_v2");
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    return real(d, sp, n);
}
SHIM_API CUresult CUDAAPI cuMemcpyDtoD(CUdeviceptr d, CUdeviceptr sp, size_t n) {
    REAL(cuMemcpyDtoD, "cuMemcpyDtoD_v2");
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    return real(d, sp, n);
}

static CUresult CopyCommon(CopyKind kind, CUdeviceptr dst, CUdeviceptr src, size_t n, CUstream s) {
    s = Normalize(s);
    auto xq = Route(s);
    if (xq) {
        // Pageable host memory makes the copy synchronous for its caller (the source may be reused, the
        // destination read, as soon as the call returns).  Sources are captured now unless they are
        // large; a pageable destination, or a large pageable source, waits for the copy.
        constexpr size_t kStageLimit = 32u << 20;
        const bool src_host = kind == CopyKind::kHtoD || kind == CopyKind::kGeneric;
        const bool dst_host = kind == CopyKind::kDtoH || kind == CopyKind::kGeneric;
        const bool src_pageable = src_host && IsPageableHost((const void *)(uintptr_t)src);
        const bool dst_pageable = dst_host && IsPageableHost((const void *)(uintptr_t)dst);
        const bool stage = src_pageable && n <= kStageLimit;
        auto cmd = std::make_shared<CudaMemcpyCommand>(kind, dst, src, n, stage);
        const bool wait = dst_pageable || (src_pageable && !stage);
        if (wait) cmd->EnableSynchronization();
        xq->Submit(cmd);
        if (wait) { xq->Wait(cmd); g_stats.copies_waited++; }
        g_stats.copies_queued++;
        return CUDA_SUCCESS;
    }
    g_stats.copies_direct++;
    const DriverApi &d = Driver();
    switch (kind) {
    case CopyKind::kHtoD: return d.cuMemcpyHtoDAsync(dst, (const void *)src, n, s);
    case CopyKind::kDtoH: return d.cuMemcpyDtoHAsync((void *)dst, src, n, s);
    case CopyKind::kDtoD: return d.cuMemcpyDtoDAsync(dst, src, n, s);
    default: return d.cuMemcpyAsync(dst, src, n, s);
    }
}
SHIM_API CUresult CUDAAPI cuMemcpyAsync(CUdeviceptr dst, CUdeviceptr src, size_t n, CUstream s) { return CopyCommon(CopyKind::kGeneric, dst, src, n, s); }
SHIM_API CUresult CUDAAPI cuMemcpyHtoDAsync(CUdeviceptr dst, const void *src, size_t n, CUstream s) { return CopyCommon(CopyKind::kHtoD, dst, (CUdeviceptr)(uintptr_t)src, n, s); }
SHIM_API CUresult CUDAAPI cuMemcpyDtoHAsync(void *dst, CUdeviceptr src, size_t n, CUstream s) { return CopyCommon(CopyKind::kDtoH, (CUdeviceptr)(uintptr_t)dst, src, n, s); }
SHIM_API CUresult CUDAAPI cuMemcpyDtoDAsync(CUdeviceptr dst, CUdeviceptr src, size_t n, CUstream s) { return CopyCommon(CopyKind::kDtoD, dst, src, n, s); }

SHIM_API CUresult CUDAAPI cuMemsetD8Async(CUdeviceptr dst, unsigned char v, size_t n, CUstream s) {
    s = Normalize(s);
    if (auto xq = Route(s)) { xq->Submit(std::make_shared<CudaMemsetCommand>(dst, v, n, 1)); return CUDA_SUCCESS; }
    return Driver().cuMemsetD8Async(dst, v, n, s);
}
SHIM_API CUresult CUDAAPI cuMemsetD32Async(CUdeviceptr dst, unsigned v, size_t n, CUstream s) {
    s = Normalize(s);
    if (auto xq = Route(s)) { xq->Submit(std::make_shared<CudaMemsetCommand>(dst, v, n, 4)); return CUDA_SUCCESS; }
    return Driver().cuMemsetD32Async(dst, v, n, s);
}

SHIM_API CUresult CUDAAPI cuLaunchHostFunc(CUstream s, CUhostFn fn, void *data) {
    s = Normalize(s);
    if (auto xq = Route(s)) { xq->Submit(std::make_shared<CudaHostFuncCommand>(fn, data)); return CUDA_SUCCESS; }
    return Driver().cuLaunchHostFunc(s, fn, data);
}

SHIM_API CUresult CUDAAPI cuEventRecord(CUevent ev, CUstream s) {
    s = Normalize(s);
    auto xq = Route(s);
    if (!xq) {
        { std::lock_guard<std::mutex> lk(g_ev_mu); g_events.erase(ev); }
        return Driver().cuEventRecord(ev, s);
    }
    auto cmd = std::make_shared<CudaEventRecordCommand>(ev);
    { std::lock_guard<std::mutex> lk(g_ev_mu); g_events[ev] = cmd; }
    xq->Submit(cmd);
    g_stats.events_queued++;
    return CUDA_SUCCESS;
}

SHIM_API CUresult CUDAAPI cuEventRecordWithFlags(CUevent ev, CUstream s, unsigned flags) {
    s = Normalize(s);
    REAL(cuEventRecordWithFlags, "cuEventRecordWithFlags");
    auto xq = Route(s);
    if (!xq) {
        { std::lock_guard<std::mutex> lk(g_ev_mu); g_events.erase(ev); }
        return real(ev, s, flags);
    }
    auto cmd = std::make_shared<CudaEventRecordCommand>(ev, flags, true);
    { std::lock_guard<std::mutex> lk(g_ev_mu); g_events[ev] = cmd; }
    xq->Submit(cmd);
    g_stats.events_queued++;
    return CUDA_SUCCESS;
}

SHIM_API CUresult CUDAAPI cuEventSynchronize(CUevent ev) {
    if (auto rec = FindRecord(ev)) { rec->Wait(); return CUDA_SUCCESS; }
    return Driver().cuEventSynchronize(ev);
}

SHIM_API CUresult CUDAAPI cuEventQuery(CUevent ev) {
    if (auto rec = FindRecord(ev)) {
        if (rec->GetState() >= kCommandStateCompleted) return CUDA_SUCCESS;
        if (rec->GetState() < kCommandStateInFlight) return CUDA_ERROR_NOT_READY;
    }
    return Driver().cuEventQuery(ev);
}

SHIM_API CUresult CUDAAPI cuEventDestroy(CUevent ev) {
    REAL(cuEventDestroy, "cuEventDestroy_v2");
    std::shared_ptr<CudaEventRecordCommand> rec;
    { std::lock_guard<std::mutex> lk(g_ev_mu); auto it = g_events.find(ev); if (it != g_events.end()) { rec = it->second; g_events.erase(it); } }
    if (rec) rec->WaitUntil(kCommandStateInFlight);     // the record must have reached the driver before the event goes away
    return real(ev);
}

SHIM_API CUresult CUDAAPI cuStreamWaitEvent(CUstream s, CUevent ev, unsigned flags) {
    s = Normalize(s);
    auto rec = FindRecord(ev);
    auto xq = Route(s);
    if (xq) {
        xq->Submit(std::make_shared<CudaEventWaitCommand>(ev, flags, rec));
        return CUDA_SUCCESS;
    }
    if (rec) rec->WaitUntil(kCommandStateInFlight);     // the record is still pending in another XQueue
    return Driver().cuStreamWaitEvent(s, ev, flags);
}

// The XQueue is waited for first (its commands may not have reached the driver yet), then the stream itself:
// stream-ordered calls that are not turned into commands (the generated trampolines) are only known to the
// driver.  (The reference stops after the XQueue, platforms/cuda/shim/src/shim.cpp:413-419.)
SHIM_API CUresult CUDAAPI cuStreamSynchronize(CUstream s) {
    s = Normalize(s);
    if (auto xq = Route(s)) {
        xq->WaitAll();
        g_stats.syncs_via_xqueue++;
    }
    return Driver().cuStreamSynchronize(s);
}

SHIM_API CUresult CUDAAPI cuStreamQuery(CUstream s) {
    s = Normalize(s);
    if (auto xq = Route(s)) {
        if (xq->Query() != kQueueStateIdle) return CUDA_ERROR_NOT_READY;
    }
    return Driver().cuStreamQuery(s);
}

SHIM_API CUresult CUDAAPI cuCtxSynchronize(void) {
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    return Driver().cuCtxSynchronize();
}

SHIM_API CUresult CUDAAPI cuMemFree(CUdeviceptr p) {
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();     // queued commands may still use the memory
    return Driver().cuMemFree(p);
}

// XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS=ON: every stream the program creates is the same stream (the first
// creation makes it, with that call's flags and priority; later ones add a reference), so the whole process is
// one XQueue and its work is serialised; the stream is destroyed with its last reference.
static std::mutex g_single_mu;
static CUstream g_single_stream = nullptr;
static int64_t g_single_refs = 0;
static bool SingleStreamMode() {
    static const bool on = GetEnvOption(XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS_ENV_NAME, false);
    return on;
}
extern "C++" {
template <class Create> static CUresult CreateStream(CUstream *s, Create &&create) {
    if (s == nullptr) return CUDA_ERROR_INVALID_VALUE;
    if (!SingleStreamMode()) {
        const CUresult r = create(s);
        if (r == CUDA_SUCCESS) AutoCreate(*s);
        return r;
    }
    std::lock_guard<std::mutex> lk(g_single_mu);
    if (g_single_refs == 0) {
        const CUresult r = create(&g_single_stream);
        if (r != CUDA_SUCCESS) return r;
        AutoCreate(g_single_stream);
    }
    ++g_single_refs;
    g_stats.single_stream_refs++;
    *s = g_single_stream;
    return CUDA_SUCCESS;
}
} // extern "C++"

SHIM_API CUresult CUDAAPI cuStreamCreate(CUstream *s, unsigned flags) {
    REAL(cuStreamCreate, "cuStreamCreate");
    return CreateStream(s, [&](CUstream *out) { return real(out, flags); });
}

SHIM_API CUresult CUDAAPI cuStreamCreateWithPriority(CUstream *s, unsigned flags, int prio) {
    return CreateStream(s, [&](CUstream *out) { return Driver().cuStreamCreateWithPriority(out, flags, prio); });
}

SHIM_API CUresult CUDAAPI cuStreamDestroy(CUstream s) {
    if (SingleStreamMode()) {
        std::lock_guard<std::mutex> lk(g_single_mu);
        if (s == g_single_stream && g_single_refs > 0) {
            if (--g_single_refs > 0) return CUDA_SUCCESS;
            g_single_stream = nullptr;
        }
    }
    if (HwQueueManager::GetXQueue((HwQueueHandle)(uintptr_t)s)) XQueueManager::AutoDestroy((HwQueueHandle)(uintptr_t)s);
    return Driver().cuStreamDestroy(s);
}

// Stream capture.  While any stream is being captured every entry point bypasses the XQueues (Route() returns
// nullptr): a command launched later by a worker thread would be recorded into the graph, and the completion
// write behind it would be as well.  Before the first capture starts, everything queued so far is drained, so
// that nothing submitted earlier runs inside the capture and direct launches cannot overtake queued ones.
// (The reference keeps the same counter, platforms/cuda/shim/src/shim.cpp:61-119.)
static std::mutex g_capture_mu;
static void CaptureBegins() {
    std::lock_guard<std::mutex> lk(g_capture_mu);
    if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();
    g_capturing.fetch_add(1);
}
static void CaptureEnded() {
    std::lock_guard<std::mutex> lk(g_capture_mu);
    if (g_capturing.load() > 0) g_capturing.fetch_sub(1);
}

SHIM_API CUresult CUDAAPI cuStreamBeginCapture(CUstream s, CUstreamCaptureMode mode) {
    s = Normalize(s);
    REAL(cuStreamBeginCapture, "cuStreamBeginCapture_v2");
    CaptureBegins();
    const CUresult r = real(s, mode);
    if (r != CUDA_SUCCESS) CaptureEnded();
    return r;
}

SHIM_API CUresult CUDAAPI cuStreamBeginCaptureToGraph(CUstream s, CUgraph g, const CUgraphNode *deps, const CUgraphEdgeData *dep_data, size_t n_deps,
                                                      CUstreamCaptureMode mode) {
    s = Normalize(s);
    REAL(cuStreamBeginCaptureToGraph, "cuStreamBeginCaptureToGraph");
    CaptureBegins();
    const CUresult r = real(s, g, deps, dep_data, n_deps, mode);
    if (r != CUDA_SUCCESS) CaptureEnded();
    return r;
}

// The counter goes down only when this call really ended a capture: ending on the wrong stream, or on one that
// was not capturing, leaves the capture (and the bypass) in place.
SHIM_API CUresult CUDAAPI cuStreamEndCapture(CUstream s, CUgraph *g) {
    s = Normalize(s);
    REAL(cuStreamEndCapture, "cuStreamEndCapture");
    using IsCapturingFn = CUresult (*)(CUstream, CUstreamCaptureStatus *);
    static const IsCapturingFn is_capturing = (IsCapturingFn)Driver().Sym("cuStreamIsCapturing");
    CUstreamCaptureStatus before = CU_STREAM_CAPTURE_STATUS_NONE, after = CU_STREAM_CAPTURE_STATUS_NONE;
    const bool known = is_capturing && is_capturing(s, &before) == CUDA_SUCCESS;
    const CUresult r = real(s, g);
    if (!known) { if (r == CUDA_SUCCESS) CaptureEnded(); return r; }
    if (before != CU_STREAM_CAPTURE_STATUS_NONE && r != CUDA_ERROR_STREAM_CAPTURE_UNMATCHED &&
        is_capturing(s, &after) == CUDA_SUCCESS && after == CU_STREAM_CAPTURE_STATUS_NONE)
        CaptureEnded();
    return r;
}


// ---- per-thread-default-stream twins --------------------------------------------------------------------
// Same handlers; while one runs, the NULL stream means "this thread's default stream" (Normalize()).  The
// synchronous copies (`_ptds`) are ordered after everything this process has queued, then go to the driver.
#define XSHIM_TWIN(call) { PtszScope in_twin; return call; }
SHIM_API CUresult CUDAAPI cuLaunchKernel_ptsz(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz, unsigned shmem,
                                              CUstream s, void **params, void **extra) XSHIM_TWIN(cuLaunchKernel(f, gx, gy, gz, bx, by, bz, shmem, s, params, extra))
SHIM_API CUresult CUDAAPI cuLaunchKernelEx_ptsz(const CUlaunchConfig *c, CUfunction f, void **params, void **extra) XSHIM_TWIN(cuLaunchKernelEx(c, f, params, extra))
SHIM_API CUresult CUDAAPI cuLaunchCooperativeKernel_ptsz(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz, unsigned shmem,
                                                         CUstream s, void **params) XSHIM_TWIN(cuLaunchCooperativeKernel(f, gx, gy, gz, bx, by, bz, shmem, s, params))
SHIM_API CUresult CUDAAPI cuLaunchHostFunc_ptsz(CUstream s, CUhostFn fn, void *data) XSHIM_TWIN(cuLaunchHostFunc(s, fn, data))
SHIM_API CUresult CUDAAPI cuMemAllocAsync_ptsz(CUdeviceptr *p, size_t n, CUstream s) XSHIM_TWIN(cuMemAllocAsync(p, n, s))
SHIM_API CUresult CUDAAPI cuMemFreeAsync_ptsz(CUdeviceptr p, CUstream s) XSHIM_TWIN(cuMemFreeAsync(p, s))
SHIM_API CUresult CUDAAPI cuMemcpyAsync_ptsz(CUdeviceptr d, CUdeviceptr sp, size_t n, CUstream s) XSHIM_TWIN(cuMemcpyAsync(d, sp, n, s))
SHIM_API CUresult CUDAAPI cuMemcpyHtoDAsync_v2_ptsz(CUdeviceptr d, const void *sp, size_t n, CUstream s) XSHIM_TWIN(cuMemcpyHtoDAsync(d, sp, n, s))
SHIM_API CUresult CUDAAPI cuMemcpyDtoHAsync_v2_ptsz(void *d, CUdeviceptr sp, size_t n, CUstream s) XSHIM_TWIN(cuMemcpyDtoHAsync(d, sp, n, s))
SHIM_API CUresult CUDAAPI cuMemcpyDtoDAsync_v2_ptsz(CUdeviceptr d, CUdeviceptr sp, size_t n, CUstream s) XSHIM_TWIN(cuMemcpyDtoDAsync(d, sp, n, s))
SHIM_API CUresult CUDAAPI cuMemcpy2DAsync_v2_ptsz(const CUDA_MEMCPY2D *c, CUstream s) XSHIM_TWIN(cuMemcpy2DAsync(c, s))
SHIM_API CUresult CUDAAPI cuMemcpy3DAsync_v2_ptsz(const CUDA_MEMCPY3D *c, CUstream s) XSHIM_TWIN(cuMemcpy3DAsync(c, s))
SHIM_API CUresult CUDAAPI cuMemcpyPeerAsync_ptsz(CUdeviceptr d, CUcontext dc, CUdeviceptr sp, CUcontext sc, size_t n, CUstream s) XSHIM_TWIN(cuMemcpyPeerAsync(d, dc, sp, sc, n, s))
SHIM_API CUresult CUDAAPI cuMemsetD8Async_ptsz(CUdeviceptr d, unsigned char v, size_t n, CUstream s) XSHIM_TWIN(cuMemsetD8Async(d, v, n, s))
SHIM_API CUresult CUDAAPI cuMemsetD16Async_ptsz(CUdeviceptr d, unsigned short v, size_t n, CUstream s) XSHIM_TWIN(cuMemsetD16Async(d, v, n, s))
SHIM_API CUresult CUDAAPI cuMemsetD32Async_ptsz(CUdeviceptr d, unsigned v, size_t n, CUstream s) XSHIM_TWIN(cuMemsetD32Async(d, v, n, s))
SHIM_API CUresult CUDAAPI cuMemsetD2D8Async_ptsz(CUdeviceptr d, size_t pitch, unsigned char v, size_t w, size_t h, CUstream s) XSHIM_TWIN(cuMemsetD2D8Async(d, pitch, v, w, h, s))
SHIM_API CUresult CUDAAPI cuMemsetD2D16Async_ptsz(CUdeviceptr d, size_t pitch, unsigned short v, size_t w, size_t h, CUstream s) XSHIM_TWIN(cuMemsetD2D16Async(d, pitch, v, w, h, s))
SHIM_API CUresult CUDAAPI cuMemsetD2D32Async_ptsz(CUdeviceptr d, size_t pitch, unsigned v, size_t w, size_t h, CUstream s) XSHIM_TWIN(cuMemsetD2D32Async(d, pitch, v, w, h, s))
SHIM_API CUresult CUDAAPI cuGraphLaunch_ptsz(CUgraphExec g, CUstream s) XSHIM_TWIN(cuGraphLaunch(g, s))
SHIM_API CUresult CUDAAPI cuGraphUpload_ptsz(CUgraphExec g, CUstream s) XSHIM_TWIN(cuGraphUpload(g, s))
SHIM_API CUresult CUDAAPI cuStreamAddCallback_ptsz(CUstream s, CUstreamCallback cb, void *data, unsigned flags) XSHIM_TWIN(cuStreamAddCallback(s, cb, data, flags))
SHIM_API CUresult CUDAAPI cuEventRecord_ptsz(CUevent ev, CUstream s) XSHIM_TWIN(cuEventRecord(ev, s))
SHIM_API CUresult CUDAAPI cuEventRecordWithFlags_ptsz(CUevent ev, CUstream s, unsigned flags) XSHIM_TWIN(cuEventRecordWithFlags(ev, s, flags))
SHIM_API CUresult CUDAAPI cuStreamWaitEvent_ptsz(CUstream s, CUevent ev, unsigned flags) XSHIM_TWIN(cuStreamWaitEvent(s, ev, flags))
SHIM_API CUresult CUDAAPI cuStreamSynchronize_ptsz(CUstream s) XSHIM_TWIN(cuStreamSynchronize(s))
SHIM_API CUresult CUDAAPI cuStreamQuery_ptsz(CUstream s) XSHIM_TWIN(cuStreamQuery(s))
SHIM_API CUresult CUDAAPI cuStreamBeginCapture_v2_ptsz(CUstream s, CUstreamCaptureMode mode) XSHIM_TWIN(cuStreamBeginCapture(s, mode))
SHIM_API CUresult CUDAAPI cuStreamBeginCaptureToGraph_ptsz(CUstream s, CUgraph g, const CUgraphNode *deps, const CUgraphEdgeData *dep_data, size_t n_deps,
                                                           CUstreamCaptureMode mode) XSHIM_TWIN(cuStreamBeginCaptureToGraph(s, g, deps, dep_data, n_deps, mode))
SHIM_API CUresult CUDAAPI cuStreamEndCapture_ptsz(CUstream s, CUgraph *g) XSHIM_TWIN(cuStreamEndCapture(s, g))
#undef XSHIM_TWIN
#define XSHIM_SYNC_COPY_PTDS(name, sym, params, args)                                              \
    SHIM_API CUresult CUDAAPI name params {                                                        \
        typedef CUresult(CUDAAPI * Fn) params;                                                     \
        static const Fn real = Real<Fn>(sym);                                                      \
        if (g_capturing.load() == 0) XQueueManager::ForEachWaitAll();                              \
        return real args;                                                                          \
    }
XSHIM_SYNC_COPY_PTDS(cuMemcpy_ptds, "cuMemcpy_ptds", (CUdeviceptr d, CUdeviceptr sp, size_t n), (d, sp, n))
XSHIM_SYNC_COPY_PTDS(cuMemcpyDtoH_v2_ptds, "cuMemcpyDtoH_v2_ptds", (void *d, CUdeviceptr sp, size_t n), (d, sp, n))
XSHIM_SYNC_COPY_PTDS(cuMemcpyHtoD_v2_ptds, "cuMemcpyHtoD_v2_ptds", (CUdeviceptr d, const void *sp, size_t n), (d, sp, n))
XSHIM_SYNC_COPY_PTDS(cuMemcpyDtoD_v2_ptds, "cuMemcpyDtoD_v2_ptds", (CUdeviceptr d, CUdeviceptr sp, size_t n), (d, sp, n))
#undef XSHIM_SYNC_COPY_PTDS

// ---- cuGetProcAddress: the CUDA runtime resolves everything through it ----
// `twin` answers lookups made with CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM (nullptr: the plain handler has no stream).
struct Hook { const char *name; void *fn; int min_version; void *twin; };
static const Hook kHooks[] = {
    {"cuLaunchKernel", (void *)&cuLaunchKernel, 4000, (void *)&cuLaunchKernel_ptsz},
    {"cuLaunchKernelEx", (void *)&cuLaunchKernelEx, 11060, (void *)&cuLaunchKernelEx_ptsz},
    {"cuLaunchCooperativeKernel", (void *)&cuLaunchCooperativeKernel, 9000, (void *)&cuLaunchCooperativeKernel_ptsz},
    {"cuMemAllocAsync", (void *)&cuMemAllocAsync, 11020, (void *)&cuMemAllocAsync_ptsz},
    {"cuMemFreeAsync", (void *)&cuMemFreeAsync, 11020, (void *)&cuMemFreeAsync_ptsz},
    {"cuMemcpy2DAsync", (void *)&cuMemcpy2DAsync, 3020, (void *)&cuMemcpy2DAsync_v2_ptsz},
    {"cuMemcpy3DAsync", (void *)&cuMemcpy3DAsync, 3020, (void *)&cuMemcpy3DAsync_v2_ptsz},
    {"cuMemsetD2D8Async", (void *)&cuMemsetD2D8Async, 3020, (void *)&cuMemsetD2D8Async_ptsz},
    {"cuMemsetD2D16Async", (void *)&cuMemsetD2D16Async, 3020, (void *)&cuMemsetD2D16Async_ptsz},
    {"cuMemsetD2D32Async", (void *)&cuMemsetD2D32Async, 3020, (void *)&cuMemsetD2D32Async_ptsz},
    {"cuGraphUpload", (void *)&cuGraphUpload, 11010, (void *)&cuGraphUpload_ptsz},
    {"cuEventRecordWithFlags", (void *)&cuEventRecordWithFlags, 11010, (void *)&cuEventRecordWithFlags_ptsz},
    {"cuMemcpyPeerAsync", (void *)&cuMemcpyPeerAsync, 4000, (void *)&cuMemcpyPeerAsync_ptsz},
    {"cuMemsetD16Async", (void *)&cuMemsetD16Async, 3020, (void *)&cuMemsetD16Async_ptsz},
    {"cuGraphLaunch", (void *)&cuGraphLaunch, 10000, (void *)&cuGraphLaunch_ptsz},
    {"cuStreamAddCallback", (void *)&cuStreamAddCallback, 5000, (void *)&cuStreamAddCallback_ptsz},
    {"cuMemcpy", (void *)&cuMemcpy, 4000, (void *)&cuMemcpy_ptds},
    {"cuMemcpyDtoH", (void *)&cuMemcpyDtoH, 3020, (void *)&cuMemcpyDtoH_v2_ptds},
    {"cuMemcpyHtoD", (void *)&cuMemcpyHtoD, 3020, (void *)&cuMemcpyHtoD_v2_ptds},
    {"cuMemcpyDtoD", (void *)&cuMemcpyDtoD, 3020, (void *)&cuMemcpyDtoD_v2_ptds},
    {"cuMemcpyAsync", (void *)&cuMemcpyAsync, 4000, (void *)&cuMemcpyAsync_ptsz},
    {"cuMemcpyHtoDAsync", (void *)&cuMemcpyHtoDAsync, 3020, (void *)&cuMemcpyHtoDAsync_v2_ptsz},
    {"cuMemcpyDtoHAsync", (void *)&cuMemcpyDtoHAsync, 3020, (void *)&cuMemcpyDtoHAsync_v2_ptsz},
    {"cuMemcpyDtoDAsync", (void *)&cuMemcpyDtoDAsync, 3020, (void *)&cuMemcpyDtoDAsync_v2_ptsz},
    {"cuMemsetD8Async", (void *)&cuMemsetD8Async, 3020, (void *)&cuMemsetD8Async_ptsz},
    {"cuMemsetD32Async", (void *)&cuMemsetD32Async, 3020, (void *)&cuMemsetD32Async_ptsz},
    {"cuLaunchHostFunc", (void *)&cuLaunchHostFunc, 10000, (void *)&cuLaunchHostFunc_ptsz},
    {"cuEventRecord", (void *)&cuEventRecord, 2000, (void *)&cuEventRecord_ptsz},
    {"cuEventSynchronize", (void *)&cuEventSynchronize, 2000, nullptr},
    {"cuEventQuery", (void *)&cuEventQuery, 2000, nullptr},
    {"cuEventDestroy", (void *)&cuEventDestroy, 4000, nullptr},
    {"cuStreamWaitEvent", (void *)&cuStreamWaitEvent, 3020, (void *)&cuStreamWaitEvent_ptsz},
    {"cuStreamSynchronize", (void *)&cuStreamSynchronize, 2000, (void *)&cuStreamSynchronize_ptsz},
    {"cuStreamQuery", (void *)&cuStreamQuery, 2000, (void *)&cuStreamQuery_ptsz},
    {"cuCtxSynchronize", (void *)&cuCtxSynchronize, 2000, nullptr},
    {"cuMemFree", (void *)&cuMemFree, 3020, nullptr},
    {"cuStreamCreate", (void *)&cuStreamCreate, 2000, nullptr},
    {"cuStreamCreateWithPriority", (void *)&cuStreamCreateWithPriority, 5050, nullptr},
    {"cuStreamDestroy", (void *)&cuStreamDestroy, 4000, nullptr},
    {"cuStreamBeginCapture", (void *)&cuStreamBeginCapture, 10010, (void *)&cuStreamBeginCapture_v2_ptsz},
    {"cuStreamBeginCaptureToGraph", (void *)&cuStreamBeginCaptureToGraph, 12030, (void *)&cuStreamBeginCaptureToGraph_ptsz},
    {"cuStreamEndCapture", (void *)&cuStreamEndCapture, 10000, (void *)&cuStreamEndCapture_ptsz},
};

static void *FindHook(const char *symbol, int version, cuuint64_t flags);

SHIM_API CUresult CUDAAPI cuGetProcAddress(const char *symbol, void **pfn, int version, cuuint64_t flags, CUdriverProcAddressQueryResult *status) {
    REAL(cuGetProcAddress, "cuGetProcAddress_v2");
    const CUresult r = real(symbol, pfn, version, flags, status);
    if (r != CUDA_SUCCESS || pfn == nullptr || *pfn == nullptr || symbol == nullptr) return r;
    if (void *h = FindHook(symbol, version, flags)) { *pfn = h; g_stats.getproc_hooked++; }
    return r;
}

#undef cuGetProcAddress
SHIM_API CUresult CUDAAPI cuGetProcAddress(const char *symbol, void **pfn, int version, cuuint64_t flags) {
    typedef CUresult(CUDAAPI * Fn)(const char *, void **, int, cuuint64_t);
    static const Fn real = Real<Fn>("cuGetProcAddress");
    const CUresult r = real(symbol, pfn, version, flags);
    if (r != CUDA_SUCCESS || pfn == nullptr || *pfn == nullptr || symbol == nullptr) return r;
    if (void *h = FindHook(symbol, version, flags)) { *pfn = h; g_stats.getproc_hooked++; }
    return r;
}

static void *FindHook(const char *symbol, int version, cuuint64_t flags) {
    const bool per_thread = (flags & CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM) != 0;
    if (std::strcmp(symbol, "cuGetProcAddress") == 0) {
        extern CUresult CUDAAPI cuGetProcAddress_v2(const char *, void **, int, cuuint64_t, CUdriverProcAddressQueryResult *);
        return version >= 12000 ? (void *)&cuGetProcAddress_v2 : (void *)&cuGetProcAddress;
    }
    for (const Hook &h : kHooks) {
        if (std::strcmp(symbol, h.name) != 0) continue;
        if (version < h.min_version) return nullptr;
        if (per_thread && h.twin) { g_stats.getproc_hooked_ptsz++; return h.twin; }
        return h.fn;       // entry points without a stream argument are the same in both modes
    }
    return nullptr;
}

} // extern "C"

// ======================================================================================= forwarders
// One pointer + one `jmp *pointer(%rip)` per driver entry point that is not handled above.
#define XSHIM_FWD(name)                                                                  \
    extern "C" { __attribute__((visibility("hidden"))) void *xshim_ptr_##name = nullptr; } \
    asm(".text\n.globl " #name "\n.type " #name ", @function\n" #name ":\n\tjmp *xshim_ptr_" #name "(%rip)\n.size " #name ", .-" #name "\n");
#include "shim_exports.inc"
#undef XSHIM_FWD

namespace {
struct FwdEntry { const char *name; void **slot; };
#define XSHIM_FWD(name) {#name, &xshim_ptr_##name},
const FwdEntry kForwarders[] = {
#include "shim_exports.inc"
};
#undef XSHIM_FWD

struct Init {
    Init() {
        const DriverApi &d = Driver();
        for (const FwdEntry &e : kForwarders) {
            void *p = d.Sym(e.name);
            *e.slot = p ? p : (void *)&Unsupported;
        }
        std::atexit(DumpStats);
    }
} g_init __attribute__((init_priority(200)));
} // namespace
