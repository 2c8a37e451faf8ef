// libcuda_fake.so — TEST INFRASTRUCTURE: a host-only stand-in for the CUDA driver, just faithful enough to run
// the CUDA HAL and the libcuda interposer of this repository on a machine without a GPU.
//
//   * a stream is a FIFO served by its own thread: work is asynchronous to the caller and ordered per stream;
//   * "device memory" is host memory the fake remembers; memory from cuMemHostAlloc is remembered as pinned;
//   * a CUfunction is a FakeFunction registered through fakeRegisterFunction(): a host function plus the sizes
//     of its parameters (what cuFuncGetParamInfo reports).  A launch copies the arguments at call time, as the
//     real driver does, and runs the host function on the stream's thread;
//   * copies that involve memory the fake does not know ("pageable") are synchronous for the caller, like
//     the real driver's: a pageable source is read before the call returns, a pageable destination is
//     written before it returns;
//   * events, cross-stream waits, host functions, 32/64-bit stream memory writes, memsets;
//   * stream capture into a graph (the recorded closures) and graph launches.
// Only the entry points the HAL loads and the test programs call exist.  Nothing here is shipped.
#include <cuda.h>

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <thread>
#include <vector>
#include <dlfcn.h>

namespace {

struct FakeFunction {
    void (*fn)(void **params, unsigned grid_x, unsigned block_x);
    std::vector<size_t> sizes;
    std::vector<size_t> offsets;
    size_t total = 0;
};

struct Stream {
    unsigned flags = 0;
    int priority = 0;
    std::mutex mu;
    std::condition_variable cv, idle_cv;
    std::deque<std::function<void()>> q;
    bool busy = false, stop = false;
    std::thread th;
    Stream() {
        th = std::thread([this] {
            std::unique_lock<std::mutex> lk(mu);
            while (true) {
                cv.wait(lk, [this] { return stop || !q.empty(); });
                if (q.empty()) return;
                auto f = std::move(q.front());
                q.pop_front();
                busy = true;
                lk.unlock();
                f();
                lk.lock();
                busy = false;
                if (q.empty()) idle_cv.notify_all();
            }
        });
    }
    ~Stream() {
        { std::lock_guard<std::mutex> lk(mu); stop = true; }
        cv.notify_all();
        if (th.joinable()) th.join();
    }
    // While a stream is capturing, work given to it is recorded instead of run.
    std::shared_ptr<std::vector<std::function<void()>>> capture;
    void Push(std::function<void()> f) {
        {
            std::lock_guard<std::mutex> lk(mu);
            if (capture) { capture->push_back(std::move(f)); return; }
            q.push_back(std::move(f));
        }
        cv.notify_one();
    }
    void Drain() {
        std::unique_lock<std::mutex> lk(mu);
        idle_cv.wait(lk, [this] { return q.empty() && !busy; });
    }
    bool Idle() {
        std::lock_guard<std::mutex> lk(mu);
        return q.empty() && !busy;
    }
};

struct Event {
    std::mutex mu;
    std::condition_variable cv;
    uint64_t recorded = 0, completed = 0;
};

struct State {
    std::mutex mu;
    std::map<const void *, std::pair<size_t, int>> mem;      // base -> (size, type: 1 pinned host, 2 device)
    std::set<Stream *> streams;
    Stream legacy;
    int ctx_token = 0;                                         // its address is "the context"
    std::atomic<uint64_t> launches{0}, copies{0}, writes{0};
};
State &S() { static State *s = new State(); return *s; }      // leaked on purpose: streams may outlive static destruction

thread_local std::vector<CUcontext> t_ctx_stack;
thread_local CUcontext t_ctx = nullptr;
CUcontext TheContext() { return (CUcontext)&S().ctx_token; }

// 0 = unknown to the fake (pageable host memory), 1 = pinned host, 2 = device
int TypeOf(const void *p) {
    std::lock_guard<std::mutex> lk(S().mu);
    auto it = S().mem.upper_bound(p);
    if (it == S().mem.begin()) return 0;
    --it;
    const char *base = (const char *)it->first;
    return ((const char *)p < base + it->second.first) ? it->second.second : 0;
}

// Legacy-default-stream rule, simplified to the strict side: work for the legacy stream is accepted only after
// everything already given to blocking streams (created without CU_STREAM_NON_BLOCKING) has finished, and work
// for a blocking stream only after the legacy stream has drained.
// Set while a `_ptsz` entry point runs: there NULL names the calling thread's default stream.
thread_local bool t_null_is_per_thread = false;
std::atomic<uint64_t> g_per_thread_stream_ops{0};          // operations the fake itself resolved to a per-thread default stream
Stream *PerThreadStream();

Stream *Of(CUstream s) {
    if (s == CU_STREAM_PER_THREAD || (s == nullptr && t_null_is_per_thread)) { g_per_thread_stream_ops++; return PerThreadStream(); }
    if (s == nullptr || s == CU_STREAM_LEGACY) {
        std::vector<Stream *> blocking;
        { std::lock_guard<std::mutex> lk(S().mu); for (Stream *x : S().streams) if (!(x->flags & CU_STREAM_NON_BLOCKING)) blocking.push_back(x); }
        for (Stream *x : blocking) x->Drain();
        return &S().legacy;
    }
    Stream *st = (Stream *)s;
    if (!(st->flags & CU_STREAM_NON_BLOCKING)) S().legacy.Drain();
    return st;
}

CUresult CopyAsync(void *dst, const void *src, size_t n, CUstream s) {
    S().copies++;
    const int ts = TypeOf(src), td = TypeOf(dst);
    Stream *st = Of(s);
    if (ts == 0 && td != 0) {                        // pageable source: read now
        auto staged = std::make_shared<std::vector<unsigned char>>((const unsigned char *)src, (const unsigned char *)src + n);
        st->Push([=] { std::memcpy(dst, staged->data(), n); });
        return CUDA_SUCCESS;
    }
    st->Push([=] { std::memcpy(dst, src, n); });
    if (td == 0) st->Drain();                        // pageable destination: written before the call returns
    return CUDA_SUCCESS;
}

} // namespace

extern "C" {

// ---- test hooks (not part of CUDA) ----
__attribute__((visibility("default"))) CUfunction fakeRegisterFunction(void (*fn)(void **, unsigned, unsigned), const size_t *sizes, int count) {
    auto *f = new FakeFunction();
    f->fn = fn;
    size_t off = 0;
    for (int i = 0; i < count; ++i) {
        const size_t align = sizes[i] >= 8 ? 8 : (sizes[i] >= 4 ? 4 : 1);
        off = (off + align - 1) / align * align;
        f->sizes.push_back(sizes[i]);
        f->offsets.push_back(off);
        off += sizes[i];
    }
    f->total = off;
    return (CUfunction)f;
}
__attribute__((visibility("default"))) void fakeCounters(uint64_t *launches, uint64_t *copies, uint64_t *writes) {
    if (launches) *launches = S().launches.load();
    if (copies) *copies = S().copies.load();
    if (writes) *writes = S().writes.load();
}

#define API __attribute__((visibility("default"))) CUresult CUDAAPI

API cuInit(unsigned) { return CUDA_SUCCESS; }
API cuDriverGetVersion(int *v) { *v = 12090; return CUDA_SUCCESS; }
API cuGetErrorString(CUresult r, const char **s) { *s = r == CUDA_SUCCESS ? "no error" : "fake driver error"; return CUDA_SUCCESS; }
API cuGetErrorName(CUresult r, const char **s) { *s = r == CUDA_SUCCESS ? "CUDA_SUCCESS" : "CUDA_ERROR_FAKE"; return CUDA_SUCCESS; }
API cuDeviceGetCount(int *n) { *n = 1; return CUDA_SUCCESS; }
API cuDeviceGet(CUdevice *d, int ordinal) { if (ordinal != 0) return CUDA_ERROR_INVALID_DEVICE; *d = 0; return CUDA_SUCCESS; }
API cuDeviceGetAttribute(int *v, CUdevice_attribute a, CUdevice) {
    switch (a) {
    case CU_DEVICE_ATTRIBUTE_PCI_BUS_ID: *v = 0x1b; break;
    case CU_DEVICE_ATTRIBUTE_PCI_DEVICE_ID: *v = 0; break;
    case CU_DEVICE_ATTRIBUTE_PCI_DOMAIN_ID: *v = 0; break;
    case CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT: *v = 4; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *v = 10; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *v = 0; break;
    default: *v = 0; break;
    }
    return CUDA_SUCCESS;
}
API cuDevicePrimaryCtxRetain(CUcontext *c, CUdevice) { *c = TheContext(); return CUDA_SUCCESS; }
API cuDevicePrimaryCtxRelease(CUdevice) { return CUDA_SUCCESS; }
API cuCtxGetCurrent(CUcontext *c) { *c = t_ctx; return CUDA_SUCCESS; }
API cuCtxSetCurrent(CUcontext c) { t_ctx = c; return CUDA_SUCCESS; }
API cuCtxPushCurrent(CUcontext c) { t_ctx_stack.push_back(t_ctx); t_ctx = c; return CUDA_SUCCESS; }
API cuCtxPopCurrent(CUcontext *c) {
    if (c) *c = t_ctx;
    if (t_ctx_stack.empty()) { t_ctx = nullptr; return CUDA_SUCCESS; }
    t_ctx = t_ctx_stack.back();
    t_ctx_stack.pop_back();
    return CUDA_SUCCESS;
}
API cuCtxGetDevice(CUdevice *d) { *d = 0; return t_ctx ? CUDA_SUCCESS : CUDA_ERROR_INVALID_CONTEXT; }
API cuCtxGetStreamPriorityRange(int *lo, int *hi) { if (lo) *lo = 0; if (hi) *hi = -5; return CUDA_SUCCESS; }
API cuCtxSynchronize(void) {
    std::vector<Stream *> all;
    { std::lock_guard<std::mutex> lk(S().mu); all.assign(S().streams.begin(), S().streams.end()); }
    for (Stream *s : all) s->Drain();
    S().legacy.Drain();
    return CUDA_SUCCESS;
}

// ---- streams ----
// (entry points never call one another through their exported names: under an interposer such a call
// would bind to the interposer's export of the same name)
static CUresult NewStream(CUstream *out, unsigned flags, int prio) {
    auto *s = new Stream();
    s->flags = flags; s->priority = prio;
    { std::lock_guard<std::mutex> lk(S().mu); S().streams.insert(s); }
    *out = (CUstream)s;
    return CUDA_SUCCESS;
}
} // extern "C"
namespace {
// The per-thread default stream of the real driver behaves like a non-blocking stream owned by the thread.
Stream *PerThreadStream() {
    thread_local Stream *mine = nullptr;
    if (!mine) { CUstream h = nullptr; NewStream(&h, CU_STREAM_NON_BLOCKING, 0); mine = (Stream *)h; }
    return mine;
}
} // namespace
extern "C" {
API cuStreamCreateWithPriority(CUstream *out, unsigned flags, int prio) { return NewStream(out, flags, prio); }
API cuStreamCreate(CUstream *out, unsigned flags) { return NewStream(out, flags, 0); }
API cuStreamDestroy(CUstream s) {
    Stream *st = (Stream *)s;
    { std::lock_guard<std::mutex> lk(S().mu); if (!S().streams.erase(st)) return CUDA_ERROR_INVALID_HANDLE; }
    st->Drain();
    delete st;
    return CUDA_SUCCESS;
}
API cuStreamGetCtx(CUstream, CUcontext *c) { *c = TheContext(); return CUDA_SUCCESS; }
API cuStreamGetFlags(CUstream s, unsigned *f) { *f = Of(s)->flags; return CUDA_SUCCESS; }
API cuStreamSynchronize(CUstream s) { Of(s)->Drain(); return CUDA_SUCCESS; }
API cuStreamQuery(CUstream s) { return Of(s)->Idle() ? CUDA_SUCCESS : CUDA_ERROR_NOT_READY; }
API cuStreamWriteValue32(CUstream s, CUdeviceptr addr, cuuint32_t v, unsigned) {
    S().writes++;
    Of(s)->Push([=] { __atomic_store_n((volatile uint32_t *)(uintptr_t)addr, v, __ATOMIC_RELEASE); });
    return CUDA_SUCCESS;
}
API cuStreamWriteValue64(CUstream s, CUdeviceptr addr, cuuint64_t v, unsigned) {
    S().writes++;
    Of(s)->Push([=] { __atomic_store_n((volatile uint64_t *)(uintptr_t)addr, v, __ATOMIC_RELEASE); });
    return CUDA_SUCCESS;
}
API cuLaunchHostFunc(CUstream s, CUhostFn fn, void *data) { Of(s)->Push([=] { fn(data); }); return CUDA_SUCCESS; }

// ---- events ----
// A CUevent is a heap-allocated shared_ptr: queued work keeps the event alive after cuEventDestroy, as the
// real driver does for an event destroyed while a record or a wait on it is pending.
using EventRef = std::shared_ptr<Event>;
static EventRef Ev(CUevent e) { return *(EventRef *)e; }
API cuEventCreate(CUevent *e, unsigned) { *e = (CUevent) new EventRef(std::make_shared<Event>()); return CUDA_SUCCESS; }
API cuEventDestroy(CUevent e) { delete (EventRef *)e; return CUDA_SUCCESS; }
static CUresult Record(CUevent e, CUstream s) {
    EventRef ev = Ev(e);
    uint64_t seq;
    { std::lock_guard<std::mutex> lk(ev->mu); seq = ++ev->recorded; }
    Of(s)->Push([=] {
        { std::lock_guard<std::mutex> lk(ev->mu); if (ev->completed < seq) ev->completed = seq; }
        ev->cv.notify_all();
    });
    return CUDA_SUCCESS;
}
API cuEventRecord(CUevent e, CUstream s) { return Record(e, s); }
API cuEventRecordWithFlags(CUevent e, CUstream s, unsigned) { return Record(e, s); }
API cuEventQuery(CUevent e) {
    EventRef ev = Ev(e);
    std::lock_guard<std::mutex> lk(ev->mu);
    return ev->completed >= ev->recorded ? CUDA_SUCCESS : CUDA_ERROR_NOT_READY;
}
API cuEventSynchronize(CUevent e) {
    EventRef ev = Ev(e);
    std::unique_lock<std::mutex> lk(ev->mu);
    const uint64_t target = ev->recorded;
    ev->cv.wait(lk, [&] { return ev->completed >= target; });
    return CUDA_SUCCESS;
}
API cuStreamWaitEvent(CUstream s, CUevent e, unsigned) {
    EventRef ev = Ev(e);
    uint64_t target;
    { std::lock_guard<std::mutex> lk(ev->mu); target = ev->recorded; }
    Of(s)->Push([=] {
        std::unique_lock<std::mutex> lk(ev->mu);
        ev->cv.wait(lk, [&] { return ev->completed >= target; });
    });
    return CUDA_SUCCESS;
}

// ---- memory ----
API cuMemAlloc(CUdeviceptr *p, size_t n) {
    void *m = std::calloc(1, n ? n : 1);
    { std::lock_guard<std::mutex> lk(S().mu); S().mem[m] = {n, 2}; }
    *p = (CUdeviceptr)(uintptr_t)m;
    return CUDA_SUCCESS;
}
API cuMemFree(CUdeviceptr p) {
    void *m = (void *)(uintptr_t)p;
    { std::lock_guard<std::mutex> lk(S().mu); if (!S().mem.erase(m)) return CUDA_ERROR_INVALID_VALUE; }
    std::free(m);
    return CUDA_SUCCESS;
}
static CUresult HostAlloc(void **p, size_t n) {
    void *m = nullptr;
    if (posix_memalign(&m, 64, n ? n : 64) != 0) return CUDA_ERROR_OUT_OF_MEMORY;
    std::memset(m, 0, n);
    { std::lock_guard<std::mutex> lk(S().mu); S().mem[m] = {n, 1}; }
    *p = m;
    return CUDA_SUCCESS;
}
API cuMemHostAlloc(void **p, size_t n, unsigned) { return HostAlloc(p, n); }
API cuMemAllocHost(void **p, size_t n) { return HostAlloc(p, n); }
API cuMemFreeHost(void *p) {
    { std::lock_guard<std::mutex> lk(S().mu); if (!S().mem.erase(p)) return CUDA_ERROR_INVALID_VALUE; }
    std::free(p);
    return CUDA_SUCCESS;
}
API cuMemHostGetDevicePointer(CUdeviceptr *d, void *h, unsigned) { *d = (CUdeviceptr)(uintptr_t)h; return CUDA_SUCCESS; }
API cuPointerGetAttribute(void *data, CUpointer_attribute attr, CUdeviceptr p) {
    const int t = TypeOf((const void *)(uintptr_t)p);
    if (t == 0) return CUDA_ERROR_INVALID_VALUE;
    if (attr == CU_POINTER_ATTRIBUTE_MEMORY_TYPE) { *(unsigned *)data = t == 2 ? CU_MEMORYTYPE_DEVICE : CU_MEMORYTYPE_HOST; return CUDA_SUCCESS; }
    return CUDA_ERROR_NOT_SUPPORTED;
}
API cuMemsetD32(CUdeviceptr d, unsigned v, size_t n) { for (size_t i = 0; i < n; ++i) ((unsigned *)(uintptr_t)d)[i] = v; return CUDA_SUCCESS; }
API cuMemsetD8Async(CUdeviceptr d, unsigned char v, size_t n, CUstream s) { Of(s)->Push([=] { std::memset((void *)(uintptr_t)d, v, n); }); return CUDA_SUCCESS; }
API cuMemsetD32Async(CUdeviceptr d, unsigned v, size_t n, CUstream s) {
    Of(s)->Push([=] { for (size_t i = 0; i < n; ++i) ((unsigned *)(uintptr_t)d)[i] = v; });
    return CUDA_SUCCESS;
}
API cuMemcpyAsync(CUdeviceptr d, CUdeviceptr s_, size_t n, CUstream s) { return CopyAsync((void *)(uintptr_t)d, (const void *)(uintptr_t)s_, n, s); }
API cuMemcpyHtoDAsync(CUdeviceptr d, const void *h, size_t n, CUstream s) { return CopyAsync((void *)(uintptr_t)d, h, n, s); }
API cuMemcpyDtoHAsync(void *h, CUdeviceptr d, size_t n, CUstream s) { return CopyAsync(h, (const void *)(uintptr_t)d, n, s); }
API cuMemcpyDtoDAsync(CUdeviceptr d, CUdeviceptr s_, size_t n, CUstream s) { return CopyAsync((void *)(uintptr_t)d, (const void *)(uintptr_t)s_, n, s); }

// ---- launches ----
API cuFuncGetParamInfo(CUfunction f, size_t i, size_t *off, size_t *size) {
    auto *ff = (FakeFunction *)f;
    if (i >= ff->sizes.size()) return CUDA_ERROR_INVALID_VALUE;
    if (off) *off = ff->offsets[i];
    if (size) *size = ff->sizes[i];
    return CUDA_SUCCESS;
}
static CUresult Launch(CUfunction f, unsigned gx, unsigned bx, CUstream s, void **params) {
    auto *ff = (FakeFunction *)f;
    S().launches++;
    // arguments are read at launch time
    auto bytes = std::make_shared<std::vector<unsigned char>>(ff->total);
    for (size_t i = 0; i < ff->sizes.size(); ++i) std::memcpy(bytes->data() + ff->offsets[i], params[i], ff->sizes[i]);
    Of(s)->Push([=] {
        std::vector<void *> ptrs(ff->sizes.size());
        for (size_t i = 0; i < ptrs.size(); ++i) ptrs[i] = bytes->data() + ff->offsets[i];
        ff->fn(ptrs.data(), gx, bx);
    });
    return CUDA_SUCCESS;
}
API cuLaunchKernel(CUfunction f, unsigned gx, unsigned, unsigned, unsigned bx, unsigned, unsigned, unsigned, CUstream s, void **params, void **) {
    return Launch(f, gx, bx, s, params);
}
API cuLaunchKernelEx(const CUlaunchConfig *c, CUfunction f, void **params, void **) { return Launch(f, c->gridDimX, c->blockDimX, c->hStream, params); }

// ---- stream capture and graphs: a graph is the list of closures recorded while the stream was capturing ----
using Recorded = std::vector<std::function<void()>>;
API cuStreamBeginCapture(CUstream s, CUstreamCaptureMode) {
    Stream *st = (Stream *)s;
    std::lock_guard<std::mutex> lk(st->mu);
    if (st->capture) return CUDA_ERROR_ILLEGAL_STATE;
    st->capture = std::make_shared<Recorded>();
    return CUDA_SUCCESS;
}
API cuStreamIsCapturing(CUstream s, CUstreamCaptureStatus *status) {
    Stream *st = (s == nullptr || s == CU_STREAM_LEGACY || s == CU_STREAM_PER_THREAD) ? &S().legacy : (Stream *)s;
    std::lock_guard<std::mutex> lk(st->mu);
    *status = st->capture ? CU_STREAM_CAPTURE_STATUS_ACTIVE : CU_STREAM_CAPTURE_STATUS_NONE;
    return CUDA_SUCCESS;
}
API cuStreamEndCapture(CUstream s, CUgraph *g) {
    Stream *st = (Stream *)s;
    std::lock_guard<std::mutex> lk(st->mu);
    if (!st->capture) return CUDA_ERROR_STREAM_CAPTURE_UNMATCHED;
    *g = (CUgraph) new std::shared_ptr<Recorded>(st->capture);
    st->capture.reset();
    return CUDA_SUCCESS;
}
API cuGraphInstantiate(CUgraphExec *exec, CUgraph g, unsigned long long) {
    *exec = (CUgraphExec) new std::shared_ptr<Recorded>(*(std::shared_ptr<Recorded> *)g);
    return CUDA_SUCCESS;
}
API cuGraphUpload(CUgraphExec, CUstream) { return CUDA_SUCCESS; }
API cuGraphLaunch(CUgraphExec exec, CUstream s) {
    std::shared_ptr<Recorded> rec = *(std::shared_ptr<Recorded> *)exec;
    Stream *st = Of(s);
    for (const auto &f : *rec) st->Push(f);
    return CUDA_SUCCESS;
}
API cuGraphExecDestroy(CUgraphExec exec) { delete (std::shared_ptr<Recorded> *)exec; return CUDA_SUCCESS; }
API cuGraphDestroy(CUgraph g) { delete (std::shared_ptr<Recorded> *)g; return CUDA_SUCCESS; }

// ---- symbol lookup ----
// A few per-thread-default-stream twins, enough for the interposer tests (launch, copies, memset, event, sync).
struct NullIsPerThread { bool prev; NullIsPerThread() : prev(t_null_is_per_thread) { t_null_is_per_thread = true; } ~NullIsPerThread() { t_null_is_per_thread = prev; } };
API cuLaunchKernel_ptsz(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz, unsigned sh, CUstream s, void **p, void **e) {
    NullIsPerThread scope; return cuLaunchKernel(f, gx, gy, gz, bx, by, bz, sh, s, p, e);
}
API cuMemcpyHtoDAsync_v2_ptsz(CUdeviceptr d, const void *h, size_t n, CUstream s) { NullIsPerThread scope; return cuMemcpyHtoDAsync(d, h, n, s); }
API cuMemcpyDtoHAsync_v2_ptsz(void *h, CUdeviceptr d, size_t n, CUstream s) { NullIsPerThread scope; return cuMemcpyDtoHAsync(h, d, n, s); }
API cuMemsetD32Async_ptsz(CUdeviceptr d, unsigned v, size_t n, CUstream s) { NullIsPerThread scope; return cuMemsetD32Async(d, v, n, s); }
API cuEventRecord_ptsz(CUevent e, CUstream s) { NullIsPerThread scope; return cuEventRecord(e, s); }
API cuStreamSynchronize_ptsz(CUstream s) { NullIsPerThread scope; return cuStreamSynchronize(s); }
API cuStreamQuery_ptsz(CUstream s) { NullIsPerThread scope; return cuStreamQuery(s); }
__attribute__((visibility("default"))) uint64_t fakePerThreadStreamOps() { return g_per_thread_stream_ops.load(); }

API cuGetProcAddress(const char *symbol, void **pfn, int, cuuint64_t lookup_flags, CUdriverProcAddressQueryResult *status) {
    Dl_info info;
    void *self = dladdr((void *)&cuInit, &info) ? dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD) : nullptr;
    void *p = nullptr;
    if (self) {
        char name[128];
        if (lookup_flags & CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM) {
            std::snprintf(name, sizeof(name), "%s_v2_ptsz", symbol);
            p = dlsym(self, name);
            if (!p) { std::snprintf(name, sizeof(name), "%s_ptsz", symbol); p = dlsym(self, name); }
        }
        std::snprintf(name, sizeof(name), "%s_v2", symbol);
        if (!p) p = dlsym(self, name);
        if (!p) p = dlsym(self, symbol);
    }
    *pfn = p;
    if (status) *status = p ? CU_GET_PROC_ADDRESS_SUCCESS : CU_GET_PROC_ADDRESS_SYMBOL_NOT_FOUND;
    return p ? CUDA_SUCCESS : CUDA_ERROR_NOT_FOUND;
}

} // extern "C"
