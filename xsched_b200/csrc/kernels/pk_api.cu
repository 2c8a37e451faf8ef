// C ABI of the preemptible-kernel library (declared in include/xsched_b200/pk.h).
// Host-side bookkeeping only: control-block allocation, launch geometry, mailbox reads.
#include "xsched_b200/pk.h"
#include "pk_common.cuh"

#include <cuda.h>
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>

namespace xpk {
// stream_kernels.cu
cudaError_t launch_stream(int op, bool preemptible, Ctl *ctl, float *out, const float *x, const float *y, float s,
                          unsigned long long n, unsigned long long tile_elems, unsigned long long launch_no,
                          int grid, cudaStream_t stream);
int stream_ctas_per_sm();
// radix_sort.cu
size_t sort_smem_bytes();
cudaError_t sort_prepare();
int sort_ctas_per_sm(bool preemptible);
unsigned long long sort_tiles(unsigned long long n);
cudaError_t launch_sort(bool preemptible, Ctl *ctl, uint32_t *keys, uint32_t *tmp, uint32_t *hist, uint32_t *state,
                        unsigned long long n, unsigned long long launch_no, int grid, cudaStream_t stream);
// gemm_tcgen05.cu
int gemm_make_map(void *map_out, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows);
cudaError_t gemm_prepare();
unsigned long long gemm_tiles(uint32_t M, uint32_t N);
cudaError_t launch_gemm(bool preemptible, bool abort_inflight, Ctl *ctl, const void *map_a, const void *map_b, void *C,
                        uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no, int grid, cudaStream_t stream);
// gemm_pair.cu
cudaError_t gemm_pair_prepare();
unsigned long long gemm_pair_tiles(uint32_t M, uint32_t N);
cudaError_t launch_gemm_pair(bool preemptible, bool abort_inflight, Ctl *ctl, const void *map_a, const void *map_b, void *C,
                             uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no, int grid, cudaStream_t stream);
} // namespace xpk

using xpk::Ctl;
using xpk::Mailbox;

struct xpkTask_st {
    uint32_t kind = 0;
    uint32_t flags = 0;
    int device = 0;
    int sm_count = 0;
    Ctl *ctl = nullptr;               // device
    Mailbox *mb_host = nullptr;       // mapped pinned host memory
    Mailbox *mb_dev = nullptr;        // device alias
    uint32_t *flag = nullptr;         // flag the kernels poll
    unsigned long long total = 0;
    // Written by whichever thread launches or resets the task (an XQueue worker, the scheduler's thread on a
    // relaunch), read by application threads in xpkTaskQuery / xpkTaskWait.
    std::atomic<unsigned long long> launches{0};        // launch counter echoed by the mailbox
    std::atomic<unsigned long long> reset_at{0};        // value of `launches` at the last reset
    std::atomic<cudaStream_t> last_stream{nullptr};     // stream of the most recent launch
    // operands
    void *p0 = nullptr; const void *p1 = nullptr; const void *p2 = nullptr;
    float s = 0.f;
    unsigned long long n = 0;
    unsigned long long tile_elems = 0;
    uint32_t *sort_hist = nullptr, *sort_state = nullptr;
    size_t sort_scratch_bytes = 0;
    uint32_t M = 0, N = 0, K = 0;
    bool gemm_pair = false;           // the two-CTA form (tensor maps with 128-row boxes)
    alignas(64) unsigned char map_a[128];
    alignas(64) unsigned char map_b[128];
};

namespace {

constexpr bool kGemmPairByDefault = true;
std::atomic<uint64_t> g_launches{0};
} // namespace
namespace xpk { void note_launches(unsigned n) { g_launches.fetch_add(n); } }
namespace {

constexpr size_t kSortScratchHeader = 4096;   // hist[4][256] u32

typedef CUresult (*WriteValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

WriteValue32Fn write_value32() {
    static WriteValue32Fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (WriteValue32Fn)p;
    });
    return fn;
}

struct DeviceState {
    int sm_count = 0;
    int stream_ctas = 0;
    int sort_ctas = 0;
    bool sort_ready = false, gemm_ready = false;
    cudaStream_t ctrl = nullptr;
};
std::mutex g_dev_mtx;
DeviceState g_dev[64];

DeviceState *device_state(int *dev_out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_dev_mtx);
    DeviceState &d = g_dev[dev];
    if (d.sm_count == 0) {
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (cudaStreamCreateWithPriority(&d.ctrl, cudaStreamNonBlocking, hi) != cudaSuccess) return nullptr;
    }
    if (dev_out) *dev_out = dev;
    return &d;
}

// Makes the task's device current for the duration of a call and puts the caller's device back.  The
// entry points that take a task may be called from any thread (a worker thread that never called
// cudaSetDevice is on device 0), while the task's memory and streams belong to the device it was
// created on.
class DeviceGuard {
public:
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev_) != cudaSuccess) { prev_ = -1; return; }
        if (prev_ != device) { if (cudaSetDevice(device) == cudaSuccess) switched_ = true; }
    }
    ~DeviceGuard() { if (switched_) cudaSetDevice(prev_); }
    DeviceGuard(const DeviceGuard &) = delete;
    DeviceGuard &operator=(const DeviceGuard &) = delete;
private:
    int prev_ = -1;
    bool switched_ = false;
};

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

xpkResult task_common(xpkTask_st *t, uint32_t kind, uint32_t flags, unsigned long long total, uint32_t *flag_dev) {
    DeviceState *d = device_state(&t->device);
    if (!d) return XPK_ERR_CUDA;
    t->kind = kind;
    t->flags = flags;
    t->sm_count = d->sm_count;
    t->total = total;
    if (cudaMalloc(&t->ctl, sizeof(Ctl)) != cudaSuccess) return XPK_ERR_CUDA;
    if (cudaMemset(t->ctl, 0, sizeof(Ctl)) != cudaSuccess) return XPK_ERR_CUDA;
    if (cudaHostAlloc(&t->mb_host, sizeof(Mailbox), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
        return XPK_ERR_CUDA;
    std::memset(t->mb_host, 0, sizeof(Mailbox));
    if (cudaHostGetDevicePointer(&t->mb_dev, t->mb_host, 0) != cudaSuccess) return XPK_ERR_CUDA;
    t->flag = flag_dev ? flag_dev : &t->ctl->own_flag;
    struct Tail { unsigned long long total; const uint32_t *flag; Mailbox *mailbox; } tail{total, t->flag, t->mb_dev};
    if (cudaMemcpy(&t->ctl->total, &tail, sizeof(tail), cudaMemcpyHostToDevice) != cudaSuccess) return XPK_ERR_CUDA;
    return XPK_SUCCESS;
}

void task_free(xpkTask_st *t) {
    if (!t) return;
    if (t->ctl) cudaFree(t->ctl);
    if (t->mb_host) cudaFreeHost(t->mb_host);
    delete t;
}

} // namespace

extern "C" {

const char *xpkResultString(xpkResult r) {
    switch (r) {
    case XPK_SUCCESS: return "success";
    case XPK_ERR_INVALID_VALUE: return "invalid value";
    case XPK_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case XPK_ERR_CUDA: return "CUDA call failed";
    case XPK_ERR_NOT_SUPPORTED: return "shape not supported";
    case XPK_ERR_BUSY: return "task busy / wait timed out";
    case XPK_ERR_DEVICE_TIMEOUT: return "bounded device-side wait expired";
    case XPK_ERR_TOO_LARGE: return "size exceeds a static capacity";
    }
    return "unknown";
}

xpkResult xpkDeviceSmCount(int *sm_count) {
    if (!sm_count) return XPK_ERR_INVALID_VALUE;
    DeviceState *d = device_state(nullptr);
    if (!d) return XPK_ERR_CUDA;
    *sm_count = d->sm_count;
    return XPK_SUCCESS;
}

uint64_t xpkLaunchCount(void) { return g_launches.load(); }

xpkResult xpkFlagCreate(uint32_t **flag_dev) {
    if (!flag_dev) return XPK_ERR_INVALID_VALUE;
    void *p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return XPK_ERR_CUDA;
    if (cudaMemset(p, 0, 256) != cudaSuccess) { cudaFree(p); return XPK_ERR_CUDA; }
    *flag_dev = (uint32_t *)p;
    return XPK_SUCCESS;
}

xpkResult xpkFlagDestroy(uint32_t *flag_dev) {
    if (!flag_dev) return XPK_ERR_INVALID_VALUE;
    return cudaFree(flag_dev) == cudaSuccess ? XPK_SUCCESS : XPK_ERR_CUDA;
}

xpkResult xpkFlagSet(uint32_t *flag_dev, uint32_t value, void *ctrl_stream) {
    if (!flag_dev) return XPK_ERR_INVALID_VALUE;
    // The write goes through a stream of the device that owns the flag, whatever device the caller is on.
    cudaPointerAttributes attr;
    int owner = -1;
    if (cudaPointerGetAttributes(&attr, flag_dev) == cudaSuccess && attr.type == cudaMemoryTypeDevice) owner = attr.device;
    else cudaGetLastError();
    int cur = 0;
    cudaGetDevice(&cur);
    DeviceGuard on_flag_device(owner >= 0 ? owner : cur);
    DeviceState *d = device_state(nullptr);
    if (!d) return XPK_ERR_CUDA;
    cudaStream_t s = ctrl_stream ? (cudaStream_t)ctrl_stream : d->ctrl;
    WriteValue32Fn fn = write_value32();
    if (fn) {
        if (fn((CUstream)s, (CUdeviceptr)(uintptr_t)flag_dev, value, 0) == CUDA_SUCCESS) return XPK_SUCCESS;
    }
    // Fallback: a 4-byte memset node on the control stream.
    if (value <= 0xFFu || value == 0xFFFFFFFFu) {
        if (cudaMemsetAsync(flag_dev, (int)(value & 0xFF), 4, s) == cudaSuccess) return XPK_SUCCESS;
    }
    return XPK_ERR_CUDA;
}

xpkResult xpkFlagAttachRelay(uint32_t *flag_dev, volatile uint32_t **relay_host) {
    if (!flag_dev || !relay_host || (reinterpret_cast<uintptr_t>(flag_dev) & 15u)) return XPK_ERR_INVALID_VALUE;
    void *host = nullptr, *alias = nullptr;
    if (cudaHostAlloc(&host, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return XPK_ERR_CUDA;
    std::memset(host, 0, 64);
    if (cudaHostGetDevicePointer(&alias, host, 0) != cudaSuccess) { cudaFreeHost(host); return XPK_ERR_CUDA; }
    const unsigned long long value = (unsigned long long)(uintptr_t)alias;
    if (cudaMemcpy((unsigned char *)flag_dev + 8, &value, 8, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFreeHost(host); return XPK_ERR_CUDA; }
    *relay_host = (volatile uint32_t *)host;
    return XPK_SUCCESS;
}

xpkResult xpkFlagDetachRelay(uint32_t *flag_dev, volatile uint32_t *relay_host) {
    if (!flag_dev || !relay_host) return XPK_ERR_INVALID_VALUE;
    const unsigned long long none = 0;
    const bool ok = cudaMemcpy((unsigned char *)flag_dev + 8, &none, 8, cudaMemcpyHostToDevice) == cudaSuccess;
    cudaFreeHost((void *)relay_host);
    return ok ? XPK_SUCCESS : XPK_ERR_CUDA;
}

static xpkResult create_stream_task(xpkTask_t *task, uint32_t kind, float *out, const float *x, const float *y,
                                    float s, uint64_t n, uint32_t tile_elems, uint32_t flags, uint32_t *flag_dev) {
    if (!task || !out || !x || !y || n == 0) return XPK_ERR_INVALID_VALUE;
    if (!aligned16(out) || !aligned16(x) || !aligned16(y)) return XPK_ERR_ALIGNMENT;
    if (tile_elems == 0) tile_elems = 16384;
    if (tile_elems % 4096 != 0) return XPK_ERR_INVALID_VALUE;
    xpkTask_st *t = new (std::nothrow) xpkTask_st();
    if (!t) return XPK_ERR_CUDA;
    const unsigned long long total = (n + tile_elems - 1) / tile_elems;
    xpkResult r = task_common(t, kind, flags, total, flag_dev);
    if (r != XPK_SUCCESS) { task_free(t); return r; }
    t->p0 = out; t->p1 = x; t->p2 = y; t->s = s; t->n = n; t->tile_elems = tile_elems;
    DeviceState *d = device_state(nullptr);
    {
        std::lock_guard<std::mutex> lk(g_dev_mtx);
        if (d->stream_ctas == 0) d->stream_ctas = xpk::stream_ctas_per_sm();
    }
    *task = t;
    return XPK_SUCCESS;
}

xpkResult xpkTaskCreateTriad(xpkTask_t *task, float *a, const float *b, const float *c, float s, uint64_t n,
                             uint32_t tile_elems, uint32_t flags, uint32_t *flag_dev) {
    return create_stream_task(task, XPK_KIND_TRIAD, a, b, c, s, n, tile_elems, flags, flag_dev);
}

xpkResult xpkTaskCreateVecAdd(xpkTask_t *task, float *c, const float *a, const float *b, uint64_t n,
                              uint32_t tile_elems, uint32_t flags, uint32_t *flag_dev) {
    return create_stream_task(task, XPK_KIND_VECADD, c, a, b, 0.f, n, tile_elems, flags, flag_dev);
}

size_t xpkSortScratchBytes(uint64_t n) {
    const unsigned long long T = xpk::sort_tiles(n);
    return kSortScratchHeader + (size_t)4 * T * 256 * sizeof(uint32_t);
}

xpkResult xpkTaskCreateSort(xpkTask_t *task, int32_t *keys, int32_t *tmp, void *scratch, uint64_t n, uint32_t flags,
                            uint32_t *flag_dev) {
    if (!task || !keys || !tmp || !scratch || n == 0) return XPK_ERR_INVALID_VALUE;
    if (n > (1ull << 30)) return XPK_ERR_TOO_LARGE;
    if (!aligned16(keys) || !aligned16(tmp) || (reinterpret_cast<uintptr_t>(scratch) & 255u)) return XPK_ERR_ALIGNMENT;
    xpkTask_st *t = new (std::nothrow) xpkTask_st();
    if (!t) return XPK_ERR_CUDA;
    const unsigned long long T = xpk::sort_tiles(n);
    xpkResult r = task_common(t, XPK_KIND_SORT, flags, 5 * T, flag_dev);
    if (r != XPK_SUCCESS) { task_free(t); return r; }
    t->p0 = keys; t->p1 = tmp; t->n = n;
    t->sort_hist = (uint32_t *)scratch;
    t->sort_state = (uint32_t *)((unsigned char *)scratch + kSortScratchHeader);
    t->sort_scratch_bytes = xpkSortScratchBytes(n);
    DeviceState *d = device_state(nullptr);
    {
        std::lock_guard<std::mutex> lk(g_dev_mtx);
        if (!d->sort_ready) {
            if (xpk::sort_prepare() != cudaSuccess) { task_free(t); return XPK_ERR_CUDA; }
            d->sort_ctas = std::min(xpk::sort_ctas_per_sm(true), xpk::sort_ctas_per_sm(false));
            d->sort_ready = true;
        }
    }
    if (cudaMemset(scratch, 0, t->sort_scratch_bytes) != cudaSuccess) { task_free(t); return XPK_ERR_CUDA; }
    *task = t;
    return XPK_SUCCESS;
}

xpkResult xpkTaskCreateGemm(xpkTask_t *task, void *C, const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K,
                            uint32_t flags, uint32_t *flag_dev) {
    if (!task || !C || !A || !B || M == 0 || N == 0 || K == 0) return XPK_ERR_INVALID_VALUE;
    if (M % 128 || N % 256 || K % 64) return XPK_ERR_NOT_SUPPORTED;
    if (!aligned16(C) || !aligned16(A) || !aligned16(B)) return XPK_ERR_ALIGNMENT;
    xpkTask_st *t = new (std::nothrow) xpkTask_st();
    if (!t) return XPK_ERR_CUDA;
    // Which form runs the task: a flag decides, else XPK_GEMM_FORM=one|pair, else the library's choice.  A pair needs two SMs.
    bool use_pair = kGemmPairByDefault;
    if (const char *form = std::getenv("XPK_GEMM_FORM")) use_pair = std::strcmp(form, "one") != 0;
    if (flags & XPK_FLAG_GEMM_ONE_CTA) use_pair = false;
    else if (flags & XPK_FLAG_GEMM_CTA_PAIR) use_pair = true;
    {
        int sms = 0, dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { task_free(t); return XPK_ERR_CUDA; }
        if (sms < 2) use_pair = false;
    }
    xpkResult r = task_common(t, XPK_KIND_GEMM, flags, use_pair ? xpk::gemm_pair_tiles(M, N) : xpk::gemm_tiles(M, N), flag_dev);
    if (r != XPK_SUCCESS) { task_free(t); return r; }
    t->p0 = C; t->p1 = A; t->p2 = B; t->M = M; t->N = N; t->K = K;
    t->gemm_pair = use_pair;
    DeviceState *d = device_state(nullptr);
    {
        std::lock_guard<std::mutex> lk(g_dev_mtx);
        if (!d->gemm_ready) {
            if (xpk::gemm_prepare() != cudaSuccess || xpk::gemm_pair_prepare() != cudaSuccess) { task_free(t); return XPK_ERR_CUDA; }
            d->gemm_ready = true;
        }
    }
    const uint32_t box_rows = t->gemm_pair ? 128 : 256;
    if (xpk::gemm_make_map(t->map_a, A, M, K, box_rows) != 0 || xpk::gemm_make_map(t->map_b, B, N, K, box_rows) != 0) {
        task_free(t);
        return XPK_ERR_CUDA;
    }
    *task = t;
    return XPK_SUCCESS;
}

xpkResult xpkTaskLaunch(xpkTask_t t, void *stream, int sm_limit) {
    if (!t) return XPK_ERR_INVALID_VALUE;
    DeviceGuard on_task_device(t->device);
    DeviceState *d = device_state(nullptr);
    if (!d) return XPK_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    const bool preemptible = !(t->flags & XPK_FLAG_NON_PREEMPTIBLE);
    int sms = t->sm_count;
    if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
    const unsigned long long launch_no = t->launches.fetch_add(1) + 1;
    cudaError_t e = cudaSuccess;
    unsigned long long grid;
    switch (t->kind) {
    case XPK_KIND_TRIAD:
    case XPK_KIND_VECADD:
        grid = (unsigned long long)sms * d->stream_ctas;
        if (grid > t->total) grid = t->total;
        e = xpk::launch_stream(t->kind == XPK_KIND_TRIAD ? 0 : 1, preemptible, t->ctl, (float *)t->p0,
                               (const float *)t->p1, (const float *)t->p2, t->s, t->n, t->tile_elems, launch_no,
                               (int)grid, s);
        break;
    case XPK_KIND_SORT:
        grid = (unsigned long long)sms * d->sort_ctas;
        if (grid > t->total) grid = t->total;
        e = xpk::launch_sort(preemptible, t->ctl, (uint32_t *)t->p0, (uint32_t *)t->p1, t->sort_hist, t->sort_state,
                             t->n, launch_no, (int)grid, s);
        break;
    case XPK_KIND_GEMM:
        grid = (unsigned long long)sms;
        if (t->gemm_pair) {
            // Whole pairs only, one pair per tile at most; an SM limit of one still gets a pair.
            if (grid > 2 * t->total) grid = 2 * t->total;
            grid = grid < 2 ? 2 : grid & ~1ull;
            e = xpk::launch_gemm_pair(preemptible, (t->flags & XPK_FLAG_ABORT_INFLIGHT) != 0, t->ctl, t->map_a, t->map_b, t->p0,
                                      t->M, t->N, t->K, launch_no, (int)grid, s);
            break;
        }
        if (grid > t->total) grid = t->total;
        e = xpk::launch_gemm(preemptible, (t->flags & XPK_FLAG_ABORT_INFLIGHT) != 0, t->ctl, t->map_a, t->map_b, t->p0,
                             t->M, t->N, t->K, launch_no, (int)grid, s);
        break;
    default:
        return XPK_ERR_INVALID_VALUE;
    }
    if (e != cudaSuccess) return XPK_ERR_CUDA;
    t->last_stream.store(s);
    g_launches.fetch_add(1);
    return XPK_SUCCESS;
}

xpkResult xpkTaskQuery(xpkTask_t t, xpkTaskInfo *info) {
    if (!t || !info) return XPK_ERR_INVALID_VALUE;
    volatile Mailbox *m = t->mb_host;
    // One reading of each counter per query: a launch from another thread may land in between.
    const unsigned long long launches = t->launches.load(), reset_at = t->reset_at.load();
    const unsigned long long seq = m->seq;
    std::atomic_thread_fence(std::memory_order_acquire);
    info->tiles_total = t->total;
    info->launches = launches;
    if (launches == reset_at) {                  // nothing launched since creation / reset
        info->status = XPK_STATUS_IDLE;
        info->error = 0; info->tiles_done = 0; info->preemptions = 0;
    } else if (seq < launches) {                 // the newest launch has not published yet
        info->status = XPK_STATUS_RUNNING;
        info->error = 0;
        info->tiles_done = seq > reset_at ? m->tiles_done : 0;
        info->preemptions = seq > reset_at ? m->preemptions : 0;
    } else {
        info->status = m->status;
        info->error = m->error;
        info->tiles_done = m->tiles_done;
        info->preemptions = m->preemptions;
    }
    return XPK_SUCCESS;
}

xpkResult xpkTaskWait(xpkTask_t t, uint64_t timeout_us, xpkTaskInfo *info) {
    if (!t) return XPK_ERR_INVALID_VALUE;
    volatile Mailbox *m = t->mb_host;
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t spins = 0;
    while (t->launches.load() != t->reset_at.load() && m->seq < t->launches.load()) {
        if (++spins > 2000) {
            std::this_thread::yield();
            if ((spins & 1023u) == 0) {
                // A faulted context never publishes: surface the CUDA error instead of timing out.
                const cudaError_t qe = cudaStreamQuery(t->last_stream.load());
                if (qe != cudaSuccess && qe != cudaErrorNotReady) return XPK_ERR_CUDA;
                const auto us = std::chrono::duration_cast<std::chrono::microseconds>(
                                    std::chrono::steady_clock::now() - t0).count();
                if ((uint64_t)us > timeout_us) return XPK_ERR_BUSY;
            }
        }
    }
    xpkTaskInfo local;
    xpkResult r = xpkTaskQuery(t, info ? info : &local);
    if (r != XPK_SUCCESS) return r;
    const uint32_t st = (info ? info : &local)->status;
    return st == XPK_STATUS_ERROR ? XPK_ERR_DEVICE_TIMEOUT : XPK_SUCCESS;
}

xpkResult xpkTaskTimes(xpkTask_t t, uint64_t *start_ns, uint64_t *exit_ns) {
    if (!t || !start_ns || !exit_ns) return XPK_ERR_INVALID_VALUE;
    volatile Mailbox *m = t->mb_host;
    if (m->seq == 0) return XPK_ERR_BUSY;
    std::atomic_thread_fence(std::memory_order_acquire);
    *start_ns = m->start_ns;
    *exit_ns = m->exit_ns;
    return XPK_SUCCESS;
}

xpkResult xpkTaskReset(xpkTask_t t, void *stream) {
    if (!t) return XPK_ERR_INVALID_VALUE;
    DeviceGuard on_task_device(t->device);
    cudaStream_t s = (cudaStream_t)stream;
    // A task that was never launched, or whose newest launch has published COMPLETED, already stands at tile 0
    // (a finishing kernel re-arms its control block): nothing to clear.  Anything else — running, preempted,
    // failed — is rewound by a stream-ordered memset.
    volatile Mailbox *m = t->mb_host;
    const unsigned long long launches = t->launches.load();
    const bool at_start = launches == t->reset_at.load() || (m->seq == launches && m->status == XPK_STATUS_COMPLETED);
    if (!at_start && cudaMemsetAsync(t->ctl, 0, xpk::kCtlResetBytes, s) != cudaSuccess) return XPK_ERR_CUDA;
    if (t->kind == XPK_KIND_SORT) {
        if (cudaMemsetAsync(t->sort_hist, 0, t->sort_scratch_bytes, s) != cudaSuccess) return XPK_ERR_CUDA;
    }
    t->reset_at.store(t->launches.load());
    return XPK_SUCCESS;
}

xpkResult xpkTaskFlag(xpkTask_t t, uint32_t **flag_dev) {
    if (!t || !flag_dev) return XPK_ERR_INVALID_VALUE;
    *flag_dev = t->flag;
    return XPK_SUCCESS;
}

xpkResult xpkTaskKind(xpkTask_t t, uint32_t *kind) {
    if (!t || !kind) return XPK_ERR_INVALID_VALUE;
    *kind = t->kind;
    return XPK_SUCCESS;
}

xpkResult xpkTaskDestroy(xpkTask_t t) {
    if (!t) return XPK_ERR_INVALID_VALUE;
    DeviceGuard on_task_device(t->device);
    task_free(t);
    return XPK_SUCCESS;
}

} // extern "C"
