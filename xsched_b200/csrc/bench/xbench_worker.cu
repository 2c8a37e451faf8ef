// xbench_worker — native workload driver for the preemption benchmarks.  One process = one role:
//
//   --role lp    a low-priority loop of preemptible tasks (gemm | triad | sort) submitted through an
//                XQueue at the given preemption level until --duration-s elapses (or SIGTERM);
//   --role hp    a high-priority request every --period-us (vecadd | sort), latency = submit -> wait;
//   --role both  the two roles as two threads / two XQueues of ONE process (in-process scheduler);
//   --role idle  a process that holds a CUDA context, buffers and a suspended queue but runs nothing, and
//   --role spin-lp  one that runs --kernel-us sleep kernels back to back on a plain stream (no XQueue): the two
//                control arms beside which a high-priority process shows what another context costs by itself;
//   --role level-sweep   the reference's level-1 suspend-latency sweep over sleep kernels of 10..2000 us;
//   --role preempt-latency
//                the reference's preemption-latency experiment (platforms/cuda/test/main/level.cu:37-86):
//                a background thread keeps the queue full while the main thread times
//                XQueueSuspend(xq, kQueueSuspendFlagSyncHwQueue) / XQueueResume pairs at random moments.
//
// Everything goes through the public C ABI (XQueue*, XHint*, CudaQueue*, xpk*).  Results are printed as
// one JSON line on stdout; "READY" is printed once the role has warmed up.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cinttypes>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <numeric>
#include <vector>
#include <cuda_runtime.h>
#include <sys/prctl.h>
#include <cuda_bf16.h>

#include "xsched/xsched.h"
#include "xsched/cuda/hal.h"
#include "xsched_b200/pk.h"
#include "xsched/utils/trace.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s -> %s\n", #x, cudaGetErrorString(e_)); std::exit(3); } } while (0)
#define XK(x) do { XResult r_ = (x); if (r_ != kXSchedSuccess) { std::fprintf(stderr, "%s -> %d\n", #x, (int)r_); std::exit(4); } } while (0)
#define PK(x) do { xpkResult r_ = (x); if (r_ != XPK_SUCCESS) { std::fprintf(stderr, "%s -> %s\n", #x, xpkResultString(r_)); std::exit(5); } } while (0)

static std::atomic<bool> g_stop{false};
static void OnTerm(int) { g_stop.store(true); }
// SIGUSR1 delimits the measurement window of a long-running low-priority loop: the first one restarts the
// count (the high-priority process has warmed up and begins its requests now), the second one freezes it
// (the requests are over), so that the reported rate covers exactly the co-run interval.
static std::atomic<int> g_marks{0};
static void OnMark(int) { g_marks.fetch_add(1); }
static int64_t NowNs() { return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static void SleepUs(int64_t us) { if (us > 0) std::this_thread::sleep_for(std::chrono::microseconds(us)); }
static double Pct(std::vector<double> v, double p) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    return v[std::min(v.size() - 1, (size_t)(p * (v.size() - 1) + 0.5))];
}

struct Args {
    std::string role = "lp", kernel = "gemm", hp_kernel = "vecadd";
    int level = 2, prio = 0, threshold = 16, batch = 8, depth = 8, abort_inflight = 1, count = 500, device = 0, e2e = 0;
    int M = 8192, N = 8192, K = 8192;
    float b_std = 1.0f;       // standard deviation of the GEMM's B operand (0.02 = weight-like)
    uint64_t n = 1ull << 26, hp_n = 1ull << 26, seed = 1;
    double duration_s = 5, warmup_s = 0.5;
    int64_t period_us = 10000, kernel_us = 500, laxity_us = -1;
    int poisson = 0;
    int tamper_at = -1;       // self-test of the output check: spoil one sample of the output of this iteration before it is verified
    std::string samples_path;
};

static Args Parse(int argc, char **argv) {
    Args a;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string k = argv[i], v = argv[i + 1];
        if (k == "--role") a.role = v; else if (k == "--kernel") a.kernel = v; else if (k == "--hp-kernel") a.hp_kernel = v;
        else if (k == "--level") a.level = std::atoi(v.c_str()); else if (k == "--prio") a.prio = std::atoi(v.c_str());
        else if (k == "--threshold") a.threshold = std::atoi(v.c_str()); else if (k == "--batch") a.batch = std::atoi(v.c_str());
        else if (k == "--depth") a.depth = std::atoi(v.c_str()); else if (k == "--abort") a.abort_inflight = std::atoi(v.c_str());
        else if (k == "--count") a.count = std::atoi(v.c_str()); else if (k == "--device") a.device = std::atoi(v.c_str());
        else if (k == "--M") a.M = std::atoi(v.c_str()); else if (k == "--N") a.N = std::atoi(v.c_str()); else if (k == "--K") a.K = std::atoi(v.c_str());
        else if (k == "--n") a.n = std::strtoull(v.c_str(), nullptr, 10); else if (k == "--hp-n") a.hp_n = std::strtoull(v.c_str(), nullptr, 10);
        else if (k == "--b-std") a.b_std = (float)std::atof(v.c_str());
        else if (k == "--seed") a.seed = std::strtoull(v.c_str(), nullptr, 10);
        else if (k == "--duration-s") a.duration_s = std::atof(v.c_str()); else if (k == "--warmup-s") a.warmup_s = std::atof(v.c_str());
        else if (k == "--period-us") a.period_us = std::atoll(v.c_str()); else if (k == "--kernel-us") a.kernel_us = std::atoll(v.c_str());
        else if (k == "--laxity-us") a.laxity_us = std::atoll(v.c_str());
        else if (k == "--poisson") a.poisson = std::atoi(v.c_str()); else if (k == "--e2e") a.e2e = std::atoi(v.c_str());
        else if (k == "--samples") a.samples_path = v;
        else if (k == "--tamper-at") a.tamper_at = std::atoi(v.c_str());
        else { std::fprintf(stderr, "unknown option %s\n", k.c_str()); std::exit(2); }
    }
    return a;
}

// ---- deterministic device-side initialisation (synthetic inputs; no host copy of multi-GiB arrays) ----
__device__ __forceinline__ uint32_t Mix(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return (uint32_t)x;
}
__global__ void FillUniform(float *p, uint64_t n, uint64_t seed) {           // U(-1, 1)
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        p[i] = (float)(Mix(i * 2654435761ull + seed) >> 8) * (2.0f / 16777216.0f) - 1.0f;
}
__global__ void FillNormalBf16(__nv_bfloat16 *p, uint64_t n, uint64_t seed, float std) {   // N(0, std) by Box-Muller
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float u1 = ((float)(Mix(i * 2 + seed) >> 8) + 1.0f) * (1.0f / 16777217.0f);
        const float u2 = (float)(Mix(i * 2 + 1 + seed * 31) >> 8) * (1.0f / 16777216.0f);
        p[i] = __float2bfloat16(std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
    }
}
__global__ void FillKeys(int32_t *p, uint64_t n, uint64_t seed) {            // U[0, 2^31)
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        p[i] = (int32_t)(Mix(i + seed * 0x9E3779B97F4A7C15ull) & 0x7FFFFFFFu);
}
// Output check of the low-priority loops.  A tile that a preempted-and-resumed iteration never wrote must be
// visible, so every iteration's output starts out spoiled and is looked at before the buffer is reused:
//   * SamplePoison writes a NaN pattern into one 32-byte sector every `stride_words` words of the buffer,
//     SampleHash reads exactly those sectors back (order-sensitive 64-bit sum, the formula of the CPU oracle's
//     checksum restricted to the sampled words).  The stride is chosen so that every
//     row of every GEMM tile (512 bytes) and every quarter of a streaming tile (16 KiB) holds a sample: a tile
//     that was skipped, or written only in part, keeps poison in at least one of them.
//   * both run on a side stream, on a buffer no in-flight task touches (each slot of the loop owns its output).
// A whole-buffer hash (stride 8 words = every sector) is taken where it is cheap against the iteration.
constexpr uint32_t kPoisonWord = 0xFFFFFFFFu;            // NaN as bf16 pair and as fp32; never produced by a sort of non-negative keys
__global__ void SamplePoison(uint32_t *p, uint64_t words, uint64_t stride_words) {
    const uint64_t samples = (words + stride_words - 1) / stride_words;
    for (uint64_t k = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; k < samples; k += (uint64_t)gridDim.x * blockDim.x)
        for (uint64_t w = k * stride_words; w < k * stride_words + 8 && w < words; ++w) p[w] = kPoisonWord;
}
__global__ void SampleHash(const uint32_t *p, uint64_t words, uint64_t stride_words, unsigned long long *out) {
    const uint64_t samples = (words + stride_words - 1) / stride_words;
    unsigned long long h = 0;
    for (uint64_t k = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; k < samples; k += (uint64_t)gridDim.x * blockDim.x)
        for (uint64_t w = k * stride_words; w < k * stride_words + 8 && w < words; ++w)
            h += (unsigned long long)p[w] * ((w & 0xFFFFu) + 1u);
    for (int o = 16; o; o >>= 1) h += __shfl_down_sync(0xffffffffu, h, o);
    if ((threadIdx.x & 31) == 0 && h) atomicAdd(out, h);
}
// The checks run on a side stream while the next iterations' kernels occupy the GPU: blocks of 128 threads (5 K
// registers) still find room on an SM beside a CTA of the two-CTA GEMM, which holds 59 K of its 64 K registers.
constexpr int kCheckBlocks = 1184, kCheckThreads = 128;
struct Verifier {
    cudaStream_t side = nullptr;
    unsigned long long *dev = nullptr, *host = nullptr;
    void Init() {
        CK(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
        CK(cudaMalloc(&dev, 8));
        CK(cudaMallocHost(&host, 8));
    }
    unsigned long long Hash(const void *p, uint64_t words, uint64_t stride_words) {
        CK(cudaMemsetAsync(dev, 0, 8, side));
        SampleHash<<<kCheckBlocks, kCheckThreads, 0, side>>>((const uint32_t *)p, words, stride_words, dev);
        CK(cudaMemcpyAsync(host, dev, 8, cudaMemcpyDeviceToHost, side));
        CK(cudaStreamSynchronize(side));
        return *host;
    }
    void Poison(void *p, uint64_t words, uint64_t stride_words) {
        SamplePoison<<<kCheckBlocks, kCheckThreads, 0, side>>>((uint32_t *)p, words, stride_words);
        CK(cudaStreamSynchronize(side));
    }
};

// ---- timeline support: device clock against the host's monotonic clock --------------------------------------
// A one-thread kernel publishes %globaltimer to a mapped host word for a fraction of a millisecond while the
// host reads the word and its own clock; the smallest (host - device) difference seen is the offset plus the
// shortest time a device write takes to become visible to the host (well under a microsecond).  The two clocks
// drift against each other (tens of microseconds per second were seen), so a process calibrates when it starts and
// again when it is done, and readers interpolate.
__global__ void PublishClock(volatile unsigned long long *out, int rounds) {
    for (int i = 0; i < rounds; ++i) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        *out = t;
        __threadfence_system();
    }
}
static void CalibrateGpuClock() {
    if (!XTraceEnabled()) return;
    unsigned long long *h = nullptr, *d = nullptr;
    CK(cudaHostAlloc(&h, 64, cudaHostAllocMapped));
    *h = 0;
    CK(cudaHostGetDevicePointer(&d, h, 0));
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    int64_t best = INT64_MAX, worst_seen = 0;
    for (int rep = 0; rep < 3; ++rep) {
        PublishClock<<<1, 1, 0, s>>>(d, 20000);
        unsigned long long last = 0;
        while (cudaStreamQuery(s) == cudaErrorNotReady) {
            for (int i = 0; i < 200; ++i) {
                const unsigned long long v = *(volatile unsigned long long *)h;
                const int64_t now = NowNs();
                if (v != 0 && v != last) { const int64_t diff = now - (int64_t)v; if (diff < best) best = diff; if (diff > worst_seen) worst_seen = diff; last = v; }
            }
        }
        CK(cudaStreamSynchronize(s));
    }
    XTraceStamp(xsched::utils::kTraceGpuClockOffset, (uint64_t)best, 1000);
    CK(cudaStreamDestroy(s));
    CK(cudaFreeHost(h));
}

struct Queue {
    cudaStream_t stream = nullptr;
    HwQueueHandle hwq = 0;
    XQueueHandle xq = 0;
    uint32_t *flag = nullptr;
};
static Queue MakeQueue(const Args &a, int level, int prio) {
    Queue q;
    CK(cudaStreamCreateWithFlags(&q.stream, cudaStreamNonBlocking));
    XK(CudaQueueCreate(&q.hwq, (CUstream)q.stream));
    XK(XQueueCreate(&q.xq, q.hwq, level, kQueueCreateFlagNone));
    XK(XQueueSetLaunchConfig(q.xq, a.threshold, a.batch));
    XK(XHintPriority(q.xq, prio));
    if (a.laxity_us >= 0 && prio > 0) XK(XHintLaxity(q.xq, a.laxity_us, 0, prio));
    XK(CudaQueueGetPreemptFlag(q.hwq, &q.flag));
    return q;
}

// ---- low-priority workload ------------------------------------------------------------------------
struct LpWork {
    std::vector<xpkTask_t> tasks;       // `depth` tasks over the same inputs, each with an output buffer of its own
    std::vector<void *> outs;           // output of task i (the sort has one task and sorts in place)
    uint64_t out_words = 0;
    uint64_t sample_stride_words = 8;   // distance between the sampled sectors of the per-iteration check (8 = every sector)
    bool full_hash_cheap = true;        // also hash the whole output after every iteration
    double work_per_iter = 0;           // flop or bytes
    const char *unit = "";
    // sort needs its input restored before every iteration
    int32_t *keys = nullptr, *keys0 = nullptr;
    uint64_t nkeys = 0;
};

static LpWork BuildLp(const Args &a, const Queue &q, uint32_t task_flags) {
    LpWork w;
    cudaStream_t s = q.stream;
    if (a.kernel == "gemm") {
        __nv_bfloat16 *A, *B;
        CK(cudaMalloc(&A, (size_t)a.M * a.K * 2)); CK(cudaMalloc(&B, (size_t)a.N * a.K * 2));
        FillNormalBf16<<<1184, 256, 0, s>>>(A, (uint64_t)a.M * a.K, a.seed, 1.0f);
        FillNormalBf16<<<1184, 256, 0, s>>>(B, (uint64_t)a.N * a.K, a.seed + 7, a.b_std);
        CK(cudaStreamSynchronize(s));
        for (int i = 0; i < a.depth; ++i) {
            xpkTask_t t;
            void *C;
            CK(cudaMalloc(&C, (size_t)a.M * a.N * 2));
            PK(xpkTaskCreateGemm(&t, C, A, B, a.M, a.N, a.K, task_flags | (a.abort_inflight ? XPK_FLAG_ABORT_INFLIGHT : 0), q.flag));
            w.tasks.push_back(t);
            w.outs.push_back(C);
        }
        w.out_words = (uint64_t)a.M * a.N / 2;
        w.sample_stride_words = 128;          // one sector per 512 bytes: every row of every 256-column tile
        w.work_per_iter = 2.0 * a.M * a.N * a.K; w.unit = "TFLOP/s";
    } else if (a.kernel == "triad") {
        float *y, *z;
        CK(cudaMalloc(&y, a.n * 4)); CK(cudaMalloc(&z, a.n * 4));
        FillUniform<<<1184, 256, 0, s>>>(y, a.n, a.seed);
        FillUniform<<<1184, 256, 0, s>>>(z, a.n, a.seed + 11);
        CK(cudaStreamSynchronize(s));
        for (int i = 0; i < a.depth; ++i) {
            xpkTask_t t;
            float *x;
            CK(cudaMalloc(&x, a.n * 4));
            PK(xpkTaskCreateTriad(&t, x, y, z, 1.5f, a.n, 0, task_flags, q.flag));
            w.tasks.push_back(t);
            w.outs.push_back(x);
        }
        w.out_words = a.n;
        w.sample_stride_words = 4096;         // one sector per 16 KiB: four per 16 Ki-element tile
        w.full_hash_cheap = a.n <= (1ull << 28);   // re-reading 8 GiB per iteration would take a third of the loop's bandwidth
        w.work_per_iter = 12.0 * a.n; w.unit = "GB/s";
    } else if (a.kernel == "sort") {
        int32_t *tmp; void *scratch;
        CK(cudaMalloc(&w.keys, a.n * 4)); CK(cudaMalloc(&w.keys0, a.n * 4)); CK(cudaMalloc(&tmp, a.n * 4));
        CK(cudaMalloc(&scratch, xpkSortScratchBytes(a.n)));
        FillKeys<<<1184, 256, 0, s>>>(w.keys0, a.n, a.seed);
        CK(cudaStreamSynchronize(s));
        xpkTask_t t;                     // one task: the scratch area is per task
        PK(xpkTaskCreateSort(&t, w.keys, tmp, scratch, a.n, task_flags, q.flag));
        w.tasks.push_back(t);
        w.nkeys = a.n;
        w.outs.push_back(w.keys); w.out_words = a.n;
        w.work_per_iter = 36.0 * a.n; w.unit = "GB/s";
    } else {
        std::fprintf(stderr, "unknown --kernel %s\n", a.kernel.c_str());
        std::exit(2);
    }
    return w;
}

struct LpResult {
    uint64_t iters = 0; double seconds = 0, rate = 0; unsigned long long want = 0, got = 0; uint64_t preemptions = 0; CudaQueueStats stats{};
    uint64_t verified_iters = 0, verified_preempted_iters = 0, mismatched_iters = 0;    // per-iteration output checks
};

static XResult RestoreKeys(HwQueueHandle hwq, void *data) {
    LpWork *w = (LpWork *)data;
    return cudaMemcpyAsync(w->keys, w->keys0, w->nkeys * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)(uintptr_t)hwq) == cudaSuccess
               ? kXSchedSuccess : kXSchedErrorHardware;
}

// Expected hashes of one task's output: a straight run with the flag never raised, outside any XQueue.
struct LpExpect { unsigned long long full = 0, sampled = 0; };
static LpExpect StraightRun(const Queue &q, LpWork &w, Verifier &v) {
    if (w.keys) CK(cudaMemcpyAsync(w.keys, w.keys0, w.nkeys * 4, cudaMemcpyDeviceToDevice, q.stream));
    PK(xpkTaskReset(w.tasks[0], q.stream));
    PK(xpkTaskLaunch(w.tasks[0], q.stream, 0));
    CK(cudaStreamSynchronize(q.stream));
    LpExpect e;
    e.full = v.Hash(w.outs[0], w.out_words, 8);
    e.sampled = v.Hash(w.outs[0], w.out_words, w.sample_stride_words);
    return e;
}

// Looks at the output of the iteration that just completed in `slot` and spoils the buffer for the next one.
// Returns false when the output is not the straight run's.
static bool CheckSlot(const LpWork &w, Verifier &v, size_t slot, const LpExpect &want, bool tamper) {
    if (tamper) v.Poison((uint32_t *)w.outs[slot] + (w.out_words / 2 / w.sample_stride_words) * w.sample_stride_words, 8, 8);
    bool ok = v.Hash(w.outs[slot], w.out_words, w.sample_stride_words) == want.sampled;
    if (w.full_hash_cheap && w.sample_stride_words != 8) ok = ok && v.Hash(w.outs[slot], w.out_words, 8) == want.full;
    if (!w.keys) v.Poison(w.outs[slot], w.out_words, w.sample_stride_words);      // the sort's input is restored by its own command
    return ok;
}

static LpResult RunLp(const Args &a, const Queue &q, LpWork &w, std::atomic<bool> *ready, double duration_s) {
    LpResult r;
    Verifier v;
    v.Init();
    const LpExpect want = StraightRun(q, w, v);
    r.want = want.full;
    for (void *o : w.outs) if (!w.keys) v.Poison(o, w.out_words, w.sample_stride_words);

    auto submit = [&](size_t slot) {
        if (w.keys) {                                   // sort: restore the unsorted input first
            HwCommandHandle c;
            XK(HwCommandCreateCallback(&c, RestoreKeys, &w));
            XK(XQueueSubmit(q.xq, c));
        }
        HwCommandHandle c;
        XK(CudaXpkCommandCreate(&c, w.tasks[slot], 1));
        XK(XQueueSubmit(q.xq, c));
    };
    const size_t depth = w.tasks.size();
    std::vector<uint64_t> uses(depth, 0), preempt_seen(depth, 0);
    std::vector<bool> unchecked(depth, false);
    // A task object may be re-submitted only after its previous command completed.  That is read from
    // the task's mailbox (no queue drain).  A preempted command is launched more than once, so the launch
    // count alone does not tell which submission a COMPLETED status belongs to: the slot remembers the
    // launch count at which its previous submission was seen complete, and the next one is complete when
    // the task reports COMPLETED at a larger count (a completed task is not launched again before it is
    // re-submitted).
    std::vector<uint64_t> seen_complete_at(depth, 0);
    for (size_t i = 0; i < depth; ++i) { xpkTaskInfo info; PK(xpkTaskQuery(w.tasks[i], &info)); seen_complete_at[i] = info.launches; preempt_seen[i] = info.preemptions; }
    uint64_t checked = 0;
    // Every completed iteration is checked before its buffer is handed out again: the output must hash to the
    // straight run's, and it was spoiled before the iteration, so a tile the iteration (or the replay after a
    // preemption) never wrote shows.
    auto check_slot = [&](size_t slot) {
        if (!unchecked[slot]) return;
        xpkTaskInfo info;
        PK(xpkTaskQuery(w.tasks[slot], &info));
        const bool was_preempted = info.preemptions != preempt_seen[slot];
        preempt_seen[slot] = info.preemptions;
        const bool ok = CheckSlot(w, v, slot, want, a.tamper_at >= 0 && checked == (uint64_t)a.tamper_at);
        ++checked;
        ++r.verified_iters;
        if (was_preempted) ++r.verified_preempted_iters;
        if (!ok) ++r.mismatched_iters;
        unchecked[slot] = false;
    };
    auto wait_slot = [&](size_t slot) {
        if (uses[slot] == 0) return;
        while (!g_stop.load()) {
            xpkTaskInfo info;
            PK(xpkTaskQuery(w.tasks[slot], &info));
            if (info.launches > seen_complete_at[slot] && info.status == XPK_STATUS_COMPLETED) { seen_complete_at[slot] = info.launches; check_slot(slot); return; }
            if (info.status == XPK_STATUS_ERROR) { std::fprintf(stderr, "task error %#x\n", info.error); std::exit(7); }
            SleepUs(20);
        }
    };
    int64_t t_begin = 0, t_frozen = 0;
    uint64_t submitted = 0, counted_from = 0, frozen_at = 0;
    int marks_seen = 0;
    const int64_t t_start = NowNs();
    while (!g_stop.load()) {
        const int marks = g_marks.load();
        if (marks != marks_seen && t_begin) {
            if (marks_seen == 0) { counted_from = submitted; t_begin = NowNs(); }               // window opens
            if (marks >= 2 && !t_frozen) { frozen_at = submitted; t_frozen = NowNs(); }        // window closes
            marks_seen = marks;
        }
        const double el = (NowNs() - t_start) / 1e9;
        if (t_begin == 0 && el >= a.warmup_s) {
            XK(XQueueWaitAll(q.xq));
            counted_from = submitted;
            t_begin = NowNs();
            if (ready) ready->store(true);
            std::printf("READY\n"); std::fflush(stdout);
        }
        if (t_begin && (NowNs() - t_begin) / 1e9 >= duration_s) break;
        const size_t slot = submitted % depth;
        wait_slot(slot);
        if (g_stop.load()) break;
        submit(slot);
        unchecked[slot] = true;
        ++uses[slot];
        ++submitted;
    }
    XK(XQueueWaitAll(q.xq));
    r.seconds = t_begin ? ((t_frozen ? t_frozen : NowNs()) - t_begin) / 1e9 : 0;
    r.iters = (t_frozen ? frozen_at : submitted) - counted_from;
    r.rate = r.seconds > 0 ? r.iters * w.work_per_iter / r.seconds : 0;
    // The iterations still unchecked (at most one per slot), then a whole-buffer hash of the newest output.
    const size_t last = submitted ? (submitted - 1) % depth : 0;
    r.got = submitted ? v.Hash(w.outs[last], w.out_words, 8) : want.full;
    for (size_t i = 0; i < depth; ++i) check_slot(i);
    for (auto t : w.tasks) { xpkTaskInfo info; PK(xpkTaskQuery(t, &info)); r.preemptions += info.preemptions; }
    CudaQueueGetStats(q.hwq, &r.stats);
    return r;
}
static bool LpOk(const LpResult &r) { return r.want == r.got && r.mismatched_iters == 0; }

static void PrintLp(const Args &a, const LpWork &w, const LpResult &r) {
    const double scale = std::strcmp(w.unit, "TFLOP/s") == 0 ? 1e12 : 1e9;
    std::printf("{\"role\": \"lp\", \"kernel\": \"%s\", \"level\": %d, \"iters\": %" PRIu64 ", \"seconds\": %.4f, \"rate\": %.3f, \"unit\": \"%s\", "
                "\"bit_exact\": %s, \"checksum\": \"%llx\", \"verified_iters\": %" PRIu64 ", \"verified_preempted_iters\": %" PRIu64 ", \"mismatched_iters\": %" PRIu64 ", "
                "\"deactivations\": %" PRIu64 ", \"relaunches\": %" PRIu64 ", \"launched\": %" PRIu64 ", \"xpk_launches\": %" PRIu64 "}\n",
                a.kernel.c_str(), a.level, r.iters, r.seconds, r.rate / scale, w.unit, LpOk(r) ? "true" : "false", r.got,
                r.verified_iters, r.verified_preempted_iters, r.mismatched_iters,
                (uint64_t)r.stats.deactivations, (uint64_t)r.stats.relaunches, (uint64_t)r.stats.launched, (uint64_t)xpkLaunchCount());
    std::fflush(stdout);
}

// ---- high-priority workload -----------------------------------------------------------------------
struct HpWork {
    xpkTask_t task = nullptr;
    float *a = nullptr, *b = nullptr, *c = nullptr, *ha = nullptr, *hb = nullptr, *hc = nullptr;
    int32_t *keys = nullptr, *keys0 = nullptr;
    uint64_t n = 0;
    bool e2e = false;
    cudaStream_t stream = nullptr;
    double bytes_algo = 0;
};

static XResult HpCopyIn(HwQueueHandle hwq, void *data) {
    HpWork *w = (HpWork *)data;
    cudaStream_t s = (cudaStream_t)(uintptr_t)hwq;
    return cudaMemcpyAsync(w->keys, w->keys0, w->n * 4, cudaMemcpyDeviceToDevice, s) == cudaSuccess ? kXSchedSuccess : kXSchedErrorHardware;
}
static HpWork BuildHp(const Args &a, const Queue &q) {
    HpWork w;
    w.n = a.hp_n; w.e2e = a.e2e != 0; w.stream = q.stream;
    if (a.hp_kernel == "vecadd") {
        CK(cudaMalloc(&w.a, w.n * 4)); CK(cudaMalloc(&w.b, w.n * 4)); CK(cudaMalloc(&w.c, w.n * 4));
        FillUniform<<<1184, 256, 0, q.stream>>>(w.a, w.n, a.seed + 100);
        FillUniform<<<1184, 256, 0, q.stream>>>(w.b, w.n, a.seed + 101);
        if (w.e2e) {
            CK(cudaMallocHost(&w.ha, w.n * 4)); CK(cudaMallocHost(&w.hb, w.n * 4)); CK(cudaMallocHost(&w.hc, w.n * 4));
            CK(cudaMemcpyAsync(w.ha, w.a, w.n * 4, cudaMemcpyDeviceToHost, q.stream));
            CK(cudaMemcpyAsync(w.hb, w.b, w.n * 4, cudaMemcpyDeviceToHost, q.stream));
        }
        CK(cudaStreamSynchronize(q.stream));
        // The high-priority kernel is the non-preemptible form: nothing ever needs to stop it.
        PK(xpkTaskCreateVecAdd(&w.task, w.c, w.a, w.b, w.n, 0, XPK_FLAG_NON_PREEMPTIBLE, nullptr));
        w.bytes_algo = 12.0 * w.n;
    } else if (a.hp_kernel == "sort") {
        int32_t *tmp; void *scratch;
        CK(cudaMalloc(&w.keys, w.n * 4)); CK(cudaMalloc(&w.keys0, w.n * 4)); CK(cudaMalloc(&tmp, w.n * 4));
        CK(cudaMalloc(&scratch, xpkSortScratchBytes(w.n)));
        FillKeys<<<1184, 256, 0, q.stream>>>(w.keys0, w.n, a.seed + 5);
        CK(cudaStreamSynchronize(q.stream));
        PK(xpkTaskCreateSort(&w.task, w.keys, tmp, scratch, w.n, XPK_FLAG_NON_PREEMPTIBLE, nullptr));
        w.bytes_algo = 36.0 * w.n;
    } else {
        std::fprintf(stderr, "unknown --hp-kernel %s\n", a.hp_kernel.c_str());
        std::exit(2);
    }
    return w;
}

static double HpOnce(const Queue &q, HpWork &w, uint64_t index = 0) {
    const bool trace = XTraceEnabled() != 0;
    if (trace) XTraceStamp(xsched::utils::kTraceAppSubmit, index, 0);
    const int64_t t0 = NowNs();
    HwCommandHandle c;
    if (w.keys) { XK(HwCommandCreateCallback(&c, HpCopyIn, &w)); XK(XQueueSubmit(q.xq, c)); }       // the sort's unsorted input (device to device)
    else if (w.e2e) {
        // The request's inputs from pinned host memory, as copy commands of the CUDA backend: they carry the
        // transfer-only property, which XSCHED_TRANSFER_AWARE_READY=ON uses to leave lower priorities running
        // until the kernel is about to start.
        XK(CudaMemcpyCommandCreate(&c, w.a, w.ha, w.n * 4, 0)); XK(XQueueSubmit(q.xq, c));
        XK(CudaMemcpyCommandCreate(&c, w.b, w.hb, w.n * 4, 0)); XK(XQueueSubmit(q.xq, c));
    }
    XK(CudaXpkCommandCreate(&c, w.task, 1));
    XK(XQueueSubmit(q.xq, c));
    if (w.e2e && !w.keys) { XK(CudaMemcpyCommandCreate(&c, w.hc, w.c, w.n * 4, 1)); XK(XQueueSubmit(q.xq, c)); }
    XK(XQueueWaitAll(q.xq));
    const double us = (NowNs() - t0) / 1e3;
    if (trace) {
        XTraceStamp(xsched::utils::kTraceAppDone, index, 0);
        uint64_t start_ns = 0, exit_ns = 0;
        if (xpkTaskTimes(w.task, &start_ns, &exit_ns) == XPK_SUCCESS) XTraceStamp(xsched::utils::kTraceAppGpuTimes, start_ns, exit_ns);
    }
    return us;
}

struct HpResult { std::vector<double> lat_us; double seconds = 0; };

static HpResult RunHp(const Args &a, const Queue &q, HpWork &w, int count, std::atomic<bool> *stop_early) {
    HpResult r;
    for (int i = 0; i < 5; ++i) HpOnce(q, w);                 // warm-up
    std::mt19937_64 rng(a.seed);
    std::exponential_distribution<double> gap(1e6 / (double)a.period_us);
    const int64_t t_begin = NowNs();
    int64_t next = t_begin;
    for (int i = 0; i < count && !g_stop.load() && !(stop_early && stop_early->load()); ++i) {
        next += a.poisson ? (int64_t)(gap(rng) * 1e9) : a.period_us * 1000;
        while (NowNs() < next) {
            const int64_t left = next - NowNs();
            if (left > 200000) SleepUs(left / 2000); else std::this_thread::yield();
        }
        r.lat_us.push_back(HpOnce(q, w, (uint64_t)i + 1));
        if (NowNs() > next + a.period_us * 1000) next = NowNs();      // overrun: do not accumulate a backlog
    }
    r.seconds = (NowNs() - t_begin) / 1e9;
    return r;
}

static void PrintHp(const Args &a, const HpWork &w, const HpResult &r, bool verify_ok) {
    std::printf("{\"role\": \"hp\", \"kernel\": \"%s\", \"n\": %zu, \"e2e\": %d, \"p50_us\": %.2f, \"p90_us\": %.2f, \"p99_us\": %.2f, \"max_us\": %.2f, "
                "\"mean_us\": %.2f, \"seconds\": %.3f, \"verified\": %s, \"h2d_bytes\": %.0f, \"d2h_bytes\": %.0f, \"xpk_launches\": %" PRIu64 "}\n",
                a.hp_kernel.c_str(), r.lat_us.size(), a.e2e, Pct(r.lat_us, 0.5), Pct(r.lat_us, 0.9), Pct(r.lat_us, 0.99), Pct(r.lat_us, 1.0),
                r.lat_us.empty() ? 0.0 : std::accumulate(r.lat_us.begin(), r.lat_us.end(), 0.0) / r.lat_us.size(), r.seconds,
                verify_ok ? "true" : "false", (w.e2e && !w.keys) ? 8.0 * w.n : 0.0, (w.e2e && !w.keys) ? 4.0 * w.n : 0.0, (uint64_t)xpkLaunchCount());
    std::fflush(stdout);
    if (!a.samples_path.empty()) {
        if (FILE *f = std::fopen(a.samples_path.c_str(), "w")) {
            for (double v : r.lat_us) std::fprintf(f, "%.2f\n", v);
            std::fclose(f);
        }
    }
}

static bool VerifyHp(const Queue &q, HpWork &w) {
    if (w.keys) {               // sorted and same multiset size; exact content is covered by the parity tests
        std::vector<int32_t> h(std::min<uint64_t>(w.n, 1 << 20));
        CK(cudaMemcpy(h.data(), w.keys, h.size() * 4, cudaMemcpyDeviceToHost));
        return std::is_sorted(h.begin(), h.end());
    }
    std::vector<float> ha(4096), hb(4096), hc(4096);
    const uint64_t off = w.n > 8192 ? w.n / 2 : 0;
    const size_t cnt = (size_t)std::min<uint64_t>(4096, w.n - off);
    CK(cudaMemcpy(ha.data(), w.a + off, cnt * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(hb.data(), w.b + off, cnt * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(hc.data(), w.c + off, cnt * 4, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < cnt; ++i) if (hc[i] != ha[i] + hb[i]) return false;
    (void)q;
    return true;
}

// ---- preemption latency (reference experiment) ----------------------------------------------------
static int PreemptLatency(const Args &a) {
    Queue q = MakeQueue(a, a.level, 0);
    Args la = a;
    LpWork w = BuildLp(la, q, 0);
    Verifier v;
    v.Init();
    const LpExpect want = StraightRun(q, w, v);
    for (void *o : w.outs) if (!w.keys) v.Poison(o, w.out_words, w.sample_stride_words);
    std::atomic<bool> stop{false};
    std::atomic<uint64_t> rounds_checked{0}, mismatches{0}, preempted_checked{0};
    std::thread bg([&] {
        CK(cudaSetDevice(a.device));
        size_t i = 0;
        const size_t depth = w.tasks.size();
        std::vector<uint64_t> preempt_seen(depth, 0);
        // Rounds of `depth` submissions; after each round every output is compared with the straight run's
        // (each was spoiled before the round) and spoiled again.
        auto check_round = [&](size_t used) {
            for (size_t sl = 0; sl < used; ++sl) {
                xpkTaskInfo info;
                PK(xpkTaskQuery(w.tasks[sl], &info));
                if (info.preemptions != preempt_seen[sl]) preempted_checked.fetch_add(1);
                preempt_seen[sl] = info.preemptions;
                const bool tamper = a.tamper_at >= 0 && rounds_checked.load() == (uint64_t)a.tamper_at && sl == 0;
                if (!CheckSlot(w, v, sl, want, tamper)) mismatches.fetch_add(1);
            }
            rounds_checked.fetch_add(1);
        };
        while (!stop.load()) {
            if (i && i % depth == 0) { XK(XQueueWaitAll(q.xq)); check_round(depth); }
            if (w.keys) { HwCommandHandle c; XK(HwCommandCreateCallback(&c, RestoreKeys, &w)); XK(XQueueSubmit(q.xq, c)); }
            HwCommandHandle c;
            XK(CudaXpkCommandCreate(&c, w.tasks[i % depth], 1));
            XK(XQueueSubmit(q.xq, c));
            ++i;
        }
        XK(XQueueWaitAll(q.xq));
        check_round(i % depth == 0 ? depth : i % depth);
    });
    SleepUs(300000);
    std::mt19937 rng((unsigned)a.seed);
    std::vector<double> pre, res;
    for (int i = 0; i < a.count; ++i) {
        SleepUs(rng() % 800);
        int64_t t0 = NowNs();
        XK(XQueueSuspend(q.xq, kQueueSuspendFlagSyncHwQueue));
        pre.push_back((NowNs() - t0) / 1e3);
        SleepUs(800 + rng() % 800);
        t0 = NowNs();
        XK(XQueueResume(q.xq, kQueueResumeFlagNone));
        res.push_back((NowNs() - t0) / 1e3);
    }
    stop.store(true);
    bg.join();
    CudaQueueStats st{};
    CudaQueueGetStats(q.hwq, &st);
    const bool ok = mismatches.load() == 0 && rounds_checked.load() > 0;
    std::printf("{\"role\": \"preempt-latency\", \"kernel\": \"%s\", \"level\": %d, \"abort\": %d, \"n\": %zu, \"preempt_avg_us\": %.2f, \"preempt_p50_us\": %.2f, "
                "\"preempt_p95_us\": %.2f, \"preempt_p99_us\": %.2f, \"preempt_max_us\": %.2f, \"resume_avg_us\": %.2f, \"resume_p99_us\": %.2f, "
                "\"bit_exact\": %s, \"rounds_checked\": %" PRIu64 ", \"preempted_outputs_checked\": %" PRIu64 ", \"mismatched_outputs\": %" PRIu64 ", "
                "\"deactivations\": %" PRIu64 ", \"relaunches\": %" PRIu64 ", \"xpk_launches\": %" PRIu64 "}\n",
                a.kernel.c_str(), a.level, a.abort_inflight, pre.size(), std::accumulate(pre.begin(), pre.end(), 0.0) / std::max<size_t>(1, pre.size()),
                Pct(pre, 0.5), Pct(pre, 0.95), Pct(pre, 0.99), Pct(pre, 1.0), std::accumulate(res.begin(), res.end(), 0.0) / std::max<size_t>(1, res.size()),
                Pct(res, 0.99), ok ? "true" : "false", rounds_checked.load(), preempted_checked.load(), mismatches.load(),
                (uint64_t)st.deactivations, (uint64_t)st.relaunches, (uint64_t)xpkLaunchCount());
    return ok ? 0 : 6;
}

#include <numeric>

// ---- the reference's level-1 latency sweep ------------------------------------------------------------
// Same experiment as the reference's platforms/cuda/test/main/level.cu:37-176 at preemption level 1: a
// background thread keeps rounds of 64 `Sleep<<<64,64>>>` kernels of a fixed duration going through an
// XQueue with launch configuration (8, 4); the main thread times `count` XQueueSuspend(SyncHwQueue) /
// XQueueResume pairs at random moments.  At level 1 a suspension waits for the kernels already handed to
// the driver, so the latency is about (commands in flight) x (kernel duration).
__global__ void SleepKernel(long long ns) {
    long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while (true) {
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 >= ns) break;
    }
}
static XResult LaunchSleep(HwQueueHandle hwq, void *data) {
    SleepKernel<<<64, 64, 0, (cudaStream_t)(uintptr_t)hwq>>>((long long)(intptr_t)data * 1000);
    return cudaGetLastError() == cudaSuccess ? kXSchedSuccess : kXSchedErrorHardware;
}
static int LevelSweep(const Args &a) {
    Args qa = a;
    qa.threshold = 8; qa.batch = 4;
    Queue q = MakeQueue(qa, kPreemptLevelBlock, 0);
    std::printf("{\"role\": \"level-sweep\", \"level\": 1, \"launch_config\": [8, 4], \"pairs\": %d, \"sweep\": [", a.count);
    bool first = true;
    for (int64_t us : {10, 30, 90, 100, 500, 1000, 2000}) {
        std::atomic<bool> stop{false};
        std::thread bg([&] {
            CK(cudaSetDevice(a.device));
            while (!stop.load()) {
                for (int i = 0; i < 64; ++i) {
                    HwCommandHandle c;
                    XK(HwCommandCreateCallback(&c, LaunchSleep, (void *)(intptr_t)us));
                    XK(XQueueSubmit(q.xq, c));
                }
                XK(XQueueWaitAll(q.xq));
            }
        });
        SleepUs(50000);
        std::mt19937 rng((unsigned)a.seed);
        std::vector<double> pre;
        for (int i = 0; i < a.count; ++i) {
            SleepUs(rng() % (2 * us + 200));
            const int64_t t0 = NowNs();
            XK(XQueueSuspend(q.xq, kQueueSuspendFlagSyncHwQueue));
            pre.push_back((NowNs() - t0) / 1e3);
            SleepUs(200 + rng() % 300);
            XK(XQueueResume(q.xq, kQueueResumeFlagNone));
        }
        stop.store(true);
        bg.join();
        std::printf("%s{\"kernel_us\": %lld, \"avg_us\": %.1f, \"p50_us\": %.1f, \"p95_us\": %.1f, \"p99_us\": %.1f}", first ? "" : ", ", (long long)us,
                    std::accumulate(pre.begin(), pre.end(), 0.0) / std::max<size_t>(1, pre.size()), Pct(pre, 0.5), Pct(pre, 0.95), Pct(pre, 0.99));
        first = false;
    }
    std::printf("]}\n");
    return 0;
}

// ---- baseline without XSched: native CUDA stream priorities, one process, two streams ----------------
// LP: the non-preemptible twin of the low-priority kernel back-to-back on a least-priority stream (two
// launches kept in flight); HP: the high-priority kernel every period on a greatest-priority stream.
static int NativePriority(const Args &a) {
    int lo = 0, hi = 0;
    CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    Queue ql, qh;                       // plain streams, no XQueue
    CK(cudaStreamCreateWithPriority(&ql.stream, cudaStreamNonBlocking, lo));
    CK(cudaStreamCreateWithPriority(&qh.stream, cudaStreamNonBlocking, hi));
    Args la = a;
    la.depth = 2;
    LpWork lw = BuildLp(la, ql, XPK_FLAG_NON_PREEMPTIBLE);
    HpWork hw = BuildHp(a, qh);
    auto hp_once = [&]() {
        const int64_t t0 = NowNs();
        PK(xpkTaskReset(hw.task, qh.stream));
        PK(xpkTaskLaunch(hw.task, qh.stream, 0));
        CK(cudaStreamSynchronize(qh.stream));
        return (NowNs() - t0) / 1e3;
    };
    std::vector<double> alone;
    for (int i = 0; i < 5; ++i) hp_once();
    for (int i = 0; i < 100; ++i) { alone.push_back(hp_once()); SleepUs(2000); }
    std::atomic<bool> stop{false};
    std::atomic<uint64_t> iters{0};
    std::thread lp([&] {
        CK(cudaSetDevice(a.device));
        cudaEvent_t ev[2];
        CK(cudaEventCreateWithFlags(&ev[0], cudaEventDisableTiming)); CK(cudaEventCreateWithFlags(&ev[1], cudaEventDisableTiming));
        uint64_t i = 0;
        while (!stop.load()) {
            if (i >= 2) CK(cudaEventSynchronize(ev[i & 1]));
            PK(xpkTaskReset(lw.tasks[i & 1], ql.stream));
            PK(xpkTaskLaunch(lw.tasks[i & 1], ql.stream, 0));
            CK(cudaEventRecord(ev[i & 1], ql.stream));
            ++i;
        }
        CK(cudaStreamSynchronize(ql.stream));
        iters.store(i);
    });
    SleepUs(300000);
    std::vector<double> lat;
    const int64_t t_begin = NowNs();
    int64_t next = t_begin;
    for (int i = 0; i < a.count; ++i) {
        next += a.period_us * 1000;
        while (NowNs() < next) { const int64_t left = next - NowNs(); if (left > 200000) SleepUs(left / 2000); else std::this_thread::yield(); }
        lat.push_back(hp_once());
    }
    stop.store(true);
    lp.join();
    std::printf("{\"role\": \"native-priority\", \"n\": %zu, \"standalone_p50_us\": %.2f, \"standalone_p99_us\": %.2f, \"p50_us\": %.2f, \"p99_us\": %.2f, "
                "\"max_us\": %.2f, \"ratio_p99\": %.3f}\n", lat.size(), Pct(alone, 0.5), Pct(alone, 0.99), Pct(lat, 0.5), Pct(lat, 0.99), Pct(lat, 1.0),
                Pct(lat, 0.99) / std::max(1.0, Pct(alone, 0.99)));
    return 0;
}

// ---- control arms: what a second process costs the high-priority one when nothing is ever preempted -------
// idle: the process owns a context, the GEMM's buffers and a level-2 queue, and never launches anything.
static int IdleContext(const Args &a) {
    Queue q = MakeQueue(a, a.level, 0);
    LpWork w = BuildLp(a, q, 0);
    (void)w;
    std::printf("READY\n"); std::fflush(stdout);
    while (!g_stop.load()) SleepUs(2000);
    std::printf("{\"role\": \"idle\"}\n");
    return 0;
}
// spin-lp: sleep kernels of --kernel-us, two in flight, on a plain stream outside XSched.
static int SpinLp(const Args &a) {
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaEvent_t ev[2];
    CK(cudaEventCreateWithFlags(&ev[0], cudaEventDisableTiming)); CK(cudaEventCreateWithFlags(&ev[1], cudaEventDisableTiming));
    std::printf("READY\n"); std::fflush(stdout);
    uint64_t i = 0;
    const int64_t t0 = NowNs();
    while (!g_stop.load()) {
        if (i >= 2) CK(cudaEventSynchronize(ev[i & 1]));
        SleepKernel<<<64, 64, 0, s>>>((long long)a.kernel_us * 1000);
        CK(cudaEventRecord(ev[i & 1], s));
        ++i;
    }
    CK(cudaStreamSynchronize(s));
    std::printf("{\"role\": \"spin-lp\", \"kernel_us\": %lld, \"kernels\": %" PRIu64 ", \"seconds\": %.3f}\n", (long long)a.kernel_us, i, (NowNs() - t0) / 1e9);
    return 0;
}

int main(int argc, char **argv) {
    Args a = Parse(argc, argv);
    std::signal(SIGUSR1, OnMark);
    std::signal(SIGTERM, OnTerm);
    std::signal(SIGINT, OnTerm);
    CK(cudaSetDevice(a.device));
    CK(cudaFree(0));
    prctl(PR_SET_TIMERSLACK, 1000UL, 0, 0, 0);
    CalibrateGpuClock();
    if (a.role == "idle") return IdleContext(a);
    if (a.role == "spin-lp") return SpinLp(a);
    if (a.role == "preempt-latency") return PreemptLatency(a);
    if (a.role == "native-priority") return NativePriority(a);
    if (a.role == "level-sweep") return LevelSweep(a);
    if (a.role == "lp") {
        Queue q = MakeQueue(a, a.level, a.prio);
        LpWork w = BuildLp(a, q, 0);
        LpResult r = RunLp(a, q, w, nullptr, a.duration_s);
        CalibrateGpuClock();          // a second reading: the two clocks drift by tens of microseconds per second
        PrintLp(a, w, r);
        return LpOk(r) ? 0 : 6;
    }
    if (a.role == "hp") {
        Queue q = MakeQueue(a, a.level, a.prio);
        HpWork w = BuildHp(a, q);
        std::printf("READY\n"); std::fflush(stdout);
        HpResult r = RunHp(a, q, w, a.count, nullptr);
        std::printf("DONE\n"); std::fflush(stdout);              // requests are over; what follows is verification
        CalibrateGpuClock();
        PrintHp(a, w, r, VerifyHp(q, w));
        return 0;
    }
    if (a.role == "both") {
        XK(XHintSetScheduler(kSchedulerLocal, a.laxity_us >= 0 ? kPolicyLaxity : kPolicyHighestPriorityFirst));
        Queue ql = MakeQueue(a, a.level, 0), qh = MakeQueue(a, a.level, 1);
        LpWork lw = BuildLp(a, ql, 0);
        HpWork hw = BuildHp(a, qh);
        std::atomic<bool> ready{false}, lp_done{false};
        LpResult lr;
        std::thread lp([&] { CK(cudaSetDevice(a.device)); lr = RunLp(a, ql, lw, &ready, a.duration_s); lp_done.store(true); });
        while (!ready.load()) SleepUs(1000);
        HpResult hr = RunHp(a, qh, hw, a.count, &lp_done);
        g_stop.store(true);
        lp.join();
        PrintHp(a, hw, hr, VerifyHp(qh, hw));
        PrintLp(a, lw, lr);
        return LpOk(lr) ? 0 : 6;
    }
    std::fprintf(stderr, "unknown --role %s\n", a.role.c_str());
    return 2;
}
