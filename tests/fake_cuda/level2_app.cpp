// level2_app — TEST INFRASTRUCTURE: the level-2 path of the CUDA HAL on the fake driver with fake preemptible
// tasks (fake_xpk.cpp).  A low-priority XQueue (level 2, window 2/1) runs tasks of 40 tiles x 200 us in a loop
// over three task objects; a high-priority XQueue gets a 300 us kernel every 7 ms; in-process HPF.  Checks:
// every tile of every finished task ran exactly once whatever the number of preemptions, a high-priority
// request waits about one tile (not one task), and the low-priority queue makes progress.  One JSON line.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include <dlfcn.h>
#include "xsched/xsched.h"
#include "xsched/cuda/hal.h"
#include "xsched_b200/pk.h"

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)
#define XK(x) do { XResult r_ = (x); if (r_ != kXSchedSuccess) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)
extern "C" xpkTask_t fakeXpkTaskCreate(uint64_t tiles, int tile_us, uint32_t *flag);
extern "C" uint32_t fakeXpkTileRuns(xpkTask_t t, uint64_t tile);

using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);
static int64_t NowUs() { return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static void Busy(void **p, unsigned, unsigned) { std::this_thread::sleep_for(std::chrono::microseconds(*(int *)p[0])); }
static CUfunction g_busy;
static XResult LaunchBusy(HwQueueHandle hwq, void *) {
    int us = 300;
    void *args[] = {&us};
    return cuLaunchKernel(g_busy, 1, 1, 1, 1, 1, 1, 0, (CUstream)(uintptr_t)hwq, args, nullptr) == CUDA_SUCCESS ? kXSchedSuccess : kXSchedErrorHardware;
}

int main() {
    const char *fake = std::getenv("FAKE_CUDA_LIB");
    void *h = fake ? dlopen(fake, RTLD_NOW) : nullptr;
    RegisterFn reg = h ? (RegisterFn)dlsym(h, "fakeRegisterFunction") : nullptr;
    if (!reg) { std::printf("FAIL FAKE_CUDA_LIB must name libcuda_fake.so\n"); return 1; }
    const size_t sizes[] = {4};
    g_busy = reg(Busy, sizes, 1);
    CK(cuInit(0));
    CUdevice dev; CK(cuDeviceGet(&dev, 0));
    CUcontext ctx; CK(cuDevicePrimaryCtxRetain(&ctx, dev)); CK(cuCtxSetCurrent(ctx));
    // L2_LP_ONLY=1: only the low-priority loop, under whatever scheduler the environment selects (a high-priority
    // process elsewhere, one xserver); otherwise both queues in this process under the in-process HPF scheduler.
    const bool lp_only = std::getenv("L2_LP_ONLY") != nullptr;
    if (!lp_only) XK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    CUstream s_lp, s_hp;
    CK(cuStreamCreate(&s_lp, CU_STREAM_NON_BLOCKING)); CK(cuStreamCreate(&s_hp, CU_STREAM_NON_BLOCKING));
    HwQueueHandle hq_lp, hq_hp; XQueueHandle lp, hp;
    XK(CudaQueueCreate(&hq_lp, s_lp)); XK(CudaQueueCreate(&hq_hp, s_hp));
    XK(XQueueCreate(&lp, hq_lp, kPreemptLevelDeactivate, kQueueCreateFlagNone)); XK(XQueueCreate(&hp, hq_hp, kPreemptLevelDeactivate, kQueueCreateFlagNone));
    XK(XQueueSetLaunchConfig(lp, 2, 1));
    XK(XHintPriority(lp, 0)); XK(XHintPriority(hp, 1));
    uint32_t *flag = nullptr;
    XK(CudaQueueGetPreemptFlag(hq_lp, &flag));

    const uint64_t tiles = 40;
    const int tile_us = 200, depth = 3, iterations = std::getenv("L2_ITERATIONS") ? std::atoi(std::getenv("L2_ITERATIONS")) : 24;
    std::vector<xpkTask_t> tasks;
    for (int i = 0; i < depth; ++i) tasks.push_back(fakeXpkTaskCreate(tiles, tile_us, flag));
    std::atomic<int> bad_tiles{0}, finished{0};
    std::atomic<bool> lp_done{false};
    std::thread lp_thread([&] {
        cuCtxSetCurrent(ctx);
        std::vector<uint64_t> seen(depth, 0);
        for (int it = 0; it < iterations; ++it) {
            const int slot = it % depth;
            if (it >= depth) {                       // the slot's previous submission must be complete: check it, then reuse
                while (true) {
                    xpkTaskInfo info; xpkTaskQuery(tasks[slot], &info);
                    if (info.launches > seen[slot] && info.status == XPK_STATUS_COMPLETED) { seen[slot] = info.launches; break; }
                    std::this_thread::sleep_for(std::chrono::microseconds(100));
                }
                for (uint64_t t = 0; t < tiles; ++t) if (fakeXpkTileRuns(tasks[slot], t) != 1) bad_tiles.fetch_add(1);
                finished.fetch_add(1);
            }
            HwCommandHandle c; XK(CudaXpkCommandCreate(&c, tasks[slot], 1)); XK(XQueueSubmit(lp, c));
        }
        XK(XQueueWaitAll(lp));
        for (int slot = 0; slot < depth; ++slot) {
            for (uint64_t t = 0; t < tiles; ++t) if (fakeXpkTileRuns(tasks[slot], t) != 1) bad_tiles.fetch_add(1);
            finished.fetch_add(1);
        }
        lp_done.store(true);
    });
    std::vector<double> lat;
    if (lp_only) std::printf("READY\n"), std::fflush(stdout);
    while (!lp_only && !lp_done.load()) {
        std::this_thread::sleep_for(std::chrono::milliseconds(7));
        const int64_t t0 = NowUs();
        HwCommandHandle c; XK(HwCommandCreateCallback(&c, LaunchBusy, nullptr)); XK(XQueueSubmit(hp, c));
        XK(XQueueWaitAll(hp));
        lat.push_back((double)(NowUs() - t0));
    }
    lp_thread.join();
    uint64_t preemptions = 0;
    for (auto t : tasks) { xpkTaskInfo info; xpkTaskQuery(t, &info); preemptions += info.preemptions; }
    CudaQueueStats st{};
    CudaQueueGetStats(hq_lp, &st);
    std::sort(lat.begin(), lat.end());
    std::printf("{\"finished\": %d, \"expected\": %d, \"bad_tiles\": %d, \"requests\": %zu, \"hp_p50_us\": %.0f, \"hp_max_us\": %.0f, "
                "\"preemptions\": %llu, \"deactivations\": %llu, \"relaunches\": %llu}\n",
                finished.load(), iterations, bad_tiles.load(), lat.size(), lat.empty() ? 0.0 : lat[lat.size() / 2], lat.empty() ? 0.0 : lat.back(),
                (unsigned long long)preemptions, (unsigned long long)st.deactivations, (unsigned long long)st.relaunches);
    XK(XQueueDestroy(lp)); XK(XQueueDestroy(hp));
    return 0;
}
