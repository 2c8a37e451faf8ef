// hal_app — TEST INFRASTRUCTURE: a program that USES XSched (XQueue C API + CudaQueueCreate) on top of the fake
// driver.  Two streams under the in-process scheduler with HPF: a low-priority stream kept full of 500 us
// "kernels" (host functions) through callback commands, a high-priority stream with one 300 us kernel per
// request.  Level 1 with launch configuration (4, 2): a request waits at most for the window to drain.
// Also times XQueueSuspend(SyncHwQueue) / XQueueResume pairs on the busy queue.  Prints one JSON line.
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

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)
#define XK(x) do { XResult r_ = (x); if (r_ != kXSchedSuccess) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)

using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);
static int64_t NowUs() { return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static std::atomic<long> g_ran{0};
static void Busy(void **p, unsigned, unsigned) {            // params: int microseconds
    const int us = *(int *)p[0];
    const int64_t t0 = NowUs();
    while (NowUs() - t0 < us) {}
    g_ran.fetch_add(1);
}
static CUfunction g_busy;
struct LaunchArg { int us; };
static XResult LaunchBusy(HwQueueHandle hwq, void *data) {
    int us = ((LaunchArg *)data)->us;
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
    XK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    CUstream s_lp, s_hp;
    CK(cuStreamCreate(&s_lp, CU_STREAM_NON_BLOCKING)); CK(cuStreamCreate(&s_hp, CU_STREAM_NON_BLOCKING));
    HwQueueHandle hq_lp, hq_hp; XQueueHandle lp, hp;
    XK(CudaQueueCreate(&hq_lp, s_lp)); XK(CudaQueueCreate(&hq_hp, s_hp));
    XK(XQueueCreate(&lp, hq_lp, kPreemptLevelBlock, kQueueCreateFlagNone)); XK(XQueueCreate(&hp, hq_hp, kPreemptLevelBlock, kQueueCreateFlagNone));
    XK(XQueueSetLaunchConfig(lp, 4, 2)); XK(XQueueSetLaunchConfig(hp, 4, 2));
    XK(XHintPriority(lp, 0)); XK(XHintPriority(hp, 1));

    static LaunchArg lp_arg{500}, hp_arg{300};
    const int lp_count = 300;
    std::thread lp_thread([&] {
        cuCtxSetCurrent(ctx);
        for (int i = 0; i < lp_count; ++i) { HwCommandHandle c; XK(HwCommandCreateCallback(&c, LaunchBusy, &lp_arg)); XK(XQueueSubmit(lp, c)); }
        XK(XQueueWaitAll(lp));
    });
    std::vector<double> lat, susp;
    for (int i = 0; i < 6; ++i) {
        std::this_thread::sleep_for(std::chrono::milliseconds(12));
        const int64_t t0 = NowUs();
        HwCommandHandle c; XK(HwCommandCreateCallback(&c, LaunchBusy, &hp_arg)); XK(XQueueSubmit(hp, c));
        XK(XQueueWaitAll(hp));
        lat.push_back((double)(NowUs() - t0));
    }
    for (int i = 0; i < 5; ++i) {
        std::this_thread::sleep_for(std::chrono::milliseconds(3));
        const int64_t t0 = NowUs();
        XK(XQueueSuspend(lp, kQueueSuspendFlagSyncHwQueue));
        susp.push_back((double)(NowUs() - t0));
        const long ran_at_suspend = g_ran.load();
        std::this_thread::sleep_for(std::chrono::milliseconds(4));
        if (g_ran.load() != ran_at_suspend) { std::printf("FAIL low-priority kernels ran while suspended\n"); return 1; }
        XK(XQueueResume(lp, kQueueResumeFlagNone));
    }
    lp_thread.join();
    XK(XQueueWaitAll(hp));
    std::sort(lat.begin(), lat.end()); std::sort(susp.begin(), susp.end());
    std::printf("{\"hp_max_us\": %.0f, \"hp_min_us\": %.0f, \"suspend_max_us\": %.0f, \"ran\": %ld, \"expected\": %d}\n", lat.back(), lat.front(), susp.back(),
                g_ran.load(), lp_count + 6);
    XK(XQueueDestroy(lp)); XK(XQueueDestroy(hp));
    XK(HwQueueDestroy(hq_lp)); XK(HwQueueDestroy(hq_hp));
    CK(cuStreamDestroy(s_lp)); CK(cuStreamDestroy(s_hp));
    return 0;
}
