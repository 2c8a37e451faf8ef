// transfer_app — TEST INFRASTRUCTURE: requests of the shape "copy the inputs in, run one kernel, copy the result out"
// on a high-priority XQueue, next to a low-priority queue that is kept full of 500 us kernels, under the
// in-process HPF scheduler on the fake driver.  The copies are CudaMemcpyCommandCreate commands over 96 MiB of
// pinned memory each (tens of milliseconds on the fake driver's stream thread), the kernel takes 3 ms.
// Prints how long the low-priority queue's kernels were kept off the "device" in total: with
// XSCHED_TRANSFER_AWARE_READY=ON that is a little more than the kernels' time, without it the copies count too.
#include <cuda.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>
#include <dlfcn.h>
#include "xsched/xsched.h"
#include "xsched/cuda/hal.h"

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)
#define XK(x) do { XResult r_ = (x); if (r_ != kXSchedSuccess) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)

using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);
static int64_t NowUs() { return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static std::atomic<int64_t> g_lp_last_end{0}, g_lp_gap_us{0}, g_hp_kernel_us{0};
static std::atomic<long> g_lp_ran{0};
// params: int microseconds, int is_lp.  Low-priority kernels account for the time between two of them.
static void Busy(void **p, unsigned, unsigned) {
    const int us = *(int *)p[0], is_lp = *(int *)p[1];
    const int64_t t0 = NowUs();
    if (is_lp) {
        const int64_t last = g_lp_last_end.load();
        if (last && t0 - last > 1000) g_lp_gap_us.fetch_add(t0 - last);       // gaps above 1 ms: the queue was held back
    }
    while (NowUs() - t0 < us) {}
    if (is_lp) { g_lp_last_end.store(NowUs()); g_lp_ran.fetch_add(1); } else g_hp_kernel_us.fetch_add(us);
}
static CUfunction g_busy;
struct LaunchArg { int us, is_lp; };
static XResult LaunchBusy(HwQueueHandle hwq, void *data) {
    LaunchArg a = *(LaunchArg *)data;
    void *args[] = {&a.us, &a.is_lp};
    return cuLaunchKernel(g_busy, 1, 1, 1, 1, 1, 1, 0, (CUstream)(uintptr_t)hwq, args, nullptr) == CUDA_SUCCESS ? kXSchedSuccess : kXSchedErrorHardware;
}

int main(int argc, char **argv) {
    const int requests = argc > 1 ? std::atoi(argv[1]) : 4;
    const size_t bytes = 96u << 20;
    const char *fake = std::getenv("FAKE_CUDA_LIB");
    void *h = fake ? dlopen(fake, RTLD_NOW) : nullptr;
    RegisterFn reg = h ? (RegisterFn)dlsym(h, "fakeRegisterFunction") : nullptr;
    if (!reg) { std::printf("FAIL FAKE_CUDA_LIB must name libcuda_fake.so\n"); return 1; }
    const size_t sizes[] = {4, 4};
    g_busy = reg(Busy, sizes, 2);
    CK(cuInit(0));
    CUdevice dev; CK(cuDeviceGet(&dev, 0));
    CUcontext ctx; CK(cuDevicePrimaryCtxRetain(&ctx, dev)); CK(cuCtxSetCurrent(ctx));
    XK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    CUstream s_lp, s_hp;
    CK(cuStreamCreate(&s_lp, CU_STREAM_NON_BLOCKING)); CK(cuStreamCreate(&s_hp, CU_STREAM_NON_BLOCKING));
    HwQueueHandle hq_lp, hq_hp; XQueueHandle lp, hp;
    XK(CudaQueueCreate(&hq_lp, s_lp)); XK(CudaQueueCreate(&hq_hp, s_hp));
    XK(XQueueCreate(&lp, hq_lp, kPreemptLevelBlock, kQueueCreateFlagNone)); XK(XQueueCreate(&hp, hq_hp, kPreemptLevelBlock, kQueueCreateFlagNone));
    XK(XQueueSetLaunchConfig(lp, 2, 1)); XK(XQueueSetLaunchConfig(hp, 8, 4));
    XK(XHintPriority(lp, 0)); XK(XHintPriority(hp, 1));
    void *hin, *hout; CUdeviceptr din, dout;
    CK(cuMemHostAlloc(&hin, bytes, 0)); CK(cuMemHostAlloc(&hout, bytes, 0));
    CK(cuMemAlloc(&din, bytes)); CK(cuMemAlloc(&dout, bytes));
    std::memset(hin, 7, bytes);

    static LaunchArg lp_arg{500, 1}, hp_arg{3000, 0};
    std::atomic<bool> stop{false};
    std::thread lp_thread([&] {
        cuCtxSetCurrent(ctx);
        while (!stop.load()) {
            for (int i = 0; i < 8; ++i) { HwCommandHandle c; XK(HwCommandCreateCallback(&c, LaunchBusy, &lp_arg)); XK(XQueueSubmit(lp, c)); }
            XK(XQueueWaitAll(lp));
        }
    });
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
    const int64_t t_begin = NowUs();
    g_lp_gap_us.store(0);
    for (int r = 0; r < requests; ++r) {
        HwCommandHandle c;
        XK(CudaMemcpyCommandCreate(&c, (void *)(uintptr_t)din, hin, bytes, 0)); XK(XQueueSubmit(hp, c));
        XK(HwCommandCreateCallback(&c, LaunchBusy, &hp_arg)); XK(XQueueSubmit(hp, c));
        XK(CudaMemcpyCommandCreate(&c, hout, (void *)(uintptr_t)din, bytes, 1)); XK(XQueueSubmit(hp, c));
        XK(XQueueWaitAll(hp));
        if (((unsigned char *)hout)[bytes - 1] != 7) { std::printf("FAIL request %d: wrong data\n", r); return 1; }
        std::memset(hout, 0, 64);
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    const int64_t elapsed = NowUs() - t_begin;
    stop.store(true);
    lp_thread.join();
    std::printf("{\"requests\": %d, \"elapsed_us\": %lld, \"lp_held_back_us\": %lld, \"hp_kernel_us\": %lld, \"lp_kernels\": %ld}\n", requests, (long long)elapsed,
                (long long)g_lp_gap_us.load(), (long long)g_hp_kernel_us.load(), g_lp_ran.load());
    XK(XQueueDestroy(lp)); XK(XQueueDestroy(hp));
    return 0;
}
