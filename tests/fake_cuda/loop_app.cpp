// loop_app — TEST INFRASTRUCTURE: an XSched-unaware driver-API program for multi-process tests on the fake
// driver.  --role lp: one stream, back-to-back 300 us "kernels" until SIGTERM; every kernel appends its start
// time (microseconds since the epoch) to --log.  --role hp: `count` requests, each a burst of 40 such kernels
// followed by cuStreamSynchronize; request intervals go to --log.  Prints READY when warmed up.
#include <cuda.h>

#include <atomic>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include <dlfcn.h>

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); return 1; } } while (0)
using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);
static int64_t EpochUs() { return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::system_clock::now().time_since_epoch()).count(); }
static std::mutex g_mu;
static std::vector<int64_t> g_starts;
static void Busy(void **p, unsigned, unsigned) {
    const int us = *(int *)p[0];
    const int64_t t0 = EpochUs();
    { std::lock_guard<std::mutex> lk(g_mu); g_starts.push_back(t0); }
    // sleeps rather than spins: several of these programs plus a polling server share a small test host
    std::this_thread::sleep_for(std::chrono::microseconds(us));
}
static std::atomic<bool> g_stop{false};
static void OnTerm(int) { g_stop.store(true); }

int main(int argc, char **argv) {
    std::string role = "lp", log;
    int count = 5;
    for (int i = 1; i + 1 < argc; i += 2) {
        if (!std::strcmp(argv[i], "--role")) role = argv[i + 1];
        else if (!std::strcmp(argv[i], "--log")) log = argv[i + 1];
        else if (!std::strcmp(argv[i], "--count")) count = std::atoi(argv[i + 1]);
    }
    std::signal(SIGTERM, OnTerm);
    const char *fake = std::getenv("FAKE_CUDA_LIB");
    void *h = fake ? dlopen(fake, RTLD_NOW) : nullptr;
    RegisterFn reg = h ? (RegisterFn)dlsym(h, "fakeRegisterFunction") : nullptr;
    if (!reg) { std::printf("FAIL FAKE_CUDA_LIB must name libcuda_fake.so\n"); return 1; }
    const size_t sizes[] = {4};
    CUfunction busy = reg(Busy, sizes, 1);
    CK(cuInit(0));
    CUdevice dev; CK(cuDeviceGet(&dev, 0));
    CUcontext ctx; CK(cuDevicePrimaryCtxRetain(&ctx, dev)); CK(cuCtxSetCurrent(ctx));
    CUstream s; CK(cuStreamCreate(&s, CU_STREAM_NON_BLOCKING));
    int us = 300;
    void *args[] = {&us};
    FILE *f = log.empty() ? nullptr : std::fopen(log.c_str(), "w");
    if (role == "lp") {
        CUevent ev[4];
        for (auto &e : ev) CK(cuEventCreate(&e, CU_EVENT_DISABLE_TIMING));
        std::printf("READY\n"); std::fflush(stdout);
        for (uint64_t i = 0; !g_stop.load(); ++i) {
            if (i >= 4) CK(cuEventSynchronize(ev[i & 3]));              // at most four kernels ahead of the GPU
            CK(cuLaunchKernel(busy, 1, 1, 1, 1, 1, 1, 0, s, args, nullptr));
            CK(cuEventRecord(ev[i & 3], s));
        }
        CK(cuStreamSynchronize(s));
        if (f) { std::lock_guard<std::mutex> lk(g_mu); for (int64_t t : g_starts) std::fprintf(f, "%lld\n", (long long)t); }
    } else {
        CK(cuLaunchKernel(busy, 1, 1, 1, 1, 1, 1, 0, s, args, nullptr));
        CK(cuStreamSynchronize(s));
        std::printf("READY\n"); std::fflush(stdout);
        for (int r = 0; r < count; ++r) {
            std::this_thread::sleep_for(std::chrono::milliseconds(25));
            const int64_t t0 = EpochUs();
            for (int k = 0; k < 40; ++k) CK(cuLaunchKernel(busy, 1, 1, 1, 1, 1, 1, 0, s, args, nullptr));
            CK(cuStreamSynchronize(s));
            if (f) std::fprintf(f, "%lld %lld\n", (long long)t0, (long long)EpochUs());
        }
    }
    if (f) std::fclose(f);
    std::printf("DONE\n");
    return 0;
}
