// ptds_app — TEST INFRASTRUCTURE: a driver-API program that works on the per-thread default stream, the two ways a
// program built with `--default-stream per-thread` does: CU_STREAM_PER_THREAD passed to the ordinary entry points,
// and the NULL stream passed to `_ptsz` entry points obtained through cuGetProcAddress with
// CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM.  Several threads run the same sequence (copy in, kernel, memset of
// a guard word, kernel, copy out, synchronise) on their own default streams and check the result.
// argv[1] = threads, argv[2] = rounds.  With "single" as argv[3] the program instead creates several streams, which
// under XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS=ON must all be one stream.  Prints "OK <checksum>".
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>
#include <dlfcn.h>

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); std::exit(1); } } while (0)

using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);

// c[i] = a[i] * k + c[i]        params: int *c, const int *a, int k, int n
static void Axpy(void **p, unsigned, unsigned) {
    int *c = *(int **)p[0]; const int *a = *(const int **)p[1]; const int k = *(int *)p[2]; const int n = *(int *)p[3];
    for (int i = 0; i < n; ++i) c[i] += a[i] * k;
}

typedef CUresult (*LaunchFn)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void **, void **);
typedef CUresult (*H2DFn)(CUdeviceptr, const void *, size_t, CUstream);
typedef CUresult (*D2HFn)(void *, CUdeviceptr, size_t, CUstream);
typedef CUresult (*SyncFn)(CUstream);
typedef CUresult (*Set32Fn)(CUdeviceptr, unsigned, size_t, CUstream);

template <class F> static F Lookup(const char *name) {
    void *p = nullptr;
    CUdriverProcAddressQueryResult st;
    CK(cuGetProcAddress(name, &p, 12000, CU_GET_PROC_ADDRESS_PER_THREAD_DEFAULT_STREAM, &st));
    if (!p) { std::printf("FAIL no per-thread entry point %s\n", name); std::exit(1); }
    return (F)p;
}

int main(int argc, char **argv) {
    const int threads = argc > 1 ? std::atoi(argv[1]) : 3, rounds = argc > 2 ? std::atoi(argv[2]) : 20;
    const bool single = argc > 3 && std::strcmp(argv[3], "single") == 0;
    const int n = 1 << 10;
    const char *fake = std::getenv("FAKE_CUDA_LIB");
    void *h = fake ? dlopen(fake, RTLD_NOW) : nullptr;
    RegisterFn reg = h ? (RegisterFn)dlsym(h, "fakeRegisterFunction") : nullptr;
    if (!reg) { std::printf("FAIL FAKE_CUDA_LIB must name libcuda_fake.so\n"); return 1; }
    const size_t sizes[] = {8, 8, 4, 4};
    CUfunction f = reg(Axpy, sizes, 4);
    CK(cuInit(0));
    CUdevice dev; CK(cuDeviceGet(&dev, 0));
    CUcontext ctx; CK(cuDevicePrimaryCtxRetain(&ctx, dev));
    CK(cuCtxSetCurrent(ctx));

    if (single) {
        // Four creations, one underlying stream: handles equal, work on any of them is ordered, and the stream
        // survives until the last handle is destroyed.
        CUstream s[4];
        for (int i = 0; i < 4; ++i) CK(i & 1 ? cuStreamCreateWithPriority(&s[i], CU_STREAM_NON_BLOCKING, 0) : cuStreamCreate(&s[i], CU_STREAM_NON_BLOCKING));
        const bool same = s[0] == s[1] && s[1] == s[2] && s[2] == s[3];
        CUdeviceptr da, dc;
        CK(cuMemAlloc(&da, n * 4)); CK(cuMemAlloc(&dc, n * 4));
        std::vector<int> ha(n, 3), hc(n, 0);
        CK(cuMemcpyHtoDAsync(da, ha.data(), n * 4, s[0]));
        CK(cuMemsetD32Async(dc, 1, n, s[1]));
        for (int r = 0; r < rounds; ++r) {
            int k = r + 1, nn = n;
            void *args[] = {&dc, &da, &k, &nn};
            CK(cuLaunchKernel(f, 1, 1, 1, 1, 1, 1, 0, s[r & 3], args, nullptr));
        }
        for (int i = 0; i < 3; ++i) CK(cuStreamDestroy(s[i]));
        CK(cuMemcpyDtoHAsync(hc.data(), dc, n * 4, s[3]));
        CK(cuStreamSynchronize(s[3]));
        CK(cuStreamDestroy(s[3]));
        long long want = 1;
        for (int r = 0; r < rounds; ++r) want += 3 * (r + 1);
        for (int i = 0; i < n; ++i) if (hc[i] != want) { std::printf("FAIL element %d = %d, want %lld\n", i, hc[i], want); return 1; }
        std::printf("OK %lld same_handles=%d\n", want, same ? 1 : 0);
        return 0;
    }

    std::atomic<long long> checksum{0};
    std::atomic<int> failures{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back([&, t] {
        CK(cuCtxSetCurrent(ctx));
        const LaunchFn launch_ptsz = Lookup<LaunchFn>("cuLaunchKernel");
        const H2DFn h2d_ptsz = Lookup<H2DFn>("cuMemcpyHtoDAsync");
        const D2HFn d2h_ptsz = Lookup<D2HFn>("cuMemcpyDtoHAsync");
        const SyncFn sync_ptsz = Lookup<SyncFn>("cuStreamSynchronize");
        const Set32Fn set_ptsz = Lookup<Set32Fn>("cuMemsetD32Async");
        CUdeviceptr da, dc;
        CK(cuMemAlloc(&da, n * 4)); CK(cuMemAlloc(&dc, n * 4));
        void *pin_a, *pin_c;
        CK(cuMemHostAlloc(&pin_a, n * 4, 0)); CK(cuMemHostAlloc(&pin_c, n * 4, 0));
        int *ha = (int *)pin_a, *hc = (int *)pin_c;
        for (int r = 0; r < rounds; ++r) {
            for (int i = 0; i < n; ++i) ha[i] = t * 1000 + r + i;
            int k = r % 5 + 1, nn = n;
            void *args[] = {&dc, &da, &k, &nn};
            if (r & 1) {            // the ordinary entry points with the per-thread handle
                CK(cuMemcpyHtoDAsync(da, ha, n * 4, CU_STREAM_PER_THREAD));
                CK(cuMemsetD32Async(dc, 7, n, CU_STREAM_PER_THREAD));
                CK(cuLaunchKernel(f, 1, 1, 1, 1, 1, 1, 0, CU_STREAM_PER_THREAD, args, nullptr));
                CK(cuLaunchKernel(f, 1, 1, 1, 1, 1, 1, 0, CU_STREAM_PER_THREAD, args, nullptr));
                CK(cuMemcpyDtoHAsync(hc, dc, n * 4, CU_STREAM_PER_THREAD));
                CK(cuStreamSynchronize(CU_STREAM_PER_THREAD));
            } else {                // the _ptsz twins with the NULL stream
                CK(h2d_ptsz(da, ha, n * 4, nullptr));
                CK(set_ptsz(dc, 7, n, nullptr));
                CK(launch_ptsz(f, 1, 1, 1, 1, 1, 1, 0, nullptr, args, nullptr));
                CK(launch_ptsz(f, 1, 1, 1, 1, 1, 1, 0, nullptr, args, nullptr));
                CK(d2h_ptsz(hc, dc, n * 4, nullptr));
                CK(sync_ptsz(nullptr));
            }
            for (int i = 0; i < n; ++i) {
                const int want = 7 + 2 * k * ha[i];
                if (hc[i] != want) { failures.fetch_add(1); break; }
                checksum.fetch_add(hc[i]);
            }
        }
        CK(cuMemFree(da)); CK(cuMemFree(dc));
    });
    for (auto &th : pool) th.join();
    if (failures.load()) { std::printf("FAIL %d rounds produced wrong data\n", failures.load()); return 1; }
    std::printf("OK %lld\n", checksum.load());
    return 0;
}
