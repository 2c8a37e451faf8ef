// driver_app — TEST INFRASTRUCTURE: an XSched-unaware program written against the CUDA driver API whose
// "kernels" are host functions registered with the fake driver (fake_cuda.cpp).  It exercises what the
// interposer has to get right without a GPU in sight:
//   * per-stream order of copies, launches, memsets and host functions;
//   * a cross-stream dependency through an event;
//   * copies from pageable host memory whose source is overwritten right after the call returns, and copies
//     into pageable memory whose destination is read right after the call returns;
//   * launch arguments that live on the caller's stack;
//   * stream / event queries and synchronisation;
//   * the legacy default stream against a blocking stream, stream capture and graph launches, destruction of
//     events and streams with work pending.
// Prints "OK <checksum>" — the same line with and without the interposer in front of the driver.
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <dlfcn.h>

#define CK(x) do { CUresult r_ = (x); if (r_ != CUDA_SUCCESS) { std::printf("FAIL %s -> %d\n", #x, (int)r_); return 1; } } while (0)

using RegisterFn = CUfunction (*)(void (*)(void **, unsigned, unsigned), const size_t *, int);

// c[i] = a[i] + b[i]        params: int *c, const int *a, const int *b, int n
static void VecAdd(void **p, unsigned, unsigned) {
    int *c = *(int **)p[0]; const int *a = *(const int **)p[1]; const int *b = *(const int **)p[2]; const int n = *(int *)p[3];
    for (int i = 0; i < n; ++i) c[i] = a[i] + b[i];
}
// c[i] *= k                 params: int *c, int k, int n
static void Scale(void **p, unsigned, unsigned) {
    int *c = *(int **)p[0]; const int k = *(int *)p[1]; const int n = *(int *)p[2];
    for (int i = 0; i < n; ++i) c[i] *= k;
}
static std::atomic<int> g_host_calls{0};
static void HostFn(void *) { g_host_calls.fetch_add(1); }

int main(int argc, char **argv) {
    const int rounds = argc > 1 ? std::atoi(argv[1]) : 30;
    const int n = 1 << 12;
    const char *fake = std::getenv("FAKE_CUDA_LIB");
    void *h = fake ? dlopen(fake, RTLD_NOW) : nullptr;
    RegisterFn reg = h ? (RegisterFn)dlsym(h, "fakeRegisterFunction") : nullptr;
    if (!reg) { std::printf("FAIL FAKE_CUDA_LIB must name libcuda_fake.so\n"); return 1; }
    const size_t add_sizes[] = {8, 8, 8, 4}, scale_sizes[] = {8, 4, 4};
    CUfunction f_add = reg(VecAdd, add_sizes, 4), f_scale = reg(Scale, scale_sizes, 3);

    CK(cuInit(0));
    CUdevice dev; CK(cuDeviceGet(&dev, 0));
    CUcontext ctx; CK(cuDevicePrimaryCtxRetain(&ctx, dev)); CK(cuCtxSetCurrent(ctx));
    CUstream s[2];
    CUdeviceptr da[2], db[2], dc[2];
    for (int k = 0; k < 2; ++k) {
        CK(cuStreamCreate(&s[k], CU_STREAM_NON_BLOCKING));
        CK(cuMemAlloc(&da[k], n * 4)); CK(cuMemAlloc(&db[k], n * 4)); CK(cuMemAlloc(&dc[k], n * 4));
    }
    CUevent ev; CK(cuEventCreate(&ev, CU_EVENT_DISABLE_TIMING));
    std::vector<int> ha(n), hb(n), hc0(n), hc1(n);           // pageable
    unsigned long long checksum = 0;
    for (int r = 0; r < rounds; ++r) {
        for (int k = 0; k < 2; ++k) {
            for (int i = 0; i < n; ++i) { ha[i] = r * 7 + i + k; hb[i] = i % 13; }
            CK(cuMemcpyHtoDAsync(da[k], ha.data(), n * 4, s[k]));
            CK(cuMemcpyHtoDAsync(db[k], hb.data(), n * 4, s[k]));
            std::fill(ha.begin(), ha.end(), -1);              // the source may be reused at once
            std::fill(hb.begin(), hb.end(), -1);
            CK(cuMemsetD32Async(dc[k], 0xdeadbeef, n, s[k]));
            int count = n;                                    // arguments on the stack, gone after the call
            void *args[] = {&dc[k], &da[k], &db[k], &count};
            CK(cuLaunchKernel(f_add, 4, 1, 1, 64, 1, 1, 0, s[k], args, nullptr));
            count = -12345;
        }
        // stream 1 scales its result only after stream 0 finished its add
        CK(cuEventRecord(ev, s[0]));
        CK(cuStreamWaitEvent(s[1], ev, 0));
        { int k3 = 3, count = n; void *args[] = {&dc[1], &k3, &count}; CK(cuLaunchKernel(f_scale, 4, 1, 1, 64, 1, 1, 0, s[1], args, nullptr)); }
        CK(cuLaunchHostFunc(s[1], HostFn, nullptr));
        CK(cuMemcpyDtoHAsync(hc0.data(), dc[0], n * 4, s[0]));   // pageable destinations: readable on return
        CK(cuMemcpyDtoHAsync(hc1.data(), dc[1], n * 4, s[1]));
        for (int i = 0; i < n; i += 97) {
            const int want0 = (r * 7 + i + 0) + i % 13, want1 = 3 * ((r * 7 + i + 1) + i % 13);
            if (hc0[i] != want0 || hc1[i] != want1) { std::printf("FAIL round %d index %d: %d %d (want %d %d)\n", r, i, hc0[i], hc1[i], want0, want1); return 1; }
            checksum = checksum * 31 + (unsigned)hc0[i] + 7u * (unsigned)hc1[i];
        }
        if (r % 5 == 0) {
            CK(cuStreamSynchronize(s[0])); CK(cuStreamSynchronize(s[1]));
            if (cuStreamQuery(s[0]) != CUDA_SUCCESS || cuEventQuery(ev) != CUDA_SUCCESS) { std::printf("FAIL queries after synchronize\n"); return 1; }
        }
    }
    // A blocking stream and the legacy default stream: work on the NULL stream is ordered after everything
    // submitted to the blocking stream before it.
    {
        CUstream sb; CK(cuStreamCreate(&sb, CU_STREAM_DEFAULT));
        CUdeviceptr x, y, z;
        CK(cuMemAlloc(&x, n * 4)); CK(cuMemAlloc(&y, n * 4)); CK(cuMemAlloc(&z, n * 4));
        for (int r = 0; r < 5; ++r) {
            CK(cuMemsetD32Async(x, (unsigned)(r + 1), n, sb));
            CK(cuMemsetD32Async(y, 10, n, sb));
            int count = n;
            void *a1[] = {&z, &x, &y, &count};
            CK(cuLaunchKernel(f_add, 4, 1, 1, 64, 1, 1, 0, sb, a1, nullptr));             // z = r + 11 on the blocking stream
            int k2 = 2;
            void *a2[] = {&z, &k2, &count};
            CK(cuLaunchKernel(f_scale, 4, 1, 1, 64, 1, 1, 0, nullptr, a2, nullptr));        // z *= 2 on the legacy stream
            CK(cuMemcpyDtoHAsync(hc0.data(), z, n * 4, nullptr));
            if (hc0[0] != 2 * (r + 11) || hc0[n - 1] != 2 * (r + 11)) { std::printf("FAIL legacy-stream order, round %d: %d\n", r, hc0[0]); return 1; }
            checksum = checksum * 31 + (unsigned)hc0[0];
        }
        CK(cuStreamSynchronize(sb));
        CK(cuMemFree(x)); CK(cuMemFree(y)); CK(cuMemFree(z)); CK(cuStreamDestroy(sb));
    }
    // Stream capture: three launches recorded into a graph (x -> 2x + 3), the graph launched between ordinary work.
    {
        CUdeviceptr v; CK(cuMemAlloc(&v, n * 4));
        CK(cuMemsetD32Async(v, 1, n, s[0]));                                               // queued before the capture
        int one_n = n, two = 2;
        CUdeviceptr ones; CK(cuMemAlloc(&ones, n * 4)); CK(cuMemsetD32Async(ones, 1, n, s[0]));
        CUgraph graph; CUgraphExec exec;
        CK(cuStreamBeginCapture(s[0], CU_STREAM_CAPTURE_MODE_THREAD_LOCAL));
        { void *a[] = {&v, &v, &ones, &one_n}; CK(cuLaunchKernel(f_add, 4, 1, 1, 64, 1, 1, 0, s[0], a, nullptr)); }      // +1
        // ending a capture on a stream that is not capturing fails and must not end the one in progress
        CUgraph wrong = nullptr;
        if (cuStreamEndCapture(s[1], &wrong) == CUDA_SUCCESS) { std::printf("FAIL ending a capture on a stream that is not capturing succeeded\n"); return 1; }
        { void *a[] = {&v, &two, &one_n}; CK(cuLaunchKernel(f_scale, 4, 1, 1, 64, 1, 1, 0, s[0], a, nullptr)); }         // *2
        { void *a[] = {&v, &v, &ones, &one_n}; CK(cuLaunchKernel(f_add, 4, 1, 1, 64, 1, 1, 0, s[0], a, nullptr)); }      // +1
        CK(cuStreamEndCapture(s[0], &graph));
        CK(cuGraphInstantiate(&exec, graph, 0));
        CK(cuMemcpyDtoHAsync(hc0.data(), v, 4, s[0]));
        if (hc0[0] != 1) { std::printf("FAIL captured work ran during the capture: %d\n", hc0[0]); return 1; }
        int expect = 1;
        for (int r = 0; r < 5; ++r) {
            CK(cuGraphLaunch(exec, s[0]));                                                   // x -> 2(x + 1) + 1
            { void *a[] = {&v, &v, &ones, &one_n}; CK(cuLaunchKernel(f_add, 4, 1, 1, 64, 1, 1, 0, s[0], a, nullptr)); }  // +1
            expect = 2 * (expect + 1) + 1 + 1;
        }
        CK(cuMemcpyDtoHAsync(hc0.data(), v, n * 4, s[0]));
        if (hc0[0] != expect || hc0[n - 1] != expect) { std::printf("FAIL graph launches: %d (want %d)\n", hc0[0], expect); return 1; }
        checksum = checksum * 31 + (unsigned)hc0[0];
        CK(cuGraphExecDestroy(exec)); CK(cuGraphDestroy(graph));
        CK(cuStreamSynchronize(s[0]));
        CK(cuMemFree(v)); CK(cuMemFree(ones));
    }
    // An event is destroyed while its record is still queued; a stream is destroyed with work pending.
    {
        CUstream st; CK(cuStreamCreate(&st, CU_STREAM_NON_BLOCKING));
        CUdeviceptr w; CK(cuMemAlloc(&w, n * 4));
        CUevent e2; CK(cuEventCreate(&e2, CU_EVENT_DISABLE_TIMING));
        for (int i = 0; i < 20; ++i) CK(cuMemsetD32Async(w, (unsigned)i, n, st));
        CK(cuEventRecord(e2, st));
        CK(cuEventDestroy(e2));
        CK(cuLaunchHostFunc(st, HostFn, nullptr));
        CK(cuStreamDestroy(st));                       // implies completion of what was submitted
        CK(cuMemcpyDtoHAsync(hc1.data(), w, 4, s[0]));
        if (hc1[0] != 19) { std::printf("FAIL work pending at stream destruction was lost: %d\n", hc1[0]); return 1; }
        CK(cuMemFree(w));
    }
    CK(cuEventSynchronize(ev));
    CK(cuCtxSynchronize());
    if (g_host_calls.load() != rounds + 1) { std::printf("FAIL host function ran %d times\n", g_host_calls.load()); return 1; }
    for (int k = 0; k < 2; ++k) { CK(cuMemFree(da[k])); CK(cuMemFree(db[k])); CK(cuMemFree(dc[k])); CK(cuStreamDestroy(s[k])); }
    CK(cuEventDestroy(ev));
    std::printf("OK %llx\n", checksum);
    return 0;
}
