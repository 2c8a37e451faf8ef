// A plain CUDA-runtime program with no knowledge of XSched that uses the stream-ordered calls beyond
// launches and 1-D copies: stream capture -> graph -> repeated graph launches, stream-ordered allocation,
// 2-D memset and copy, a cooperative launch, a host function and a stream callback.  Each round's result is
// checked on the host.  Used to test the libcuda interposer: same "OK" line with and without it.
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cooperative_groups.h>
#include <cuda_runtime.h>

namespace cg = cooperative_groups;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("FAIL %s: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)

__global__ void add_one(int *p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] += 1;
}
__global__ void times_two(int *p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] *= 2;
}
// grid-wide reduction in two phases separated by a grid sync
__global__ void coop_sum(const int *p, int n, unsigned long long *partial, unsigned long long *out) {
    cg::grid_group grid = cg::this_grid();
    unsigned long long s = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) s += (unsigned long long)p[i];
    for (int o = 16; o; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&partial[blockIdx.x], s);
    grid.sync();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t = 0;
        for (unsigned b = 0; b < gridDim.x; ++b) { t += partial[b]; partial[b] = 0; }
        *out = t;
    }
}

static std::atomic<int> g_host_calls{0}, g_callbacks{0};
static void CUDART_CB HostFn(void *) { g_host_calls.fetch_add(1); }
static void CUDART_CB StreamCb(cudaStream_t, cudaError_t, void *) { g_callbacks.fetch_add(1); }

int main(int argc, char **argv) {
    const int n = 1 << 18, rounds = argc > 1 ? std::atoi(argv[1]) : 20;
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    int *d;
    CK(cudaMalloc(&d, n * 4));
    unsigned long long *partial, *out, *h_out;
    CK(cudaMalloc(&partial, 64 * 8)); CK(cudaMemset(partial, 0, 64 * 8));
    CK(cudaMalloc(&out, 8));
    CK(cudaMallocHost(&h_out, 8));

    // graph: (+1) -> (*2) -> (+1)   ==>  x -> 2x + 3
    cudaGraph_t graph; cudaGraphExec_t exec;
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    add_one<<<n / 256, 256, 0, s>>>(d, n);
    times_two<<<n / 256, 256, 0, s>>>(d, n);
    add_one<<<n / 256, 256, 0, s>>>(d, n);
    CK(cudaStreamEndCapture(s, &graph));
    CK(cudaGraphInstantiate(&exec, graph, 0));
    CK(cudaGraphUpload(exec, s));

    for (int r = 0; r < rounds; ++r) {
        CK(cudaMemset2DAsync(d, 1024 * 4, 0, 1024 * 4, n / 1024, s));          // all zero, as a 2-D memset
        add_one<<<n / 256, 256, 0, s>>>(d, n);                                 // 1
        CK(cudaGraphLaunch(exec, s));                                          // 5
        CK(cudaGraphLaunch(exec, s));                                          // 13
        int *tmp;
        CK(cudaMallocAsync(&tmp, n * 4, s));
        CK(cudaMemcpy2DAsync(tmp, 1024 * 4, d, 1024 * 4, 1024 * 4, n / 1024, cudaMemcpyDeviceToDevice, s));
        times_two<<<n / 256, 256, 0, s>>>(tmp, n);                             // 26 in tmp
        void *args[] = {(void *)&tmp, (void *)&n, (void *)&partial, (void *)&out};
        CK(cudaLaunchCooperativeKernel((void *)coop_sum, dim3(64), dim3(256), args, 0, s));
        CK(cudaFreeAsync(tmp, s));
        CK(cudaMemcpyAsync(h_out, out, 8, cudaMemcpyDeviceToHost, s));
        CK(cudaLaunchHostFunc(s, HostFn, nullptr));
        CK(cudaStreamAddCallback(s, StreamCb, nullptr, 0));
        CK(cudaStreamSynchronize(s));
        if (*h_out != 26ull * n) { std::printf("FAIL round %d: %llu\n", r, *h_out); return 1; }
    }
    CK(cudaDeviceSynchronize());
    if (g_host_calls.load() != rounds || g_callbacks.load() != rounds) { std::printf("FAIL host calls %d callbacks %d\n", g_host_calls.load(), g_callbacks.load()); return 1; }
    CK(cudaGraphExecDestroy(exec)); CK(cudaGraphDestroy(graph));
    CK(cudaFree(d)); CK(cudaFree(partial)); CK(cudaFree(out)); CK(cudaFreeHost(h_out)); CK(cudaStreamDestroy(s));
    std::printf("OK rounds=%d\n", rounds);
    return 0;
}
