// A plain CUDA-runtime program built with `nvcc --default-stream per-thread`: two host threads work on "the default
// stream" (stream 0 / no stream argument), which in this build is a different stream per thread.  Each thread runs
// rounds of H2D copy -> kernel -> kernel -> D2H copy -> synchronise and checks its own result.  Used to test that
// the libcuda interposer schedules per-thread-default-stream work: same "OK" line with and without it.
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <thread>
#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("FAIL %s: %s\n", #x, cudaGetErrorString(e_)); std::exit(1); } } while (0)

__global__ void axpy(float *c, const float *a, float k, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) c[i] = a[i] * k + c[i];
}

int main(int argc, char **argv) {
    const int n = 1 << 20, rounds = argc > 1 ? std::atoi(argv[1]) : 30;
    std::atomic<int> bad{0};
    auto work = [&](int t) {
        float *ha, *hc, *da, *dc;
        CK(cudaMallocHost(&ha, n * 4)); CK(cudaMallocHost(&hc, n * 4));
        CK(cudaMalloc(&da, n * 4)); CK(cudaMalloc(&dc, n * 4));
        for (int r = 0; r < rounds; ++r) {
            for (int i = 0; i < n; i += 257) ha[i] = (float)((i + r + t) % 1000);
            CK(cudaMemcpyAsync(da, ha, n * 4, cudaMemcpyHostToDevice, 0));
            CK(cudaMemsetAsync(dc, 0, n * 4, 0));
            axpy<<<(n + 255) / 256, 256>>>(dc, da, 2.0f, n);
            axpy<<<(n + 255) / 256, 256, 0, cudaStreamPerThread>>>(dc, da, 0.5f, n);
            CK(cudaMemcpyAsync(hc, dc, n * 4, cudaMemcpyDeviceToHost, 0));
            CK(cudaStreamSynchronize(0));
            for (int i = 0; i < n; i += 257) if (hc[i] != ha[i] * 2.5f) { bad.fetch_add(1); break; }
        }
        CK(cudaFree(da)); CK(cudaFree(dc)); CK(cudaFreeHost(ha)); CK(cudaFreeHost(hc));
    };
    CK(cudaFree(0));
    std::thread a(work, 0), b(work, 1);
    a.join(); b.join();
    CK(cudaDeviceSynchronize());
    if (bad.load()) { std::printf("FAIL %d rounds with wrong data\n", bad.load()); return 1; }
    std::printf("OK rounds=%d threads=2\n", rounds);
    return 0;
}
