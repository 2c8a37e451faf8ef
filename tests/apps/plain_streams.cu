// A plain CUDA-runtime program with no knowledge of XSched: two streams, each running rounds of
// H2D copy -> vector_add kernel -> D2H copy, chained across the streams with an event, checked on the host.
// Used to test the libcuda interposer: the same binary must print the same "OK" line with and without it.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("FAIL %s: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)

__global__ void vector_add(const float *a, const float *b, float *c, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) c[i] = a[i] + b[i];
}
__global__ void scale(float *c, float s, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) c[i] *= s;
}

int main(int argc, char **argv) {
    const int n = 1 << 20, rounds = argc > 1 ? std::atoi(argv[1]) : 60;
    float *ha, *hb, *hc[2];
    CK(cudaMallocHost(&ha, n * 4)); CK(cudaMallocHost(&hb, n * 4)); CK(cudaMallocHost(&hc[0], n * 4)); CK(cudaMallocHost(&hc[1], n * 4));
    for (int i = 0; i < n; ++i) { ha[i] = (float)(i % 1000) * 0.5f; hb[i] = (float)(i % 77); }
    cudaStream_t s[2];
    float *da[2], *db[2], *dc[2];
    for (int k = 0; k < 2; ++k) {
        CK(cudaStreamCreateWithFlags(&s[k], cudaStreamNonBlocking));
        CK(cudaMalloc(&da[k], n * 4)); CK(cudaMalloc(&db[k], n * 4)); CK(cudaMalloc(&dc[k], n * 4));
    }
    cudaEvent_t ev;
    CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    for (int r = 0; r < rounds; ++r) {
        for (int k = 0; k < 2; ++k) {
            CK(cudaMemcpyAsync(da[k], ha, n * 4, cudaMemcpyHostToDevice, s[k]));
            CK(cudaMemcpyAsync(db[k], hb, n * 4, cudaMemcpyHostToDevice, s[k]));
            vector_add<<<(n + 255) / 256, 256, 0, s[k]>>>(da[k], db[k], dc[k], n);
        }
        // stream 1 scales its result only after stream 0 finished its add (cross-stream dependency)
        CK(cudaEventRecord(ev, s[0]));
        CK(cudaStreamWaitEvent(s[1], ev, 0));
        scale<<<(n + 255) / 256, 256, 0, s[1]>>>(dc[1], 2.0f, n);
        for (int k = 0; k < 2; ++k) CK(cudaMemcpyAsync(hc[k], dc[k], n * 4, cudaMemcpyDeviceToHost, s[k]));
        CK(cudaStreamSynchronize(s[0]));
        CK(cudaStreamSynchronize(s[1]));
        for (int i = 0; i < n; i += 4097) {
            if (hc[0][i] != ha[i] + hb[i] || hc[1][i] != 2.0f * (ha[i] + hb[i])) { std::printf("FAIL round %d index %d\n", r, i); return 1; }
        }
    }
    CK(cudaEventSynchronize(ev));
    CK(cudaDeviceSynchronize());
    for (int k = 0; k < 2; ++k) { CK(cudaFree(da[k])); CK(cudaFree(db[k])); CK(cudaFree(dc[k])); CK(cudaStreamDestroy(s[k])); }
    std::printf("OK rounds=%d\n", rounds);
    return 0;
}
