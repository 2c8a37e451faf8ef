// plain_worker — the benchmark workloads as an XSched-UNAWARE CUDA program: it uses only the CUDA runtime and
// the kernel library (non-preemptible kernels), never an XQueue or hint call.  Scheduling, if any, comes
// from whichever libcuda interposer is on LD_LIBRARY_PATH (this repository's libshimcuda.so or the
// reference's own shim built under oracle/_ref) together with the XSCHED_* environment variables — the
// "transparent" way of using XSched (reference: examples/Linux/1_transparent_sched).
//
//   --role lp   non-preemptible bf16 GEMM launched back-to-back on one stream until SIGTERM
//   --role hp   fp32 vector add every --period-us; latency = launch -> cudaStreamSynchronize
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cinttypes>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <string>
#include <thread>
#include <vector>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "xsched_b200/pk.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s -> %s\n", #x, cudaGetErrorString(e_)); std::exit(3); } } while (0)
#define PK(x) do { xpkResult r_ = (x); if (r_ != XPK_SUCCESS) { std::fprintf(stderr, "%s -> %s\n", #x, xpkResultString(r_)); std::exit(5); } } while (0)

static std::atomic<bool> g_stop{false};
static void OnTerm(int) { g_stop.store(true); }
// SIGUSR1: first = restart the count (co-run begins), second = freeze it (co-run over).
static std::atomic<int> g_marks{0};
static void OnMark(int) { g_marks.fetch_add(1); }
static int64_t NowNs() { return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static double Pct(std::vector<double> v, double p) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    return v[std::min(v.size() - 1, (size_t)(p * (v.size() - 1) + 0.5))];
}
__global__ void FillBf16(__nv_bfloat16 *p, size_t n, float v) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = __float2bfloat16(v * (float)((i * 2654435761u >> 16) & 255) / 255.f - 0.5f * v);
}
__global__ void FillF32(float *p, size_t n, float v) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v * (float)(i & 1023);
}

int main(int argc, char **argv) {
    std::string role = "lp";
    int device = 0, count = 300, M = 8192, N = 8192, K = 8192, in_flight = 2;
    int64_t period_us = 10000;
    uint64_t n = 1ull << 26;
    double duration_s = 3600;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string k = argv[i], v = argv[i + 1];
        if (k == "--role") role = v; else if (k == "--device") device = std::atoi(v.c_str()); else if (k == "--count") count = std::atoi(v.c_str());
        else if (k == "--period-us") period_us = std::atoll(v.c_str()); else if (k == "--hp-n") n = std::strtoull(v.c_str(), nullptr, 10);
        else if (k == "--M") M = std::atoi(v.c_str()); else if (k == "--N") N = std::atoi(v.c_str()); else if (k == "--K") K = std::atoi(v.c_str());
        else if (k == "--in-flight") in_flight = std::atoi(v.c_str()); else if (k == "--duration-s") duration_s = std::atof(v.c_str());
    }
    std::signal(SIGUSR1, OnMark);
    std::signal(SIGTERM, OnTerm);
    std::signal(SIGINT, OnTerm);
    CK(cudaSetDevice(device));
    CK(cudaFree(0));
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));        // an interposer may attach an XQueue here

    if (role == "lp") {
        __nv_bfloat16 *A, *B, *C;
        CK(cudaMalloc(&A, (size_t)M * K * 2)); CK(cudaMalloc(&B, (size_t)N * K * 2)); CK(cudaMalloc(&C, (size_t)M * N * 2));
        FillBf16<<<1184, 256, 0, s>>>(A, (size_t)M * K, 1.0f);
        FillBf16<<<1184, 256, 0, s>>>(B, (size_t)N * K, 1.0f);
        CK(cudaStreamSynchronize(s));
        std::vector<xpkTask_t> tasks(in_flight);
        std::vector<cudaEvent_t> done(in_flight);
        for (int i = 0; i < in_flight; ++i) {
            PK(xpkTaskCreateGemm(&tasks[i], C, A, B, M, N, K, XPK_FLAG_NON_PREEMPTIBLE, nullptr));
            CK(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        uint64_t iters = 0, counted_from = 0, frozen_at = 0;
        int64_t t_begin = 0, t_frozen = 0;
        int marks_seen = 0;
        const int64_t t_start = NowNs();
        while (!g_stop.load()) {
            const int marks = g_marks.load();
            if (marks != marks_seen && t_begin) {
                if (marks_seen == 0) { counted_from = iters; t_begin = NowNs(); }
                if (marks >= 2 && !t_frozen) { frozen_at = iters; t_frozen = NowNs(); }
                marks_seen = marks;
            }
            if (!t_begin && (NowNs() - t_start) > 500000000) {
                CK(cudaStreamSynchronize(s));
                counted_from = iters;
                t_begin = NowNs();
                std::printf("READY\n"); std::fflush(stdout);
            }
            if (t_begin && (NowNs() - t_begin) / 1e9 >= duration_s) break;
            const int slot = (int)(iters % in_flight);
            if (iters >= (uint64_t)in_flight) CK(cudaEventSynchronize(done[slot]));
            PK(xpkTaskReset(tasks[slot], s));
            PK(xpkTaskLaunch(tasks[slot], s, 0));
            CK(cudaEventRecord(done[slot], s));
            ++iters;
        }
        CK(cudaStreamSynchronize(s));
        const double sec = t_begin ? ((t_frozen ? t_frozen : NowNs()) - t_begin) / 1e9 : 0;
        const uint64_t counted = (t_frozen ? frozen_at : iters) - counted_from;
        std::printf("{\"role\": \"plain-lp\", \"iters\": %" PRIu64 ", \"seconds\": %.4f, \"rate\": %.3f, \"unit\": \"TFLOP/s\"}\n", counted, sec,
                    sec > 0 ? counted * 2.0 * M * N * K / sec / 1e12 : 0.0);
        return 0;
    }

    float *a, *b, *c;
    CK(cudaMalloc(&a, n * 4)); CK(cudaMalloc(&b, n * 4)); CK(cudaMalloc(&c, n * 4));
    FillF32<<<1184, 256, 0, s>>>(a, n, 1.0f);
    FillF32<<<1184, 256, 0, s>>>(b, n, 2.0f);
    CK(cudaStreamSynchronize(s));
    xpkTask_t t;
    PK(xpkTaskCreateVecAdd(&t, c, a, b, n, 0, XPK_FLAG_NON_PREEMPTIBLE, nullptr));
    auto once = [&]() {
        const int64_t t0 = NowNs();
        PK(xpkTaskReset(t, s));
        PK(xpkTaskLaunch(t, s, 0));
        CK(cudaStreamSynchronize(s));
        return (NowNs() - t0) / 1e3;
    };
    for (int i = 0; i < 5; ++i) once();
    std::printf("READY\n"); std::fflush(stdout);
    std::vector<double> lat;
    int64_t next = NowNs();
    for (int i = 0; i < count && !g_stop.load(); ++i) {
        next += period_us * 1000;
        while (NowNs() < next) { const int64_t left = next - NowNs(); if (left > 200000) std::this_thread::sleep_for(std::chrono::microseconds(left / 2000)); else std::this_thread::yield(); }
        lat.push_back(once());
        if (NowNs() > next + period_us * 1000) next = NowNs();
    }
    std::printf("DONE\n"); std::fflush(stdout);
    float h[4];
    CK(cudaMemcpy(h, c + 1000, 16, cudaMemcpyDeviceToHost));
    const bool ok = h[0] == 3.0f * 1000 && h[1] == 3.0f * 1001;
    std::printf("{\"role\": \"plain-hp\", \"n\": %zu, \"p50_us\": %.2f, \"p99_us\": %.2f, \"max_us\": %.2f, \"mean_us\": %.2f, \"verified\": %s}\n", lat.size(),
                Pct(lat, 0.5), Pct(lat, 0.99), Pct(lat, 1.0), lat.empty() ? 0.0 : std::accumulate(lat.begin(), lat.end(), 0.0) / lat.size(), ok ? "true" : "false");
    return 0;
}
