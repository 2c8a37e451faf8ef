// Preemptible persistent streaming kernels: fp32 triad a = b + s*c and fp32 vector add.
//
// HBM-bound.  Algorithmic traffic is 12 bytes per element (two 4-byte reads, one 4-byte
// write); nothing is re-read.  Every access is a 128-bit, fully coalesced load or store
// with a streaming cache hint, issued UNROLL-deep per thread so that each SM keeps well
// over latency x bandwidth bytes in flight.  Indexing is 64-bit throughout (2^31 elements
// per array overflows 32-bit byte offsets).
//
// Both forms claim one tile (tile_elems elements) at a time through xpk::claim_tile; the
// preemptible one reads the preempt flag before each claim, the twin (kPreemptible = false:
// the high-priority kernels, and the measurement of what the check costs) never does.  Tiles
// handed out dynamically also balance the HBM channels better than a static stride does.
#include "pk_common.cuh"

namespace xpk {

constexpr int kStreamThreads = 256;
constexpr int kStreamUnroll  = 4;                                   // float4 per thread per array per chunk
constexpr int kChunkElems    = kStreamThreads * kStreamUnroll * 4;  // 4096 elements

enum StreamOp { kOpTriad = 0, kOpVecAdd = 1 };

__device__ __forceinline__ float4 ld_stream(const float4 *p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(float4 *p, const float4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int OP>
__device__ __forceinline__ float apply1(float x, float y, float s) {
    // Triad: out = x + s*y with one rounding.  Vector add: out = x + y.
    return OP == kOpTriad ? __fmaf_rn(s, y, x) : __fadd_rn(x, y);
}
template <int OP>
__device__ __forceinline__ float4 apply4(const float4 &x, const float4 &y, float s) {
    return make_float4(apply1<OP>(x.x, y.x, s), apply1<OP>(x.y, y.y, s),
                       apply1<OP>(x.z, y.z, s), apply1<OP>(x.w, y.w, s));
}

// Process elements [lo, hi) of the arrays; lo is a multiple of kChunkElems.
template <int OP>
__device__ __forceinline__ void stream_tile(float *__restrict__ out, const float *__restrict__ x,
                                            const float *__restrict__ y, float s,
                                            unsigned long long lo, unsigned long long hi) {
    const int tid = threadIdx.x;
    unsigned long long pos = lo;
    // Whole chunks: no bounds checks, all loads issued before the first use.
    for (; pos + kChunkElems <= hi; pos += kChunkElems) {
        const float4 *x4 = reinterpret_cast<const float4 *>(x + pos) + tid;
        const float4 *y4 = reinterpret_cast<const float4 *>(y + pos) + tid;
        float4 *o4 = reinterpret_cast<float4 *>(out + pos) + tid;
        float4 xv[kStreamUnroll], yv[kStreamUnroll];
#pragma unroll
        for (int u = 0; u < kStreamUnroll; ++u) {
            xv[u] = ld_stream(x4 + u * kStreamThreads);
            yv[u] = ld_stream(y4 + u * kStreamThreads);
        }
#pragma unroll
        for (int u = 0; u < kStreamUnroll; ++u)
            st_stream(o4 + u * kStreamThreads, apply4<OP>(xv[u], yv[u], s));
    }
    // Ragged end of the array (only the last tile gets here).
    if (pos < hi) {
        const unsigned long long vec_end = pos + ((hi - pos) & ~3ull);
        for (unsigned long long i = pos + 4ull * tid; i < vec_end; i += 4ull * kStreamThreads) {
            float4 xv = ld_stream(reinterpret_cast<const float4 *>(x + i));
            float4 yv = ld_stream(reinterpret_cast<const float4 *>(y + i));
            st_stream(reinterpret_cast<float4 *>(out + i), apply4<OP>(xv, yv, s));
        }
        for (unsigned long long i = vec_end + tid; i < hi; i += kStreamThreads)
            out[i] = apply1<OP>(x[i], y[i], s);
    }
}

constexpr unsigned kRelayCtas = 8;

template <int OP, bool kPreemptible>
__global__ void __launch_bounds__(kStreamThreads, 6)
stream_kernel(Ctl *ctl, float *__restrict__ out, const float *__restrict__ x,
              const float *__restrict__ y, float s, unsigned long long n,
              unsigned long long tile_elems, unsigned long long launch_no) {
    unsigned long long done = 0;
    note_start(ctl);
    __shared__ unsigned long long s_tile;
    // Relay of the host's early flag (see pk_common.cuh): in the grid's first kRelayCtas CTAs one thread of the second
    // warp looks at the host word while thread 0 claims the next tile, and raises the device flag itself.  The
    // kernel then stops even when the stream-ordered write of the flag is held up behind it (seen under MPS, where
    // a client's streams can share a hardware queue).  Eight CTAs with ~27 us tiles look every ~3 us between them.
    const uint32_t *relay_src = nullptr;
    if constexpr (kPreemptible) {
        if (blockIdx.x < kRelayCtas && threadIdx.x == 32) relay_src = flag_relay_source(ctl->flag);
    }
    while (true) {
        if (threadIdx.x == 0) s_tile = claim_tile<kPreemptible>(ctl);
        if constexpr (kPreemptible) {
            if (relay_src != nullptr && ld_host_word(relay_src) != 0u) atomicExch(const_cast<uint32_t *>(ctl->flag), 1u);
        }
        __syncthreads();
        const unsigned long long tile = s_tile;
        if (tile == kNoTile) break;
        const unsigned long long lo = tile * tile_elems;
        unsigned long long hi = lo + tile_elems;
        if (hi > n) hi = n;
        stream_tile<OP>(out, x, y, s, lo, hi);
        ++done;
        __syncthreads();          // s_tile is rewritten next iteration
    }
    __syncthreads();
    if (threadIdx.x == 0) cta_exit(ctl, done, launch_no);
}

// Host-side launcher used by the C ABI.
cudaError_t launch_stream(int op, bool preemptible, Ctl *ctl, float *out, const float *x,
                          const float *y, float s, unsigned long long n,
                          unsigned long long tile_elems, unsigned long long launch_no,
                          int grid, cudaStream_t stream) {
    dim3 g(grid), b(kStreamThreads);
    if (op == kOpTriad) {
        if (preemptible) stream_kernel<kOpTriad, true><<<g, b, 0, stream>>>(ctl, out, x, y, s, n, tile_elems, launch_no);
        else             stream_kernel<kOpTriad, false><<<g, b, 0, stream>>>(ctl, out, x, y, s, n, tile_elems, launch_no);
    } else {
        if (preemptible) stream_kernel<kOpVecAdd, true><<<g, b, 0, stream>>>(ctl, out, x, y, s, n, tile_elems, launch_no);
        else             stream_kernel<kOpVecAdd, false><<<g, b, 0, stream>>>(ctl, out, x, y, s, n, tile_elems, launch_no);
    }
    return cudaGetLastError();
}

int stream_ctas_per_sm() {
    int a = 0, b = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&a, stream_kernel<kOpTriad, true>, kStreamThreads, 0);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, stream_kernel<kOpVecAdd, true>, kStreamThreads, 0);
    int m = a < b ? a : b;
    return m < 1 ? 1 : m;
}

} // namespace xpk
