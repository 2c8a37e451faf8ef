/*
 * kernels_oracle.c — CPU restatement of the arithmetic of the preemptible kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped libraries links, loads or calls this
 * file; it is used by tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline leg
 * as the checker the CUDA results are compared with.
 *
 * Provenance.  The reference (XSched) contains no triad, radix-sort or GEMM kernel: its
 * Level-2 device code is a guardian prologue patched into arbitrary application kernels
 * (platforms/cuda/hal/inject/inject.cu:43-140) and its only arithmetic kernel is the example
 * `vector_add`, C[i] = A[i] + B[i] in fp32 (examples/Linux/1_transparent_sched/app.cu:18-23).
 * oracle_vecadd follows that kernel line for line.  The other three functions restate the
 * definitions the workload configs give (a = b + s*c as one fused multiply-add; ascending
 * int32 sort by 8-bit LSD radix; C = A*B^T in bf16 with wide accumulation) — there is no
 * reference source or golden vector for them, so for these three the parity is "unpinned
 * by the reference" and pinned instead by cross-checks against independent implementations
 * (qsort, numpy, an fp64 product) in tests/test_oracle_kernels.py.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared -o liboracle_kernels.so kernels_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* examples/Linux/1_transparent_sched/app.cu:18-23 — C[i] = A[i] + B[i]. */
void oracle_vecadd(float *c, const float *a, const float *b, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) c[i] = a[i] + b[i];
}

/* STREAM triad with a single rounding per element: a[i] = fma(s, c[i], b[i]). */
void oracle_triad(float *a, const float *b, const float *c, float s, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) a[i] = fmaf(s, c[i], b[i]);
}

/* 64-bit checksum used for full-size arrays: sum of the raw 32-bit patterns, each
 * multiplied by (index mod 2^16 + 1) so that permutations and shifts are caught. */
uint64_t oracle_checksum_u32(const uint32_t *x, uint64_t n) {
    uint64_t h = 0;
    for (uint64_t i = 0; i < n; ++i) h += (uint64_t)x[i] * ((i & 0xFFFFu) + 1u);
    return h;
}

/* Ascending int32 LSD radix sort, 8-bit digits, 4 passes, sign bit flipped for the order.
 * `keys` is sorted in place; `tmp` has room for n keys.  Stable counting sort per pass. */
void oracle_radix_sort_i32(int32_t *keys, int32_t *tmp, uint64_t n) {
    uint32_t *src = (uint32_t *)keys, *dst = (uint32_t *)tmp;
    for (int pass = 0; pass < 4; ++pass) {
        uint64_t count[256];
        memset(count, 0, sizeof(count));
        const int shift = 8 * pass;
        for (uint64_t i = 0; i < n; ++i) count[((src[i] ^ 0x80000000u) >> shift) & 255u]++;
        uint64_t run = 0;
        for (int d = 0; d < 256; ++d) { uint64_t c = count[d]; count[d] = run; run += c; }
        for (uint64_t i = 0; i < n; ++i) dst[count[((src[i] ^ 0x80000000u) >> shift) & 255u]++] = src[i];
        uint32_t *t = src; src = dst; dst = t;
    }
    /* 4 passes: the data is back in `keys`. */
}

/* 256-bin histogram of byte `pass` of the order-preserving key (phase 0 of the sort). */
void oracle_digit_hist(const int32_t *keys, uint64_t n, int pass, uint32_t *hist256) {
    memset(hist256, 0, 256 * sizeof(uint32_t));
    for (uint64_t i = 0; i < n; ++i)
        hist256[((((uint32_t)keys[i]) ^ 0x80000000u) >> (8 * pass)) & 255u]++;
}

static int cmp_i32(const void *a, const void *b) {
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return (x > y) - (x < y);
}
/* Independent check of the radix restatement. */
void oracle_qsort_i32(int32_t *keys, uint64_t n) { qsort(keys, (size_t)n, sizeof(int32_t), cmp_i32); }

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* Round-to-nearest-even fp32 -> bf16 (finite inputs; NaN kept quiet). */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* C[m,n] = sum_k A[m,k] * B[n,k] for the listed rows only, accumulated in fp64 from the exact
 * bf16 inputs (each product of two bf16 values is exact in fp64).  A is M x K, B is N x K,
 * both row-major bf16 bit patterns.  `rows` holds `nrows` row indices; out is nrows x N fp64. */
void oracle_gemm_bf16_rows(double *out, const uint16_t *A, const uint16_t *B, uint32_t N, uint32_t K,
                           const uint32_t *rows, uint32_t nrows) {
    float *brow = (float *)malloc((size_t)K * sizeof(float));
    float *arow = (float *)malloc((size_t)K * sizeof(float));
    for (uint32_t r = 0; r < nrows; ++r) {
        const uint16_t *a = A + (size_t)rows[r] * K;
        for (uint32_t k = 0; k < K; ++k) arow[k] = bf16_to_f32(a[k]);
        for (uint32_t n = 0; n < N; ++n) {
            const uint16_t *b = B + (size_t)n * K;
            for (uint32_t k = 0; k < K; ++k) brow[k] = bf16_to_f32(b[k]);
            double acc = 0.0;
            for (uint32_t k = 0; k < K; ++k) acc += (double)arow[k] * (double)brow[k];
            out[(size_t)r * N + n] = acc;
        }
    }
    free(brow);
    free(arow);
}
