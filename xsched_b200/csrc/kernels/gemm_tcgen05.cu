// Preemptible persistent bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulate.
//
// Tensor-pipe bound: 2*M*N*K flop.  One CTA per SM owns a 256x256 output tile at a time:
//
//   warp 0 (one lane)   claims tiles (xpk::claim_tile: flag poll + ticket), publishes the tile
//                       id on a 4-slot ring, and streams 256x64 A / 256x64 B k-blocks (64 KB) into
//                       a 3-stage shared-memory ring with TMA (cp.async.bulk.tensor, 128-byte
//                       swizzle, no multicast: every CTA fetches its own operands);
//   warp 1 (one lane)   issues tcgen05.mma.cta_group::1.kind::f16 (M128 N256 K16) from
//                       shared-memory descriptors: per K=16 step one MMA for rows 0-127 and one
//                       for rows 128-255, both reading the same B tile, into two 256-column fp32
//                       accumulators that together fill tensor memory (512 columns);
//                       tcgen05.commit releases the smem stage / publishes the accumulators;
//   warps 2-9           two groups of four warps, one per accumulator, read it with tcgen05.ld
//                       (32 lanes x 32 columns per instruction), round to bf16 and store rows;
//   warp 10 (one lane,  relays an early copy of the preempt flag from mapped host memory into the device flag
//   first CTA only)     (see pk_common.cuh); idle in every other CTA.
//
// A 256x256 tile moves 64 KB of operands per 64-deep k-block for 2*256*256*64 flop — one third less
// L2->SM traffic per flop than a 128x256 tile, which measured as the limiter of that shape (tensor pipe
// 74 % busy at 15 TB/s of operand traffic over the chip).  The price: both accumulators belong to the
// same tile, so the epilogue no longer overlaps the next tile's MMAs (it overlaps its TMA prefetch);
// eight epilogue warps keep that window to a few microseconds per ~120 us tile.
//
// Preemption.  Between tiles the producer stops claiming once the flag is up; tiles already
// claimed are finished.  With kAbort it also polls the flag every kAbortPollEvery (4) k-blocks inside a tile
// and, when raised, stops loading, hands the tile back (xpk::abandon_tile) and tells the MMA
// and epilogue warps which k-block / tile sequence number was the first not issued; they
// finish everything older and drop the abandoned tile, whose C is untouched and which is
// recomputed from k = 0 after resume.  A tile's accumulation order is fixed (k ascending,
// one accumulator, no split-K, no atomics), so its bf16 result does not depend on which CTA
// or launch produced it.
//
// Every mbarrier wait is bounded (2 s); on expiry the CTA raises an error, all roles leave
// their loops, outstanding TMA loads and MMAs are waited for (bounded), tensor memory is
// freed and the kernel returns with status ERROR.
#include "gemm_ptx.cuh"

namespace xpk {

constexpr int kBM = 256, kBN = 256, kBK = 64;   // CTA tile
constexpr int kMmaM = 128;                      // rows per MMA / per accumulator
constexpr int kStages = 3;
constexpr int kAccBufs = 2;                     // the two row-halves of one tile
constexpr int kSchedSlots = 4;
constexpr int kEpiWarps = 8;
constexpr int kRelayWarp = 2 + kEpiWarps;                // one more warp: in the grid's first CTA its first lane relays the host's early flag
constexpr int kGemmThreads = 64 + 32 * kEpiWarps + 32;
constexpr uint32_t kABytes = kBM * kBK * 2;          // 32 KiB
constexpr uint32_t kBBytes = kBN * kBK * 2;          // 32 KiB
constexpr uint32_t kTmemCols = 512;
constexpr int kAbortPollEvery = 4;

constexpr uint32_t kErrGemmProducer = 0x60000001u;
constexpr uint32_t kErrGemmMma      = 0x60000002u;
constexpr uint32_t kErrGemmEpilogue = 0x60000003u;
constexpr uint32_t kErrGemmDrain    = 0x60000004u;

struct GemmShared {
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long tmem_full;                 // both accumulators of the tile are complete
    unsigned long long tmem_empty[kAccBufs];      // one per accumulator: its epilogue group has drained it
    unsigned long long sched_full[kSchedSlots];
    unsigned long long sched_empty[kSchedSlots];
    unsigned long long drain;
    unsigned long long sched_tile[kSchedSlots];
    unsigned long long abort_kseq;       // first k-block sequence number that was not loaded
    unsigned long long abort_tile_seq;   // sequence number of the abandoned tile
    uint32_t abort;                      // 1: abandon from abort_* on; 2: error, leave now
    uint32_t tmem_base;
    uint32_t relay_stop;                 // the producer is done: nothing left for an early flag to stop
};
constexpr size_t kGemmSmemBytes = 1024 /*align slack*/ + kStages * (kABytes + kBBytes) + sizeof(GemmShared);

// ---- instructions with the .cta_group::1 qualifier ------------------------------------
__device__ __forceinline__ void tc_commit(void *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Instruction descriptor for kind::f16: D fp32, A/B bf16, both K-major, N=256, M=128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kMmaM >> 4) << 24);

// Bounded wait.  `quit()` is evaluated between polls; returns false when it fired or on timeout.
template <class Quit>
__device__ __forceinline__ bool bounded_wait(void *bar, uint32_t parity, GemmShared *sh, Ctl *ctl,
                                             uint32_t errcode, Quit quit) {
    uint32_t it = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (quit()) return false;
        if ((++it & 0xFFu) == 0) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) {
                raise_error(ctl, errcode);
                *(volatile uint32_t *)&sh->abort = 2u;
                return false;
            }
        }
    }
    return true;
}

template <bool kPreemptible, bool kAbort>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(Ctl *ctl, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 __nv_bfloat16 *__restrict__ C, uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *smem_a = smem;
    unsigned char *smem_b = smem + kStages * kABytes;
    GemmShared *sh = reinterpret_cast<GemmShared *>(smem + kStages * (kABytes + kBBytes));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (M + kBM - 1) / kBM, n_tiles = N / kBN;   // M is a multiple of 128: the last row-block may be half full
    const uint32_t k_blocks = K / kBK;
    volatile uint32_t *v_abort = &sh->abort;
    note_start(ctl);

    if constexpr (kPreemptible) {
        // A kernel that starts with the flag already raised (it was queued behind the one being flushed)
        // leaves before setting up barriers or tensor memory, so a flush of several queued launches costs
        // little more than their launch overhead.
        __shared__ uint32_t s_stop;
        if (threadIdx.x == 0) s_stop = ld_flag(ctl->flag);
        __syncthreads();
        if (s_stop != 0) {
            if (threadIdx.x == 0) cta_exit(ctl, 0, launch_no);
            return;
        }
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
        mbar_init(&sh->tmem_full, 1);
        for (int i = 0; i < kAccBufs; ++i) mbar_init(&sh->tmem_empty[i], 4);
        for (int i = 0; i < kSchedSlots; ++i) { mbar_init(&sh->sched_full[i], 1); mbar_init(&sh->sched_empty[i], 1 + kEpiWarps); }
        mbar_init(&sh->drain, 1);
        sh->abort = 0;
        sh->relay_stop = 0;
        sh->abort_kseq = ~0ull;
        sh->abort_tile_seq = ~0ull;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&sh->tmem_base;

    unsigned long long tiles_done = 0;     // counted by warp 2 lane 0

    if (warp == 0) {
        // ======================= producer: claim + TMA =======================
        if (lane == 0) {
            unsigned long long kseq = 0, tseq = 0;
            bool live = true;
            while (live) {
                const unsigned long long tile = claim_tile<kPreemptible>(ctl);     // the twin takes the same tickets without reading the flag
                const int slot = (int)(tseq % kSchedSlots);
                const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
                if (!bounded_wait(&sh->sched_empty[slot], sph ^ 1u, sh, ctl, kErrGemmProducer,
                                  [&] { return *v_abort == 2u; })) break;
                sh->sched_tile[slot] = tile;
                mbar_arrive(&sh->sched_full[slot]);
                if (tile == kNoTile) break;
                uint32_t m_blk, n_blk;
                tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if constexpr (kAbort) {
                        if ((kb % kAbortPollEvery) == 0 && ld_flag(ctl->flag) != 0) {
                            abandon_tile(ctl, tile);
                            sh->abort_kseq = kseq;
                            sh->abort_tile_seq = tseq;
                            __threadfence_block();
                            *v_abort = 1u;
                            live = false;
                            break;
                        }
                    }
                    const int stage = (int)(kseq % kStages);
                    const uint32_t ph = (uint32_t)((kseq / kStages) & 1);
                    if (!bounded_wait(&sh->empty[stage], ph ^ 1u, sh, ctl, kErrGemmProducer,
                                      [&] { return *v_abort == 2u; })) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->full[stage], kABytes + kBBytes);
                    tma_load_2d(smem_a + stage * kABytes, &map_a, &sh->full[stage], (int)(kb * kBK), (int)(m_blk * kBM));
                    tma_load_2d(smem_b + stage * kBBytes, &map_b, &sh->full[stage], (int)(kb * kBK), (int)(n_blk * kBN));
                    ++kseq;
                }
                ++tseq;
            }
            *(volatile uint32_t *)&sh->relay_stop = 1u;
            // Leave only after every load this thread issued has landed in shared memory.
            const unsigned long long first = kseq > (unsigned long long)kStages ? kseq - kStages : 0;
            for (unsigned long long s = first; s < kseq; ++s) {
                const int stage = (int)(s % kStages);
                const uint32_t ph = (uint32_t)((s / kStages) & 1);
                bounded_wait(&sh->full[stage], ph, sh, ctl, kErrGemmDrain, [] { return false; });
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ======================= MMA issuer =======================
        if (lane == 0) {
            unsigned long long kseq = 0, tseq = 0;
            bool issued_any = false;
            while (true) {
                const int slot = (int)(tseq % kSchedSlots);
                const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
                if (!bounded_wait(&sh->sched_full[slot], sph, sh, ctl, kErrGemmMma,
                                  [&] { return *v_abort == 2u || (*v_abort == 1u && tseq > *(volatile unsigned long long *)&sh->abort_tile_seq); })) break;
                const unsigned long long tile = sh->sched_tile[slot];
                mbar_arrive(&sh->sched_empty[slot]);
                if (tile == kNoTile) break;
                // Both accumulators must have been drained by the previous tile's epilogue.
                const uint32_t aph = (uint32_t)(tseq & 1);
                if (!bounded_wait(&sh->tmem_empty[0], aph ^ 1u, sh, ctl, kErrGemmMma, [&] { return *v_abort == 2u; })) break;
                if (!bounded_wait(&sh->tmem_empty[1], aph ^ 1u, sh, ctl, kErrGemmMma, [&] { return *v_abort == 2u; })) break;
                tc_fence_after();
                const uint32_t d_tmem0 = tmem_base, d_tmem1 = tmem_base + (uint32_t)kBN;
                bool abandoned = false;
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    const int stage = (int)(kseq % kStages);
                    const uint32_t ph = (uint32_t)((kseq / kStages) & 1);
                    if (!bounded_wait(&sh->full[stage], ph, sh, ctl, kErrGemmMma,
                                      [&] { return *v_abort == 2u || (*v_abort == 1u && kseq >= *(volatile unsigned long long *)&sh->abort_kseq); })) {
                        abandoned = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + stage * kABytes);
                    const uint32_t b_addr = smem_u32(smem_b + stage * kBBytes);
                    const uint64_t adesc0 = make_kmajor_sw128_desc(a_addr);
                    const uint64_t adesc1 = make_kmajor_sw128_desc(a_addr + kMmaM * kBK * 2);   // rows 128..255
                    const uint64_t bdesc = make_kmajor_sw128_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // +32 bytes per K=16 step inside the 128-byte swizzle atom (address field is >>4).
                        const uint32_t acc_flag = (kb | (uint32_t)k) != 0u;
                        tc_mma_bf16(d_tmem0, adesc0 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), kIdesc, acc_flag);
                        tc_mma_bf16(d_tmem1, adesc1 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), kIdesc, acc_flag);
                    }
                    issued_any = true;
                    tc_commit(&sh->empty[stage]);
                    ++kseq;
                }
                if (abandoned) break;
                tc_commit(&sh->tmem_full);
                ++tseq;
            }
            // All issued MMAs must have retired before tensor memory is freed.
            if (issued_any) {
                tc_commit(&sh->drain);
                bounded_wait(&sh->drain, 0u, sh, ctl, kErrGemmDrain, [] { return false; });
            }
        }
        __syncwarp();
    } else if (warp == kRelayWarp) {
        // ======================= relay of the host's early flag (first CTA only) =======================
        // The host raises a word in its own (mapped) memory a few microseconds before its write of the device
        // flag lands; this thread looks at that word about twice per microsecond and raises the device flag
        // itself.  Correctness never depends on it: the host's own write of the flag follows in any case.
        if constexpr (kPreemptible) {
            if (blockIdx.x == 0 && lane == 0) {
                const uint32_t *src = flag_relay_source(ctl->flag);
                if (src != nullptr) {
                    const unsigned long long t0 = global_ns();
                    uint32_t it = 0;
                    while (*(volatile uint32_t *)&sh->relay_stop == 0u) {
                        if (ld_host_word(src) != 0u) { atomicExch(const_cast<uint32_t *>(ctl->flag), 1u); break; }
                        __nanosleep(400);
                        if ((++it & 1023u) == 0 && global_ns() - t0 > kWaitLimitNs) break;      // a very long kernel just loses its relay
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ======================= epilogue (warps 2..9: two groups of four) =======================
        const uint32_t half = (uint32_t)(warp - 2) / 4u;         // which accumulator / row-half of the tile
        const uint32_t quarter = (uint32_t)(warp & 3);           // TMEM lanes [32q, 32q+32)
        unsigned long long tseq = 0;
        while (true) {
            const int slot = (int)(tseq % kSchedSlots);
            const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
            bool ok = bounded_wait(&sh->sched_full[slot], sph, sh, ctl, kErrGemmEpilogue,
                                   [&] { return *v_abort == 2u || (*v_abort == 1u && tseq > *(volatile unsigned long long *)&sh->abort_tile_seq); });
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const unsigned long long tile = sh->sched_tile[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->sched_empty[slot]);
            if (tile == kNoTile) break;
            const uint32_t aph = (uint32_t)(tseq & 1);
            ok = bounded_wait(&sh->tmem_full, aph, sh, ctl, kErrGemmEpilogue,
                              [&] { return *v_abort == 2u || (*v_abort == 1u && tseq >= *(volatile unsigned long long *)&sh->abort_tile_seq); });
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t m_blk, n_blk;
            tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
            const uint32_t row = m_blk * kBM + half * kMmaM + quarter * 32u + (uint32_t)lane;
            if (m_blk * kBM + half * kMmaM < M) {                    // the last row-block may have only its first half
                __nv_bfloat16 *crow = C + (size_t)row * N + (size_t)n_blk * kBN;
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + half * (uint32_t)kBN;
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    uint32_t r[32];
                    tc_ld32(taddr + (uint32_t)c, r);
                    tc_wait_ld();
                    store_row32_bf16(crow + c, r);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty[half]);
            if (warp == 2 && lane == 0) ++tiles_done;
            ++tseq;
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (warp == 2 && lane == 0) cta_exit(ctl, tiles_done, launch_no);
}

// ---- host side --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = (EncodeTiledFn)p;
    return fn;
}

// rows x cols bf16, row-major (cols contiguous); box = box_rows x 64 columns, 128-byte swizzle.
int gemm_make_map(void *map_out, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return 1;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};     // rows past the end of the tensor read as zero
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn((CUtensorMap *)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

cudaError_t gemm_prepare() {
    cudaError_t e;
    e = cudaFuncSetAttribute(gemm_bf16_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_bf16_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_bf16_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes);
}

unsigned long long gemm_tiles(uint32_t M, uint32_t N) { return (unsigned long long)((M + kBM - 1) / kBM) * (N / kBN); }

cudaError_t launch_gemm(bool preemptible, bool abort_inflight, Ctl *ctl, const void *map_a, const void *map_b,
                        void *C, uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no, int grid,
                        cudaStream_t stream) {
    const CUtensorMap &ma = *(const CUtensorMap *)map_a;
    const CUtensorMap &mb = *(const CUtensorMap *)map_b;
    __nv_bfloat16 *c = (__nv_bfloat16 *)C;
    if (!preemptible)
        gemm_bf16_kernel<false, false><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    else if (abort_inflight)
        gemm_bf16_kernel<true, true><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    else
        gemm_bf16_kernel<true, false><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    return cudaGetLastError();
}

} // namespace xpk
