// Preemptible persistent bf16 GEMM for sm_100a, two-CTA form: C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulate.
//
// What bounds the one-CTA form (gemm_tcgen05.cu) is not the tensor pipe but the delivery of operands from L2 to
// the SMs: its 256x256 tile needs 64 bytes per SM and tensor-pipe cycle, and three tile shapes measured the same
// ~11 TB/s of operand traffic over the chip whatever their demand.  Without multicast loads the only way down is a
// larger tile per unit of tensor memory, and the largest one is a pair of CTAs (the two SMs of a TPC) sharing a
// 512x256 tile through tcgen05.mma.cta_group::2: per 64-deep k-block each CTA stages 2 x 128 rows of A and its
// 128-row half of B (48 KB; 48 bytes per SM and tensor-pipe cycle, a quarter less) and holds the two 128x256 fp32
// accumulators of its rows in its 512 tensor-memory columns.  Two MMAs (M256 N256 K16) per K step, one per
// 256-row half of the tile, read the same B.  No load is multicast: every CTA fetches its own operand blocks with
// its own TMA loads.
//
// Roles per CTA (352 threads; rank = position in the pair, rank 0 = leader):
//   warp 0, one lane   leader: claims tiles (a ticket taken one tile ahead, so that the atomic's round trip passes
//                      under the loads of the tile before; handed back if the flag goes up first), publishes
//                      each tile id on a 4-slot ring in BOTH CTAs' shared memory and loads its operand blocks;
//                      with kAbort it stores, every kAbortPollEvery k-blocks, how far the tile will be loaded
//                      into the peer's `permit` word;
//                      peer: takes tiles from its ring and issues exactly as many k-blocks as `permit` allows
//                      (whole tiles without kAbort), so the two rings never disagree and an abort needs no
//                      negotiation.
//                      Both CTAs' loads complete on the LEADER's `full` barrier (cp.async.bulk.tensor
//                      .cta_group::2), which expects the bytes of both.
//   warp 1, one lane   leader only: issues the MMAs; tcgen05.commit ... multicast::cluster arrives on the
//                      `empty` (stage consumed) and `tmem_full` (accumulators complete) barriers of both CTAs.
//   warps 2-9          epilogue of the CTA's own 2 x 128 rows: two groups of four warps, one per accumulator,
//                      tcgen05.ld, round to bf16, store; they free the accumulators by arriving on the
//                      leader's `tmem_empty` barrier (2 x 8 arrivals).
//   warp 10, one lane  leader only: watches the preempt flag (three looks per microsecond) and notes a raised flag
//                      in shared memory for the producer; in the grid's first CTA it also relays the host's
//                      early flag (see pk_common.cuh).
//
// Preemption is the one-CTA form's: no tile is started after the flag is up; with kAbort the leader's producer looks
// at the watcher's word every kAbortPollEvery k-blocks, stops loading, hands the tile back and tells both CTAs which
// k-block and tile sequence number were the first not issued.  A tile's accumulation order is fixed (k ascending,
// one accumulator per output element), so its bf16 result does not depend on which pair or launch produced it —
// nor on which of the two forms.
//
// Life of the pair.  Remote shared memory may only be touched while its CTA runs, so: (1) a cluster barrier
// before anything remote; the leader's reading of the flag decides for both whether the launch leaves at once;
// (2) a cluster barrier after barrier initialisation and tensor-memory allocation; (3) a cluster barrier before
// either CTA frees tensor memory and leaves.  Every other wait is bounded (2 s): on expiry the CTA raises an
// error in both CTAs, all roles leave their loops, loads and MMAs in flight are waited for (bounded), tensor
// memory is freed and the kernel returns with status ERROR.
#include "gemm_ptx.cuh"

namespace xpk {
namespace pair {

constexpr int kTileM = 512, kTileN = 256, kBK = 64;     // tile of the pair
constexpr int kMmaM = 256;                              // rows per MMA of the pair (128 per CTA), one accumulator each
constexpr int kHalf = 128;                              // rows of one operand block in one CTA
constexpr int kStages = 4;
constexpr int kSchedSlots = 4;
constexpr int kEpiWarps = 8;
constexpr int kRelayWarp = 2 + kEpiWarps;
constexpr int kThreads = 64 + 32 * kEpiWarps + 32;
constexpr uint32_t kOperandBytes = kHalf * kBK * 2;     // 16 KiB
constexpr uint32_t kStageBytes = 3 * kOperandBytes;     // per CTA and stage: two blocks of A, one of B
constexpr uint32_t kTmemCols = 512;
// 11 warps sit 3+3+3+2 on the SM's four register files of 16 K: at 128 registers per thread every file keeps room
// for warps of other kernels beside this CTA (four warps of 40 registers, say).
constexpr int kMaxRegs = 128;
constexpr int kAbortPollEvery = 2;
constexpr uint32_t kParkNs = 1000;                      // longest a waiting thread stays parked before it looks at the abort word again
constexpr int kPairRasterGroup = 8;                     // row-blocks per raster group (8 x 512 rows)

constexpr unsigned long long kTileMask = (1ull << 40) - 1;     // kNoTile + 1 == 0 under the mask

constexpr uint32_t kErrProducer = 0x61000001u;
constexpr uint32_t kErrMma      = 0x61000002u;
constexpr uint32_t kErrEpilogue = 0x61000003u;
constexpr uint32_t kErrDrain    = 0x61000004u;
constexpr uint32_t kErrPermit   = 0x61000005u;

struct PairShared {
    unsigned long long full[kStages];             // used in the leader: bytes of both CTAs' loads
    unsigned long long empty[kStages];            // each CTA's own; the leader's commit arrives on both
    unsigned long long tmem_full;                 // each CTA's own; the leader's commit arrives on both
    unsigned long long tmem_empty;                // used in the leader: 2 x kEpiWarps arrivals
    unsigned long long sched_full[kSchedSlots];   // each CTA's own ring of tiles, filled by its own producer
    unsigned long long sched_empty[kSchedSlots];  // used in the leader: MMA thread + peer producer + 2 x kEpiWarps
    unsigned long long drain;
    unsigned long long sched_tile[kSchedSlots];
    unsigned long long tile_word[kSchedSlots];    // peer: (use count of the slot << 40 | tile + 1), stored by the leader in one piece
    unsigned long long permit;           // peer: k-blocks the leader has issued since the launch began
    unsigned long long abort_kseq;       // first k-block sequence number that was not loaded
    unsigned long long abort_tile_seq;   // sequence number of the abandoned tile
    uint32_t abort;                      // 1: abandon from abort_* on; 2: error, leave now
    uint32_t tmem_base;
    uint32_t relay_stop;
    uint32_t stop_at_start;              // leader: the flag was already up when the launch began
    uint32_t flag_seen;                  // leader: the watcher has seen the preempt flag raised
    uint32_t watch_off;                  // leader: the watcher has given up (a launch longer than its limit); poll the flag directly
};
constexpr uint32_t kStagingBytes = 32 * 64 * 2;         // per epilogue warp: 32 rows x 64 bf16, where rows are regrouped for coalesced stores
constexpr size_t kSharedBlockBytes = (sizeof(PairShared) + 127) & ~(size_t)127;
constexpr size_t kSmemBytes = 1024 /*align slack*/ + kStages * kStageBytes + kSharedBlockBytes + kEpiWarps * kStagingBytes;

// ---- cluster and .cta_group::2 instructions ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `p` (own shared memory) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t in_cta(const void *p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
// Arrival on a barrier of either CTA.  No data travels with it (the arrivals that use it only say "done reading"),
// so it carries no cluster-scope release: that fence costs about a microsecond.
__device__ __forceinline__ void remote_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void remote_st_u64(uint32_t addr, unsigned long long v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" :: "r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ void remote_st_relaxed_u64(uint32_t addr, unsigned long long v) {
    asm volatile("st.relaxed.cluster.shared::cluster.u64 [%0], %1;" :: "r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ void remote_st_release_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.release.cluster.shared::cluster.u32 [%0], %1;" :: "r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t remote_ld_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const void *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.cluster.shared::cta.u64 %0, [%1];" : "=l"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
// Tile load into this CTA's shared memory whose bytes are counted on `bar`, a barrier of either CTA of the pair
// (an address in the cluster's shared window).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Arrives on the barrier at this offset in both CTAs once the MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_both(void *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_commit_own(void *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Instruction descriptor for kind::f16: D fp32, A/B bf16, both K-major, N=256, M=256 (128 rows per CTA).
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kMmaM >> 4) << 24);


struct Ctx {
    PairShared *sh;
    Ctl *ctl;
    uint32_t peer_abort;     // the other CTA's `abort` word
};

__device__ __forceinline__ void raise_in_both(const Ctx &cx, uint32_t errcode) {
    raise_error(cx.ctl, errcode);
    *(volatile uint32_t *)&cx.sh->abort = 2u;
    remote_st_release_u32(cx.peer_abort, 2u);
}

// Bounded wait.  kRemote only documents that threads of the other CTA arrive on the barrier.
// `quit()` is evaluated between polls; returns false when it fired or on timeout.
template <bool kRemote, class Quit>
__device__ __forceinline__ bool bounded_wait(void *bar, uint32_t parity, const Ctx &cx, uint32_t errcode, Quit quit) {
    uint32_t it = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait_hint(bar, parity, kParkNs)) {
        if (quit()) return false;
        if ((++it & 0xFFu) == 0) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) {
                raise_in_both(cx, errcode);
                return false;
            }
        }
    }
    return true;
}

template <bool kPreemptible, bool kAbort>
__global__ void __cluster_dims__(2, 1, 1) __maxnreg__(kMaxRegs)
gemm_bf16_pair_kernel(Ctl *ctl, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      __nv_bfloat16 *__restrict__ C, uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *smem_a0 = smem;                                   // rows [0,256) of the tile: this CTA's 128 of them
    unsigned char *smem_a1 = smem + kStages * kOperandBytes;         // rows [256,512)
    unsigned char *smem_b = smem + 2 * kStages * kOperandBytes;
    PairShared *sh = reinterpret_cast<PairShared *>(smem + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const uint32_t m_tiles = (M + kTileM - 1) / kTileM, n_tiles = N / kTileN;   // M is a multiple of 128: the last row-block may be half full
    const uint32_t k_blocks = K / kBK;
    note_start(ctl);

    // (1) Both CTAs run from here on.  A launch that starts with the flag already raised (it was queued behind
    // the one being flushed) leaves before setting anything up; the leader's reading decides for the pair.
    if (threadIdx.x == 0) sh->stop_at_start = (kPreemptible && leader) ? ld_flag(ctl->flag) : 0u;
    cluster_sync_all();
    if constexpr (kPreemptible) {
        const uint32_t stop = remote_ld_u32(in_cta(&sh->stop_at_start, 0));
        if (stop != 0) {
            cluster_sync_all();          // the leader stays until the peer has read its word
            if (threadIdx.x == 0) cta_exit(ctl, 0, launch_no);
            return;
        }
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 2 * kEpiWarps);
        for (int i = 0; i < kSchedSlots; ++i) { mbar_init(&sh->sched_full[i], 1); mbar_init(&sh->sched_empty[i], 2 + 2 * kEpiWarps); }
        mbar_init(&sh->drain, 1);
        sh->abort = 0;
        sh->relay_stop = 0;
        sh->flag_seen = 0;
        sh->watch_off = 0;
        sh->permit = 0;
        for (int i = 0; i < kSchedSlots; ++i) sh->tile_word[i] = 0;
        sh->abort_kseq = ~0ull;
        sh->abort_tile_seq = ~0ull;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // One warp of each CTA of the pair allocates (and later frees) the pair's columns.
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                  // (2) barriers and tensor memory of both CTAs are ready
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&sh->tmem_base;

    Ctx cx;
    cx.sh = sh;
    cx.ctl = ctl;
    cx.peer_abort = in_cta(&sh->abort, rank ^ 1u);
    // The abort word, written by this CTA or (with a cluster-scope release, after the words it guards) by the other.
    auto aborted = [&]() -> uint32_t {
        const uint32_t a = *(volatile uint32_t *)&sh->abort;
        if (a != 0u) asm volatile("fence.acq_rel.cluster;" ::: "memory");
        return a;
    };
    unsigned long long tiles_done = 0;     // counted by the leader's first epilogue warp

    if (warp == 0) {
        if (lane == 0 && leader) {
            // ======================= leader's producer: claim + publish + TMA =======================
            const uint32_t peer_tile_word = in_cta(&sh->tile_word[0], 1);
            const uint32_t peer_permit = in_cta(&sh->permit, 1);
            const uint32_t peer_abort_kseq = in_cta(&sh->abort_kseq, 1), peer_abort_tile_seq = in_cta(&sh->abort_tile_seq, 1);
            const uint32_t my_full = smem_u32(&sh->full[0]);
            const ClaimCtx cc = load_claim_ctx(ctl);          // frozen while a launch runs
            // The flag as the watcher (warp kRelayWarp) last saw it: a shared-memory read instead of a round trip
            // to L2 in the middle of the load stream.  The twin never looks.
            auto flag_up = [&]() -> bool {
                if constexpr (!kPreemptible) return false;
                if (*(volatile uint32_t *)&sh->watch_off != 0u) return ld_flag(ctl->flag) != 0;
                return *(volatile uint32_t *)&sh->flag_seen != 0u;
            };
            auto hand_back = [&](unsigned long long ticket) {        // a ticket taken ahead whose tile will not be run here
                const unsigned long long t = resolve_ticket(ctl, cc, ticket);
                if (t != kNoTile) abandon_tile(ctl, t);
            };
            unsigned long long kseq = 0, tseq = 0;
            bool live = true;
            // Tickets are taken one tile ahead: the atomic's round trip passes under the loads of the tile before.
            // A ticket in hand when the flag goes up is handed back (its tile is untouched).
            unsigned long long ticket = take_ticket(ctl);
            while (live) {
                unsigned long long tile;
                if (flag_up()) { hand_back(ticket); tile = kNoTile; }
                else tile = resolve_ticket(ctl, cc, ticket);
                const int slot = (int)(tseq % kSchedSlots);
                const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
                if (!bounded_wait<true>(&sh->sched_empty[slot], sph ^ 1u, cx, kErrProducer, [&] { return aborted() == 2u; })) break;
                sh->sched_tile[slot] = tile;
                mbar_arrive(&sh->sched_full[slot]);
                // To the peer the tile travels as one tagged 64-bit word (no ordering against anything else needed).
                remote_st_relaxed_u64(peer_tile_word + 8u * slot, ((tseq / kSchedSlots + 1) << 40) | ((tile + 1) & kTileMask));
                if (tile == kNoTile) break;
                ticket = take_ticket(ctl);
                uint32_t m_blk, n_blk;
                tile_coords<kPairRasterGroup>(tile, m_tiles, n_tiles, m_blk, n_blk);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if constexpr (kAbort) {
                        if ((kb % kAbortPollEvery) == 0) {
                            if (flag_up()) {
                                abandon_tile(ctl, tile);
                                hand_back(ticket);
                                sh->abort_kseq = kseq;
                                sh->abort_tile_seq = tseq;
                                __threadfence_block();
                                *(volatile uint32_t *)&sh->abort = 1u;
                                remote_st_u64(peer_abort_kseq, kseq);
                                remote_st_u64(peer_abort_tile_seq, tseq);
                                remote_st_release_u32(cx.peer_abort, 1u);
                                live = false;
                                break;
                            }
                            // The peer may issue its halves of the k-blocks up to the next poll (a bare count: it orders no data).
                            remote_st_relaxed_u64(peer_permit, kseq + min((uint32_t)kAbortPollEvery, k_blocks - kb));
                        }
                    }
                    const int stage = (int)(kseq % kStages);
                    const uint32_t ph = (uint32_t)((kseq / kStages) & 1);
                    if (!bounded_wait<false>(&sh->empty[stage], ph ^ 1u, cx, kErrProducer, [&] { return aborted() == 2u; })) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->full[stage], 2 * kStageBytes);
                    tma_load_2d_pair(smem_a0 + stage * kOperandBytes, &map_a, my_full + 8u * stage, (int)(kb * kBK), (int)(m_blk * kTileM));
                    tma_load_2d_pair(smem_a1 + stage * kOperandBytes, &map_a, my_full + 8u * stage, (int)(kb * kBK), (int)(m_blk * kTileM + kMmaM));
                    tma_load_2d_pair(smem_b + stage * kOperandBytes, &map_b, my_full + 8u * stage, (int)(kb * kBK), (int)(n_blk * kTileN));
                    ++kseq;
                }
                ++tseq;
            }
            *(volatile uint32_t *)&sh->relay_stop = 1u;
            // Leave only after every load of the pair that counts on these barriers has landed.
            const unsigned long long first = kseq > (unsigned long long)kStages ? kseq - kStages : 0;
            for (unsigned long long s = first; s < kseq; ++s) {
                const int stage = (int)(s % kStages);
                const uint32_t ph = (uint32_t)((s / kStages) & 1);
                bounded_wait<false>(&sh->full[stage], ph, cx, kErrDrain, [] { return false; });
            }
        } else if (lane == 0) {
            // ======================= peer's producer: follow the leader =======================
            const uint32_t leader_full = in_cta(&sh->full[0], 0), leader_sched_empty = in_cta(&sh->sched_empty[0], 0);
            unsigned long long kseq = 0, tseq = 0;
            bool live = true;
            while (live) {
                const int slot = (int)(tseq % kSchedSlots);
                // The leader's word for this use of the slot; then the tile goes on this CTA's own ring for its epilogue warps.
                unsigned long long word = 0;
                {
                    const unsigned long long want = tseq / kSchedSlots + 1;
                    uint32_t it = 0;
                    unsigned long long t0 = 0;
                    while (((word = ld_relaxed_u64(&sh->tile_word[slot])) >> 40) != want) {
                        __nanosleep(64);
                        if (*(volatile uint32_t *)&sh->abort != 0u) {
                            const uint32_t a = aborted();
                            if (a == 2u || (a == 1u && tseq > *(volatile unsigned long long *)&sh->abort_tile_seq)) { live = false; break; }
                        }
                        if ((++it & 0xFFu) == 0) {
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > kWaitLimitNs) { raise_in_both(cx, kErrProducer); live = false; break; }
                        }
                    }
                    if (!live) break;
                }
                const unsigned long long tile = (word & kTileMask) == 0 ? kNoTile : (word & kTileMask) - 1;
                sh->sched_tile[slot] = tile;
                mbar_arrive(&sh->sched_full[slot]);
                remote_arrive(leader_sched_empty + 8u * slot);
                if (tile == kNoTile) break;
                uint32_t m_blk, n_blk;
                tile_coords<kPairRasterGroup>(tile, m_tiles, n_tiles, m_blk, n_blk);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    // With in-flight aborts the leader says, kAbortPollEvery k-blocks at a time, how far this tile will be loaded;
                    // without them a published tile is always loaded whole.
                    if constexpr (kAbort) {
                        uint32_t it = 0;
                        unsigned long long t0 = 0;
                        while (ld_relaxed_u64(&sh->permit) <= kseq) {
                            __nanosleep(200);                      // a permit comes every kAbortPollEvery k-blocks (about a microsecond and a half)
                            if (*(volatile uint32_t *)&sh->abort != 0u) {
                                const uint32_t a = aborted();
                                if (a == 2u || (a == 1u && kseq >= *(volatile unsigned long long *)&sh->abort_kseq)) { live = false; break; }
                            }
                            if ((++it & 0xFFu) == 0) {
                                const unsigned long long now = global_ns();
                                if (t0 == 0) t0 = now;
                                else if (now - t0 > kWaitLimitNs) { raise_in_both(cx, kErrPermit); live = false; break; }
                            }
                        }
                        if (!live) break;
                    }
                    const int stage = (int)(kseq % kStages);
                    const uint32_t ph = (uint32_t)((kseq / kStages) & 1);
                    if (!bounded_wait<false>(&sh->empty[stage], ph ^ 1u, cx, kErrProducer, [&] { return aborted() == 2u; })) { live = false; break; }
                    tma_load_2d_pair(smem_a0 + stage * kOperandBytes, &map_a, leader_full + 8u * stage, (int)(kb * kBK), (int)(m_blk * kTileM + kHalf));
                    tma_load_2d_pair(smem_a1 + stage * kOperandBytes, &map_a, leader_full + 8u * stage, (int)(kb * kBK), (int)(m_blk * kTileM + kMmaM + kHalf));
                    tma_load_2d_pair(smem_b + stage * kOperandBytes, &map_b, leader_full + 8u * stage, (int)(kb * kBK), (int)(n_blk * kTileN + kHalf));
                    ++kseq;
                }
                ++tseq;
            }
            // This CTA's loads are counted in the leader.  Every k-block issued here is issued there too and is consumed
            // by an MMA whose commit arrives on `empty` here: waiting for the last of those proves that the loads
            // have landed and that no arrival is still on its way to this CTA's barriers.  After an error (some wait
            // of two seconds ran out) nothing will consume them: loads issued in the last moments get 50 us to land.
            if (aborted() == 2u) {
                for (int i = 0; i < 50; ++i) __nanosleep(1000);
            } else {
                const unsigned long long first = kseq > (unsigned long long)kStages ? kseq - kStages : 0;
                for (unsigned long long s = first; s < kseq; ++s) {
                    const int stage = (int)(s % kStages);
                    const uint32_t ph = (uint32_t)((s / kStages) & 1);
                    bounded_wait<false>(&sh->empty[stage], ph, cx, kErrDrain, [&] { return aborted() == 2u; });
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ======================= MMA issuer (leader only) =======================
        if (lane == 0 && leader) {
            unsigned long long kseq = 0, tseq = 0;
            bool issued_any = false;
            while (true) {
                const int slot = (int)(tseq % kSchedSlots);
                const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
                if (!bounded_wait<false>(&sh->sched_full[slot], sph, cx, kErrMma,
                                         [&] { const uint32_t a = aborted(); return a == 2u || (a == 1u && tseq > *(volatile unsigned long long *)&sh->abort_tile_seq); })) break;
                const unsigned long long tile = sh->sched_tile[slot];
                mbar_arrive(&sh->sched_empty[slot]);
                if (tile == kNoTile) break;
                // Both accumulators must have been drained by both CTAs' epilogues of the previous tile.
                const uint32_t aph = (uint32_t)(tseq & 1);
                if (!bounded_wait<true>(&sh->tmem_empty, aph ^ 1u, cx, kErrMma, [&] { return aborted() == 2u; })) break;
                tc_fence_after();
                const uint32_t d_tmem0 = tmem_base, d_tmem1 = tmem_base + (uint32_t)kTileN;
                bool abandoned = false;
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    const int stage = (int)(kseq % kStages);
                    const uint32_t ph = (uint32_t)((kseq / kStages) & 1);
                    if (!bounded_wait<false>(&sh->full[stage], ph, cx, kErrMma,
                                             [&] { const uint32_t a = aborted(); return a == 2u || (a == 1u && kseq >= *(volatile unsigned long long *)&sh->abort_kseq); })) {
                        abandoned = true;
                        break;
                    }
                    tc_fence_after();
                    // The descriptors name this CTA's shared memory; the peer's tensor core reads the same offsets of its own.
                    const uint64_t adesc0 = make_kmajor_sw128_desc(smem_u32(smem_a0 + stage * kOperandBytes));
                    const uint64_t adesc1 = make_kmajor_sw128_desc(smem_u32(smem_a1 + stage * kOperandBytes));
                    const uint64_t bdesc = make_kmajor_sw128_desc(smem_u32(smem_b + stage * kOperandBytes));
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // +32 bytes per K=16 step inside the 128-byte swizzle atom (address field is >>4).
                        const uint32_t acc_flag = (kb | (uint32_t)k) != 0u;
                        tc_mma_bf16_pair(d_tmem0, adesc0 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), kIdesc, acc_flag);
                        tc_mma_bf16_pair(d_tmem1, adesc1 + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), kIdesc, acc_flag);
                    }
                    issued_any = true;
                    tc_commit_both(&sh->empty[stage]);
                    ++kseq;
                }
                if (abandoned) break;
                tc_commit_both(&sh->tmem_full);
                ++tseq;
            }
            // All issued MMAs must have retired before tensor memory is freed.
            if (issued_any) {
                tc_commit_own(&sh->drain);
                bounded_wait<false>(&sh->drain, 0u, cx, kErrDrain, [] { return false; });
            }
        }
        __syncwarp();
    } else if (warp == kRelayWarp) {
        // ======================= flag watcher (leader only) =======================
        // One thread per pair looks at the preempt flag about three times per microsecond and notes a raised flag in
        // shared memory, where the producer reads it between loads.  In the grid's first CTA it also relays the
        // host's early word into the flag (see pk_common.cuh).  It ends with the producer; past its time limit it
        // hands the polling back to the producer.
        if constexpr (kPreemptible) {
            if (leader && lane == 0) {
                const uint32_t *src = blockIdx.x == 0 ? flag_relay_source(ctl->flag) : nullptr;
                const unsigned long long t0 = global_ns();
                uint32_t it = 0;
                while (*(volatile uint32_t *)&sh->relay_stop == 0u) {
                    if (ld_flag(ctl->flag) != 0u) { *(volatile uint32_t *)&sh->flag_seen = 1u; break; }
                    if (src != nullptr && ld_host_word(src) != 0u) {
                        atomicExch(const_cast<uint32_t *>(ctl->flag), 1u);
                        *(volatile uint32_t *)&sh->flag_seen = 1u;
                        break;
                    }
                    __nanosleep(250);
                    if ((++it & 1023u) == 0 && global_ns() - t0 > 4 * kWaitLimitNs) { *(volatile uint32_t *)&sh->watch_off = 1u; break; }
                }
            }
        }
        __syncwarp();
    } else {
        // ======================= epilogue (warps 2..9: two groups of four): this CTA's 2 x 128 rows =======================
        const uint32_t acc = (uint32_t)(warp - 2) / 4u;           // which accumulator / 256-row half of the tile
        const uint32_t quarter = (uint32_t)(warp & 3);            // TMEM lanes [32q, 32q+32)
        const uint32_t leader_sched_empty = in_cta(&sh->sched_empty[0], 0), leader_tmem_empty = in_cta(&sh->tmem_empty, 0);
        unsigned long long tseq = 0;
        while (true) {
            const int slot = (int)(tseq % kSchedSlots);
            const uint32_t sph = (uint32_t)((tseq / kSchedSlots) & 1);
            // One lane per warp waits (a barrier wakes few waiters sooner than many); the warp follows it.
            bool ok = true;
            if (lane == 0)
                ok = bounded_wait<false>(&sh->sched_full[slot], sph, cx, kErrEpilogue,
                                         [&] { const uint32_t a = aborted(); return a == 2u || (a == 1u && tseq > *(volatile unsigned long long *)&sh->abort_tile_seq); });
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const unsigned long long tile = *(volatile unsigned long long *)&sh->sched_tile[slot];
            __syncwarp();
            if (lane == 0) { if (leader) mbar_arrive(&sh->sched_empty[slot]); else remote_arrive(leader_sched_empty + 8u * slot); }
            if (tile == kNoTile) break;
            uint32_t m_blk, n_blk;
            tile_coords<kPairRasterGroup>(tile, m_tiles, n_tiles, m_blk, n_blk);     // before the wait: its divisions are off the critical path
            const uint32_t aph = (uint32_t)(tseq & 1);
            if (lane == 0)
                ok = bounded_wait<false>(&sh->tmem_full, aph, cx, kErrEpilogue,
                                         [&] { const uint32_t a = aborted(); return a == 2u || (a == 1u && tseq >= *(volatile unsigned long long *)&sh->abort_tile_seq); });
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            // 64 columns at a time: two tensor-memory loads in flight (a load takes several hundred cycles to come
            // back), rounded to bf16, written to this warp's staging block in shared memory with the 16-byte pieces of a
            // row XOR-swizzled by the row number, read back so that eight lanes hold the 128 contiguous bytes of one
            // row, and stored: a store instruction then covers 4 rows x 128 bytes instead of 32 rows x 16 bytes.
            // Tensor memory goes back to the MMA thread as soon as the last loads have landed in registers.
            const uint32_t row0 = m_blk * kTileM + acc * kMmaM + rank * kHalf;
            const bool in_range = row0 < M;                           // the last row-block may be filled in part (M is a multiple of 128)
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * (uint32_t)kTileN;
            uint4 *stg = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(sh) + kSharedBlockBytes + (size_t)(warp - 2) * kStagingBytes);
            __nv_bfloat16 *cbase = C + (size_t)(row0 + quarter * 32u) * N + (size_t)n_blk * kTileN;
#pragma unroll 1
            for (int c = 0; c < kTileN / 64; ++c) {
                uint32_t r[64];
                if (in_range) {
                    tc_ld32(taddr + (uint32_t)(64 * c), *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
                    tc_ld32(taddr + (uint32_t)(64 * c + 32), *reinterpret_cast<uint32_t (*)[32]>(&r[32]));
                    tc_wait_ld();
                }
                if (c == kTileN / 64 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { if (leader) mbar_arrive(&sh->tmem_empty); else remote_arrive(leader_tmem_empty); }
                }
                if (in_range) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 o;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                        o.x = *reinterpret_cast<uint32_t *>(&p0);
                        o.y = *reinterpret_cast<uint32_t *>(&p1);
                        o.z = *reinterpret_cast<uint32_t *>(&p2);
                        o.w = *reinterpret_cast<uint32_t *>(&p3);
                        stg[lane * 8 + (j ^ (lane & 7))] = o;
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3), ch = lane & 7;
                        const uint4 o = stg[rr * 8 + (ch ^ (rr & 7))];
                        *reinterpret_cast<uint4 *>(cbase + (size_t)rr * N + 64 * c + 8 * ch) = o;
                    }
                    __syncwarp();
                }
            }
            if (leader && warp == 2 && lane == 0) ++tiles_done;
            ++tseq;
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                  // (3) nothing of either CTA is still in use by the other
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (warp == 2 && lane == 0) cta_exit(ctl, tiles_done, launch_no);
}

} // namespace pair


cudaError_t gemm_pair_prepare() {
    cudaError_t e;
    e = cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair::kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(pair::gemm_bf16_pair_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair::kSmemBytes);
}

unsigned long long gemm_pair_tiles(uint32_t M, uint32_t N) { return (unsigned long long)((M + pair::kTileM - 1) / pair::kTileM) * (N / pair::kTileN); }

// `grid` must be even (whole pairs); `map_a` / `map_b` are tensor maps with 128-row boxes.
cudaError_t launch_gemm_pair(bool preemptible, bool abort_inflight, Ctl *ctl, const void *map_a, const void *map_b,
                             void *C, uint32_t M, uint32_t N, uint32_t K, unsigned long long launch_no, int grid,
                             cudaStream_t stream) {
    if (grid < 2 || (grid & 1)) return cudaErrorInvalidValue;
    const CUtensorMap &ma = *(const CUtensorMap *)map_a;
    const CUtensorMap &mb = *(const CUtensorMap *)map_b;
    __nv_bfloat16 *c = (__nv_bfloat16 *)C;
    if (!preemptible)
        pair::gemm_bf16_pair_kernel<false, false><<<grid, pair::kThreads, pair::kSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    else if (abort_inflight)
        pair::gemm_bf16_pair_kernel<true, true><<<grid, pair::kThreads, pair::kSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    else
        pair::gemm_bf16_pair_kernel<true, false><<<grid, pair::kThreads, pair::kSmemBytes, stream>>>(ctl, ma, mb, c, M, N, K, launch_no);
    return cudaGetLastError();
}

} // namespace xpk
