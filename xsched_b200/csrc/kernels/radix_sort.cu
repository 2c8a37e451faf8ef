// Preemptible persistent int32 LSD radix sort (8-bit digits, 4 passes, ascending).
//
// One persistent kernel walks a single ticket sequence of 5*T tiles (T = ceil(n / 4096)):
//   phase 0, tickets [0,T):       digit histograms of all four bytes of every key, summed
//                                 into hist[4][256] with integer atomics (order-free, exact);
//   phase p=1..4, tickets [pT,(p+1)T): scatter pass p-1 over tile j = ticket - pT.
// A tile of phase p starts only after all T tiles of phase p-1 have finished (a counter per
// phase in the control block).  Tickets are claimed in increasing order by resident CTAs and
// a claimed tile only ever waits on smaller tickets, so the waits cannot deadlock; they are
// bounded all the same and raise an error instead of spinning forever.
//
// Inside a scatter tile (256 threads x 16 keys, keys held warp-striped so that load order is
// preserved; four CTAs per SM, so that one CTA's barriers and look-back waits are covered by the others):
//   * each warp ranks its keys item by item: every lane ORs its lane bit into a shared-memory word
//     selected by (warp, digit), reads the word back — the mask of lanes holding the same digit — and the
//     warp's running counter of that digit; its rank is counter + number of lower lanes in the mask; the
//     lowest lane of the mask advances the counter and clears the word (stable within the warp; two
//     alternating mask tables make two warp barriers per item enough);
//   * warp counters are prefix-summed across warps, giving stable ranks within the tile;
//   * the tile's per-digit counts are published and the exclusive prefix over earlier tiles
//     is obtained by decoupled look-back (one thread per digit);
//   * keys are staged in shared memory in ranked order and written out so that consecutive
//     threads write consecutive addresses of the same digit's run.
//
// HBM traffic: one read for the histograms plus a read and a write per pass:
// (1 + 2*4) * 4n bytes.  Source keys are read with ld.global.cg: a buffer read in pass p is
// rewritten by other CTAs in pass p+1 and read again in pass p+2 by this same kernel, so a
// line cached in L1 would be stale.
//
// The cursor is the ticket counter: a preempted launch leaves every claimed tile finished,
// the phase counters and look-back words stay in global memory, and the relaunch continues
// with the next ticket.  Integer arithmetic only, so the result is bit-exact by construction.
#include "pk_common.cuh"
#include "xsched_b200/pk.h"

#include <mutex>

namespace xpk {

void note_launches(unsigned n);      // pk_api.cu: the library-wide launch counter

constexpr int kSortThreads = 256;
constexpr int kSortWarps   = kSortThreads / 32;
constexpr int kSortItems   = 16;                  // keys per thread (even: ranks are kept two per register; 20 and 24 measured no faster)
constexpr int kSortTile    = kSortThreads * kSortItems;   // 4096 keys
static_assert(kSortItems % 2 == 0 && kSortTile <= 65536, "ranks are packed as 16-bit pairs");
constexpr int kSortCtasPerSm = 4;
static_assert(kSortThreads == 256, "one thread per digit: the scans and the look-back assume 256 threads");
constexpr int kRadix       = 256;
constexpr uint32_t kFlagAgg  = 1u << 30;
constexpr uint32_t kFlagInc  = 2u << 30;
constexpr uint32_t kValMask  = (1u << 30) - 1u;
constexpr unsigned long long kSpinLimitNs = 2000000000ull;   // 2 s per wait

constexpr uint32_t kErrSortPhaseWait = 0x50000001u;
constexpr uint32_t kErrSortLookback  = 0x50000002u;

struct SortSmem {
    uint32_t warp_hist[kSortWarps][kRadix];   // per-warp digit counters -> exclusive prefix over warps
    uint32_t match[2][kSortWarps][kRadix];    // lane masks per (item parity, warp, digit); all zero between uses
    uint32_t keys[kSortTile];                 // ranked staging / phase-0 histograms
    uint32_t tile_off[kRadix];                // exclusive digit offsets inside the tile
    uint32_t gbase[kRadix];                   // dst index = gbase[digit] + rank in tile (mod 2^32)
    uint32_t scan_tmp[kSortWarps];
    ClaimCtx claim;                           // thread 0's copy of the frozen cursor fields
    uint32_t tile;                            // tile handed from thread 0 to the CTA (kNoTile32 = none)
    uint32_t bail;
};
constexpr uint32_t kNoTile32 = 0xFFFFFFFFu;   // 5 * T tickets always fit 32 bits (n <= 2^30)

__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed(uint32_t *p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Signed ascending order == unsigned order of the key with its sign bit flipped.
__device__ __forceinline__ uint32_t twiddle(uint32_t k) { return k ^ 0x80000000u; }

// Exclusive scan of 256 values, one per thread; all threads call.
__device__ __forceinline__ uint32_t block_excl_scan256(uint32_t v, SortSmem &sm, uint32_t *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sm.scan_tmp[warp] = inc;
    __syncthreads();
    uint32_t add = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
        uint32_t t = sm.scan_tmp[w];
        if (w < warp) add += t;
        tot += t;
    }
    __syncthreads();
    if (total) *total = tot;
    return inc - v + add;
}

// Wait until *counter >= target.  Thread 0 spins; returns false (and raises `code`) on timeout
// or when another CTA has already raised an error.
__device__ __forceinline__ bool wait_counter(Ctl *ctl, const unsigned long long *counter,
                                             unsigned long long target, uint32_t code) {
    if (ld_acquire64(counter) >= target) return true;
    const unsigned long long t0 = global_ns();
    uint32_t it = 0;
    while (ld_acquire64(counter) < target) {
        __nanosleep(64);
        if ((++it & 255u) == 0) {
            if (ld_relaxed(&ctl->error) != 0) return false;
            if (global_ns() - t0 > kSpinLimitNs) { raise_error(ctl, code); return false; }
        }
    }
    return true;
}

constexpr int kLookbackWindow = 8;      // predecessor tiles read per round of the look-back

// The ticket claim is two dependent round trips to L2 (flag, then the ticket atomic) that one thread makes while
// 255 wait; measured at a fifth of a tile's time when done at the top of the loop.  It is therefore spread over
// the tile: thread 0 reads the preempt flag at the top of tile i (used much later), takes the ticket of tile
// i+1 just before it starts writing tile i out, and hands the tile id to the CTA at the closing barrier.  The
// ticket is taken late on purpose: tickets must be taken in the order in which CTAs become free, or the
// look-back of ticket t+1 waits for a CTA that still has most of another tile to do before it ranks ticket t.
// So the flag a CTA acts on is at most one tile old: after the flag is raised a CTA finishes the tile it is in
// and possibly one more (about 10 us each).  A claimed ticket is always processed by the CTA that took it, which
// the look-back of later tickets relies on.
template <bool kPoll>
__global__ void __launch_bounds__(kSortThreads, kSortCtasPerSm)
radix_sort_kernel(Ctl *ctl, uint32_t *keys, uint32_t *tmp, uint32_t *hist, uint32_t *state,
                  unsigned long long n64, unsigned long long T64, unsigned long long launch_no) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmem &sm = *reinterpret_cast<SortSmem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n = (uint32_t)n64, T = (uint32_t)T64;     // n <= 2^30
    unsigned long long *phase_done = ctl->user;       // [0..4]
    uint32_t done = 0;
    uint32_t goff = 0;            // exclusive global offset of digit `tid` in pass `goff_pass`
    int goff_pass = -1;
    note_start(ctl);
    // The mask tables are all zero whenever no warp is between its two barriers of an item.
    for (int i = tid; i < 2 * kSortWarps * kRadix; i += kSortThreads) (&sm.match[0][0][0])[i] = 0;
    if (tid == 0) {
        sm.claim = load_claim_ctx(ctl);               // frozen while a launch runs
        const unsigned long long first = claim_tile<kPoll>(ctl);
        sm.tile = first == kNoTile ? kNoTile32 : (uint32_t)first;
        sm.bail = 0;
    }
    __syncthreads();
    uint32_t ticket = sm.tile;
    uint32_t cur_phase = kNoTile32;                   // phase whose predecessor is known to be complete

    while (ticket != kNoTile32) {
        const uint32_t phase = ticket / T;
        if (phase != cur_phase) {
            // First tile of a phase for this CTA: every tile of the phase before must have finished.  (Uniform.)
            if (tid == 0 && phase > 0 && !wait_counter(ctl, &phase_done[phase - 1], T, kErrSortPhaseWait)) sm.bail = 1;
            __syncthreads();
            if (sm.bail) break;
            cur_phase = phase;
        }
        const uint32_t j = ticket - phase * T;
        const uint32_t lo = j * (uint32_t)kSortTile;
        const uint32_t count = min(n - lo, (uint32_t)kSortTile);
        uint32_t flag_now = 0;
        if constexpr (kPoll) { if (tid == 0) flag_now = ld_flag(ctl->flag); }       // consumed a barrier later
        unsigned long long next_seq = kNoTile;        // thread 0: ticket number taken for the next tile
        uint32_t next = kNoTile32;

        if (phase == 0) {
            // ---- histograms of all four digits of this tile's keys ----
            uint32_t *h = sm.keys;                     // [4][256]
            for (int i = tid; i < 4 * kRadix; i += kSortThreads) h[i] = 0;
            __syncthreads();
            for (uint32_t i = tid; i < count; i += kSortThreads) {
                const uint32_t k = twiddle(__ldcg(keys + lo + i));
                atomicAdd(&h[0 * kRadix + (k & 255u)], 1u);
                atomicAdd(&h[1 * kRadix + ((k >> 8) & 255u)], 1u);
                atomicAdd(&h[2 * kRadix + ((k >> 16) & 255u)], 1u);
                atomicAdd(&h[3 * kRadix + (k >> 24)], 1u);
            }
            __syncthreads();
            if (tid == 0 && flag_now == 0) next_seq = take_ticket(ctl);
            for (int i = tid; i < 4 * kRadix; i += kSortThreads) {
                const uint32_t c = h[i];
                if (c) atomicAdd(&hist[i], c);
            }
        } else {
            const int pass = (int)phase - 1;
            const int shift = pass * 8;
            const uint32_t *src = (pass & 1) ? tmp : keys;
            uint32_t *dst = (pass & 1) ? keys : tmp;
            uint32_t *st = state + ((unsigned long long)pass * T + j) * kRadix;      // 4 * T * 256 words can pass 2^32 bytes

            // ---- load (warp-striped) ----
            uint32_t key[kSortItems];
            uint32_t rank2[kSortItems / 2];            // two 16-bit ranks per word (a rank is below the tile size)
            const uint32_t wbase = warp * (32 * kSortItems);
#pragma unroll
            for (int i = 0; i < kSortItems; ++i) {
                const uint32_t idx = wbase + i * 32 + lane;
                key[i] = idx < count ? twiddle(__ldcg(src + lo + idx)) : 0xFFFFFFFFu;
            }
            // Each warp clears its own counter row (no other warp touches it before the block barrier below).
            volatile uint32_t *wh = sm.warp_hist[warp];
#pragma unroll
            for (int i = 0; i < kRadix / 32; ++i) wh[i * 32 + lane] = 0;
            __syncwarp();

            // ---- stable rank inside the warp ----
            const uint32_t lane_bit = 1u << lane, lower = lane_bit - 1u;
#pragma unroll
            for (int i = 0; i < kSortItems; ++i) {
                const uint32_t d = (key[i] >> shift) & 255u;
                uint32_t *mw = &sm.match[i & 1][warp][d];
                atomicOr(mw, lane_bit);
                __syncwarp();
                const uint32_t mask = *(volatile uint32_t *)mw;      // lanes of this item with the same digit
                const uint32_t base = wh[d];                         // keys of earlier items with that digit
                __syncwarp();
                if ((mask & lower) == 0) {                           // lowest lane of the group
                    wh[d] = base + __popc(mask);
                    *(volatile uint32_t *)mw = 0;
                }
                const uint32_t r = base + __popc(mask & lower);
                if (i & 1) rank2[i >> 1] |= r << 16; else rank2[i >> 1] = r;
                // No barrier here: the next item uses the other mask table, and its first barrier orders this
                // counter update before the next read of the counters.
            }
            __syncthreads();

            // ---- per-digit totals, exclusive prefix over warps (thread t owns digit t) ----
            uint32_t cnt = 0;
#pragma unroll
            for (int w = 0; w < kSortWarps; ++w) {
                const uint32_t c = sm.warp_hist[w][tid];
                sm.warp_hist[w][tid] = cnt;
                cnt += c;
            }
            // Publish early so later tiles can look back through this one.
            st_relaxed(st + tid, (j == 0 ? kFlagInc : kFlagAgg) | cnt);
            const uint32_t toff = block_excl_scan256(cnt, sm, nullptr);
            // Global start of each digit in this pass: the same for every tile of a pass, so it is computed when
            // this CTA meets the pass for the first time and kept in a register (the condition is uniform).
            if (goff_pass != pass) {
                goff = block_excl_scan256(__ldcg(hist + pass * kRadix + tid), sm, nullptr);
                goff_pass = pass;
            }

            // ---- decoupled look-back over earlier tiles of this pass, kLookbackWindow tiles per round ----
            uint32_t excl = 0;
            bool ok = true;
            if (j > 0) {
                long long k = (long long)j - 1;                  // nearest tile not yet accounted for
                const uint32_t *row0 = state + (unsigned long long)pass * T * kRadix + tid;
                unsigned long long t0 = 0;
                uint32_t it = 0;
                bool found = false;
                while (!found) {
                    // The nearest unaccounted tile first, alone: while it is unpublished nothing else is worth reading.
                    uint32_t s0 = ld_relaxed(row0 + (unsigned long long)k * kRadix);
                    while ((s0 & ~kValMask) == 0) {
                        __nanosleep(32);
                        if ((++it & 127u) == 0) {
                            if (ld_relaxed(&ctl->error) != 0) { ok = false; break; }
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > kSpinLimitNs) { raise_error(ctl, kErrSortLookback); ok = false; break; }
                        }
                        s0 = ld_relaxed(row0 + (unsigned long long)k * kRadix);
                    }
                    if (!ok) break;
                    excl += s0 & kValMask;
                    if ((s0 & ~kValMask) == kFlagInc) break;
                    --k;
                    // Then a window of older tiles in one round trip; they are accounted for in order up to the
                    // first inclusive word, or up to the first word that is not published yet.
                    uint32_t sv[kLookbackWindow];
#pragma unroll
                    for (int w = 0; w < kLookbackWindow; ++w)
                        sv[w] = (k - w) >= 0 ? ld_relaxed(row0 + (unsigned long long)(k - w) * kRadix) : kFlagInc;   // before tile 0: nothing
                    int used = 0;
#pragma unroll
                    for (int w = 0; w < kLookbackWindow; ++w) {
                        const uint32_t f = sv[w] & ~kValMask;
                        if (found || used != w || f == 0) continue;
                        excl += sv[w] & kValMask;
                        used = w + 1;
                        if (f == kFlagInc) found = true;
                    }
                    k -= used;
                }
                if (ok) st_relaxed(st + tid, kFlagInc | ((excl + cnt) & kValMask));
            }
            sm.tile_off[tid] = toff;
            sm.gbase[tid] = goff + excl - toff;
            if (!ok) sm.bail = 1;
            __syncthreads();
            if (sm.bail) break;

            // ---- stage in ranked order ----
#pragma unroll
            for (int i = 0; i < kSortItems; ++i) {
                const uint32_t d = (key[i] >> shift) & 255u;
                const uint32_t r = (i & 1) ? rank2[i >> 1] >> 16 : rank2[i >> 1] & 0xFFFFu;
                sm.keys[sm.tile_off[d] + sm.warp_hist[warp][d] + r] = key[i];
            }
            __syncthreads();

            if (tid == 0 && flag_now == 0) next_seq = take_ticket(ctl);      // result needed after the write-out

            // ---- write out: consecutive threads -> consecutive addresses per digit run ----
#pragma unroll 4
            for (uint32_t idx = tid; idx < count; idx += kSortThreads) {
                const uint32_t k = sm.keys[idx];
                const uint32_t d = (k >> shift) & 255u;
                dst[sm.gbase[d] + idx] = twiddle(k);
            }
        }
        if (tid == 0) {
            const unsigned long long nt = next_seq == kNoTile ? kNoTile : resolve_ticket(ctl, sm.claim, next_seq);
            sm.tile = nt == kNoTile ? kNoTile32 : (uint32_t)nt;
        }
        __syncthreads();
        next = sm.tile;
        if (tid == 0) {
            __threadfence();
            atomicAdd(&phase_done[phase], 1ull);
        }
        ++done;
        ticket = next;
    }
    __syncthreads();
    if (tid == 0) cta_exit(ctl, done, launch_no);
}

size_t sort_smem_bytes() { return sizeof(SortSmem); }

cudaError_t sort_prepare() {
    cudaError_t e = cudaFuncSetAttribute(radix_sort_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SortSmem));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(radix_sort_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SortSmem));
}

int sort_ctas_per_sm(bool preemptible) {
    int a = 0;
    if (preemptible) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&a, radix_sort_kernel<true>, kSortThreads, sizeof(SortSmem));
    else             cudaOccupancyMaxActiveBlocksPerMultiprocessor(&a, radix_sort_kernel<false>, kSortThreads, sizeof(SortSmem));
    return a < 1 ? 1 : a;
}

unsigned long long sort_tiles(unsigned long long n) { return (n + kSortTile - 1) / kSortTile; }

cudaError_t launch_sort(bool preemptible, Ctl *ctl, uint32_t *keys, uint32_t *tmp, uint32_t *hist,
                        uint32_t *state, unsigned long long n, unsigned long long launch_no,
                        int grid, cudaStream_t stream) {
    const unsigned long long T = sort_tiles(n);
    if (preemptible)
        radix_sort_kernel<true><<<grid, kSortThreads, sizeof(SortSmem), stream>>>(ctl, keys, tmp, hist, state, n, T, launch_no);
    else
        radix_sort_kernel<false><<<grid, kSortThreads, sizeof(SortSmem), stream>>>(ctl, keys, tmp, hist, state, n, T, launch_no);
    return cudaGetLastError();
}

} // namespace xpk

// ---------------------------------------------------------------------------------------------------
// xpkSortNoAlloc: the same sort for callers that must not allocate.
//
// Everything the kernel needs beyond the caller's two key buffers — the control block, the four digit
// histograms and the look-back words — lives in one statically sized array in device memory that is part
// of this library's image.  The host side only ever handles its address, obtained once per device with
// cudaGetSymbolAddress (the array's name is not a device pointer in host code).
namespace {

constexpr unsigned long long kNoAllocMaxKeys = XPK_SORT_NOALLOC_MAX_KEYS;
constexpr unsigned long long kNoAllocMaxTiles = (kNoAllocMaxKeys + xpk::kSortTile - 1) / xpk::kSortTile;
constexpr size_t kNoAllocCtlBytes = (sizeof(xpk::Ctl) + 255) / 256 * 256;
constexpr size_t kNoAllocHistBytes = 4096;
constexpr size_t kNoAllocStateBytes = (size_t)4 * kNoAllocMaxTiles * xpk::kRadix * sizeof(uint32_t);
constexpr size_t kNoAllocBytes = kNoAllocCtlBytes + kNoAllocHistBytes + kNoAllocStateBytes;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// Prepares the control block in place: cursor at tile 0, private flag lowered, no mailbox.
__global__ void noalloc_init_ctl(xpk::Ctl *ctl, unsigned long long total) {
    unsigned long long *w = reinterpret_cast<unsigned long long *>(ctl);
    for (unsigned i = threadIdx.x; i < 256 / 8; i += blockDim.x) w[i] = 0;     // bytes [0,256): state + header
    __syncthreads();
    if (threadIdx.x == 0) {
        ctl->total = total;
        ctl->own_flag = 0;
        ctl->flag = &ctl->own_flag;
        ctl->mailbox = nullptr;
    }
}

struct NoAllocDevice {
    unsigned char *base = nullptr;     // device address of g_noalloc_scratch on this device
    int grid_limit = 0;                // SMs x resident CTAs per SM
};
std::mutex g_noalloc_mu;
NoAllocDevice g_noalloc_dev[64];

} // namespace

extern "C" xpkResult xpkSortNoAlloc(int32_t *keys, int32_t *tmp, uint64_t n, void *stream) {
    if (keys == nullptr || tmp == nullptr || n == 0) return XPK_ERR_INVALID_VALUE;
    if (n > kNoAllocMaxKeys) return XPK_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(keys) & 15u) || (reinterpret_cast<uintptr_t>(tmp) & 15u)) return XPK_ERR_ALIGNMENT;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return XPK_ERR_CUDA;
    NoAllocDevice d;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (g_noalloc_dev[dev].base == nullptr) {
            // First call on this device: resolve the array's device address and size the grid.  None of
            // these calls allocates, but they are not stream operations, so make this first call outside
            // any stream capture.
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return XPK_ERR_CUDA;
            if (xpk::sort_prepare() != cudaSuccess) return XPK_ERR_CUDA;
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return XPK_ERR_CUDA;
            g_noalloc_dev[dev].grid_limit = sms * xpk::sort_ctas_per_sm(/*preemptible=*/false);
            g_noalloc_dev[dev].base = static_cast<unsigned char *>(p);
        }
        d = g_noalloc_dev[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    xpk::Ctl *ctl = reinterpret_cast<xpk::Ctl *>(d.base);
    uint32_t *hist = reinterpret_cast<uint32_t *>(d.base + kNoAllocCtlBytes);
    uint32_t *state = reinterpret_cast<uint32_t *>(d.base + kNoAllocCtlBytes + kNoAllocHistBytes);
    const unsigned long long T = xpk::sort_tiles(n);
    // The array keeps whatever the previous call left: the histograms and the look-back words of the T
    // tiles this call uses must start at zero.
    if (cudaMemsetAsync(hist, 0, kNoAllocHistBytes + (size_t)4 * T * xpk::kRadix * sizeof(uint32_t), s) != cudaSuccess) return XPK_ERR_CUDA;
    noalloc_init_ctl<<<1, 32, 0, s>>>(ctl, 5 * T);
    if (cudaGetLastError() != cudaSuccess) return XPK_ERR_CUDA;
    unsigned long long grid = (unsigned long long)d.grid_limit;
    if (grid > 5 * T) grid = 5 * T;
    if (xpk::launch_sort(/*preemptible=*/false, ctl, reinterpret_cast<uint32_t *>(keys), reinterpret_cast<uint32_t *>(tmp), hist, state, n,
                         /*launch_no=*/1, (int)grid, s) != cudaSuccess)
        return XPK_ERR_CUDA;
    xpk::note_launches(2);       // the control-block set-up kernel and the sort kernel
    return XPK_SUCCESS;
}
