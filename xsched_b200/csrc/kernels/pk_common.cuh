// Device-side control block and tile-claim protocol shared by every preemptible kernel.
//
// Role in the preemption path: this replaces the reference's Level-2 preempt buffer
//   | u32 global_exit_flag | u32 rsvd | u64 preempt_idx | {exit_flag, restore_flag} x blocks |
// (platforms/cuda/hal/src/level2/instrument.cpp:177-180, hal/inject/inject.cu:39-42), which
// checkpoints at thread-block granularity from a patched-in prologue.  Here the unit is a
// tile of a persistent kernel and the checkpoint is a cursor:
//
//   * CTAs claim tiles through one ticket counter.  Before each claim they read the
//     preempt flag; once it is raised no further ticket is taken.
//   * A claimed tile is either finished or (GEMM with abort) handed back on a small
//     "returned" list.  Nothing else is in flight when the last CTA leaves.
//   * The last CTA folds the tickets into the cursor {base, returned[]}, publishes
//     {status, tiles_done} to a mailbox in mapped host memory, and re-arms the block.
//   * A relaunch hands out returned tiles first, then fresh tiles from `base`.
//
// Because a tile's result never depends on which CTA computed it or on when, a task that
// is preempted and resumed any number of times writes exactly the bytes of one straight run.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace xpk {

constexpr uint32_t kStatusIdle      = 0;
constexpr uint32_t kStatusRunning   = 1;
constexpr uint32_t kStatusCompleted = 2;
constexpr uint32_t kStatusPreempted = 3;
constexpr uint32_t kStatusError     = 4;

constexpr uint32_t kMaxReturned = 1024;     // >= persistent CTAs x tiles a CTA can hold

// Host-visible result of the most recent launch.  Lives in mapped pinned host memory so
// the host learns the outcome with a plain load.  `seq` is written last.
struct Mailbox {
    unsigned long long tiles_done;
    unsigned long long tiles_total;
    uint32_t status;
    uint32_t error;
    unsigned long long preemptions;
    unsigned long long seq;          // == launch number once the fields above are valid
    unsigned long long start_ns;     // %globaltimer when the launch's first CTA started
    unsigned long long exit_ns;      // %globaltimer when its last CTA left
    unsigned long long pad[1];
};
static_assert(sizeof(Mailbox) == 64, "mailbox is one 64-byte line");

struct __align__(256) Ctl {
    // --- bytes [0,64): claim state; cleared by a task reset ---
    unsigned long long claim_seq;    // tickets handed out by the current launch
    unsigned long long base;         // first tile never claimed (frozen during a launch)
    unsigned long long tiles_done;   // completed tiles over the task's life
    unsigned long long preemptions;  // launches that ended PREEMPTED
    uint32_t n_returned;             // valid entries of returned[cur] (frozen during a launch)
    uint32_t n_abandoned;            // entries appended to returned[cur ^ 1] by this launch
    uint32_t cur;                    // which returned[] buffer this launch consumes
    uint32_t ctas_exited;
    uint32_t error;                  // first error code raised by any CTA (0 = none)
    uint32_t status;
    unsigned long long start_ns;     // %globaltimer at the start of this launch's block 0 (for latency break-downs)
    // --- bytes [64,192): kernel-specific persistent words (radix sort phase counters);
    //     cleared by a task reset ---
    unsigned long long user[16];
    // --- bytes [192,256): set once at task creation ---
    unsigned long long total;        // tiles in the task
    const uint32_t *flag;            // preempt flag polled before each claim
    Mailbox *mailbox;                // device alias of the mapped host mailbox
    uint32_t own_flag;               // storage for a private flag
    uint32_t pad1[9];
    unsigned long long returned[2][kMaxReturned];
};
constexpr size_t kCtlResetBytes = 192;
static_assert(offsetof(Ctl, start_ns) == 56 && offsetof(Ctl, user) == 64 && offsetof(Ctl, total) == 192, "Ctl layout");
static_assert(offsetof(Ctl, returned) == 256, "Ctl layout");

constexpr unsigned long long kNoTile = ~0ull;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// First statement of every kernel: block 0 notes when the launch began to run.
__device__ __forceinline__ void note_start(Ctl *ctl) {
    if (blockIdx.x == 0 && threadIdx.x == 0) ctl->start_ns = global_ns();
}

// A preempt flag is the first word of a 16-byte block.  Bytes [8,16) of the block may hold the device address of a
// word in mapped host memory that the host sets (with a plain store, visible to the GPU within a couple of
// microseconds) just before it enqueues the write of the flag itself (which takes 6-14 us to land): a kernel that
// runs a relay (the GEMM: one spare thread of its first CTA; the stream kernels: one thread in each of their first CTAs) copies a raised host word into the flag, so that the
// tile loops, which only ever poll device memory, see it early.  0 = no such word.
__device__ __forceinline__ const uint32_t *flag_relay_source(const uint32_t *flag) {
    return reinterpret_cast<const uint32_t *>(*reinterpret_cast<const unsigned long long *>(flag + 2));
}
__device__ __forceinline__ uint32_t ld_host_word(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t ld_flag(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The claim in its parts, for kernels that overlap it with work: the cursor fields are frozen while a launch
// runs, so they may be read once; a ticket is one atomic; a ticket number maps to a tile.
struct ClaimCtx {
    unsigned long long nret;     // tickets below this are tiles handed back by an earlier launch
    unsigned long long fresh;    // tiles never claimed so far
    unsigned long long base;     // first of them
    uint32_t cur;                // which returned[] list this launch consumes
};
__device__ __forceinline__ ClaimCtx load_claim_ctx(const Ctl *ctl) {
    ClaimCtx c;
    c.nret = ctl->n_returned;
    c.base = ctl->base;
    c.fresh = ctl->total - c.base;
    c.cur = ctl->cur;
    return c;
}
__device__ __forceinline__ unsigned long long take_ticket(Ctl *ctl) { return atomicAdd(&ctl->claim_seq, 1ull); }
__device__ __forceinline__ unsigned long long resolve_ticket(const Ctl *ctl, const ClaimCtx &c, unsigned long long t) {
    if (t < c.nret) return ctl->returned[c.cur][t];
    t -= c.nret;
    return t < c.fresh ? c.base + t : kNoTile;
}

// One thread per CTA calls this.  Returns a tile index or kNoTile (flag raised or work
// exhausted).  Tickets < n_returned map to tiles handed back by an earlier launch.
// kPoll = false is the twin used to measure what the check costs: the same ticket sequence, the same
// atomics, the flag never read.
template <bool kPoll = true>
__device__ __forceinline__ unsigned long long claim_tile(Ctl *ctl) {
    if constexpr (kPoll) { if (ld_flag(ctl->flag) != 0) return kNoTile; }
    const ClaimCtx c = load_claim_ctx(ctl);
    return resolve_ticket(ctl, c, take_ticket(ctl));
}

// Hand a claimed tile back (its output has not been written, or may be rewritten whole).
__device__ __forceinline__ void abandon_tile(Ctl *ctl, unsigned long long tile) {
    uint32_t slot = atomicAdd(&ctl->n_abandoned, 1u);
    if (slot < kMaxReturned) ctl->returned[ctl->cur ^ 1u][slot] = tile;
    else atomicCAS(&ctl->error, 0u, 0xA0000001u);
}

__device__ __forceinline__ void raise_error(Ctl *ctl, uint32_t code) {
    atomicCAS(&ctl->error, 0u, code);
}

// Called by one thread per CTA after all of the CTA's global writes are ordered before it
// (the caller does __syncthreads(); this function fences).  `done_by_cta` = tiles this CTA
// finished in this launch; `launch_no` = the host's launch counter for this task, echoed
// into the mailbox so the host can tell this launch's result from the previous one's.  The last CTA to arrive folds the launch into the cursor.
__device__ __forceinline__ void cta_exit(Ctl *ctl, unsigned long long done_by_cta,
                                         unsigned long long launch_no) {
    if (done_by_cta) atomicAdd(&ctl->tiles_done, done_by_cta);
    __threadfence();
    const uint32_t prev = atomicAdd(&ctl->ctas_exited, 1u);
    if (prev + 1u != gridDim.x) return;
    __threadfence();

    volatile Ctl *v = ctl;
    const unsigned long long nret   = v->n_returned;
    const unsigned long long fresh  = v->total - v->base;
    unsigned long long consumed     = v->claim_seq;
    if (consumed > nret + fresh) consumed = nret + fresh;
    const unsigned long long ret_used   = consumed < nret ? consumed : nret;
    const unsigned long long fresh_used = consumed - ret_used;
    const uint32_t cur = v->cur, nxt = cur ^ 1u;
    uint32_t n_ab = v->n_abandoned;
    if (n_ab > kMaxReturned) n_ab = kMaxReturned;
    // Returned tiles this launch never reached stay on the list, after the abandoned ones.
    uint32_t out = n_ab;
    for (unsigned long long i = ret_used; i < nret; ++i) {
        if (out < kMaxReturned) ctl->returned[nxt][out++] = ctl->returned[cur][i];
        else { atomicCAS(&ctl->error, 0u, 0xA0000002u); break; }
    }
    ctl->cur = nxt;
    ctl->n_returned = out;
    ctl->n_abandoned = 0;
    ctl->base = v->base + fresh_used;
    ctl->claim_seq = 0;
    ctl->ctas_exited = 0;

    const unsigned long long done = v->tiles_done;
    const uint32_t err = v->error;
    uint32_t st = err ? kStatusError : (done >= v->total ? kStatusCompleted : kStatusPreempted);
    if (st == kStatusPreempted) ctl->preemptions = v->preemptions + 1;
    ctl->status = st;
    const unsigned long long preemptions = v->preemptions, start_ns = v->start_ns;
    if (st == kStatusCompleted) {
        // A finished task re-arms itself: the claim state goes back to what a reset leaves, so that the next
        // submission of the same task needs no memset in front of its kernel (the outcome lives in the mailbox).
        unsigned long long *w = reinterpret_cast<unsigned long long *>(ctl);
        for (unsigned i = 0; i < kCtlResetBytes / 8; ++i) w[i] = 0;
    }
    __threadfence();

    Mailbox *mb = v->mailbox;
    if (mb) {
        volatile Mailbox *m = mb;
        m->tiles_done = done;
        m->tiles_total = v->total;
        m->status = st;
        m->error = err;
        m->preemptions = preemptions;
        m->start_ns = start_ns;
        m->exit_ns = global_ns();
        __threadfence_system();
        m->seq = launch_no;
        __threadfence_system();
    }
}

} // namespace xpk
