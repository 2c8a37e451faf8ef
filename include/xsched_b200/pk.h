/*
 * pk.h — C ABI of the preemptible persistent-kernel library (libxpk.so) for sm_100a.
 *
 * This is the device-side half of XSched's Level-2 ("deactivate") preemption on B200.
 * The reference obtains Level-2 by patching a guardian prologue into every application
 * kernel (platforms/cuda/hal/src/level2/instrument.cpp:15-231,
 * platforms/cuda/hal/inject/inject.cu:43-140): each thread block checks a global exit
 * flag, records exit/restore flags per block, and the host relaunches from `preempt_idx`
 * (platforms/cuda/hal/src/level2/cuda_queue.cpp:29-41).  That guardian exists only as
 * sm35/sm70/sm86 machine code (platforms/cuda/hal/src/arch/arch.cpp:26-39), so on B200 the
 * reference has no Level-2 at all.  Here the same contract is provided cooperatively:
 * every kernel below is persistent, claims its work tile by tile, polls a device-visible
 * preempt flag at each tile boundary, and on preemption leaves a resumable cursor in a
 * control block.  Relaunching the same task continues from the cursor; the output of a
 * task preempted and resumed any number of times is bit-identical to an unpreempted run.
 *
 * All entry points take plain pointers and sizes.  Device pointers are raw CUDA device
 * addresses; streams are CUstream/cudaStream_t passed as void*.  Every function returns
 * an xpkResult; nothing here allocates behind the caller's back except xpkTaskCreate*
 * (one device control block of about 16.6 KB — claim state plus two lists of handed-back
 * tiles — and one 64-byte mapped host mailbox per task).
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    XPK_SUCCESS            = 0,
    XPK_ERR_INVALID_VALUE  = 1,  /* null pointer, zero size, bad shape            */
    XPK_ERR_ALIGNMENT      = 2,  /* a device pointer is not 16-byte aligned       */
    XPK_ERR_CUDA           = 3,  /* a CUDA runtime/driver call failed             */
    XPK_ERR_NOT_SUPPORTED  = 4,  /* shape outside what the kernel was built for   */
    XPK_ERR_BUSY           = 5,  /* task still in flight                          */
    XPK_ERR_DEVICE_TIMEOUT = 6,  /* a bounded device-side wait gave up            */
    XPK_ERR_TOO_LARGE      = 7,  /* exceeds a static capacity                     */
} xpkResult;

/* Task status as published by the kernel in the mailbox. */
typedef enum {
    XPK_STATUS_IDLE      = 0,  /* created or reset, never launched                 */
    XPK_STATUS_RUNNING   = 1,  /* launched, final CTA has not yet published        */
    XPK_STATUS_COMPLETED = 2,  /* every tile done                                   */
    XPK_STATUS_PREEMPTED = 3,  /* stopped on the preempt flag; cursor is resumable */
    XPK_STATUS_ERROR     = 4,  /* a bounded wait expired; output undefined         */
} xpkStatus;

typedef enum {
    XPK_KIND_TRIAD  = 1,  /* a[i] = fmaf(s, c[i], b[i]), fp32, 128-bit accesses   */
    XPK_KIND_VECADD = 2,  /* c[i] = a[i] + b[i], fp32                              */
    XPK_KIND_SORT   = 3,  /* int32 ascending LSD radix sort, 8-bit digits          */
    XPK_KIND_GEMM   = 4,  /* bf16 C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulate      */
} xpkKind;

/* Launch-time flags for xpkTaskCreate*. */
enum {
    XPK_FLAG_NONE           = 0,
    XPK_FLAG_NON_PREEMPTIBLE = 1, /* the twin: same tile loop and the same ticket claim, the
                                     preempt flag never read.  For kernels nothing needs to
                                     stop, and to measure what the check costs.            */
    XPK_FLAG_ABORT_INFLIGHT = 2, /* GEMM only: on preemption abandon tiles whose main
                                     loop is still running and recompute them on resume
                                     (keeps the preemption latency below one tile).     */
    XPK_FLAG_GEMM_ONE_CTA   = 4, /* GEMM only: run the form in which one CTA owns a 256x256
                                     tile (tcgen05 .cta_group::1).                         */
    XPK_FLAG_GEMM_CTA_PAIR  = 8, /* GEMM only: run the form in which the two SMs of a TPC
                                     share a 256x256 tile (tcgen05 .cta_group::2).  With
                                     neither flag the library chooses (XPK_GEMM_FORM=one|pair
                                     in the environment overrides its choice).  Both forms
                                     write the same bytes.                                 */
};

typedef struct xpkTask_st *xpkTask_t;

/* Snapshot returned by xpkTaskQuery; mirrors the mailbox the final CTA writes. */
typedef struct {
    uint32_t status;       /* xpkStatus                                             */
    uint32_t error;        /* 0, or a kernel-specific code naming the wait that expired */
    uint64_t tiles_done;   /* tiles completed over the task's life (the cursor)     */
    uint64_t tiles_total;  /* tiles in the task                                     */
    uint64_t launches;     /* kernel launches issued for this task since reset      */
    uint64_t preemptions;  /* launches that ended PREEMPTED                         */
} xpkTaskInfo;

/* ---- library / device --------------------------------------------------------------- */

/* Number of SMs of the current device (the persistent grids are sized from it). */
xpkResult xpkDeviceSmCount(int *sm_count);
const char *xpkResultString(xpkResult r);

/* ---- preempt flag -------------------------------------------------------------------
 * A flag is one 32-bit word in device memory.  One flag is normally shared by all tasks
 * of one hardware queue (that is what HwQueue::Deactivate raises — reference contract
 * preempt/include/xsched/preempt/hal/hw_queue.h:36-44).  Raise/clear are enqueued as a
 * 32-bit stream memory write on `ctrl_stream`, which should not be the stream the
 * persistent kernel occupies.                                                          */
xpkResult xpkFlagCreate(uint32_t **flag_dev);
xpkResult xpkFlagDestroy(uint32_t *flag_dev);
xpkResult xpkFlagSet(uint32_t *flag_dev, uint32_t value, void *ctrl_stream);
/* A stream write needs 6-14 us to reach device memory.  A flag (256 bytes from xpkFlagCreate, or any zeroed
 * 16-byte-aligned block whose first word is the flag) can be given an early-warning word in mapped host memory:
 * the caller stores a non-zero value there (a plain host store, on the GPU within about 2 us) immediately before
 * xpkFlagSet(flag, 1, ..), and zero before lowering the flag.  Kernels that run a relay (the GEMM, the triad and the vector add) copy the raised
 * word into the flag; every kernel still honours the flag itself.  The word is freed with the flag's owner
 * calling xpkFlagDetachRelay.                                                                          */
xpkResult xpkFlagAttachRelay(uint32_t *flag_dev, volatile uint32_t **relay_host);
xpkResult xpkFlagDetachRelay(uint32_t *flag_dev, volatile uint32_t *relay_host);

/* ---- task creation ------------------------------------------------------------------
 * `flag_dev` may be NULL: the task then owns a private flag (see xpkTaskFlag).
 * `tile_elems`/tile shape 0 selects the default.                                        */

/* a = b + s*c computed as one fused multiply-add per element.  n in elements. */
xpkResult xpkTaskCreateTriad(xpkTask_t *task, float *a, const float *b, const float *c,
                             float s, uint64_t n, uint32_t tile_elems, uint32_t flags,
                             uint32_t *flag_dev);

/* c = a + b. */
xpkResult xpkTaskCreateVecAdd(xpkTask_t *task, float *c, const float *a, const float *b,
                              uint64_t n, uint32_t tile_elems, uint32_t flags,
                              uint32_t *flag_dev);

/* Ascending sort of n int32 keys.  `keys` holds the input and, after completion, the
 * sorted output (4 passes: the data ends in the buffer it started in).  `tmp` is a
 * caller-provided buffer of n keys.  `scratch` is caller-provided device memory of at
 * least xpkSortScratchBytes(n) bytes, 256-byte aligned; the library clears what it needs. */
size_t    xpkSortScratchBytes(uint64_t n);
xpkResult xpkTaskCreateSort(xpkTask_t *task, int32_t *keys, int32_t *tmp, void *scratch,
                            uint64_t n, uint32_t flags, uint32_t *flag_dev);

/* bf16 GEMM, C[M,N] (row-major, bf16) = A[M,K] (row-major) * B[N,K]^T (row-major, i.e.
 * both operands K-major), fp32 accumulation in tensor memory.  M % 128 == 0,
 * N % 256 == 0, K % 64 == 0.  A tile (the unit of xpkTaskInfo.tiles_*) is 512x256 in the
 * pair form and 256x256 in the one-CTA form (XPK_FLAG_GEMM_*); the pair form launches whole
 * pairs of CTAs (an `sm_limit` is rounded down to an even number, at least 2).           */
xpkResult xpkTaskCreateGemm(xpkTask_t *task, void *C, const void *A, const void *B,
                            uint32_t M, uint32_t N, uint32_t K, uint32_t flags,
                            uint32_t *flag_dev);

/* ---- task control ------------------------------------------------------------------- *
 * A task belongs to the device that was current when it was created.  xpkTaskLaunch,
 * xpkTaskReset and xpkTaskDestroy (and xpkFlagSet, for the flag's device) make that device
 * current for the duration of the call and restore the caller's, so they may be called
 * from any thread; `stream` must be a stream of the task's device.                       */

/* Enqueue the task's kernel on `stream`.  A fresh or reset task starts at tile 0; a
 * PREEMPTED task continues from its cursor; a COMPLETED task has re-armed itself and runs
 * again from tile 0 (callers whose inputs changed in place, like the sort's keys, restore them
 * first).  Never blocks.  `sm_limit` > 0 caps the persistent grid to that many SMs (0 = all).          */
xpkResult xpkTaskLaunch(xpkTask_t task, void *stream, int sm_limit);

/* Read the mailbox (mapped host memory; no CUDA call, no synchronisation). */
xpkResult xpkTaskQuery(xpkTask_t task, xpkTaskInfo *info);

/* Spin (with back-off) on the mailbox until the launch issued most recently has
 * published COMPLETED, PREEMPTED or ERROR, or `timeout_us` elapses (XPK_ERR_BUSY).      */
xpkResult xpkTaskWait(xpkTask_t task, uint64_t timeout_us, xpkTaskInfo *info);

/* Device-clock stamps (%globaltimer, nanoseconds) of the launch whose result the mailbox holds: when its
 * first CTA started and when its last CTA left.  For latency break-downs; XPK_ERR_BUSY before any launch
 * has published.  The GPU clock is not the host's: callers calibrate an offset themselves.            */
xpkResult xpkTaskTimes(xpkTask_t task, uint64_t *start_ns, uint64_t *exit_ns);

/* Rewind the cursor to tile 0 (enqueued on `stream`, ordered after prior work on it).  Costs nothing on the
 * device for a task that was never launched or has completed; the sort's scratch is cleared in any case. */
xpkResult xpkTaskReset(xpkTask_t task, void *stream);

/* The flag this task polls (its own, or the shared one given at creation). */
xpkResult xpkTaskFlag(xpkTask_t task, uint32_t **flag_dev);
xpkResult xpkTaskKind(xpkTask_t task, uint32_t *kind);
xpkResult xpkTaskDestroy(xpkTask_t task);

/* ---- sorting without any allocation ---------------------------------------------------
 * (No counterpart in the reference, which has no sort kernel and no allocation-free entry points.)
 *
 * For callers that cannot allocate device or pinned memory at the point where they need a sort —
 * code running while a memory pool is frozen, a plugin that was handed two buffers and a stream and
 * nothing else, a latency-critical section where cudaMalloc's implicit device synchronisation is not
 * acceptable.  xpkTaskCreateSort needs a control block, a mailbox and caller-provided scratch; this
 * entry point needs none of them: its control block, digit histograms and look-back words live in a
 * fixed array inside the library's device image (about 4.2 MB, held by every GPU that loads the
 * library until the process exits).
 *
 * Sorts `n` int32 keys ascending, in place in `keys`, using `tmp` (n keys) as the second buffer, on
 * `stream`; asynchronous, the result is ready when the stream reaches this point.  Not preemptible.
 *   - n > XPK_SORT_NOALLOC_MAX_KEYS  -> XPK_ERR_TOO_LARGE; keys/tmp must be 16-byte aligned.
 *   - Calls no cudaMalloc/cudaFree/cudaHostAlloc and no library routine that allocates.
 *   - The first call on each device resolves the array's address (cudaGetSymbolAddress) and sets a
 *     kernel attribute; make that first call outside any stream capture.
 *   - `stream` must be a stream of the device that is current in the calling thread: the array
 *     that is used is the current device's copy.
 *   - There is no status channel: a bounded wait inside the kernel that gives up (none has been
 *     seen to) leaves the keys unsorted and is not reported; callers that need a status use the
 *     task form (xpkTaskCreateSort / xpkTaskWait).
 *   - All calls on one device share the one array.  It keeps the previous call's contents (the entry
 *     point clears what it needs), and two calls whose kernels overlap on the GPU — different
 *     streams, or different host threads without ordering between their streams — race on it:
 *     serialise them.                                                                      */
#define XPK_SORT_NOALLOC_MAX_KEYS (4ull << 20)
xpkResult xpkSortNoAlloc(int32_t *keys, int32_t *tmp, uint64_t n, void *stream);

/* Kernels launched by this library in this process since load (all tasks, and the sort kernels
 * of xpkSortNoAlloc). */
uint64_t xpkLaunchCount(void);

#ifdef __cplusplus
}
#endif
