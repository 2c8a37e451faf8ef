// fake_xpk — TEST INFRASTRUCTURE: the three libxpk entry points the CUDA HAL calls (xpkTaskReset, xpkTaskLaunch,
// xpkTaskQuery) over the fake driver, so that the level-2 path of the HAL — raise the flag, kernels stop at a
// tile boundary and leave a cursor, Reactivate relaunches from the first unfinished task — can be run and raced
// on a machine without a GPU.  A task is `tiles` tiles of `tile_us` microseconds; a launch is a host function on
// the stream that works through the tiles from the cursor on, looks at the preempt flag before every tile, and
// publishes COMPLETED or PREEMPTED like the real kernels' last CTA does.  Every tile counts how often it ran.
#include <cuda.h>

#include <atomic>
#include <chrono>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>
#include "xsched_b200/pk.h"

struct xpkTask_st {
    uint64_t tiles = 0;
    int tile_us = 0;
    volatile uint32_t *flag = nullptr;
    std::mutex mu;                         // the published state, as the mailbox holds it
    uint64_t cursor = 0;                   // next tile to run
    uint64_t launches = 0, reset_at = 0, published_for = 0, preemptions = 0;
    uint32_t status = XPK_STATUS_IDLE;
    std::vector<std::atomic<uint32_t>> runs;          // per tile, since the last reset
    explicit xpkTask_st(uint64_t n) : runs(n) {}
};

namespace {
struct LaunchArg { xpkTask_st *t; uint64_t launch_no; };
void RunTask(void *p) {
    std::unique_ptr<LaunchArg> a((LaunchArg *)p);
    xpkTask_st *t = a->t;
    uint64_t tile;
    { std::lock_guard<std::mutex> lk(t->mu); tile = t->cursor; }
    uint32_t st = XPK_STATUS_COMPLETED;
    for (; tile < t->tiles; ++tile) {
        if (__atomic_load_n(t->flag, __ATOMIC_ACQUIRE) != 0) { st = XPK_STATUS_PREEMPTED; break; }
        std::this_thread::sleep_for(std::chrono::microseconds(t->tile_us));
        t->runs[tile].fetch_add(1);
    }
    std::lock_guard<std::mutex> lk(t->mu);
    t->cursor = tile;
    t->status = st;
    if (st == XPK_STATUS_PREEMPTED) ++t->preemptions;
    t->published_for = a->launch_no;
}
} // namespace

extern "C" {

__attribute__((visibility("default"))) xpkTask_t fakeXpkTaskCreate(uint64_t tiles, int tile_us, uint32_t *flag) {
    auto *t = new xpkTask_st(tiles);
    t->tiles = tiles; t->tile_us = tile_us; t->flag = flag;
    return t;
}
__attribute__((visibility("default"))) uint32_t fakeXpkTileRuns(xpkTask_t t, uint64_t tile) { return t->runs[tile].load(); }

__attribute__((visibility("default"))) xpkResult xpkTaskReset(xpkTask_t t, void *) {
    std::lock_guard<std::mutex> lk(t->mu);
    t->cursor = 0;
    t->reset_at = t->launches;
    t->status = XPK_STATUS_IDLE;
    for (auto &r : t->runs) r.store(0);
    return XPK_SUCCESS;
}
__attribute__((visibility("default"))) xpkResult xpkTaskLaunch(xpkTask_t t, void *stream, int) {
    uint64_t no;
    { std::lock_guard<std::mutex> lk(t->mu); no = ++t->launches; }
    return cuLaunchHostFunc((CUstream)stream, RunTask, new LaunchArg{t, no}) == CUDA_SUCCESS ? XPK_SUCCESS : XPK_ERR_CUDA;
}
__attribute__((visibility("default"))) xpkResult xpkTaskTimes(xpkTask_t, uint64_t *, uint64_t *) { return XPK_ERR_BUSY; }
__attribute__((visibility("default"))) xpkResult xpkTaskQuery(xpkTask_t t, xpkTaskInfo *info) {
    std::lock_guard<std::mutex> lk(t->mu);
    info->tiles_total = t->tiles;
    info->launches = t->launches;
    info->error = 0;
    info->tiles_done = t->cursor;
    info->preemptions = t->preemptions;
    if (t->launches == t->reset_at) info->status = XPK_STATUS_IDLE;
    else if (t->published_for < t->launches) info->status = XPK_STATUS_RUNNING;
    else info->status = t->status;
    return XPK_SUCCESS;
}

} // extern "C"
