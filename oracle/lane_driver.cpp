// lane_driver — scenario runner over the public C API (XQueue*, XHint*, HwQueue*, HostLane*).
//
// TEST INFRASTRUCTURE.  The file uses nothing but the C entry points, so it is compiled twice:
//   oracle/_ref/lane_driver_ref   against the reference's headers + its compiled host core
//   oracle/lane_driver_new        against this repository's headers + libpreempt.so / libhalhost.so
// and tests compare what the two print for the same scenario.  Each scenario prints one JSON object.
//
//   lane_driver api_contract
//   lane_driver window   <threshold> <batch> <count> <spin_us>
//   lane_driver suspend  <level> <count> <spin_us>
//   lane_driver drop     <level> <count> <spin_us>
//   lane_driver hpf      <level> <lp_count> <lp_us> <hp_count> <hp_us> <hp_gap_us> <threshold> <batch> [LCL|GLB]
//   lane_driver config0  <level> <lp_count> <lp_us> <hp_us> <hp_rate_per_s> <seed (0 = periodic)> <threshold> <batch> <sched:APP|LCL>
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "xsched/types.h"
#include "xsched/xqueue.h"
#include "xsched/hint.h"

extern "C" {
XResult HostLaneQueueCreate(HwQueueHandle *hwq, uint32_t lane_id);
XResult HostLaneCommandCreate(HwCommandHandle *hw_cmd, int64_t spin_us);
XResult HostLaneCommandTimes(HwCommandHandle hw_cmd, int64_t *start_ns, int64_t *finish_ns);
XResult HostLaneCommandLaunchTime(HwCommandHandle hw_cmd, int64_t *launch_ns);
XResult HostLaneCommandRelease(HwCommandHandle hw_cmd);
XResult HostLaneStats(uint32_t lane_id, uint64_t *executed, uint64_t *flushed);
XResult HostLaneSetAffinity(uint32_t lane_id, int cpu);
}

static int64_t NowNs() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
static void SleepUs(int64_t us) { std::this_thread::sleep_for(std::chrono::microseconds(us)); }
static uint32_t LaneId();
static uint64_t Executed() { uint64_t e = 0, f = 0; HostLaneStats(LaneId(), &e, &f); return e; }
static uint64_t Flushed() { uint64_t e = 0, f = 0; HostLaneStats(LaneId(), &e, &f); return f; }
static double Pct(std::vector<double> v, double p) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    size_t i = (size_t)(p * (v.size() - 1) + 0.5);
    return v[std::min(i, v.size() - 1)];
}
#define CHECK(x) do { XResult r_ = (x); if (r_ != kXSchedSuccess) { std::fprintf(stderr, "%s -> %d\n", #x, (int)r_); std::exit(2); } } while (0)

// The lane (= XDevice id) is taken from LANE_ID so that several driver processes can stand for several devices.
static uint32_t LaneId() { const char *v = std::getenv("LANE_ID"); return v ? (uint32_t)std::atoi(v) : 0u; }

static XQueueHandle MakeQueue(int64_t level, int64_t threshold, int64_t batch, HwQueueHandle *hwq_out = nullptr) {
    HwQueueHandle hwq = 0;
    XQueueHandle xq = 0;
    CHECK(HostLaneQueueCreate(&hwq, LaneId()));
    CHECK(XQueueCreate(&xq, hwq, level, kQueueCreateFlagNone));
    if (threshold > 0 || batch > 0) CHECK(XQueueSetLaunchConfig(xq, threshold, batch));
    if (hwq_out) *hwq_out = hwq;
    return xq;
}
static HwCommandHandle SubmitSpin(XQueueHandle xq, int64_t us) {
    HwCommandHandle c = 0;
    CHECK(HostLaneCommandCreate(&c, us));
    CHECK(XQueueSubmit(xq, c));
    return c;
}
static int WaitState(XQueueHandle xq, XQueueState want, int64_t timeout_ms) {
    const int64_t t0 = NowNs();
    while (NowNs() - t0 < timeout_ms * 1000000) {
        XQueueState s = kQueueStateUnknown;
        XQueueQuery(xq, &s);
        if (s == want) return 1;
        SleepUs(200);
    }
    return 0;
}

// ---- error codes and ownership rules of the C API -------------------------------------------------
static int ApiContract() {
    std::printf("{");
    HwQueueHandle hwq = 0;
    XQueueHandle xq = 0, xq2 = 0, got = 0;
    std::printf("\"create_null_out\": %d", (int)XQueueCreate(nullptr, 1, 1, 0));
    CHECK(HostLaneQueueCreate(&hwq, 0));
    std::printf(", \"create_level0\": %d", (int)XQueueCreate(&xq, hwq, 0, 0));
    std::printf(", \"create_level4\": %d", (int)XQueueCreate(&xq, hwq, 4, 0));
    std::printf(", \"create_blocking\": %d", (int)XQueueCreate(&xq, hwq, 1, kQueueCreateFlagBlockingSubmit));
    std::printf(", \"create_unknown_hwq\": %d", (int)XQueueCreate(&xq, 0xdeadbeef, 1, 0));
    std::printf(", \"get_before_create\": %d", (int)XQueueGet(&got, hwq));
    std::printf(", \"create_ok\": %d", (int)XQueueCreate(&xq, hwq, 1, 0));
    std::printf(", \"create_twice\": %d", (int)XQueueCreate(&xq2, hwq, 1, 0));
    std::printf(", \"create_twice_same_handle\": %d", (int)(xq == xq2));
    std::printf(", \"get_ok\": %d", (int)XQueueGet(&got, hwq));
    std::printf(", \"get_same\": %d", (int)(got == xq));
    std::printf(", \"get_null\": %d", (int)XQueueGet(nullptr, hwq));
    std::printf(", \"handle_has_pid\": %d", (int)((xq >> 48) != 0));
    XQueueState st = kQueueStateUnknown;
    std::printf(", \"query_ok\": %d", (int)XQueueQuery(xq, &st));
    std::printf(", \"query_initial_state\": %d", (int)st);
    std::printf(", \"query_null\": %d", (int)XQueueQuery(xq, nullptr));
    std::printf(", \"query_unknown\": %d", (int)XQueueQuery(0x1234, &st));
    std::printf(", \"destroy_hwq_attached\": %d", (int)HwQueueDestroy(hwq));
    std::printf(", \"setlevel_bad\": %d", (int)XQueueSetPreemptLevel(xq, (XPreemptLevel)0));
    std::printf(", \"setlevel_2\": %d", (int)XQueueSetPreemptLevel(xq, kPreemptLevelDeactivate));
    std::printf(", \"setlevel_unknown_xq\": %d", (int)XQueueSetPreemptLevel(0x1234, kPreemptLevelBlock));
    std::printf(", \"setconfig_noop\": %d", (int)XQueueSetLaunchConfig(xq, 0, -1));
    std::printf(", \"setconfig_ok\": %d", (int)XQueueSetLaunchConfig(xq, 4, 2));
    std::printf(", \"setconfig_unknown\": %d", (int)XQueueSetLaunchConfig(0x1234, 4, 2));
    HwCommandHandle c = 0;
    std::printf(", \"cmd_create_null\": %d", (int)HostLaneCommandCreate(nullptr, 10));
    CHECK(HostLaneCommandCreate(&c, 100));
    std::printf(", \"submit_unknown_xq\": %d", (int)XQueueSubmit(0x1234, c));
    std::printf(", \"submit_ok\": %d", (int)XQueueSubmit(xq, c));
    std::printf(", \"submit_consumed\": %d", (int)XQueueSubmit(xq, c));
    std::printf(", \"wait_consumed\": %d", (int)XQueueWait(xq, c));
    std::printf(", \"cmd_destroy_consumed\": %d", (int)HwCommandDestroy(c));
    std::printf(", \"waitall_ok\": %d", (int)XQueueWaitAll(xq));
    std::printf(", \"waitall_unknown\": %d", (int)XQueueWaitAll(0x1234));
    int64_t cnt = -1;
    std::printf(", \"count_ok\": %d", (int)XQueueProfileHwCommandCount(xq, &cnt));
    std::printf(", \"count_value\": %" PRId64, cnt);
    std::printf(", \"count_null\": %d", (int)XQueueProfileHwCommandCount(xq, nullptr));
    std::printf(", \"idle_after_waitall\": %d", WaitState(xq, kQueueStateIdle, 2000));
    std::printf(", \"suspend_ok\": %d", (int)XQueueSuspend(xq, 0));
    std::printf(", \"suspend_again\": %d", (int)XQueueSuspend(xq, 0));
    std::printf(", \"resume_ok\": %d", (int)XQueueResume(xq, 0));
    std::printf(", \"resume_again\": %d", (int)XQueueResume(xq, 0));
    std::printf(", \"suspend_unknown\": %d", (int)XQueueSuspend(0x1234, 0));
    std::printf(", \"hint_prio_ok\": %d", (int)XHintPriority(xq, 3));
    std::printf(", \"hint_prio_unknown\": %d", (int)XHintPriority(0x1234, 3));
    std::printf(", \"hint_lax_unknown\": %d", (int)XHintLaxity(0x1234, 10, 0, 1));
    std::printf(", \"hint_timeslice\": %d", (int)XHintTimeslice(5000));
    std::printf(", \"set_scheduler_bad\": %d", (int)XHintSetScheduler((XSchedulerType)0, kPolicyUnknown));
    std::printf(", \"set_scheduler_lcl_badpolicy\": %d", (int)XHintSetScheduler(kSchedulerLocal, kPolicyUnknown));
    std::printf(", \"set_scheduler_lcl_hpf\": %d", (int)XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    std::printf(", \"set_scheduler_app\": %d", (int)XHintSetScheduler(kSchedulerAppManaged, kPolicyUnknown));
    HwCommandHandle cb = 0;
    static std::atomic<int> cb_runs{0};
    std::printf(", \"cb_create_null\": %d", (int)HwCommandCreateCallback(nullptr, nullptr, nullptr));
    CHECK(HwCommandCreateCallback(&cb, [](HwQueueHandle, void *) -> XResult { cb_runs++; return kXSchedSuccess; }, nullptr));
    std::printf(", \"cb_submit\": %d", (int)XQueueSubmit(xq, cb));
    XQueueWaitAll(xq);
    std::printf(", \"cb_runs\": %d", cb_runs.load());
    CHECK(HwCommandCreateCallback(&cb, [](HwQueueHandle, void *) -> XResult { cb_runs++; return kXSchedSuccess; }, nullptr));
    std::printf(", \"cb_destroy\": %d", (int)HwCommandDestroy(cb));
    std::printf(", \"cb_destroy_again\": %d", (int)HwCommandDestroy(cb));
    std::printf(", \"hwq_sync\": %d", (int)HwQueueSynchronize(hwq));
    std::printf(", \"hwq_sync_unknown\": %d", (int)HwQueueSynchronize(0x77));
    CHECK(HostLaneCommandCreate(&c, 50));
    std::printf(", \"hwq_launch_direct\": %d", (int)HwQueueLaunch(hwq, c));
    std::printf(", \"hwq_launch_consumed\": %d", (int)HwQueueLaunch(hwq, c));
    HwQueueSynchronize(hwq);
    std::printf(", \"destroy_xq\": %d", (int)XQueueDestroy(xq));
    std::printf(", \"destroy_xq_again\": %d", (int)XQueueDestroy(xq));
    std::printf(", \"get_after_destroy\": %d", (int)XQueueGet(&got, hwq));
    std::printf(", \"destroy_hwq\": %d", (int)HwQueueDestroy(hwq));
    std::printf(", \"destroy_hwq_again\": %d", (int)HwQueueDestroy(hwq));
    std::printf("}\n");
    return 0;
}

// ---- the in-flight window ---------------------------------------------------------------------
static int Window(int64_t threshold, int64_t batch, int count, int64_t spin_us) {
    XQueueHandle xq = MakeQueue(1, threshold, batch);
    std::vector<HwCommandHandle> cmds;
    for (int i = 0; i < count; ++i) cmds.push_back(SubmitSpin(xq, spin_us));
    XQueueState st = kQueueStateUnknown;
    XQueueQuery(xq, &st);
    const int ready_after_submit = st == kQueueStateReady;
    CHECK(XQueueWaitAll(xq));
    std::vector<int64_t> launch(count), start(count), finish(count);
    for (int i = 0; i < count; ++i) {
        HostLaneCommandLaunchTime(cmds[i], &launch[i]);
        HostLaneCommandTimes(cmds[i], &start[i], &finish[i]);
    }
    // Commands in flight right after launch i = launched so far minus finished before launch[i].
    int max_inflight = 0, in_order = 1, all_ran = 1;
    for (int i = 0; i < count; ++i) {
        int fin = 0;
        for (int j = 0; j < i; ++j) if (finish[j] != 0 && finish[j] <= launch[i]) ++fin;
        max_inflight = std::max(max_inflight, i + 1 - fin);
        if (i && start[i] < start[i - 1]) in_order = 0;
        if (!finish[i]) all_ran = 0;
    }
    std::printf("{\"threshold\": %" PRId64 ", \"batch\": %" PRId64 ", \"count\": %d, \"ready_after_submit\": %d, "
                "\"max_inflight\": %d, \"window_respected\": %d, \"in_order\": %d, \"all_ran\": %d, \"idle_at_end\": %d}\n",
                threshold, batch, count, ready_after_submit, max_inflight, (int)(max_inflight <= threshold), in_order, all_ran,
                WaitState(xq, kQueueStateIdle, 2000));
    for (auto c : cmds) HostLaneCommandRelease(c);
    XQueueDestroy(xq);
    return 0;
}

// ---- suspend / resume -------------------------------------------------------------------------
static int Suspend(int64_t level, int count, int64_t spin_us) {
    XQueueHandle xq = MakeQueue(level, 8, 4);
    std::vector<HwCommandHandle> cmds;
    for (int i = 0; i < count; ++i) cmds.push_back(SubmitSpin(xq, spin_us));
    SleepUs(3 * spin_us);
    const int64_t t0 = NowNs();
    CHECK(XQueueSuspend(xq, kQueueSuspendFlagSyncHwQueue));
    const double suspend_us = (NowNs() - t0) / 1e3;
    const uint64_t exec_at_suspend = Executed();
    SleepUs(20 * spin_us + 20000);
    const uint64_t exec_later = Executed();
    const uint64_t flushed = Flushed();
    XQueueState st = kQueueStateUnknown;
    XQueueQuery(xq, &st);
    CHECK(XQueueResume(xq, kQueueResumeFlagNone));
    CHECK(XQueueWaitAll(xq));
    const uint64_t exec_end = Executed();
    std::printf("{\"level\": %" PRId64 ", \"count\": %d, \"suspend_us\": %.1f, \"suspend_bound_us\": %.1f, "
                "\"frozen_while_suspended\": %d, \"partial_at_suspend\": %d, \"flushed_any\": %d, \"state_while_suspended\": %d, "
                "\"all_ran_once\": %d}\n",
                level, count, suspend_us, (double)(level >= 2 ? 2 : 9) * spin_us + 1500.0 /* scheduling noise of a shared host */,
                (int)(exec_at_suspend == exec_later), (int)(exec_at_suspend < (uint64_t)count), (int)(flushed > 0), (int)st,
                (int)(exec_end == (uint64_t)count));
    for (auto c : cmds) HostLaneCommandRelease(c);
    XQueueDestroy(xq);
    return 0;
}

static int Drop(int64_t level, int count, int64_t spin_us) {
    XQueueHandle xq = MakeQueue(level, 8, 4);
    std::vector<HwCommandHandle> cmds;
    for (int i = 0; i < count; ++i) cmds.push_back(SubmitSpin(xq, spin_us));
    SleepUs(2 * spin_us);
    CHECK(XQueueSuspend(xq, kQueueSuspendFlagSyncHwQueue));
    CHECK(XQueueResume(xq, kQueueResumeFlagDropCommands));
    const int64_t t0 = NowNs();
    CHECK(XQueueWaitAll(xq));
    const double waitall_us = (NowNs() - t0) / 1e3;
    const uint64_t exec = Executed();
    // the queue works again after a drop
    HwCommandHandle c = SubmitSpin(xq, spin_us);
    CHECK(XQueueWaitAll(xq));
    int64_t s = 0, f = 0;
    HostLaneCommandTimes(c, &s, &f);
    int64_t cnt = 0;
    XQueueProfileHwCommandCount(xq, &cnt);
    // At level 1 commands already handed to the lane still run after the drop; wait for the lane so
    // that the statistics are final.
    SleepUs((level >= 2 ? 2 : 10) * spin_us + 5000);
    std::printf("{\"level\": %" PRId64 ", \"dropped_some\": %d, \"waitall_quick\": %d, \"works_after_drop\": %d, \"submitted_count\": %" PRId64 "}\n",
                level, (int)(exec < (uint64_t)count), (int)(waitall_us < 3.0 * spin_us + 3000), (int)(f != 0), cnt);
    for (auto h : cmds) HostLaneCommandRelease(h);
    HostLaneCommandRelease(c);
    XQueueDestroy(xq);
    return 0;
}

// ---- seeded random walk over the C API ------------------------------------------------------------
// Two XQueues on one lane, a seeded sequence of API calls (submit bursts, wait, suspend/resume with random
// flags, launch-config and level changes, hints, queries, profile counts).  Everything printed is
// independent of timing: the result code of every call, the submitted-command counters, the queue state at
// quiescent points, and at the end whether everything that was not dropped ran exactly once.
static int Fuzz(uint64_t seed, int steps) {
    CHECK(XHintSetScheduler(kSchedulerAppManaged, kPolicyUnknown));
    std::mt19937_64 rng(seed);
    struct Q { XQueueHandle xq; HwQueueHandle hwq; bool suspended = false; int64_t level; int64_t submitted = 0; bool dropped = false; };
    Q q[2];
    for (int i = 0; i < 2; ++i) { q[i].level = 1 + (int64_t)(rng() % 2); q[i].xq = MakeQueue(q[i].level, 4, 2, &q[i].hwq); }
    std::printf("{\"seed\": %" PRIu64 ", \"codes\": [", seed);
    bool first = true;
    auto out = [&](const char *op, int64_t v) { std::printf("%s[\"%s\", %" PRId64 "]", first ? "" : ", ", op, v); first = false; };
    const uint64_t exec0 = Executed();
    int64_t total_submitted = 0;
    for (int s = 0; s < steps; ++s) {
        Q &x = q[rng() % 2];
        switch (rng() % 10) {
        case 0: case 1: case 2: {                                  // a burst of short commands
            const int n = 1 + (int)(rng() % 6);
            for (int i = 0; i < n; ++i) {
                HwCommandHandle c = 0;
                CHECK(HostLaneCommandCreate(&c, 50 + (int64_t)(rng() % 150)));
                HostLaneCommandRelease(c);
                out("submit", (int64_t)XQueueSubmit(x.xq, c));
                ++x.submitted; ++total_submitted;
            }
            break;
        }
        case 3:
            if (!x.suspended) {
                out("wait_all", (int64_t)XQueueWaitAll(x.xq));
                XQueueState st = kQueueStateUnknown;
                out("query", (int64_t)XQueueQuery(x.xq, &st));
                // the worker marks the queue idle a moment after the wait returns: poll, do not sample
                out("idle_after_wait", (int64_t)WaitState(x.xq, kQueueStateIdle, 2000));
            }
            break;
        case 4: {
            const int64_t flags = (rng() % 2) ? kQueueSuspendFlagSyncHwQueue : kQueueSuspendFlagNone;
            out("suspend", (int64_t)XQueueSuspend(x.xq, flags));
            x.suspended = true;
            break;
        }
        case 5: {
            const bool drop = x.suspended && (rng() % 4 == 0);
            out("resume", (int64_t)XQueueResume(x.xq, drop ? kQueueResumeFlagDropCommands : kQueueResumeFlagNone));
            if (drop && x.level >= 2) x.dropped = true;                 // level 1 ignores the drop flag
            x.suspended = false;
            break;
        }
        case 6:
            if (!x.suspended) {
                const int64_t bs = 1 + (int64_t)(rng() % 4), th = bs + (int64_t)(rng() % 6);
                out("config", (int64_t)XQueueSetLaunchConfig(x.xq, th, bs));
            }
            break;
        case 7:
            if (!x.suspended) {
                const int64_t level = 1 + (int64_t)(rng() % 2);
                const XResult r = XQueueSetPreemptLevel(x.xq, (XPreemptLevel)level);
                out("level", (int64_t)r);
                if (r == kXSchedSuccess) x.level = level;
            }
            break;
        case 8: {
            int64_t cnt = -1;
            out("count_rc", (int64_t)XQueueProfileHwCommandCount(x.xq, &cnt));
            out("count", cnt);
            break;
        }
        default:
            out("hint", (int64_t)XHintPriority(x.xq, (Priority)((int)(rng() % 600) - 300)));
            break;
        }
        if (rng() % 3 == 0) SleepUs((int64_t)(rng() % 400));
    }
    bool any_drop = false;
    for (Q &x : q) {
        if (x.suspended) out("final_resume", (int64_t)XQueueResume(x.xq, kQueueResumeFlagNone));
        out("final_wait", (int64_t)XQueueWaitAll(x.xq));
        out("final_idle", (int64_t)WaitState(x.xq, kQueueStateIdle, 2000));
        any_drop = any_drop || x.dropped;
    }
    SleepUs(3000);
    const uint64_t ran = Executed() - exec0;
    std::printf("], \"submitted\": %" PRId64 ", \"all_ran_unless_dropped\": %d, \"none_ran_twice\": %d}\n", total_submitted,
                (int)(any_drop || ran == (uint64_t)total_submitted), (int)(ran <= (uint64_t)total_submitted));
    for (Q &x : q) { XQueueDestroy(x.xq); }
    return 0;
}

// ---- suspend/resume stress: many short rounds; a lost wake-up or a lost command shows as a stuck round ----
static int Stress(int64_t level, int rounds, int64_t spin_us) {
    CHECK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    XQueueHandle xq = MakeQueue(level, 4, 2);
    CHECK(XHintPriority(xq, 3));
    std::atomic<int> round{0};
    std::atomic<bool> done{false};
    std::thread watchdog([&] {
        int last = -1;
        int64_t since = NowNs();
        while (!done.load()) {
            SleepUs(100000);
            const int r = round.load();
            if (r != last) { last = r; since = NowNs(); continue; }
            if (NowNs() - since > 5000000000ll) {
                std::printf("{\"stuck_in_round\": %d, \"executed\": %" PRIu64 ", \"flushed\": %" PRIu64 "}\n", r, Executed(), Flushed());
                std::fflush(stdout);
                std::_Exit(3);
            }
        }
    });
    const uint64_t exec0 = Executed();
    for (int r = 0; r < rounds; ++r) {
        round.store(r);
        for (int i = 0; i < 6; ++i) { HwCommandHandle c = 0; CHECK(HostLaneCommandCreate(&c, spin_us)); HostLaneCommandRelease(c); CHECK(XQueueSubmit(xq, c)); }
        CHECK(XQueueSuspend(xq, kQueueSuspendFlagSyncHwQueue));
        CHECK(XQueueResume(xq, kQueueResumeFlagNone));
        CHECK(XQueueWaitAll(xq));
    }
    done.store(true);
    watchdog.join();
    std::printf("{\"rounds\": %d, \"executed\": %" PRIu64 ", \"expected\": %d}\n", rounds, Executed() - exec0, rounds * 6);
    XQueueDestroy(xq);
    return 0;
}

// ---- concurrent callers: one thread submits and waits, one suspends and resumes, one queries and hints ----
// Nothing is dropped, so every command must run exactly once and the submitter's waits must all return.
static int MtFuzz(uint64_t seed, int64_t level, int bursts) {
    CHECK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    XQueueHandle xq = MakeQueue(level, 4, 2);
    std::atomic<bool> done{false};
    std::atomic<int> progress{0};
    const uint64_t exec0 = Executed();
    int64_t submitted = 0;
    std::thread submitter([&] {
        std::mt19937_64 rng(seed);
        for (int b = 0; b < bursts; ++b) {
            const int n = 1 + (int)(rng() % 8);
            for (int i = 0; i < n; ++i) { HwCommandHandle c = 0; CHECK(HostLaneCommandCreate(&c, 20 + (int64_t)(rng() % 120))); HostLaneCommandRelease(c); CHECK(XQueueSubmit(xq, c)); ++submitted; }
            if (rng() % 2) CHECK(XQueueWaitAll(xq));
            progress.fetch_add(1);
        }
        CHECK(XQueueWaitAll(xq));
        done.store(true);
    });
    std::thread suspender([&] {
        std::mt19937_64 rng(seed * 31 + 7);
        while (!done.load()) {
            SleepUs((int64_t)(rng() % 600));
            CHECK(XQueueSuspend(xq, (rng() % 2) ? kQueueSuspendFlagSyncHwQueue : kQueueSuspendFlagNone));
            SleepUs((int64_t)(rng() % 300));
            CHECK(XQueueResume(xq, kQueueResumeFlagNone));
        }
    });
    std::thread prober([&] {
        std::mt19937_64 rng(seed * 131 + 3);
        while (!done.load()) {
            XQueueState st; int64_t cnt;
            CHECK(XQueueQuery(xq, &st));
            CHECK(XQueueProfileHwCommandCount(xq, &cnt));
            CHECK(XHintPriority(xq, (Priority)(rng() % 5)));
            SleepUs((int64_t)(rng() % 200));
        }
    });
    std::thread watchdog([&] {
        int last = -1;
        int64_t since = NowNs();
        while (!done.load()) {
            SleepUs(100000);
            const int p = progress.load();
            if (p != last) { last = p; since = NowNs(); continue; }
            if (NowNs() - since > 8000000000ll) { std::printf("{\"stuck_at_burst\": %d}\n", p); std::fflush(stdout); std::_Exit(3); }
        }
    });
    submitter.join(); suspender.join(); prober.join(); watchdog.join();
    SleepUs(2000);
    std::printf("{\"submitted\": %" PRId64 ", \"executed\": %" PRIu64 "}\n", submitted, Executed() - exec0);
    XQueueDestroy(xq);
    return 0;
}

// ---- host-path cost: zero-length commands through one XQueue --------------------------------------
// Submit rate of the application thread and end-to-end rate (submit .. last command retired) with the
// window doing its work (every batch-th command is waited for).  Round trips: submit -> WaitAll of a
// single zero-length command, the shortest path a synchronous caller sees.
static int Tput(int64_t level, int count, int64_t th, int64_t bs) {
    XQueueHandle xq = MakeQueue(level, th, bs);
    for (int i = 0; i < 2000; ++i) { HwCommandHandle c = 0; CHECK(HostLaneCommandCreate(&c, 0)); HostLaneCommandRelease(c); CHECK(XQueueSubmit(xq, c)); }
    CHECK(XQueueWaitAll(xq));
    const int64_t t0 = NowNs();
    for (int i = 0; i < count; ++i) {
        HwCommandHandle c = 0;
        CHECK(HostLaneCommandCreate(&c, 0));
        HostLaneCommandRelease(c);
        CHECK(XQueueSubmit(xq, c));
    }
    const int64_t t1 = NowNs();
    CHECK(XQueueWaitAll(xq));
    const int64_t t2 = NowNs();
    std::vector<double> rt;
    for (int i = 0; i < 2000; ++i) {
        const int64_t a = NowNs();
        HwCommandHandle c = 0;
        CHECK(HostLaneCommandCreate(&c, 0));
        HostLaneCommandRelease(c);
        CHECK(XQueueSubmit(xq, c));
        CHECK(XQueueWaitAll(xq));
        rt.push_back((NowNs() - a) / 1e3);
    }
    std::printf("{\"level\": %" PRId64 ", \"count\": %d, \"submit_ns_per_cmd\": %.1f, \"end_to_end_ns_per_cmd\": %.1f, "
                "\"round_trip_p50_us\": %.2f, \"round_trip_p99_us\": %.2f}\n",
                level, count, (double)(t1 - t0) / count, (double)(t2 - t0) / count, Pct(rt, 0.5), Pct(rt, 0.99));
    XQueueDestroy(xq);
    return 0;
}

// ---- two queues under highest-priority-first ------------------------------------------------------
struct HpResult { std::vector<double> lat_us; double lp_total_ms = 0; };

static HpResult RunTwoQueues(int64_t level, int lp_count, int64_t lp_us, const std::vector<int64_t> &hp_arrivals_us, int64_t hp_us,
                             int64_t threshold, int64_t batch, bool with_lp, int64_t lax_us = -1) {
    XQueueHandle lp = MakeQueue(level, threshold, batch);
    XQueueHandle hp = MakeQueue(level, threshold, batch);
    if (lax_us < 0) {
        CHECK(XHintPriority(lp, 0));
        CHECK(XHintPriority(hp, 1));
    } else {
        // laxity policy: the low-priority queue stays un-hinted (priority 0); the other one is relaxed
        // (priority 0) for lax_us after it becomes ready and critical (priority 1) from then on
        CHECK(XHintLaxity(hp, lax_us, 0, 1));
    }
    HpResult res;
    std::atomic<bool> lp_done{false};
    const int64_t t_begin = NowNs();
    std::thread lp_thread([&] {
        if (with_lp) {
            for (int i = 0; i < lp_count; ++i) {
                HwCommandHandle c = 0;
                CHECK(HostLaneCommandCreate(&c, lp_us));
                HostLaneCommandRelease(c);                 // timing of LP commands is not needed
                CHECK(XQueueSubmit(lp, c));
            }
            CHECK(XQueueWaitAll(lp));
        }
        res.lp_total_ms = (NowNs() - t_begin) / 1e6;
        lp_done.store(true);
    });
    for (int64_t at : hp_arrivals_us) {
        if (with_lp && lp_done.load()) break;
        const int64_t target = t_begin + at * 1000;
        while (NowNs() < target) SleepUs(std::min<int64_t>(200, std::max<int64_t>(1, (target - NowNs()) / 2000)));
        const int64_t t0 = NowNs();
        HwCommandHandle c = 0;
        CHECK(HostLaneCommandCreate(&c, hp_us));
        HostLaneCommandRelease(c);
        CHECK(XQueueSubmit(hp, c));
        CHECK(XQueueWaitAll(hp));
        res.lat_us.push_back((NowNs() - t0) / 1e3);
    }
    lp_thread.join();
    XQueueDestroy(hp);
    XQueueDestroy(lp);
    return res;
}

static void PrintHp(const char *name, const HpResult &r) {
    std::printf("\"%s\": {\"n\": %zu, \"p50_us\": %.1f, \"p99_us\": %.1f, \"max_us\": %.1f, \"lp_total_ms\": %.2f}", name,
                r.lat_us.size(), Pct(r.lat_us, 0.50), Pct(r.lat_us, 0.99), Pct(r.lat_us, 1.0), r.lp_total_ms);
}

static int Hpf(int64_t level, int lp_count, int64_t lp_us, int hp_count, int64_t hp_us, int64_t hp_gap_us, int64_t th, int64_t bs,
               const std::string &sched, int64_t lax_us = -1) {
    if (sched == "GLB") CHECK(XHintSetScheduler(kSchedulerGlobal, kPolicyUnknown));      // needs a running xserver
    else CHECK(XHintSetScheduler(kSchedulerLocal, lax_us < 0 ? kPolicyHighestPriorityFirst : kPolicyLaxity));
    std::vector<int64_t> arrivals;
    for (int i = 0; i < hp_count; ++i) arrivals.push_back((i + 1) * hp_gap_us);
    HpResult r = RunTwoQueues(level, lp_count, lp_us, arrivals, hp_us, th, bs, true, lax_us);
    std::printf("{\"level\": %" PRId64 ", ", level);
    PrintHp("hp", r);
    std::printf(", \"flushed\": %" PRIu64 "}\n", Flushed());
    return 0;
}

static int Config0(int64_t level, int lp_count, int64_t lp_us, int64_t hp_us, double hp_rate, uint64_t seed, int64_t th, int64_t bs,
                   const std::string &sched) {
    if (sched == "LCL") CHECK(XHintSetScheduler(kSchedulerLocal, kPolicyHighestPriorityFirst));
    else CHECK(XHintSetScheduler(kSchedulerAppManaged, kPolicyUnknown));
    // Poisson arrivals: exponential gaps with mean 1/rate, seeded.
    std::mt19937_64 rng(seed);
    std::exponential_distribution<double> gap(hp_rate);
    std::vector<int64_t> arrivals;
    double t = 0;
    const double horizon_us = (double)lp_count * lp_us * 1.5 + 1e6;
    // seed 0 selects a fixed period of 1/rate instead of Poisson arrivals
    while (t < horizon_us) { t += (seed == 0 ? 1.0 / hp_rate : gap(rng)) * 1e6; arrivals.push_back((int64_t)t); }
    // standalone: the same arrivals (first 200 at most) with no low-priority work
    std::vector<int64_t> solo(arrivals.begin(), arrivals.begin() + std::min<size_t>(arrivals.size(), 50));
    for (size_t i = 0; i < solo.size(); ++i) solo[i] = (int64_t)(i + 1) * (hp_us + 3000);
    HpResult alone = RunTwoQueues(level, 0, lp_us, solo, hp_us, th, bs, false);
    HpResult both = RunTwoQueues(level, lp_count, lp_us, arrivals, hp_us, th, bs, true);
    const double ideal_ms = ((double)lp_count * lp_us + (double)both.lat_us.size() * hp_us) / 1e3;
    std::printf("{\"level\": %" PRId64 ", \"sched\": \"%s\", \"threshold\": %" PRId64 ", \"batch\": %" PRId64 ", \"lp_count\": %d, ",
                level, sched.c_str(), th, bs, lp_count);
    PrintHp("standalone", alone);
    std::printf(", ");
    PrintHp("corun", both);
    std::printf(", \"p99_ratio\": %.3f, \"lp_ideal_ms\": %.2f, \"lp_kept_pct\": %.2f, \"cores\": %u}\n",
                Pct(both.lat_us, 0.99) / std::max(1.0, Pct(alone.lat_us, 0.99)), ideal_ms, 100.0 * ideal_ms / std::max(1e-9, both.lp_total_ms),
                std::thread::hardware_concurrency());
    return 0;
}

int main(int argc, char **argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: lane_driver <scenario> ...\n"); return 1; }
    const std::string s = argv[1];
    auto I = [&](int i, int64_t d) -> int64_t { return argc > i ? std::atoll(argv[i]) : d; };
    if (s == "api_contract") return ApiContract();
    if (s == "window") return Window(I(2, 4), I(3, 2), (int)I(4, 40), I(5, 300));
    if (s == "suspend") return Suspend(I(2, 1), (int)I(3, 40), I(4, 500));
    if (s == "drop") return Drop(I(2, 1), (int)I(3, 40), I(4, 500));
    if (s == "hpf") return Hpf(I(2, 1), (int)I(3, 400), I(4, 1000), (int)I(5, 10), I(6, 2000), I(7, 30000), I(8, 16), I(9, 8), argc > 10 ? argv[10] : "LCL");
    if (s == "mtfuzz") return MtFuzz((uint64_t)I(2, 1), I(3, 2), (int)I(4, 300));
    if (s == "stress") return Stress(I(2, 2), (int)I(3, 2000), I(4, 100));
    if (s == "fuzz") return Fuzz((uint64_t)I(2, 1), (int)I(3, 200));
    if (s == "tput") return Tput(I(2, 1), (int)I(3, 200000), I(4, 16), I(5, 8));
    if (s == "lax") return Hpf(I(2, 2), (int)I(3, 400), I(4, 1000), (int)I(5, 10), I(6, 2000), I(7, 30000), I(8, 16), I(9, 8), argc > 10 ? argv[10] : "LCL", I(11, 5000));
    if (s == "config0") return Config0(I(2, 1), (int)I(3, 3000), I(4, 1000), I(5, 2000), (double)I(6, 20), (uint64_t)I(7, 42), I(8, 16), I(9, 8),
                                       argc > 10 ? argv[10] : "LCL");
    std::fprintf(stderr, "unknown scenario %s\n", s.c_str());
    return 1;
}
