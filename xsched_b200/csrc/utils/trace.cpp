#include "xsched/utils/trace.h"

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>
#include <unistd.h>

namespace xsched::utils {
namespace {

struct Record { int64_t ns; uint32_t stage; uint64_t a, b; };
constexpr uint64_t kRing = 1u << 18;          // 8 MB when tracing is on; nothing is allocated otherwise

struct State {
    bool on = false;
    std::string path;
    Record *ring = nullptr;
    std::atomic<uint64_t> next{0};
    std::mutex flush_mu;
    uint64_t flushed = 0;
    State() {
        const char *p = std::getenv("XSCHED_TRACE_FILE");
        if (p == nullptr || *p == '\0') return;
        path = std::string(p) + "." + std::to_string((long)getpid());
        ring = new Record[kRing];
        on = true;
        std::atexit([] { TraceFlush(); });
    }
};
// Never destroyed: the flush registered with atexit runs after function-local statics would have gone.
State &S() { static State *s = new State; return *s; }

const char *const kNames[] = {"none", "ready_sent", "idle_sent", "event_recv", "decision", "op_sent", "op_recv", "suspend_begin", "suspend_end",
                              "resume_begin", "resume_end", "deactivate_issued", "hwq_synced", "task_gpu_times", "gpu_clock_offset", "app_submit",
                              "app_done", "app_gpu_times"};
static_assert(sizeof(kNames) / sizeof(kNames[0]) == kTraceStageMax, "one name per stage");

} // namespace

const char *TraceStageName(uint32_t stage) { return stage < kTraceStageMax ? kNames[stage] : "?"; }

bool TraceEnabled() { return S().on; }

void TraceStamp(uint32_t stage, uint64_t a, uint64_t b) {
    State &s = S();
    if (!s.on) return;
    const int64_t ns = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
    const uint64_t i = s.next.fetch_add(1, std::memory_order_relaxed);
    s.ring[i % kRing] = Record{ns, stage, a, b};
}

void TraceFlush() {
    State &s = S();
    if (!s.on) return;
    std::lock_guard<std::mutex> lk(s.flush_mu);
    const uint64_t end = s.next.load();
    uint64_t begin = s.flushed;
    if (end - begin > kRing) begin = end - kRing;       // the ring wrapped: the oldest records are gone
    if (begin == end) return;
    FILE *f = std::fopen(s.path.c_str(), "a");
    if (!f) return;
    for (uint64_t i = begin; i < end; ++i) {
        const Record &r = s.ring[i % kRing];
        std::fprintf(f, "%lld %s %llu %llu\n", (long long)r.ns, TraceStageName(r.stage), (unsigned long long)r.a, (unsigned long long)r.b);
    }
    std::fclose(f);
    s.flushed = end;
}

} // namespace xsched::utils

extern "C" {
__attribute__((visibility("default"))) int XTraceEnabled(void) { return xsched::utils::TraceEnabled() ? 1 : 0; }
__attribute__((visibility("default"))) void XTraceStamp(uint32_t stage, uint64_t a, uint64_t b) { xsched::utils::TraceStamp(stage, a, b); }
__attribute__((visibility("default"))) void XTraceFlush(void) { xsched::utils::TraceFlush(); }
}
