// sched_probe (this repository's build) — TEST INFRASTRUCTURE.  Same script and output format as
// sched_probe_ref.cpp, driving this repository's LocalScheduler (csrc/sched/local_scheduler.cpp).
//   usage: sched_probe_new <policy> [--virtual <t0_us>] < script
// With --virtual the scheduler runs on the calling thread against a virtual clock that starts at t0_us:
// a round after every event, `sleep_ms` / `sleep_us` serve the policy's timers at their exact times, `flush` lets
// 30 ms pass first (as the real-time mode does), `peek` reports without letting time pass.  Outcomes are then
// exactly reproducible.
#include <chrono>
#include <cstdio>
#include <iostream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "xsched/protocol/names.h"
#include "xsched/sched/scheduler.h"

using namespace xsched::sched;

static std::vector<unsigned char> Unhex(const std::string &s) {
    std::vector<unsigned char> out;
    for (size_t i = 0; i + 1 < s.size(); i += 2) out.push_back((unsigned char)std::stoi(s.substr(i, 2), nullptr, 16));
    return out;
}

int main(int argc, char **argv) {
    const XPolicyType policy = xsched::protocol::GetPolicyType(argc > 1 ? argv[1] : "HPF");
    LocalScheduler sched(policy);
    const bool virt = argc > 3 && std::string(argv[2]) == "--virtual";
    int64_t vnow = virt ? std::atoll(argv[3]) : 0;
    if (virt) sched.SetClock([&vnow] { return vnow; });
    auto advance = [&](int64_t until) {
        while (sched.NextTimerUs() <= until) {
            vnow = std::max(vnow, sched.NextTimerUs());
            sched.StepInline(nullptr, 0);
        }
        vnow = until;
    };
    std::mutex mu;
    std::map<int32_t, std::pair<std::vector<uint64_t>, std::vector<uint64_t>>> last;
    sched.SetExecutor([&](const Operation &op) {
        if (op.Meta().type != kOperationSched) return;
        const OpSchedHeader &h = *reinterpret_cast<const OpSchedHeader *>(op.bytes.data());
        const uint64_t *handles = reinterpret_cast<const uint64_t *>(op.bytes.data() + sizeof(OpSchedHeader));
        {
            std::lock_guard<std::mutex> lk(mu);
            auto &e = last[h.meta.pid];
            e.first.assign(handles, handles + h.running_cnt);
            e.second.assign(handles + h.running_cnt, handles + h.running_cnt + h.suspended_cnt);
        }
        if (virt) return;
        Event ack = Event::OperationComplete(h.meta.id);
        reinterpret_cast<EventMeta *>(ack.bytes)->pid = h.meta.pid;
        sched.RecvEvent(ack);
    });
    if (!virt) sched.Run();
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream is(line);
        std::string cmd;
        is >> cmd;
        if (cmd == "event") {
            std::string hex;
            is >> hex;
            auto bytes = Unhex(hex);
            Event e;
            if (!e.Assign(bytes.data(), bytes.size())) { std::printf("malformed\n"); continue; }
            if (virt) sched.StepInline(&e, 1); else sched.RecvEvent(e);
        } else if (cmd == "sleep_ms") {
            int ms = 0;
            is >> ms;
            if (virt) advance(vnow + (int64_t)ms * 1000); else std::this_thread::sleep_for(std::chrono::milliseconds(ms));
        } else if (cmd == "sleep_us") {                  // virtual clock only: finer steps than sleep_ms
            long long us = 0;
            is >> us;
            if (virt) advance(vnow + us); else std::this_thread::sleep_for(std::chrono::microseconds(us));
        } else if (cmd == "flush" || cmd == "peek") {    // peek: the same report without letting time pass first
            if (cmd == "flush") { if (virt) advance(vnow + 30000); else std::this_thread::sleep_for(std::chrono::milliseconds(30)); }
            std::lock_guard<std::mutex> lk(mu);
            std::printf("flush");
            for (auto &[pid, rs] : last) {
                std::printf(" | pid %d run", (int)pid);
                for (auto h : rs.first) std::printf(" %llx", (unsigned long long)h);
                std::printf(" susp");
                for (auto h : rs.second) std::printf(" %llx", (unsigned long long)h);
            }
            std::printf("\n");
        }
    }
    if (!virt) sched.Stop();
    return 0;
}
