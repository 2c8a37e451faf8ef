// sched_probe (reference build) — TEST INFRASTRUCTURE.
// Feeds raw agent->server event records (hex, one per line) into the REFERENCE's LocalScheduler
// (sched/src/scheduler/local.cpp, policies sched/src/policy/{hpf,lax}.cpp) through
// Event::CopyConstructor, and prints, at every `flush`, the newest Sched operation sent to each process.
//   usage: sched_probe_ref <HPF|LAX> < script
//   script lines:  event <hex bytes> | flush | sleep_ms <n>
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
#include "xsched/sched/protocol/event.h"
#include "xsched/sched/protocol/operation.h"
#include "xsched/sched/scheduler/local.h"

using namespace xsched::sched;

static std::vector<unsigned char> Unhex(const std::string &s) {
    std::vector<unsigned char> out;
    for (size_t i = 0; i + 1 < s.size(); i += 2) out.push_back((unsigned char)std::stoi(s.substr(i, 2), nullptr, 16));
    return out;
}

int main(int argc, char **argv) {
    const XPolicyType policy = xsched::protocol::GetPolicyType(argc > 1 ? argv[1] : "HPF");
    LocalScheduler sched(policy);
    std::mutex mu;
    std::map<PID, std::pair<std::vector<uint64_t>, std::vector<uint64_t>>> last;
    uint64_t ops = 0;
    sched.SetExecutor([&](std::shared_ptr<const Operation> op) {
        if (op->Type() != kOperationSched) return;
        auto so = std::dynamic_pointer_cast<const SchedOperation>(op);
        std::lock_guard<std::mutex> lk(mu);
        auto &e = last[so->Pid()];
        e.first.assign(so->Handles(), so->Handles() + so->RunningCnt());
        e.second.assign(so->Handles() + so->RunningCnt(), so->Handles() + so->RunningCnt() + so->SuspendedCnt());
        ++ops;
        // acknowledge, as a client would
        struct { EventMeta meta; OperationId id; } ack{{kEventOperationComplete, so->Pid()}, so->Id()};
        sched.RecvEvent(Event::CopyConstructor(&ack));
    });
    sched.Run();
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream is(line);
        std::string cmd;
        is >> cmd;
        if (cmd == "event") {
            std::string hex;
            is >> hex;
            auto bytes = Unhex(hex);
            bytes.resize(512, 0);
            sched.RecvEvent(Event::CopyConstructor(bytes.data()));
        } else if (cmd == "sleep_ms") {
            int ms = 0;
            is >> ms;
            std::this_thread::sleep_for(std::chrono::milliseconds(ms));
        } else if (cmd == "flush") {
            std::this_thread::sleep_for(std::chrono::milliseconds(30));
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
    sched.Stop();
    return 0;
}
