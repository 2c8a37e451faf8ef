// xserver <POLICY> [port] — the scheduling server of one box.
//
// One policy instance decides for every XQueue of every client process on all GPUs of the box; state is
// kept per XDevice, so the 8 GPUs are independent XQueue sets under one policy.  Clients (processes
// running with XSCHED_SCHEDULER=GLB) send events to channel key 1; operations go back on the channel
// whose key is the client's pid.  A client that dies without saying goodbye is noticed through a pidfd
// and removed, which lets the policy resume whatever it had suspended on the survivor's behalf.
//
// Role of the reference's service/server (server.cpp:47-202, main.cpp:20-44).  The HTTP/JSON routes
// that serve `xcli` there are not part of this program; `port` is accepted for command-line
// compatibility and ignored.  With --status-interval-ms N the server prints one JSON line with the
// queue table every N ms (what `xcli list` would show).
#include <atomic>
#include <chrono>
#include <csignal>
#include <deque>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include <poll.h>
#include <sys/syscall.h>
#include <unistd.h>

#include "xsched/protocol/def.h"
#include "xsched/protocol/names.h"
#include "xsched/sched/ipc.h"
#include "xsched/sched/scheduler.h"
#include "xsched/utils/trace.h"
#include "xsched/utils/xassert.h"

using namespace xsched::sched;

namespace {

std::atomic<bool> g_stop{false};
IpcEndpoint *g_recv = nullptr;

void OnSignal(int) {
    g_stop.store(true);
    if (g_recv) g_recv->Close();
}

class Server {
public:
    explicit Server(XPolicyType policy) : sched_(policy) {
        sched_.SetExecutor([this](const Operation &op) { Send(op); });
    }

    int Run(int status_interval_ms) {
        if (!recv_.Bind(XSCHED_SERVER_CHANNEL_KEY)) {
            std::fprintf(stderr, "xserver: cannot bind the server channel (another xserver running?)\n");
            return 1;
        }
        XASSERT(send_.OpenSender(), "cannot open the operation socket");
        g_recv = &recv_;
        const bool spin = GetEnvOption(XSCHED_IPC_SPIN_ENV_NAME, false);
        if (!spin) sched_.Run();
        std::thread watcher([this] { WatchClients(); });
        std::thread status;
        if (status_interval_ms > 0) status = std::thread([this, status_interval_ms] { PrintStatus(status_interval_ms); });
        std::printf("xserver ready policy=%s pid=%d mode=%s\n", xsched::protocol::GetPolicyTypeName(sched_.GetPolicy()), (int)getpid(),
                    spin ? "polling" : "blocking");
        std::fflush(stdout);

        alignas(8) unsigned char buf[4096];
        if (spin) {
            // Polling mode: one thread receives, updates the status, runs the policy and sends the
            // operations — no hand-off to a worker thread, no sleep between a ready event and the suspend
            // operation it causes.  Policy timers are served from the same loop.
            std::vector<Event> batch;
            while (!g_stop.load()) {
                batch.clear();
                while (batch.size() < 64) {
                    const long n = recv_.TryReceive(buf, sizeof(buf));
                    if (n == -2) break;
                    if (n <= 0) { g_stop.store(true); break; }
                    Event e;
                    if (!e.Assign(buf, (size_t)n)) continue;
                    XTRACE(xsched::utils::kTraceEventRecv, (uint64_t)e.Type(), (uint64_t)e.Pid());
                    if (e.Type() == kEventProcessCreate) Track(e.Pid());
                    if (e.Type() == kEventProcessDestroy) Untrack(e.Pid());
                    batch.push_back(e);
                }
                {
                    std::lock_guard<std::mutex> lk(inject_mu_);
                    for (auto &e : injected_) batch.push_back(e);
                    injected_.clear();
                }
                FlushOutbox();
                if (!batch.empty() || NowEpochUs() >= sched_.NextTimerUs()) sched_.StepInline(batch.data(), batch.size());
                else for (int i = 0; i < 16; ++i) __builtin_ia32_pause();
            }
        } else {
            while (!g_stop.load()) {
                // Operations are parked by the scheduler's thread; wake up regularly to retry them
                // (every millisecond while some are parked, every 20 ms otherwise).
                if (!recv_.WaitReadable(FlushOutbox() ? 1 : 20)) continue;
                const long n = recv_.Receive(buf, sizeof(buf));
                if (n <= 0) break;
                Event e;
                if (!e.Assign(buf, (size_t)n)) { XWARN("malformed event of %ld bytes dropped", n); continue; }
                XTRACE(xsched::utils::kTraceEventRecv, (uint64_t)e.Type(), (uint64_t)e.Pid());
                if (e.Type() == kEventProcessCreate) Track(e.Pid());
                if (e.Type() == kEventProcessDestroy) Untrack(e.Pid());
                if (e.Type() == kEventSchedulerTerminate) continue;      // clients cannot stop the server
                sched_.RecvEvent(e);
            }
        }
        g_stop.store(true);
        watcher.join();
        if (status.joinable()) status.join();
        if (!spin) sched_.Stop();
        return 0;
    }

private:
    // The server must never block in a send: a client whose receive queue is full may itself be blocked
    // sending to the server, and two blocked senders would wait for each other forever (datagram queues
    // hold only a handful of records).  An operation that cannot be delivered now is parked per client and
    // retried from the main loop; since a Sched operation carries the client's complete running/suspended
    // sets, a newer one simply replaces a parked older one.
    void Send(const Operation &op) {
        const int32_t pid = op.Meta().pid;
        std::lock_guard<std::mutex> lk(out_mu_);
        auto it = outbox_.find(pid);
        if (it != outbox_.end()) {
            if (op.Meta().type == kOperationSched && it->second.back().Meta().type == kOperationSched) it->second.back() = op;
            else it->second.push_back(op);
            return;
        }
        const int r = send_.TrySendTo((uint64_t)pid, op.bytes.data(), op.bytes.size());
        if (r == 1) return;
        if (r == 0) { outbox_[pid].push_back(op); return; }
        AckOnBehalf(op);        // the client is gone or not listening yet: nobody should wait for it
    }

    void AckOnBehalf(const Operation &op) {
        Event ack = Event::OperationComplete(op.Meta().id);
        reinterpret_cast<EventMeta *>(ack.bytes)->pid = op.Meta().pid;
        Deliver(ack);
    }

    /// Retry parked operations.  Returns true while something is still parked.
    bool FlushOutbox() {
        std::lock_guard<std::mutex> lk(out_mu_);
        for (auto it = outbox_.begin(); it != outbox_.end();) {
            auto &q = it->second;
            while (!q.empty()) {
                const int r = send_.TrySendTo((uint64_t)it->first, q.front().bytes.data(), q.front().bytes.size());
                if (r == 0) break;
                if (r < 0) AckOnBehalf(q.front());
                q.pop_front();
            }
            it = q.empty() ? outbox_.erase(it) : std::next(it);
        }
        return !outbox_.empty();
    }

    // Events produced inside the server (client death, acknowledgements on behalf of a dead client).
    void Deliver(const Event &e) {
        static const bool spin = GetEnvOption(XSCHED_IPC_SPIN_ENV_NAME, false);
        if (!spin) { sched_.RecvEvent(e); return; }
        std::lock_guard<std::mutex> lk(inject_mu_);
        injected_.push_back(e);
    }

    void Track(int32_t pid) {
        std::lock_guard<std::mutex> lk(mu_);
        if (clients_.count(pid)) return;
        const int fd = (int)syscall(SYS_pidfd_open, pid, 0);
        clients_[pid] = fd;      // fd < 0: fall back to kill(pid, 0) probing
    }
    void Untrack(int32_t pid) {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = clients_.find(pid);
        if (it == clients_.end()) return;
        if (it->second >= 0) ::close(it->second);
        clients_.erase(it);
    }

    void WatchClients() {
        while (!g_stop.load()) {
            std::vector<std::pair<int32_t, int>> snap;
            { std::lock_guard<std::mutex> lk(mu_); snap.assign(clients_.begin(), clients_.end()); }
            std::vector<pollfd> fds;
            for (auto &[pid, fd] : snap) if (fd >= 0) fds.push_back(pollfd{fd, POLLIN, 0});
            if (!fds.empty()) ::poll(fds.data(), fds.size(), 50);
            else std::this_thread::sleep_for(std::chrono::milliseconds(50));
            size_t k = 0;
            for (auto &[pid, fd] : snap) {
                bool dead = false;
                if (fd >= 0) dead = (fds[k++].revents & (POLLIN | POLLHUP | POLLERR)) != 0;
                else dead = (::kill(pid, 0) != 0 && errno == ESRCH);
                if (!dead) continue;
                XINFO("client %d is gone; removing its XQueues", pid);
                Untrack(pid);
                Deliver(Event::ProcessDestroy(pid));
            }
        }
    }

    void PrintStatus(int interval_ms) {
        while (!g_stop.load()) {
            std::this_thread::sleep_for(std::chrono::milliseconds(interval_ms));
            const Status st = sched_.Snapshot();
            std::string out = "{\"xqueues\": [";
            bool first = true;
            for (const auto &[h, q] : st.xqueues) {
                char line[256];
                std::snprintf(line, sizeof(line), "%s{\"handle\": \"0x%llx\", \"device\": \"0x%llx\", \"level\": %d, \"pid\": %d, "
                              "\"threshold\": %lld, \"batch_size\": %lld, \"ready\": %s, \"suspended\": %s}",
                              first ? "" : ", ", (unsigned long long)h, (unsigned long long)q.device, q.level, (int)q.pid,
                              (long long)q.threshold, (long long)q.batch_size, q.ready ? "true" : "false", q.suspended ? "true" : "false");
                out += line;
                first = false;
            }
            out += "], \"rounds\": " + std::to_string(sched_.Rounds()) + "}";
            std::printf("%s\n", out.c_str());
            std::fflush(stdout);
        }
    }

    LocalScheduler sched_;
    IpcEndpoint recv_, send_;
    std::mutex mu_;
    std::map<int32_t, int> clients_;
    std::mutex inject_mu_;
    std::vector<Event> injected_;
    std::mutex out_mu_;
    std::map<int32_t, std::deque<Operation>> outbox_;
};

} // namespace

int main(int argc, char **argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: xserver <HPF|HHPF|CHPF|UP|PUP|KEDF|LAX|AWF|CFS|MLFQ> [port] [--status-interval-ms N]\n");
        return 2;
    }
    const XPolicyType policy = xsched::protocol::GetPolicyType(argv[1]);
    if (xsched::sched::CreatePolicy(policy) == nullptr) {
        std::fprintf(stderr, "xserver: policy '%s' is not provided\n", argv[1]);
        return 2;
    }
    int status_ms = 0;
    for (int i = 2; i + 1 < argc; ++i) if (std::strcmp(argv[i], "--status-interval-ms") == 0) status_ms = std::atoi(argv[i + 1]);
    std::signal(SIGINT, OnSignal);
    std::signal(SIGTERM, OnSignal);
    Server server(policy);
    return server.Run(status_ms);
}
