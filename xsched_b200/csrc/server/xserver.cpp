// xserver <POLICY> [port] — the scheduling server of one box.
//
// One policy instance decides for every XQueue of every client process on all GPUs of the box; state is
// kept per XDevice, so the 8 GPUs are independent XQueue sets under one policy.  Clients (processes
// running with XSCHED_SCHEDULER=GLB) send events to channel key 1; operations go back on the channel
// whose key is the client's pid.  A client that dies without saying goodbye is noticed through a pidfd
// and removed, which lets the policy resume whatever it had suspended on the survivor's behalf.
//
// Role of the reference's service/server (server.cpp:47-202, main.cpp:20-44).  `port` is where the control
// interface listens (HTTP/JSON, the routes `xcli` and scripts use; reference: server.cpp:28-39,228-544):
//   GET  /xqueues                 every XQueue {handle, device, level, pid, threshold, batch_size, ready, suspended}
//                                 and every client process {pid, cmdline}
//   GET  /xqueue/<hex handle>     one XQueue and its process
//   POST /config/<hex handle>     ?level=&threshold=&batch_size=   -> a Config operation to the owning process
//   GET  /policy  |  POST /policy ?policy=<number>                  -> hot swap (everything is resumed first)
//   POST /hint                    JSON body {"hint_type": n, ...}   -> the hint reaches the policy like a client's
// It binds 127.0.0.1 (--http-addr changes that); a port that cannot be bound is reported and the server runs on
// without the interface.  With --status-interval-ms N the server also prints the queue table every N ms.
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
#include "server/http.h"
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

    int Run(int status_interval_ms, const std::string &http_addr, int http_port) {
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
        uint16_t bound = 0;
        if (http_port > 0) {
            InstallRoutes();
            bound = http_.Start(http_addr, (uint16_t)http_port);
            if (!bound) XWARN("control interface: cannot listen on %s:%d (%s); continuing without it", http_addr.c_str(), http_port, std::strerror(errno));
        }
        std::printf("xserver ready policy=%s pid=%d mode=%s http=%s\n", xsched::protocol::GetPolicyTypeName(sched_.GetPolicy()), (int)getpid(),
                    spin ? "polling" : "blocking", bound ? std::to_string(bound).c_str() : "off");
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
                if (!batch.empty() || NowEpochUs() >= sched_.NextTimerUs()) {
                    std::lock_guard<std::mutex> step(step_mu_);       // a policy swap from the control interface waits here
                    sched_.StepInline(batch.data(), batch.size());
                }
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
        http_.Stop();
        watcher.join();
        if (status.joinable()) status.join();
        if (!spin) sched_.Stop();
        return 0;
    }

private:
    // ---- control interface ----------------------------------------------------------------------------
    static std::string QueueJson(const XQueueStatus &q) {
        char line[320];
        std::snprintf(line, sizeof(line), "{\"handle\": %llu, \"device\": %llu, \"level\": %d, \"pid\": %d, \"threshold\": %lld, \"batch_size\": %lld, "
                      "\"ready\": %s, \"suspended\": %s}", (unsigned long long)q.handle, (unsigned long long)q.device, (int)q.level, (int)q.pid,
                      (long long)q.threshold, (long long)q.batch_size, q.ready ? "true" : "false", q.suspended ? "true" : "false");
        return line;
    }
    static std::string ProcessJson(const ProcessStatus &p) {
        return "{\"pid\": " + std::to_string((int)p.pid) + ", \"cmdline\": \"" + xsched::service::JsonEscape(p.cmdline) + "\"}";
    }
    static bool ParseHandle(const std::string &hex, uint64_t *out) {
        if (hex.empty()) return false;
        char *end = nullptr;
        errno = 0;
        const unsigned long long v = std::strtoull(hex.c_str(), &end, 16);
        if (errno != 0 || end == nullptr || *end != '\0' || v == 0) return false;
        *out = v;
        return true;
    }
    static bool ParseInt(const std::string &text, long long *out) {
        if (text.empty()) return false;
        char *end = nullptr;
        errno = 0;
        const long long v = std::strtoll(text.c_str(), &end, 10);
        if (errno != 0 || end == nullptr || *end != '\0') return false;
        *out = v;
        return true;
    }
    static void Fail(xsched::service::HttpResponse &res, int status, const char *why) {
        res.status = status;
        res.body = why ? std::string("{\"error\": \"") + why + "\"}" : "";
    }

    void InstallRoutes() {
        using xsched::service::HttpRequest;
        using xsched::service::HttpResponse;
        http_.Route("GET", "/xqueues", false, [this](const HttpRequest &, HttpResponse &res) {
            const Status st = sched_.Snapshot();
            std::string out = "{\"xqueues\": [";
            bool first = true;
            for (const auto &[h, q] : st.xqueues) { out += (first ? "" : ", ") + QueueJson(q); first = false; }
            out += "], \"processes\": [";
            first = true;
            for (const auto &[pid, p] : st.processes) { out += (first ? "" : ", ") + ProcessJson(p); first = false; }
            res.body = out + "]}";
        });
        http_.Route("GET", "/xqueue/", true, [this](const HttpRequest &req, HttpResponse &res) {
            uint64_t handle = 0;
            if (!ParseHandle(req.Get("_tail"), &handle)) return Fail(res, 400, nullptr);
            const Status st = sched_.Snapshot();
            auto it = st.xqueues.find(handle);
            if (it == st.xqueues.end()) return Fail(res, 404, nullptr);
            auto pit = st.processes.find(it->second.pid);
            ProcessStatus none;
            none.pid = it->second.pid;
            res.body = "{\"xqueue\": " + QueueJson(it->second) + ", \"process\": " + ProcessJson(pit == st.processes.end() ? none : pit->second) + "}";
        });
        http_.Route("POST", "/config/", true, [this](const HttpRequest &req, HttpResponse &res) {
            uint64_t handle = 0;
            if (!ParseHandle(req.Get("_tail"), &handle)) return Fail(res, 400, nullptr);
            long long level = kPreemptLevelUnknown, threshold = -1, batch = -1;
            if (req.Has("level") && (!ParseInt(req.Get("level"), &level) || level <= kPreemptLevelUnknown || level >= kPreemptLevelMax)) return Fail(res, 400, "invalid level");
            if (req.Has("threshold") && (!ParseInt(req.Get("threshold"), &threshold) || threshold <= 0)) return Fail(res, 400, "invalid command threshold");
            if (req.Has("batch_size") && (!ParseInt(req.Get("batch_size"), &batch) || batch <= 0)) return Fail(res, 400, "invalid command batch size");
            const Status st = sched_.Snapshot();
            auto it = st.xqueues.find(handle);
            if (it == st.xqueues.end()) return Fail(res, 404, "XQueue not found");
            const long long new_threshold = threshold > 0 ? threshold : it->second.threshold, new_batch = batch > 0 ? batch : it->second.batch_size;
            // The XQueue itself requires threshold >= batch size (the reference's route asks for strictly less,
            // its core asserts >=: preempt/src/xqueue/launch_worker.cpp:14); follow the core.
            if (new_batch > new_threshold) return Fail(res, 400, "batch size must not exceed threshold");
            if (level == kPreemptLevelUnknown && threshold == -1 && batch == -1) { res.body = "{\"warning\": \"no change\"}"; return; }
            const uint64_t id = sched_.NextOperationId(it->second.pid);
            Send(Operation::Config(id, it->second.pid, handle, (int32_t)level, threshold, batch));
            res.body = "{\"info\": \"success\"}";
        });
        http_.Route("GET", "/policy", false, [this](const HttpRequest &, HttpResponse &res) {
            res.body = "{\"policy\": " + std::to_string((int)sched_.GetPolicy()) + ", \"name\": \"" + xsched::protocol::GetPolicyTypeName(sched_.GetPolicy()) + "\"}";
        });
        http_.Route("POST", "/policy", false, [this](const HttpRequest &req, HttpResponse &res) {
            long long type = 0;
            if (!req.Has("policy") || !ParseInt(req.Get("policy"), &type) || type <= kPolicyUnknown || type >= kPolicyMax) return Fail(res, 400, nullptr);
            if (xsched::sched::CreatePolicy((XPolicyType)type) == nullptr) return Fail(res, 400, "policy not provided");
            {
                std::lock_guard<std::mutex> step(step_mu_);
                sched_.SetPolicy((XPolicyType)type);
            }
            res.body = "{\"info\": \"success\"}";
        });
        http_.Route("POST", "/hint", false, [this](const HttpRequest &req, HttpResponse &res) {
            std::map<std::string, std::string> j;
            if (!xsched::service::ParseFlatJson(req.body, &j)) return Fail(res, 400, nullptr);
            auto num = [&](const char *k, long long *out) { auto it = j.find(k); return it != j.end() && ParseInt(it->second, out); };
            auto handle_of = [&]() -> uint64_t { auto it = j.find("handle"); return it == j.end() ? 0 : std::strtoull(it->second.c_str(), nullptr, 10); };
            long long type = 0;
            if (!j.count("hint_type")) return Fail(res, 400, "missing hint type");
            if (!num("hint_type", &type) || type <= kHintTypeUnknown || type >= kHintTypeMax) return Fail(res, 400, "invalid hint type");
            long long v = 0, pid = 0;
            num("pid", &pid);
            switch (type) {
            case kHintTypePriority: {
                const uint64_t h = handle_of();
                if (h == 0) return Fail(res, 400, "invalid handle");
                if (!j.count("priority")) return Fail(res, 400, "missing priority");
                if (!num("priority", &v) || v < PRIORITY_MIN || v > PRIORITY_MAX) return Fail(res, 400, "invalid priority");
                const HintPriority hint{kHintTypePriority, 0, h, (int32_t)v, 0};
                Deliver(Event::Hint(&hint, sizeof(hint)));
                break;
            }
            case kHintTypeUtilization: {
                const uint64_t h = handle_of();
                if (h == 0 && pid == 0) return Fail(res, 400, "handle or pid is required");
                if (!j.count("utilization")) return Fail(res, 400, "missing utilization");
                if (!num("utilization", &v) || v < UTILIZATION_MIN || v > UTILIZATION_MAX) return Fail(res, 400, "invalid utilization");
                const HintUtilization hint{kHintTypeUtilization, (int32_t)pid, h, (int32_t)v, 0};
                Deliver(Event::Hint(&hint, sizeof(hint)));
                break;
            }
            case kHintTypeTimeslice: {
                if (!j.count("timeslice")) return Fail(res, 400, "missing timeslice");
                if (!num("timeslice", &v) || v <= 0) return Fail(res, 400, "invalid timeslice");
                const HintTimeslice hint{kHintTypeTimeslice, 0, v};
                Deliver(Event::Hint(&hint, sizeof(hint)));
                break;
            }
            case kHintTypeLaxity: {
                const uint64_t h = handle_of();
                long long lax_prio = 0, crit_prio = 0;
                if (h == 0) return Fail(res, 400, "invalid handle");
                if (!num("laxity", &v) || v < 0) return Fail(res, 400, "invalid laxity");
                num("lax_priority", &lax_prio);
                num("critical_priority", &crit_prio);
                const HintLaxity hint{kHintTypeLaxity, 0, h, v, (int32_t)lax_prio, (int32_t)crit_prio};
                Deliver(Event::Hint(&hint, sizeof(hint)));
                break;
            }
            case kHintTypeWindowActive: {
                long long display = 0;
                if (!j.count("pid")) return Fail(res, 400, "missing pid");
                if (!j.count("display") || !num("display", &display)) return Fail(res, 400, "missing display");
                const HintWindowActive hint{kHintTypeWindowActive, (int32_t)pid, (uint64_t)display};
                Deliver(Event::Hint(&hint, sizeof(hint)));
                break;
            }
            default:
                return Fail(res, 400, "invalid hint type");
            }
            res.body = "{\"info\": \"success\"}";
        });
    }

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
    xsched::service::HttpServer http_;
    std::mutex step_mu_;                 // the policy loop of the polling mode against a policy swap from the control interface
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
        std::fprintf(stderr, "usage: xserver <HPF|HHPF|CHPF|UP|PUP|KEDF|LAX|AWF|CFS|MLFQ> [port] [--http-addr A] [--status-interval-ms N]\n");
        return 2;
    }
    const XPolicyType policy = xsched::protocol::GetPolicyType(argv[1]);
    if (xsched::sched::CreatePolicy(policy) == nullptr) {
        std::fprintf(stderr, "xserver: policy '%s' is not provided\n", argv[1]);
        return 2;
    }
    int status_ms = 0;
    int port = argc > 2 && argv[2][0] != '-' ? std::atoi(argv[2]) : XSCHED_SERVER_DEFAULT_PORT;
    std::string http_addr = "127.0.0.1";
    for (int i = 2; i + 1 < argc; ++i) {
        if (std::strcmp(argv[i], "--status-interval-ms") == 0) status_ms = std::atoi(argv[i + 1]);
        if (std::strcmp(argv[i], "--http-addr") == 0) http_addr = argv[i + 1];
    }
    std::signal(SIGINT, OnSignal);
    std::signal(SIGTERM, OnSignal);
    Server server(policy);
    return server.Run(status_ms, http_addr, port);
}
