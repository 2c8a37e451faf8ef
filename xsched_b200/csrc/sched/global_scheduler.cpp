// GlobalScheduler: the client side of the scheduling server.  Events go to the server's channel
// (key 1); operations arrive on this process's channel (key = pid) and are executed on a worker
// thread.  Role as in the reference's sched/src/scheduler/global.cpp:7-69; a lost server ends the
// process there (XASSERT) and here as well.
#include "xsched/sched/scheduler.h"

#include "xsched/protocol/def.h"
#include "xsched/sched/ipc.h"
#include "xsched/utils/xassert.h"

namespace xsched::sched {

struct GlobalScheduler::Impl {
    IpcEndpoint recv;
    IpcEndpoint send;
    std::thread worker;
    std::atomic<bool> running{false};
};

GlobalScheduler::GlobalScheduler() : Scheduler(kSchedulerGlobal), impl_(std::make_unique<Impl>()) {}
GlobalScheduler::~GlobalScheduler() { Stop(); }

void GlobalScheduler::Run() {
    if (impl_->running) return;
    XASSERT(impl_->recv.Bind((uint64_t)GetProcessId()), "cannot open the operation channel of process %d", GetProcessId());
    XASSERT(impl_->send.OpenSender(), "cannot open the event channel");
    impl_->running = true;
    impl_->worker = std::thread([this] {
        alignas(8) unsigned char buf[65536];
        while (true) {
            const long n = impl_->recv.ReceiveAuto(buf, sizeof(buf));
            if (n <= 0) return;
            Operation op;
            if (!op.Assign(buf, (size_t)n)) { XWARN("malformed operation of %ld bytes dropped", n); continue; }
            if (op.Meta().type == kOperationTerminate) return;
            Execute(op);
        }
    });
}

void GlobalScheduler::Stop() {
    if (!impl_->running) return;
    impl_->running = false;
    impl_->recv.Close();
    if (impl_->worker.joinable()) impl_->worker.join();
    impl_->send.Close();
}

void GlobalScheduler::RecvEvent(const Event &event) {
    if (!impl_->running) return;
    if (LIKELY(impl_->send.SendTo(XSCHED_SERVER_CHANNEL_KEY, event.bytes, event.size))) return;
    // Nothing to tell when the process is on its way out anyway.
    if (event.Type() == kEventProcessDestroy || event.Type() == kEventXQueueDestroy) return;
    Stop();
    XASSERT(false, "failed to send event %d to the scheduling server (is xserver running?)", event.Type());
}

std::shared_ptr<Scheduler> CreateScheduler(XSchedulerType scheduler, XPolicyType policy) {
    // A valid policy selects the in-process scheduler regardless of the scheduler type.
    if (policy > kPolicyUnknown && policy < kPolicyMax) return std::make_shared<LocalScheduler>(policy);
    if (scheduler == kSchedulerGlobal) return std::make_shared<GlobalScheduler>();
    return std::make_shared<AppManagedScheduler>();
}

} // namespace xsched::sched
