// Builders and parsers of the agent <-> server records (layouts in xsched/sched/wire.h).
#include "xsched/sched/wire.h"

#include <algorithm>

namespace xsched::sched {

static size_t ExpectedEventSize(int32_t type, const void *data, size_t n) {
    switch (type) {
    case kEventHint: {
        if (n < offsetof(EvHint, hint)) return 0;
        const uint64_t sz = reinterpret_cast<const EvHint *>(data)->size;
        return (sz >= offsetof(EvHint, hint) + 4 && sz <= sizeof(EvHint)) ? (size_t)sz : 0;
    }
    case kEventSchedulerTerminate:
    case kEventProcessDestroy: return sizeof(EvPlain);
    case kEventProcessCreate: return sizeof(EvProcessCreate);
    case kEventXQueueCreate:
    case kEventXQueueConfigUpdate: return sizeof(EvXQueueConfig);
    case kEventXQueueDestroy:
    case kEventXQueueIdle: return sizeof(EvXQueueHandle);
    case kEventXQueueReady: return sizeof(EvXQueueReady);
    case kEventOperationComplete: return sizeof(EvOpComplete);
    default: return 0;
    }
}

bool Event::Assign(const void *data, size_t n) {
    if (!data || n < sizeof(EventMeta) || n > sizeof(bytes)) return false;
    const size_t want = ExpectedEventSize(reinterpret_cast<const EventMeta *>(data)->type, data, n);
    if (want == 0 || n < want) return false;
    std::memcpy(bytes, data, want);
    size = (uint32_t)want;
    return true;
}

Event Event::Terminate() { Event e; e.Init<EvPlain>(kEventSchedulerTerminate); return e; }

Event Event::ProcessCreate(const std::string &cmdline) {
    Event e;
    EvProcessCreate &d = e.Init<EvProcessCreate>(kEventProcessCreate);
    std::strncpy(d.cmdline, cmdline.c_str(), sizeof(d.cmdline) - 1);
    return e;
}

Event Event::ProcessDestroy(int32_t pid) {
    Event e;
    e.Init<EvPlain>(kEventProcessDestroy).meta.pid = pid;
    return e;
}

static Event MakeConfig(int32_t type, uint64_t handle, uint64_t device, int32_t level, int64_t threshold, int64_t batch) {
    Event e;
    EvXQueueConfig &d = e.Init<EvXQueueConfig>(type);
    d.handle = handle; d.device = device; d.level = level; d.threshold = threshold; d.batch_size = batch;
    return e;
}
Event Event::XQueueCreate(uint64_t h, uint64_t dev, int32_t lvl, int64_t th, int64_t bs) { return MakeConfig(kEventXQueueCreate, h, dev, lvl, th, bs); }
Event Event::XQueueConfigUpdate(uint64_t h, uint64_t dev, int32_t lvl, int64_t th, int64_t bs) { return MakeConfig(kEventXQueueConfigUpdate, h, dev, lvl, th, bs); }

Event Event::XQueueDestroy(uint64_t handle) { Event e; e.Init<EvXQueueHandle>(kEventXQueueDestroy).handle = handle; return e; }
Event Event::XQueueIdle(uint64_t handle) { Event e; e.Init<EvXQueueHandle>(kEventXQueueIdle).handle = handle; return e; }

Event Event::XQueueReady(uint64_t handle, int64_t ready_time_us) {
    Event e;
    EvXQueueReady &d = e.Init<EvXQueueReady>(kEventXQueueReady);
    d.handle = handle; d.ready_time_us = ready_time_us;
    return e;
}

Event Event::OperationComplete(uint64_t op_id) { Event e; e.Init<EvOpComplete>(kEventOperationComplete).op_id = op_id; return e; }

Event Event::Hint(const void *hint, size_t hint_size) {
    Event e;
    hint_size = std::min(hint_size, sizeof(EvHint::hint));
    EvHint &d = e.Init<EvHint>(kEventHint, offsetof(EvHint, hint) + hint_size);
    d.size = offsetof(EvHint, hint) + hint_size;
    std::memcpy(d.hint, hint, hint_size);
    return e;
}

bool Operation::Assign(const void *data, size_t n) {
    if (!data || n < sizeof(OperationMeta)) return false;
    const OperationMeta *m = reinterpret_cast<const OperationMeta *>(data);
    size_t want = 0;
    switch (m->type) {
    case kOperationTerminate: want = sizeof(OperationMeta); break;
    case kOperationConfig: want = sizeof(OpConfig); break;
    case kOperationSched: {
        if (n < sizeof(OpSchedHeader)) return false;
        const OpSchedHeader *h = reinterpret_cast<const OpSchedHeader *>(data);
        want = sizeof(OpSchedHeader) + (size_t)(h->running_cnt + h->suspended_cnt) * sizeof(uint64_t);
        if (h->size != want) return false;
        break;
    }
    default: return false;
    }
    if (n < want) return false;
    bytes.assign((const unsigned char *)data, (const unsigned char *)data + want);
    return true;
}

Operation Operation::Terminate(int32_t pid) {
    Operation op;
    op.bytes.resize(sizeof(OperationMeta));
    OperationMeta m{0, kOperationTerminate, pid};
    std::memcpy(op.bytes.data(), &m, sizeof(m));
    return op;
}

Operation Operation::Sched(uint64_t id, int32_t pid, const std::vector<uint64_t> &running, const std::vector<uint64_t> &suspended) {
    Operation op;
    const size_t total = sizeof(OpSchedHeader) + (running.size() + suspended.size()) * sizeof(uint64_t);
    op.bytes.resize(total);
    OpSchedHeader h{};
    h.meta = OperationMeta{id, kOperationSched, pid};
    h.size = total; h.running_cnt = running.size(); h.suspended_cnt = suspended.size();
    std::memcpy(op.bytes.data(), &h, sizeof(h));
    uint64_t *handles = reinterpret_cast<uint64_t *>(op.bytes.data() + sizeof(h));
    std::copy(running.begin(), running.end(), handles);
    std::copy(suspended.begin(), suspended.end(), handles + running.size());
    return op;
}

Operation Operation::Config(uint64_t id, int32_t pid, uint64_t handle, int32_t level, int64_t threshold, int64_t batch) {
    Operation op;
    op.bytes.resize(sizeof(OpConfig));
    OpConfig c{};
    c.meta = OperationMeta{id, kOperationConfig, pid};
    c.handle = handle; c.level = level; c.threshold = threshold; c.batch_size = batch;
    std::memcpy(op.bytes.data(), &c, sizeof(c));
    return op;
}

} // namespace xsched::sched
