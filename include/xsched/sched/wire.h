// Wire format between a client process's scheduling agent and the scheduling server: tagged, fixed
// layout byte records.  A record's first field is its tag.  The layouts reproduce, byte for byte on
// x86-64 / aarch64 Linux, the POD structs the reference sends:
//   events      sched/include/xsched/sched/protocol/event.h:17-433
//   operations  sched/include/xsched/sched/protocol/operation.h:15-140
//   hints       sched/include/xsched/sched/protocol/hint.h:16-264
// so that a client and a server from the two code bases can be mixed.  The static_asserts pin sizes
// and offsets.  Query events carry a raw pointer in the reference and never leave the process; here
// the in-process status query is a direct call and has no record.
#pragma once
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>
#include "xsched/types.h"
#include "xsched/utils/common.h"

namespace xsched::sched {

enum EventType : int32_t {
    kEventHint = 0, kEventSchedulerTerminate = 1, kEventProcessCreate = 2, kEventProcessDestroy = 3,
    kEventXQueueCreate = 4, kEventXQueueDestroy = 5, kEventXQueueReady = 6, kEventXQueueIdle = 7,
    kEventXQueueConfigUpdate = 8, kEventXQueueQuery = 9, kEventXQueueQueryAll = 10, kEventOperationComplete = 11,
};
enum HintType : int32_t {
    kHintTypeUnknown = 0, kHintTypePriority = 1, kHintTypeUtilization = 2, kHintTypeTimeslice = 3,
    kHintTypeDeadline = 4, kHintTypeKDeadline = 5, kHintTypeLaxity = 6, kHintTypeWindowActive = 7, kHintTypeMax = 8,
};
enum OperationType : int32_t { kOperationNone = 0, kOperationTerminate = 1, kOperationSched = 2, kOperationConfig = 4 };
typedef uint64_t OperationId;

struct EventMeta { int32_t type; int32_t pid; };

// ---- hints (payload of a hint event) ----
struct HintPriority    { int32_t type; int32_t pad0; uint64_t handle; int32_t prio; int32_t pad1; };
struct HintUtilization { int32_t type; int32_t pid; uint64_t handle; int32_t util; int32_t pad1; };
struct HintTimeslice   { int32_t type; int32_t pad0; int64_t ts_us; };
struct HintDeadline    { int32_t type; int32_t pad0; uint64_t handle; int64_t ddl_us; };
struct HintKDeadline   { int32_t type; int32_t pad0; uint64_t k; };
struct HintLaxity      { int32_t type; int32_t pad0; uint64_t handle; int64_t lax_us; int32_t lax_prio; int32_t crit_prio; };
struct HintWindowActive { int32_t type; int32_t pid; uint64_t display; };
static_assert(sizeof(HintPriority) == 24 && offsetof(HintPriority, prio) == 16, "wire");
static_assert(sizeof(HintUtilization) == 24 && offsetof(HintUtilization, util) == 16, "wire");
static_assert(sizeof(HintTimeslice) == 16 && sizeof(HintDeadline) == 24 && sizeof(HintKDeadline) == 16, "wire");
static_assert(sizeof(HintLaxity) == 32 && offsetof(HintLaxity, lax_prio) == 24, "wire");
static_assert(sizeof(HintWindowActive) == 16 && offsetof(HintWindowActive, display) == 8, "wire");

// ---- events ----
struct EvHint          { EventMeta meta; uint64_t size; char hint[64]; };   // `size` bytes are sent
struct EvPlain         { EventMeta meta; };                                 // terminate, process destroy
struct EvProcessCreate { EventMeta meta; char cmdline[256]; };
struct EvXQueueConfig  { EventMeta meta; uint64_t handle; uint64_t device; int32_t level; int32_t pad0;
                         int64_t threshold; int64_t batch_size; };          // create, config update
struct EvXQueueHandle  { EventMeta meta; uint64_t handle; };                // destroy, idle
struct EvXQueueReady   { EventMeta meta; uint64_t handle; int64_t ready_time_us; };  // us since the epoch
struct EvOpComplete    { EventMeta meta; uint64_t op_id; };
static_assert(offsetof(EvHint, hint) == 16 && sizeof(EvPlain) == 8 && sizeof(EvProcessCreate) == 264, "wire");
static_assert(sizeof(EvXQueueConfig) == 48 && offsetof(EvXQueueConfig, threshold) == 32, "wire");
static_assert(sizeof(EvXQueueHandle) == 16 && sizeof(EvXQueueReady) == 24 && sizeof(EvOpComplete) == 16, "wire");

// ---- operations ----
struct OperationMeta { uint64_t id; int32_t type; int32_t pid; };
struct OpSchedHeader { OperationMeta meta; uint64_t size; uint64_t running_cnt; uint64_t suspended_cnt; };
//   followed by running_cnt + suspended_cnt XQueue handles: first the ones to run, then the ones to suspend
struct OpConfig      { OperationMeta meta; uint64_t handle; int32_t level; int32_t pad0; int64_t threshold; int64_t batch_size; };
static_assert(sizeof(OperationMeta) == 16 && sizeof(OpSchedHeader) == 40 && sizeof(OpConfig) == 48, "wire");

/// An event with its bytes.  Small enough to copy.
struct Event {
    uint32_t size = 0;
    alignas(8) unsigned char bytes[272];

    int32_t Type() const { return reinterpret_cast<const EventMeta *>(bytes)->type; }
    int32_t Pid() const { return reinterpret_cast<const EventMeta *>(bytes)->pid; }
    template <class T> const T &As() const { return *reinterpret_cast<const T *>(bytes); }
    template <class T> T &Init(int32_t type, size_t sz = sizeof(T)) {
        std::memset(bytes, 0, sizeof(T));
        size = (uint32_t)sz;
        T &t = *reinterpret_cast<T *>(bytes);
        t.meta.type = type;
        t.meta.pid = (int32_t)GetProcessId();
        return t;
    }
    /// Parse received bytes; false if the record is truncated or its tag is unknown.
    bool Assign(const void *data, size_t n);

    static Event Terminate();
    static Event ProcessCreate(const std::string &cmdline);
    static Event ProcessDestroy(int32_t pid);
    static Event XQueueCreate(uint64_t handle, uint64_t device, int32_t level, int64_t threshold, int64_t batch);
    static Event XQueueConfigUpdate(uint64_t handle, uint64_t device, int32_t level, int64_t threshold, int64_t batch);
    static Event XQueueDestroy(uint64_t handle);
    static Event XQueueReady(uint64_t handle, int64_t ready_time_us);
    static Event XQueueIdle(uint64_t handle);
    static Event OperationComplete(uint64_t op_id);
    static Event Hint(const void *hint, size_t hint_size);
};

/// An operation with its bytes (variable length for kOperationSched).
struct Operation {
    std::vector<unsigned char> bytes;
    const OperationMeta &Meta() const { return *reinterpret_cast<const OperationMeta *>(bytes.data()); }
    bool Assign(const void *data, size_t n);
    static Operation Terminate(int32_t pid);
    static Operation Sched(uint64_t id, int32_t pid, const std::vector<uint64_t> &running, const std::vector<uint64_t> &suspended);
    static Operation Config(uint64_t id, int32_t pid, uint64_t handle, int32_t level, int64_t threshold, int64_t batch);
};

inline int64_t NowEpochUs() {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

} // namespace xsched::sched
