// Small shared helpers of the host runtime.  Macro and function names follow the reference's
// utils/include/xsched/utils/common.h so that HAL sources written against it compile unchanged.
#pragma once
#include <cerrno>
#include <cinttypes>
#include <cstdint>
#include <cstring>
#include <string>
#include <unistd.h>
#include <sys/syscall.h>
#include <sys/types.h>

#define LIKELY(x)   __builtin_expect(!!(x), 1)
#define UNLIKELY(x) __builtin_expect(!!(x), 0)

#define NO_COPY_CLASS(T) T(const T &) = delete; T &operator=(const T &) = delete;
#define NO_MOVE_CLASS(T) T(T &&) = delete; T &operator=(T &&) = delete;
#define STATIC_CLASS(T)  T() = delete; ~T() = delete; NO_COPY_CLASS(T) NO_MOVE_CLASS(T)

#define UNUSED(expr) do { (void)(expr); } while (0)
#define ROUND_UP(x, a)   ((((x) + (a) - 1) / (a)) * (a))
#define ROUND_DOWN(x, a) ((x) / (a) * (a))

#ifdef __cplusplus
#define EXPORT_C_FUNC   extern "C" __attribute__((visibility("default")))
#define EXPORT_CXX_FUNC __attribute__((visibility("default")))
#else
#define EXPORT_C_FUNC   __attribute__((visibility("default")))
#endif

#define FMT_32D "%" PRId32
#define FMT_32U "%" PRIu32
#define FMT_32X "%" PRIx32
#define FMT_64D "%" PRId64
#define FMT_64U "%" PRIu64
#define FMT_64X "%" PRIx64
typedef pid_t TID;
typedef pid_t PID;
#define FMT_TID FMT_32D
#define FMT_PID FMT_32D

inline TID GetThreadId() {
    static thread_local const TID tid = (TID)syscall(SYS_gettid);
    return tid;
}
inline PID GetProcessId() { return getpid(); }   // not cached: must stay right after fork()
