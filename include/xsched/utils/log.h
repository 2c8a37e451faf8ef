// Logging: XDEBG / XINFO / XWARN / XERRO (fatal) with the runtime filter XLOG_LEVEL=ERRO|WARN|INFO|DEBG,
// the same user-facing contract as the reference's utils/include/xsched/utils/log.h:40-126.
// XDEBG compiles to nothing when RELEASE_MODE is defined.
#pragma once
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include "xsched/utils/common.h"
#include "xsched/utils/env.h"

namespace xsched::utils {
enum LogLevel { kLogErro = 0, kLogWarn = 1, kLogInfo = 2, kLogDebg = 3 };
inline int LogLevelFromEnv() {
    const std::string v = GetEnv("XLOG_LEVEL");
    if (v.empty()) return kLogDebg;
    if (v == "ERRO") return kLogErro;
    if (v == "WARN") return kLogWarn;
    if (v == "DEBG") return kLogDebg;
    return kLogInfo;
}
inline int CurrentLogLevel() { static const int lvl = LogLevelFromEnv(); return lvl; }
inline void LogPrefix(const char *tag) {
    using namespace std::chrono;
    const auto now = system_clock::now();
    const time_t tt = system_clock::to_time_t(now);
    std::tm lt{};
    localtime_r(&tt, &lt);
    const long us = (long)(duration_cast<microseconds>(now.time_since_epoch()).count() % 1000000);
    std::fprintf(stderr, "[XSCHED %s @ T " FMT_TID " @ %02d:%02d:%02d.%06ld] ", tag, GetThreadId(), lt.tm_hour, lt.tm_min, lt.tm_sec, us);
}
} // namespace xsched::utils

#define XLOG_AT(level, tag, format, ...)                                          \
    do {                                                                          \
        if ((level) <= ::xsched::utils::CurrentLogLevel()) {                      \
            ::xsched::utils::LogPrefix(tag);                                      \
            std::fprintf(stderr, format " @ %s:%d\n" __VA_OPT__(,) __VA_ARGS__, __FILE__, __LINE__); \
        }                                                                         \
    } while (0)

#ifdef RELEASE_MODE
#define XDEBG(format, ...) do { } while (0)
#else
#define XDEBG(format, ...) XLOG_AT(::xsched::utils::kLogDebg, "DEBG", format __VA_OPT__(,) __VA_ARGS__)
#endif
#define XINFO(format, ...) XLOG_AT(::xsched::utils::kLogInfo, "INFO", format __VA_OPT__(,) __VA_ARGS__)
#define XWARN(format, ...) XLOG_AT(::xsched::utils::kLogWarn, "WARN", format __VA_OPT__(,) __VA_ARGS__)
#define XERRO_NOEXIT(format, ...) XLOG_AT(::xsched::utils::kLogErro, "ERRO", format __VA_OPT__(,) __VA_ARGS__)
#define XERRO(format, ...)                                                        \
    do {                                                                          \
        XLOG_AT(::xsched::utils::kLogErro, "ERRO", format __VA_OPT__(,) __VA_ARGS__); \
        std::fflush(stderr);                                                      \
        std::exit(EXIT_FAILURE);                                                  \
    } while (0)
