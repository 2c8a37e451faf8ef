// Environment-variable getters (names as in the reference's utils/include/xsched/utils/env.h).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <string>
#include <strings.h>

inline std::string GetEnv(const std::string &name) {
    const char *v = std::getenv(name.c_str());
    return v ? std::string(v) : std::string();
}
inline bool GetEnvInt64(const std::string &name, int64_t &val) {
    const char *v = std::getenv(name.c_str());
    if (!v || !*v) return false;
    char *end = nullptr;
    errno = 0;
    long long x = std::strtoll(v, &end, 10);
    if (end == v || errno != 0) return false;
    val = (int64_t)x;
    return true;
}
// "1"/"on" -> true, "0"/"off" -> false (case-insensitive), anything else -> default_val.
inline bool GetEnvOption(const std::string &name, bool default_val = false) {
    const std::string v = GetEnv(name);
    if (v == "1" || strcasecmp(v.c_str(), "on") == 0) return true;
    if (v == "0" || strcasecmp(v.c_str(), "off") == 0) return false;
    return default_val;
}
