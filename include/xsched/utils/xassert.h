// XASSERT: a failed invariant logs and ends the process, as in the reference
// (utils/include/xsched/utils/xassert.h:9-15) — internal errors are not recoverable states.
#pragma once
#include "xsched/utils/log.h"
#define XASSERT(expr, format, ...)                                                \
    do {                                                                          \
        if (UNLIKELY(!static_cast<bool>(expr))) {                                 \
            XERRO("Assertion failed: " format __VA_OPT__(,) __VA_ARGS__);         \
        }                                                                         \
    } while (0)
