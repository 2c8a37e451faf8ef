#pragma once
#include "xsched/utils/common.h"
#include "xsched/utils/env.h"
#include "xsched/utils/log.h"
#include "xsched/utils/xassert.h"
