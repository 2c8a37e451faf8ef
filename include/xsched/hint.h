/* Forwarding header: the whole public C ABI lives in xsched/xsched.h. */
#pragma once
#include "xsched/xsched.h"
