#include "xsched/protocol/names.h"

#include <strings.h>

namespace xsched::protocol {

namespace {
struct PolicyName { XPolicyType type; const char *name; };
const PolicyName kPolicies[] = {
    {kPolicyHighestPriorityFirst, XSCHED_POLICY_NAME_HPF}, {kPolicyHeterogeneousHighestPriorityFirst, XSCHED_POLICY_NAME_HHPF},
    {kPolicyCPUHighestPriorityFirst, XSCHED_POLICY_NAME_CHPF}, {kPolicyUtilizationPartition, XSCHED_POLICY_NAME_UP},
    {kPolicyProcessUtilizationPartition, XSCHED_POLICY_NAME_PUP}, {kPolicyStrictProcessUtilizationPartition, XSCHED_POLICY_NAME_SPUP},
    {kPolicyKEarliestDeadlineFirst, XSCHED_POLICY_NAME_KEDF}, {kPolicyLaxity, XSCHED_POLICY_NAME_LAX},
    {kPolicyActiveWindowFirst, XSCHED_POLICY_NAME_AWF}, {kPolicyCompletelyFairScheduler, XSCHED_POLICY_NAME_CFS},
    {kPolicyMultiLevelFeedbackQueue, XSCHED_POLICY_NAME_MLFQ},
};
struct SchedName { XSchedulerType type; const char *name; };
const SchedName kSchedulers[] = {
    {kSchedulerAppManaged, XSCHED_SCHEDULER_NAME_APP}, {kSchedulerLocal, XSCHED_SCHEDULER_NAME_LCL}, {kSchedulerGlobal, XSCHED_SCHEDULER_NAME_GLB},
};
} // namespace

XSchedulerType GetSchedulerType(const std::string &name) {
    for (const auto &s : kSchedulers) if (strcasecmp(name.c_str(), s.name) == 0) return s.type;
    return kSchedulerUnknown;
}
XPolicyType GetPolicyType(const std::string &name) {
    for (const auto &p : kPolicies) if (strcasecmp(name.c_str(), p.name) == 0) return p.type;
    return kPolicyUnknown;
}
const char *GetSchedulerTypeName(XSchedulerType t) {
    for (const auto &s : kSchedulers) if (s.type == t) return s.name;
    return XSCHED_UNKNOWN_NAME;
}
const char *GetPolicyTypeName(XPolicyType t) {
    for (const auto &p : kPolicies) if (p.type == t) return p.name;
    return XSCHED_UNKNOWN_NAME;
}
const char *GetPreemptLevelName(XPreemptLevel l) {
    switch (l) {
    case kPreemptLevelBlock: return "Block";
    case kPreemptLevelDeactivate: return "Deactivate";
    case kPreemptLevelInterrupt: return "Interrupt";
    default: return XSCHED_UNKNOWN_NAME;
    }
}

} // namespace xsched::protocol
