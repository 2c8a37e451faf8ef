// Name <-> enumerator tables for schedulers and policies, and XDevice packing
// (reference: protocol/src/names.cpp, protocol/src/device.cpp:6-19).
#pragma once
#include <string>
#include "xsched/types.h"
#include "xsched/protocol/def.h"

namespace xsched::protocol {

inline XDeviceId GetDeviceId(XDevice dev) { return (XDeviceId)(dev & 0xFFFFFFFFull); }
inline XDeviceType GetDeviceType(XDevice dev) { return (XDeviceType)(dev >> 32); }
inline XDevice MakeDevice(XDeviceType type, XDeviceId id) { return ((uint64_t)type << 32) | (uint64_t)id; }
/// PCI address as the reference packs it (utils/include/xsched/utils/pci.h:5-8).
inline uint32_t MakePciId(uint32_t domain, uint32_t bus, uint32_t device, uint32_t function) {
    return (domain << 16) | (bus << 8) | (device << 3) | function;
}

XSchedulerType GetSchedulerType(const std::string &name);   // kSchedulerUnknown if not a known name
XPolicyType GetPolicyType(const std::string &name);         // kPolicyUnknown if not a known name
const char *GetSchedulerTypeName(XSchedulerType t);
const char *GetPolicyTypeName(XPolicyType t);
const char *GetPreemptLevelName(XPreemptLevel l);

} // namespace xsched::protocol
