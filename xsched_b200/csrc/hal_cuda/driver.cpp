#include "hal_cuda/driver.h"

#include <dlfcn.h>
#include <limits.h>
#include <mutex>
#include <stdlib.h>
#include <sys/stat.h>
#include <vector>
#include "xsched/protocol/def.h"
#include "xsched/utils/xassert.h"

namespace xsched::cuda {

namespace {

// Marker exported by the interposer (libshimcuda.so); a candidate that has it is not the real driver.
constexpr const char *kShimMarker = "XSchedShimMarker";

bool IsRegularFile(const std::string &p) {
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

std::string SelfDirectory() {
    Dl_info info;
    if (dladdr((void *)&SelfDirectory, &info) == 0 || !info.dli_fname) return "";
    char buf[PATH_MAX];
    if (!realpath(info.dli_fname, buf)) return "";
    std::string s(buf);
    const size_t k = s.rfind('/');
    return k == std::string::npos ? "" : s.substr(0, k);
}

} // namespace

std::string FindRealDriver() {
    const std::string env = GetEnv(XSCHED_CUDA_LIB_ENV_NAME);
    if (!env.empty()) return IsRegularFile(env) ? env : "";
    const std::string self_dir = SelfDirectory();
    static const char *kDirs[] = {
        "/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/lib", "/lib/x86_64-linux-gnu", "/usr/lib/aarch64-linux-gnu",
        "/usr/local/nvidia/lib64", "/usr/local/nvidia/lib", "/usr/lib/wsl/lib", "/usr/local/cuda/compat", "/usr/lib/x86_64-linux-gnu/nvidia/current",
    };
    for (const char *d : kDirs) {
        for (const char *name : {"libcuda.so.1", "libcuda.so"}) {
            const std::string p = std::string(d) + "/" + name;
            if (!IsRegularFile(p)) continue;
            char real[PATH_MAX];
            if (!realpath(p.c_str(), real)) continue;
            const std::string rp(real);
            if (!self_dir.empty() && rp.compare(0, self_dir.size(), self_dir) == 0) continue;   // our own tree
            return rp;
        }
    }
    return "";
}

void *DriverApi::Sym(const char *name) const { return handle ? dlsym(handle, name) : nullptr; }

const DriverApi &Driver() {
    static DriverApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        std::string path = FindRealDriver();
        // Last resort: let the dynamic loader search by name (finds the driver in non-standard
        // locations listed in ld.so.conf / LD_LIBRARY_PATH; the marker check below rejects the shim).
        if (path.empty()) path = "libcuda.so.1";
        // RTLD_DEEPBIND: the driver's own cross-calls must bind to itself, not to the interposer's exports of
        // the same names.  Sanitizer runtimes refuse that flag; sanitizer builds define XSCHED_NO_DEEPBIND.
#ifdef XSCHED_NO_DEEPBIND
        const int deep = 0;
#else
        const int deep = RTLD_DEEPBIND;
#endif
        void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL | deep);
        if (!h) XERRO("cannot open the CUDA driver (%s): %s; set %s to the path of the real libcuda.so.1", path.c_str(), dlerror(), XSCHED_CUDA_LIB_ENV_NAME);
        if (dlsym(h, kShimMarker)) XERRO("%s is the XSched interposer, not the CUDA driver; set %s", path.c_str(), XSCHED_CUDA_LIB_ENV_NAME);
        api.handle = h;
        api.path = path;
        auto need = [&](const char *versioned, const char *plain) -> void * {
            void *p = dlsym(h, versioned);
            if (!p && plain) p = dlsym(h, plain);
            if (!p) XERRO("CUDA driver %s lacks %s", path.c_str(), versioned);
            return p;
        };
#define LOAD(name) api.name = (decltype(api.name))need(#name, nullptr);
#define LOAD_V(name, sym) api.name = (decltype(api.name))need(sym, #name);
        LOAD(cuInit) LOAD(cuGetErrorString) LOAD(cuCtxGetCurrent) LOAD(cuCtxSetCurrent) LOAD_V(cuCtxPushCurrent, "cuCtxPushCurrent_v2") LOAD_V(cuCtxPopCurrent, "cuCtxPopCurrent_v2") LOAD(cuCtxGetDevice)
        LOAD(cuCtxGetStreamPriorityRange) LOAD(cuCtxSynchronize) LOAD(cuDeviceGetAttribute) LOAD(cuStreamGetCtx)
        LOAD(cuStreamGetFlags) LOAD(cuStreamSynchronize) LOAD(cuStreamQuery) LOAD(cuStreamCreateWithPriority)
        LOAD_V(cuStreamDestroy, "cuStreamDestroy_v2") LOAD(cuStreamWaitEvent)
        LOAD_V(cuStreamWriteValue32, "cuStreamWriteValue32_v2") LOAD_V(cuStreamWriteValue64, "cuStreamWriteValue64_v2")
        LOAD_V(cuMemHostAlloc, "cuMemHostAlloc") LOAD_V(cuMemHostGetDevicePointer, "cuMemHostGetDevicePointer_v2")
        LOAD(cuMemFreeHost) LOAD_V(cuMemAlloc, "cuMemAlloc_v2") LOAD_V(cuMemFree, "cuMemFree_v2")
        LOAD_V(cuMemsetD32, "cuMemsetD32_v2") LOAD(cuMemsetD8Async) LOAD(cuMemsetD32Async) LOAD(cuMemcpyAsync)
        LOAD_V(cuMemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2") LOAD_V(cuMemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2")
        LOAD_V(cuMemcpyDtoDAsync, "cuMemcpyDtoDAsync_v2") LOAD(cuLaunchKernel) LOAD(cuLaunchKernelEx) LOAD(cuLaunchHostFunc)
        LOAD(cuFuncGetParamInfo) LOAD(cuPointerGetAttribute) LOAD(cuEventCreate) LOAD_V(cuEventDestroy, "cuEventDestroy_v2") LOAD(cuEventRecord)
        LOAD(cuEventQuery) LOAD(cuEventSynchronize) LOAD_V(cuGetProcAddress, "cuGetProcAddress_v2")
#undef LOAD
#undef LOAD_V
    });
    return api;
}

const char *ErrorString(CUresult r) {
    const char *s = nullptr;
    if (Driver().cuGetErrorString(r, &s) != CUDA_SUCCESS || !s) return "unknown";
    return s;
}

} // namespace xsched::cuda
