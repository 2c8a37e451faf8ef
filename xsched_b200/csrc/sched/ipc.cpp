#include "xsched/sched/ipc.h"

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <string>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include "xsched/protocol/def.h"
#include "xsched/utils/env.h"

namespace xsched::sched {

static socklen_t MakeAddr(uint64_t key, sockaddr_un &addr) {
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    const std::string ns = GetEnv(XSCHED_IPC_NAMESPACE_ENV_NAME);
    const int n = std::snprintf(addr.sun_path + 1, sizeof(addr.sun_path) - 1, "%sxsched.ipc.%llu", ns.c_str(), (unsigned long long)key);
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

IpcEndpoint::~IpcEndpoint() {
    if (fd_ >= 0) ::close(fd_);
}

bool IpcEndpoint::OpenSender() {
    fd_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    return fd_ >= 0;
}

bool IpcEndpoint::Bind(uint64_t key) {
    if (!OpenSender()) return false;
    int sz = 4 << 20;
    ::setsockopt(fd_, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
    sockaddr_un addr;
    const socklen_t len = MakeAddr(key, addr);
    if (::bind(fd_, (sockaddr *)&addr, len) != 0) { ::close(fd_); fd_ = -1; return false; }
    key_ = key;
    static_assert(sizeof(sockaddr_un) <= sizeof(self_addr_), "own address does not fit");
    std::memcpy(self_addr_, &addr, sizeof(addr));
    self_addr_len_ = (unsigned)len;
    bound_ = true;
    return true;
}

bool IpcEndpoint::SendTo(uint64_t key, const void *data, size_t size) {
    if (fd_ < 0 || closed_) return false;
    sockaddr_un addr;
    const socklen_t len = MakeAddr(key, addr);
    return ::sendto(fd_, data, size, 0, (sockaddr *)&addr, len) == (ssize_t)size;
}

int IpcEndpoint::TrySendTo(uint64_t key, const void *data, size_t size) {
    if (fd_ < 0 || closed_) return -1;
    sockaddr_un addr;
    const socklen_t len = MakeAddr(key, addr);
    const ssize_t n = ::sendto(fd_, data, size, MSG_DONTWAIT, (sockaddr *)&addr, len);
    if (n == (ssize_t)size) return 1;
    return (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) ? 0 : -1;
}

bool IpcEndpoint::WaitReadable(int timeout_ms) {
    if (fd_ < 0 || closed_) return true;
    pollfd p{fd_, POLLIN, 0};
    return ::poll(&p, 1, timeout_ms) > 0;
}

long IpcEndpoint::Receive(void *buf, size_t cap) {
    if (fd_ < 0) return -1;
    if (closed_) return 0;
    const ssize_t n = ::recv(fd_, buf, cap, 0);
    if (closed_) return 0;
    return n < 0 ? -1 : (long)n;
}

long IpcEndpoint::TryReceive(void *buf, size_t cap) {
    if (fd_ < 0) return -1;
    if (closed_) return 0;
    const ssize_t n = ::recv(fd_, buf, cap, MSG_DONTWAIT);
    if (closed_) return 0;
    if (n < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? -2 : -1;
    return (long)n;
}

long IpcEndpoint::ReceiveAuto(void *buf, size_t cap) {
    static const bool spin = GetEnvOption(XSCHED_IPC_SPIN_ENV_NAME, false);
    if (!spin) return Receive(buf, cap);
    while (true) {
        const long n = TryReceive(buf, cap);
        if (n != -2) return n;
        for (int i = 0; i < 16; ++i) __builtin_ia32_pause();
    }
}

// Async-signal-safe (socket / sendto / close only): the server calls it from its signal handler.
void IpcEndpoint::Close() {
    if (closed_.exchange(true)) return;
    if (fd_ >= 0 && bound_) {
        // wake a blocked Receive with an empty datagram to ourselves
        const int s = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
        if (s >= 0) {
            char z = 0;
            ::sendto(s, &z, 0, 0, (const sockaddr *)self_addr_, (socklen_t)self_addr_len_);
            ::close(s);
        }
    }
}

} // namespace xsched::sched
