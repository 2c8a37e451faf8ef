// Stand-in for the reference's un-vendored `ipc` dependency (3rdparty/ipc is an empty submodule;
// its version is not pinned by the reference tree).  TEST INFRASTRUCTURE: this header exists only
// so that the reference's own scheduler sources compile into oracle/_ref/.
//
// It provides the whole surface those sources use — ipc::ChannelKey, ipc::NodeType,
// ipc::Node{Send, Receive, Remove}, ipc::Channel::Remove (call sites:
// sched/src/scheduler/global.cpp:19-31,51,60-65 and service/server/src/server.cpp:49-51,98-103,
// 130-131,173,200) — over abstract-namespace Unix datagram sockets named "\0xsched.ipc.<key>".
// Delivery order / capacity semantics of the real library are unknown ("parity unpinned" at this
// boundary); datagram sockets give in-order, message-preserving, blocking delivery on one host.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>
#include <atomic>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace ipc {

using ChannelKey = uint64_t;
enum class NodeType { kSender, kReceiver };

class Message {
public:
    explicit Message(std::vector<char> &&d) : data_(std::move(d)) {}
    const void *Data() const { return data_.data(); }
    size_t Size() const { return data_.size(); }
private:
    std::vector<char> data_;
};

inline socklen_t MakeAddr(ChannelKey key, sockaddr_un &addr) {
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    int n = std::snprintf(addr.sun_path + 1, sizeof(addr.sun_path) - 1, "xsched.ipc.%llu", (unsigned long long)key);
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

class Node {
public:
    Node(ChannelKey key, NodeType type) : key_(key), type_(type) {
        fd_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
        if (fd_ < 0) return;
        sockaddr_un addr;
        socklen_t len = MakeAddr(key, addr);
        if (type == NodeType::kReceiver) {
            int sz = 4 << 20;
            ::setsockopt(fd_, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
            if (::bind(fd_, (sockaddr *)&addr, len) != 0) { ::close(fd_); fd_ = -1; }
        }
    }
    ~Node() { if (fd_ >= 0) ::close(fd_); }

    bool Send(const void *data, size_t size) {
        if (fd_ < 0 || closed_.load()) return false;
        sockaddr_un addr;
        socklen_t len = MakeAddr(key_, addr);
        ssize_t n = ::sendto(fd_, data, size, 0, (sockaddr *)&addr, len);
        return n == (ssize_t)size;
    }

    std::shared_ptr<Message> Receive() {
        if (fd_ < 0 || closed_.load()) return nullptr;
        std::vector<char> buf(65536);
        ssize_t n = ::recv(fd_, buf.data(), buf.size(), 0);
        if (n <= 0 || closed_.load()) return nullptr;
        buf.resize((size_t)n);
        return std::make_shared<Message>(std::move(buf));
    }

    // Closes the node; a Receive() blocked on a receiver node returns nullptr.
    void Remove() {
        if (closed_.exchange(true)) return;
        if (fd_ >= 0 && type_ == NodeType::kReceiver) {
            int s = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
            if (s >= 0) {
                sockaddr_un addr;
                socklen_t len = MakeAddr(key_, addr);
                char z = 0;
                ::sendto(s, &z, 0, 0, (sockaddr *)&addr, len);
                ::close(s);
            }
        }
    }

private:
    ChannelKey key_;
    NodeType type_;
    int fd_ = -1;
    std::atomic<bool> closed_{false};
};

struct Channel {
    static void Remove(ChannelKey) {}
};

} // namespace ipc
