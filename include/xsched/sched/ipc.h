// Same-host message channel between scheduling agents and the server: a datagram per record, in order,
// over abstract-namespace Unix sockets named "<namespace>xsched.ipc.<key>" (key 1 = server, otherwise
// the client's pid — the reference's key assignment, protocol/include/xsched/protocol/def.h:35-37).
// The reference uses its un-vendored `ipc` library here, whose transport is not part of its tree.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <vector>

namespace xsched::sched {

class IpcEndpoint {
public:
    IpcEndpoint() = default;
    ~IpcEndpoint();
    IpcEndpoint(const IpcEndpoint &) = delete;
    IpcEndpoint &operator=(const IpcEndpoint &) = delete;

    bool Bind(uint64_t key);                       // become the receiver of `key`
    bool OpenSender();                             // unbound socket for SendTo
    bool SendTo(uint64_t key, const void *data, size_t size);        // may block while the receiver's queue is full
    /// Never blocks: 1 = sent, 0 = the receiver's queue is full right now, -1 = no such receiver / error.
    int TrySendTo(uint64_t key, const void *data, size_t size);
    /// Wait until a record can be received or `timeout_ms` passed (-1 = forever).  False on timeout.
    bool WaitReadable(int timeout_ms);
    /// Blocks.  Returns bytes received, 0 after Close(), -1 on error.
    long Receive(void *buf, size_t cap);
    /// Non-blocking: bytes received, -2 when nothing is queued, 0 after Close(), -1 on error.  A thread
    /// that polls this in a loop sees a record a few microseconds after it was sent, instead of after a
    /// scheduler wake-up; XSCHED_IPC_SPIN=ON selects that mode for the agent's and the server's receivers.
    long TryReceive(void *buf, size_t cap);
    /// Receive with the mode chosen by XSCHED_IPC_SPIN (spinning TryReceive or blocking Receive).
    long ReceiveAuto(void *buf, size_t cap);
    void Close();                                  // wakes a blocked Receive
    bool Ok() const { return fd_ >= 0; }
private:
    int fd_ = -1;
    uint64_t key_ = 0;
    bool bound_ = false;
    std::atomic<bool> closed_{false};
    // Own address, kept from Bind() so that Close() needs no allocation (it may run in a signal handler).
    unsigned char self_addr_[128] = {};
    unsigned self_addr_len_ = 0;
};

} // namespace xsched::sched
