// HwCommands of the CUDA backend.  Completion of a command is observed through a per-queue counter in
// mapped pinned host memory that the GPU front-end bumps with a 64-bit stream memory write placed
// right behind the command: waiting for a command is a load loop on a host word, not a driver call.
// (The reference waits with cuEventSynchronize on pooled blocking events:
// platforms/cuda/hal/src/common/cuda_command.cpp:39-52, event_pool.cpp:5-43.)
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>
#include <cuda.h>
#include "xsched/preempt/hal/hw_command.h"

namespace xsched::cuda {

class CudaQueue;

/// Shared between a queue and its commands: the counter the GPU writes and the ticket dispenser.
struct CompletionCounter {
    volatile uint64_t *host = nullptr;     // mapped pinned host word
    CUdeviceptr dev = 0;                   // its device address
    std::atomic<uint64_t> next_ticket{0};
    std::mutex issue_mu;                   // ticket order must equal stream order of the writes
    CUstream stream = nullptr;             // the queue's stream and context: asked for errors during long waits
    CUcontext ctx = nullptr;
    /// Take the next ticket and enqueue its write on `stream`; returns the ticket (0 on failure).
    uint64_t Issue(CUstream stream, CUresult *res);
    /// Wait until *host >= ticket.  Spin briefly, then back off.  When the caller knows that the work
    /// behind the ticket still needs about `expected_remaining_us` (a task that was timed on its previous
    /// run), half of that is slept away first, so that a loop of millisecond kernels does not keep a core
    /// busy; 0 = unknown, no sleep.  A wait that lasts asks the driver about the stream every few
    /// milliseconds: a context that has taken an error never executes the write, and neither does a stream
    /// that went idle without it; both end the process with the driver's error, which is what a failed
    /// cuEventSynchronize does in the reference (platforms/cuda/hal/src/common/cuda_command.cpp:39-44 under
    /// CUDA_ASSERT).
    void Wait(uint64_t ticket, int64_t expected_remaining_us = 0) const;
    /// CUDA_SUCCESS / CUDA_ERROR_NOT_READY, or the error the stream's context is in.
    CUresult QueryStream() const;
    /// The counter as the GPU last wrote it.
    uint64_t Load() const { return __atomic_load_n(const_cast<const uint64_t *>(host), __ATOMIC_ACQUIRE); }
};

class CudaCommand : public preempt::HwCommand {
public:
    explicit CudaCommand(preempt::XCommandProperties props) : HwCommand(props) {}
    ~CudaCommand() override = default;

    void Synchronize() override;
    bool Synchronizable() override { return want_sync_.load(std::memory_order_acquire); }
    bool EnableSynchronization() override { want_sync_.store(true, std::memory_order_release); return true; }

    /// Enqueue the work on `stream`, then (if waitable) the counter write that marks its completion.
    CUresult LaunchOn(CUstream stream, const std::shared_ptr<CompletionCounter> &counter);
    /// One line for the log when the driver refuses the command.
    virtual std::string Describe() const { return "command"; }
    /// Ticket of the completion write behind the latest launch of this command (0 = none).
    uint64_t Ticket() const { return ticket_.load(std::memory_order_acquire); }
    /// Microseconds the work of this command is still expected to take; 0 = unknown.
    virtual int64_t ExpectedRemainingUs() const { return 0; }
    /// Called after a wait on this command returned.
    virtual void OnWaited() {}

protected:
    virtual CUresult Enqueue(CUstream stream) = 0;

private:
    std::atomic<bool> want_sync_{false};       // set by the window worker, read by waiting application threads
    std::shared_ptr<CompletionCounter> counter_;
    std::atomic<uint64_t> ticket_{0};      // 0 = not issued yet
};

/// cuLaunchKernel with a private copy of the argument block (the caller's argument array is only
/// valid during the call that was intercepted).  Not deactivatable: an arbitrary kernel cannot be
/// stopped cooperatively.
/// When the driver cannot describe the kernel's parameters the command borrows the caller's argument
/// array instead and is marked "blocking submit": XQueue::Submit returns only after the launch, so the
/// array is still valid when it is read, the stream's XQueue does not have to drain, and the scheduler
/// keeps seeing the work.
class CudaKernelLaunchCommand final : public CudaCommand {
public:
    CudaKernelLaunchCommand(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                            unsigned shmem, void **params, void **extra);
    /// cuLaunchKernelEx form: the launch attributes (cluster shape, priority, ...) are copied as well.
    CudaKernelLaunchCommand(const CUlaunchConfig *config, CUfunction f, void **params, void **extra);
    /// False when the arguments are borrowed from the caller (blocking submit).
    bool ParamsCopied() const { return !borrowed_; }
    std::string Describe() const override;
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CUfunction f_;
    unsigned g_[3], b_[3], shmem_;
    std::vector<unsigned char> arg_bytes_;
    std::vector<void *> arg_ptrs_;
    std::vector<unsigned char> extra_bytes_;
    void *extra_[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    bool use_extra_ = false;
    bool borrowed_ = false;
    void **caller_params_ = nullptr, **caller_extra_ = nullptr;
    bool use_ex_ = false;
    std::vector<CUlaunchAttribute> attrs_;
    void CopyArgs(void **params, void **extra);
};

enum class CopyKind { kHtoD, kDtoH, kDtoD, kGeneric };
/// True when the driver does not know `p`: ordinary (pageable) host memory.
bool IsPageableHost(const void *p);

/// An asynchronous copy.  With `stage_source` the source bytes are captured at construction: a copy
/// from pageable host memory returns to its caller only after the source was read, so the caller may
/// reuse the buffer at once, long before a queued command reaches the driver (the reference stages
/// such sources into pinned memory, platforms/cuda/hal/include/xsched/cuda/hal/common/cuda_command.h:175-199).
class CudaMemcpyCommand final : public CudaCommand {
public:
    CudaMemcpyCommand(CopyKind kind, CUdeviceptr dst, CUdeviceptr src, size_t bytes, bool stage_source = false);
    std::string Describe() const override;
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CopyKind kind_;
    CUdeviceptr dst_, src_;
    size_t bytes_;
    std::vector<unsigned char> staged_;
};

class CudaMemsetCommand final : public CudaCommand {
public:
    CudaMemsetCommand(CUdeviceptr dst, unsigned value, size_t count, int width)
        : CudaCommand(preempt::kCommandPropertyNone), dst_(dst), value_(value), count_(count), width_(width) {}
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CUdeviceptr dst_;
    unsigned value_;
    size_t count_;
    int width_;
};

/// Any other stream-ordered driver call (graph launch and upload, 2D/3D/peer copies, the remaining
/// memsets, stream-ordered allocation, cooperative launches, stream callbacks), kept as a closure over
/// its copied arguments.  Calls whose arguments are only valid during the intercepted call, or whose
/// result the caller reads on return, are created with the blocking-submit property.  (The reference has
/// one generated command class per entry point, platforms/cuda/hal/include/xsched/cuda/hal/common/cuda_command.h:121-233.)
class CudaCallCommand final : public CudaCommand {
public:
    CudaCallCommand(const char *what, std::function<CUresult(CUstream)> call, preempt::XCommandProperties props = preempt::kCommandPropertyNone)
        : CudaCommand(props), what_(what), call_(std::move(call)) {}
    std::string Describe() const override { return what_; }
protected:
    CUresult Enqueue(CUstream stream) override { return call_(stream); }
private:
    const char *what_;
    std::function<CUresult(CUstream)> call_;
};

/// cuEventRecord[WithFlags]: re-executable, always individually waitable.
class CudaEventRecordCommand final : public CudaCommand {
public:
    explicit CudaEventRecordCommand(CUevent ev, unsigned flags = 0, bool with_flags = false)
        : CudaCommand(preempt::kCommandPropertyIdempotent), ev_(ev), flags_(flags), with_flags_(with_flags) { EnableSynchronization(); }
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CUevent ev_;
    unsigned flags_;
    bool with_flags_;
};

/// cuStreamWaitEvent: before it is launched, the command that records the event must have been
/// launched (it may sit in another XQueue's pending list).
class CudaEventWaitCommand final : public CudaCommand {
public:
    CudaEventWaitCommand(CUevent ev, unsigned flags, std::shared_ptr<preempt::HwCommand> record_cmd)
        : CudaCommand(preempt::kCommandPropertyIdempotent), ev_(ev), flags_(flags), record_(std::move(record_cmd)) {}
    void BeforeLaunch() override;
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CUevent ev_;
    unsigned flags_;
    std::shared_ptr<preempt::HwCommand> record_;
};

class CudaHostFuncCommand final : public CudaCommand {
public:
    CudaHostFuncCommand(CUhostFn fn, void *data) : CudaCommand(preempt::kCommandPropertyNone), fn_(fn), data_(data) {}
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    CUhostFn fn_;
    void *data_;
};

/// A task of the preemptible-kernel library: the deactivatable command of this backend.
class CudaXpkCommand final : public CudaCommand {
public:
    CudaXpkCommand(void *task, bool rewind) : CudaCommand(preempt::kCommandPropertyDeactivatable), task_(task), rewind_(rewind) {}
    /// Completed on the device (valid once the stream has drained).
    bool TaskCompleted() const;
    void *Task() const { return task_; }
    /// From the duration the same task showed the last time a wait for it returned.
    int64_t ExpectedRemainingUs() const override;
    void OnWaited() override;
protected:
    CUresult Enqueue(CUstream stream) override;
private:
    void *task_;
    bool rewind_;
    bool launched_once_ = false;
    std::atomic<int64_t> launched_at_ns_{0};    // written at every (re)launch, read by waiters
};

} // namespace xsched::cuda
