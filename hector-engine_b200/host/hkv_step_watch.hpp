// hkv_step_watch.hpp — host-side failure detection for the multi-GPU decode step. Nothing here
// touches a GPU: a stuck or departed peer must surface as a host-side status, never as a device
// hang, so both pieces are plain C++ and are tested among CPU ranks.
//
//   watch_step   polls "is the step's stream done?" and "does the communicator report an error?"
//                until one answers or a deadline passes (the pattern NCCL documents around
//                ncclCommGetAsyncError); the caller aborts the communicator on anything but Done.
//   NodeRoster   a roster of the ranks of one node in POSIX shared memory: every rank publishes
//                the step it is about to launch and whether it has left. Before a launch each
//                rank checks that all peers are present and not behind, so a rank that left
//                BETWEEN steps is noticed before a collective is enqueued that would wait for it.
//
// The reference engine is single-GPU and has no counterpart (its README lists multi-GPU as absent).
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>

namespace hkv {

enum class WatchResult : int { Done = 0, PeerError = 1, TimedOut = 2 };

inline const char* watch_result_name(WatchResult r) {
    switch (r) {
        case WatchResult::Done: return "done";
        case WatchResult::PeerError: return "communicator reported an asynchronous error";
        case WatchResult::TimedOut: return "timed out waiting for the step (a peer is stuck or gone)";
    }
    return "?";
}

// done():       true once the work enqueued for the step has completed (cudaStreamQuery == success)
// peer_error(): true when the communicator has recorded an asynchronous error
// Both are polled every `poll`; the error check comes first so that a failed collective is not
// mistaken for a slow one. Clock is a template parameter so tests can run on a fake clock.
template <class Done, class PeerError, class Clock = std::chrono::steady_clock>
WatchResult watch_step(Done&& done, PeerError&& peer_error, std::chrono::milliseconds timeout,
                       std::chrono::microseconds poll = std::chrono::microseconds(200)) {
    const auto deadline = Clock::now() + timeout;
    for (;;) {
        if (peer_error()) return WatchResult::PeerError;
        if (done()) return WatchResult::Done;
        if (Clock::now() >= deadline) return WatchResult::TimedOut;
        if (poll.count() > 0) std::this_thread::sleep_for(poll);
    }
}

// ---------------------------------------------------------------------------
// Roster of one node's ranks in shared memory (shm_open + mmap; lock-free 64-bit atomics).
// ---------------------------------------------------------------------------
class NodeRoster {
public:
    static constexpr int kMaxRanks = 64;
    enum class Check : int { Ok = 0, PeerLeft = 1, PeerBehind = 2 };

    // Every rank of the job opens the same `name` (e.g. "/hkv-<job id>"); whoever comes first
    // creates and sizes the segment. `fresh` unlinks a leftover segment of that name first and
    // should be set by exactly one rank (rank 0) before the others open it.
    NodeRoster(const std::string& name, int world, int rank, bool fresh = false)
        : name_(name), world_(world), rank_(rank) {
        if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
            throw std::runtime_error("NodeRoster: rank/world out of range");
        if (fresh) shm_unlink(name.c_str());
        fd_ = shm_open(name.c_str(), O_CREAT | O_RDWR, 0600);
        if (fd_ < 0) throw std::runtime_error("NodeRoster: shm_open failed for " + name);
        if (ftruncate(fd_, sizeof(Segment)) != 0) {
            close(fd_);
            throw std::runtime_error("NodeRoster: ftruncate failed");
        }
        void* p = mmap(nullptr, sizeof(Segment), PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
        if (p == MAP_FAILED) {
            close(fd_);
            throw std::runtime_error("NodeRoster: mmap failed");
        }
        seg_ = static_cast<Segment*>(p);   // a fresh segment is zero-filled: nobody joined, nobody left
        seg_->slot[rank].step.store(0, std::memory_order_relaxed);
        seg_->slot[rank].left.store(0, std::memory_order_relaxed);
        seg_->slot[rank].joined.store(1, std::memory_order_release);
    }
    ~NodeRoster() {
        if (seg_) munmap(seg_, sizeof(Segment));
        if (fd_ >= 0) close(fd_);
    }
    NodeRoster(const NodeRoster&) = delete;
    NodeRoster& operator=(const NodeRoster&) = delete;

    // Removes the name (call once, after every rank is done; mappings stay valid until unmapped).
    void unlink() { shm_unlink(name_.c_str()); }

    int world() const { return world_; }
    int rank() const { return rank_; }
    bool joined(int r) const { return seg_->slot[r].joined.load(std::memory_order_acquire) != 0; }

    // "I am about to launch step `step`" (steps count from 1).
    void announce(uint64_t step) { seg_->slot[rank_].step.store(step, std::memory_order_release); }
    // "I am leaving": call between steps, with none of this rank's kernels or collectives in flight.
    void leave() { seg_->slot[rank_].left.store(1, std::memory_order_release); }
    uint64_t step_of(int r) const { return seg_->slot[r].step.load(std::memory_order_acquire); }
    bool has_left(int r) const { return seg_->slot[r].left.load(std::memory_order_acquire) != 0; }

    // Before launching `step`: has any peer left, or is any peer more than one step behind (it
    // would not join this step's collective in time)? Waits up to `grace` for stragglers to
    // announce `step - 1` at least — ranks run a step apart at most, the collective of step - 1
    // having synchronised them. `who` receives the offending rank.
    Check check_before_launch(uint64_t step, std::chrono::milliseconds grace, int* who = nullptr) const {
        const auto deadline = std::chrono::steady_clock::now() + grace;
        for (;;) {
            int behind = -1;
            for (int r = 0; r < world_; ++r) {
                if (r == rank_) continue;
                if (has_left(r)) {
                    if (who) *who = r;
                    return Check::PeerLeft;
                }
                if (!joined(r) || step_of(r) + 1 < step) behind = r;
            }
            if (behind < 0) return Check::Ok;
            if (std::chrono::steady_clock::now() >= deadline) {
                if (who) *who = behind;
                return Check::PeerBehind;
            }
            std::this_thread::sleep_for(std::chrono::microseconds(100));
        }
    }

private:
    struct Slot {
        std::atomic<uint64_t> step;
        std::atomic<uint32_t> joined;
        std::atomic<uint32_t> left;
        char pad[48];   // one cache line per rank
    };
    struct Segment {
        Slot slot[kMaxRanks];
    };
    static_assert(sizeof(Slot) == 64, "one cache line per rank");
    std::string name_;
    int world_, rank_;
    int fd_ = -1;
    Segment* seg_ = nullptr;
};

}  // namespace hkv
