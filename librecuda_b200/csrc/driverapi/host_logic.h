// Host-side decision logic of the stream layer that needs no CUDA call to be exercised: the polling wait with
// an optional deadline, the accumulation of event timestamps over a chain of epochs, and the record of what
// the kernels still in flight on a lane may be writing.  Pure C++ so that tests/cpp/host_logic_test.cpp can
// drive it on a machine without a GPU, with stubbed query functions.
#pragma once

#include <chrono>
#include <cstddef>
#include <cstdint>
#include <thread>
#include <vector>

namespace lcu {

// ---- polling wait ---------------------------------------------------------------------------------------
enum class PollResult { Done, Pending, Failed };
enum class WaitOutcome { Done, TimedOut, Failed };

// Polls `query` until it reports Done or Failed, or until `limit_ms` milliseconds have passed (0 = no limit,
// which is the reference's behaviour: signalWaitCpu spins without a bound, driverapi/src/cmdqueue.cpp:346-352).
// `now_ms` is the clock (injected so that a test can run it forward); `yield` = give the core away between polls.
template <typename Query, typename Clock>
WaitOutcome poll_until(Query query, Clock now_ms, uint64_t limit_ms, bool yield) {
    const uint64_t start = limit_ms ? now_ms() : 0;
    for (uint64_t spins = 0;; ++spins) {
        const PollResult r = query();
        if (r == PollResult::Done) return WaitOutcome::Done;
        if (r == PollResult::Failed) return WaitOutcome::Failed;
        // the clock is read every 64th poll only: a poll costs well under a microsecond
        if (limit_ms && (spins & 63) == 63 && now_ms() - start >= limit_ms) return WaitOutcome::TimedOut;
        if (yield) std::this_thread::yield();
    }
}

inline uint64_t steady_ms() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// ---- event timestamps ---------------------------------------------------------------------------------------
// CUDA reports the distance between two events as a float in milliseconds (24 significant bits).  Measured
// from one fixed origin that is 60 ns of resolution after a second, 62 us after seventeen minutes, 250 us
// after an hour.  Timestamps are therefore taken against the newest of a chain of epochs, at most a few
// seconds old, and the epochs' own offsets are summed in 64-bit nanoseconds.
inline uint64_t add_elapsed_ns(uint64_t base_ns, float elapsed_ms) {
    if (!(elapsed_ms > 0.0f)) return base_ns;  // also NaN
    return base_ns + (uint64_t)((double)elapsed_ms * 1.0e6 + 0.5);
}

// base_ns[k] = offset of epoch k from epoch 0.  `elapsed(a, b, &ms)` returns false while the distance between
// epochs a and b is not known yet (one of them has not been reached on the GPU).  Resolves as far as `upto`
// and returns false if it could not get there.
template <typename Elapsed>
bool resolve_epochs(std::vector<uint64_t> &base_ns, size_t &resolved, size_t upto, Elapsed elapsed) {
    if (base_ns.empty()) return false;
    if (resolved == 0) {
        base_ns[0] = 0;
        resolved = 1;
    }
    while (resolved <= upto) {
        float ms = 0.f;
        if (!elapsed(resolved - 1, resolved, &ms)) return false;
        base_ns[resolved] = add_elapsed_ns(base_ns[resolved - 1], ms);
        ++resolved;
    }
    return true;
}

// ---- what may still be written on a lane ---------------------------------------------------------------------------
// The library's kernels are launched so that the NEXT kernel's CTAs become resident while the previous one
// drains; a copy whose source nothing in flight writes may start loading at once (LCB_COPY_SRC_STABLE).  This
// log holds the byte ranges written by the library kernels submitted to one CUDA stream since the last
// operation that fully serialises the stream (a copy-engine transfer, a host wait).  It is conservative:
// `unknown` (a user kernel or a collective, whose writes are not tracked) or an overflow makes every query say
// "may be written".
class WriteLog {
public:
    void clear() {
        n_ = 0;
        unknown_ = false;
    }
    void add(const void *p, size_t bytes) {
        if (bytes == 0) return;
        const uintptr_t lo = reinterpret_cast<uintptr_t>(p), hi = lo + bytes;
        for (int i = 0; i < n_; ++i)
            if (lo_[i] <= lo && hi <= hi_[i]) return;  // already covered (the same buffer written again and again)
        if (n_ == kMax) {
            unknown_ = true;
            return;
        }
        lo_[n_] = reinterpret_cast<uintptr_t>(p);
        hi_[n_] = lo_[n_] + bytes;
        ++n_;
    }
    void add_unknown() { unknown_ = true; }
    bool may_be_written(const void *p, size_t bytes) const {
        if (unknown_) return true;
        const uintptr_t lo = reinterpret_cast<uintptr_t>(p), hi = lo + bytes;
        for (int i = 0; i < n_; ++i)
            if (lo < hi_[i] && lo_[i] < hi) return true;
        return false;
    }

private:
    static constexpr int kMax = 16;
    uintptr_t lo_[kMax] = {}, hi_[kMax] = {};
    int n_ = 0;
    bool unknown_ = false;
};

}  // namespace lcu
