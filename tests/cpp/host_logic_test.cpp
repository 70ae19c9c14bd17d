// Host-only exercise of the stream layer's decision logic (csrc/driverapi/host_logic.h): the polling wait
// with a deadline against a query that never succeeds, the 64-bit accumulation of event timestamps over a
// chain of epochs, and the record of byte ranges that kernels in flight may write.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "host_logic.h"

#define CHECK(cond)                                                   \
    do {                                                              \
        if (!(cond)) {                                                \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                 \
        }                                                             \
    } while (0)

using namespace lcu;

int main() {
    // ---- polling wait: a query that never succeeds runs into the deadline; the clock is a counter --------
    {
        uint64_t fake_now = 1000, polls = 0;
        auto never = [&] { ++polls; return PollResult::Pending; };
        auto clock = [&] { return fake_now += 7; };  // 7 ms per look at the clock
        CHECK(poll_until(never, clock, 50, false) == WaitOutcome::TimedOut);
        CHECK(polls >= 64 && polls <= 64 * 16);  // the clock is read every 64th poll
        polls = 0;
        auto tenth = [&] { return ++polls == 10 ? PollResult::Done : PollResult::Pending; };
        CHECK(poll_until(tenth, clock, 50, true) == WaitOutcome::Done && polls == 10);
        polls = 0;
        auto fails = [&] { return ++polls == 3 ? PollResult::Failed : PollResult::Pending; };
        CHECK(poll_until(fails, clock, 0, false) == WaitOutcome::Failed && polls == 3);
        polls = 0;
        auto late = [&] { return ++polls == 100000 ? PollResult::Done : PollResult::Pending; };
        CHECK(poll_until(late, clock, 0, false) == WaitOutcome::Done);  // no limit: waits as long as it takes
    }
    // ---- timestamps: 3600 epochs one second apart, then an event 0.1 ms after the last one ----------------
    {
        CHECK(add_elapsed_ns(5, 0.0f) == 5 && add_elapsed_ns(5, -1.0f) == 5);
        CHECK(add_elapsed_ns(1000, 1.5f) == 1000 + 1500000);
        const size_t n = 3601;
        std::vector<uint64_t> base(n, 0);
        size_t resolved = 0, reachable = 1800;  // the GPU has only reached the first half at first
        auto elapsed = [&](size_t a, size_t b, float *ms) {
            if (b > reachable) return false;
            *ms = (float)(1000.0 * (double)(b - a));
            return true;
        };
        CHECK(!resolve_epochs(base, resolved, n - 1, elapsed));
        CHECK(resolved == 1801);
        reachable = n;
        CHECK(resolve_epochs(base, resolved, n - 1, elapsed));
        CHECK(base[n - 1] == 3600ull * 1000000000ull);
        // an event a tenth of a millisecond after the last epoch keeps that tenth ...
        const uint64_t ts = add_elapsed_ns(base[n - 1], 0.1f);
        CHECK(ts == 3600ull * 1000000000ull + 100000ull);
        // ... where a single float distance from the origin cannot: floats step by 0.25 ms at 3 600 000 ms
        const float from_origin = 3600000.1f;
        CHECK((uint64_t)((double)from_origin * 1.0e6) == 3600ull * 1000000000ull);
    }
    // ---- write log -------------------------------------------------------------------------------------------
    {
        WriteLog log;
        char *p = reinterpret_cast<char *>(0x10000);
        CHECK(!log.may_be_written(p, 100));
        log.add(p + 100, 50);
        CHECK(!log.may_be_written(p, 100));         // touches, does not overlap
        CHECK(log.may_be_written(p, 101));
        CHECK(log.may_be_written(p + 149, 1));
        CHECK(!log.may_be_written(p + 150, 1000));
        log.add(p, 0);                               // empty ranges are ignored
        CHECK(!log.may_be_written(p, 1));
        for (int i = 0; i < 40; ++i) log.add(p + 100000 + 64 * i, 8);  // more ranges than it holds: everything suspect
        CHECK(log.may_be_written(p + 900000, 1));
        log.clear();
        CHECK(!log.may_be_written(p + 100, 50));
        for (int i = 0; i < 1000; ++i) log.add(p + 64, 32);  // the same range over and over takes one slot
        for (int i = 0; i < 1000; ++i) log.add(p + 70, 8);   // and so does a part of it
        CHECK(log.may_be_written(p + 95, 1) && !log.may_be_written(p + 96, 1000) && !log.may_be_written(p, 64));
        log.clear();
        log.add_unknown();
        CHECK(log.may_be_written(p, 1));
        log.clear();
        CHECK(!log.may_be_written(p, 1));
    }
    std::printf("host logic ok\n");
    return 0;
}
