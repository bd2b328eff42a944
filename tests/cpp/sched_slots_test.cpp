// Host-only test of the work-item counter slot policy (csrc/sched_slots.h): compiled and run by
// tests/test_cpu_sched_slots.py.  Exit code 0 = every check passed.
#include "sched_slots.h"

#include <atomic>
#include <cstdio>
#include <set>
#include <thread>
#include <vector>

using ttk::SlotRing;

static int failures = 0;
#define CHECK(cond)                                                         \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED line %d: %s\n", __LINE__, #cond);           \
            ++failures;                                                     \
        }                                                                   \
    } while (0)

int main() {
    {   // round robin; a slot nobody used before never needs a wait
        SlotRing ring(4);
        bool w = true;
        for (int i = 0; i < 4; ++i) {
            const int s = ring.acquire([](int) { return true; }, &w);
            CHECK(s == i && !w);
            ring.release(s);
        }
        // second lap: every slot has a previous user; the caller's "still running" test decides
        for (int i = 0; i < 4; ++i) {
            const int s = ring.acquire([](int slot) { return slot == 2; }, &w);
            CHECK(s == i && w == (i == 2));
            ring.release(s);
        }
    }
    {   // one long launch + more short launches than slots: the long launch's slot comes round again and
        // is flagged, so the short launch that gets it is ordered behind the long one instead of sharing
        SlotRing ring(8);
        bool w = false;
        const int long_slot = ring.acquire([](int) { return false; }, &w);
        ring.release(long_slot);          // its event is recorded; the kernel is still running
        int flagged = 0, shared_unflagged = 0;
        for (int i = 0; i < 100; ++i) {
            const int s = ring.acquire([&](int slot) { return slot == long_slot; }, &w);
            if (s == long_slot) (w ? flagged : shared_unflagged)++;
            ring.release(s);
        }
        CHECK(flagged >= 12 && shared_unflagged == 0);
    }
    {   // a slot held by another host thread (between acquire and release) is skipped
        SlotRing ring(3);
        bool w = false;
        const int a = ring.acquire([](int) { return false; }, &w);
        const int b = ring.acquire([](int) { return false; }, &w);
        CHECK(a == 0 && b == 1);
        const int c = ring.acquire([](int) { return false; }, &w);
        CHECK(c == 2);
        ring.release(b);
        const int d = ring.acquire([](int) { return false; }, &w);   // 0 and 2 are held: only 1 is free
        CHECK(d == 1);
        ring.release(a); ring.release(c); ring.release(d);
    }
    {   // many threads: two holders never own one slot at the same time; a thread that finds every slot
        // held waits for a release instead of failing
        SlotRing ring(4);
        std::atomic<int> owners[4];
        for (auto& o : owners) o = 0;
        std::atomic<int> clashes{0};
        std::vector<std::thread> th;
        for (int t = 0; t < 8; ++t)
            th.emplace_back([&] {
                for (int i = 0; i < 2000; ++i) {
                    bool w;
                    const int s = ring.acquire([](int) { return false; }, &w);
                    if (owners[s].fetch_add(1) != 0) ++clashes;
                    owners[s].fetch_sub(1);
                    ring.release(s);
                }
            });
        for (auto& x : th) x.join();
        CHECK(clashes.load() == 0);
    }
    if (failures == 0) std::printf("ok\n");
    return failures == 0 ? 0 : 1;
}
