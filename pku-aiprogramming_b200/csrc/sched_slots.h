// Slot allocator for the work-item counters of the persistent kernels (pure C++, no CUDA: the
// caller supplies the "is the slot's last user still running" test, so the policy can be tested on a
// machine without a GPU).
//
// A launch holds a slot from acquire() until release(); between the two it clears the slot's counter
// on its stream, launches its kernel and records an event on the slot.  Slots are handed out round
// robin.  A slot that another host thread still holds is skipped.  A slot whose previous launch has
// not finished is still handed out, but flagged: the caller must order its own launch behind that
// launch (stream-wait on the slot's event) before touching the counter.  So two launches that are in
// flight at the same time never read the same counter, however many launches overlap.
#pragma once
#include <mutex>
#include <thread>
#include <vector>

namespace ttk {

class SlotRing {
public:
    explicit SlotRing(int n) : held_(n, false), used_(n, false), next_(0) {}
    int size() const { return (int)held_.size(); }

    // busy(slot) -> true when the launch that last used `slot` may still be running.
    // Returns the slot; *must_wait says whether the caller has to wait for that launch first.
    template <class BusyFn>
    int acquire(BusyFn busy, bool* must_wait) {
        for (;;) {
            {
                std::lock_guard<std::mutex> lk(mu_);
                const int n = size();
                for (int tries = 0; tries < n; ++tries) {
                    const int s = (int)(next_++ % (unsigned)n);
                    if (held_[s]) continue;   // another thread is between acquire and release on it
                    held_[s] = true;
                    *must_wait = used_[s] && busy(s);
                    used_[s] = true;
                    return s;
                }
            }
            std::this_thread::yield();        // every slot is held by a launching thread: wait for one
        }
    }
    void release(int slot) {
        std::lock_guard<std::mutex> lk(mu_);
        held_[slot] = false;
    }

private:
    std::mutex mu_;
    std::vector<bool> held_, used_;
    unsigned next_;
};

}  // namespace ttk
