// A host-side wait with a limit.  `poll()` returns 0 while the awaited work is still running, 1 when it
// has finished and a negative value when it failed; the wait ends with MASCOT_OK, with the negative value
// or - when `timeout_ms` have passed - with MASCOT_ERR_TIMEOUT.  Nothing here blocks inside a driver call,
// so a peer that never shows up costs the caller the limit, not the process.  Header-only and free of
// CUDA, so that a host-only test can exercise it.
#pragma once
#include <chrono>
#include <thread>

namespace mascot {

constexpr int kWaitTimedOut = -6;      // the value of MASCOT_ERR_TIMEOUT (include/mascot.h)

template <class Poll>
int bounded_wait(Poll poll, unsigned timeout_ms, unsigned sleep_us = 50) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        const int s = poll();
        if (s > 0) return 0;
        if (s < 0) return s;
        if (std::chrono::steady_clock::now() >= deadline) return kWaitTimedOut;
        if (sleep_us) std::this_thread::sleep_for(std::chrono::microseconds(sleep_us));
    }
}

}  // namespace mascot
