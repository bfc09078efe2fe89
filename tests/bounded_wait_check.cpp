// Host-only exercise of csrc/bounded_wait.h for the CPU tests: argv[1] = "ready_after_polls",
// argv[2] = timeout in ms, argv[3] = value the poll returns when it fails (0 = never fails).
// Prints the status and the milliseconds the wait took.
#include <chrono>
#include <cstdio>
#include <cstdlib>

#include "bounded_wait.h"

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    const long ready_after = std::atol(argv[1]);
    const unsigned timeout_ms = (unsigned)std::atoi(argv[2]);
    const int fail_with = std::atoi(argv[3]);
    long polls = 0;
    const auto t0 = std::chrono::steady_clock::now();
    const int rc = mascot::bounded_wait([&]() -> int {
        polls++;
        if (fail_with && polls == 3) return fail_with;
        return (ready_after >= 0 && polls > ready_after) ? 1 : 0;
    }, timeout_ms);
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    std::printf("%d %.1f %ld\n", rc, ms, polls);
    return 0;
}
