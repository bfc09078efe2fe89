// Host-only exercise of csrc/launch_cache.h for the CPU tests: replays a sequence of launches given on
// the command line ("device:block:smem" triples) against fake CUDA calls and prints what the cache asked
// of them.  The largest request of the kernel is the second argument.
#include <cstdio>
#include <cstdlib>

#include "launch_cache.h"

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const size_t smem_max = std::strtoull(argv[1], nullptr, 10);
    const int fail_raise = std::atoi(argv[2]);
    mascot::LaunchCache cache;
    for (int a = 3; a < argc; a++) {
        int dev = 0, block = 0; unsigned long long smem = 0;
        if (std::sscanf(argv[a], "%d:%d:%llu", &dev, &block, &smem) != 3) return 2;
        int fit = -1;
        const int rc = cache.lookup(
            dev, block, (size_t)smem, smem_max,
            [&](size_t bytes) { std::printf("raise dev=%d bytes=%zu\n", dev, bytes); return fail_raise; },
            [&](int blk, size_t sm, int* f) { std::printf("query dev=%d block=%d smem=%zu\n", dev, blk, sm); *f = (int)(200000 / (sm + 1)); return 0; },
            &fit);
        std::printf("launch dev=%d block=%d smem=%llu rc=%d fit=%d\n", dev, block, smem, rc, fit);
    }
    return 0;
}
