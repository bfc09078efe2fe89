// Prints the row layout of the library (csrc/layout.cuh) for the CPU tests: for K = 64 and 128 the
// logical element stored at every physical position, and a few values of the seeded permutation.
#include <cstdio>
#include <cstdlib>
#include <initializer_list>

#include "layout.cuh"

int main(int argc, char** argv) {
    if (argc >= 2 && argv[1][0] == 'p') {            // permutation: n seed
        const unsigned long long n = std::strtoull(argv[2], nullptr, 10), seed = std::strtoull(argv[3], nullptr, 10);
        for (unsigned long long j = 0; j < n; j++) std::printf("%llu\n", (unsigned long long)mascot::permute_index(j, n, seed));
        return 0;
    }
    for (int K : {64, 128}) {
        std::printf("K %d\n", K);
        for (int p = 0; p < K; p++) std::printf("%d %d\n", mascot::logical_of_phys(K, p), mascot::phys_of_logical(K, mascot::logical_of_phys(K, p)));
    }
    return 0;
}
