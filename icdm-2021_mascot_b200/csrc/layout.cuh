// Factor-row storage layout and the team reduction that goes with it.
//
// The reference gives lane l of a warp the elements l, l+32 [, l+64, l+96] of a row, adds the
// lane's products pairwise and then folds the 32 lane partials with shfl_down 16,8,4,2,1
// (sgd/sgd_kernel.h:42-63, mascot/mascot_sgd_kernel.h:193-210).  Floating-point addition is
// not associative, so a bit-exact engine has to add the same pairs in the same tree - but it need
// not keep the strided 2/4-byte accesses.  Rows are therefore stored PERMUTED so that one 64-bit
// (fp16) or 128-bit (fp32) access per lane fetches exactly the operands of one or two reference
// lanes, and a xor-butterfly over a "team" of K/4 lanes reproduces the reference tree:
//
//   K = 128, team of 32 lanes, lane t holds physical elements 4t..4t+3 =
//            slots 0..3 of reference lane  (t>>1) + 16*(t&1)
//   K =  64, team of 16 lanes, lane t holds physical elements 4t..4t+3 =
//            slots 0,1 of reference lane A = (t>>1) + 8*(t&1)  followed by slots 0,1 of lane A+16
//
// In both cases the lane partial is (fma(a0,b0,a1*b1)) + (fma(a2,b2,a3*b3)) - for K=64 the outer
// add is the reference's shfl_down-16 step - and the remaining tree steps are xor 1, T/2, .., 2.
// Addition is commutative, so after the butterfly every lane holds the reference's lane-0 value.
#pragma once
#include <cstdint>

#ifndef __CUDACC__
#define MASCOT_HD
#else
#define MASCOT_HD __host__ __device__
#endif

namespace mascot {

// physical position of logical element e (0 <= e < K) inside a row
MASCOT_HD inline int phys_of_logical(int K, int e) {
    const int lane = e & 31, slot = e >> 5;
    if (K == 128) return 8 * (lane & 15) + 4 * (lane >> 4) + slot;
    return 8 * (lane & 7) + 4 * ((lane >> 3) & 1) + 2 * ((lane >> 4) & 1) + slot;
}

// logical element stored at physical position p
MASCOT_HD inline int logical_of_phys(int K, int p) {
    const int t = p >> 2, s = p & 3;
    if (K == 128) return (t >> 1) + 16 * (t & 1) + 32 * s;
    return (t >> 1) + 8 * (t & 1) + 16 * (s >> 1) + 32 * (s & 1);
}

// Seeded bijection of [0, n): a 4-round Feistel network over the next even power-of-two domain,
// cycle-walked back into range.  Integer-only, so host and device agree exactly.
MASCOT_HD inline uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
    return x;
}

MASCOT_HD inline uint64_t permute_index(uint64_t j, uint64_t n, uint64_t seed) {
    if (n < 2) return j;
    int bits = 2;
    while ((1ull << bits) < n) bits += 2;
    const int hb = bits >> 1;
    const uint32_t mask = (hb >= 32) ? 0xffffffffU : ((1u << hb) - 1u);
    uint64_t x = j;
    do {
        uint32_t L = (uint32_t)(x >> hb) & mask, R = (uint32_t)x & mask;
        for (int round = 0; round < 4; round++) {
            const uint32_t key = mix32((uint32_t)(seed >> (16 * (round & 1))) + 0x9e3779b9U * (uint32_t)(round + 1) + (uint32_t)(seed >> 32));
            const uint32_t F = mix32(R ^ key) & mask;
            const uint32_t nl = R;
            R = L ^ F;
            L = nl;
        }
        x = ((uint64_t)L << hb) | R;
    } while (x >= n);
    return x;
}

// Bit 31 of a stream id selects the arena a row lives in: 0 binary16, 1 fp32.
constexpr uint32_t kPrecBit = 0x80000000u;
constexpr uint32_t kIdMask = 0x7fffffffu;

}  // namespace mascot
