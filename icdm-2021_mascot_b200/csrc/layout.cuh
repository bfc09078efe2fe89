// Factor-row storage layout and the worker reduction that goes with it.
//
// The reference gives lane l of a warp the elements l, l+32 [, l+64, l+96] of a row, adds the
// lane's products pairwise and then folds the 32 lane partials with shfl_down 16,8,4,2,1
// (sgd/sgd_kernel.h:42-63, mascot/mascot_sgd_kernel.h:193-210).  Floating-point addition is
// not associative, so a bit-exact engine has to add the same pairs in the same tree - but it need
// not keep the strided 2/4-byte accesses.  Rows are therefore stored PERMUTED so that lane m of a
// "worker" of K/8 lanes owns the eight consecutive physical elements 8m..8m+7 (one 128-bit access
// in binary16, two in fp32), which are the operands of two (k=128) or four (k=64) reference lanes:
//
//   K = 128:  e0..e3 = slots 0..3 of reference lane m,       e4..e7 = slots 0..3 of lane m+16
//   K =  64:  e0,e1 = slots 0,1 of lane m,  e2,e3 = of lane m+16,  e4,e5 = of m+8,  e6,e7 = of m+24
//
// and inside the lane they are stored in the order  e0 e4 e1 e5 e2 e6 e3 e7, i.e. as the four
// binary16 pairs (e0,e4) (e1,e5) (e2,e6) (e3,e7).  With that order two packed multiplies, two
// packed fused multiply-adds and one packed add give (f0+f1, f2+f3) for the pair products
// f_j = fma(e_2j, e'_2j, e_2j+1 * e'_2j+1) without moving a single half between registers; one more
// add finishes the lane partial (f0+f1)+(f2+f3).  For k=128 that last add is the reference's
// shfl_down-16 step, for k=64 the packed add is its 16 step and the last add its 8 step; the
// remaining steps are a xor butterfly over the worker's lanes.  Addition is commutative, so after
// the butterfly every lane holds the reference's lane-0 value.
#pragma once
#include <cstdint>

#ifndef __CUDACC__
#define MASCOT_HD
#else
#define MASCOT_HD __host__ __device__
#endif

namespace mascot {

// position inside a lane's eight elements: e_s is stored at 2*(s&3) + (s>>2)
MASCOT_HD inline int lane_pos_of_elem(int s) { return 2 * (s & 3) + (s >> 2); }
MASCOT_HD inline int lane_elem_of_pos(int q) { return (q >> 1) + 4 * (q & 1); }

// physical position of logical element e (0 <= e < K) inside a row
MASCOT_HD inline int phys_of_logical(int K, int e) {
    const int lane = e & 31, slot = e >> 5;
    int m, s;
    if (K == 128) { m = lane & 15; s = 4 * (lane >> 4) + slot; }
    else { m = lane & 7; s = 4 * ((lane >> 3) & 1) + 2 * ((lane >> 4) & 1) + slot; }
    return 8 * m + lane_pos_of_elem(s);
}

// logical element stored at physical position p
MASCOT_HD inline int logical_of_phys(int K, int p) {
    const int m = p >> 3, s = lane_elem_of_pos(p & 7);
    if (K == 128) return m + 16 * (s >> 2) + 32 * (s & 3);
    return m + 8 * (s >> 2) + 16 * ((s >> 1) & 1) + 32 * (s & 1);
}

// The fp32 arena stores a row as two halves of K/2 floats: lane m's first four values (positions
// 8m..8m+3 of the binary16 order) at floats 4m..4m+3 of the first half, its last four at 4m..4m+3 of the
// second half.  A worker then reads or writes a row with two 128-bit accesses per lane, each of which
// covers a CONTIGUOUS quarter kilobyte across the worker's lanes (whole 32-byte sectors), instead of two
// interleaved accesses that each touch half of every sector.
MASCOT_HD inline int f32_pos_of_phys(int K, int p) { return ((p & 4) ? K / 2 : 0) + 4 * (p >> 3) + (p & 3); }

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

// Bit 31 of a stream id selects the arena a row lives in: 0 binary16, 1 fp32.  Bit 30 marks a user
// row that so many workers update at the same time that only one in 2^shift of its updates is written
// back (see the update kernel; the shift is one number per engine).  The per-row byte tables carry the
// same two flags in bits 0 and 1.
constexpr uint32_t kPrecBit = 0x80000000u;
constexpr uint32_t kHotBit = 0x40000000u;
constexpr uint32_t kIdMask = 0x3fffffffu;
constexpr uint8_t kRowPrec = 1, kRowHot = 2;
MASCOT_HD inline uint32_t row_flags_to_code(uint8_t b) { return ((b & kRowPrec) ? kPrecBit : 0u) | ((b & kRowHot) ? kHotBit : 0u); }

// Where the row of sorted index s lives in an arena.
//   parts <= 1          : row s (a single engine).
//   parts > 1, !snake   : items of a sharded run - `parts` blocks, sorted index s belongs to block
//                         s % parts and is row s / parts of that block, so every block holds the same mix
//                         of popular and rare items and is one contiguous range of rows_per_part rows.
//   parts > 1, snake    : users of a sharded run - dealt to `parts` ranks from the highest degree down,
//                         reversing direction every round, so that the rating counts of the ranks stay
//                         close for heavy-tailed degrees; rank p owns rows [p * rows_per_part, ...).
// The last rows of a part stay unused when n is not a multiple of parts.
struct RowLayout {
    uint32_t parts = 1;
    uint32_t rows_per_part = 0;
    uint32_t n = 0;
    uint32_t snake = 0;
};
MASCOT_HD inline uint32_t layout_rows(const RowLayout& L) { return L.parts <= 1 ? L.n : L.parts * L.rows_per_part; }
MASCOT_HD inline uint32_t arena_row(const RowLayout& L, uint32_t s) {
    if (L.parts <= 1) return s;
    if (!L.snake) return (s % L.parts) * L.rows_per_part + s / L.parts;
    const uint32_t pos = L.n - 1 - s, rnd = pos / L.parts, idx = pos % L.parts;
    return ((rnd & 1) ? L.parts - 1 - idx : idx) * L.rows_per_part + rnd;
}
MASCOT_HD inline uint32_t part_of_row(const RowLayout& L, uint32_t row) { return L.parts <= 1 ? 0 : row / L.rows_per_part; }
// Inverse of arena_row; returns 0xffffffff for an unused (padding) row.
MASCOT_HD inline uint32_t sorted_of_row(const RowLayout& L, uint32_t row) {
    if (L.parts <= 1) return row;
    const uint32_t part = row / L.rows_per_part, within = row % L.rows_per_part;
    if (!L.snake) { const uint64_t s = (uint64_t)within * L.parts + part; return s < L.n ? (uint32_t)s : 0xffffffffu; }
    const uint32_t idx = (within & 1) ? L.parts - 1 - part : part;
    const uint64_t pos = (uint64_t)within * L.parts + idx;
    return pos < L.n ? (uint32_t)(L.n - 1 - pos) : 0xffffffffu;
}

}  // namespace mascot
