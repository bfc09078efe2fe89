/* Host check of two shortcuts the fixed-point trainers' kernels take (csrc/train_kernels.cu: round_away,
 * pow2_rev), restated here with the same integer and float operations:
 *   1. trunc(x + copysign(largest float below 1/2, x)) == roundf(x) for every one of the 2^32 float patterns;
 *   2. for every power of two s with s and 1/s normal, the mirrored exponent 0x7f000000 - bits(s) == 1/s.
 * Prints "ok" and returns 0 when both hold. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static inline float from_bits(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }
static inline uint32_t bits_of(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }

static inline float round_away(float x) {
    const float h = from_bits((bits_of(x) & 0x80000000u) | 0x3effffffu);
    volatile float s = x + h;                     /* one correctly rounded fp32 addition, as __fadd_rn */
    return truncf(s);
}

int main(void) {
    unsigned long long bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (long long i = 0; i < (1ll << 32); i++) {
        const float x = from_bits((uint32_t)i);
        const float a = roundf(x), c = round_away(x);
        if (bits_of(a) != bits_of(c) && !(isnan(a) && isnan(c))) bad++;
    }
    if (bad) { printf("round_away differs from roundf on %llu patterns\n", bad); return 1; }
    for (int e = -126; e <= 126; e++) {
        const float s = ldexpf(1.0f, e);
        const uint32_t b = bits_of(s);
        if (!(b >= 0x00800000u && b < 0x7f000000u && !(b & 0x007fffffu))) { printf("2^%d not taken by the shortcut\n", e); return 1; }
        if (from_bits(0x7f000000u - b) != 1.0f / s) { printf("mirrored exponent wrong for 2^%d\n", e); return 1; }
    }
    /* what the shortcut must leave to the division */
    const uint32_t left[] = {bits_of(ldexpf(1.0f, 127)), 0x7f800000u, 0x00400000u, bits_of(3.0f), 0u};
    for (unsigned j = 0; j < sizeof left / sizeof left[0]; j++) {
        const uint32_t b = left[j];
        if (b >= 0x00800000u && b < 0x7f000000u && !(b & 0x007fffffu)) { printf("pattern %08x must not take the shortcut\n", b); return 1; }
    }
    printf("ok\n");
    return 0;
}
