/* Host check of the integer shortcut the AFP trainer's kernel takes for ceil((float)log2((double)x))
 * (csrc/train_kernels.cu: ceil_log2_rounded), restated here with the same integer operations and compared
 * with the double-precision formula of the CPU restatement (oracle/mascot_oracle.c) on every positive finite
 * float.  Prints "ok" and returns 0 when they agree everywhere. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static inline float from_bits(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }

/* x = (1 + M / 2^23) * 2^E.  log2(x) = E + log2(1 + M / 2^23) lies in [E, E + 1); rounded to float it is E itself
 * when M = 0, or when the fraction is below half the spacing of the floats next to E on the side of E + 1 - which
 * happens for the first few M only, the more the larger |E| - and otherwise something in (E, E + 1], whose ceiling
 * is E + 1. */
static inline int ceil_log2_rounded(uint32_t bits) {
    int E = (int)(bits >> 23) - 127;
    uint32_t M = bits & 0x7fffffu;
    if ((bits >> 23) == 0) {                       /* denormal: normalise */
        int lz = __builtin_clz(M) - 9;             /* zeros above the leading one inside the 23-bit field */
        E = -126 - (lz + 1);
        M = (M << (lz + 1)) & 0x7fffffu;
    }
    if (M == 0) return E;
    /* largest M whose log2 still rounds down to E: floor(0.34657 * 2^j) with 2^j <= |value next to E| < 2^(j+1) */
    uint32_t a = (uint32_t)(E < 0 ? -E : E);       /* |E| */
    if (E < 0) a -= 1;                             /* the floats between E and E + 1 are smaller in magnitude than |E| */
    if (E <= 0 && a == 0) return E + 1;            /* E = 0 or -1: floats next to it are far finer than any fraction */
    int j = 31 - __builtin_clz(a);                 /* 2^j <= a */
    static const uint32_t limit[8] = {0, 0, 1, 2, 5, 11, 22, 44};
    return M <= limit[j] ? E : E + 1;
}

int main(void) {
    unsigned long long bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (long long i = 1; i < 0x7f800000ll; i++) {
        const float x = from_bits((uint32_t)i);
        const float want = ceilf((float)log2((double)x));
        const int got = ceil_log2_rounded((uint32_t)i);
        if ((float)got != want) {
            if (bad < 5) {
#pragma omp critical
                printf("x=%a bits=%08x want %g got %d\n", x, (unsigned)i, want, got);
            }
            bad++;
        }
    }
    if (bad) { printf("%llu mismatches\n", bad); return 1; }
    printf("ok\n");
    return 0;
}
