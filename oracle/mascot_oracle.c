/* CPU oracle for the MASCOT training hot path - TEST INFRASTRUCTURE ONLY (see mascot_oracle.h).
 *
 * Compile with -ffp-contract=off: every fused multiply-add below is written explicitly with
 * fmaf()/fma(), every other operator must round on its own.
 */
#include "mascot_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Contraction pattern of the reference as compiled by nvcc 12.9 -O3 for sm_100 (see
 * mo_rules_reference_build); determined empirically from the golden vectors:
 *   (a0*b0)+(a1*b1)      -> fma(a0, b0, a1*b1)          fp32 and binary16
 *   e*q - lam*p          -> fma(e, q, -(lam*p))          fp32 and binary16
 *   p + lr*t             -> fma(lr, t, p)
 *   a0*b0+a1*b1+a2*b2+.. -> fma(a3,b3, fma(a2,b2, fma(a0,b0, a1*b1)))
 * The sum-of-squares statistic and the fp16-storage trainer are insensitive to the choice within
 * what the golden vectors can resolve; they follow the same pattern. */
#define MO_REF_DOT_F32 1
#define MO_REF_INNER_F32 1
#define MO_REF_OUTER_F32 1
#define MO_REF_CHAIN_F32 1
#define MO_REF_NORM_F32 1
#define MO_REF_DOT_F16 1
#define MO_REF_INNER_F16 1
#define MO_REF_MPT_OUTER 1
/* MuPPET binary16 passes: hmul2(a,b) + hmul2(c,d) -> hfma2(a, b, hmul2(c, d)); the sum of the two
 * halves of ONE hmul2 result stays an unfused add. */
#define MO_REF_MUP_FWD_F16 1
#define MO_REF_MUP_BWD_F16 0
/* AFP moving average: follows the general pattern; the golden vectors cannot tell the variants apart. */
#define MO_REF_AFP_AVG 1

/* ------------------------------------------------------------------------------------------ */
/* contraction rule sets                                                                       */
/* ------------------------------------------------------------------------------------------ */
void mo_rules_literal(mo_rules* r) { memset(r, 0, sizeof(*r)); }

/* The reference built with nvcc 12.9 (-O3, default -fmad=true) for sm_100: found by matching the
 * golden vectors of tests/golden/harness_out.bin. */
void mo_rules_reference_build(mo_rules* r) {
    memset(r, 0, sizeof(*r));
    r->dot_f32 = MO_REF_DOT_F32;
    r->inner_f32 = MO_REF_INNER_F32;
    r->outer_f32 = MO_REF_OUTER_F32;
    r->chain_f32 = MO_REF_CHAIN_F32;
    r->norm_f32 = MO_REF_NORM_F32;
    r->dot_f16 = MO_REF_DOT_F16;
    r->mup_fwd_f16 = MO_REF_MUP_FWD_F16;
    r->mup_bwd_f16 = MO_REF_MUP_BWD_F16;
    r->afp_avg = MO_REF_AFP_AVG;
    r->inner_f16 = MO_REF_INNER_F16;
    r->mpt_outer = MO_REF_MPT_OUTER;
}

/* ------------------------------------------------------------------------------------------ */
/* binary16                                                                                    */
/* ------------------------------------------------------------------------------------------ */
static inline uint64_t d_bits(double d) { uint64_t u; memcpy(&u, &d, 8); return u; }
static inline double bits_d(uint64_t u) { double d; memcpy(&d, &u, 8); return d; }

/* double -> binary16, round to nearest even, done on the bit pattern so that there is exactly
 * one rounding (model_init.cu:51-54 uses __float2half_rn; float -> double is exact). */
static uint16_t d2h(double d) {
    uint64_t b = d_bits(d);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    int64_t exp = (int64_t)((b >> 52) & 0x7ff);
    uint64_t man = b & 0xfffffffffffffull;
    if (exp == 0x7ff) return (uint16_t)(sign | (man ? 0x7fffu : 0x7c00u)); /* CUDA canonical NaN */
    if (exp == 0 && man == 0) return sign;
    int64_t e = exp - 1023;                 /* unbiased; subnormal doubles are far below half range */
    if (exp == 0) return sign;              /* |d| < 2^-1022 -> 0 */
    uint64_t sig = man | (1ull << 52);      /* 53-bit significand, value = sig * 2^(e-52) */
    int shift;                              /* number of low bits to drop */
    int64_t he;                             /* resulting biased half exponent */
    if (e >= -14) { shift = 42; he = e + 15; }          /* normal: keep 11 bits */
    else { shift = (int)(42 + (-14 - e)); he = 0; }     /* subnormal: keep fewer */
    if (shift > 63) return sign;                         /* far too small even for rounding up */
    uint64_t kept = sig >> shift;
    uint64_t rem = sig & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (kept & 1))) kept++;
    uint32_t out;
    if (he == 0) out = (uint32_t)kept;                   /* may carry into the smallest normal: fine */
    else out = (uint32_t)(((uint64_t)(he - 1) << 10) + kept); /* kept has the implicit bit: carries bump exp */
    if (out >= 0x7c00u) out = 0x7c00u;                   /* overflow -> inf */
    return (uint16_t)(sign | out);
}

uint16_t mo_f2h(float f) { return d2h((double)f); }

float mo_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) out = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 0x1f) out = sign | 0x7f800000u | (man << 13);
    else out = sign | ((exp + 112) << 23) | (man << 13);
    float f; memcpy(&f, &out, 4); return f;
}

/* One binary16 operation computed in fp32 and rounded once more is correctly rounded
 * (24 >= 2*11+2), so +,-,* go through float. */
uint16_t mo_hadd(uint16_t a, uint16_t b) { return mo_f2h(mo_h2f(a) + mo_h2f(b)); }
uint16_t mo_hsub(uint16_t a, uint16_t b) { return mo_f2h(mo_h2f(a) - mo_h2f(b)); }
uint16_t mo_hmul(uint16_t a, uint16_t b) { return mo_f2h(mo_h2f(a) * mo_h2f(b)); }

/* Fused multiply-add with a single rounding: the product is exact in double; the sum is formed
 * in double with its rounding error recovered (TwoSum) and folded in as round-to-odd, after which
 * the final rounding to 11 bits is exact. */
uint16_t mo_hfma(uint16_t a, uint16_t b, uint16_t c) {
    double p = (double)mo_h2f(a) * (double)mo_h2f(b);
    double cc = (double)mo_h2f(c);
    double s = p + cc;
    if (isnan(s) || isinf(s)) return d2h(s);
    double bb = s - p;
    double err = (p - (s - bb)) + (cc - bb);
    if (err != 0.0) {
        uint64_t u = d_bits(s);
        if (!(u & 1)) {
            /* move one ulp toward the exact value: that neighbour has an odd significand */
            int toward_larger_magnitude = ((err > 0) == (s > 0));
            if (s == 0.0) return d2h(err);
            u = toward_larger_magnitude ? u + 1 : u - 1;
            s = bits_d(u);
        }
    }
    return d2h(s);
}

static inline uint16_t hneg(uint16_t a) { return (uint16_t)(a ^ 0x8000u); }

/* ------------------------------------------------------------------------------------------ */
/* schedule / control                                                                          */
/* ------------------------------------------------------------------------------------------ */
/* mf_methods.cu:94-97 (identical in every trainer): evaluated in double, stored as float. */
void mo_lr_schedule(float alpha, float decay, int epochs, float* out) {
    for (int i = 0; i < epochs; i++) out[i] = (float)((double)alpha / (1.0 + ((double)decay * pow((double)i, 1.5))));
}

/* Host twin of the engine's seeded factor initialisation (it replaces init_rand_feature_single,
 * model_init.cu:19-28, whose cuRAND states are seeded with clock()).  Element t of stream `sid`:
 * two splitmix64 draws -> u1 in (0,1], u2 in [0,1) -> Box-Muller, with a logarithm and a cosine
 * built from single IEEE-754 operations in a fixed order (this file is compiled with
 * -ffp-contract=off), so that the device reaches the same bits. */
static uint64_t mo_splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}
static double mo_exact_log(double x) {
    uint64_t bits; memcpy(&bits, &x, 8);
    int e = (int)((bits >> 52) & 0x7ff) - 1023;
    uint64_t mb = (bits & 0xfffffffffffffull) | 0x3ff0000000000000ull;
    double m; memcpy(&m, &mb, 8);
    if (m > 1.4142135623730951) { m = m * 0.5; e += 1; }
    const double f = m + -1.0;
    const double s = f / (2.0 + f);
    const double z = s * s;
    static const double c[10] = {1.0 / 19.0, 1.0 / 17.0, 1.0 / 15.0, 1.0 / 13.0, 1.0 / 11.0, 1.0 / 9.0, 1.0 / 7.0, 1.0 / 5.0, 1.0 / 3.0, 1.0};
    double p = 1.0 / 21.0;
    for (int j = 0; j < 10; j++) { const double t = p * z; p = t + c[j]; }
    const double a = (double)e * 0.6931471805599453, b = 2.0 * s;
    return a + b * p;
}
static double mo_exact_cospi(double y) {
    const int q = (int)floor(y * 2.0 + 0.5);
    const double r = y + -((double)q * 0.5);
    const double t = r * 3.141592653589793, t2 = t * t;
    static const double cc[8] = {-1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0, 1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -0.5, 1.0};
    static const double sc[8] = {-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0, -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0, 1.0};
    double c = 1.0 / 20922789888000.0, sn = 1.0 / 355687428096000.0;
    for (int j = 0; j < 8; j++) { const double u = c * t2; c = u + cc[j]; }
    for (int j = 0; j < 8; j++) { const double u = sn * t2; sn = u + sc[j]; }
    sn = sn * t;
    switch (q & 3) { case 0: return c; case 1: return -sn; case 2: return -c; default: return sn; }
}
void mo_init_normal(float* dst, uint64_t count, uint64_t seed, uint64_t sid) {
    const uint64_t base = mo_splitmix64(seed ^ (sid * 0xd1342543de82ef95ull));
    for (uint64_t t = 0; t < count; t++) {
        const uint64_t z = mo_splitmix64(base + t);
        const double u1 = (double)((z >> 11) + 1) * (1.0 / 9007199254740992.0);
        const uint64_t z2 = mo_splitmix64(z);
        const double u2 = (double)(z2 >> 11) * (1.0 / 9007199254740992.0);
        const double l = mo_exact_log(u1);
        const double radius = sqrt(-2.0 * l);
        const double cv = mo_exact_cospi(2.0 * u2);
        const double v = radius * cv;
        dst[t] = (float)(v * 0.01);
    }
}

/* mf_methods.cu:168-175: first check at epoch index 5, then every `interval`, never the last. */
int mo_is_check_epoch(int e, int epochs, int interval) {
    const int start_idx = 5;
    return (e >= start_idx) && (e % interval == (start_idx % interval)) && (epochs - 1 != e);
}

/* preprocess_utils.h:54-99: histogram of training degrees, then sort_by_key ascending.  Ties are
 * kept in ascending id order (a stable sort, which is what the radix sort behind
 * thrust::sort_by_key does for integer keys). */
void mo_degree_sort(const uint32_t* ids, uint64_t n, uint64_t stride_words, uint32_t n_entities,
                    uint32_t* sorted2orig, uint32_t* orig2sorted, uint32_t* cnt_sorted) {
    uint32_t* cnt = (uint32_t*)calloc(n_entities ? n_entities : 1, sizeof(uint32_t));
    uint32_t maxc = 0;
    for (uint64_t j = 0; j < n; j++) cnt[ids[j * stride_words]]++;
    for (uint32_t e = 0; e < n_entities; e++) if (cnt[e] > maxc) maxc = cnt[e];
    uint64_t* start = (uint64_t*)calloc((size_t)maxc + 2, sizeof(uint64_t));
    for (uint32_t e = 0; e < n_entities; e++) start[cnt[e] + 1]++;
    for (uint32_t c = 0; c <= maxc; c++) start[c + 1] += start[c];
    for (uint32_t e = 0; e < n_entities; e++) {
        uint64_t pos = start[cnt[e]]++;
        sorted2orig[pos] = e;
        orig2sorted[e] = (uint32_t)pos;
        cnt_sorted[pos] = cnt[e];
    }
    free(start); free(cnt);
}

/* preprocess_utils.h:101-213: T = ceil(N / requested); walk the distinct degrees upward, summing
 * the number of entities per degree class; close a group at the last entity of a class once the
 * running count reaches T, and always close one at the maximum degree. */
int mo_grouping(const uint32_t* cnt_sorted, uint32_t n_entities, uint32_t requested_groups,
                uint32_t* end_idx, uint32_t* group_of_sorted) {
    uint32_t threshold = (uint32_t)ceilf((float)n_entities / (float)requested_groups);
    uint32_t max_cnt = cnt_sorted[n_entities - 1];
    int groups = 0;
    uint32_t acc = 0;
    uint32_t pos = 0, prev = 0;
    while (pos < n_entities) {
        uint32_t c = cnt_sorted[pos];
        uint32_t last = pos;
        while (last + 1 < n_entities && cnt_sorted[last + 1] == c) last++;
        if (c >= 1) {   /* the reference's walk starts at degree 1 (preprocess_utils.h:139) */
            acc += last - prev + 1;
            if (acc >= threshold) { end_idx[groups++] = last; acc = 0; }
            else if (c == max_cnt) end_idx[groups++] = last;
            prev = last + 1;
        }
        pos = last + 1;
    }
    if (group_of_sorted) {
        uint32_t s = 0;
        for (int g = 0; g < groups; g++) { for (; s <= end_idx[g]; s++) group_of_sorted[s] = (uint32_t)g; }
    }
    return groups;
}

/* mf_methods.cu:325-379: err_g = sum_d (grad_sum[g][d])^2 / sum_parts norm_sum[g][part] / initial. */
void mo_group_errors(const float* grad_sum, const float* norm_sum, int n_norm_parts, int groups, int k,
                     const uint8_t* prec, const float* initial_err, float* err_out) {
    for (int g = 0; g < groups; g++) {
        if (prec[g]) { err_out[g] = -1.0f; continue; }
        float num = 0.f, den = 0.f;
        for (int d = 0; d < k; d++) num += powf(grad_sum[(size_t)g * k + d], 2);
        for (int j = 0; j < n_norm_parts; j++) den += norm_sum[(size_t)g * n_norm_parts + j];
        float e = num / den;
        err_out[g] = e / initial_err[g];
    }
}

/* ------------------------------------------------------------------------------------------ */
/* expression helpers under a contraction rule set                                             */
/* ------------------------------------------------------------------------------------------ */
static inline float pair_f32(float a0, float b0, float a1, float b1, int mode) {
    if (mode == 1) return fmaf(a0, b0, a1 * b1);
    if (mode == 2) return fmaf(a1, b1, a0 * b0);
    return (a0 * b0) + (a1 * b1);
}
static inline float inner_f32(float e, float q, float lam, float p, int mode) {
    if (mode == 1) return fmaf(e, q, -(lam * p));
    if (mode == 2) return fmaf(-lam, p, e * q);
    return (e * q) - (lam * p);
}
static inline float outer_f32(float p, float lr, float t, int mode) {
    if (mode == 1) return fmaf(lr, t, p);
    return p + lr * t;
}
static inline float chain4_f32(const float* a, const float* b, int stride, int n, int mode) {
    /* a0*b0 + a1*b1 + ... left to right */
    float acc;
    if (mode == 1) acc = fmaf(a[0], b[0], a[stride] * b[stride]);
    else if (mode == 2) acc = fmaf(a[stride], b[stride], a[0] * b[0]);
    else acc = a[0] * b[0] + a[stride] * b[stride];
    for (int j = 2; j < n; j++) {
        if (mode) acc = fmaf(a[j * stride], b[j * stride], acc);
        else acc = acc + a[j * stride] * b[j * stride];
    }
    return acc;
}
static inline uint16_t pair_f16(uint16_t a0, uint16_t b0, uint16_t a1, uint16_t b1, int mode) {
    if (mode == 1) return mo_hfma(a0, b0, mo_hmul(a1, b1));
    if (mode == 2) return mo_hfma(a1, b1, mo_hmul(a0, b0));
    return mo_hadd(mo_hmul(a0, b0), mo_hmul(a1, b1));
}
static inline uint16_t inner_f16(uint16_t e, uint16_t q, uint16_t lam, uint16_t p, int mode) {
    if (mode == 1) return mo_hfma(e, q, hneg(mo_hmul(lam, p)));
    if (mode == 2) return mo_hfma(hneg(lam), p, mo_hmul(e, q));
    return mo_hsub(mo_hmul(e, q), mo_hmul(lam, p));
}

/* The warp reduction every kernel uses (e.g. sgd/sgd_kernel.h:57-63): x += shfl_down(x, d) for
 * d = 16,8,4,2,1 on 32 lanes, result taken from lane 0.  Only lane 0's dependency cone matters. */
static float tree32_f32(float* x) {
    for (int d = 16; d >= 1; d >>= 1) for (int l = 0; l < d; l++) x[l] = x[l] + x[l + d];
    return x[0];
}
static uint16_t tree32_f16(uint16_t* x) {
    for (int d = 16; d >= 1; d >>= 1) for (int l = 0; l < d; l++) x[l] = mo_hadd(x[l], x[l + d]);
    return x[0];
}

/* Lane l of the warp owns elements l, l+32[, l+64, l+96] of a row (sgd_kernel.h:42-52). */
static float dot_f32(int k, const float* p, const float* q, int mode) {
    float x[32];
    for (int l = 0; l < 32; l++) {
        if (k == 128) x[l] = pair_f32(p[l], q[l], p[l + 32], q[l + 32], mode) + pair_f32(p[l + 64], q[l + 64], p[l + 96], q[l + 96], mode);
        else x[l] = pair_f32(p[l], q[l], p[l + 32], q[l + 32], mode);
    }
    return tree32_f32(x);
}
static uint16_t dot_f16(int k, const uint16_t* p, const uint16_t* q, int mode) {
    uint16_t x[32];
    for (int l = 0; l < 32; l++) {
        if (k == 128) x[l] = mo_hadd(pair_f16(p[l], q[l], p[l + 32], q[l + 32], mode), pair_f16(p[l + 64], q[l + 64], p[l + 96], q[l + 96], mode));
        else x[l] = pair_f16(p[l], q[l], p[l + 32], q[l + 32], mode);
    }
    return tree32_f16(x);
}
/* sum of squares of a gradient vector, same per-lane grouping and tree (mascot_sgd_kernel.h:244-257) */
static float sumsq_f32(int k, const float* g, int mode) { return dot_f32(k, g, g, mode); }

/* ------------------------------------------------------------------------------------------ */
/* FP32 SGD: sgd/sgd_kernel.h:35-76, sgd_kernel_k64.h:33-64                                    */
/* ------------------------------------------------------------------------------------------ */
static inline void sgd_update(int k, float* p, float* q, float r, float lr, float lam, const mo_rules* ru) {
    float dot = dot_f32(k, p, q, ru->dot_f32);
    float e = r - dot;
    for (int d = 0; d < k; d++) {
        float pv = p[d], qv = q[d];
        p[d] = outer_f32(pv, lr, inner_f32(e, qv, lam, pv, ru->inner_f32), ru->outer_f32);
        q[d] = outer_f32(qv, lr, inner_f32(e, pv, lam, qv, ru->inner_f32), ru->outer_f32);
    }
}

void mo_sgd_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, const mo_rules* rules) {
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        sgd_update(k, P + (size_t)n->u * k, Q + (size_t)n->i * k, n->r, lr, lam, rules);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* MASCOT: mascot/mascot_sgd_kernel.h:188-443 (k=128), mascot_sgd_kernel_k64.h:188-383 (k=64)  */
/* ------------------------------------------------------------------------------------------ */
typedef struct { float* gsum_p; float* gsum_q; float* nsum_p; float* nsum_q; } mascot_stats;

static inline void mascot_update(int k, uint16_t* p16, float* p32, int uprec, uint16_t* q16, float* q32, int iprec,
                                 float r, float lr, float lam, uint16_t lr_h, uint16_t lam_h,
                                 int sampled, float* gs_p, float* gs_q, float* ns_p, float* ns_q, const mo_rules* ru) {
    float gp[128], gq[128];
    if (!uprec && !iprec) {
        /* all binary16: mascot_sgd_kernel.h:188-278 */
        uint16_t r_h = mo_f2h(r);
        uint16_t e = mo_hsub(r_h, dot_f16(k, p16, q16, ru->dot_f16));
        for (int d = 0; d < k; d++) {
            uint16_t pv = p16[d], qv = q16[d];
            uint16_t tp = inner_f16(e, qv, lam_h, pv, ru->inner_f16);
            uint16_t tq = inner_f16(e, pv, lam_h, qv, ru->inner_f16);
            p16[d] = mo_hfma(lr_h, tp, pv);
            q16[d] = mo_hfma(lr_h, tq, qv);
            gp[d] = mo_h2f(tp); gq[d] = mo_h2f(tq);
        }
        if (sampled) {
            *ns_p += sumsq_f32(k, gp, ru->norm_f32);
            *ns_q += sumsq_f32(k, gq, ru->norm_f32);
            for (int d = 0; d < k; d++) { gs_p[d] += gp[d]; gs_q[d] += gq[d]; }
        }
    } else if (!uprec && iprec) {
        /* binary16 user row, fp32 item row: mascot_sgd_kernel.h:279-342 */
        float pf[128];
        for (int d = 0; d < k; d++) pf[d] = mo_h2f(p16[d]);
        float e = r - dot_f32(k, pf, q32, ru->dot_f32);
        for (int d = 0; d < k; d++) {
            float pv = pf[d], qv = q32[d];
            gp[d] = inner_f32(e, qv, lam, pv, ru->inner_f32);
            p16[d] = mo_f2h(fmaf(lr, gp[d], pv));
            q32[d] = fmaf(lr, inner_f32(e, pv, lam, qv, ru->inner_f32), qv);
        }
        if (sampled) {
            *ns_p += sumsq_f32(k, gp, ru->norm_f32);
            for (int d = 0; d < k; d++) gs_p[d] += gp[d];
        }
    } else if (uprec && !iprec) {
        /* fp32 user row, binary16 item row: mascot_sgd_kernel.h:343-407 */
        float qf[128];
        for (int d = 0; d < k; d++) qf[d] = mo_h2f(q16[d]);
        float e = r - dot_f32(k, p32, qf, ru->dot_f32);
        for (int d = 0; d < k; d++) {
            float pv = p32[d], qv = qf[d];
            gq[d] = inner_f32(e, pv, lam, qv, ru->inner_f32);
            p32[d] = fmaf(lr, inner_f32(e, qv, lam, pv, ru->inner_f32), pv);
            q16[d] = mo_f2h(fmaf(lr, gq[d], qv));
        }
        if (sampled) {
            *ns_q += sumsq_f32(k, gq, ru->norm_f32);
            for (int d = 0; d < k; d++) gs_q[d] += gq[d];
        }
    } else {
        /* all fp32 with explicit fmaf: mascot_sgd_kernel.h:408-443; no statistics */
        float e = r - dot_f32(k, p32, q32, ru->dot_f32);
        for (int d = 0; d < k; d++) {
            float pv = p32[d], qv = q32[d];
            p32[d] = fmaf(lr, inner_f32(e, qv, lam, pv, ru->inner_f32), pv);
            q32[d] = fmaf(lr, inner_f32(e, pv, lam, qv, ru->inner_f32), qv);
        }
    }
}

void mo_mascot_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq,
                   uint16_t* P16, float* P32, const uint8_t* uprec_row, const uint32_t* ugroup,
                   uint16_t* Q16, float* Q32, const uint8_t* iprec_row, const uint32_t* igroup,
                   float lr, float lam, uint64_t first_sample_pos,
                   float* gsum_p, float* gsum_q, float* nsum_p, float* nsum_q, int item_stats_by_run,
                   const mo_rules* rules) {
    uint16_t lr_h = mo_f2h(lr), lam_h = mo_f2h(lam);   /* mascot_sgd_kernel.h:79-80 */
    float dummy_vec[128]; float dummy = 0;
    /* item side of a run of equal item groups, when summed per run (see mascot_oracle.h) */
    float run_g[128]; float run_n = 0; int64_t run_group = -1;
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        int sampled = (t >= first_sample_pos) && gsum_p;
        uint32_t gu = ugroup ? ugroup[n->u] : 0, gi = igroup ? igroup[n->i] : 0;
        if (sampled && item_stats_by_run) {
            float gq[128]; float nq = 0;
            memset(gq, 0, sizeof gq);
            mascot_update(k, P16 + (size_t)n->u * k, P32 + (size_t)n->u * k, uprec_row[n->u],
                          Q16 + (size_t)n->i * k, Q32 + (size_t)n->i * k, iprec_row[n->i],
                          n->r, lr, lam, lr_h, lam_h, 1, gsum_p + (size_t)gu * k, gq, nsum_p + gu, &nq, rules);
            if (!iprec_row[n->i]) {
                if ((int64_t)gi != run_group) {
                    if (run_group >= 0) {
                        for (int d = 0; d < k; d++) gsum_q[(size_t)run_group * k + d] += run_g[d];
                        nsum_q[run_group] += run_n;
                    }
                    run_group = gi; run_n = 0; memset(run_g, 0, sizeof run_g);
                }
                for (int d = 0; d < k; d++) run_g[d] += gq[d];
                run_n += nq;
            }
        } else {
            mascot_update(k, P16 + (size_t)n->u * k, P32 + (size_t)n->u * k, uprec_row[n->u],
                          Q16 + (size_t)n->i * k, Q32 + (size_t)n->i * k, iprec_row[n->i],
                          n->r, lr, lam, lr_h, lam_h, sampled,
                          sampled ? gsum_p + (size_t)gu * k : dummy_vec, sampled ? gsum_q + (size_t)gi * k : dummy_vec,
                          sampled ? nsum_p + gu : &dummy, sampled ? nsum_q + gi : &dummy, rules);
        }
    }
    if (run_group >= 0) {
        for (int d = 0; d < k; d++) gsum_q[(size_t)run_group * k + d] += run_g[d];
        nsum_q[run_group] += run_n;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* MPT: mpt/mpt_sgd_kernel.h:15-16, 38-91 (fp32 master weights, binary16 arithmetic, x1000)    */
/* ------------------------------------------------------------------------------------------ */
void mo_mpt_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, const mo_rules* ru) {
    const float scaling = 1000.0f;
    const float rev = 1 / scaling;
    const uint16_t scaling_h = mo_f2h(scaling);
    const uint16_t lam_h = mo_f2h(lam * scaling);      /* mf_methods.cu:764-765 */
    uint16_t ph[128], qh[128];
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        float* p = P + (size_t)n->u * k; float* q = Q + (size_t)n->i * k;
        uint16_t r_h = mo_f2h(n->r);
        for (int d = 0; d < k; d++) { ph[d] = mo_f2h(p[d]); qh[d] = mo_f2h(q[d]); }
        uint16_t e = mo_hmul(scaling_h, mo_hsub(r_h, dot_f16(k, ph, qh, ru->dot_f16)));
        for (int d = 0; d < k; d++) {
            float gp = mo_h2f(inner_f16(e, qh[d], lam_h, ph[d], ru->inner_f16));
            float gq = mo_h2f(inner_f16(e, ph[d], lam_h, qh[d], ru->inner_f16));
            if (ru->mpt_outer) { p[d] = fmaf(lr, rev * gp, p[d]); q[d] = fmaf(lr, rev * gq, q[d]); }
            else { p[d] = p[d] + (lr * (rev * gp)); q[d] = q[d] + (lr * (rev * gq)); }
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* MuPPET (-v 3): muppet/muppet_sgd_kernel.h:7-48 (helpers), 50-292 (k=128), _k64.h:1-212     */
/* ------------------------------------------------------------------------------------------ */
/* get_only_scaling_factor (muppet_sgd_kernel.h:7-19) followed by the assignment to an unsigned
 * index (a negative float becomes 0 on the device) and exp2f of that index. */
static float muppet_scale(int bits, float max_v, float min_v) {
    if (max_v == 0 && min_v == 0) return 1.0f;                 /* index 0 */
    float val = (float)(1 << (bits - 1));
    float top = (val - 1) + 0.5f, bottom = (-val) - 0.5f;
    float range_best = fminf(fabsf(top / max_v), fabsf(bottom / min_v));
    float idx = floorf((float)log2((double)range_best));
    if (!(idx > 0)) return 1.0f;
    if (idx > 4294967295.0f) idx = 4294967295.0f;
    return exp2f(idx);
}
/* Squared norm of both gradients in the grouping of muppet_sgd_kernel.h:267-277 and
 * sgd_kernel.h:266-276: per lane (norm_p + norm_q), then the lane tree. */
static float norm_pq_tree(int k, const float* gp, const float* gq, int mode) {
    float x[32];
    for (int l = 0; l < 32; l++) {
        float np_, nq_;
        if (k == 128) {
            np_ = pair_f32(gp[l], gp[l], gp[l + 32], gp[l + 32], mode) + pair_f32(gp[l + 64], gp[l + 64], gp[l + 96], gp[l + 96], mode);
            nq_ = pair_f32(gq[l], gq[l], gq[l + 32], gq[l + 32], mode) + pair_f32(gq[l + 64], gq[l + 64], gq[l + 96], gq[l + 96], mode);
        } else {
            np_ = pair_f32(gp[l], gp[l], gp[l + 32], gp[l + 32], mode);
            nq_ = pair_f32(gq[l], gq[l], gq[l + 32], gq[l + 32], mode);
        }
        x[l] = np_ + nq_;
    }
    return tree32_f32(x);
}
static inline int sat8(float v) { return v > 127.f ? 127 : (v < -128.f ? -128 : (int)v); }
static inline float fix_round(float v, float s, float s_rev) { return roundf(v * s) * s_rev; }

void mo_muppet_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                   float lr, float lam, int bits_fwd, int bits_bwd, uint64_t first_sample_pos,
                   float* sum_updated_val, float* sum_norms, const mo_rules* ru) {
    const int slots = k / 32;
    float gp[128], gq[128], x[32];
    float norm_total = 0.f;
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        float* p = P + (size_t)n->u * k; float* q = Q + (size_t)n->i * k;
        float pmin = p[0], pmax = p[0], qmin = q[0], qmax = q[0];
        float sp = 1.f, sq = 1.f, pred;
        if (bits_fwd != 32) {
            for (int d = 1; d < k; d++) { pmin = fminf(pmin, p[d]); pmax = fmaxf(pmax, p[d]); qmin = fminf(qmin, q[d]); qmax = fmaxf(qmax, q[d]); }
            sp = muppet_scale(bits_fwd, pmax, pmin); sq = muppet_scale(bits_fwd, qmax, qmin);
        }
        if (bits_fwd == 8) {
            int acc = 0;
            for (int d = 0; d < k; d++) acc += sat8(roundf(p[d] * sp)) * sat8(roundf(q[d] * sq));
            pred = (float)acc / (sp * sq);
        } else if (bits_fwd == 32) {
            pred = dot_f32(k, p, q, ru->dot_f32);
        } else {
            /* binary16 pairs (slot 0, slot 1) and (slot 2, slot 3) of every lane; both halves go
             * through the lane tree separately and are added at the end (muppet_sgd_kernel.h:170-194) */
            const float sp_rev = 1 / sp, sq_rev = 1 / sq;
            uint16_t xs[32], ys[32];
            for (int l = 0; l < 32; l++) {
                uint16_t ph[4], qh[4];
                for (int s = 0; s < slots; s++) {
                    ph[s] = mo_f2h(fix_round(p[l + 32 * s], sp, sp_rev));
                    qh[s] = mo_f2h(fix_round(q[l + 32 * s], sq, sq_rev));
                }
                if (slots == 4) {
                    xs[l] = pair_f16(ph[0], qh[0], ph[2], qh[2], ru->mup_fwd_f16);
                    ys[l] = pair_f16(ph[1], qh[1], ph[3], qh[3], ru->mup_fwd_f16);
                } else {
                    xs[l] = mo_hmul(ph[0], qh[0]); ys[l] = mo_hmul(ph[1], qh[1]);
                }
            }
            pred = mo_h2f(mo_hadd(tree32_f16(xs), tree32_f16(ys)));
        }
        const float ruv = n->r - pred;
        float sb = 1.f;
        if (bits_bwd != 32) {
            /* with a 32-bit forward pass the extrema were never computed on the device; the host
             * policy always runs both passes at the same width, so that case does not occur */
            float bmin = fminf(fminf(pmin, qmin), fminf(-1 * lam, ruv));
            float bmax = fmaxf(fmaxf(pmax, qmax), fmaxf(-1 * lam, ruv));
            sb = muppet_scale(bits_bwd, bmax, bmin);
        }
        if (bits_bwd == 8) {
            const float rev2 = 1 / (sb * sb);
            const int e_i = sat8(roundf(ruv * sb)), l_i = sat8(roundf(-1.0f * lam * sb));
            for (int d = 0; d < k; d++) {
                const int pi = sat8(roundf(p[d] * sb)), qi = sat8(roundf(q[d] * sb));
                gp[d] = (float)(qi * e_i + pi * l_i) * rev2;
                gq[d] = (float)(pi * e_i + qi * l_i) * rev2;
            }
        } else if (bits_bwd == 32) {
            for (int d = 0; d < k; d++) {
                gp[d] = inner_f32(ruv, q[d], lam, p[d], ru->inner_f32);
                gq[d] = inner_f32(ruv, p[d], lam, q[d], ru->inner_f32);
            }
        } else {
            const float sb_rev = 1 / sb;
            const uint16_t e_h = mo_f2h(fix_round(ruv, sb, sb_rev)), l_h = mo_f2h(fix_round(-1 * lam, sb, sb_rev));
            for (int d = 0; d < k; d++) {
                const uint16_t ph = mo_f2h(fix_round(p[d], sb, sb_rev)), qh = mo_f2h(fix_round(q[d], sb, sb_rev));
                gp[d] = mo_h2f(pair_f16(qh, e_h, ph, l_h, ru->mup_bwd_f16));
                gq[d] = mo_h2f(pair_f16(ph, e_h, qh, l_h, ru->mup_bwd_f16));
            }
        }
        for (int d = 0; d < k; d++) {
            p[d] = outer_f32(p[d], lr, gp[d], ru->outer_f32);
            q[d] = outer_f32(q[d], lr, gq[d], ru->outer_f32);
        }
        if (bits_fwd != 32 && bits_bwd != 32 && t >= first_sample_pos && sum_updated_val) {
            norm_total += norm_pq_tree(k, gp, gq, ru->norm_f32);
            for (int d = 0; d < k; d++) sum_updated_val[d] += gp[d] + gq[d];
        }
    }
    if (sum_norms) *sum_norms = norm_total;
}

/* ------------------------------------------------------------------------------------------ */
/* whole-model switching trainer (-v 8): sgd/sgd_kernel.h:166-330                               */
/* ------------------------------------------------------------------------------------------ */
void mo_switching_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, void* Pv, void* Qv, int precision,
                      float lr, float lam, uint64_t first_sample_pos, float* sum_updated_val, float* sum_norms,
                      const mo_rules* ru) {
    if (precision) {
        /* fmaf(lr, e*q - lam*p, p): the compiled form of the plain fp32 trainer */
        mo_sgd_run(k, R, seq, nseq, (float*)Pv, (float*)Qv, lr, lam, ru);
        if (sum_norms) *sum_norms = 0.f;
        return;
    }
    uint16_t* P = (uint16_t*)Pv; uint16_t* Q = (uint16_t*)Qv;
    const uint16_t lr_h = mo_f2h(lr), lam_h = mo_f2h(lam);
    float gp[128], gq[128], norm_total = 0.f;
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        uint16_t* p = P + (size_t)n->u * k; uint16_t* q = Q + (size_t)n->i * k;
        const uint16_t e = mo_hsub(mo_f2h(n->r), dot_f16(k, p, q, ru->dot_f16));
        for (int d = 0; d < k; d++) {
            const uint16_t pv = p[d], qv = q[d];
            const uint16_t tp = inner_f16(e, qv, lam_h, pv, ru->inner_f16), tq = inner_f16(e, pv, lam_h, qv, ru->inner_f16);
            p[d] = mo_hfma(lr_h, tp, pv); q[d] = mo_hfma(lr_h, tq, qv);
            gp[d] = mo_h2f(tp); gq[d] = mo_h2f(tq);
        }
        if (t >= first_sample_pos && sum_updated_val) {
            norm_total += norm_pq_tree(k, gp, gq, ru->norm_f32);
            for (int d = 0; d < k; d++) sum_updated_val[d] += gp[d] + gq[d];
        }
    }
    if (sum_norms) *sum_norms = norm_total;
}

/* ------------------------------------------------------------------------------------------ */
/* AFP (-v 2): afp/afp_sgd_kernel.h:1-125 (helpers), 127-376 (k=128), _k64.h:1-277             */
/* ------------------------------------------------------------------------------------------ */
/* log2 as the restatement computes it: in double precision, rounded once to float (the device code
 * of this repository does the same, so that both sides take identical decisions). */
static inline float log2_rounded(float x) { return (float)log2((double)x); }

/* |ceil(log2(range / (2^(bits-1) - 1)))| (afp_sgd_kernel.h:8-16, 112-118), kept inside the range of
 * float exponents (an all-zero row would give infinity). */
static int afp_exponent(int bits, float range) {
    if (range == 0) return 0;
    float e = fabsf(ceilf(log2_rounded(range / (exp2f((float)(bits - 1)) - 1))));
    return e > 126.f ? 126 : (int)e;
}

typedef struct { int n; float scale; float mov_avg; int64_t next; } afp_side;

/* QEM / QEM_BP (afp_sgd_kernel.h:31-104): relative loss of the sum of magnitudes under 8-bit
 * fixed point; `vals` holds, per lane, the lane's values in the order the reference adds them. */
static float afp_qem(float vals[32][10], int per_lane, float max_val) {
    const float scale = exp2f((float)afp_exponent(8, max_val)), rev = 1 / scale;
    float xq[32], x[32];
    for (int l = 0; l < 32; l++) {
        float sq = fabsf(roundf(vals[l][0] * scale) * rev), sv = fabsf(vals[l][0]);
        for (int j = 1; j < per_lane; j++) { sq = sq + fabsf(roundf(vals[l][j] * scale) * rev); sv = sv + fabsf(vals[l][j]); }
        xq[l] = sq; x[l] = sv;
    }
    const float sum_q = tree32_f32(xq), sum = tree32_f32(x);
    return log2_rounded(fabsf((sum - sum_q) / sum) + 1);
}

/* QPA (afp_sgd_kernel.h:106-125) plus the bookkeeping around it (196-206). */
static void afp_requantize(afp_side* s, float diff, float range, int64_t cur_iter, int epoch, int init_threshold, int avg_mode) {
    const float threshold = 0.0005, alpha = 0.04, beta = 0.1, delta = 100, gamma = 2;
    if (cur_iter == 0) s->mov_avg = range;
    const float prev = s->mov_avg;
    if (diff <= threshold) { s->n = 8; s->scale = exp2f((float)afp_exponent(8, range)); }
    else { s->n = 16; s->scale = exp2f((float)afp_exponent(16, range)); }
    const float keep = 1.0f - alpha;
    if (avg_mode == 1) s->mov_avg = fmaf(alpha, range, keep * prev);
    else if (avg_mode == 2) s->mov_avg = fmaf(keep, prev, alpha * range);
    else s->mov_avg = alpha * range + keep * prev;
    const float i1 = delta * diff * diff, i2 = fabsf(s->mov_avg - prev);
    const float f = (beta / fmaxf(i1, i2)) - gamma;
    int64_t itv = (f != f) ? 0 : (f >= 2147483648.0f ? 2147483647 : (f <= -2147483648.0f ? -2147483647 - 1 : (int64_t)f));
    if (epoch == 0 && cur_iter < init_threshold) itv = 1;
    s->next += itv;
}

void mo_afp_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, int epoch, int init_threshold, const mo_rules* ru) {
    const int slots = k / 32;
    afp_side us = {8, 1.f, 0.f, 0}, is = {8, 1.f, 0.f, 0}, bs = {8, 1.f, 0.f, 0};
    float vals[32][10], gp[128], gq[128];
    for (uint64_t t = 0; t < nseq; t++) {
        const int64_t cur = (int64_t)t;
        const mo_node* n = &R[seq ? seq[t] : t];
        float* p = P + (size_t)n->u * k; float* q = Q + (size_t)n->i * k;
        float pmax = 0.f, qmax = 0.f;
        for (int d = 0; d < k; d++) { pmax = fmaxf(pmax, fabsf(p[d])); qmax = fmaxf(qmax, fabsf(q[d])); }
        if (cur == us.next) {
            for (int l = 0; l < 32; l++) for (int s = 0; s < slots; s++) vals[l][s] = p[l + 32 * s];
            afp_requantize(&us, afp_qem(vals, slots, pmax), pmax, cur, epoch, init_threshold, ru->afp_avg);
        }
        if (cur == is.next) {
            for (int l = 0; l < 32; l++) for (int s = 0; s < slots; s++) vals[l][s] = q[l + 32 * s];
            afp_requantize(&is, afp_qem(vals, slots, qmax), qmax, cur, epoch, init_threshold, ru->afp_avg);
        }
        float pred;
        if (us.n == 8 && is.n == 8) {
            int acc = 0;
            for (int d = 0; d < k; d++) acc += sat8(roundf(p[d] * us.scale)) * sat8(roundf(q[d] * is.scale));
            pred = (float)acc / (us.scale * is.scale);
        } else {
            const float sp_rev = 1 / us.scale, sq_rev = 1 / is.scale;
            uint16_t xs[32], ys[32];
            for (int l = 0; l < 32; l++) {
                uint16_t ph[4], qh[4];
                for (int s = 0; s < slots; s++) {
                    ph[s] = mo_f2h(fix_round(p[l + 32 * s], us.scale, sp_rev));
                    qh[s] = mo_f2h(fix_round(q[l + 32 * s], is.scale, sq_rev));
                }
                if (slots == 4) {
                    xs[l] = pair_f16(ph[0], qh[0], ph[2], qh[2], ru->mup_fwd_f16);
                    ys[l] = pair_f16(ph[1], qh[1], ph[3], qh[3], ru->mup_fwd_f16);
                } else {
                    xs[l] = mo_hmul(ph[0], qh[0]); ys[l] = mo_hmul(ph[1], qh[1]);
                }
            }
            pred = mo_h2f(mo_hadd(tree32_f16(xs), tree32_f16(ys)));
        }
        const float ruv = n->r - pred;
        if (cur == bs.next) {
            const float range = fmaxf(fmaxf(fmaxf(pmax, qmax), fabsf(lam)), fabsf(ruv));
            for (int l = 0; l < 32; l++) {
                int j = 0;
                for (int s = 0; s < slots; s++) vals[l][j++] = p[l + 32 * s];
                for (int s = 0; s < slots; s++) vals[l][j++] = q[l + 32 * s];
                vals[l][j++] = lam; vals[l][j++] = ruv;       /* every lane adds them (afp_sgd_kernel.h:84-86) */
            }
            afp_requantize(&bs, afp_qem(vals, 2 * slots + 2, range), range, cur, epoch, init_threshold, ru->afp_avg);
        }
        if (bs.n == 8) {
            const float rev2 = 1 / (bs.scale * bs.scale);
            const int e_i = sat8(roundf(ruv * bs.scale)), l_i = sat8(roundf(-1.0f * lam * bs.scale));
            for (int d = 0; d < k; d++) {
                const int pi = sat8(roundf(p[d] * bs.scale)), qi = sat8(roundf(q[d] * bs.scale));
                gp[d] = (float)(qi * e_i + pi * l_i) * rev2;
                gq[d] = (float)(pi * e_i + qi * l_i) * rev2;
            }
        } else {
            const float sb_rev = 1 / bs.scale;
            const uint16_t e_h = mo_f2h(fix_round(ruv, bs.scale, sb_rev)), l_h = mo_f2h(fix_round(-1.0f * lam, bs.scale, sb_rev));
            for (int d = 0; d < k; d++) {
                const uint16_t ph = mo_f2h(fix_round(p[d], bs.scale, sb_rev)), qh = mo_f2h(fix_round(q[d], bs.scale, sb_rev));
                gp[d] = mo_h2f(pair_f16(qh, e_h, ph, l_h, ru->mup_bwd_f16));
                gq[d] = mo_h2f(pair_f16(ph, e_h, qh, l_h, ru->mup_bwd_f16));
            }
        }
        for (int d = 0; d < k; d++) {
            p[d] = outer_f32(p[d], lr, gp[d], ru->outer_f32);
            q[d] = outer_f32(q[d], lr, gq[d], ru->outer_f32);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* fp16 storage, fp32 arithmetic (-v 7): sgd/sgd_kernel.h:110-161, sgd_kernel_k64.h:98-137     */
/* ------------------------------------------------------------------------------------------ */
void mo_memquant_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, uint16_t* P, uint16_t* Q,
                     float lr, float lam, const mo_rules* ru) {
    float pf[128], qf[128], x[32];
    for (uint64_t t = 0; t < nseq; t++) {
        const mo_node* n = &R[seq ? seq[t] : t];
        uint16_t* p = P + (size_t)n->u * k; uint16_t* q = Q + (size_t)n->i * k;
        for (int d = 0; d < k; d++) { pf[d] = mo_h2f(p[d]); qf[d] = mo_h2f(q[d]); }
        for (int l = 0; l < 32; l++) x[l] = chain4_f32(pf + l, qf + l, 32, k / 32, ru->chain_f32);
        float e = n->r - tree32_f32(x);
        for (int d = 0; d < k; d++) {
            float pv = pf[d], qv = qf[d];
            p[d] = mo_f2h(outer_f32(pv, lr, inner_f32(e, qv, lam, pv, ru->inner_f32), ru->outer_f32));
            q[d] = mo_f2h(outer_f32(qv, lr, inner_f32(e, pv, lam, qv, ru->inner_f32), ru->outer_f32));
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* test RMSE: rmse.h:26-98 (k=128), 100-166 (k=64), host reduce 168-189                        */
/* ------------------------------------------------------------------------------------------ */
float mo_rmse_literal(int k, const mo_node* T, uint32_t n, const float* P, const float* Q,
                      float* block_err, const mo_rules* ru) {
    uint32_t blocks = (n + 511) / 512;
    float total = 0.f;
    float tmp[512], x[32];
    for (uint32_t b = 0; b < blocks; b++) {
        for (int j = 0; j < 512; j++) {
            uint64_t idx = (uint64_t)b * 512 + j;
            if (idx >= n) { tmp[j] = 0.f; continue; }
            const float* p = P + (size_t)T[idx].u * k; const float* q = Q + (size_t)T[idx].i * k;
            for (int l = 0; l < 32; l++) x[l] = chain4_f32(p + l, q + l, 32, k / 32, ru->chain_f32);
            float d = T[idx].r - tree32_f32(x);
            tmp[j] = d * d;       /* pow(x, 2) of a float: the exact square rounded once */
        }
        for (int s = 256; s >= 1; s >>= 1) for (int j = 0; j < s; j++) tmp[j] = tmp[j] + tmp[j + s];
        if (block_err) block_err[b] = tmp[0];
        total += tmp[0];
    }
    return (float)sqrt(total / (double)n);
}

double mo_rmse_double(int k, const mo_node* T, uint64_t n, const float* P, const float* Q) {
    double total = 0;
    for (uint64_t j = 0; j < n; j++) {
        const float* p = P + (size_t)T[j].u * k; const float* q = Q + (size_t)T[j].i * k;
        double dot = 0;
        for (int d = 0; d < k; d++) dot += (double)p[d] * (double)q[d];
        double e = (double)T[j].r - dot;
        total += e * e;
    }
    return sqrt(total / (double)(n ? n : 1));
}

/* ------------------------------------------------------------------------------------------ */
/* Hogwild epochs on host threads (CPU baseline)                                               */
/* ------------------------------------------------------------------------------------------ */
int mo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void mo_sgd_epoch_hogwild(int k, const mo_node* R, uint64_t n, float* P, float* Q, float lr, float lam,
                          int threads, const mo_rules* rules) {
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t t = 0; t < (int64_t)n; t++)
        sgd_update(k, P + (size_t)R[t].u * k, Q + (size_t)R[t].i * k, R[t].r, lr, lam, rules);
}

void mo_mascot_epoch_hogwild(int k, const mo_node* R, uint64_t n,
                             uint16_t* P16, float* P32, const uint8_t* uprec_row,
                             uint16_t* Q16, float* Q32, const uint8_t* iprec_row,
                             float lr, float lam, int threads, const mo_rules* rules) {
    uint16_t lr_h = mo_f2h(lr), lam_h = mo_f2h(lam);
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t t = 0; t < (int64_t)n; t++) {
        float dv[128]; float ds = 0;
        const mo_node* nd = &R[t];
        mascot_update(k, P16 + (size_t)nd->u * k, P32 + (size_t)nd->u * k, uprec_row[nd->u],
                      Q16 + (size_t)nd->i * k, Q32 + (size_t)nd->i * k, iprec_row[nd->i],
                      nd->r, lr, lam, lr_h, lam_h, 0, dv, dv, &ds, &ds, rules);
    }
}
