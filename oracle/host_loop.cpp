// Host-core baseline: a plain C++ Hogwild loop of the update rule the engine runs, for the
// `cpu_baseline` / `--impl reference` legs of bench.py.  MEASUREMENT INFRASTRUCTURE, not the product and
// not the parity checker: the bit-exact restatement is mascot_oracle.c (software binary16, ~50k updates/s
// per thread); this file trades bit-exactness for speed - hardware half<->float conversions (F16C),
// 8-wide AVX2 arithmetic, every binary16 operation computed in fp32 and rounded back to binary16 (exact
// for add and multiply; a fused multiply-add rounds twice) - and is checked against the oracle by final
// RMSE (tests/test_host_loop.py), not bit for bit.
//
// Rules (the reference's kernels as built, see mascot_oracle.c for the citations):
//   hl_mascot_half_epoch : both rows stored in binary16, arithmetic in binary16
//                          (mascot/mascot_sgd_kernel.h:188-238)
//   hl_sgd_epoch         : fp32 rows, fp32 arithmetic (sgd/sgd_kernel.h:35-76)
// Threads split the rating array into contiguous slices and race on the rows, like the GPU warps.
#include <immintrin.h>
#include <omp.h>
#include <stdint.h>
#include <string.h>

extern "C" {

struct hl_node { float r; uint32_t u; uint32_t i; };

static inline __m256 round_half(__m256 x) {           // to binary16 (nearest even) and back
    return _mm256_cvtph_ps(_mm256_cvtps_ph(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
}
static inline float round_half1(float x) {
    return _cvtsh_ss(_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
}
static inline float hsum_half(__m256 v) {             // tree sum, rounding to binary16 after every add
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    __m128 s = _mm_add_ps(lo, hi);
    s = _mm_cvtph_ps(_mm_cvtps_ph(s, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_cvtph_ps(_mm_cvtps_ph(s, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
    return round_half1(_mm_cvtss_f32(s));
}
static inline float hsum_f32(__m256 v) {
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
    return _mm_cvtss_f32(s);
}

void hl_mascot_half_epoch(int k, const hl_node* R, uint64_t n, uint16_t* P, uint16_t* Q, float lr, float lam, int threads) {
    const float lr_h = round_half1(lr), lam_h = round_half1(lam);
    const __m256 vlr = _mm256_set1_ps(lr_h), vlam = _mm256_set1_ps(lam_h);
    const int nv = k / 8;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t t = 0; t < (int64_t)n; t++) {
        uint16_t* p = P + (size_t)R[t].u * k;
        uint16_t* q = Q + (size_t)R[t].i * k;
        __m256 pv[16], qv[16];
        __m256 acc = _mm256_setzero_ps();
        for (int v = 0; v < nv; v++) {
            pv[v] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(p + 8 * v)));
            qv[v] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(q + 8 * v)));
            acc = round_half(_mm256_add_ps(acc, round_half(_mm256_mul_ps(pv[v], qv[v]))));
        }
        const float e = round_half1(round_half1(R[t].r) - hsum_half(acc));
        const __m256 ve = _mm256_set1_ps(e);
        for (int v = 0; v < nv; v++) {
            const __m256 gp = round_half(_mm256_sub_ps(_mm256_mul_ps(ve, qv[v]), round_half(_mm256_mul_ps(vlam, pv[v]))));
            const __m256 gq = round_half(_mm256_sub_ps(_mm256_mul_ps(ve, pv[v]), round_half(_mm256_mul_ps(vlam, qv[v]))));
            const __m256 pn = _mm256_fmadd_ps(vlr, gp, pv[v]), qn = _mm256_fmadd_ps(vlr, gq, qv[v]);
            _mm_storeu_si128((__m128i*)(p + 8 * v), _mm256_cvtps_ph(pn, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
            _mm_storeu_si128((__m128i*)(q + 8 * v), _mm256_cvtps_ph(qn, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
        }
    }
}

void hl_sgd_epoch(int k, const hl_node* R, uint64_t n, float* P, float* Q, float lr, float lam, int threads) {
    const __m256 vlr = _mm256_set1_ps(lr), vlam = _mm256_set1_ps(lam);
    const int nv = k / 8;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t t = 0; t < (int64_t)n; t++) {
        float* p = P + (size_t)R[t].u * k;
        float* q = Q + (size_t)R[t].i * k;
        __m256 pv[16], qv[16];
        __m256 acc = _mm256_setzero_ps();
        for (int v = 0; v < nv; v++) {
            pv[v] = _mm256_loadu_ps(p + 8 * v); qv[v] = _mm256_loadu_ps(q + 8 * v);
            acc = _mm256_fmadd_ps(pv[v], qv[v], acc);
        }
        const __m256 ve = _mm256_set1_ps(R[t].r - hsum_f32(acc));
        for (int v = 0; v < nv; v++) {
            const __m256 gp = _mm256_fmsub_ps(ve, qv[v], _mm256_mul_ps(vlam, pv[v]));
            const __m256 gq = _mm256_fmsub_ps(ve, pv[v], _mm256_mul_ps(vlam, qv[v]));
            _mm256_storeu_ps(p + 8 * v, _mm256_fmadd_ps(vlr, gp, pv[v]));
            _mm256_storeu_ps(q + 8 * v, _mm256_fmadd_ps(vlr, gq, qv[v]));
        }
    }
}

// fp32 -> binary16 rows and back (round to nearest even), for setting the model up and reading it out
void hl_to_half(const float* src, uint16_t* dst, uint64_t n) {
    for (uint64_t j = 0; j < n; j++) dst[j] = _cvtss_sh(src[j], _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
}
void hl_to_float(const uint16_t* src, float* dst, uint64_t n) {
    for (uint64_t j = 0; j < n; j++) dst[j] = _cvtsh_ss(src[j]);
}

int hl_max_threads(void) { return omp_get_max_threads(); }
int hl_supported(void) { return __builtin_cpu_supports("f16c") && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); }

}  // extern "C"
