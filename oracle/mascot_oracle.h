/* CPU oracle for the MASCOT training hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product library includes, links or calls this file;
 * it is the checker that the parity tests, the smoke test and the CPU-baseline leg of the
 * benchmark compare the CUDA path against.
 *
 * It restates, in plain C with a software binary16, the per-rating update rules and the
 * host-side control logic of the reference (Yujaeseo/ICDM-2021_MASCOT).  Each function cites the
 * reference file:line it follows.  Parity status: PINNED against outputs of the reference's own
 * kernels (golden vectors produced by oracle/ref_harness.cu on a B200, committed under
 * tests/golden/); the reference itself ships no tests or golden vectors.
 *
 * All factor matrices passed here are in the reference's LOGICAL element order (row-major, k
 * consecutive elements per row).
 */
#ifndef MASCOT_ORACLE_H
#define MASCOT_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One training / test rating: same 12-byte record as the reference's Node (common_struct.h:8-12). */
typedef struct { float r; uint32_t u; uint32_t i; } mo_node;

/* How floating-point expressions that the reference writes with plain operators were contracted
 * into fused multiply-adds by the compiler.  0 everywhere = source-literal (every operator rounds
 * separately).  The values that reproduce the reference as built by nvcc 12.9 for sm_100 were
 * found by comparing against the golden vectors and are returned by mo_rules_reference_build(). */
typedef struct {
    int dot_f32;    /* (a0*b0)+(a1*b1):  0 literal | 1 fma(a0,b0,a1*b1) | 2 fma(a1,b1,a0*b0)          */
    int inner_f32;  /* e*q - lam*p:      0 literal | 1 fma(e,q,-(lam*p)) | 2 fma(-lam,p,e*q)           */
    int outer_f32;  /* p + lr*t:         0 literal | 1 fma(lr,t,p)                                      */
    int chain_f32;  /* a0*b0+a1*b1+a2*b2+a3*b3 left to right: 0 literal | 1 fma chain seeded a1*b1 | 2 seeded a0*b0 */
    int norm_f32;   /* (a*a)+(b*b): same coding as dot_f32                                              */
    int dot_f16;    /* binary16 versions of the above                                                   */
    int inner_f16;
    int mpt_outer;  /* p + lr*(rev*g):   0 literal | 1 fma(lr, rev*g, p)                                */
    int stats_sum;  /* (gp + gq) in MuPPET statistics etc.: reserved                                    */
    int mup_fwd_f16; /* MuPPET/AFP binary16 forward pass, hmul2(a,b) + hmul2(c,d): coding as dot_f32    */
    int mup_bwd_f16; /* MuPPET/AFP binary16 backward pass, result.x + result.y of one hmul2: as dot_f32 */
    int afp_avg;     /* AFP moving average alpha*range + (1-alpha)*prev: coding as dot_f32                */
} mo_rules;

void mo_rules_literal(mo_rules* r);
void mo_rules_reference_build(mo_rules* r);

/* ---- binary16 primitives (round-to-nearest-even, subnormals, inf/nan) ---- */
uint16_t mo_f2h(float f);
float    mo_h2f(uint16_t h);
uint16_t mo_hadd(uint16_t a, uint16_t b);
uint16_t mo_hsub(uint16_t a, uint16_t b);
uint16_t mo_hmul(uint16_t a, uint16_t b);
uint16_t mo_hfma(uint16_t a, uint16_t b, uint16_t c);

/* ---- schedule and control logic ---- */
void mo_lr_schedule(float alpha, float decay, int epochs, float* out);
/* g-switching check epochs: returns 1 when epoch e (0-based) computes group errors. */
int mo_is_check_epoch(int e, int epochs, int interval);
/* Degree histogram + ascending stable sort; fills sorted2orig, orig2sorted, cnt_sorted. */
void mo_degree_sort(const uint32_t* ids, uint64_t n, uint64_t stride_words, uint32_t n_entities,
                    uint32_t* sorted2orig, uint32_t* orig2sorted, uint32_t* cnt_sorted);
/* Grouping of degree-sorted entities; returns the number of groups written to end_idx. */
int mo_grouping(const uint32_t* cnt_sorted, uint32_t n_entities, uint32_t requested_groups,
                uint32_t* end_idx, uint32_t* group_of_sorted);
/* Normalised group errors from the sampled statistics; already-fp32 groups report -1. */
void mo_group_errors(const float* grad_sum, const float* norm_sum, int n_norm_parts, int groups, int k,
                     const uint8_t* prec, const float* initial_err, float* err_out);

/* ---- per-rating update engines; seq[t] indexes R, processed sequentially ----
 * Sampled statistics: the reference adds each sampled rating's gradient to the per-group sums with
 * unordered atomics, so the order of that floating-point sum is not defined by the reference.  With
 * item_stats_by_run == 0 the sums grow rating by rating (what one reference warp does, and what the
 * golden vectors hold); with 1 the item side is first summed over each run of consecutive sampled
 * ratings whose items fall in the same group and then added once (what the engine does). */
void mo_sgd_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, const mo_rules* rules);
void mo_mascot_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq,
                   uint16_t* P16, float* P32, const uint8_t* uprec_row, const uint32_t* ugroup,
                   uint16_t* Q16, float* Q32, const uint8_t* iprec_row, const uint32_t* igroup,
                   float lr, float lam, uint64_t first_sample_pos,
                   float* gsum_p, float* gsum_q, float* nsum_p, float* nsum_q, int item_stats_by_run,
                   const mo_rules* rules);
void mo_mpt_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, const mo_rules* rules);
/* MuPPET (-v 3): muppet/muppet_sgd_kernel.h:50-292, muppet_sgd_kernel_k64.h:1-212.  fp32 factors,
 * forward and backward pass in `bits_fwd` / `bits_bwd` (8: int8 dot products, 32: fp32, else
 * fixed-point-rounded binary16).  Ratings at sequence positions >= first_sample_pos add to
 * sum_updated_val[k] and *sum_norms when neither pass is 32-bit. */
void mo_muppet_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                   float lr, float lam, int bits_fwd, int bits_bwd, uint64_t first_sample_pos,
                   float* sum_updated_val, float* sum_norms, const mo_rules* rules);
/* Whole-model switching trainer (-v 8, k=128 in the reference): sgd/sgd_kernel.h:166-330.
 * precision 0: every row binary16, arithmetic of MASCOT's all-binary16 case, sampled statistics in
 * MuPPET's form (one norm sum, one k-vector of summed updates); precision 1: fp32 with explicit fmaf,
 * no statistics.  P/Q point to uint16_t (precision 0) or float (precision 1) rows. */
void mo_switching_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, void* P, void* Q, int precision,
                      float lr, float lam, uint64_t first_sample_pos, float* sum_updated_val, float* sum_norms,
                      const mo_rules* rules);
/* AFP (-v 2): afp/afp_sgd_kernel.h:1-376, afp_sgd_kernel_k64.h:1-277.  One sequential worker: the
 * per-warp state of the reference (three sets of quantization parameters and their re-estimation
 * counters) lives for the whole sequence.  `epoch` and `init_threshold` are the kernel arguments
 * that force re-estimation at every rating early in the first epoch. */
void mo_afp_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, float* P, float* Q,
                float lr, float lam, int epoch, int init_threshold, const mo_rules* rules);
void mo_memquant_run(int k, const mo_node* R, const uint32_t* seq, uint64_t nseq, uint16_t* P, uint16_t* Q,
                     float lr, float lam, const mo_rules* rules);

/* ---- initialisation ---- */
/* The engine's seeded N(0, 0.01^2) factor generator, restated for the host: element t of stream
 * `sid` (1 = user factors, 2 = item factors, both in the caller's row order). */
void mo_init_normal(float* dst, uint64_t count, uint64_t seed, uint64_t sid);

/* ---- evaluation ---- */
/* Reference-literal test RMSE: fp32 dot, 512-rating block trees, float sum of block partials. */
float mo_rmse_literal(int k, const mo_node* T, uint32_t n, const float* P, const float* Q,
                      float* block_err, const mo_rules* rules);
double mo_rmse_double(int k, const mo_node* T, uint64_t n, const float* P, const float* Q);

/* ---- multi-threaded Hogwild epochs (CPU baseline; racy by design like the reference) ---- */
void mo_sgd_epoch_hogwild(int k, const mo_node* R, uint64_t n, float* P, float* Q, float lr, float lam,
                          int threads, const mo_rules* rules);
void mo_mascot_epoch_hogwild(int k, const mo_node* R, uint64_t n,
                             uint16_t* P16, float* P32, const uint8_t* uprec_row,
                             uint16_t* Q16, float* Q32, const uint8_t* iprec_row,
                             float lr, float lam, int threads, const mo_rules* rules);
int mo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
