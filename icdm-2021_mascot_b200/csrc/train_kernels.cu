// Per-rating SGD update kernels for sm_100a.
//
// WORKERS.  The reference runs `-wg` warps, each applying one rating at a time; the number of such
// sequential workers decides how many updates of a popular row are lost to races, i.e. how fast the
// model converges per epoch.  This engine keeps that meaning of `-wg` - a worker is a group of
// K/8 lanes (16 for k=128, 8 for k=64; two or four workers per warp) that applies its ratings
// strictly one after the other - and gets its speed from making each worker fast instead of adding
// workers:
//   * every lane holds eight consecutive physical elements of a row (one 128-bit access for
//     binary16 storage, two for fp32);
//   * the rating records of a chunk (one rating per lane) are loaded one chunk ahead, tagged
//     (repeated user, start of an item run, repeated item) and put into shared memory, from where
//     the worker reads one rating with a single 128-bit broadcast load;
//   * rows travel global -> shared memory by cp.async into small per-worker rings, user rows a few
//     ratings ahead, item rows one rating ahead; copy groups complete in order, so the wait for the
//     row of rating j leaves the younger copies in flight (register loads cannot do that: the wait
//     for an old load also waits for every younger load on the same scoreboard);
//   * the row of an item that repeats (the stream is item-sorted inside shuffle windows) stays in
//     registers for the whole run and is written back once;
//   * chunks are handed out in runs of up to eight through one atomic ticket per run; the runs shrink
//     to single chunks near the end of the stream, so that all workers finish together.
//   * user rows are written back as vector reductions of their change whenever several workers run,
//     so racing updates of one user add up instead of overwriting each other (add_row_delta).
// The item lead is short on purpose.  Between the request of an item row and its write-back (a plain
// store, once per run) every update another worker makes to that row is lost, so the loss grows with
// (workers x lead); measured on the 100M-rating configuration with plain stores on both sides, a lead
// of seven ratings costs 1.5 % of final RMSE where three (users) and one (items) cost nothing.
//
// ELEMENT ORDER.  layout.cuh stores rows permuted so that lane m of a worker holds the elements of
// reference lanes m and m+16 (k=128) or m, m+16, m+8, m+24 (k=64).  With pair products
// f_j = fma(a_2j, b_2j, a_2j+1 * b_2j+1) the lane partial (f_0 + f_1) + (f_2 + f_3) and a xor
// butterfly over the worker's lanes add exactly the pairs that the reference's per-lane sum and
// shfl_down 16-8-4-2-1 tree add, so results are bit-identical to the reference kernels:
//   all binary16      mascot/mascot_sgd_kernel.h:188-278     binary16 user / fp32 item  :279-342
//   fp32 / binary16   mascot/mascot_sgd_kernel.h:343-407     all fp32                   :408-443
//   (sgd/sgd_kernel.h:35-76 compiles to the same operations as the all-fp32 case)
//   MPT               mpt/mpt_sgd_kernel.h:38-91              fp16 storage (-v 7)  sgd/sgd_kernel.h:110-161
//   MuPPET            muppet/muppet_sgd_kernel.h:121-285      AFP                  afp/afp_sgd_kernel.h:194-371
//   whole-model switching (-v 8)  sgd/sgd_kernel.h:205-326 (binary16 phase = the all-binary16 case above
//   with MuPPET's form of the statistics; fp32 phase = the fp32 trainer)
// including the fused multiply-adds the compiled reference executes.  Every operation is written
// with a rounding-mode intrinsic so that ptxas cannot contract or re-associate anything further.
//
// Bit 31 of a stream id says which arena (binary16 or fp32) the row lives in, which replaces the
// reference's per-rating group search (mascot_sgd_kernel.h:104-180).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "engine.h"
#include "launch_cache.h"
#include "layout.cuh"

namespace mascot {

namespace {

constexpr uint32_t kNoRow = 0xffffffffu;     // never a valid stream id

struct V8h { __half2 v[4]; };                // eight binary16 values, physical order
struct V8f { float x[8]; };

// How the rows of one side are stored in a launch.  Known on the host, so the common cases carry no
// per-rating precision test, no unused registers and no oversized ring slots.  The mixed-precision
// trainer keeps its stream partitioned by (user precision, item precision), and every part runs the
// instantiation made for it; ROWS_DYN (precision read from bit 31 of the id, per rating) remains for
// the deterministic single-worker mode, which must follow the stream in its original order.
enum RowMode { ROWS_HALF = 0, ROWS_F32 = 1, ROWS_DYN = 2 };

// A lane's slice of a row as fetched: 16 bytes for binary16 storage, 32 bytes for fp32 storage.
template <int MODE> struct Raw { uint4 a, b; };
template <> struct Raw<ROWS_HALF> { uint4 a; };

__device__ __forceinline__ V8h v8h_of(const uint4& a) {
    V8h h;
    h.v[0] = *reinterpret_cast<const __half2*>(&a.x); h.v[1] = *reinterpret_cast<const __half2*>(&a.y);
    h.v[2] = *reinterpret_cast<const __half2*>(&a.z); h.v[3] = *reinterpret_cast<const __half2*>(&a.w);
    return h;
}
__device__ __forceinline__ V8f v8f_of(const uint4& a, const uint4& b) {
    V8f f;
    f.x[0] = __uint_as_float(a.x); f.x[1] = __uint_as_float(a.y); f.x[2] = __uint_as_float(a.z); f.x[3] = __uint_as_float(a.w);
    f.x[4] = __uint_as_float(b.x); f.x[5] = __uint_as_float(b.y); f.x[6] = __uint_as_float(b.z); f.x[7] = __uint_as_float(b.w);
    return f;
}
template <int MODE> __device__ __forceinline__ V8h as_v8h(const Raw<MODE>& r) { return v8h_of(r.a); }
template <int MODE> __device__ __forceinline__ V8f as_v8f(const Raw<MODE>& r) {
    if constexpr (MODE != ROWS_HALF) return v8f_of(r.a, r.b); else return v8f_of(r.a, r.a);   // fp32 rows never occur in ROWS_HALF
}

template <int MODE> __device__ __forceinline__ void put(Raw<MODE>& r, const V8h& h) {
    r.a.x = *reinterpret_cast<const unsigned*>(&h.v[0]); r.a.y = *reinterpret_cast<const unsigned*>(&h.v[1]);
    r.a.z = *reinterpret_cast<const unsigned*>(&h.v[2]); r.a.w = *reinterpret_cast<const unsigned*>(&h.v[3]);
}
template <int MODE> __device__ __forceinline__ void put(Raw<MODE>& r, const V8f& f) {
    if constexpr (MODE != ROWS_HALF) {
        r.a = make_uint4(__float_as_uint(f.x[0]), __float_as_uint(f.x[1]), __float_as_uint(f.x[2]), __float_as_uint(f.x[3]));
        r.b = make_uint4(__float_as_uint(f.x[4]), __float_as_uint(f.x[5]), __float_as_uint(f.x[6]), __float_as_uint(f.x[7]));
    }
}

__device__ __forceinline__ V8f widen(const V8h& h) {
    V8f f;
#pragma unroll
    for (int s = 0; s < 4; s++) { const float2 t = __half22float2(h.v[s]); f.x[2 * s] = t.x; f.x[2 * s + 1] = t.y; }
    return f;
}
__device__ __forceinline__ V8h narrow(const V8f& f) {
    V8h h;
#pragma unroll
    for (int s = 0; s < 4; s++) h.v[s] = __halves2half2(__float2half_rn(f.x[2 * s]), __float2half_rn(f.x[2 * s + 1]));
    return h;
}

// Is the row behind this stream id stored in fp32?
template <int MODE> __device__ __forceinline__ bool is_f32(uint32_t code) {
    return MODE == ROWS_F32 || (MODE == ROWS_DYN && (code & kPrecBit));
}

// Row slice of lane m: L2-only loads/stores (rows are shared between SMs and never reused from L1).
template <int K, int MODE>
__device__ __forceinline__ Raw<MODE> ld_row(const Arena& A, uint32_t code, int m) {
    const uint32_t row = code & kIdMask;
    Raw<MODE> r;
    if (is_f32<MODE>(code)) {
        const uint4* p = reinterpret_cast<const uint4*>(A.f32 + (size_t)row * K) + m;     // first half; second half K/8 uint4 on
        r.a = __ldcg(p);
        if constexpr (MODE != ROWS_HALF) r.b = __ldcg(p + K / 8);
    } else {
        r.a = __ldcg(reinterpret_cast<const uint4*>(A.f16 + (size_t)row * K) + m);
    }
    return r;
}
template <int K, int MODE>
__device__ __forceinline__ void st_row(const Arena& A, uint32_t code, int m, const Raw<MODE>& r) {
    const uint32_t row = code & kIdMask;
    if (is_f32<MODE>(code)) {
        uint4* p = reinterpret_cast<uint4*>(A.f32 + (size_t)row * K) + m;
        __stcg(p, r.a);
        if constexpr (MODE != ROWS_HALF) __stcg(p + K / 8, r.b);
    } else {
        __stcg(reinterpret_cast<uint4*>(A.f16 + (size_t)row * K) + m, r.a);
    }
}

// Adds (now - before) to a row instead of storing `now`: with several workers on the same row at the
// same time a plain store erases what the others wrote since this worker read the row, a reduction
// keeps it.  (Not used for rows flagged kHotBit: summing the changes of very many concurrent updates
// that all started from the same stale value multiplies the step; there the plain store stays.)  When nobody else touched the row the result equals `now` (the difference of two nearby
// values is exact).  128-bit vector reductions, fire and forget.
template <int K, int MODE>
__device__ __forceinline__ void add_row_delta(const Arena& A, uint32_t code, int m, const Raw<MODE>& now, const Raw<MODE>& before) {
    const uint32_t row = code & kIdMask;
    if (is_f32<MODE>(code)) {
        if constexpr (MODE != ROWS_HALF) {
            float4* p = reinterpret_cast<float4*>(A.f32 + (size_t)row * K) + m;
            const V8f n = v8f_of(now.a, now.b), o = v8f_of(before.a, before.b);
            atomicAdd(p, make_float4(__fsub_rn(n.x[0], o.x[0]), __fsub_rn(n.x[1], o.x[1]), __fsub_rn(n.x[2], o.x[2]), __fsub_rn(n.x[3], o.x[3])));
            atomicAdd(p + K / 8, make_float4(__fsub_rn(n.x[4], o.x[4]), __fsub_rn(n.x[5], o.x[5]), __fsub_rn(n.x[6], o.x[6]), __fsub_rn(n.x[7], o.x[7])));
        }
    } else {
        const V8h n = v8h_of(now.a), o = v8h_of(before.a);
        unsigned d[4];
#pragma unroll
        for (int t = 0; t < 4; t++) { const __half2 x = __hsub2(n.v[t], o.v[t]); d[t] = *reinterpret_cast<const unsigned*>(&x); }
        uint4* p = reinterpret_cast<uint4*>(A.f16 + (size_t)row * K) + m;
        asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d[0]), "r"(d[1]), "r"(d[2]), "r"(d[3]) : "memory");
    }
}

// ---- lane partials -------------------------------------------------------------------------
// A lane's elements e0..e7 sit at positions 0 2 4 6 1 3 5 7 (layout.cuh), i.e. as the binary16 pairs
// (e0,e4) (e1,e5) (e2,e6) (e3,e7).  Lane partial: (f_0 + f_1) + (f_2 + f_3) with
// f_j = fma(e_2j, e'_2j, e_2j+1 * e'_2j+1).
// fp32 arithmetic runs on the packed two-lane instructions of sm_100 (fma / mul / add .f32x2): each lane
// is rounded on its own, exactly like the scalar instruction, and a row slice needs half as many issue
// slots - which is what bounds this kernel.
__device__ __forceinline__ float2 pr(const V8f& v, int j) { return make_float2(v.x[2 * j], v.x[2 * j + 1]); }
__device__ __forceinline__ void set_pr(V8f& v, int j, float2 t) { v.x[2 * j] = t.x; v.x[2 * j + 1] = t.y; }

__device__ __forceinline__ float pair_partial(const V8f& a, const V8f& b) {
    // (f0, f2) = (a0 b0 + a2 b2, a1 b1 + a3 b3), (f1, f3) likewise from positions 4..7
    const float2 f02 = __ffma2_rn(pr(a, 0), pr(b, 0), __fmul2_rn(pr(a, 1), pr(b, 1)));
    const float2 f13 = __ffma2_rn(pr(a, 2), pr(b, 2), __fmul2_rn(pr(a, 3), pr(b, 3)));
    const float2 t = __fadd2_rn(f02, f13);                                     // (f0+f1, f2+f3)
    return __fadd_rn(t.x, t.y);
}
__device__ __forceinline__ __half pair_partial(const V8h& p, const V8h& q) {
    const __half2 f02 = __hfma2(p.v[0], q.v[0], __hmul2_rn(p.v[1], q.v[1]));   // (f_0, f_2)
    const __half2 f13 = __hfma2(p.v[2], q.v[2], __hmul2_rn(p.v[3], q.v[3]));   // (f_1, f_3)
    const __half2 t = __hadd2_rn(f02, f13);                                     // (f_0+f_1, f_2+f_3)
    return __hadd_rn(__low2half(t), __high2half(t));
}
// k=128 only: the left-to-right product chain of a reference lane over its four elements,
// fma(a3,b3, fma(a2,b2, fma(a0,b0, a1*b1))), for the two reference lanes this lane holds
// (fp16-storage trainer sgd/sgd_kernel.h:124, RMSE rmse.h:75).
__device__ __forceinline__ float chain_partial_k128(const V8f& a, const V8f& b) {
    float c[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {          // h = 0: e0..e3 at positions 0 2 4 6;  h = 1: e4..e7 at 1 3 5 7
        float acc = __fmaf_rn(a.x[h], b.x[h], __fmul_rn(a.x[2 + h], b.x[2 + h]));
        acc = __fmaf_rn(a.x[4 + h], b.x[4 + h], acc);
        c[h] = __fmaf_rn(a.x[6 + h], b.x[6 + h], acc);
    }
    return __fadd_rn(c[0], c[1]);
}

template <int TS>
__device__ __forceinline__ float worker_sum(float x, unsigned wmask) {
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) x = __fadd_rn(x, __shfl_xor_sync(wmask, x, d));
    return x;
}
template <int TS>
__device__ __forceinline__ __half worker_sum(__half x, unsigned wmask) {
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) x = __hadd_rn(x, __shfl_xor_sync(wmask, x, d));
    return x;
}

// t = fma(e, y, -(lam*x)) and x' = fma(lr, t, x), element-wise
__device__ __forceinline__ V8f grad(float e, const V8f& y, float lam, const V8f& x) {
    V8f g;
    const float2 e2 = make_float2(e, e), nlam2 = make_float2(-lam, -lam);      // (-lam) * x == -(lam * x), bit for bit
#pragma unroll
    for (int j = 0; j < 4; j++) set_pr(g, j, __ffma2_rn(e2, pr(y, j), __fmul2_rn(nlam2, pr(x, j))));
    return g;
}
__device__ __forceinline__ V8h grad(__half2 e, const V8h& y, __half2 lam, const V8h& x) {
    V8h g;
#pragma unroll
    for (int s = 0; s < 4; s++) g.v[s] = __hfma2(e, y.v[s], __hneg2(__hmul2_rn(lam, x.v[s])));
    return g;
}
__device__ __forceinline__ V8f step(float lr, const V8f& g, const V8f& x) {
    V8f o;
    const float2 lr2 = make_float2(lr, lr);
#pragma unroll
    for (int j = 0; j < 4; j++) set_pr(o, j, __ffma2_rn(lr2, pr(g, j), pr(x, j)));
    return o;
}
__device__ __forceinline__ V8h step(__half2 lr, const V8h& g, const V8h& x) {
    V8h o;
#pragma unroll
    for (int s = 0; s < 4; s++) o.v[s] = __hfma2(lr, g.v[s], x.v[s]);
    return o;
}

struct Consts {
    float lr, lam;
    __half2 lr_h, lam_h;          // mascot_sgd_kernel.h:79-80
    __half mpt_scale;             // mpt_sgd_kernel.h:15-16
    __half2 mpt_lam;              // mf_methods.cu:764-765
    float mpt_rev;
    int bits;                     // MuPPET: width of the forward and the backward pass
    int afp_epoch, afp_init_threshold;   // AFP: epoch index; ratings per worker / 10 (afp_sgd_kernel.h:143)
};

// Sampled statistics (mascot_sgd_kernel.h:240-277): per group the element-wise sum of the gradients
// and the sum of their squared norms.  They go to global memory as 128-bit fire-and-forget
// reductions.  The reference adds every rating's gradient with scalar atomics in no particular
// order; here the user side does the same per rating, while the item side - whose ratings arrive in
// runs of the same group, because shuffle windows are item-sorted - is summed in registers over a run
// of equal item groups and flushed once per run, which removes the contention on popular items.
struct Sample {
    V8f gp, gq;
    bool user, item;      // which sides of this rating contribute (binary16-stored rows only)
};

__device__ __forceinline__ void red_add8(float* dst, const V8f& g) {
    atomicAdd(reinterpret_cast<float4*>(dst), make_float4(g.x[0], g.x[1], g.x[2], g.x[3]));
    atomicAdd(reinterpret_cast<float4*>(dst) + 1, make_float4(g.x[4], g.x[5], g.x[6], g.x[7]));
}

struct KernelArgs {
    Stream s;
    Arena P, Q;
    float lr, lam;
    SampleStats st;
    int bits;                     // MuPPET pass width
    int epoch;                    // AFP: epoch index
    int add_user_delta;           // user rows are written back as reductions of the change (concurrent launches)
    unsigned workers;             // concurrent sequential workers actually launched
    unsigned long long* next_chunk;   // work counter, zero at launch: chunks beyond the first two runs per
                                      // worker are handed out dynamically, so the launch never depends on
                                      // every block being resident at the same time
    unsigned long long* zero_counter; // another counter, which this launch resets for a later launch
    unsigned hot_user_shift;          // one in 2^this of the updates of a marked user row is written back
};

// ---- MuPPET (muppet/muppet_sgd_kernel.h:7-48, 121-264; _k64.h) -------------------------------
// Power-of-two scale for a `bits`-wide fixed-point grid that covers [lo, hi]: the reference takes
// floor(log2(min(|qmax/hi|, |qmin/lo|))) with qmax = 2^(bits-1)-0.5, qmin = -2^(bits-1)-0.5, stores
// it in an unsigned index (negative -> 0) and scales by 2^index.
__device__ __forceinline__ float muppet_scale(int bits, float hi, float lo) {
    if (hi == 0.f && lo == 0.f) return 1.f;
    const float val = (float)(1 << (bits - 1));
    const float top = __fadd_rn(__fsub_rn(val, 1.f), 0.5f), bottom = __fsub_rn(-val, 0.5f);
    const float best = fminf(fabsf(__fdiv_rn(top, hi)), fabsf(__fdiv_rn(bottom, lo)));
    const float idx = floorf(log2f(best));
    if (!(idx > 0.f)) return 1.f;
    const int e = idx > 127.f ? 128 : (int)idx;
    return e >= 128 ? __int_as_float(0x7f800000) : __int_as_float((e + 127) << 23);
}
// roundf (halves away from zero) in three instructions: trunc(x + copysign(largest float below one half, x)).
// The sum is rounded to nearest-even, which is what makes it exact: x = n + f with f < 1/2 cannot reach n + 1,
// f >= 1/2 always does.  Equal to roundf for every one of the 2^32 float patterns (checked exhaustively on the
// host, tests/round_check.c); the library routine costs about three times as much and these trainers call it
// 34 times per rating and lane.
__device__ __forceinline__ float round_away(float x) {
    const float h = __uint_as_float((__float_as_uint(x) & 0x80000000u) | 0x3effffffu);
    return truncf(__fadd_rn(x, h));
}
// 1 / s for a scale that is a power of two: the exponent mirrored around zero, exact while both s and 1 / s are
// normal numbers; anything else (2^127, infinity) takes the division.
__device__ __forceinline__ float pow2_rev(float s) {
    const uint32_t b = __float_as_uint(s);
    return (b >= 0x00800000u && b < 0x7f000000u && !(b & 0x007fffffu)) ? __uint_as_float(0x7f000000u - b) : __fdiv_rn(1.f, s);
}
__device__ __forceinline__ float fix_round(float v, float s, float s_rev) { return __fmul_rn(round_away(__fmul_rn(v, s)), s_rev); }
// Clamp to the int8 range, then to integer.  Every caller passes a value that round_away has already made
// integral, so the one conversion instruction with saturation (truncating, which changes nothing then) equals
// v > 127 ? 127 : (v < -128 ? -128 : (int)v).
__device__ __forceinline__ int sat8(float v) {
    int r;
    asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ V8h fix_round_half(const V8f& x, float s, float s_rev) {
    V8h h;
#pragma unroll
    for (int t = 0; t < 4; t++)
        h.v[t] = __floats2half2_rn(fix_round(x.x[2 * t], s, s_rev), fix_round(x.x[2 * t + 1], s, s_rev));
    return h;
}
template <int TS> __device__ __forceinline__ float worker_min(float x, unsigned wmask) {
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) x = fminf(x, __shfl_xor_sync(wmask, x, d));
    return x;
}
template <int TS> __device__ __forceinline__ float worker_max(float x, unsigned wmask) {
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) x = fmaxf(x, __shfl_xor_sync(wmask, x, d));
    return x;
}
// Squared norm of both gradients the way the reference groups it: per reference lane
// (norm_p + norm_q), then the lane tree.  A lane here holds two (k=128) or four (k=64) reference lanes.
template <int K>
__device__ __forceinline__ float muppet_norm_partial(const V8f& gp, const V8f& gq) {
    auto sq = [](const V8f& g, int a, int b) { return __fmaf_rn(g.x[a], g.x[a], __fmul_rn(g.x[b], g.x[b])); };
    if (K == 128) {
        const float la = __fadd_rn(__fadd_rn(sq(gp, 0, 2), sq(gp, 4, 6)), __fadd_rn(sq(gq, 0, 2), sq(gq, 4, 6)));
        const float lb = __fadd_rn(__fadd_rn(sq(gp, 1, 3), sq(gp, 5, 7)), __fadd_rn(sq(gq, 1, 3), sq(gq, 5, 7)));
        return __fadd_rn(la, lb);
    }
    const float l0 = __fadd_rn(sq(gp, 0, 2), sq(gq, 0, 2)), l1 = __fadd_rn(sq(gp, 4, 6), sq(gq, 4, 6));
    const float l2 = __fadd_rn(sq(gp, 1, 3), sq(gq, 1, 3)), l3 = __fadd_rn(sq(gp, 5, 7), sq(gq, 5, 7));
    return __fadd_rn(__fadd_rn(l0, l1), __fadd_rn(l2, l3));
}

// ---- passes shared by MuPPET and AFP ------------------------------------------------------------
// int8 forward pass: saturated fixed-point values, exact integer dot product, one division
template <int TS>
__device__ __forceinline__ float forward_int8(const V8f& p, const V8f& q, float sp, float sq, unsigned wmask) {
    int acc = 0;
#pragma unroll
    for (int t = 0; t < 8; t++) acc += sat8(round_away(__fmul_rn(p.x[t], sp))) * sat8(round_away(__fmul_rn(q.x[t], sq)));
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) acc += __shfl_xor_sync(wmask, acc, d);
    return __fdiv_rn((float)acc, __fmul_rn(sp, sq));
}
// binary16 forward pass on the fixed-point grid; the two halves of the reference's half2 accumulator
// go through the lane tree separately and meet at the end (muppet_sgd_kernel.h:170-194,
// afp_sgd_kernel.h:252-273)
template <int K>
__device__ __forceinline__ float forward_half(const V8f& p, const V8f& q, float sp, float sq, unsigned wmask) {
    constexpr int TS = K / 8;
    const V8h ph = fix_round_half(p, sp, pow2_rev(sp)), qh = fix_round_half(q, sq, pow2_rev(sq));
    __half2 xy;
    if (K == 128) {
        const __half2 xab = __hfma2(ph.v[0], qh.v[0], __hmul2_rn(ph.v[2], qh.v[2]));   // (x of lane m, x of lane m+16)
        const __half2 yab = __hfma2(ph.v[1], qh.v[1], __hmul2_rn(ph.v[3], qh.v[3]));
        xy = __hadd2_rn(__lows2half2(xab, yab), __highs2half2(xab, yab));              // tree step 16
    } else {
        const __half2 x = __hadd2_rn(__hmul2_rn(ph.v[0], qh.v[0]), __hmul2_rn(ph.v[2], qh.v[2]));   // step 16: (m)+(m+16), (m+8)+(m+24)
        const __half2 y = __hadd2_rn(__hmul2_rn(ph.v[1], qh.v[1]), __hmul2_rn(ph.v[3], qh.v[3]));
        xy = __hadd2_rn(__lows2half2(x, y), __highs2half2(x, y));                                   // step 8
    }
#pragma unroll
    for (int d = TS / 2; d >= 1; d >>= 1) {
        const unsigned o = __shfl_xor_sync(wmask, *reinterpret_cast<unsigned*>(&xy), d);
        xy = __hadd2_rn(xy, *reinterpret_cast<const __half2*>(&o));
    }
    return __half2float(__hadd_rn(__low2half(xy), __high2half(xy)));
}
// backward passes: g_p = q*e + p*(-lam), g_q = p*e + q*(-lam) in int8 or binary16 fixed point
__device__ __forceinline__ void backward_int8(const V8f& p, const V8f& q, float ruv, float nlam, float sb, V8f& gp, V8f& gq) {
    const float rev2 = __fdiv_rn(1.f, __fmul_rn(sb, sb));
    const int ei = sat8(round_away(__fmul_rn(ruv, sb))), li = sat8(round_away(__fmul_rn(nlam, sb)));
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const int pi = sat8(round_away(__fmul_rn(p.x[t], sb))), qi = sat8(round_away(__fmul_rn(q.x[t], sb)));
        gp.x[t] = __fmul_rn((float)(qi * ei + pi * li), rev2);
        gq.x[t] = __fmul_rn((float)(pi * ei + qi * li), rev2);
    }
}
__device__ __forceinline__ void backward_half(const V8f& p, const V8f& q, float ruv, float nlam, float sb, V8f& gp, V8f& gq) {
    const float sb_rev = pow2_rev(sb);
    const __half2 e2 = __half2half2(__float2half_rn(fix_round(ruv, sb, sb_rev)));
    const __half2 l2 = __half2half2(__float2half_rn(fix_round(nlam, sb, sb_rev)));
    const V8h ph = fix_round_half(p, sb, sb_rev), qh = fix_round_half(q, sb, sb_rev);
    V8h gph, gqh;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        gph.v[t] = __hadd2_rn(__hmul2_rn(qh.v[t], e2), __hmul2_rn(ph.v[t], l2));
        gqh.v[t] = __hadd2_rn(__hmul2_rn(ph.v[t], e2), __hmul2_rn(qh.v[t], l2));
    }
    gp = widen(gph); gq = widen(gqh);
}

template <int K>
__device__ __forceinline__ void muppet_update(const Consts& c, float r, V8f& p, V8f& q, V8f& gp, V8f& gq, unsigned wmask) {
    constexpr int TS = K / 8;
    const int bits = c.bits;
    float pmin = 0.f, pmax = 0.f, qmin = 0.f, qmax = 0.f, sp = 1.f, sq = 1.f, pred;
    if (bits != 32) {
        pmin = pmax = p.x[0]; qmin = qmax = q.x[0];
#pragma unroll
        for (int t = 1; t < 8; t++) {
            pmin = fminf(pmin, p.x[t]); pmax = fmaxf(pmax, p.x[t]);
            qmin = fminf(qmin, q.x[t]); qmax = fmaxf(qmax, q.x[t]);
        }
        pmin = worker_min<TS>(pmin, wmask); pmax = worker_max<TS>(pmax, wmask);
        qmin = worker_min<TS>(qmin, wmask); qmax = worker_max<TS>(qmax, wmask);
        sp = muppet_scale(bits, pmax, pmin); sq = muppet_scale(bits, qmax, qmin);
    }
    if (bits == 8) pred = forward_int8<TS>(p, q, sp, sq, wmask);
    else if (bits == 32) pred = worker_sum<TS>(pair_partial(p, q), wmask);
    else pred = forward_half<K>(p, q, sp, sq, wmask);
    const float ruv = __fsub_rn(r, pred);
    const float nlam = -c.lam;
    float sb = 1.f;
    if (bits != 32) {
        const float bmin = fminf(fminf(pmin, qmin), fminf(nlam, ruv)), bmax = fmaxf(fmaxf(pmax, qmax), fmaxf(nlam, ruv));
        sb = muppet_scale(bits, bmax, bmin);
    }
    if (bits == 8) backward_int8(p, q, ruv, nlam, sb, gp, gq);
    else if (bits == 32) { gp = grad(ruv, q, c.lam, p); gq = grad(ruv, p, c.lam, q); }
    else backward_half(p, q, ruv, nlam, sb, gp, gq);
    p = step(c.lr, gp, p); q = step(c.lr, gq, q);
}

// ---- AFP (afp/afp_sgd_kernel.h:1-125 helpers, 127-376 k=128; afp_sgd_kernel_k64.h) ----------------
// One side's quantization parameters and the rating count at which they are estimated next.  The
// reference keeps three of these per warp for a whole kernel launch; here per worker.
struct AfpSide { int n; float scale; float mov_avg; long long next; };
struct AfpState { AfpSide user, item, back; long long cur; };

// log2 in double precision, rounded once to float: the CPU restatement computes it the same way, so
// both take identical re-estimation decisions (it runs only when parameters are re-estimated).
// The re-estimation helpers below are deliberately NOT inlined: they run once in many ratings, and inlined -
// six copies of the double-precision logarithm per update, times the unrolled ring - they made the AFP kernel
// so large that its warps waited 5 cycles per issued instruction for instruction fetches.
__device__ __noinline__ float log2_rounded(float x) { return (float)log2((double)x); }

// ceil((float)log2((double)x)) for x > 0 without the logarithm.  x = (1 + M / 2^23) * 2^E: log2(x) lies in
// [E, E + 1); rounded to float it is E itself when M = 0, or when the fraction is below half the spacing of the
// floats next to E on the side of E + 1 - the first few M only, the more the larger |E| - and otherwise a value in
// (E, E + 1], whose ceiling is E + 1.  Equal to the double-precision formula of the CPU restatement for every
// positive finite float (checked exhaustively on the host, tests/ceil_log2_check.c).  Zero gives a large negative
// number, as the logarithm would.
__device__ __forceinline__ int ceil_log2_rounded(float x) {
    const uint32_t bits = __float_as_uint(x) & 0x7fffffffu;
    if (bits == 0u) return -100000;
    int E = (int)(bits >> 23) - 127;
    uint32_t M = bits & 0x7fffffu;
    if ((bits >> 23) == 0u) {                      // denormal: normalise
        const int lz = __clz((int)M) - 9;
        E = -126 - (lz + 1);
        M = (M << (lz + 1)) & 0x7fffffu;
    }
    if (M == 0u) return E;
    uint32_t a = (uint32_t)(E < 0 ? -E : E);
    if (E < 0) a -= 1u;                            // the floats between E and E + 1 are smaller in magnitude than |E|
    if (E <= 0 && a == 0u) return E + 1;
    const int j = 31 - __clz((int)a);
    const uint32_t limit = j <= 1 ? 0u : (j == 2 ? 1u : (j == 3 ? 2u : (j == 4 ? 5u : (j == 5 ? 11u : (j == 6 ? 22u : 44u)))));
    return M <= limit ? E : E + 1;
}

// 2^|ceil(log2(range / (2^(bits-1) - 1)))| (afp_sgd_kernel.h:8-16, 112-118); exponent capped at 126
__device__ __forceinline__ float afp_scale(int bits, float range) {
    if (range == 0.f) return 1.f;
    const float top = bits == 8 ? 127.f : 32767.f;
    const int c = ceil_log2_rounded(__fdiv_rn(range, top));
    const int e = c < 0 ? -c : c;
    const int ei = e > 126 ? 126 : e;
    return __int_as_float((ei + 127) << 23);
}
// Sum of magnitudes of the values a reference lane adds, left to right, before and after 8-bit
// rounding; `G` reference lanes live in this lane, `N` values each, v[g][j].
template <int G, int N>
__device__ __forceinline__ void afp_lane_sums(const float (&v)[G][N], float scale, float rev, float& sum, float& sum_q) {
    float s[G], sq[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        s[g] = fabsf(v[g][0]); sq[g] = fabsf(__fmul_rn(round_away(__fmul_rn(v[g][0], scale)), rev));
#pragma unroll
        for (int j = 1; j < N; j++) {
            s[g] = __fadd_rn(s[g], fabsf(v[g][j]));
            sq[g] = __fadd_rn(sq[g], fabsf(__fmul_rn(round_away(__fmul_rn(v[g][j], scale)), rev)));
        }
    }
    if (G == 2) { sum = __fadd_rn(s[0], s[1]); sum_q = __fadd_rn(sq[0], sq[1]); }
    else { sum = __fadd_rn(__fadd_rn(s[0], s[1]), __fadd_rn(s[2], s[3])); sum_q = __fadd_rn(__fadd_rn(sq[0], sq[1]), __fadd_rn(sq[2], sq[3])); }
}
// QEM / QEM_BP (afp_sgd_kernel.h:31-104): log2(1 + relative loss of the magnitude sum under 8 bits)
template <int K>
__device__ __noinline__ float afp_qem(V8f x, float max_val, unsigned wmask) {
    constexpr int TS = K / 8;
    const float scale = afp_scale(8, max_val), rev = __fdiv_rn(1.f, scale);
    float sum, sum_q;
    if (K == 128) {
        const float v[2][4] = {{x.x[0], x.x[2], x.x[4], x.x[6]}, {x.x[1], x.x[3], x.x[5], x.x[7]}};
        afp_lane_sums<2, 4>(v, scale, rev, sum, sum_q);
    } else {
        const float v[4][2] = {{x.x[0], x.x[2]}, {x.x[4], x.x[6]}, {x.x[1], x.x[3]}, {x.x[5], x.x[7]}};
        afp_lane_sums<4, 2>(v, scale, rev, sum, sum_q);
    }
    sum = worker_sum<TS>(sum, wmask); sum_q = worker_sum<TS>(sum_q, wmask);
    return log2_rounded(__fadd_rn(fabsf(__fdiv_rn(__fsub_rn(sum, sum_q), sum)), 1.f));
}
template <int K>
__device__ __noinline__ float afp_qem_back(V8f p, V8f q, float lam, float ruv, float max_val, unsigned wmask) {
    constexpr int TS = K / 8;
    const float scale = afp_scale(8, max_val), rev = __fdiv_rn(1.f, scale);
    float sum, sum_q;
    if (K == 128) {
        const float v[2][10] = {{p.x[0], p.x[2], p.x[4], p.x[6], q.x[0], q.x[2], q.x[4], q.x[6], lam, ruv},
                                {p.x[1], p.x[3], p.x[5], p.x[7], q.x[1], q.x[3], q.x[5], q.x[7], lam, ruv}};
        afp_lane_sums<2, 10>(v, scale, rev, sum, sum_q);
    } else {
        const float v[4][6] = {{p.x[0], p.x[2], q.x[0], q.x[2], lam, ruv}, {p.x[4], p.x[6], q.x[4], q.x[6], lam, ruv},
                               {p.x[1], p.x[3], q.x[1], q.x[3], lam, ruv}, {p.x[5], p.x[7], q.x[5], q.x[7], lam, ruv}};
        afp_lane_sums<4, 6>(v, scale, rev, sum, sum_q);
    }
    sum = worker_sum<TS>(sum, wmask); sum_q = worker_sum<TS>(sum_q, wmask);
    return log2_rounded(__fadd_rn(fabsf(__fdiv_rn(__fsub_rn(sum, sum_q), sum)), 1.f));
}
// QPA (afp_sgd_kernel.h:106-125) and the bookkeeping around each call (196-206)
__device__ __noinline__ AfpSide afp_requantize(AfpSide s, float diff, float range, long long cur, int epoch, int init_threshold) {
    const float threshold = 0.0005, alpha = 0.04, beta = 0.1, delta = 100, gamma = 2;
    if (cur == 0) s.mov_avg = range;
    const float prev = s.mov_avg;
    s.n = diff <= threshold ? 8 : 16;
    s.scale = afp_scale(s.n, range);
    s.mov_avg = __fmaf_rn(alpha, range, __fmul_rn(__fsub_rn(1.0f, alpha), prev));
    const float i1 = __fmul_rn(__fmul_rn(delta, diff), diff), i2 = fabsf(__fsub_rn(s.mov_avg, prev));
    int itv = __float2int_rz(__fsub_rn(__fdiv_rn(beta, fmaxf(i1, i2)), gamma));     // saturates; NaN -> 0
    if (epoch == 0 && cur < init_threshold) itv = 1;
    s.next += itv;
    return s;
}
__device__ __forceinline__ float abs_max8(const V8f& x) {
    float m = fabsf(x.x[0]);
#pragma unroll
    for (int t = 1; t < 8; t++) m = fmaxf(m, fabsf(x.x[t]));
    return m;
}

template <int K>
__device__ __forceinline__ void afp_update(const Consts& c, AfpState& st, float r, V8f& p, V8f& q, unsigned wmask) {
    constexpr int TS = K / 8;
    const long long cur = st.cur;
    float pmax = 0.f, qmax = 0.f;
    const bool need_back = cur == st.back.next;
    if (cur == st.user.next || need_back) pmax = worker_max<TS>(abs_max8(p), wmask);
    if (cur == st.item.next || need_back) qmax = worker_max<TS>(abs_max8(q), wmask);
    if (cur == st.user.next) st.user = afp_requantize(st.user, afp_qem<K>(p, pmax, wmask), pmax, cur, c.afp_epoch, c.afp_init_threshold);
    if (cur == st.item.next) st.item = afp_requantize(st.item, afp_qem<K>(q, qmax, wmask), qmax, cur, c.afp_epoch, c.afp_init_threshold);
    const float pred = (st.user.n == 8 && st.item.n == 8) ? forward_int8<TS>(p, q, st.user.scale, st.item.scale, wmask)
                                                          : forward_half<K>(p, q, st.user.scale, st.item.scale, wmask);
    const float ruv = __fsub_rn(r, pred);
    if (need_back) {
        const float range = fmaxf(fmaxf(fmaxf(pmax, qmax), fabsf(c.lam)), fabsf(ruv));
        st.back = afp_requantize(st.back, afp_qem_back<K>(p, q, c.lam, ruv, range, wmask), range, cur, c.afp_epoch, c.afp_init_threshold);
    }
    V8f gp, gq;
    if (st.back.n == 8) backward_int8(p, q, ruv, -c.lam, st.back.scale, gp, gq);
    else backward_half(p, q, ruv, -c.lam, st.back.scale, gp, gq);
    p = step(c.lr, gp, p); q = step(c.lr, gq, q);
    st.cur = cur + 1;
}

// One update.  p_raw / q_raw are the row slices in their storage precision; both are replaced by the
// updated values.  Statistics go to `acc` when the rating is sampled.
template <int K, int KIND, int UM, int IM, bool STATS>
__device__ __forceinline__ void update_one(const Consts& c, float r, uint32_t uc, uint32_t ic, Raw<UM>& p_raw, Raw<IM>& q_raw,
                                           bool sampled, Sample& smp, AfpState& afp, unsigned wmask) {
    constexpr int TS = K / 8;
    if (STATS) { smp.user = false; smp.item = false; }
    if constexpr (KIND == KIND_MPT) {
        const V8f p = as_v8f(p_raw), q = as_v8f(q_raw);
        const V8h ph = narrow(p), qh = narrow(q);
        const __half dot = worker_sum<TS>(pair_partial(ph, qh), wmask);
        const __half2 e = __half2half2(__hmul_rn(c.mpt_scale, __hsub_rn(__float2half_rn(r), dot)));
        const V8f gp = widen(grad(e, qh, c.mpt_lam, ph)), gq = widen(grad(e, ph, c.mpt_lam, qh));
        V8f po, qo;
        const float2 lr2 = make_float2(c.lr, c.lr), rev2 = make_float2(c.mpt_rev, c.mpt_rev);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            set_pr(po, j, __ffma2_rn(lr2, __fmul2_rn(rev2, pr(gp, j)), pr(p, j)));
            set_pr(qo, j, __ffma2_rn(lr2, __fmul2_rn(rev2, pr(gq, j)), pr(q, j)));
        }
        put(p_raw, po); put(q_raw, qo);
    } else if constexpr (KIND == KIND_MUPPET) {
        V8f p = as_v8f(p_raw), q = as_v8f(q_raw);
        muppet_update<K>(c, r, p, q, smp.gp, smp.gq, wmask);
        put(p_raw, p); put(q_raw, q);
        if (STATS && sampled && c.bits != 32) smp.user = true;
    } else if constexpr (KIND == KIND_AFP) {
        V8f p = as_v8f(p_raw), q = as_v8f(q_raw);
        afp_update<K>(c, afp, r, p, q, wmask);
        put(p_raw, p); put(q_raw, q);
    } else if constexpr (KIND == KIND_MEMQUANT) {
        const V8f p = widen(as_v8h(p_raw)), q = widen(as_v8h(q_raw));
        const float part = (K == 128) ? chain_partial_k128(p, q) : pair_partial(p, q);
        const float e = __fsub_rn(r, worker_sum<TS>(part, wmask));
        put(p_raw, narrow(step(c.lr, grad(e, q, c.lam, p), p)));
        put(q_raw, narrow(step(c.lr, grad(e, p, c.lam, q), q)));
    } else {
        const bool uf = is_f32<UM>(uc), itf = is_f32<IM>(ic);
        auto both_half = [&]() {
            const V8h p = as_v8h(p_raw), q = as_v8h(q_raw);
            const __half dot = worker_sum<TS>(pair_partial(p, q), wmask);
            const __half2 e = __half2half2(__hsub_rn(__float2half_rn(r), dot));
            const V8h gp = grad(e, q, c.lam_h, p), gq = grad(e, p, c.lam_h, q);
            put(p_raw, step(c.lr_h, gp, p));
            put(q_raw, step(c.lr_h, gq, q));
            if (STATS && sampled) { smp.gp = widen(gp); smp.gq = widen(gq); smp.user = true; smp.item = true; }
        };
        auto some_f32 = [&]() {
            const V8f p = uf ? as_v8f(p_raw) : widen(as_v8h(p_raw));
            const V8f q = itf ? as_v8f(q_raw) : widen(as_v8h(q_raw));
            const float e = __fsub_rn(r, worker_sum<TS>(pair_partial(p, q), wmask));
            const V8f gp = grad(e, q, c.lam, p), gq = grad(e, p, c.lam, q);
            const V8f po = step(c.lr, gp, p), qo = step(c.lr, gq, q);
            if (uf) put(p_raw, po); else put(p_raw, narrow(po));
            if (itf) put(q_raw, qo); else put(q_raw, narrow(qo));
            if (STATS && sampled) { smp.gp = gp; smp.gq = gq; smp.user = !uf; smp.item = !itf; }
        };
        if constexpr (UM == ROWS_HALF && IM == ROWS_HALF) both_half();
        else if constexpr (UM != ROWS_DYN && IM != ROWS_DYN) some_f32();
        else { if (!uf && !itf) both_half(); else some_f32(); }
    }
}

// ---- asynchronous row copies (global -> the worker's shared-memory rings) ----------------------
// Rows are fetched with cp.async, not with loads into registers: a register load ties the wait for
// an old row to every younger load that shares its scoreboard, which exposes one full memory
// latency per rating; copy groups complete in order, so waiting for the group of rating j leaves
// the copies of ratings j+1 .. j+D in flight.
__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Slot layout = row layout: the first 16 bytes of every lane, then (fp32 rows) the second 16 bytes of
// every lane (layout.cuh), so that neither the 128-bit shared-memory accesses of neighbouring lanes collide
// on a bank nor the global accesses of a worker touch partial sectors.
template <int K, int MODE>
__device__ __forceinline__ void cp_row(unsigned char* slot, const Arena& A, uint32_t code, int m) {
    const uint32_t row = code & kIdMask;
    if (is_f32<MODE>(code)) {
        const unsigned char* g = reinterpret_cast<const unsigned char*>(A.f32 + (size_t)row * K) + 16 * m;
        cp16(slot + 16 * m, g);
        if constexpr (MODE != ROWS_HALF) cp16(slot + 2 * K + 16 * m, g + 2 * K);       // second half of the row
    } else {
        cp16(slot + 16 * m, reinterpret_cast<const unsigned char*>(A.f16 + (size_t)row * K) + 16 * m);
    }
}
template <int K, int MODE>
__device__ __forceinline__ Raw<MODE> lds_row(const unsigned char* slot, uint32_t code, int m) {
    Raw<MODE> r;
    r.a = *reinterpret_cast<const uint4*>(slot + 16 * m);
    if constexpr (MODE != ROWS_HALF) {
        if (is_f32<MODE>(code)) r.b = *reinterpret_cast<const uint4*>(slot + 2 * K + 16 * m);
    }
    return r;
}

// One rating as the worker's lanes read it from shared memory (one 128-bit broadcast load).
constexpr uint32_t F_VALID = 1u;    // there is a rating at this position
constexpr uint32_t F_UDUP = 2u;     // its user also occurs among the NS ratings before it: read the row at use
constexpr uint32_t F_RS = 4u;       // its item differs from the item of the rating before it (a run starts)
constexpr uint32_t F_IDUP = 8u;     // run start whose item also occurs among the NS ratings before it

constexpr int kSpan = 8;            // consecutive chunks handed out together (the longest run of one ticket)

// Shared memory of one worker: two chunks of records, then the user ring, then the item ring.  A ring
// slot is as large as the widest row its side can hold in this launch.
template <int K, int UM, int IM, int NS, int NSI> struct WorkerSmem {
    static constexpr int TS = K / 8;
    static constexpr int kURowBytes = K * (UM == ROWS_HALF ? 2 : 4);
    static constexpr int kIRowBytes = K * (IM == ROWS_HALF ? 2 : 4);
    static constexpr int kRecBytes = 2 * TS * 16;
    static constexpr int kBytes = kRecBytes + NS * kURowBytes + NSI * kIRowBytes;
};

// NS / NSI: slots of the user / item ring.  User rows are requested D ratings ahead, item rows DI
// ratings ahead (DI <= D <= NS-1, DI <= NSI-1).  The lead is kept as short as the memory latency allows: a row that another
// worker updates between the request and the write-back loses that update, and the chance of that
// grows with the lead.
template <int K, int KIND, int UM, int IM, bool STATS, int NS, int NSI, int D, int DI>
__global__ void __launch_bounds__(256, (UM == ROWS_HALF && IM == ROWS_HALF && !STATS) ? 4 : ((UM == ROWS_DYN || STATS || KIND == KIND_AFP) ? 2 : 3)) train_kernel(const KernelArgs a) {
    using SM = WorkerSmem<K, UM, IM, NS, NSI>;
    constexpr int TS = SM::TS;                     // lanes per worker = ratings per chunk
    static_assert(TS % NS == 0, "the ring must divide the chunk");
    static_assert(DI >= 1 && DI <= D && D == NS - 1 && DI <= NSI - 1 && NS % NSI == 0, "leads must fit the rings");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int m = lane % TS;
    const unsigned wmask = (TS == 32) ? 0xffffffffu : (((1u << TS) - 1u) << (lane - m));
    const uint64_t worker = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) / TS;
    const uint64_t W = a.workers;
    const uint64_t nchunks = (a.s.n + TS - 1) / TS;

    unsigned char* const mine = smem_raw + (size_t)(threadIdx.x / TS) * SM::kBytes;
    uint4* const recs = reinterpret_cast<uint4*>(mine);                  // [2][TS]
    unsigned char* const uring = mine + SM::kRecBytes;                    // [NS][kURowBytes]
    unsigned char* const iring = uring + NS * SM::kURowBytes;             // [NSI][kIRowBytes]

    Consts c;
    c.lr = a.lr; c.lam = a.lam;
    c.lr_h = __half2half2(__float2half_rn(a.lr));
    c.lam_h = __half2half2(__float2half_rn(a.lam));
    c.mpt_scale = __float2half_rn(1000.0f);
    c.mpt_lam = __half2half2(__float2half_rn(__fmul_rn(a.lam, 1000.0f)));
    c.mpt_rev = __fdiv_rn(1.0f, 1000.0f);
    c.bits = a.bits;
    c.afp_epoch = a.epoch;
    c.afp_init_threshold = (int)((float)((a.s.n + W - 1) / W) / 10.0f);
    // only the mixed-precision mode reads the precision bit of an id
    constexpr uint32_t kKeep = (UM == ROWS_DYN || IM == ROWS_DYN) ? 0xffffffffu : (kIdMask | kHotBit);

    if (worker >= W) return;

    // ---- which chunks this worker processes ----
    // Runs of consecutive chunks: first the static runs [worker*kSpan, +kSpan) and [(worker+W)*kSpan,
    // +kSpan), then runs handed out by the shared counter, which counts chunks beyond the static part.
    // A dynamic run is kSpan chunks long while plenty of work is left and shrinks to a single chunk as
    // the counter nears the end (its length is what is left, as seen at the previous ticket, divided by
    // twice the number of workers), so that the workers finish within about one chunk of each other.  A
    // ticket is requested one run before it is needed and stays in lane 0 until then, so the launch
    // neither waits for the counter nor depends on all blocks being resident.
    const uint64_t static_chunks = 2 * W * kSpan;
    const uint64_t dyn_chunks = nchunks > static_chunks ? nchunks - static_chunks : 0;
    auto run_length = [&](unsigned long long seen) -> unsigned {
        const uint64_t left = dyn_chunks > seen ? dyn_chunks - seen : 0;
        const uint64_t g = left / (2 * W);
        return g >= (uint64_t)kSpan ? (unsigned)kSpan : (g < 1 ? 1u : (unsigned)g);
    };
    uint64_t run_cur = worker * kSpan, run_next = (worker + W) * kSpan;
    unsigned len_cur = kSpan, len_next = kSpan, kin = 0;
    unsigned tlen = run_length(0);
    unsigned long long ticket = (m == 0) ? atomicAdd(a.next_chunk, (unsigned long long)tlen) : 0ull;
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.zero_counter = 0ull;      // the counter of the launch after next
    auto next_chunk_id = [&]() -> uint64_t {
        if (run_cur >= nchunks) return ~0ull;
        const uint64_t ci = run_cur + kin;
        if (++kin == len_cur) {
            kin = 0;
            run_cur = run_next; len_cur = len_next;
            const unsigned lo = __shfl_sync(wmask, (unsigned)ticket, 0, TS), hi = __shfl_sync(wmask, (unsigned)(ticket >> 32), 0, TS);
            len_next = __shfl_sync(wmask, tlen, 0, TS);
            run_next = static_chunks + (((uint64_t)hi << 32) | lo);
            if (m == 0) { tlen = run_length(ticket); ticket = atomicAdd(a.next_chunk, (unsigned long long)tlen); }
        }
        return ci < nchunks ? ci : ~0ull;
    };

    // ---- chunk pipeline: global loads (registers) -> flags -> records in shared memory -> use ----
    struct Loaded { float r; uint32_t u, i; int cnt; uint64_t base; };
    auto fetch_chunk = [&](uint64_t ci) {
        Loaded k; k.r = 0.f; k.u = kNoRow; k.i = kNoRow; k.cnt = 0; k.base = 0;
        if (ci < nchunks) {
            k.base = ci * TS;
            const uint64_t left = a.s.n - k.base;
            k.cnt = left < (uint64_t)TS ? (int)left : TS;
            if (m < k.cnt) {
                k.r = __ldg(a.s.r + k.base + m);
                k.u = __ldg(a.s.u + k.base + m) & kKeep;
                k.i = __ldg(a.s.i + k.base + m) & kKeep;
            }
        }
        return k;
    };
    uint32_t prev_u = kNoRow, prev_i = kNoRow;        // lane m: rating m of the chunk before `inflight`
    Loaded inflight = fetch_chunk(next_chunk_id());
    uint64_t base0 = 0, base1 = 0;              // stream position of the first rating of each buffer
    // Turns `inflight` into records in buffer `b` and starts loading the chunk after it.
    auto publish = [&](int b) {
        bool udup = false, idup = false, rs = false;
#pragma unroll
        for (int d = 1; d <= NS; d++) {
            // the rating d places earlier: lane m-d of this chunk, or lane m-d+TS of the previous one;
            // the SOURCE lane knows which of its two values a reader d lanes further on wants
            const bool from_this = m < TS - d;
            const uint32_t su = __shfl_sync(wmask, from_this ? inflight.u : prev_u, (m - d) & (TS - 1), TS);
            const uint32_t si = __shfl_sync(wmask, from_this ? inflight.i : prev_i, (m - d) & (TS - 1), TS);
            udup |= su == inflight.u;
            if (d == 1) rs = si != inflight.i; else idup |= si == inflight.i;
        }
        uint32_t f = 0;
        if (m < inflight.cnt) f = F_VALID | (udup ? F_UDUP : 0u) | (rs ? F_RS : 0u) | ((rs && idup) ? F_IDUP : 0u);
        recs[b * TS + m] = make_uint4(f, inflight.i, inflight.u, __float_as_uint(inflight.r));
        if (b) base1 = inflight.base; else base0 = inflight.base;
        prev_u = inflight.u; prev_i = inflight.i;
        inflight = (inflight.cnt > 0) ? fetch_chunk(next_chunk_id()) : inflight;
        __syncwarp(wmask);
    };
    publish(0);
    publish(1);

    unsigned hot_seen = worker;                       // counts the ratings of marked users this worker has met
    const unsigned hot_mask = (1u << a.hot_user_shift) - 1u;
    // item row of the current run
    uint32_t cur_ic = kNoRow;
    Raw<IM> q;

    // item-side statistics of the current run of equal item groups
    V8f gq_acc; float nq_acc = 0.f; uint32_t acc_group = kNoRow;
#pragma unroll
    for (int t = 0; t < 8; t++) gq_acc.x[t] = 0.f;
    // this block's private set of accumulators (fewer workers per address, less serialisation)
    const size_t my_set = STATS ? (size_t)(blockIdx.x % (unsigned)a.st.copies) * a.st.copy_stride : 0;
    float* const gsum_p = a.st.gsum_p + my_set; float* const gsum_q = a.st.gsum_q + my_set;
    float* const nsum_p = a.st.nsum_p + my_set; float* const nsum_q = a.st.nsum_q + my_set;
    auto flush_item_stats = [&]() {
        if (acc_group != kNoRow) {
            red_add8(gsum_q + (size_t)acc_group * K + 8 * m, gq_acc);
            if (m == 0) atomicAdd(nsum_q + acc_group, nq_acc);
        }
    };
    auto record = [&](const Sample& smp, uint32_t uc, uint32_t ic) {
        if constexpr (KIND == KIND_MUPPET || KIND == KIND_SWITCH) {
            // muppet_sgd_kernel.h:266-285, sgd_kernel.h:266-285: the squared norm of both gradients goes to the
            // worker's running sum, the element-wise sum of both gradients to k shared accumulators
            if (smp.user) {
                const float n = worker_sum<TS>(muppet_norm_partial<K>(smp.gp, smp.gq), wmask);
                V8f both;
#pragma unroll
                for (int t = 0; t < 8; t++) both.x[t] = __fadd_rn(smp.gp.x[t], smp.gq.x[t]);
                red_add8(gsum_p + 8 * m, both);
                nq_acc = __fadd_rn(nq_acc, n);
            }
            return;
        }
        if (smp.user) {
            const uint32_t g = a.st.ugroup[uc & kIdMask];
            const float n = worker_sum<TS>(pair_partial(smp.gp, smp.gp), wmask);
            red_add8(gsum_p + (size_t)g * K + 8 * m, smp.gp);
            if (m == 0) atomicAdd(nsum_p + g, n);
        }
        if (smp.item) {
            const uint32_t g = a.st.igroup[ic & kIdMask];
            const float n = worker_sum<TS>(pair_partial(smp.gq, smp.gq), wmask);
            if (g != acc_group) {
                flush_item_stats();
                acc_group = g; nq_acc = 0.f;
#pragma unroll
                for (int t = 0; t < 8; t++) gq_acc.x[t] = 0.f;
            }
#pragma unroll
            for (int t = 0; t < 8; t++) gq_acc.x[t] = __fadd_rn(gq_acc.x[t], smp.gq.x[t]);
            nq_acc = __fadd_rn(nq_acc, n);
        }
    };
    Sample smp;
    AfpState afp;
    afp.user = AfpSide{8, 1.f, 0.f, 0}; afp.item = afp.user; afp.back = afp.user; afp.cur = 0;

    // requests the user row of the rating with record `rx` / the item row of the rating whose first
    // two record words are `ri`, into ring slot `slot`
    auto request_user = [&](const uint4& rx, int slot) {
        if ((rx.x & (F_VALID | F_UDUP)) == F_VALID) cp_row<K, UM>(uring + slot * SM::kURowBytes, a.P, rx.z, m);
    };
    auto request_item = [&](const uint2& ri, int slot) {
        if ((ri.x & (F_VALID | F_RS | F_IDUP)) == (F_VALID | F_RS)) cp_row<K, IM>(iring + slot * SM::kIRowBytes, a.Q, ri.y, m);
    };
    // Copy groups complete in order.  Every iteration commits two: first the item row of the rating
    // DI ahead, then the user row of the rating D ahead.  When rating j is used, the groups younger
    // than its item row's are 2*DI-1 and those younger than its user row's are 2*(D-1); waiting for
    // exactly that many to remain pending leaves every younger copy in flight.
    constexpr int kPendUser = 2 * (D - 1);
    constexpr int kPendItem = (2 * DI - 1 < kPendUser) ? 2 * DI - 1 : kPendUser;
    // The records of the ratings j .. j+D live in a register queue indexed like the user ring (the
    // record of rating x in slot x mod NS): each record is read from shared memory once, D ratings
    // before its rating is processed, and serves the user request, the item request and the update.
    uint4 rq[NS];
    // prologue: the groups of the iterations -D .. -1
#pragma unroll
    for (int t = 0; t < D; t++) {
        rq[t] = recs[t];
        if (t - (D - DI) >= 0) request_item(make_uint2(rq[t - (D - DI)].x, rq[t - (D - DI)].y), (t - (D - DI)) & (NSI - 1));
        cp_commit();
        request_user(rq[t], t);
        cp_commit();
    }

    int cb = 0;                                     // buffer of the chunk in use
    for (;;) {
        const uint4* const rc = recs + cb * TS;
        const uint4* const rn = recs + (cb ^ 1) * TS;
        bool more = true;
#pragma unroll 1
        for (int jb = 0; jb < TS && more; jb += NS) {
#pragma unroll
            for (int t = 0; t < NS; t++) {
                const int j = jb + t;
                {   // the record of the rating D ahead takes the slot of the rating processed last
                    const int x = j + D;
                    rq[(t + D) & (NS - 1)] = (x < TS) ? rc[x] : rn[x - TS];
                }
                const uint4 rec = rq[t];
                if (!(rec.x & F_VALID)) { more = false; break; }
                const uint32_t uc = rec.z, ic = rec.y;
                const float r = __uint_as_float(rec.w);
                const bool sampled = STATS && ((cb ? base1 : base0) + j >= a.st.first_sample_pos);
                if (rec.x & F_RS) {
                    cp_wait<kPendItem>();
                    if (cur_ic != kNoRow) st_row<K, IM>(a.Q, cur_ic, m, q);
                    if (rec.x & F_IDUP) q = ld_row<K, IM>(a.Q, ic, m);
                    else q = lds_row<K, IM>(iring + (t & (NSI - 1)) * SM::kIRowBytes, ic, m);
                    cur_ic = ic;
                } else {
                    cp_wait<kPendUser>();
                }
                Raw<UM> p;
                if (rec.x & F_UDUP) p = ld_row<K, UM>(a.P, uc, m);
                else p = lds_row<K, UM>(uring + t * SM::kURowBytes, uc, m);
                // request the user row of the rating D ahead and the item row of the rating DI ahead,
                // into slots whose previous contents have been consumed
                {
                    const uint4& ri = rq[(t + DI) & (NS - 1)];
                    request_item(make_uint2(ri.x, ri.y), (t + DI) & (NSI - 1));
                    cp_commit();
                    request_user(rq[(t + D) & (NS - 1)], (t + D) & (NS - 1));
                    cp_commit();
                }
                const Raw<UM> p_before = p;
                update_one<K, KIND, UM, IM, STATS>(c, r, uc, ic, p, q, sampled, smp, afp, wmask);
                if (a.add_user_delta) {
                    // A marked user (see the set-up): every 2^shift-th update of a marked row that this worker meets
                    // is written back; the others are dropped.
                    bool keep = true;
                    if (uc & kHotBit) keep = ((++hot_seen) & hot_mask) == 0u;
                    if (keep) add_row_delta<K, UM>(a.P, uc, m, p, p_before);
                } else {
                    st_row<K, UM>(a.P, uc, m, p);
                }
                if (STATS && sampled) record(smp, uc, ic);
            }
        }
        if (!more) break;
        __syncwarp(wmask);           // every lane has read this buffer's records
        publish(cb);                 // the chunk after next takes the buffer of the finished one
        cb ^= 1;
    }
    cp_wait<0>();
    if (cur_ic != kNoRow) st_row<K, IM>(a.Q, cur_ic, m, q);
    if (STATS) {
        if constexpr (KIND == KIND_MUPPET || KIND == KIND_SWITCH) { if (m == 0) atomicAdd(nsum_p, nq_acc); }
        else flush_item_stats();
    }
}

__global__ void reduce_stats_kernel(float* sets, int copies, size_t stride, size_t n) {
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (size_t)gridDim.x * blockDim.x) {
        float acc = sets[j];
        for (int c = 1; c < copies; c++) acc = __fadd_rn(acc, sets[(size_t)c * stride + j]);
        sets[j] = acc;
    }
}

template <int K, int KIND, int UM, int IM, bool STATS, int NS, int NSI, int D, int DI>
cudaError_t launch_ns(KernelArgs a, unsigned warps_per_sm, unsigned workers, cudaStream_t st, LaunchShape* shape, bool dry) {
    constexpr int TS = K / 8;
    constexpr int kPerWarp = 32 / TS;
    using SM = WorkerSmem<K, UM, IM, NS, NSI>;
    auto kern = train_kernel<K, KIND, UM, IM, STATS, NS, NSI, D, DI>;
    // the most dynamic shared memory a launch of this instantiation can ask for: a block of 8 warps
    constexpr size_t kSmemMax = (size_t)8 * kPerWarp * SM::kBytes;
    static LaunchCache cache;                    // one per instantiation; see launch_cache.h
    int grid, block;
    const unsigned warps = (workers + kPerWarp - 1) / kPerWarp;
    if (workers <= 1) a.add_user_delta = 0;      // a single worker has nobody to race with: plain stores
    unsigned blocks_per_sm = 1, warps_per_block = warps;
    if (warps > 8) {
        // the same number of warps on every SM, in blocks of at most 8 warps
        blocks_per_sm = (warps_per_sm + 7) / 8;
        warps_per_block = (warps_per_sm + blocks_per_sm - 1) / blocks_per_sm;
    }
    block = (int)(32 * warps_per_block);
    const size_t smem = (size_t)warps_per_block * kPerWarp * SM::kBytes;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    int fit = 0;
    const int rc = cache.lookup(
        dev, block, smem, kSmemMax,
        [&](size_t bytes) { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); },
        [&](int blk, size_t sm, int* f) { return (int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(f, kern, blk, sm); }, &fit);
    if (rc != 0) return (cudaError_t)rc;
    if (fit < 1) return cudaErrorLaunchOutOfResources;
    size_t smem_used = smem;
    if (warps > 8 && blocks_per_sm > (unsigned)fit && warps_per_block < 8) {
        // The SM cannot hold as many blocks as the even split asked for: blocks of the full eight warps then put
        // more warps on it (42 warps wanted: six blocks of seven, of which four fit = 28 warps; four blocks of
        // eight = 32).
        int fit8 = 0;
        const size_t smem8 = (size_t)8 * kPerWarp * SM::kBytes;
        const int rc8 = cache.lookup(
            dev, 256, smem8, kSmemMax,
            [&](size_t bytes) { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); },
            [&](int blk, size_t sm, int* f) { return (int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(f, kern, blk, sm); }, &fit8);
        if (rc8 != 0) return (cudaError_t)rc8;
        if (fit8 * 8 > fit * (int)warps_per_block) {
            warps_per_block = 8; block = 256; smem_used = smem8; fit = fit8;
            blocks_per_sm = (warps_per_sm + 7) / 8;
        }
    }
    if (warps <= 8) {
        // a single block (deterministic runs, tiny worker counts) uses exactly the requested workers
        grid = 1;
        a.workers = workers;
    } else {
        // no more blocks than the SM can hold at once (registers, shared memory)
        if (blocks_per_sm > (unsigned)fit) blocks_per_sm = (unsigned)fit;
        grid = (int)((unsigned)sm_count() * blocks_per_sm);
        a.workers = (unsigned)grid * warps_per_block * kPerWarp;
    }
    if (!dry) kern<<<grid, block, smem_used, st>>>(a);      // a dry call stops here: the function is loaded and configured
    if (shape) { shape->grid = grid; shape->block = block; shape->smem = smem_used; shape->workers = a.workers; }
    return cudaGetLastError();
}

template <int K, int KIND, int UM, int IM, bool STATS>
cudaError_t launch_one(const KernelArgs& args, unsigned workers, cudaStream_t st, LaunchShape* shape, bool dry) {
    constexpr int TS = K / 8;
    constexpr int kPerWarp = 32 / TS;
    if (workers < 1) workers = 1;
    // more workers than can ever be resident at once (64 warps per SM) only add launch overhead
    const unsigned resident_cap = (unsigned)sm_count() * 64u * kPerWarp;
    if (workers > resident_cap) workers = resident_cap;
    const unsigned warps = (workers + kPerWarp - 1) / kPerWarp;
    const unsigned sms = (unsigned)sm_count();
    const unsigned per_sm = warps <= 8 ? warps : (warps + sms - 1) / sms;
    // User ring of four slots (rows requested three ratings ahead), item ring of two (one rating ahead).
    // Requesting user rows seven ahead was measured on the 100M- and the 252M-rating configuration and
    // changed nothing: the kernel is not waiting for memory.  With fp32 rows the slots are twice as large
    // and the occupancy query trims the number of blocks per SM accordingly.
    // (Requesting fp32 item rows two ratings ahead, into an item ring of four slots, was measured as well and
    // changed nothing either - 13.99 against 14.06 ms per promoted epoch on the 100M-rating configuration.)
    return launch_ns<K, KIND, UM, IM, STATS, 4, 2, 3, 1>(args, per_sm, workers, st, shape, dry);
}

template <int K, int KIND, int UM, int IM>
cudaError_t launch_st(const KernelArgs& a, bool stats, unsigned workers, cudaStream_t st, LaunchShape* sh, bool dry) {
    return stats ? launch_one<K, KIND, UM, IM, true>(a, workers, st, sh, dry) : launch_one<K, KIND, UM, IM, false>(a, workers, st, sh, dry);
}

template <int K>
cudaError_t launch_k(TrainKind kind, const KernelArgs& a, bool stats, RowClass cls, unsigned workers, cudaStream_t st, LaunchShape* sh, bool dry) {
    switch (kind) {
        case KIND_MIXED:
            switch (cls) {
                case ROWCLASS_HH: return launch_st<K, KIND_MIXED, ROWS_HALF, ROWS_HALF>(a, stats, workers, st, sh, dry);
                case ROWCLASS_HF: return launch_st<K, KIND_MIXED, ROWS_HALF, ROWS_F32>(a, stats, workers, st, sh, dry);
                case ROWCLASS_FH: return launch_st<K, KIND_MIXED, ROWS_F32, ROWS_HALF>(a, stats, workers, st, sh, dry);
                case ROWCLASS_FF: return launch_st<K, KIND_MIXED, ROWS_F32, ROWS_F32>(a, stats, workers, st, sh, dry);
                case ROWCLASS_ANY: return launch_st<K, KIND_MIXED, ROWS_DYN, ROWS_DYN>(a, stats, workers, st, sh, dry);
            }
            return cudaErrorInvalidValue;
        case KIND_FP32: return launch_one<K, KIND_FP32, ROWS_F32, ROWS_F32, false>(a, workers, st, sh, dry);
        case KIND_MPT: return launch_one<K, KIND_MPT, ROWS_F32, ROWS_F32, false>(a, workers, st, sh, dry);
        case KIND_MEMQUANT: return launch_one<K, KIND_MEMQUANT, ROWS_HALF, ROWS_HALF, false>(a, workers, st, sh, dry);
        case KIND_AFP: return launch_one<K, KIND_AFP, ROWS_F32, ROWS_F32, false>(a, workers, st, sh, dry);
        case KIND_SWITCH: return launch_st<K, KIND_SWITCH, ROWS_HALF, ROWS_HALF>(a, stats, workers, st, sh, dry);
        case KIND_MUPPET: return launch_st<K, KIND_MUPPET, ROWS_F32, ROWS_F32>(a, stats, workers, st, sh, dry);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_reduce_stats(float* sets, int copies, size_t copy_stride, size_t floats_per_set, cudaStream_t st) {
    if (copies <= 1 || floats_per_set == 0) return cudaSuccess;
    const int grid = (int)((floats_per_set + 255) / 256);
    reduce_stats_kernel<<<grid, 256, 0, st>>>(sets, copies, copy_stride, floats_per_set);
    return cudaGetLastError();
}

int sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    int& v = sms[dev & 63];
    if (!v) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 1;
}

cudaError_t launch_train(int K, TrainKind kind, const Stream& s, Arena P, Arena Q, float lr, float lam,
                         const SampleStats* stats, RowClass row_class, unsigned workers, WorkCounters* counters,
                         int bits, int epoch, bool add_user_delta, unsigned hot_user_shift, cudaStream_t st, LaunchShape* shape) {
    KernelArgs a;
    a.hot_user_shift = hot_user_shift;
    a.add_user_delta = add_user_delta ? 1 : 0;
    a.s = s; a.P = P; a.Q = Q; a.lr = lr; a.lam = lam; a.workers = workers; a.bits = bits; a.epoch = epoch;
    if (stats) a.st = *stats;
    if (s.n == 0) { if (shape) *shape = LaunchShape(); return cudaSuccess; }
    if (!counters) {
        // dry call: loads the instantiation this launch would use and sets its shared-memory limit, launches nothing
        if (K == 128) return launch_k<128>(kind, a, stats != nullptr, row_class, workers, st, shape, true);
        if (K == 64) return launch_k<64>(kind, a, stats != nullptr, row_class, workers, st, shape, true);
        return cudaErrorInvalidValue;
    }
    // Launches of one engine run one after the other on its stream.  Launch number L hands out chunks
    // through counter L mod 4 and resets counter (L + 2) mod 4, which the launch after next will use and
    // which no launch in flight touches; all four start at zero.
    a.next_chunk = counters->d_slots + (counters->launches & 3);
    a.zero_counter = counters->d_slots + ((counters->launches + 2) & 3);
    counters->launches++;
    if (K == 128) return launch_k<128>(kind, a, stats != nullptr, row_class, workers, st, shape, false);
    if (K == 64) return launch_k<64>(kind, a, stats != nullptr, row_class, workers, st, shape, false);
    return cudaErrorInvalidValue;
}

}  // namespace mascot
