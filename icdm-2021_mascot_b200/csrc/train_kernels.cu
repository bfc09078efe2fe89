// Per-rating SGD update kernels for sm_100a.
//
// One "team" of T = K/4 lanes owns one rating at a time; every lane holds four consecutive
// physical elements of the user row and of the item row (one 64-bit access for binary16 storage,
// one 128-bit access for fp32 storage; layout.cuh explains the element permutation that makes this
// reproduce the reference's reduction tree).  Teams walk the rating stream in chunks of T ratings,
// grid-stride over a persistent grid: the T records of a chunk are fetched with one coalesced load
// per field (lane j keeps rating j) one chunk ahead of use and broadcast with shuffles, so the only
// dependent memory round trip per rating is the row gather itself.  Bit 31 of the stream ids says
// which arena (binary16 or fp32) a row lives in, which replaces the reference's per-rating group
// search (mascot/mascot_sgd_kernel.h:104-180) with nothing at all.
//
// The arithmetic of each precision case is the reference's, including the fused multiply-adds its
// compiled kernels execute:
//   all binary16      mascot_sgd_kernel.h:188-278     binary16 user / fp32 item  :279-342
//   fp32 / binary16   mascot_sgd_kernel.h:343-407     all fp32                   :408-443
//   (sgd/sgd_kernel.h:35-76 compiles to the same operations as the all-fp32 case)
//   MPT               mpt/mpt_sgd_kernel.h:38-91      fp16 storage (-v 7)  sgd/sgd_kernel.h:110-161
// Every operation is written with a rounding-mode intrinsic so that ptxas cannot re-associate or
// contract anything further.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "engine.h"
#include "layout.cuh"

namespace mascot {

namespace {

template <int T>
__device__ __forceinline__ float team_sum(float x, unsigned mask) {
    x = __fadd_rn(x, __shfl_xor_sync(mask, x, 1));
#pragma unroll
    for (int d = T / 2; d >= 2; d >>= 1) x = __fadd_rn(x, __shfl_xor_sync(mask, x, d));
    return x;
}

template <int T>
__device__ __forceinline__ __half team_sum(__half x, unsigned mask) {
    x = __hadd_rn(x, __shfl_xor_sync(mask, x, 1));
#pragma unroll
    for (int d = T / 2; d >= 2; d >>= 1) x = __hadd_rn(x, __shfl_xor_sync(mask, x, d));
    return x;
}

struct H4 { __half2 a, b; };          // four binary16 values, physical order
struct F4 { float x[4]; };

__device__ __forceinline__ H4 ld_h4(const __half* base, uint32_t row, int K, int tl) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(base + (size_t)row * K) + tl);
    H4 h;
    h.a = *reinterpret_cast<const __half2*>(&v.x);
    h.b = *reinterpret_cast<const __half2*>(&v.y);
    return h;
}
__device__ __forceinline__ void st_h4(__half* base, uint32_t row, int K, int tl, const H4& h) {
    uint2 v;
    v.x = *reinterpret_cast<const unsigned*>(&h.a);
    v.y = *reinterpret_cast<const unsigned*>(&h.b);
    __stcg(reinterpret_cast<uint2*>(base + (size_t)row * K) + tl, v);
}
__device__ __forceinline__ F4 ld_f4(const float* base, uint32_t row, int K, int tl) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (size_t)row * K) + tl);
    F4 f;
    f.x[0] = v.x; f.x[1] = v.y; f.x[2] = v.z; f.x[3] = v.w;
    return f;
}
__device__ __forceinline__ void st_f4(float* base, uint32_t row, int K, int tl, const F4& f) {
    __stcg(reinterpret_cast<float4*>(base + (size_t)row * K) + tl, make_float4(f.x[0], f.x[1], f.x[2], f.x[3]));
}
// Raw fetch of a user row: 16 bytes per lane for fp32 storage, 8 (in .x/.y) for binary16 storage.
template <int KIND>
__device__ __forceinline__ uint4 ld_row_raw(const Arena& A, uint32_t code, int K, int tl) {
    const uint32_t row = code & kIdMask;
    const bool f32 = (KIND == KIND_MIXED) ? ((code & kPrecBit) != 0) : (KIND == KIND_FP32 || KIND == KIND_MPT);
    if (f32) return __ldcg(reinterpret_cast<const uint4*>(A.f32 + (size_t)row * K) + tl);
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(A.f16 + (size_t)row * K) + tl);
    return make_uint4(v.x, v.y, 0u, 0u);
}
__device__ __forceinline__ F4 raw_f4(const uint4& v) {
    F4 f;
    f.x[0] = __uint_as_float(v.x); f.x[1] = __uint_as_float(v.y); f.x[2] = __uint_as_float(v.z); f.x[3] = __uint_as_float(v.w);
    return f;
}
__device__ __forceinline__ H4 raw_h4(const uint4& v) {
    H4 h;
    h.a = *reinterpret_cast<const __half2*>(&v.x);
    h.b = *reinterpret_cast<const __half2*>(&v.y);
    return h;
}

__device__ __forceinline__ F4 widen(const H4& h) {
    F4 f;
    const float2 lo = __half22float2(h.a), hi = __half22float2(h.b);
    f.x[0] = lo.x; f.x[1] = lo.y; f.x[2] = hi.x; f.x[3] = hi.y;
    return f;
}
__device__ __forceinline__ H4 narrow(const F4& f) {
    H4 h;
    h.a = __halves2half2(__float2half_rn(f.x[0]), __float2half_rn(f.x[1]));
    h.b = __halves2half2(__float2half_rn(f.x[2]), __float2half_rn(f.x[3]));
    return h;
}

// Write a cached item row back to the arena its precision selects.
template <int KIND>
__device__ __forceinline__ void st_item(const Arena& Q, uint32_t code, int K, int tl, const H4& qh, const F4& qf) {
    const uint32_t row = code & kIdMask;
    const bool f32 = (KIND == KIND_MIXED) ? ((code & kPrecBit) != 0) : (KIND == KIND_FP32 || KIND == KIND_MPT);
    if (f32) st_f4(Q.f32, row, K, tl, qf); else st_h4(Q.f16, row, K, tl, qh);
}

// lane partial of the dot product: (fma(a0,b0,a1*b1)) + (fma(a2,b2,a3*b3))
__device__ __forceinline__ float pair_partial(const F4& a, const F4& b) {
    const float f01 = __fmaf_rn(a.x[0], b.x[0], __fmul_rn(a.x[1], b.x[1]));
    const float f23 = __fmaf_rn(a.x[2], b.x[2], __fmul_rn(a.x[3], b.x[3]));
    return __fadd_rn(f01, f23);
}
// lane partial of the left-to-right product chain the fp16-storage trainer and the RMSE kernel
// use for k=128: fma(a3,b3, fma(a2,b2, fma(a0,b0, a1*b1)))
__device__ __forceinline__ float chain_partial(const F4& a, const F4& b) {
    float acc = __fmaf_rn(a.x[0], b.x[0], __fmul_rn(a.x[1], b.x[1]));
    acc = __fmaf_rn(a.x[2], b.x[2], acc);
    return __fmaf_rn(a.x[3], b.x[3], acc);
}
__device__ __forceinline__ __half pair_partial(const H4& p, const H4& q) {
    const __half2 plo = __lows2half2(p.a, p.b), phi = __highs2half2(p.a, p.b);
    const __half2 qlo = __lows2half2(q.a, q.b), qhi = __highs2half2(q.a, q.b);
    const __half2 f = __hfma2(plo, qlo, __hmul2_rn(phi, qhi));   // (f01, f23)
    return __hadd_rn(__low2half(f), __high2half(f));
}
// t = fma(e, y, -(lam*x)) element-wise
__device__ __forceinline__ F4 grad(float e, const F4& y, float lam, const F4& x) {
    F4 g;
#pragma unroll
    for (int s = 0; s < 4; s++) g.x[s] = __fmaf_rn(e, y.x[s], -__fmul_rn(lam, x.x[s]));
    return g;
}
__device__ __forceinline__ H4 grad(__half2 e, const H4& y, __half2 lam, const H4& x) {
    H4 g;
    g.a = __hfma2(e, y.a, __hneg2(__hmul2_rn(lam, x.a)));
    g.b = __hfma2(e, y.b, __hneg2(__hmul2_rn(lam, x.b)));
    return g;
}
__device__ __forceinline__ F4 step(float lr, const F4& g, const F4& x) {
    F4 o;
#pragma unroll
    for (int s = 0; s < 4; s++) o.x[s] = __fmaf_rn(lr, g.x[s], x.x[s]);
    return o;
}
__device__ __forceinline__ float sumsq_partial(const F4& g) { return pair_partial(g, g); }

// Accumulators of the sampled statistics: shared memory when they fit, else straight to global.
struct StatAcc {
    float* gs_p; float* gs_q; float* ns_p; float* ns_q;
};

template <int K, int T>
__device__ __forceinline__ void sample_side(const F4& g, float* gsum, float* nsum, uint32_t group, int tl, unsigned mask) {
    const float n = team_sum<T>(sumsq_partial(g), mask);
    if (tl == 0) atomicAdd(nsum + group, n);
    float* dst = gsum + (size_t)group * K + 4 * tl;
#pragma unroll
    for (int s = 0; s < 4; s++) atomicAdd(dst + s, g.x[s]);
}

struct KernelArgs {
    Stream s;
    Arena P, Q;
    float lr, lam;
    SampleStats st;
    int stats_in_smem;
    int deterministic;
};

// ---------------------------------------------------------------------------------------------
// Fast path for k = 128 when every row of a 32-rating chunk is stored in binary16 (the common case
// of the MASCOT variant): the warp splits into two half-warps, each walking 16 of the chunk's
// ratings on its own, so every instruction serves two ratings and a row is one 128-bit access per
// lane.  Lane m of a half-warp holds physical elements 8m..8m+7 = the four elements of reference
// lane m followed by the four of reference lane m+16; adding the two lane partials is the
// reference's shfl_down-16 step and xor 8,4,2,1 inside the half-warp finishes the same tree, so
// the arithmetic is bit-identical to the 32-lane path.  The two half-warps are independent workers
// (like two warps of the reference), hence this path is not used in deterministic mode.
// ---------------------------------------------------------------------------------------------
struct H8 { __half2 v[4]; };

__device__ __forceinline__ H8 raw_h8(const uint4& x) {
    H8 h;
    h.v[0] = *reinterpret_cast<const __half2*>(&x.x); h.v[1] = *reinterpret_cast<const __half2*>(&x.y);
    h.v[2] = *reinterpret_cast<const __half2*>(&x.z); h.v[3] = *reinterpret_cast<const __half2*>(&x.w);
    return h;
}
__device__ __forceinline__ uint4 h8_raw(const H8& h) {
    uint4 x;
    x.x = *reinterpret_cast<const unsigned*>(&h.v[0]); x.y = *reinterpret_cast<const unsigned*>(&h.v[1]);
    x.z = *reinterpret_cast<const unsigned*>(&h.v[2]); x.w = *reinterpret_cast<const unsigned*>(&h.v[3]);
    return x;
}

__device__ __forceinline__ void chunk_all_half_k128(const KernelArgs& a, float r_l, uint32_t u_l, uint32_t i_l, int cnt,
                                                    __half2 lr_h, __half2 lam_h) {
    constexpr int K = 128;
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int m = lane & 15;                     // lane inside the half-warp
    const int half_id = lane >> 4;
    const int my_cnt = min(max(cnt - 16 * half_id, 0), 16);
    const int max_cnt = min(cnt, 16);            // half-warp 0 always has at least as many ratings

    uint32_t cur_i = 0xffffffffu;
    H8 q;
    q.v[0] = q.v[1] = q.v[2] = q.v[3] = __half2half2(__ushort_as_half(0));
    uint32_t u = __shfl_sync(full, u_l, 0, 16);
    uint4 p_raw = make_uint4(0u, 0u, 0u, 0u);
    if (my_cnt > 0) p_raw = __ldcg(reinterpret_cast<const uint4*>(a.P.f16 + (size_t)u * K) + m);
    for (int j = 0; j < max_cnt; j++) {
        const bool on = j < my_cnt;
        const float r = __shfl_sync(full, r_l, j, 16);
        const uint32_t i = __shfl_sync(full, i_l, j, 16);
        const int jn = (j + 1 < 16) ? j + 1 : j;
        const uint32_t u_next = __shfl_sync(full, u_l, jn, 16);
        if (on && i != cur_i) {
            if (cur_i != 0xffffffffu) __stcg(reinterpret_cast<uint4*>(a.Q.f16 + (size_t)cur_i * K) + m, h8_raw(q));
            cur_i = i;
            q = raw_h8(__ldcg(reinterpret_cast<const uint4*>(a.Q.f16 + (size_t)i * K) + m));
        }
        const H8 p = raw_h8(p_raw);
        const bool more = on && (j + 1 < my_cnt);
        const bool refetch = more && (u_next == u);
        if (more && !refetch) p_raw = __ldcg(reinterpret_cast<const uint4*>(a.P.f16 + (size_t)u_next * K) + m);

        // lane partials of reference lanes m and m+16, then the shfl_down-16 step
        const __half2 fa = __hfma2(__lows2half2(p.v[0], p.v[1]), __lows2half2(q.v[0], q.v[1]),
                                   __hmul2_rn(__highs2half2(p.v[0], p.v[1]), __highs2half2(q.v[0], q.v[1])));
        const __half2 fb = __hfma2(__lows2half2(p.v[2], p.v[3]), __lows2half2(q.v[2], q.v[3]),
                                   __hmul2_rn(__highs2half2(p.v[2], p.v[3]), __highs2half2(q.v[2], q.v[3])));
        const __half2 t = __hadd2_rn(__lows2half2(fa, fb), __highs2half2(fa, fb));
        __half x = __hadd_rn(__low2half(t), __high2half(t));
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) x = __hadd_rn(x, __shfl_xor_sync(full, x, d));
        const __half2 e = __half2half2(__hsub_rn(__float2half_rn(r), x));
        H8 po;
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const __half2 gp = __hfma2(e, q.v[s], __hneg2(__hmul2_rn(lam_h, p.v[s])));
            const __half2 gq = __hfma2(e, p.v[s], __hneg2(__hmul2_rn(lam_h, q.v[s])));
            po.v[s] = __hfma2(lr_h, gp, p.v[s]);
            if (on) q.v[s] = __hfma2(lr_h, gq, q.v[s]);
        }
        if (on) __stcg(reinterpret_cast<uint4*>(a.P.f16 + (size_t)u * K) + m, h8_raw(po));
        if (refetch) p_raw = __ldcg(reinterpret_cast<const uint4*>(a.P.f16 + (size_t)u_next * K) + m);
        u = u_next;
    }
    if (cur_i != 0xffffffffu) __stcg(reinterpret_cast<uint4*>(a.Q.f16 + (size_t)cur_i * K) + m, h8_raw(q));
}

#ifndef MASCOT_TRAIN_MIN_BLOCKS
#define MASCOT_TRAIN_MIN_BLOCKS 4
#endif

template <int K, int KIND, bool STATS>
__global__ void __launch_bounds__(256, MASCOT_TRAIN_MIN_BLOCKS) train_kernel(const KernelArgs a) {
    constexpr int T = K / 4;
    extern __shared__ float smem[];
    const int tl = threadIdx.x % T;
    const unsigned mask = (T == 32) ? 0xffffffffu : (0xffffu << (16 * ((threadIdx.x >> 4) & 1)));
    const uint64_t team = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) / T;
    const uint64_t nteams = ((uint64_t)gridDim.x * blockDim.x) / T;
    const uint64_t nchunks = (a.s.n + T - 1) / T;

    StatAcc acc = {a.st.gsum_p, a.st.gsum_q, a.st.nsum_p, a.st.nsum_q};
    if (STATS && a.stats_in_smem) {
        const int total = (a.st.ug + a.st.ig) * (K + 1);
        for (int j = threadIdx.x; j < total; j += blockDim.x) smem[j] = 0.f;
        acc.gs_p = smem;
        acc.gs_q = acc.gs_p + a.st.ug * K;
        acc.ns_p = acc.gs_q + a.st.ig * K;
        acc.ns_q = acc.ns_p + a.st.ug;
        __syncthreads();
    }

    const float lr = a.lr, lam = a.lam;
    const __half2 lr_h = __half2half2(__float2half_rn(lr));     // mascot_sgd_kernel.h:79-80
    const __half2 lam_h = __half2half2(__float2half_rn(lam));
    // MPT constants (mpt_sgd_kernel.h:15-16, mf_methods.cu:764-765)
    const __half mpt_scale = __float2half_rn(1000.0f);
    const __half2 mpt_lam = __half2half2(__float2half_rn(__fmul_rn(lam, 1000.0f)));
    const float mpt_rev = __fdiv_rn(1.0f, 1000.0f);

    // storage precision of each side: fixed by the trainer, or per row (bit 31) for the mixed one
    constexpr bool kUserF32Fixed = (KIND == KIND_FP32 || KIND == KIND_MPT);
    constexpr bool kItemF32Fixed = kUserF32Fixed;

    uint64_t c = team;
    float r_n = 0.f; uint32_t u_n = 0, i_n = 0;
    if (c < nchunks) {
        const uint64_t pos = c * T + tl;
        if (pos < a.s.n) { r_n = __ldg(a.s.r + pos); u_n = __ldg(a.s.u + pos); i_n = __ldg(a.s.i + pos); }
    }
    for (; c < nchunks; c += nteams) {
        const float r_l = r_n; const uint32_t u_l = u_n, i_l = i_n;
        const uint64_t cn = c + nteams;
        if (cn < nchunks) {
            const uint64_t pos = cn * T + tl;
            if (pos < a.s.n) { r_n = __ldg(a.s.r + pos); u_n = __ldg(a.s.u + pos); i_n = __ldg(a.s.i + pos); }
        }
        const uint64_t base = c * T;
        const int cnt = (a.s.n - base) < (uint64_t)T ? (int)(a.s.n - base) : T;

        if (K == 128 && KIND == KIND_MIXED && !a.deterministic) {
            const bool any_f32 = __ballot_sync(0xffffffffu, ((u_l | i_l) & kPrecBit) != 0) != 0;
            const bool has_samples = STATS && (base + T > a.st.first_sample_pos);
            if (!any_f32 && !has_samples) {
                chunk_all_half_k128(a, r_l, u_l, i_l, cnt, lr_h, lam_h);
                continue;
            }
        }

        // The item row of a run of equal items stays in registers (qh or qf, by its precision) and is
        // written back when the item changes or the chunk ends; within one team this is exactly the
        // sequential semantics, because nothing else of this team touches that row in between.
        uint32_t cur_ic = 0xffffffffu;          // no row cached (a real id never has all bits set)
        H4 qh; F4 qf;
        qh.a = qh.b = __half2half2(__ushort_as_half(0));
        qf.x[0] = qf.x[1] = qf.x[2] = qf.x[3] = 0.f;

        // user row of the first rating, fetched raw (low 8 bytes used for binary16 rows)
        uint32_t uc = __shfl_sync(mask, u_l, 0, T);
        uint4 p_raw = ld_row_raw<KIND>(a.P, uc, K, tl);
        for (int j = 0; j < cnt; j++) {
            const float r = __shfl_sync(mask, r_l, j, T);
            const uint32_t ic = __shfl_sync(mask, i_l, j, T);
            const uint32_t u = uc & kIdMask, i = ic & kIdMask;
            const bool uf = (KIND == KIND_MIXED) ? ((uc & kPrecBit) != 0) : kUserF32Fixed;
            const bool itf = (KIND == KIND_MIXED) ? ((ic & kPrecBit) != 0) : kItemF32Fixed;
            const bool sampled = STATS && (base + j >= a.st.first_sample_pos);

            if (ic != cur_ic) {
                if (cur_ic != 0xffffffffu) st_item<KIND>(a.Q, cur_ic, K, tl, qh, qf);
                cur_ic = ic;
                if (itf) qf = ld_f4(a.Q.f32, i, K, tl); else qh = ld_h4(a.Q.f16, i, K, tl);
            }
            // prefetch the next rating's user row while this one is processed; a repeated user is
            // re-read after the store below so that it sees this update
            const uint4 p_cur = p_raw;
            uint32_t uc_next = uc;
            bool refetch = false;
            if (j + 1 < cnt) {
                uc_next = __shfl_sync(mask, u_l, j + 1, T);
                if (uc_next != uc) p_raw = ld_row_raw<KIND>(a.P, uc_next, K, tl); else refetch = true;
            }

            if (KIND == KIND_MPT) {
                const F4 p = raw_f4(p_cur);
                const H4 ph = narrow(p), qhh = narrow(qf);
                const __half dot = team_sum<T>(pair_partial(ph, qhh), mask);
                const __half2 e = __half2half2(__hmul_rn(mpt_scale, __hsub_rn(__float2half_rn(r), dot)));
                const F4 gp = widen(grad(e, qhh, mpt_lam, ph)), gq = widen(grad(e, ph, mpt_lam, qhh));
                F4 po;
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    po.x[s] = __fmaf_rn(lr, __fmul_rn(mpt_rev, gp.x[s]), p.x[s]);
                    qf.x[s] = __fmaf_rn(lr, __fmul_rn(mpt_rev, gq.x[s]), qf.x[s]);
                }
                st_f4(a.P.f32, u, K, tl, po);
            } else if (KIND == KIND_MEMQUANT) {
                const F4 p = widen(raw_h4(p_cur)), q = widen(qh);
                const float part = (K == 128) ? chain_partial(p, q) : pair_partial(p, q);
                const float e = __fsub_rn(r, team_sum<T>(part, mask));
                st_h4(a.P.f16, u, K, tl, narrow(step(lr, grad(e, q, lam, p), p)));
                qh = narrow(step(lr, grad(e, p, lam, q), q));
            } else if (!uf && !itf) {
                const H4 p = raw_h4(p_cur);
                const __half dot = team_sum<T>(pair_partial(p, qh), mask);
                const __half2 e = __half2half2(__hsub_rn(__float2half_rn(r), dot));
                const H4 gp = grad(e, qh, lam_h, p), gq = grad(e, p, lam_h, qh);
                H4 po;
                po.a = __hfma2(lr_h, gp.a, p.a); po.b = __hfma2(lr_h, gp.b, p.b);
                qh.a = __hfma2(lr_h, gq.a, qh.a); qh.b = __hfma2(lr_h, gq.b, qh.b);
                st_h4(a.P.f16, u, K, tl, po);
                if (sampled) {
                    sample_side<K, T>(widen(gp), acc.gs_p, acc.ns_p, a.st.ugroup[u], tl, mask);
                    sample_side<K, T>(widen(gq), acc.gs_q, acc.ns_q, a.st.igroup[i], tl, mask);
                }
            } else if (!uf && itf) {
                const F4 p = widen(raw_h4(p_cur));
                const float e = __fsub_rn(r, team_sum<T>(pair_partial(p, qf), mask));
                const F4 gp = grad(e, qf, lam, p);
                st_h4(a.P.f16, u, K, tl, narrow(step(lr, gp, p)));
                qf = step(lr, grad(e, p, lam, qf), qf);
                if (sampled) sample_side<K, T>(gp, acc.gs_p, acc.ns_p, a.st.ugroup[u], tl, mask);
            } else if (uf && !itf) {
                const F4 p = raw_f4(p_cur), q = widen(qh);
                const float e = __fsub_rn(r, team_sum<T>(pair_partial(p, q), mask));
                const F4 gq = grad(e, p, lam, q);
                st_f4(a.P.f32, u, K, tl, step(lr, grad(e, q, lam, p), p));
                qh = narrow(step(lr, gq, q));
                if (sampled) sample_side<K, T>(gq, acc.gs_q, acc.ns_q, a.st.igroup[i], tl, mask);
            } else {
                const F4 p = raw_f4(p_cur);
                const float e = __fsub_rn(r, team_sum<T>(pair_partial(p, qf), mask));
                st_f4(a.P.f32, u, K, tl, step(lr, grad(e, qf, lam, p), p));
                qf = step(lr, grad(e, p, lam, qf), qf);
            }
            if (refetch) p_raw = ld_row_raw<KIND>(a.P, uc_next, K, tl);
            uc = uc_next;
        }
        if (cur_ic != 0xffffffffu) st_item<KIND>(a.Q, cur_ic, K, tl, qh, qf);
    }

    if (STATS && a.stats_in_smem) {
        __syncthreads();
        const int nvec = (a.st.ug + a.st.ig) * K;
        for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
            const float v = smem[j];
            if (v != 0.f) atomicAdd((j < a.st.ug * K) ? a.st.gsum_p + j : a.st.gsum_q + (j - a.st.ug * K), v);
        }
        for (int j = threadIdx.x; j < a.st.ug + a.st.ig; j += blockDim.x) {
            const float v = smem[nvec + j];
            if (v != 0.f) atomicAdd((j < a.st.ug) ? a.st.nsum_p + j : a.st.nsum_q + (j - a.st.ug), v);
        }
    }
}

int sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

template <int K, int KIND, bool STATS>
cudaError_t launch_one(const KernelArgs& args, bool deterministic, int grid_hint, cudaStream_t st, LaunchShape* shape) {
    auto kern = train_kernel<K, KIND, STATS>;
    KernelArgs a = args;
    a.deterministic = deterministic ? 1 : 0;
    int block = deterministic ? K / 4 : 256;
    size_t smem = 0;
    a.stats_in_smem = 0;
    if (STATS) {
        const size_t want = (size_t)(a.st.ug + a.st.ig) * (K + 1) * sizeof(float);
        if (want <= 200 * 1024) {
            smem = want;
            a.stats_in_smem = 1;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return e;
            }
        }
    }
    int grid = 1;
    if (!deterministic) {
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, block, smem);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) per_sm = 1;
        grid = grid_hint > 0 ? grid_hint : per_sm * sm_count();
    }
    kern<<<grid, block, smem, st>>>(a);
    if (shape) { shape->grid = grid; shape->block = block; shape->smem = smem; }
    return cudaGetLastError();
}

template <int K>
cudaError_t launch_k(TrainKind kind, const KernelArgs& a, bool stats, bool det, int hint, cudaStream_t st, LaunchShape* sh) {
    switch (kind) {
        case KIND_MIXED:
            return stats ? launch_one<K, KIND_MIXED, true>(a, det, hint, st, sh) : launch_one<K, KIND_MIXED, false>(a, det, hint, st, sh);
        case KIND_FP32: return launch_one<K, KIND_FP32, false>(a, det, hint, st, sh);
        case KIND_MPT: return launch_one<K, KIND_MPT, false>(a, det, hint, st, sh);
        case KIND_MEMQUANT: return launch_one<K, KIND_MEMQUANT, false>(a, det, hint, st, sh);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_train(int K, TrainKind kind, const Stream& s, Arena P, Arena Q, float lr, float lam,
                         const SampleStats* stats, bool deterministic, int grid_blocks_hint, cudaStream_t st,
                         LaunchShape* shape) {
    KernelArgs a;
    a.s = s; a.P = P; a.Q = Q; a.lr = lr; a.lam = lam; a.stats_in_smem = 0; a.deterministic = 0;
    if (stats) a.st = *stats;
    if (s.n == 0) { if (shape) *shape = LaunchShape(); return cudaSuccess; }
    if (K == 128) return launch_k<128>(kind, a, stats != nullptr, deterministic, grid_blocks_hint, st, shape);
    if (K == 64) return launch_k<64>(kind, a, stats != nullptr, deterministic, grid_blocks_hint, st, shape);
    return cudaErrorInvalidValue;
}

}  // namespace mascot
