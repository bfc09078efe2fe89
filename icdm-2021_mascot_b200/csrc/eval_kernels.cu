// Test-RMSE kernels.
//
// The reduction is the reference's, so the result is reproducible bit for bit: per rating an fp32
// dot product (per-lane left-to-right product chain, then the 16-8-4-2-1 lane tree), the squared
// error in fp32, a 512-entry pairwise tree per block of 512 consecutive test ratings
// (get_test_rmse_coalesced_k128/k64, rmse.h:26-166), and a sequential float sum of the block
// partials on the host (rmse.h:183-188).  Unlike the reference there is no device->host->device
// round trip of the factors (mf_methods.cu:248-313, rmse.h:170-171): the kernel reads the
// mixed-precision arenas in place.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>

#include "../../include/mascot.h"
#include "engine.h"
#include "layout.cuh"

namespace mascot {

namespace {

constexpr int kRmseBlock = 512;    // ratings per block partial (BLOCK_SIZE in rmse.h:3)
constexpr int kRmseThreads = 256;

__device__ __forceinline__ float block_tree_512(float* tmp) {
    // tmp[j] += tmp[j+s] for s = 256 .. 1  (rmse.h:85-91 and warpReduce, rmse.h:5-24)
    for (int s = 256; s >= 1; s >>= 1) {
        __syncthreads();
        for (int j = threadIdx.x; j < s; j += blockDim.x) tmp[j] = __fadd_rn(tmp[j], tmp[j + s]);
    }
    __syncthreads();
    return tmp[0];
}

// A lane's eight consecutive physical elements of a row as fp32 (positions: see layout.cuh).
__device__ __forceinline__ void load8(const Arena& A, uint32_t code, int K, int tl, float* x) {
    const uint32_t row = code & kIdMask;
    if (code & kPrecBit) {
        const float4* p = reinterpret_cast<const float4*>(A.f32 + (size_t)row * K) + tl;      // two half-rows (layout.cuh)
        const float4 v = __ldcg(p), w = __ldcg(p + K / 8);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w; x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
    } else {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(A.f16 + (size_t)row * K) + tl);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
    }
}

template <int K>
__global__ void __launch_bounds__(kRmseThreads) rmse_kernel(const Stream t, const Arena P, const Arena Q, float* block_err) {
    constexpr int T = K / 8;                      // lanes per rating, eight elements each
    __shared__ float tmp[kRmseBlock];
    const int tl = threadIdx.x % T;
    const int team = threadIdx.x / T;
    constexpr int kTeams = kRmseThreads / T;
    const int lane = threadIdx.x & 31;
    const unsigned mask = ((1u << T) - 1u) << (lane - tl);
    const uint64_t base = (uint64_t)blockIdx.x * kRmseBlock;
    for (int j = team; j < kRmseBlock; j += kTeams) {
        const uint64_t idx = base + j;
        float err2 = 0.f;
        if (idx < t.n) {
            const float r = __ldg(t.r + idx);
            const uint32_t uc = __ldg(t.u + idx), ic = __ldg(t.i + idx);
            float p[8], q[8];
            load8(P, uc, K, tl, p);
            load8(Q, ic, K, tl, q);
            // positions 0 2 4 6 hold e0..e3, positions 1 3 5 7 hold e4..e7
            float part;
            if (K == 128) {
                // two reference lanes (m, m+16): product chain over four elements each (rmse.h:75),
                // their sum is the tree's 16 step
                float c[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float acc = __fmaf_rn(p[h], q[h], __fmul_rn(p[2 + h], q[2 + h]));
                    acc = __fmaf_rn(p[4 + h], q[4 + h], acc);
                    c[h] = __fmaf_rn(p[6 + h], q[6 + h], acc);
                }
                part = __fadd_rn(c[0], c[1]);
            } else {
                // four reference lanes (m, m+16, m+8, m+24) with two elements each: 16 step, then 8 step
                const float f0 = __fmaf_rn(p[0], q[0], __fmul_rn(p[2], q[2]));
                const float f1 = __fmaf_rn(p[4], q[4], __fmul_rn(p[6], q[6]));
                const float f2 = __fmaf_rn(p[1], q[1], __fmul_rn(p[3], q[3]));
                const float f3 = __fmaf_rn(p[5], q[5], __fmul_rn(p[7], q[7]));
                part = __fadd_rn(__fadd_rn(f0, f1), __fadd_rn(f2, f3));
            }
#pragma unroll
            for (int d = T / 2; d >= 1; d >>= 1) part = __fadd_rn(part, __shfl_xor_sync(mask, part, d));
            const float e = __fsub_rn(r, part);
            err2 = __fmul_rn(e, e);
        }
        if (tl == 0) tmp[j] = err2;
    }
    const float s = block_tree_512(tmp);
    if (threadIdx.x == 0) block_err[blockIdx.x] = s;
}

struct NodeAos { float r; uint32_t u; uint32_t i; };

// Plain fp32 rows in the reference's own element order: lane l reads elements l, l+32, ...
template <int K>
__global__ void __launch_bounds__(kRmseThreads) rmse_plain_kernel(const NodeAos* t, uint64_t n, const float* P, const float* Q, float* block_err) {
    __shared__ float tmp[kRmseBlock];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kWarps = kRmseThreads / 32;
    const uint64_t base = (uint64_t)blockIdx.x * kRmseBlock;
    for (int j = warp; j < kRmseBlock; j += kWarps) {
        const uint64_t idx = base + j;
        float err2 = 0.f;
        if (idx < n) {
            const float r = __ldg(&t[idx].r);
            const float* p = P + (size_t)__ldg(&t[idx].u) * K;
            const float* q = Q + (size_t)__ldg(&t[idx].i) * K;
            float part = __fmaf_rn(p[lane], q[lane], __fmul_rn(p[lane + 32], q[lane + 32]));
            if (K == 128) {
                part = __fmaf_rn(p[lane + 64], q[lane + 64], part);
                part = __fmaf_rn(p[lane + 96], q[lane + 96], part);
            }
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, d));
            const float e = __fsub_rn(r, part);
            err2 = __fmul_rn(e, e);
        }
        if (lane == 0) tmp[j] = err2;
    }
    const float s = block_tree_512(tmp);
    if (threadIdx.x == 0) block_err[blockIdx.x] = s;
}

}  // namespace

cudaError_t launch_rmse(int K, const Stream& t, Arena P, Arena Q, float* block_err, cudaStream_t st) {
    if (t.n == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((t.n + kRmseBlock - 1) / kRmseBlock);
    if (K == 128) rmse_kernel<128><<<blocks, kRmseThreads, 0, st>>>(t, P, Q, block_err);
    else if (K == 64) rmse_kernel<64><<<blocks, kRmseThreads, 0, st>>>(t, P, Q, block_err);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_rmse_plain(int K, const void* d_test_aos, uint64_t n, const float* P, const float* Q,
                              float* block_err, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((n + kRmseBlock - 1) / kRmseBlock);
    const NodeAos* t = static_cast<const NodeAos*>(d_test_aos);
    if (K == 128) rmse_plain_kernel<128><<<blocks, kRmseThreads, 0, st>>>(t, n, P, Q, block_err);
    else if (K == 64) rmse_plain_kernel<64><<<blocks, kRmseThreads, 0, st>>>(t, n, P, Q, block_err);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace mascot

// ---------------------------------------------------------------------------------------------
// Evaluation without any allocation.
//
// Some callers must not allocate device memory at call time: an evaluation hook that runs between
// training steps of a host program which has handed the whole GPU to its own memory pool (a
// cudaMalloc there can fail or fragment the pool), a serving loop that cannot afford the implicit
// device-wide synchronisation of cudaMalloc/cudaFree, or a process working inside a memory budget
// that was fixed at start-up.  For them the per-block partial sums live in the fixed array below
// instead of a cudaMalloc'ed buffer.  Every GPU that loads this library holds the array (256 KiB)
// until the process exits.
// ---------------------------------------------------------------------------------------------
namespace mascot {
namespace {

constexpr uint64_t kStaticMaxBlocks = 1u << 16;                       // 65,536 partials = 256 KiB
constexpr uint64_t kStaticMaxRatings = kStaticMaxBlocks * kRmseBlock; // 33,554,432 test ratings
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_block_err[kStaticMaxBlocks];

// In host code the name above is only a stand-in for the symbol, not an address a kernel can use:
// the device address is looked up once per device (with that device current) and cached here.
float* g_static_block_err_addr[kMaxDevices] = {nullptr};
float g_static_host_partials[kStaticMaxBlocks];

}  // namespace
}  // namespace mascot

extern "C" int mascot_rmse_device_noalloc(const float* d_P, const float* d_Q, uint32_t k, const mascot_rating* d_test,
                                          uint64_t n_test, double* rmse) {
    using namespace mascot;
    char msg[256];
    if (!d_P || !d_Q || !d_test || !rmse || !n_test) { set_global_error("null pointer or empty test set"); return MASCOT_ERR_BAD_ARG; }
    if (k != 64 && k != 128) { set_global_error("k must be 64 or 128"); return MASCOT_ERR_BAD_ARG; }
    if (n_test > kStaticMaxRatings) {
        snprintf(msg, sizeof msg, "mascot_rmse_device_noalloc handles at most %llu test ratings per call (got %llu); "
                 "use mascot_rmse_device for larger sets", (unsigned long long)kStaticMaxRatings, (unsigned long long)n_test);
        set_global_error(msg);
        return MASCOT_ERR_BAD_ARG;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_global_error("no current CUDA device (or device ordinal beyond 63)");
        return MASCOT_ERR_NO_DEVICE;
    }
    if (!g_static_block_err_addr[dev]) {
        // first call on this device: resolve the symbol's device address
        float* addr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_static_block_err);
        if (e != cudaSuccess || !addr) {
            snprintf(msg, sizeof msg, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            set_global_error(msg);
            return MASCOT_ERR_CUDA;
        }
        g_static_block_err_addr[dev] = addr;
    }
    float* d_err = g_static_block_err_addr[dev];
    const size_t blocks = (size_t)((n_test + kRmseBlock - 1) / kRmseBlock);
    // every one of the `blocks` partials is overwritten by its block, so nothing has to be cleared
    e = launch_rmse_plain((int)k, d_test, n_test, d_P, d_Q, d_err, nullptr);
    if (e == cudaSuccess) e = cudaMemcpy(g_static_host_partials, d_err, sizeof(float) * blocks, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        snprintf(msg, sizeof msg, "evaluation failed: %s", cudaGetErrorString(e));
        set_global_error(msg);
        return MASCOT_ERR_CUDA;
    }
    float sum = 0;                                   // same float accumulation order as mascot_rmse_device
    for (size_t b = 0; b < blocks; b++) sum += g_static_host_partials[b];
    *rmse = (double)(float)std::sqrt(sum / (double)n_test);
    return MASCOT_OK;
}
