// Set-up and conversion kernels: stream encoding (shuffle + id remap + precision bit), factor
// scatter/gather between the caller's fp32 row-major view and the permuted mixed-precision arenas,
// group promotion, and factor initialisation.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cub/block/block_radix_sort.cuh>
#include <cub/device/device_radix_sort.cuh>

#include "engine.h"
#include "layout.cuh"

namespace mascot {

namespace {

struct NodeAos { float r; uint32_t u; uint32_t i; };

inline int grid_for(uint64_t n, int block) {
    uint64_t g = (n + block - 1) / block;
    const uint64_t cap = (uint64_t)sm_count() * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// Replaces the host random_shuffle (mf_methods.cu:38-39) and the id remap
// matrix_reconst_gpu_triplet (preprocess_utils.h:28-36): stream position j takes source rating
// permute_index(j), ids are mapped to sorted indices and tagged with the row's storage precision.
// An id outside [0, n_users) x [0, n_items) is never used as an index: the rating is replaced by a
// no-op record on row 0 (r = 0 would still train, so the host reports the raised flag as an error).
__device__ __forceinline__ NodeAos checked(NodeAos nd, uint32_t n_users, uint32_t n_items, uint32_t* err) {
    if (nd.u >= n_users || nd.i >= n_items) { atomicOr(err, 1u); nd.u = 0; nd.i = 0; nd.r = 0.f; }
    return nd;
}

__global__ void encode_kernel(const NodeAos* src, uint64_t n, int shuffle, uint64_t seed,
                              const uint32_t* umap, const uint32_t* imap,
                              const uint8_t* uprec, const uint8_t* iprec, uint32_t n_users, uint32_t n_items, uint32_t* err,
                              float* r, uint32_t* u, uint32_t* i, uint32_t* src_out, uint32_t src_base) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t s = shuffle ? permute_index(j, n, seed) : j;
        const NodeAos nd = checked(src[s], n_users, n_items, err);
        uint32_t uu = umap ? umap[nd.u] : nd.u;
        uint32_t ii = imap ? imap[nd.i] : nd.i;
        uu |= row_flags_to_code(uprec[uu]);
        ii |= row_flags_to_code(iprec[ii]);
        r[j] = nd.r; u[j] = uu; i[j] = ii;
        if (src_out) src_out[j] = src_base + (uint32_t)s;
    }
}

// Locality-aware variant used when the stream is shuffled: after the seeded permutation the stream is
// cut into windows of kWindow consecutive positions and each window is stably sorted by item row.
// Ratings of a popular item then sit next to each other, and the update kernel keeps that item's
// row in registers for the whole run instead of reading and writing it once per rating - which is
// what bounds throughput on skewed data (every update of the most popular item otherwise goes
// through the same L2 lines).  Order inside a window carries no meaning for SGD; across windows the
// stream stays randomly ordered.  src_out records which source rating landed at each position.
constexpr int kSortThreads = 256;
constexpr int kSortItemsPerThread = 16;
constexpr int kWindow = kSortThreads * kSortItemsPerThread;

__global__ void __launch_bounds__(kSortThreads) encode_sorted_kernel(
        const NodeAos* src, uint64_t n, uint64_t seed, const uint32_t* umap, const uint32_t* imap,
        const uint8_t* uprec, const uint8_t* iprec, uint32_t n_users, uint32_t n_items, uint32_t* err, int key_bits,
        float* r, uint32_t* u, uint32_t* i, uint32_t* src_out, uint32_t src_base) {
    typedef cub::BlockRadixSort<uint32_t, kSortThreads, kSortItemsPerThread, uint32_t> Sort;
    __shared__ typename Sort::TempStorage temp;
    const uint64_t windows = (n + kWindow - 1) / kWindow;
    for (uint64_t w = blockIdx.x; w < windows; w += gridDim.x) {
        const uint64_t base = w * kWindow;
        uint32_t keys[kSortItemsPerThread], vals[kSortItemsPerThread];
#pragma unroll
        for (int t = 0; t < kSortItemsPerThread; t++) {
            const uint32_t local = threadIdx.x * kSortItemsPerThread + t;
            const uint64_t pos = base + local;
            uint32_t key = 0xffffffffu >> (32 - key_bits);      // padding sorts last
            if (pos < n) {
                uint32_t it = src[permute_index(pos, n, seed)].i;
                if (it >= n_items) it = 0;                      // reported when the record is read below
                key = imap ? imap[it] : it;
            }
            keys[t] = key;
            vals[t] = local;
        }
        Sort(temp).Sort(keys, vals, 0, key_bits);
        __syncthreads();
#pragma unroll
        for (int t = 0; t < kSortItemsPerThread; t++) {
            const uint64_t out = base + threadIdx.x * kSortItemsPerThread + t;
            if (out < n) {
                const uint64_t s = permute_index(base + vals[t], n, seed);
                const NodeAos nd = checked(src[s], n_users, n_items, err);
                uint32_t uu = umap ? umap[nd.u] : nd.u;
                uint32_t ii = (imap ? imap[nd.i] : nd.i);        // equals keys[t] unless the record was replaced
                uu |= row_flags_to_code(uprec[uu]);
                ii |= row_flags_to_code(iprec[ii]);
                r[out] = nd.r; u[out] = uu; i[out] = ii;
                if (src_out) src_out[out] = src_base + (uint32_t)s;
            }
        }
    }
}

__global__ void recode_kernel(uint32_t* ids, uint64_t n, const uint8_t* prec_row) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t id = ids[j] & kIdMask;
        ids[j] = id | row_flags_to_code(prec_row[id]);
    }
}

// cpyparams2grouped_params_for_comparison_indexing (model_init.cu:30-83): caller row e goes to
// arena row row_map[e]; here both arenas are filled so a later promotion is a plain widening.
template <int K>
__global__ void scatter_kernel(const float* src, uint32_t rows, const uint32_t* row_map, int through_half,
                               __half* dst16, float* dst32) {
    const uint64_t total = (uint64_t)rows * K;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t e = (uint32_t)(t / K);
        const int d = (int)(t % K);
        const uint32_t row = row_map ? row_map[e] : e;
        const int ph = phys_of_logical(K, d);
        const float v = src[t];
        const __half h = __float2half_rn(v);
        if (dst16) dst16[(size_t)row * K + ph] = h;
        if (dst32) dst32[(size_t)row * K + f32_pos_of_phys(K, ph)] = through_half ? __half2float(h) : v;
    }
}

// Output row e is the arena row row_map[e] (caller's id order) or, without a map, the arena row of
// sorted index e (sorted-index order).
template <int K>
__global__ void gather_kernel(const __half* a16, const float* a32, const uint8_t* prec_row, uint32_t rows,
                              const uint32_t* row_map, RowLayout layout, float* dst) {
    const uint64_t total = (uint64_t)rows * K;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t e = (uint32_t)(t / K);
        const int d = (int)(t % K);
        const uint32_t row = row_map ? row_map[e] : arena_row(layout, e);
        const int ph = phys_of_logical(K, d);
        dst[t] = (prec_row[row] & kRowPrec) ? a32[(size_t)row * K + f32_pos_of_phys(K, ph)] : __half2float(a16[(size_t)row * K + ph]);
    }
}

// mem_cpy_fp162fp32 (precision_switching.h:1-6) without the re-allocation around it: widens the rows of
// the sorted indices [begin, end) - one group - wherever the layout put them, and marks them fp32.
template <int K>
__global__ void promote_kernel(const __half* a16, float* a32, uint8_t* row_flags, RowLayout layout, uint32_t begin, uint32_t end) {
    const uint64_t total = (uint64_t)(end - begin) * K;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t row = arena_row(layout, begin + (uint32_t)(t / K));
        const int ph = (int)(t % K);
        a32[(size_t)row * K + f32_pos_of_phys(K, ph)] = __half2float(a16[(size_t)row * K + ph]);
        if (ph == 0) row_flags[row] |= kRowPrec;
    }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

// ---- reproducible double arithmetic for the factor initialisation -------------------------------
// The library logarithm and cosine are accurate to a unit in the last place but not correctly rounded,
// so a host program cannot reproduce their results bit for bit.  The two functions below use only
// single IEEE-754 operations (add, multiply, divide - written as intrinsics so that nothing is fused)
// in a fixed order; the same sequence on a host gives the same bits.
__device__ __forceinline__ double rmul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double radd(double a, double b) { return __dadd_rn(a, b); }

// ln(x) for a normal x in (0, 1]: x = m * 2^e with m in (sqrt(1/2), sqrt(2)], s = (m-1)/(m+1),
// ln(m) = 2s * (1 + z/3 + z^2/5 + ... + z^10/21), z = s^2 <= 0.0295 (truncation below 1e-17).
__device__ double exact_log(double x) {
    const long long bits = __double_as_longlong(x);
    int e = (int)((bits >> 52) & 0x7ff) - 1023;
    double m = __longlong_as_double((bits & 0xfffffffffffffLL) | 0x3ff0000000000000LL);
    if (m > 1.4142135623730951) { m = rmul(m, 0.5); e += 1; }
    const double f = radd(m, -1.0);
    const double s = __ddiv_rn(f, radd(2.0, f));
    const double z = rmul(s, s);
    double p = 1.0 / 21.0;
    p = radd(rmul(p, z), 1.0 / 19.0); p = radd(rmul(p, z), 1.0 / 17.0); p = radd(rmul(p, z), 1.0 / 15.0);
    p = radd(rmul(p, z), 1.0 / 13.0); p = radd(rmul(p, z), 1.0 / 11.0); p = radd(rmul(p, z), 1.0 / 9.0);
    p = radd(rmul(p, z), 1.0 / 7.0); p = radd(rmul(p, z), 1.0 / 5.0); p = radd(rmul(p, z), 1.0 / 3.0);
    p = radd(rmul(p, z), 1.0);
    return radd(rmul((double)e, 0.6931471805599453), rmul(rmul(2.0, s), p));
}

// cos(pi * y) for y in [0, 2], y a multiple of 2^-52: y = q/2 + r with |r| <= 1/4 (exact), then the
// Taylor series of cos or sin of t = pi*r (|t| <= 0.786, truncation below 1e-17).
__device__ double exact_cospi(double y) {
    const int q = (int)floor(radd(rmul(y, 2.0), 0.5));
    const double r = radd(y, -rmul((double)q, 0.5));
    const double t = rmul(r, 3.141592653589793), t2 = rmul(t, t);
    double c = 1.0 / 20922789888000.0;                       // 1/16!
    c = radd(rmul(c, t2), -1.0 / 87178291200.0); c = radd(rmul(c, t2), 1.0 / 479001600.0);
    c = radd(rmul(c, t2), -1.0 / 3628800.0); c = radd(rmul(c, t2), 1.0 / 40320.0);
    c = radd(rmul(c, t2), -1.0 / 720.0); c = radd(rmul(c, t2), 1.0 / 24.0);
    c = radd(rmul(c, t2), -0.5); c = radd(rmul(c, t2), 1.0);
    double sn = 1.0 / 355687428096000.0;                     // 1/17!
    sn = radd(rmul(sn, t2), -1.0 / 1307674368000.0); sn = radd(rmul(sn, t2), 1.0 / 6227020800.0);
    sn = radd(rmul(sn, t2), -1.0 / 39916800.0); sn = radd(rmul(sn, t2), 1.0 / 362880.0);
    sn = radd(rmul(sn, t2), -1.0 / 5040.0); sn = radd(rmul(sn, t2), 1.0 / 120.0);
    sn = radd(rmul(sn, t2), -1.0 / 6.0); sn = radd(rmul(sn, t2), 1.0);
    sn = rmul(sn, t);
    switch (q & 3) { case 0: return c; case 1: return -sn; case 2: return -c; default: return sn; }
}

// N(0, 0.01^2) like init_rand_feature_single (model_init.cu:19-28), from a counter-based generator:
// element t of stream `sid` depends only on (seed, sid, t) - two splitmix64 draws, Box-Muller with the
// reproducible logarithm and cosine above, one rounding to float.  A host program that follows the
// same steps gets the same factors bit for bit.
__global__ void init_normal_kernel(float* dst, uint64_t count, uint64_t seed, uint64_t sid) {
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t z = splitmix64(splitmix64(seed ^ (sid * 0xd1342543de82ef95ull)) + t);
        const double u1 = rmul((double)((z >> 11) + 1), 1.0 / 9007199254740992.0);    // (0, 1]
        const uint64_t z2 = splitmix64(z);
        const double u2 = rmul((double)(z2 >> 11), 1.0 / 9007199254740992.0);         // [0, 1)
        const double radius = __dsqrt_rn(rmul(-2.0, exact_log(u1)));
        dst[t] = (float)rmul(rmul(radius, exact_cospi(rmul(2.0, u2))), 0.01);
    }
}

}  // namespace

cudaError_t launch_encode_stream(const void* d_src_aos, uint64_t n, bool shuffle, uint64_t seed,
                                 const uint32_t* user_map, const uint32_t* item_map,
                                 const uint8_t* uprec_row, const uint8_t* iprec_row, uint32_t n_users, uint32_t n_items,
                                 uint32_t item_rows, uint32_t* err_flag,
                                 float* r, uint32_t* u, uint32_t* i, uint32_t* src_out, uint32_t src_base,
                                 cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const NodeAos* src = static_cast<const NodeAos*>(d_src_aos);
    if (shuffle) {
        int key_bits = 1;
        while (key_bits < 31 && (1ull << key_bits) < (uint64_t)item_rows + 1) key_bits++;
        const uint64_t windows = (n + kWindow - 1) / kWindow;
        const uint64_t cap = (uint64_t)sm_count() * 8;
        const int grid = (int)(windows < cap ? windows : cap);
        encode_sorted_kernel<<<grid, kSortThreads, 0, st>>>(src, n, seed, user_map, item_map, uprec_row, iprec_row,
                                                             n_users, n_items, err_flag, key_bits, r, u, i, src_out, src_base);
    } else {
        encode_kernel<<<grid_for(n, 256), 256, 0, st>>>(src, n, 0, seed, user_map, item_map, uprec_row, iprec_row,
                                                         n_users, n_items, err_flag, r, u, i, src_out, src_base);
    }
    return cudaGetLastError();
}

cudaError_t launch_recode(uint32_t* ids, uint64_t n, const uint8_t* prec_row, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    recode_kernel<<<grid_for(n, 256), 256, 0, st>>>(ids, n, prec_row);
    return cudaGetLastError();
}

// ---- re-ordering of the coded stream: precision classes and item-sorted run windows --------------
// One stable radix sort by the key  ((segment * 4 + class) << window_bits | window) << item_bits | item row :
//   * class = 2 * (user row is fp32) + (item row is fp32) when the sort is by class, else 0;
//   * window = position inside the sorted range >> run_window_log2, item = the item's arena row, when the
//     sort is by item windows (window_bits + item_bits > 0), else both absent.
// By class only, the ratings of one class become contiguous inside every segment and keep their previous
// order (so runs of equal items stay runs).  By item windows, the ratings of every window of 2^run_window_log2
// positions are sorted by item: a run of equal items is then as long as the item's share of such a window,
// not of the 4096 positions the encode kernel sorts, and a worker reads and writes the item's row once per run.
struct StreamKey {
    int use_class;           // 1: the class is part of the key
    int run_window_log2;     // log2 of the window length; only read when window_bits + item_bits > 0
    int window_bits, item_bits;
};
__global__ void stream_key_kernel(const uint32_t* u, const uint32_t* i, uint64_t n, const uint64_t* seg_off, int nseg,
                                  StreamKey sk, uint64_t* key, uint32_t* idx) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        int lo = 0, hi = nseg - 1;                    // last segment whose offset is <= j
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (seg_off[mid] <= j) lo = mid; else hi = mid - 1; }
        const uint32_t ic = i[j];
        const uint64_t cls = sk.use_class ? (((u[j] & kPrecBit) ? 2u : 0u) | ((ic & kPrecBit) ? 1u : 0u)) : 0u;
        uint64_t k = (uint64_t)lo * 4 + cls;
        if (sk.window_bits + sk.item_bits > 0)
            k = (((k << sk.window_bits) | (j >> sk.run_window_log2)) << sk.item_bits) | (ic & kIdMask);
        key[j] = k;
        idx[j] = (uint32_t)j;
    }
}
__global__ void class_gather_kernel(const uint32_t* perm, uint64_t n, const float* r, const uint32_t* u, const uint32_t* i,
                                    const uint32_t* src, float* r2, uint32_t* u2, uint32_t* i2, uint32_t* src2) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t s = perm[j];
        r2[j] = r[s]; u2[j] = u[s]; i2[j] = i[s];
        if (src) src2[j] = src[s];
    }
}
// first[k] = smallest position whose (segment, class) part of the key is k (entries of absent keys keep their
// preset value)
__global__ void class_first_kernel(const uint64_t* key_sorted, uint64_t n, int low_bits, unsigned long long* first) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x)
        if (j == 0 || (key_sorted[j] >> low_bits) != (key_sorted[j - 1] >> low_bits)) first[key_sorted[j] >> low_bits] = j;
}

static StreamKey make_stream_key(uint64_t n, bool by_class, int run_window_log2, uint32_t item_rows) {
    StreamKey sk{by_class ? 1 : 0, run_window_log2, 0, 0};
    if (run_window_log2 > 0) {
        while (((n - 1) >> run_window_log2) >> sk.window_bits) sk.window_bits++;
        while (sk.item_bits < 30 && (item_rows - 1u) >> sk.item_bits) sk.item_bits++;
        if (sk.item_bits == 0) sk.item_bits = 1;
    }
    return sk;
}

size_t stream_sort_temp_bytes(uint64_t n, int segclass_bits, bool by_class, int run_window_log2, uint32_t item_rows) {
    size_t bytes = 0;
    const StreamKey sk = make_stream_key(n, by_class, run_window_log2, item_rows);
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const uint64_t*)nullptr, (uint64_t*)nullptr, (const uint32_t*)nullptr,
                                    (uint32_t*)nullptr, n, 0, segclass_bits + sk.window_bits + sk.item_bits);
    return bytes;
}

cudaError_t launch_stream_sort(const float* r, const uint32_t* u, const uint32_t* i, const uint32_t* src, uint64_t n,
                               const uint64_t* d_seg_off, int nseg, int segclass_bits, bool by_class, int run_window_log2,
                               uint32_t item_rows, uint64_t* key_a, uint64_t* key_b, uint32_t* idx_a, uint32_t* idx_b,
                               void* temp, size_t temp_bytes, unsigned long long* d_first,
                               float* r2, uint32_t* u2, uint32_t* i2, uint32_t* src2, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const int g = grid_for(n, 256);
    const StreamKey sk = make_stream_key(n, by_class, run_window_log2, item_rows);
    stream_key_kernel<<<g, 256, 0, st>>>(u, i, n, d_seg_off, nseg, sk, key_a, idx_a);
    cudaError_t e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, key_a, key_b, idx_a, idx_b, n, 0,
                                                    segclass_bits + sk.window_bits + sk.item_bits, st);
    if (e != cudaSuccess) return e;
    class_gather_kernel<<<g, 256, 0, st>>>(idx_b, n, r, u, i, src, r2, u2, i2, src2);
    if (d_first) {
        e = cudaMemsetAsync(d_first, 0xff, sizeof(unsigned long long) * (size_t)nseg * 4, st);
        if (e != cudaSuccess) return e;
        class_first_kernel<<<g, 256, 0, st>>>(key_b, n, sk.window_bits + sk.item_bits, d_first);
    }
    return cudaGetLastError();
}

cudaError_t launch_scatter_factors(int K, const float* src, uint32_t rows, const uint32_t* row_map,
                                   bool round_through_half, __half* dst16, float* dst32, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    const int g = grid_for((uint64_t)rows * K, 256);
    if (K == 128) scatter_kernel<128><<<g, 256, 0, st>>>(src, rows, row_map, round_through_half ? 1 : 0, dst16, dst32);
    else if (K == 64) scatter_kernel<64><<<g, 256, 0, st>>>(src, rows, row_map, round_through_half ? 1 : 0, dst16, dst32);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_gather_factors(int K, Arena a, const uint8_t* prec_row, uint32_t rows,
                                  const uint32_t* row_map, const RowLayout& layout, float* dst, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    const int g = grid_for((uint64_t)rows * K, 256);
    if (K == 128) gather_kernel<128><<<g, 256, 0, st>>>(a.f16, a.f32, prec_row, rows, row_map, layout, dst);
    else if (K == 64) gather_kernel<64><<<g, 256, 0, st>>>(a.f16, a.f32, prec_row, rows, row_map, layout, dst);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_promote_rows(int K, Arena a, uint8_t* row_flags, const RowLayout& layout, uint32_t sorted_begin, uint32_t sorted_end,
                                cudaStream_t st) {
    if (sorted_end <= sorted_begin) return cudaSuccess;
    const int g = grid_for((uint64_t)(sorted_end - sorted_begin) * K, 256);
    if (K == 128) promote_kernel<128><<<g, 256, 0, st>>>(a.f16, a.f32, row_flags, layout, sorted_begin, sorted_end);
    else if (K == 64) promote_kernel<64><<<g, 256, 0, st>>>(a.f16, a.f32, row_flags, layout, sorted_begin, sorted_end);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_init_normal(float* dst, uint64_t count, uint64_t seed, uint64_t stream_id, cudaStream_t st) {
    if (count == 0) return cudaSuccess;
    init_normal_kernel<<<grid_for(count, 256), 256, 0, st>>>(dst, count, seed, stream_id);
    return cudaGetLastError();
}

}  // namespace mascot
