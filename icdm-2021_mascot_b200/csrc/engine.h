// Internal interface between the host control code (mascot_api.cu) and the kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "layout.cuh"

namespace mascot {

// Structure-of-arrays rating stream.  u/i carry the row index in bits 0..30 and the storage
// precision of that row in bit 31 (kPrecBit), so the hot loop needs no group lookup.
struct Stream {
    const float* r = nullptr;
    const uint32_t* u = nullptr;
    const uint32_t* i = nullptr;
    uint64_t n = 0;
};

// Both arenas of one side exist for the whole run (rows at a fixed stride in each); a row is live
// in exactly one of them, chosen by its group's precision.
struct Arena {
    __half* f16 = nullptr;
    float* f32 = nullptr;
};

struct SampleStats {
    const uint16_t* ugroup = nullptr;   // group of each sorted user index
    const uint16_t* igroup = nullptr;
    int ug = 0, ig = 0;
    float* gsum_p = nullptr;            // [ug*K], physical element order inside each K-vector
    float* gsum_q = nullptr;
    float* nsum_p = nullptr;            // [ug]
    float* nsum_q = nullptr;
    uint64_t first_sample_pos = 0;      // stream positions >= this are sampled
    // The four arrays above are the first of `copies` private sets laid out `copy_stride` floats
    // apart; block b adds into set b % copies, and launch_reduce_stats folds them into set 0.
    int copies = 1;
    size_t copy_stride = 0;
};

enum TrainKind { KIND_MIXED = 0, KIND_FP32 = 1, KIND_MPT = 2, KIND_MEMQUANT = 3, KIND_MUPPET = 4, KIND_AFP = 5,
                 KIND_SWITCH = 6 /* all rows binary16, MASCOT arithmetic, statistics in MuPPET's form */ };

// Which storage precisions the ratings of a launch combine (mixed-precision trainer only).  The
// stream is kept partitioned by this class, so that each part runs an instantiation without
// per-rating precision tests; ROWCLASS_ANY reads the precision bit of every id instead.
enum RowClass { ROWCLASS_HH = 0,   // binary16 user row, binary16 item row
                ROWCLASS_HF = 1,   // binary16 user row, fp32 item row
                ROWCLASS_FH = 2,   // fp32 user row, binary16 item row
                ROWCLASS_FF = 3,   // both fp32
                ROWCLASS_ANY = 4 };

// Four 8-byte device counters (all zero when handed over) through which the update launches of one
// stream hand out their chunks in turn, and the number of launches made so far.
struct WorkCounters {
    unsigned long long* d_slots = nullptr;
    unsigned long long launches = 0;
};

struct LaunchShape {
    int grid = 0;
    int block = 0;
    size_t smem = 0;
    unsigned workers = 0;   // concurrent sequential workers the launch provides
};

// Update kernels.  `stats` == nullptr -> plain epoch.  `workers` = requested number of concurrent
// sequential workers (1 = fully sequential); `row_class` tells the mixed-precision trainer which
// precisions the ratings of this range combine (ignored by the other kinds); `counters` are the
// engine's chunk counters (all launches that share them must be queued on one stream); `bits` is the width of MuPPET's forward and
// backward pass (8, 12, 14, 16 or 32; ignored by the other kinds), `epoch` the epoch index (AFP
// re-estimates its formats at every rating early in epoch 0).  With `add_user_delta` (ignored for a
// single worker) user rows are written back as reductions of their change, so that concurrent
// updates of one user by several workers are not lost; of the updates of a user whose id carries the mark in bit 30
// only one in 2^hot_user_shift is then written back.  Returns the launch shape used.
// With `counters` == nullptr the call is dry: the instantiation the launch would use is loaded and configured
// (so that the first real launch does not pay for it) and nothing is launched.
// MuPPET statistics use gsum_p[0..K) (sum of the sampled updates, physical order) and nsum_p[0].
cudaError_t launch_train(int K, TrainKind kind, const Stream& s, Arena P, Arena Q, float lr, float lam,
                         const SampleStats* stats, RowClass row_class, unsigned workers,
                         WorkCounters* counters, int bits, int epoch, bool add_user_delta, unsigned hot_user_shift,
                         cudaStream_t st, LaunchShape* shape);

// Folds the private statistic sets of a launch into set 0 (sets are added in index order).
cudaError_t launch_reduce_stats(float* sets, int copies, size_t copy_stride, size_t floats_per_set, cudaStream_t st);

// Test RMSE over a coded SoA stream; block_err has ceil(n/512) floats.
cudaError_t launch_rmse(int K, const Stream& t, Arena P, Arena Q, float* block_err, cudaStream_t st);
// Test RMSE over plain fp32 rows in the reference element order and AoS ratings {r,u,i}.
cudaError_t launch_rmse_plain(int K, const void* d_test_aos, uint64_t n, const float* P, const float* Q,
                              float* block_err, cudaStream_t st);

// Set-up / conversion kernels.
// Codes n ratings {r,u,i} into the stream arrays: optional seeded permutation + item-sorted windows, ids
// mapped to arena rows (maps may be null: identity) and tagged with the row's storage flags.  Ids are
// checked against n_users / n_items first; an id out of range raises *err_flag and is not used as an
// index (the rating becomes a zero rating of row 0).  item_rows = rows of the item arena (sort key range).
cudaError_t launch_encode_stream(const void* d_src_aos, uint64_t n, bool shuffle, uint64_t seed,
                                 const uint32_t* user_map, const uint32_t* item_map,
                                 const uint8_t* uprec_row, const uint8_t* iprec_row, uint32_t n_users, uint32_t n_items,
                                 uint32_t item_rows, uint32_t* err_flag,
                                 float* r, uint32_t* u, uint32_t* i, uint32_t* src_out, uint32_t src_base,
                                 cudaStream_t st);
cudaError_t launch_recode(uint32_t* ids, uint64_t n, const uint8_t* prec_row, cudaStream_t st);
// Stable re-ordering of a coded stream inside every segment, by precision class (by_class; class = 2 * (user
// row fp32) + (item row fp32)) and / or by item inside windows of 2^run_window_log2 positions
// (run_window_log2 > 0; item_rows = rows of the item arena, which bounds the item part of the key).
// Inputs r/u/i/src (src may be null) stay untouched; the result goes to r2/u2/i2/src2.  key_* (n u64),
// idx_* (n u32) and temp (stream_sort_temp_bytes) are scratch; d_first (may be null) receives, for every
// segment * 4 + class, the first position holding it (all ones when it does not occur).  segclass_bits =
// bits of the largest segment * 4 + class.
size_t stream_sort_temp_bytes(uint64_t n, int segclass_bits, bool by_class, int run_window_log2, uint32_t item_rows);
cudaError_t launch_stream_sort(const float* r, const uint32_t* u, const uint32_t* i, const uint32_t* src, uint64_t n,
                               const uint64_t* d_seg_off, int nseg, int segclass_bits, bool by_class, int run_window_log2,
                               uint32_t item_rows, uint64_t* key_a, uint64_t* key_b, uint32_t* idx_a, uint32_t* idx_b,
                               void* temp, size_t temp_bytes, unsigned long long* d_first,
                               float* r2, uint32_t* u2, uint32_t* i2, uint32_t* src2, cudaStream_t st);
cudaError_t launch_scatter_factors(int K, const float* src, uint32_t rows, const uint32_t* row_map,
                                   bool round_through_half, __half* dst16, float* dst32, cudaStream_t st);
cudaError_t launch_gather_factors(int K, Arena a, const uint8_t* prec_row, uint32_t rows,
                                  const uint32_t* row_map, const RowLayout& layout, float* dst, cudaStream_t st);
// Widens the rows of the sorted indices [sorted_begin, sorted_end) from the binary16 into the fp32 arena
// and sets their "stored in fp32" flag.
cudaError_t launch_promote_rows(int K, Arena a, uint8_t* row_flags, const RowLayout& layout, uint32_t sorted_begin, uint32_t sorted_end,
                                cudaStream_t st);
cudaError_t launch_init_normal(float* dst, uint64_t count, uint64_t seed, uint64_t stream_id, cudaStream_t st);

// Number of SMs of the current device (cached per device).
int sm_count();

// Records the message returned by mascot_last_error(NULL) for handle-free entry points.
void set_global_error(const char* msg);

}  // namespace mascot
