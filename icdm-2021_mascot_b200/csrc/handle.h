// The engine handle and the helpers shared by the host-side translation units of libmascot
// (mascot_api.cu: C ABI and epochs; setup.cu: rating set-up on the device; shard.cu: multi-GPU schedule).
#pragma once
#include <cstdio>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/mascot.h"
#include "engine.h"
#include "layout.cuh"

namespace mascot { struct ShardCtx; }

struct mascot_handle {
    mascot_config cfg;
    int K = 0;
    mascot::TrainKind kind = mascot::KIND_MIXED;
    bool grouped = false;          // m-quantization / g-switching active (MASCOT variant)
    // MuPPET precision policy (mf_methods.cu:586-601): index into {8, 12, 14, 16, 32} and its history
    int mup_idx = 0, mup_switched_epoch = -1, mup_violations = 0;
    float mup_max_diversity = -1.f;
    std::vector<float> mup_norms_epoch, mup_sums_epoch;
    std::vector<uint32_t> urow_degree;           // training degree of every user row (row space of the arenas)
    bool switched_to_fp32 = false;               // whole-model switching trainer: the switch has happened
    float switch_initial_error = 1.f;            // its error at epoch index 5 (mf_methods.cu:1444, 1530)
    cudaStream_t stream = nullptr;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    // streamed epochs: a copy stream and two staging buffers, so that the upload of one piece of the
    // rating array overlaps the encoding and the updates of the piece before it
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_copied[2] = {nullptr, nullptr}, ev_free[2] = {nullptr, nullptr};
    mascot_rating* d_stage[2] = {nullptr, nullptr};
    uint64_t stage_ratings = 0;

    uint32_t n_users = 0, n_items = 0;
    uint64_t n_train = 0, n_test = 0;
    bool have_ratings = false, have_factors = false;

    // device
    float* tr_r = nullptr; uint32_t* tr_u = nullptr; uint32_t* tr_i = nullptr;
    uint32_t* tr_src = nullptr;     // source position of each stream entry (when n_train < 2^32)
    float* te_r = nullptr; uint32_t* te_u = nullptr; uint32_t* te_i = nullptr;
    mascot::Arena P, Q;
    uint8_t* d_uprec_row = nullptr; uint8_t* d_iprec_row = nullptr;
    uint32_t hot_user_shift = 0;    // one in 2^this of the updates of a marked (very popular) user is written back
    uint16_t* d_ugroup = nullptr; uint16_t* d_igroup = nullptr;
    uint32_t* d_umap = nullptr; uint32_t* d_imap = nullptr;
    float* d_stats = nullptr;       // stats_copies sets of: gsum_p | gsum_q | nsum_p | nsum_q
    int stats_copies = 1; size_t stats_stride = 0;
    float* d_block_err = nullptr;
    mascot::WorkCounters counters;  // chunk counters of the update launches (all on `stream`)
    // grow-only device scratch shared by mascot_reload_train (staging of the uploaded array) and by the
    // partition of the stream by precision class; released by mascot_release_scratch / mascot_destroy
    void* d_scratch = nullptr; size_t scratch_bytes = 0;
    // Mixed-precision trainer, several workers: once a group has been promoted the stream is kept
    // partitioned, inside every segment, into the four precision classes (see RowClass); cls_off holds
    // five stream positions per segment: the starts of the classes and the end of the segment.
    bool partitioned = false;
    std::vector<uint64_t> cls_off;

    // host
    std::vector<uint32_t> user2sorted, item2sorted, uend, iend;
    std::vector<uint8_t> uprec, iprec;
    std::vector<float> uerr, ierr, init_uerr, init_ierr;
    std::vector<float> lr;
    std::vector<float> h_stats;     // same layout as d_stats, gsum in LOGICAL element order
    std::vector<float> h_block_err;
    std::vector<uint64_t> udeg_sum, ideg_sum;   // ratings per group (training set), for byte accounting
    std::vector<uint64_t> seg_off;              // training stream segments: [seg_off[s], seg_off[s+1])
    uint64_t n_train_accounted = 0;
    std::string err;

    // Row placement (layout.cuh): where the row of sorted index s lives in the arenas.  A single engine
    // uses the identity; an engine of a sharded group lays users out rank by rank and items block by
    // block, so that what travels between GPUs is one contiguous range.  urows / irows = arena rows.
    mascot::RowLayout ulay, ilay;
    uint32_t urows = 0, irows = 0;
    bool sorted_space = false;      // ids go through the degree sort (m-quantization, and every sharded engine)
    uint32_t* d_err_flag = nullptr; // set by kernels that met an id out of range
    mascot::ShardCtx* shard = nullptr;   // group membership of a sharded engine (shard.cu)
    mascot_timings timings = {};         // accumulated phase times (mascot_get_timings)
    bool l2_window_set = false;          // a persisting access-policy window is installed on `stream`
    size_t l2_limit_before = 0;          // the process's persisting-L2 limit before this engine changed it
};

namespace mascot {

constexpr int kStatCopies = 256;   // private accumulator sets of the sampled statistics

// Records `msg` as the handle's last error (or as the handle-free one) and returns `code`.
int fail(mascot_handle* h, int code, const std::string& msg);

#define CU(h, call)                                                                               \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            char buf_[512];                                                                       \
            snprintf(buf_, sizeof buf_, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return ::mascot::fail(h, e_ == cudaErrorMemoryAllocation ? MASCOT_ERR_OOM : MASCOT_ERR_CUDA, buf_); \
        }                                                                                         \
    } while (0)

// Host clock in microseconds (phases that end with a synchronisation are timed with it).
double now_us();

template <typename T>
cudaError_t dev_alloc(T** p, size_t count) {
    return cudaMalloc(reinterpret_cast<void**>(p), sizeof(T) * (count ? count : 1));
}

template <typename T>
void dev_free(T*& p) { if (p) { cudaFree(p); p = nullptr; } }

// ---- mascot_api.cu ----
void free_ratings(mascot_handle* h);
int need_scratch(mascot_handle* h, size_t bytes);           // grow-only device scratch of at least `bytes`
bool any_fp32_group(const mascot_handle* h);
int warm_kernels(mascot_handle* h);                        // load the update kernels the first epochs will launch
int sort_run_windows(mascot_handle* h);                    // item-sorted run windows of a freshly encoded resident stream
int partition_all(mascot_handle* h);                        // (re)partition the stream by precision class when that pays
bool is_check_epoch(const mascot_config& c, uint32_t e);
float lr_at(const mascot_config& c, uint32_t e);
size_t stats_floats(const mascot_handle* h);
unsigned worker_count(const mascot_handle* h, uint64_t n);
int train_range(mascot_handle* h, float lr, uint32_t epoch, size_t segment, bool collect, LaunchShape* shape, uint32_t* launches,
                uint64_t policy_n = 0);
int fetch_stats(mascot_handle* h, uint32_t* launches);
int apply_stats(mascot_handle* h, uint32_t epoch, uint32_t* promoted_u, uint32_t* promoted_i, uint32_t* launches);
uint64_t algorithmic_bytes(const mascot_handle* h);
void make_groups(const std::vector<uint32_t>& cnt_sorted, uint32_t requested, std::vector<uint32_t>& end_idx);
cudaError_t encode_segments(mascot_handle* h, const mascot_rating* d_src, const std::vector<uint64_t>& seg, bool shuffle,
                            float* r, uint32_t* u, uint32_t* i, uint32_t* src_idx);

// ---- setup.cu ----
struct SetupRequest {
    const mascot_rating* train = nullptr; uint64_t n_train = 0;
    const uint64_t* segment_offsets = nullptr; uint32_t n_segments = 1;
    const mascot_rating* test = nullptr; uint64_t n_test = 0;
    uint32_t n_users = 0, n_items = 0;
    const uint32_t* user_degree = nullptr; const uint32_t* item_degree = nullptr;
    // library-side sharding: the arrays hold the WHOLE data set, the engine keeps the ratings of the
    // users dealt to `rank` and orders them into one segment per step of the block schedule
    int rank = -1, world = 1;
    uint32_t blocks = 1, blocks_per_rank = 1;
};
int setup_ratings(mascot_handle* h, const SetupRequest& rq);

// Installs / removes the persisting-L2 window over the item arena (cfg.l2_item_window).
int l2_window_install(mascot_handle* h);
void l2_window_remove(mascot_handle* h);

// NVTX range for the lifetime of the object (a no-op unless a profiler is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name);
    ~NvtxRange();
};

// ---- shard.cu ----
void shard_destroy(mascot_handle* h);
unsigned shard_worker_count(const mascot_handle* h);        // automatic worker count of an engine in a group

}  // namespace mascot
