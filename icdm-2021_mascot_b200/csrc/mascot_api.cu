// libmascot: host control code behind the C ABI of include/mascot.h.
//
// One handle = one GPU, one stream, one host control thread (like the reference: a single thread
// driving the default stream with a synchronisation after each epoch, mf_methods.cu:239).  The
// m-quantization set-up (degree sort, grouping, id maps) runs once on the host; everything per
// epoch runs on the device and only the small group statistics travel back on check epochs.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include "../../include/mascot.h"
#include "handle.h"

using namespace mascot;

namespace {

thread_local std::string g_create_error;

}  // namespace

void mascot::set_global_error(const char* msg) { g_create_error = msg ? msg : ""; }

mascot::NvtxRange::NvtxRange(const char* name) { nvtxRangePushA(name); }
mascot::NvtxRange::~NvtxRange() { nvtxRangePop(); }

// L2 residency for the item factors (north of L2-sized models the item side is what every rating of a
// run re-reads): a persisting access-policy window on the engine's stream over the arena that holds the
// binary16 item rows (or the fp32 one for fp32 variants).  The carve-out is a per-process limit of the
// device, not a GPU setting: it is restored when the engine goes away.
int mascot::l2_window_install(mascot_handle* h) {
    if (!h->cfg.l2_item_window || h->l2_window_set) return MASCOT_OK;
    int dev = h->cfg.device, max_persist = 0, max_window = 0;
    CU(h, cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev));
    CU(h, cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev));
    void* base = h->Q.f16 ? (void*)h->Q.f16 : (void*)h->Q.f32;
    const size_t bytes = (size_t)h->irows * h->K * (h->Q.f16 ? sizeof(__half) : sizeof(float));
    if (!base || !bytes || max_persist <= 0 || max_window <= 0) return MASCOT_OK;
    CU(h, cudaDeviceGetLimit(&h->l2_limit_before, cudaLimitPersistingL2CacheSize));
    const size_t carve = std::min<size_t>((size_t)max_persist, bytes);
    CU(h, cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, carve));
    cudaStreamAttrValue attr;
    std::memset(&attr, 0, sizeof attr);
    attr.accessPolicyWindow.base_ptr = base;
    attr.accessPolicyWindow.num_bytes = std::min<size_t>(bytes, (size_t)max_window);
    attr.accessPolicyWindow.hitRatio = (float)std::min(1.0, (double)carve / (double)attr.accessPolicyWindow.num_bytes);
    attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    CU(h, cudaStreamSetAttribute(h->stream, cudaStreamAttributeAccessPolicyWindow, &attr));
    h->l2_window_set = true;
    return MASCOT_OK;
}

void mascot::l2_window_remove(mascot_handle* h) {
    if (!h->l2_window_set) return;
    cudaStreamAttrValue attr;
    std::memset(&attr, 0, sizeof attr);
    attr.accessPolicyWindow.num_bytes = 0;            // an empty window switches the policy off
    cudaStreamSetAttribute(h->stream, cudaStreamAttributeAccessPolicyWindow, &attr);
    cudaCtxResetPersistingL2Cache();
    cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, h->l2_limit_before);
    h->l2_window_set = false;
}

double mascot::now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int mascot::fail(mascot_handle* h, int code, const std::string& msg) {
    if (h) h->err = msg; else g_create_error = msg;
    return code;
}

namespace mascot {

void free_ratings(mascot_handle* h) {
    dev_free(h->tr_r); dev_free(h->tr_u); dev_free(h->tr_i); dev_free(h->tr_src);
    dev_free(h->te_r); dev_free(h->te_u); dev_free(h->te_i);
    dev_free(h->P.f16); dev_free(h->P.f32); dev_free(h->Q.f16); dev_free(h->Q.f32);
    dev_free(h->d_uprec_row); dev_free(h->d_iprec_row); dev_free(h->d_ugroup); dev_free(h->d_igroup);
    dev_free(h->d_umap); dev_free(h->d_imap); dev_free(h->d_stats); dev_free(h->d_block_err);
    h->have_ratings = h->have_factors = false;
}

// mf_methods.cu:94-97: evaluated in double, stored as float.

float lr_at(const mascot_config& c, uint32_t e) {
    return (float)((double)c.learning_rate / (1.0 + ((double)c.decay * std::pow((double)e, 1.5))));
}

// mf_methods.cu:168-175: first check at epoch index 5, then every `interval`, never the last epoch.
bool is_check_epoch(const mascot_config& c, uint32_t e) {
    const uint32_t start_idx = 5;
    const uint32_t it = c.interval ? c.interval : 1;
    return e >= start_idx && (e % it == start_idx % it) && (c.epoch - 1 != e);
}

// split_group_based_equal_size_not_strict_ret_end_idx (preprocess_utils.h:101-213): target size
// T = ceil(N / requested); walk the distinct degrees upward counting entities; close a group at the
// last entity of a degree class once the count reaches T; always close one at the top degree.
void make_groups(const std::vector<uint32_t>& cnt_sorted, uint32_t requested, std::vector<uint32_t>& end_idx) {
    end_idx.clear();
    const uint32_t n = (uint32_t)cnt_sorted.size();
    if (!n) return;
    const uint32_t threshold = (uint32_t)std::ceil((float)n / (float)(requested ? requested : 1));
    const uint32_t max_cnt = cnt_sorted[n - 1];
    uint32_t acc = 0, pos = 0, prev = 0;
    while (pos < n) {
        const uint32_t c = cnt_sorted[pos];
        uint32_t last = pos;
        while (last + 1 < n && cnt_sorted[last + 1] == c) last++;
        if (c >= 1) {   // the reference's walk starts at degree 1 (preprocess_utils.h:139)
            acc += last - prev + 1;
            if (acc >= threshold) { end_idx.push_back(last); acc = 0; }
            else if (c == max_cnt) end_idx.push_back(last);
            prev = last + 1;
        }
        pos = last + 1;
    }
    if (end_idx.empty() || end_idx.back() != n - 1) end_idx.push_back(n - 1);   // only when every degree is 0
}

// bytes the update rule moves per epoch: every rating reads and writes k elements on each side
uint64_t algorithmic_bytes(const mascot_handle* h) {
    double per_side[2] = {0, 0};
    for (int side = 0; side < 2; side++) {
        const std::vector<uint64_t>& deg = side == 0 ? h->udeg_sum : h->ideg_sum;
        const std::vector<uint8_t>& prec = side == 0 ? h->uprec : h->iprec;
        for (size_t g = 0; g < deg.size(); g++) {
            // MPT / AFP / MuPPET keep fp32 masters; fp16-stored groups move 2 bytes per element
            per_side[side] += (double)deg[g] * (prec[g] ? 4.0 : 2.0);
        }
    }
    double total = 2.0 * h->K * (per_side[0] + per_side[1]);
    if (h->n_train_accounted && h->n_train != h->n_train_accounted) total *= (double)h->n_train / (double)h->n_train_accounted;
    return (uint64_t)total;
}

// MuPPET's ladder of pass widths (mf_methods.cu:597).
int muppet_width_at(int idx) {
    static const int widths[5] = {8, 12, 14, 16, 32};
    return widths[idx < 0 ? 0 : (idx < 4 ? idx : 4)];
}

size_t stats_floats(const mascot_handle* h) {
    return (size_t)(h->uend.size() + h->iend.size()) * (h->K + 1);
}

// Encodes an uploaded rating array into the structure-of-arrays stream, segment by segment: the
// seeded permutation and the item-sorted windows never cross a segment boundary.
cudaError_t encode_segments(mascot_handle* h, const mascot_rating* d_src, const std::vector<uint64_t>& seg, bool shuffle,
                            float* r, uint32_t* u, uint32_t* i, uint32_t* src_idx) {
    for (size_t sgm = 0; sgm + 1 < seg.size(); sgm++) {
        const uint64_t off = seg[sgm], n = seg[sgm + 1] - off;
        cudaError_t e = launch_encode_stream(d_src + off, n, shuffle, h->cfg.seed + 0x9e3779b97f4a7c15ull * sgm, h->d_umap, h->d_imap,
                                             h->d_uprec_row, h->d_iprec_row, h->n_users, h->n_items, h->irows, h->d_err_flag,
                                             r + off, u + off, i + off, src_idx ? src_idx + off : nullptr, (uint32_t)off, h->stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// One group fp16 -> fp32 (precision_switching.h:12-27): widen its rows into the fp32 arena and flip
// the per-row precision bytes; the stream ids are re-tagged afterwards by recode_side().
int promote_group(mascot_handle* h, bool users, size_t g) {
    const std::vector<uint32_t>& end = users ? h->uend : h->iend;
    std::vector<uint8_t>& prec = users ? h->uprec : h->iprec;
    uint8_t* prow = users ? h->d_uprec_row : h->d_iprec_row;
    const uint32_t b = g ? end[g - 1] + 1 : 0, e = end[g] + 1;
    CU(h, launch_promote_rows(h->K, users ? h->P : h->Q, prow, users ? h->ulay : h->ilay, b, e, h->stream));
    prec[g] = 1;
    return MASCOT_OK;
}

int recode_side(mascot_handle* h, bool users) {
    const uint8_t* prow = users ? h->d_uprec_row : h->d_iprec_row;
    CU(h, launch_recode(users ? h->tr_u : h->tr_i, h->n_train, prow, h->stream));
    CU(h, launch_recode(users ? h->te_u : h->te_i, h->n_test, prow, h->stream));
    return MASCOT_OK;
}

int need_scratch(mascot_handle* h, size_t bytes) {
    if (h->scratch_bytes >= bytes) return MASCOT_OK;
    dev_free(h->d_scratch); h->scratch_bytes = 0;
    CU(h, cudaMalloc(&h->d_scratch, bytes));
    h->scratch_bytes = bytes;
    return MASCOT_OK;
}

bool any_fp32_group(const mascot_handle* h) {
    for (uint8_t p : h->uprec) if (p) return true;
    for (uint8_t p : h->iprec) if (p) return true;
    return false;
}

// Re-orders the segments [seg_first, seg_first + seg_count) of the coded stream, stably, inside each segment:
//   by_class: the ratings of one precision class become contiguous (the order inside a class is the order
//     before) and the class boundaries are recorded.  Called after the precision bits of the ids changed
//     (promotion + recode) or after a stream was encoded while promoted groups exist.
//   run_window_log2 > 0: every window of 2^run_window_log2 positions is sorted by item (longer runs of equal
//     items).  Called once after a stream was encoded.
// The single-worker deterministic mode keeps the caller's order and does neither.
int reorder_segments(mascot_handle* h, size_t seg_first, size_t seg_count, bool by_class, int run_window_log2) {
    const size_t nseg_all = h->seg_off.size() - 1;
    if (by_class && h->cls_off.size() != nseg_all * 5) {
        h->cls_off.assign(nseg_all * 5, 0);
        for (size_t sg = 0; sg < nseg_all; sg++) {          // everything in the first class
            h->cls_off[sg * 5] = h->seg_off[sg];
            for (int c = 1; c <= 4; c++) h->cls_off[sg * 5 + c] = h->seg_off[sg + 1];
        }
    }
    const uint64_t begin = h->seg_off[seg_first], end = h->seg_off[seg_first + seg_count], n = end - begin;
    if (n == 0) return MASCOT_OK;
    int key_bits = 2;
    while ((1ull << key_bits) < seg_count * 4) key_bits++;
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    const size_t temp_bytes = stream_sort_temp_bytes(n, key_bits, by_class, run_window_log2, h->irows);
    const size_t b_key = up(sizeof(uint64_t) * n), b_idx = up(sizeof(uint32_t) * n), b_seg = up(sizeof(uint64_t) * (seg_count + 1));
    const size_t b_first = up(sizeof(unsigned long long) * seg_count * 4);
    const size_t total = 2 * b_key + 2 * b_idx + 4 * b_idx + b_seg + b_first + up(temp_bytes);
    int rc = need_scratch(h, total);
    if (rc != MASCOT_OK) return rc;
    unsigned char* base = static_cast<unsigned char*>(h->d_scratch);
    uint64_t* key_a = reinterpret_cast<uint64_t*>(base); base += b_key;
    uint64_t* key_b = reinterpret_cast<uint64_t*>(base); base += b_key;
    uint32_t* idx_a = reinterpret_cast<uint32_t*>(base); base += b_idx;
    uint32_t* idx_b = reinterpret_cast<uint32_t*>(base); base += b_idx;
    float* r2 = reinterpret_cast<float*>(base); base += b_idx;
    uint32_t* u2 = reinterpret_cast<uint32_t*>(base); base += b_idx;
    uint32_t* i2 = reinterpret_cast<uint32_t*>(base); base += b_idx;
    uint32_t* s2 = reinterpret_cast<uint32_t*>(base); base += b_idx;
    uint64_t* d_seg = reinterpret_cast<uint64_t*>(base); base += b_seg;
    unsigned long long* d_first = reinterpret_cast<unsigned long long*>(base); base += b_first;
    void* temp = base;
    std::vector<uint64_t> rel(seg_count + 1);
    for (size_t j = 0; j <= seg_count; j++) rel[j] = h->seg_off[seg_first + j] - begin;
    CU(h, cudaMemcpyAsync(d_seg, rel.data(), sizeof(uint64_t) * rel.size(), cudaMemcpyHostToDevice, h->stream));
    uint32_t* src = h->tr_src ? h->tr_src + begin : nullptr;
    CU(h, launch_stream_sort(h->tr_r + begin, h->tr_u + begin, h->tr_i + begin, src, n, d_seg, (int)seg_count, key_bits, by_class,
                             run_window_log2, h->irows, key_a, key_b, idx_a, idx_b, temp, temp_bytes, by_class ? d_first : nullptr,
                             r2, u2, i2, s2, h->stream));
    CU(h, cudaMemcpyAsync(h->tr_r + begin, r2, sizeof(float) * n, cudaMemcpyDeviceToDevice, h->stream));
    CU(h, cudaMemcpyAsync(h->tr_u + begin, u2, sizeof(uint32_t) * n, cudaMemcpyDeviceToDevice, h->stream));
    CU(h, cudaMemcpyAsync(h->tr_i + begin, i2, sizeof(uint32_t) * n, cudaMemcpyDeviceToDevice, h->stream));
    if (src) CU(h, cudaMemcpyAsync(src, s2, sizeof(uint32_t) * n, cudaMemcpyDeviceToDevice, h->stream));
    std::vector<unsigned long long> first(seg_count * 4);
    if (by_class) CU(h, cudaMemcpyAsync(first.data(), d_first, sizeof(unsigned long long) * first.size(), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));          // `rel` and `first` are host buffers of this call
    if (!by_class) return MASCOT_OK;
    for (size_t j = 0; j < seg_count; j++) {
        uint64_t* off = &h->cls_off[(seg_first + j) * 5];
        off[4] = h->seg_off[seg_first + j + 1];
        for (int c = 3; c >= 0; c--) off[c] = first[j * 4 + c] == ~0ull ? off[c + 1] : begin + first[j * 4 + c];
    }
    return MASCOT_OK;
}

// The stream is partitioned when that pays: mixed-precision trainer, more than one worker, at least
// one promoted group, and sizes the sort key and the 32-bit permutation can express.
bool wants_partition(const mascot_handle* h) {
    if (!(h->grouped && !h->cfg.deterministic && any_fp32_group(h) && h->n_train < (1ull << 32) && (h->seg_off.size() - 1) * 4 <= 65536)) return false;
    // Measured on one B200 with promoted groups: 100M-rating set 7.6 ms per epoch with one launch per class (14.0 ms
    // before the run windows) against 15.2 ms for one launch that reads each id's precision bit; 252M-rating set,
    // 40 epochs: 1,126 ms against 1,365 ms (the launch of the all-binary16 class keeps its 32 warps per SM, the
    // per-rating instantiation runs 16).
    return h->cfg.no_class_partition != 1;
}

int partition_all(mascot_handle* h) {
    h->partitioned = false;
    if (!wants_partition(h)) return MASCOT_OK;
    const int rc = reorder_segments(h, 0, h->seg_off.size() - 1, true, 0);
    if (rc == MASCOT_OK) h->partitioned = true;
    return rc;
}

// log2 of the item-sorted run windows of the resident stream; 0 = none beyond the encode kernel's own windows.
// The configured length (default 2^20) is shortened to the largest power of two that keeps two properties:
//   * a window is no longer than the ratings all workers of a launch hold at one time (workers x 8 chunks of
//     K/8 ratings): with longer windows every worker is on the same few items at once, and since item rows are
//     plain stores most of their updates are lost (100M-rating set, 8,288 workers: windows of 2^20 and 2^22
//     converge like the unsorted stream, 2^24 needs twice the epochs);
//   * when statistics are sampled, the sampled tail of every launched range (sample_ratio of a segment) spans
//     at least four windows, so that every item group is met there in proportion.
int run_window_log2(const mascot_handle* h) {
    if (h->cfg.deterministic || !h->cfg.shuffle || h->n_train == 0 || h->n_train >= (1ull << 32) || (h->seg_off.size() - 1) * 4 > 65536) return 0;
    uint32_t w = h->cfg.run_window_log2 ? std::min<uint32_t>(h->cfg.run_window_log2, 32) : 20;
    uint64_t limit = (uint64_t)worker_count(h, h->n_train) * 8 * (h->K / 8);
    const bool sampled = h->kind == KIND_MIXED || h->kind == KIND_SWITCH || h->kind == KIND_MUPPET;
    if (sampled && h->cfg.sample_ratio > 0.f) {
        uint64_t shortest = ~0ull;
        for (size_t sg = 0; sg + 1 < h->seg_off.size(); sg++)
            if (h->seg_off[sg + 1] > h->seg_off[sg]) shortest = std::min<uint64_t>(shortest, h->seg_off[sg + 1] - h->seg_off[sg]);
        limit = std::min<uint64_t>(limit, (uint64_t)((double)shortest * h->cfg.sample_ratio / 4.0));
    }
    while (w > 12 && (1ull << w) > limit) w--;
    return w <= 12 ? 0 : (int)w;
}

int muppet_bits(const mascot_handle* h);

// Loads and configures the update-kernel instantiations the first epochs will launch (the CUDA runtime loads
// a kernel at its first use, which otherwise costs the first epoch a few milliseconds).  The instantiations
// for promoted rows are left to their first use.
int warm_kernels(mascot_handle* h) {
    if (!h->n_train) return MASCOT_OK;
    Stream s; s.r = h->tr_r; s.u = h->tr_u; s.i = h->tr_i; s.n = h->n_train;
    const unsigned workers = worker_count(h, h->n_train);
    const RowClass cls = any_fp32_group(h) ? ROWCLASS_ANY : ROWCLASS_HH;
    SampleStats st = SampleStats();
    const bool sampled = h->kind == KIND_MIXED || h->kind == KIND_SWITCH || h->kind == KIND_MUPPET;
    for (int with_stats = 0; with_stats <= (sampled ? 1 : 0); with_stats++)
        CU(h, launch_train(h->K, h->kind, s, h->P, h->Q, 0.f, 0.f, with_stats ? &st : nullptr, cls, workers, nullptr, muppet_bits(h), 0,
                           h->cfg.plain_user_stores == 0, h->hot_user_shift, h->stream, nullptr));
    return MASCOT_OK;
}

// Sorts the freshly encoded resident stream by item inside its run windows.
int sort_run_windows(mascot_handle* h) {
    const int w = run_window_log2(h);
    if (w == 0 || h->n_train == 0) return MASCOT_OK;
    NvtxRange range("mascot: item-sorted run windows");
    return reorder_segments(h, 0, h->seg_off.size() - 1, false, w);
}

float reference_rmse_from_partials(const std::vector<float>& part, uint64_t n) {
    float sum = 0;                                  // rmse.h:183-186: float accumulation in block order
    for (float v : part) sum += v;
    return (float)std::sqrt(sum / (double)n);       // rmse.h:188, returned through a float
}

}  // namespace

extern "C" {

int mascot_abi_info(uint32_t* abi_version, uint32_t* config_bytes, uint32_t* epoch_stats_bytes) {
    if (abi_version) *abi_version = MASCOT_ABI_VERSION;
    if (config_bytes) *config_bytes = (uint32_t)sizeof(mascot_config);
    if (epoch_stats_bytes) *epoch_stats_bytes = (uint32_t)sizeof(mascot_epoch_stats);
    return MASCOT_OK;
}

int mascot_config_default(mascot_config* cfg) {
    if (!cfg) return MASCOT_ERR_BAD_ARG;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->lambda = 0.015f; cfg->learning_rate = 0.01f; cfg->decay = 0.1f; cfg->sample_ratio = 0.01f;
    cfg->error_threshold = 0.001f; cfg->interval = 1; cfg->user_group_num = 10; cfg->item_group_num = 10;
    cfg->k = 128; cfg->num_workers = 2048; cfg->epoch = 50; cfg->thread_block_size = 128; cfg->version = 7;
    cfg->shuffle = 1; cfg->seed = 1; cfg->device = 0;
    return MASCOT_OK;
}

const char* mascot_status_string(int s) {
    switch (s) {
        case MASCOT_OK: return "ok";
        case MASCOT_ERR_BAD_ARG: return "bad argument";
        case MASCOT_ERR_CUDA: return "CUDA error";
        case MASCOT_ERR_OOM: return "out of memory";
        case MASCOT_ERR_STATE: return "call order violated";
        case MASCOT_ERR_NO_DEVICE: return "no usable CUDA device";
        case MASCOT_ERR_TIMEOUT: return "timed out";
        case MASCOT_ERR_UNSUPPORTED: return "unsupported";
        case MASCOT_ERR_COMM: return "communication failure";
    }
    return "unknown status";
}

const char* mascot_last_error(const mascot_handle* h) { return h ? h->err.c_str() : g_create_error.c_str(); }

int mascot_create(const mascot_config* cfg, mascot_handle** out) {
    if (!cfg || !out) return fail(nullptr, MASCOT_ERR_BAD_ARG, "null config or output pointer");
    *out = nullptr;
    if (cfg->k != 64 && cfg->k != 128) return fail(nullptr, MASCOT_ERR_BAD_ARG, "k must be 64 or 128");
    if (cfg->epoch == 0) return fail(nullptr, MASCOT_ERR_BAD_ARG, "epoch count must be positive");
    TrainKind kind;
    switch (cfg->version) {
        case MASCOT_V_MASCOT: kind = KIND_MIXED; break;
        case MASCOT_V_SGD: kind = KIND_FP32; break;
        case MASCOT_V_MPT: kind = KIND_MPT; break;
        case MASCOT_V_MEMQUANT: kind = KIND_MEMQUANT; break;
        case MASCOT_V_NAIVE: kind = KIND_MIXED; break;
        case MASCOT_V_SWITCH_ONLY: kind = KIND_SWITCH; break;
        case MASCOT_V_MUPPET: kind = KIND_MUPPET; break;
        case MASCOT_V_AFP: kind = KIND_AFP; break;
        default: return fail(nullptr, MASCOT_ERR_BAD_ARG, "unknown training variant");
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        cudaGetLastError();
        return fail(nullptr, MASCOT_ERR_NO_DEVICE, "no CUDA device is visible; libmascot has no CPU path");
    }
    if (cfg->device < 0 || cfg->device >= ndev) return fail(nullptr, MASCOT_ERR_NO_DEVICE, "requested CUDA device does not exist");
    mascot_handle* h = new (std::nothrow) mascot_handle();
    if (!h) return fail(nullptr, MASCOT_ERR_OOM, "host allocation failed");
    h->cfg = *cfg; h->K = (int)cfg->k; h->kind = kind; h->grouped = (cfg->version == MASCOT_V_MASCOT || cfg->version == MASCOT_V_NAIVE);
    h->mup_idx = cfg->is_yahoo ? 1 : 0;            // mf_methods.cu:600-601
    for (int j = 0; j < 5; j++) if (cfg->muppet_width == (uint32_t)muppet_width_at(j)) h->mup_idx = j;
    h->lr.resize(cfg->epoch);
    for (uint32_t e = 0; e < cfg->epoch; e++) h->lr[e] = lr_at(*cfg, e);
    cudaError_t e = cudaSetDevice(cfg->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    for (int j = 0; j < 4 && e == cudaSuccess; j++) e = cudaEventCreate(&h->ev[j]);
    if (e == cudaSuccess) e = dev_alloc(&h->counters.d_slots, 4);
    if (e == cudaSuccess) e = cudaMemset(h->counters.d_slots, 0, 4 * sizeof(unsigned long long));
    if (e != cudaSuccess) {
        std::string msg = std::string("CUDA set-up failed: ") + cudaGetErrorString(e);
        mascot_destroy(h);
        return fail(nullptr, MASCOT_ERR_CUDA, msg);
    }
    *out = h;
    return MASCOT_OK;
}

int mascot_destroy(mascot_handle* h) {
    if (!h) return MASCOT_OK;
    cudaSetDevice(h->cfg.device);
    l2_window_remove(h);
    free_ratings(h);
    shard_destroy(h);
    dev_free(h->d_scratch); dev_free(h->counters.d_slots); dev_free(h->d_err_flag);
    for (auto& ev : h->ev) if (ev) cudaEventDestroy(ev);
    for (int b = 0; b < 2; b++) {
        if (h->ev_copied[b]) cudaEventDestroy(h->ev_copied[b]);
        if (h->ev_free[b]) cudaEventDestroy(h->ev_free[b]);
        if (h->d_stage[b]) cudaFree(h->d_stage[b]);
    }
    if (h->copy_stream) cudaStreamDestroy(h->copy_stream);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return MASCOT_OK;
}

int mascot_set_ratings(mascot_handle* h, const mascot_rating* train, uint64_t n_train,
                       const mascot_rating* test, uint64_t n_test, uint32_t n_users, uint32_t n_items) {
    return mascot_set_ratings_sharded(h, train, n_train, nullptr, 1, test, n_test, n_users, n_items, nullptr, nullptr);
}

int mascot_set_ratings_sharded(mascot_handle* h, const mascot_rating* train, uint64_t n_train,
                               const uint64_t* segment_offsets, uint32_t n_segments,
                               const mascot_rating* test, uint64_t n_test, uint32_t n_users, uint32_t n_items,
                               const uint32_t* user_degree, const uint32_t* item_degree) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (h->shard) return fail(h, MASCOT_ERR_STATE, "this engine belongs to a sharded group: use mascot_shard_set_ratings");
    SetupRequest rq;
    rq.train = train; rq.n_train = n_train; rq.segment_offsets = segment_offsets; rq.n_segments = n_segments;
    rq.test = test; rq.n_test = n_test; rq.n_users = n_users; rq.n_items = n_items;
    rq.user_degree = user_degree; rq.item_degree = item_degree;
    return setup_ratings(h, rq);
}

int mascot_reload_train(mascot_handle* h, const mascot_rating* train, uint64_t n_train) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!train && n_train) return fail(h, MASCOT_ERR_BAD_ARG, "null rating array");
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    if (n_train >= (1ull << 32)) return fail(h, MASCOT_ERR_BAD_ARG, "too many ratings (limit 2^32 - 1 per engine)");
    CU(h, cudaSetDevice(h->cfg.device));
    if (n_train != h->n_train) {
        dev_free(h->tr_r); dev_free(h->tr_u); dev_free(h->tr_i); dev_free(h->tr_src);
        CU(h, dev_alloc(&h->tr_r, n_train)); CU(h, dev_alloc(&h->tr_u, n_train)); CU(h, dev_alloc(&h->tr_i, n_train));
        CU(h, dev_alloc(&h->tr_src, n_train));
        h->n_train = n_train;
        h->seg_off.assign({0, n_train});           // a stream of another length is one segment
        h->cls_off.clear(); h->partitioned = false;
    }
    if (!n_train) return MASCOT_OK;
    const size_t bytes = sizeof(mascot_rating) * n_train;
    int rc = need_scratch(h, bytes);
    if (rc != MASCOT_OK) return rc;
    CU(h, cudaMemsetAsync(h->d_err_flag, 0, sizeof(uint32_t), h->stream));
    CU(h, cudaMemcpyAsync(h->d_scratch, train, bytes, cudaMemcpyHostToDevice, h->stream));
    CU(h, encode_segments(h, static_cast<const mascot_rating*>(h->d_scratch), h->seg_off, h->cfg.shuffle != 0,
                          h->tr_r, h->tr_u, h->tr_i, h->tr_src));
    uint32_t bad = 0;
    CU(h, cudaMemcpyAsync(&bad, h->d_err_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
    h->cls_off.clear();
    if ((rc = sort_run_windows(h)) != MASCOT_OK) return rc;
    if ((rc = partition_all(h)) != MASCOT_OK) return rc;      // the new stream carries the current precisions
    CU(h, cudaStreamSynchronize(h->stream));
    if (bad) return fail(h, MASCOT_ERR_BAD_ARG, "training rating with id out of range (replaced by zero ratings of row 0; reload a valid array)");
    return MASCOT_OK;
}

static int scatter_from_device(mascot_handle* h, const float* dP, const float* dQ) {
    const double t0 = now_us();
    const bool through_half = (h->kind == KIND_MPT);   // MPT masters start from fp16 values (mf_methods.cu:730-733)
    CU(h, launch_scatter_factors(h->K, dP, h->n_users, h->d_umap, through_half, h->P.f16, h->P.f32, h->stream));
    CU(h, launch_scatter_factors(h->K, dQ, h->n_items, h->d_imap, through_half, h->Q.f16, h->Q.f32, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    h->timings.copy_to_grouped_us += now_us() - t0;
    h->have_factors = true;
    return l2_window_install(h);
}

int mascot_set_factors(mascot_handle* h, const float* P, const float* Q) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!P || !Q) return fail(h, MASCOT_ERR_BAD_ARG, "null factor matrix");
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    CU(h, cudaSetDevice(h->cfg.device));
    const size_t pu = (size_t)h->n_users * h->K, qi = (size_t)h->n_items * h->K;
    float *dP = nullptr, *dQ = nullptr;
    CU(h, dev_alloc(&dP, pu));
    cudaError_t e = dev_alloc(&dQ, qi);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dP, P, sizeof(float) * pu, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dQ, Q, sizeof(float) * qi, cudaMemcpyHostToDevice, h->stream);
    int rc = MASCOT_OK;
    if (e == cudaSuccess) rc = scatter_from_device(h, dP, dQ);
    cudaFree(dP); cudaFree(dQ);
    CU(h, e);
    return rc;
}

int mascot_init_factors(mascot_handle* h) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    CU(h, cudaSetDevice(h->cfg.device));
    const size_t pu = (size_t)h->n_users * h->K, qi = (size_t)h->n_items * h->K;
    float *dP = nullptr, *dQ = nullptr;
    CU(h, dev_alloc(&dP, pu));
    cudaError_t e = dev_alloc(&dQ, qi);
    if (e == cudaSuccess) e = launch_init_normal(dP, pu, h->cfg.seed, 1, h->stream);
    if (e == cudaSuccess) e = launch_init_normal(dQ, qi, h->cfg.seed, 2, h->stream);
    int rc = MASCOT_OK;
    if (e == cudaSuccess) rc = scatter_from_device(h, dP, dQ);
    cudaFree(dP); cudaFree(dQ);
    CU(h, e);
    return rc;
}

}  // extern "C"

namespace mascot {

unsigned worker_count(const mascot_handle* h, uint64_t n) {
    // -wg 0 = automatic: one worker per 8192 ratings keeps the sequential depth per worker - and with
    // it the convergence per epoch - at the level of the reference's tuned runs; the launch caps the
    // count at what the GPU can keep resident.  Small sets (under 1.5M ratings) would leave most SMs
    // idle at that rate: they get one worker per 512 ratings, at most 1536 (measured on the 0.8M-rating
    // configuration: final RMSE still below the reference's, three times the throughput of 512 workers).
    if (h->cfg.deterministic) return 1u;
    if (h->cfg.num_workers) return h->cfg.num_workers;
    if (h->shard) return shard_worker_count(h);
    if (n < 1500000) return (unsigned)std::min<uint64_t>(std::max<uint64_t>(n / 512, 512), 1536);
    uint64_t w = std::min<uint64_t>(std::max<uint64_t>(n / 8192, 512), 1u << 20);
    return (unsigned)w;
}

// Width of MuPPET's forward and backward pass this epoch (mf_methods.cu:597, 623-624).
int muppet_bits(const mascot_handle* h) { return muppet_width_at(h->mup_idx); }

// MuPPET's switching rule after epoch e (mf_methods.cu:586-595, 660-695): over the last three epochs,
// gradient diversity = sum of the sampled squared gradient norms / squared norm of the summed sampled
// updates; when the largest diversity seen since the last switch exceeds the current one by more than a
// decaying threshold, the next wider format is used from the next epoch on.
void muppet_policy(mascot_handle* h, uint32_t epoch) {
    const int K = h->K, e = (int)epoch, resolution = 3;
    const float alpha = 1.0f, beta = 1.5f, lambda_thr = 0.3f;
    const float threshold = alpha + (beta * std::exp(-1 * lambda_thr * (e)));
    if ((int)h->mup_norms_epoch.size() <= e) { h->mup_norms_epoch.resize(e + 1, 0.f); h->mup_sums_epoch.resize((size_t)(e + 1) * K, 0.f); }
    h->mup_norms_epoch[e] = h->h_stats[(size_t)2 * K];                       // nsum_p[0]
    std::copy(h->h_stats.begin(), h->h_stats.begin() + K, h->mup_sums_epoch.begin() + (size_t)e * K);
    if (e - h->mup_switched_epoch < resolution) return;
    float norms = 0.f, sq = 0.f;
    std::vector<float> acc(K, 0.f);
    for (int w = e - resolution + 1; w <= e; w++) {
        norms += h->mup_norms_epoch[w];
        for (int d = 0; d < K; d++) acc[d] += h->mup_sums_epoch[(size_t)w * K + d];
    }
    for (int d = 0; d < K; d++) sq += powf(acc[d], 2);
    const float diversity = norms / sq;
    h->mup_max_diversity = h->mup_max_diversity < diversity ? diversity : h->mup_max_diversity;
    const float ratio = h->mup_max_diversity / diversity;
    if (ratio > threshold && ++h->mup_violations == 1) {
        if (h->mup_idx < 4) h->mup_idx++;
        h->mup_switched_epoch = e;
        h->mup_max_diversity = -1.f;
        h->mup_violations = 0;
    }
}

int promote_group(mascot_handle* h, bool users, size_t g);
int recode_side(mascot_handle* h, bool users);

// Whole-model switching trainer after a check epoch (mf_methods.cu:1515-1545): error = squared norm of
// the summed sampled updates / sum of their squared norms, relative to its value at epoch index 5;
// above the threshold every row is widened to fp32 and the fp32 trainer takes over.
int switch_only_policy(mascot_handle* h, uint32_t epoch, uint32_t* promoted_u, uint32_t* promoted_i) {
    const int K = h->K;
    float sq = 0.f;
    for (int d = 0; d < K; d++) sq += powf(h->h_stats[d], 2);
    float error = sq / h->h_stats[(size_t)2 * K];
    error = error / h->switch_initial_error;
    h->uerr[0] = error; h->ierr[0] = error;
    if (epoch == 5) h->switch_initial_error = error;
    if (epoch > 5 && error > h->cfg.error_threshold) {
        int rc;
        if ((rc = promote_group(h, true, 0)) != MASCOT_OK) return rc;
        if ((rc = promote_group(h, false, 0)) != MASCOT_OK) return rc;
        if ((rc = recode_side(h, true)) != MASCOT_OK) return rc;
        if ((rc = recode_side(h, false)) != MASCOT_OK) return rc;
        h->switched_to_fp32 = true;
        *promoted_u = 1; *promoted_i = 1;
    }
    return MASCOT_OK;
}

SampleStats stats_view(mascot_handle* h) {
    const int ug = (int)h->uend.size(), ig = (int)h->iend.size(), K = h->K;
    SampleStats st;
    st.ugroup = h->d_ugroup; st.igroup = h->d_igroup; st.ug = ug; st.ig = ig;
    st.gsum_p = h->d_stats; st.gsum_q = st.gsum_p + (size_t)ug * K;
    st.nsum_p = st.gsum_q + (size_t)ig * K; st.nsum_q = st.nsum_p + ug;
    st.copies = h->stats_copies; st.copy_stride = h->stats_stride;
    st.first_sample_pos = 0;
    return st;
}

// Runs the update kernel over stream positions [begin, end), all of whose ratings are of row class
// `cls`.  With `collect`, the last sample_ratio of the range (mf_methods.cu:102-103, 173-174) goes
// through the statistics kernel - a second launch, so that only the sampled fraction pays for the
// statistics.  `policy_n` (0 = the range's own length) is the stream length the automatic worker
// count is taken from.
int train_span(mascot_handle* h, float lr, uint32_t epoch, uint64_t begin, uint64_t end, RowClass cls, bool collect,
               LaunchShape* shape, uint32_t* launches, unsigned workers, cudaStream_t stream, WorkCounters* counters) {
    if (end <= begin) return MASCOT_OK;
    const uint64_t n = end - begin;
    // after its switch the whole-model switching trainer is the plain fp32 trainer (sgd_kernel.h:296-326)
    const TrainKind kind = (h->kind == KIND_SWITCH && h->switched_to_fp32) ? KIND_FP32 : h->kind;
    Stream s; s.r = h->tr_r + begin; s.u = h->tr_u + begin; s.i = h->tr_i + begin; s.n = n;
    uint64_t head = n;
    if (collect) {
        const uint64_t sample_num = (uint64_t)((float)n * h->cfg.sample_ratio);
        head = n - std::min<uint64_t>(sample_num, n);
    }
    if (head > 0) {
        Stream sa = s; sa.n = head;
        CU(h, launch_train(h->K, kind, sa, h->P, h->Q, lr, h->cfg.lambda, nullptr, cls, workers,
                           counters, muppet_bits(h), (int)epoch, h->cfg.plain_user_stores == 0, h->hot_user_shift, stream, shape));
        (*launches)++;
    }
    if (head < n) {
        Stream sb; sb.r = s.r + head; sb.u = s.u + head; sb.i = s.i + head; sb.n = n - head;
        const SampleStats st = stats_view(h);
        LaunchShape tail_shape;            // the caller is told the shape of the plain launch when there is one
        CU(h, launch_train(h->K, kind, sb, h->P, h->Q, lr, h->cfg.lambda, &st, cls, workers,
                           counters, muppet_bits(h), (int)epoch, h->cfg.plain_user_stores == 0, h->hot_user_shift, stream, head > 0 ? &tail_shape : shape));
        (*launches)++;
    }
    return MASCOT_OK;
}

// One segment of the stream: a single launch while every row is binary16 (or when the stream is not
// partitioned: the launch then reads each id's precision bit), else one launch per non-empty precision
// class, one after the other.  (Running the classes side by side on streams of their own, each with a
// share of the workers, was measured too: 15.7 ms per promoted epoch on the 100M-rating set against 14.0 ms
// one after the other.)  On a check epoch every launched range contributes its own sampled tail.
int train_range(mascot_handle* h, float lr, uint32_t epoch, size_t segment, bool collect, LaunchShape* shape, uint32_t* launches,
                uint64_t policy_n) {
    const uint64_t begin = h->seg_off[segment], end = h->seg_off[segment + 1];
    if (!policy_n) policy_n = end - begin;
    const unsigned workers = worker_count(h, policy_n);
    if (!h->partitioned)
        return train_span(h, lr, epoch, begin, end, any_fp32_group(h) ? ROWCLASS_ANY : ROWCLASS_HH, collect, shape, launches, workers,
                          h->stream, &h->counters);
    const uint64_t* off = &h->cls_off[segment * 5];
    for (int c = 0; c < 4; c++) {
        const int rc = train_span(h, lr, epoch, off[c], off[c + 1], (RowClass)c, collect, shape, launches, workers, h->stream, &h->counters);
        if (rc != MASCOT_OK) return rc;
    }
    return MASCOT_OK;
}

// Folds the private accumulator sets and brings the sums to the host in LOGICAL element order.
int fetch_stats(mascot_handle* h, uint32_t* launches) {
    const int ug = (int)h->uend.size(), ig = (int)h->iend.size(), K = h->K;
    const double t0 = now_us();
    if (h->stats_copies > 1) {
        CU(h, launch_reduce_stats(h->d_stats, h->stats_copies, h->stats_stride, stats_floats(h), h->stream));
        if (launches) (*launches)++;
    }
    std::vector<float> raw(stats_floats(h));
    CU(h, cudaMemcpyAsync(raw.data(), h->d_stats, sizeof(float) * raw.size(), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    for (size_t g = 0; g < (size_t)(ug + ig); g++)
        for (int p = 0; p < K; p++) h->h_stats[g * K + logical_of_phys(K, p)] = raw[g * K + p];
    std::copy(raw.begin() + (size_t)(ug + ig) * K, raw.end(), h->h_stats.begin() + (size_t)(ug + ig) * K);
    h->timings.error_computation_us += now_us() - t0;
    return MASCOT_OK;
}

// Group errors from the sums in h->h_stats and the switching that follows (mf_methods.cu:325-393,
// precision_switching.h:8-51).
int apply_stats(mascot_handle* h, uint32_t epoch, uint32_t* promoted_u, uint32_t* promoted_i, uint32_t* launches) {
    NvtxRange range("mascot: group errors and precision switching");
    const int ug = (int)h->uend.size(), ig = (int)h->iend.size(), K = h->K;
    const double t_err = now_us();
    auto errors = [&](int groups, const float* gsum, const float* nsum, const std::vector<uint8_t>& prec,
                      const std::vector<float>& initial, std::vector<float>& err) {
        for (int g = 0; g < groups; g++) {
            if (prec[g]) { err[g] = -1.f; continue; }
            float num = 0.f;
            for (int d = 0; d < K; d++) num += powf(gsum[(size_t)g * K + d], 2);
            const float den = nsum[g];
            err[g] = (num / den) / initial[g];
        }
    };
    const float* gs_p = h->h_stats.data(); const float* gs_q = gs_p + (size_t)ug * K;
    const float* ns_p = gs_q + (size_t)ig * K; const float* ns_q = ns_p + ug;
    errors(ug, gs_p, ns_p, h->uprec, h->init_uerr, h->uerr);
    errors(ig, gs_q, ns_q, h->iprec, h->init_ierr, h->ierr);
    if (epoch == 5) { h->init_uerr = h->uerr; h->init_ierr = h->ierr; }   // mf_methods.cu:381-388
    h->timings.error_computation_us += now_us() - t_err;
    if (epoch > 5) {
        int rc;
        const double t_sw = now_us();
        for (int side = 0; side < 2; side++) {
            const bool users = side == 0;
            const std::vector<uint8_t>& prec = users ? h->uprec : h->iprec;
            const std::vector<float>& err = users ? h->uerr : h->ierr;
            uint32_t& count = users ? *promoted_u : *promoted_i;
            for (size_t g = 0; g < prec.size(); g++) {
                if (!(err[g] > h->cfg.error_threshold) || prec[g]) continue;
                if ((rc = promote_group(h, users, g)) != MASCOT_OK) return rc;
                count++; if (launches) (*launches)++;
            }
            if (count) {
                if ((rc = recode_side(h, users)) != MASCOT_OK) return rc;
                if (launches) (*launches) += 2;
            }
        }
        if (*promoted_u + *promoted_i) {
            if ((rc = partition_all(h)) != MASCOT_OK) return rc;
            if (launches && h->partitioned) (*launches) += 4;
            CU(h, cudaStreamSynchronize(h->stream));
        }
        h->timings.precision_switching_us += now_us() - t_sw;
    }
    return MASCOT_OK;
}

}  // namespace

extern "C" {

int mascot_is_check_epoch(const mascot_handle* h, uint32_t epoch) {
    return (h && h->grouped && is_check_epoch(h->cfg, epoch)) ? 1 : 0;
}

int mascot_stats_begin(mascot_handle* h) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaMemsetAsync(h->d_stats, 0, sizeof(float) * h->stats_stride * h->stats_copies, h->stream));   // mf_methods.cu:178-182
    return MASCOT_OK;
}

int mascot_train_segment(mascot_handle* h, uint32_t epoch, uint32_t segment, uint32_t collect_stats, mascot_epoch_stats* out) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before training");
    if (segment + 1 >= h->seg_off.size()) return fail(h, MASCOT_ERR_BAD_ARG, "segment index out of range");
    CU(h, cudaSetDevice(h->cfg.device));
    const float lr = epoch < h->lr.size() ? h->lr[epoch] : lr_at(h->cfg, epoch);
    LaunchShape shape; uint32_t launches = 0;
    CU(h, cudaEventRecord(h->ev[0], h->stream));
    const int rc = train_range(h, lr, epoch, segment, collect_stats && h->grouped, &shape, &launches);
    if (rc != MASCOT_OK) return rc;
    CU(h, cudaEventRecord(h->ev[3], h->stream));
    if (out) {
        CU(h, cudaEventSynchronize(h->ev[3]));
        std::memset(out, 0, sizeof(*out));
        out->updates = h->seg_off[segment + 1] - h->seg_off[segment]; out->lr = lr; out->kernel_launches = launches;
        out->workers = shape.workers; out->error_check = (collect_stats && h->grouped) ? 1 : 0;
        cudaEventElapsedTime(&out->kernel_ms, h->ev[0], h->ev[3]);
        out->total_ms = out->kernel_ms;
    }
    return MASCOT_OK;
}

int mascot_stats_fetch(mascot_handle* h, float* grad_sum_p, float* grad_sum_q, float* norm_sum_p, float* norm_sum_q) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    CU(h, cudaSetDevice(h->cfg.device));
    const int rc = fetch_stats(h, nullptr);
    if (rc != MASCOT_OK) return rc;
    return mascot_get_sample_stats(h, grad_sum_p, grad_sum_q, norm_sum_p, norm_sum_q);
}

int mascot_stats_apply(mascot_handle* h, uint32_t epoch, const float* grad_sum_p, const float* grad_sum_q,
                       const float* norm_sum_p, const float* norm_sum_q, uint32_t* promoted_user_groups, uint32_t* promoted_item_groups) {
    if (!h || !grad_sum_p || !grad_sum_q || !norm_sum_p || !norm_sum_q) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set first");
    CU(h, cudaSetDevice(h->cfg.device));
    const size_t ug = h->uend.size(), ig = h->iend.size(), K = h->K;
    float* s = h->h_stats.data();
    std::copy(grad_sum_p, grad_sum_p + ug * K, s);
    std::copy(grad_sum_q, grad_sum_q + ig * K, s + ug * K);
    std::copy(norm_sum_p, norm_sum_p + ug, s + (ug + ig) * K);
    std::copy(norm_sum_q, norm_sum_q + ig, s + (ug + ig) * K + ug);
    uint32_t pu = 0, pi = 0;
    const int rc = apply_stats(h, epoch, &pu, &pi, nullptr);
    if (rc != MASCOT_OK) return rc;
    CU(h, cudaStreamSynchronize(h->stream));
    if (promoted_user_groups) *promoted_user_groups = pu;
    if (promoted_item_groups) *promoted_item_groups = pi;
    return MASCOT_OK;
}

int mascot_train_epoch(mascot_handle* h, uint32_t epoch, mascot_epoch_stats* out) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (h->shard) return fail(h, MASCOT_ERR_STATE, "this engine belongs to a sharded group: use mascot_shard_train_epoch");
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before training");
    NvtxRange range("mascot_train_epoch");
    CU(h, cudaSetDevice(h->cfg.device));
    const float lr = epoch < h->lr.size() ? h->lr[epoch] : lr_at(h->cfg, epoch);
    const bool muppet = h->kind == KIND_MUPPET;
    const int bits_this_epoch = muppet ? muppet_bits(h) : 0;
    // MuPPET samples every epoch (its statistics feed the width policy), MASCOT on its check epochs
    const bool switch_only = h->kind == KIND_SWITCH;
    const bool check = muppet || ((h->grouped || (switch_only && !h->switched_to_fp32)) && is_check_epoch(h->cfg, epoch));
    uint32_t launches = 0, promoted_u = 0, promoted_i = 0;
    const uint64_t bytes_this_epoch = algorithmic_bytes(h);    // with the precisions the kernel is about to see
    CU(h, cudaEventRecord(h->ev[0], h->stream));
    if (check) CU(h, cudaMemsetAsync(h->d_stats, 0, sizeof(float) * h->stats_stride * h->stats_copies, h->stream));   // mf_methods.cu:178-182
    CU(h, cudaEventRecord(h->ev[1], h->stream));
    LaunchShape shape;
    int rc;
    for (size_t sgm = 0; sgm + 1 < h->seg_off.size(); sgm++)
        if ((rc = train_range(h, lr, epoch, sgm, check, &shape, &launches)) != MASCOT_OK) return rc;
    if (check && h->stats_copies > 1) {
        CU(h, launch_reduce_stats(h->d_stats, h->stats_copies, h->stats_stride, stats_floats(h), h->stream));
        launches++;
    }
    CU(h, cudaEventRecord(h->ev[2], h->stream));
    if (check) {
        const int saved = h->stats_copies;
        h->stats_copies = 1;                      // already folded above, inside the timed kernel span
        rc = fetch_stats(h, nullptr);
        h->stats_copies = saved;
        if (rc != MASCOT_OK) return rc;
        if (muppet) muppet_policy(h, epoch);
        else if (switch_only) { if ((rc = switch_only_policy(h, epoch, &promoted_u, &promoted_i)) != MASCOT_OK) return rc; }
        else if ((rc = apply_stats(h, epoch, &promoted_u, &promoted_i, &launches)) != MASCOT_OK) return rc;
    }
    CU(h, cudaEventRecord(h->ev[3], h->stream));
    CU(h, cudaEventSynchronize(h->ev[3]));
    if (out) {
        std::memset(out, 0, sizeof(*out));
        out->updates = h->n_train; out->lr = lr; out->error_check = check ? 1 : 0; out->pass_bits = (uint32_t)bits_this_epoch;
        out->promoted_user_groups = promoted_u; out->promoted_item_groups = promoted_i; out->kernel_launches = launches;
        out->algorithmic_bytes = bytes_this_epoch;
        out->workers = shape.workers;
        cudaEventElapsedTime(&out->kernel_ms, h->ev[1], h->ev[2]);
        cudaEventElapsedTime(&out->total_ms, h->ev[0], h->ev[3]);
    }
    { float kms = 0.f; if (cudaEventElapsedTime(&kms, h->ev[1], h->ev[2]) == cudaSuccess) h->timings.update_us += 1e3 * kms; }
    return MASCOT_OK;
}

int mascot_train_epoch_streamed(mascot_handle* h, uint32_t epoch, const mascot_rating* train, uint64_t n_train, mascot_epoch_stats* out) {
    if (!h || (!train && n_train)) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before training");
    if (h->kind == KIND_AFP) return fail(h, MASCOT_ERR_UNSUPPORTED, "the AFP trainer keeps its per-worker state for a whole epoch: use mascot_train_epoch");
    if (h->shard) return fail(h, MASCOT_ERR_STATE, "this engine belongs to a sharded group: use mascot_shard_train_epoch");
    CU(h, cudaSetDevice(h->cfg.device));
    constexpr uint64_t kPiece = 8ull << 20;           // ratings per piece (96 MiB of input)
    if (!h->copy_stream) {
        CU(h, cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
        for (int b = 0; b < 2; b++) {
            CU(h, cudaEventCreateWithFlags(&h->ev_copied[b], cudaEventDisableTiming));
            CU(h, cudaEventCreateWithFlags(&h->ev_free[b], cudaEventDisableTiming));
        }
    }
    const uint64_t piece = std::min<uint64_t>(kPiece, std::max<uint64_t>(n_train, 1));
    if (h->stage_ratings < piece) {
        for (int b = 0; b < 2; b++) { if (h->d_stage[b]) cudaFree(h->d_stage[b]); h->d_stage[b] = nullptr; }
        h->stage_ratings = 0;
        for (int b = 0; b < 2; b++) CU(h, cudaMalloc(&h->d_stage[b], sizeof(mascot_rating) * piece));
        h->stage_ratings = piece;
    }
    if (n_train != h->n_train) {
        dev_free(h->tr_r); dev_free(h->tr_u); dev_free(h->tr_i); dev_free(h->tr_src);
        CU(h, dev_alloc(&h->tr_r, n_train)); CU(h, dev_alloc(&h->tr_u, n_train)); CU(h, dev_alloc(&h->tr_i, n_train));
        CU(h, dev_alloc(&h->tr_src, n_train));
        h->n_train = n_train;
    }
    CU(h, cudaMemsetAsync(h->d_err_flag, 0, sizeof(uint32_t), h->stream));
    // the pieces become the segments of the resident stream (seeded permutation inside each piece)
    h->seg_off.clear();
    for (uint64_t off = 0; off < n_train; off += piece) h->seg_off.push_back(off);
    h->seg_off.push_back(n_train);
    // The pieces are not partitioned by precision class: finding the class boundaries needs a read-back,
    // i.e. a host wait per piece, which would stall the upload pipeline.  With promoted groups every piece
    // runs the instantiation that reads each id's precision bit; its extra cost hides behind the upload.
    h->cls_off.clear();
    h->partitioned = false;

    const float lr = epoch < h->lr.size() ? h->lr[epoch] : lr_at(h->cfg, epoch);
    const bool muppet = h->kind == KIND_MUPPET;
    const int bits_this_epoch = muppet ? muppet_bits(h) : 0;
    const bool switch_only = h->kind == KIND_SWITCH;
    const bool check = muppet || ((h->grouped || (switch_only && !h->switched_to_fp32)) && is_check_epoch(h->cfg, epoch));
    uint32_t launches = 0, promoted_u = 0, promoted_i = 0;
    const uint64_t bytes_this_epoch = algorithmic_bytes(h);
    CU(h, cudaEventRecord(h->ev[0], h->stream));
    if (check) CU(h, cudaMemsetAsync(h->d_stats, 0, sizeof(float) * h->stats_stride * h->stats_copies, h->stream));
    CU(h, cudaEventRecord(h->ev[1], h->stream));
    LaunchShape shape;
    int rc;
    for (size_t c = 0; c + 1 < h->seg_off.size(); c++) {
        const int b = (int)(c & 1);
        const uint64_t off = h->seg_off[c], len = h->seg_off[c + 1] - off;
        if (c >= 2) CU(h, cudaStreamWaitEvent(h->copy_stream, h->ev_free[b], 0));
        CU(h, cudaMemcpyAsync(h->d_stage[b], train + off, sizeof(mascot_rating) * len, cudaMemcpyHostToDevice, h->copy_stream));
        CU(h, cudaEventRecord(h->ev_copied[b], h->copy_stream));
        CU(h, cudaStreamWaitEvent(h->stream, h->ev_copied[b], 0));
        CU(h, launch_encode_stream(h->d_stage[b], len, h->cfg.shuffle != 0, h->cfg.seed + 0x9e3779b97f4a7c15ull * c, h->d_umap, h->d_imap,
                                   h->d_uprec_row, h->d_iprec_row, h->n_users, h->n_items, h->irows, h->d_err_flag,
                                   h->tr_r + off, h->tr_u + off, h->tr_i + off, h->tr_src ? h->tr_src + off : nullptr, (uint32_t)off, h->stream));
        launches++;
        CU(h, cudaEventRecord(h->ev_free[b], h->stream));
        if ((rc = train_range(h, lr, epoch, c, check, &shape, &launches, n_train)) != MASCOT_OK) return rc;
    }
    if (check && h->stats_copies > 1) {
        CU(h, launch_reduce_stats(h->d_stats, h->stats_copies, h->stats_stride, stats_floats(h), h->stream));
        launches++;
    }
    CU(h, cudaEventRecord(h->ev[2], h->stream));
    if (check) {
        const int saved = h->stats_copies;
        h->stats_copies = 1;
        rc = fetch_stats(h, nullptr);
        h->stats_copies = saved;
        if (rc != MASCOT_OK) return rc;
        if (muppet) muppet_policy(h, epoch);
        else if (switch_only) { if ((rc = switch_only_policy(h, epoch, &promoted_u, &promoted_i)) != MASCOT_OK) return rc; }
        else if ((rc = apply_stats(h, epoch, &promoted_u, &promoted_i, &launches)) != MASCOT_OK) return rc;
    }
    uint32_t bad = 0;
    CU(h, cudaMemcpyAsync(&bad, h->d_err_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaEventRecord(h->ev[3], h->stream));
    CU(h, cudaEventSynchronize(h->ev[3]));
    if (bad) return fail(h, MASCOT_ERR_BAD_ARG, "training rating with id out of range (it was trained as a zero rating of row 0)");
    if (out) {
        std::memset(out, 0, sizeof(*out));
        out->updates = n_train; out->lr = lr; out->error_check = check ? 1 : 0; out->pass_bits = (uint32_t)bits_this_epoch;
        out->promoted_user_groups = promoted_u; out->promoted_item_groups = promoted_i; out->kernel_launches = launches;
        out->algorithmic_bytes = bytes_this_epoch;
        out->workers = shape.workers;
        cudaEventElapsedTime(&out->kernel_ms, h->ev[1], h->ev[2]);
        cudaEventElapsedTime(&out->total_ms, h->ev[0], h->ev[3]);
    }
    { float kms = 0.f; if (cudaEventElapsedTime(&kms, h->ev[1], h->ev[2]) == cudaSuccess) h->timings.update_us += 1e3 * kms; }
    return MASCOT_OK;
}

int mascot_item_rows(mascot_handle* h, uint32_t row_begin, uint32_t row_end, void** f16_ptr, uint64_t* f16_bytes,
                     void** f32_ptr, uint64_t* f32_bytes) {
    if (!h || row_end < row_begin) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    if (row_end > h->n_items) return fail(h, MASCOT_ERR_BAD_ARG, "item row range out of bounds");
    if (h->ilay.parts > 1) return fail(h, MASCOT_ERR_UNSUPPORTED, "the items of a sharded engine are laid out block by block, not by sorted index");
    const size_t b = (size_t)row_begin * h->K, n = (size_t)(row_end - row_begin) * h->K;
    if (f16_ptr) *f16_ptr = h->Q.f16 ? (void*)(h->Q.f16 + b) : nullptr;
    if (f16_bytes) *f16_bytes = h->Q.f16 ? n * sizeof(__half) : 0;
    if (f32_ptr) *f32_ptr = h->Q.f32 ? (void*)(h->Q.f32 + b) : nullptr;
    if (f32_bytes) *f32_bytes = h->Q.f32 ? n * sizeof(float) : 0;
    return MASCOT_OK;
}

int mascot_get_timings(mascot_handle* h, mascot_timings* out) {
    if (!h || !out) return MASCOT_ERR_BAD_ARG;
    *out = h->timings;
    return MASCOT_OK;
}

int mascot_get_worker_count(mascot_handle* h, uint32_t* workers) {
    if (!h || !workers) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    *workers = worker_count(h, h->n_train);
    return MASCOT_OK;
}

int mascot_release_scratch(mascot_handle* h) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaStreamSynchronize(h->stream));
    dev_free(h->d_scratch); h->scratch_bytes = 0;
    return MASCOT_OK;
}

int mascot_sync(mascot_handle* h) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaStreamSynchronize(h->stream));
    return MASCOT_OK;
}

int mascot_get_stream(mascot_handle* h, void** stream) {
    if (!h || !stream) return MASCOT_ERR_BAD_ARG;
    *stream = (void*)h->stream;
    return MASCOT_OK;
}

int mascot_eval_sq_error(mascot_handle* h, double* sum_sq, uint64_t* count) {
    if (!h || !sum_sq || !count) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before evaluation");
    *sum_sq = 0; *count = h->n_test;
    if (!h->n_test) return MASCOT_OK;
    CU(h, cudaSetDevice(h->cfg.device));
    Stream t; t.r = h->te_r; t.u = h->te_u; t.i = h->te_i; t.n = h->n_test;
    CU(h, launch_rmse(h->K, t, h->P, h->Q, h->d_block_err, h->stream));
    CU(h, cudaMemcpyAsync(h->h_block_err.data(), h->d_block_err, sizeof(float) * h->h_block_err.size(), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    double s = 0;
    for (float v : h->h_block_err) s += (double)v;
    *sum_sq = s;
    return MASCOT_OK;
}

int mascot_eval_rmse(mascot_handle* h, double* rmse) {
    if (!h || !rmse) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before evaluation");
    if (!h->n_test) return fail(h, MASCOT_ERR_STATE, "no test ratings were given");
    CU(h, cudaSetDevice(h->cfg.device));
    Stream t; t.r = h->te_r; t.u = h->te_u; t.i = h->te_i; t.n = h->n_test;
    CU(h, launch_rmse(h->K, t, h->P, h->Q, h->d_block_err, h->stream));
    CU(h, cudaMemcpyAsync(h->h_block_err.data(), h->d_block_err, sizeof(float) * h->h_block_err.size(), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    *rmse = (double)reference_rmse_from_partials(h->h_block_err, h->n_test);
    return MASCOT_OK;
}

int mascot_get_factors(mascot_handle* h, float* P, float* Q, int order) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_factors) return fail(h, MASCOT_ERR_STATE, "no factors yet");
    if (order != 0 && order != 1) return fail(h, MASCOT_ERR_BAD_ARG, "order must be 0 or 1");
    CU(h, cudaSetDevice(h->cfg.device));
    auto one = [&](float* dst, Arena a, const uint8_t* prow, uint32_t rows, const uint32_t* map, const RowLayout& lay) -> int {
        if (!dst) return MASCOT_OK;
        float* d = nullptr;
        CU(h, dev_alloc(&d, (size_t)rows * h->K));
        cudaError_t e = launch_gather_factors(h->K, a, prow, rows, order == 0 ? map : nullptr, lay, d, h->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst, d, sizeof(float) * (size_t)rows * h->K, cudaMemcpyDeviceToHost, h->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
        cudaFree(d);
        CU(h, e);
        return MASCOT_OK;
    };
    int rc = one(P, h->P, h->d_uprec_row, h->n_users, h->d_umap, h->ulay);
    if (rc != MASCOT_OK) return rc;
    return one(Q, h->Q, h->d_iprec_row, h->n_items, h->d_imap, h->ilay);
}

int mascot_get_group_info(mascot_handle* h, int side, uint32_t* n_groups, uint32_t* end_idx, uint8_t* precision, float* error) {
    if (!h || (side != 0 && side != 1)) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    const std::vector<uint32_t>& end = side == 0 ? h->uend : h->iend;
    const std::vector<uint8_t>& prec = side == 0 ? h->uprec : h->iprec;
    const std::vector<float>& err = side == 0 ? h->uerr : h->ierr;
    if (n_groups) *n_groups = (uint32_t)end.size();
    if (end_idx) std::copy(end.begin(), end.end(), end_idx);
    if (precision) std::copy(prec.begin(), prec.end(), precision);
    if (error) std::copy(err.begin(), err.end(), error);
    return MASCOT_OK;
}

int mascot_get_index_maps(mascot_handle* h, uint32_t* user2sorted, uint32_t* item2sorted) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    if (user2sorted) {
        if (h->sorted_space) std::copy(h->user2sorted.begin(), h->user2sorted.end(), user2sorted);
        else for (uint32_t e = 0; e < h->n_users; e++) user2sorted[e] = e;
    }
    if (item2sorted) {
        if (h->sorted_space) std::copy(h->item2sorted.begin(), h->item2sorted.end(), item2sorted);
        else for (uint32_t e = 0; e < h->n_items; e++) item2sorted[e] = e;
    }
    return MASCOT_OK;
}

int mascot_promote_group(mascot_handle* h, int side, uint32_t group) {
    if (!h || (side != 0 && side != 1)) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set first");
    if (!h->grouped) return fail(h, MASCOT_ERR_UNSUPPORTED, "only the MASCOT variant stores groups in switchable precision");
    const bool users = side == 0;
    std::vector<uint8_t>& prec = users ? h->uprec : h->iprec;
    if (group >= prec.size()) return fail(h, MASCOT_ERR_BAD_ARG, "group index out of range");
    if (prec[group]) return MASCOT_OK;
    CU(h, cudaSetDevice(h->cfg.device));
    int rc = promote_group(h, users, group);
    if (rc == MASCOT_OK) rc = recode_side(h, users);
    if (rc == MASCOT_OK) rc = partition_all(h);
    if (rc != MASCOT_OK) return rc;
    CU(h, cudaStreamSynchronize(h->stream));
    return MASCOT_OK;
}

int mascot_get_sample_stats(mascot_handle* h, float* grad_sum_p, float* grad_sum_q, float* norm_sum_p, float* norm_sum_q) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    const size_t ug = h->uend.size(), ig = h->iend.size(), K = h->K;
    const float* s = h->h_stats.data();
    if (grad_sum_p) std::copy(s, s + ug * K, grad_sum_p);
    if (grad_sum_q) std::copy(s + ug * K, s + (ug + ig) * K, grad_sum_q);
    if (norm_sum_p) std::copy(s + (ug + ig) * K, s + (ug + ig) * K + ug, norm_sum_p);
    if (norm_sum_q) std::copy(s + (ug + ig) * K + ug, s + (ug + ig) * K + ug + ig, norm_sum_q);
    return MASCOT_OK;
}

int mascot_get_test_ratings(mascot_handle* h, mascot_rating* out, int order) {
    if (!h || !out) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    if (order != 0 && order != 1) return fail(h, MASCOT_ERR_BAD_ARG, "order must be 0 or 1");
    CU(h, cudaSetDevice(h->cfg.device));
    const uint64_t n = h->n_test;
    std::vector<float> r(n); std::vector<uint32_t> u(n), i(n);
    CU(h, cudaMemcpy(r.data(), h->te_r, sizeof(float) * n, cudaMemcpyDeviceToHost));
    CU(h, cudaMemcpy(u.data(), h->te_u, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost));
    CU(h, cudaMemcpy(i.data(), h->te_i, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost));
    std::vector<uint32_t> s2u, s2i;
    if (order == 0 && h->sorted_space) {
        s2u.resize(h->n_users); s2i.resize(h->n_items);
        for (uint32_t e = 0; e < h->n_users; e++) s2u[h->user2sorted[e]] = e;
        for (uint32_t e = 0; e < h->n_items; e++) s2i[h->item2sorted[e]] = e;
    }
    for (uint64_t j = 0; j < n; j++) {
        // the stream holds arena rows: back to sorted indices, then (order 0) to the caller's ids
        uint32_t uu = sorted_of_row(h->ulay, u[j] & kIdMask), ii = sorted_of_row(h->ilay, i[j] & kIdMask);
        if (!s2u.empty()) { uu = s2u[uu]; ii = s2i[ii]; }
        out[j].r = r[j]; out[j].u = uu; out[j].i = ii;
    }
    return MASCOT_OK;
}

int mascot_stream_source_index(const mascot_handle* h, uint64_t pos, uint64_t* src) {
    if (!h || !src) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || pos >= h->n_train) return MASCOT_ERR_BAD_ARG;
    if (!h->cfg.shuffle) { *src = pos; return MASCOT_OK; }
    if (!h->tr_src) return MASCOT_ERR_UNSUPPORTED;       // streams of 2^32 ratings or more keep no map
    uint32_t v = 0;
    if (cudaSetDevice(h->cfg.device) != cudaSuccess ||
        cudaMemcpy(&v, h->tr_src + pos, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return MASCOT_ERR_CUDA;
    *src = v;
    return MASCOT_OK;
}

int mascot_get_stream_order(mascot_handle* h, uint32_t* src_out) {
    if (!h || !src_out) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings) return fail(h, MASCOT_ERR_STATE, "mascot_set_ratings must come first");
    if (!h->tr_src) return fail(h, MASCOT_ERR_UNSUPPORTED, "streams of 2^32 ratings or more keep no order map");
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaMemcpy(src_out, h->tr_src, sizeof(uint32_t) * h->n_train, cudaMemcpyDeviceToHost));
    return MASCOT_OK;
}

int mascot_rmse_device(const float* d_P, const float* d_Q, uint32_t k, const mascot_rating* d_test, uint64_t n_test, double* rmse) {
    if (!d_P || !d_Q || !d_test || !rmse || !n_test) return fail(nullptr, MASCOT_ERR_BAD_ARG, "null pointer or empty test set");
    if (k != 64 && k != 128) return fail(nullptr, MASCOT_ERR_BAD_ARG, "k must be 64 or 128");
    const size_t blocks = (size_t)((n_test + 511) / 512);
    float* d_err = nullptr;
    CU(nullptr, dev_alloc(&d_err, blocks));
    std::vector<float> part(blocks);
    cudaError_t e = launch_rmse_plain((int)k, d_test, n_test, d_P, d_Q, d_err, nullptr);
    if (e == cudaSuccess) e = cudaMemcpy(part.data(), d_err, sizeof(float) * blocks, cudaMemcpyDeviceToHost);
    cudaFree(d_err);
    CU(nullptr, e);
    *rmse = (double)reference_rmse_from_partials(part, n_test);
    return MASCOT_OK;
}

int mascot_rmse_host(const float* P, uint32_t n_users, const float* Q, uint32_t n_items, uint32_t k,
                     const mascot_rating* test, uint64_t n_test, int device, double* rmse) {
    if (!P || !Q || !test || !rmse || !n_test || !n_users || !n_items) return fail(nullptr, MASCOT_ERR_BAD_ARG, "null pointer or empty input");
    if (k != 64 && k != 128) return fail(nullptr, MASCOT_ERR_BAD_ARG, "k must be 64 or 128");
    for (uint64_t j = 0; j < n_test; j++)
        if (test[j].u >= n_users || test[j].i >= n_items) return fail(nullptr, MASCOT_ERR_BAD_ARG, "test rating with id out of range");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) {
        cudaGetLastError();
        return fail(nullptr, MASCOT_ERR_NO_DEVICE, "no usable CUDA device; libmascot has no CPU path");
    }
    CU(nullptr, cudaSetDevice(device));
    float *dP = nullptr, *dQ = nullptr; mascot_rating* dT = nullptr;
    cudaError_t e = dev_alloc(&dP, (size_t)n_users * k);
    if (e == cudaSuccess) e = dev_alloc(&dQ, (size_t)n_items * k);
    if (e == cudaSuccess) e = dev_alloc(&dT, n_test);
    if (e == cudaSuccess) e = cudaMemcpy(dP, P, sizeof(float) * (size_t)n_users * k, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(dQ, Q, sizeof(float) * (size_t)n_items * k, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(dT, test, sizeof(mascot_rating) * n_test, cudaMemcpyHostToDevice);
    int rc = MASCOT_OK;
    if (e == cudaSuccess) rc = mascot_rmse_device(dP, dQ, k, dT, n_test, rmse);
    cudaFree(dP); cudaFree(dQ); cudaFree(dT);
    CU(nullptr, e);
    return rc;
}

}  // extern "C"
