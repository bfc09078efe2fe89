// Rating set-up on the device: everything mascot_set_ratings* does between the caller's arrays and the
// coded training stream.
//
// The reference does this part with a device histogram and a thrust sort, then host loops over the
// entities (user_item_rating_histogram, split_group_based_equal_size_not_strict_ret_end_idx,
// matrix_reconstruction; preprocess_utils.h:54-255), after a host std::map pass over every rating
// (io_utils.h:30-240).  Here one host->device copy of the rating array is followed by kernels only; the
// host touches per-ENTITY tables (degrees, groups, maps: a few MB), never the ratings:
//   1. ids checked against n_users / n_items and degree histogram (atomics)            check_hist_kernel
//   2. entities sorted by (degree, id): stable radix sort of the degrees, ids as values  cub::DeviceRadixSort
//   3. grouping walk over the sorted degrees on the host (O(entities))                   make_groups
//   4. id -> arena row maps, per-row group / precision tables                            host, O(entities)
//   5. sharded engines: ratings of this rank's users selected and ordered by the step of the block
//      schedule at which their item block is here - a stable radix sort of a small key   select_key_kernel
//   6. seeded permutation, item-sorted windows, id remap, precision tags                 launch_encode_stream
//   7. test set: same check, (sharded: this rank's users), sorted by (user, item) like test_set_preprocess
//      (preprocess_utils.h:38-52) with a stable 64-bit radix sort, then coded without shuffling.
#include <algorithm>
#include <cmath>
#include <cstring>

#include <cub/device/device_radix_sort.cuh>

#include "handle.h"

namespace mascot {

namespace {

struct NodeAos { float r; uint32_t u; uint32_t i; };

inline int grid_for(uint64_t n, int block) {
    const uint64_t g = (n + block - 1) / block, cap = (uint64_t)sm_count() * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// An id out of range raises the flag and is NOT used as an index.
__global__ void check_hist_kernel(const NodeAos* R, uint64_t n, uint32_t n_users, uint32_t n_items,
                                  uint32_t* udeg, uint32_t* ideg, uint32_t* err) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t u = R[j].u, i = R[j].i;
        if (u >= n_users || i >= n_items) { atomicOr(err, 1u); continue; }
        if (udeg) atomicAdd(udeg + u, 1u);
        if (ideg) atomicAdd(ideg + i, 1u);
    }
}

__global__ void iota_kernel(uint32_t* v, uint64_t n) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) v[j] = (uint32_t)j;
}

// Which step of the block schedule trains rating j on this rank: users are pinned to ranks, item
// blocks pass by; ratings of other ranks' users get the key `blocks` and sort behind everything kept.
__global__ void select_key_kernel(const NodeAos* R, uint64_t n, const uint32_t* urow_of, const uint32_t* irow_of,
                                  RowLayout ulay, RowLayout ilay, uint32_t rank, uint32_t blocks_per_rank, uint32_t blocks,
                                  uint16_t* key, uint32_t* idx) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t owner = part_of_row(ulay, urow_of[R[j].u]);
        uint32_t k = blocks;
        if (owner == rank) {
            const uint32_t b = part_of_row(ilay, irow_of[R[j].i]);
            k = (b + blocks - (blocks_per_rank * rank) % blocks) % blocks;
        }
        key[j] = (uint16_t)k;
        idx[j] = (uint32_t)j;
    }
}
// test ratings: key 0 = a user of this rank, 1 = somebody else's
__global__ void owner_key_kernel(const NodeAos* R, uint64_t n, const uint32_t* urow_of, RowLayout ulay, uint32_t rank,
                                 uint16_t* key, uint32_t* idx) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        key[j] = part_of_row(ulay, urow_of[R[j].u]) == rank ? 0 : 1;
        idx[j] = (uint32_t)j;
    }
}
__global__ void gather_aos_kernel(const uint32_t* perm, uint64_t n, const NodeAos* in, NodeAos* out) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) out[j] = in[perm[j]];
}
__global__ void key_first_kernel(const uint16_t* key_sorted, uint64_t n, unsigned long long* first) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x)
        if (j == 0 || key_sorted[j] != key_sorted[j - 1]) first[key_sorted[j]] = j;
}
__global__ void compose_kernel(uint32_t* v, uint64_t n, const uint32_t* through) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) v[j] = through[v[j]];
}
__global__ void pair_key_kernel(const NodeAos* R, uint64_t n, unsigned long long* key, uint32_t* idx) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (uint64_t)gridDim.x * blockDim.x) {
        key[j] = ((unsigned long long)R[j].u << 32) | R[j].i;
        idx[j] = (uint32_t)j;
    }
}

// Simple bump allocator over the handle's scratch buffer.
struct Carver {
    unsigned char* base; size_t off = 0;
    explicit Carver(void* p) : base(static_cast<unsigned char*>(p)) {}
    static size_t up(size_t b) { return (b + 255) / 256 * 256; }
    template <typename T> T* take(size_t count) { T* p = reinterpret_cast<T*>(base + off); off += up(sizeof(T) * count); return p; }
};

int bits_for(uint64_t values) { int b = 1; while ((1ull << b) < values) b++; return b; }

// (degree, id) ascending: user_item_rating_histogram's sort_by_key (preprocess_utils.h:87-88) - a stable
// radix sort over ids that start out ascending, so equal degrees keep ascending id order.
int sort_by_degree(mascot_handle* h, const uint32_t* d_deg, uint32_t n, uint32_t* d_deg_sorted, uint32_t* d_s2o,
                   uint32_t* d_iota, void* temp, size_t temp_bytes) {
    iota_kernel<<<grid_for(n, 256), 256, 0, h->stream>>>(d_iota, n);
    CU(h, cudaGetLastError());
    CU(h, cub::DeviceRadixSort::SortPairs(temp, temp_bytes, d_deg, d_deg_sorted, d_iota, d_s2o, (int)n, 0, 32, h->stream));
    return MASCOT_OK;
}

// Host tables of one side from its sorted degrees: groups, maps, per-row flags; uploads the device copies.
int build_side(mascot_handle* h, bool users, const std::vector<uint32_t>& s2o, const std::vector<uint32_t>& cnt_sorted,
               const std::vector<uint32_t>& local_degree_by_id, uint64_t n_local) {
    const uint32_t n = users ? h->n_users : h->n_items;
    const RowLayout& L = users ? h->ulay : h->ilay;
    const uint32_t rows = layout_rows(L);
    std::vector<uint32_t>& end = users ? h->uend : h->iend;
    std::vector<uint8_t>& prec = users ? h->uprec : h->iprec;
    std::vector<uint32_t>& o2s = users ? h->user2sorted : h->item2sorted;
    std::vector<uint64_t>& deg_sum = users ? h->udeg_sum : h->ideg_sum;
    if (h->grouped) {
        make_groups(cnt_sorted, users ? h->cfg.user_group_num : h->cfg.item_group_num, end);
        if (end.size() > 65535) return fail(h, MASCOT_ERR_BAD_ARG, "more than 65535 groups");
        prec.assign(end.size(), 0);
    } else {
        end.assign(1, n - 1);
        prec.assign(1, (h->kind == KIND_MEMQUANT || h->kind == KIND_SWITCH) ? 0 : 1);
    }
    // sorted position -> id (identity when ids are not sorted), id -> sorted position, id -> arena row
    o2s.clear();
    std::vector<uint32_t> row_of_id(n);
    if (h->sorted_space) {
        o2s.resize(n);
        for (uint32_t s = 0; s < n; s++) o2s[s2o[s]] = s;
        for (uint32_t e = 0; e < n; e++) row_of_id[e] = arena_row(L, o2s[e]);
    } else {
        for (uint32_t e = 0; e < n; e++) row_of_id[e] = e;
    }
    // per arena row: group and storage flags; ratings of this engine's stream per group (byte accounting)
    std::vector<uint16_t> group(rows, 0);
    std::vector<uint8_t> flags(rows, 0);
    deg_sum.assign(end.size(), 0);
    if (users) { h->urow_degree.assign(rows, 0); h->hot_user_shift = 0; }
    uint32_t s = 0;
    // A user whose ratings are so many that many workers hold its row at any time: adding up the changes of
    // that many concurrent, equally stale updates multiplies the step and can diverge.  Expected number of
    // workers inside their read-to-write span of a row: c = workers x 4 ratings x degree / n.  Measured: 23 still
    // converges as well as the reference (20M-rating configuration), 82 diverges (252M-rating one).  Above 32 the
    // row is marked, and only one in 2^shift of the updates of marked rows is written back (as a reduction, like
    // every other user row), with 2^shift the power of two that brings the c of the most popular user to 32 or
    // less (one shift per engine: the update kernel gets it as an argument); the other updates of the row are
    // dropped, which is what a plain store does to all but one of the concurrent holders - without the cost of
    // plain stores to a line every SM writes (252M-rating set at quarter size: 10.8 ms per epoch with plain stores
    // for the marked rows, 5.2 ms with reductions for every update, 4.4 ms with no write-back at all).
    const uint64_t w_est = std::min<uint64_t>(worker_count(h, n_local), 16384);
    for (size_t g = 0; g < end.size(); g++) {
        for (; s <= end[g] && s < n; s++) {
            const uint32_t id = h->sorted_space ? s2o[s] : s;
            const uint32_t row = arena_row(L, s);
            const uint32_t deg = local_degree_by_id[id];
            group[row] = (uint16_t)g;
            flags[row] = prec[g] ? kRowPrec : 0;
            deg_sum[g] += deg;
            if (users) {
                h->urow_degree[row] = deg;
                if ((uint64_t)deg * w_est > 8 * n_local) {
                    uint32_t shift = 1;
                    while (shift < 24 && (((uint64_t)deg * w_est) >> shift) > 8 * n_local) shift++;
                    flags[row] |= kRowHot;
                    h->hot_user_shift = std::max(h->hot_user_shift, shift);
                }
            }
        }
    }
    uint16_t** dg = users ? &h->d_ugroup : &h->d_igroup;
    uint8_t** dp = users ? &h->d_uprec_row : &h->d_iprec_row;
    uint32_t** dm = users ? &h->d_umap : &h->d_imap;
    CU(h, dev_alloc(dg, rows)); CU(h, dev_alloc(dp, rows));
    CU(h, cudaMemcpyAsync(*dg, group.data(), sizeof(uint16_t) * rows, cudaMemcpyHostToDevice, h->stream));
    CU(h, cudaMemcpyAsync(*dp, flags.data(), sizeof(uint8_t) * rows, cudaMemcpyHostToDevice, h->stream));
    if (h->sorted_space) {
        CU(h, dev_alloc(dm, n));
        CU(h, cudaMemcpyAsync(*dm, row_of_id.data(), sizeof(uint32_t) * n, cudaMemcpyHostToDevice, h->stream));
    }
    CU(h, cudaStreamSynchronize(h->stream));       // the host vectors above end with this call
    return MASCOT_OK;
}

}  // namespace

int setup_ratings(mascot_handle* h, const SetupRequest& rq) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    const uint32_t n_users = rq.n_users, n_items = rq.n_items;
    if ((!rq.train && rq.n_train) || (!rq.test && rq.n_test)) return fail(h, MASCOT_ERR_BAD_ARG, "null rating array");
    if (!n_users || !n_items || n_users > kIdMask || n_items > kIdMask) return fail(h, MASCOT_ERR_BAD_ARG, "user/item count out of range");
    if (rq.n_train >= (1ull << 32) || rq.n_test >= (1ull << 32)) return fail(h, MASCOT_ERR_BAD_ARG, "too many ratings (limit 2^32 - 1 per engine)");
    if (rq.n_segments == 0 || (rq.n_segments > 1 && !rq.segment_offsets)) return fail(h, MASCOT_ERR_BAD_ARG, "bad segment table");
    if ((rq.user_degree == nullptr) != (rq.item_degree == nullptr)) return fail(h, MASCOT_ERR_BAD_ARG, "give both degree tables or none");
    const bool sharded = rq.rank >= 0;
    if (sharded && (rq.world < 1 || rq.rank >= rq.world || rq.blocks != rq.blocks_per_rank * (uint32_t)rq.world || rq.blocks > 4096))
        return fail(h, MASCOT_ERR_BAD_ARG, "bad rank / world / block count");
    std::vector<uint64_t> seg(rq.n_segments + 1);
    if (rq.segment_offsets) {
        for (uint32_t j = 0; j <= rq.n_segments; j++) seg[j] = rq.segment_offsets[j];
        if (seg[0] != 0 || seg[rq.n_segments] != rq.n_train) return fail(h, MASCOT_ERR_BAD_ARG, "segment offsets must run from 0 to n_train");
        for (uint32_t j = 0; j < rq.n_segments; j++) if (seg[j] > seg[j + 1]) return fail(h, MASCOT_ERR_BAD_ARG, "segment offsets must not decrease");
    } else { seg[0] = 0; seg[1] = rq.n_train; }
    NvtxRange range("mascot: rating set-up");
    CU(h, cudaSetDevice(h->cfg.device));
    l2_window_remove(h);
    free_ratings(h);
    h->n_users = n_users; h->n_items = n_items; h->n_test = 0; h->n_train = 0;
    h->cls_off.clear(); h->partitioned = false;
    h->sorted_space = h->grouped || sharded;
    h->ulay = RowLayout(); h->ilay = RowLayout();
    h->ulay.n = n_users; h->ilay.n = n_items;
    if (sharded && rq.world > 1) { h->ulay.parts = (uint32_t)rq.world; h->ulay.rows_per_part = (n_users + rq.world - 1) / rq.world; h->ulay.snake = 1; }
    if (sharded && rq.blocks > 1) { h->ilay.parts = rq.blocks; h->ilay.rows_per_part = (n_items + rq.blocks - 1) / rq.blocks; }
    h->urows = layout_rows(h->ulay); h->irows = layout_rows(h->ilay);
    if (!h->d_err_flag) CU(h, dev_alloc(&h->d_err_flag, 1));
    CU(h, cudaMemsetAsync(h->d_err_flag, 0, sizeof(uint32_t), h->stream));

    // ---- scratch: the uploaded arrays and the sort buffers ----
    const uint64_t n_all = rq.n_train, n_big = std::max<uint64_t>(n_all, rq.n_test);
    const uint32_t n_ent = std::max(n_users, n_items);
    size_t temp_bytes = 0, tb = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tb, (const uint32_t*)nullptr, (uint32_t*)nullptr, (const uint32_t*)nullptr, (uint32_t*)nullptr, (int)n_ent, 0, 32);
    temp_bytes = std::max(temp_bytes, tb);
    cub::DeviceRadixSort::SortPairs(nullptr, tb, (const uint16_t*)nullptr, (uint16_t*)nullptr, (const uint32_t*)nullptr, (uint32_t*)nullptr, n_big, 0, 16);
    temp_bytes = std::max(temp_bytes, tb);
    cub::DeviceRadixSort::SortPairs(nullptr, tb, (const unsigned long long*)nullptr, (unsigned long long*)nullptr, (const uint32_t*)nullptr, (uint32_t*)nullptr, rq.n_test, 0, 64);
    temp_bytes = std::max(temp_bytes, tb);
    const size_t need = Carver::up(sizeof(NodeAos) * n_big) * 2 + Carver::up(8 * n_big) * 2 + Carver::up(4 * n_big) * 2 +
                        Carver::up(4 * (size_t)n_ent) * 6 + Carver::up(temp_bytes) + Carver::up(8 * 4100) + 4096;
    int rc = need_scratch(h, need);
    if (rc != MASCOT_OK) return rc;
    Carver cv(h->d_scratch);
    NodeAos* aos = cv.take<NodeAos>(n_big);
    NodeAos* aos2 = cv.take<NodeAos>(n_big);
    unsigned long long* key64_a = cv.take<unsigned long long>(n_big);      // also used as 16-bit keys
    unsigned long long* key64_b = cv.take<unsigned long long>(n_big);
    uint32_t* idx_a = cv.take<uint32_t>(n_big);
    uint32_t* idx_b = cv.take<uint32_t>(n_big);
    uint32_t* d_udeg = cv.take<uint32_t>(n_ent);
    uint32_t* d_ideg = cv.take<uint32_t>(n_ent);
    uint32_t* d_sorted_deg = cv.take<uint32_t>(n_ent);
    uint32_t* d_s2o = cv.take<uint32_t>(n_ent);
    uint32_t* d_iota = cv.take<uint32_t>(n_ent);
    uint32_t* d_ldeg = cv.take<uint32_t>(n_ent);        // local degrees of the second side, see below
    void* temp = cv.take<unsigned char>(temp_bytes);
    unsigned long long* d_first = cv.take<unsigned long long>(4100);
    uint16_t* key16_a = reinterpret_cast<uint16_t*>(key64_a);
    uint16_t* key16_b = reinterpret_cast<uint16_t*>(key64_b);

    double t_phase = now_us();
    // ---- 1. training ratings: upload, check, degrees ----
    if (n_all) CU(h, cudaMemcpyAsync(aos, rq.train, sizeof(NodeAos) * n_all, cudaMemcpyHostToDevice, h->stream));
    CU(h, cudaMemsetAsync(d_udeg, 0, sizeof(uint32_t) * n_users, h->stream));
    CU(h, cudaMemsetAsync(d_ideg, 0, sizeof(uint32_t) * n_items, h->stream));
    if (n_all) {
        check_hist_kernel<<<grid_for(n_all, 256), 256, 0, h->stream>>>(aos, n_all, n_users, n_items, d_udeg, d_ideg, h->d_err_flag);
        CU(h, cudaGetLastError());
    }
    uint32_t bad = 0;
    CU(h, cudaMemcpyAsync(&bad, h->d_err_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    if (bad) return fail(h, MASCOT_ERR_BAD_ARG, "training rating with id out of range");
    // degrees that define the index space: those of the array (the whole data set for library-side
    // sharding) or the tables a caller-sharded engine was given
    std::vector<uint32_t> udeg_local(n_users), ideg_local(n_items);
    CU(h, cudaMemcpyAsync(udeg_local.data(), d_udeg, sizeof(uint32_t) * n_users, cudaMemcpyDeviceToHost, h->stream));
    CU(h, cudaMemcpyAsync(ideg_local.data(), d_ideg, sizeof(uint32_t) * n_items, cudaMemcpyDeviceToHost, h->stream));
    if (rq.user_degree) {
        CU(h, cudaMemcpyAsync(d_udeg, rq.user_degree, sizeof(uint32_t) * n_users, cudaMemcpyHostToDevice, h->stream));
        CU(h, cudaMemcpyAsync(d_ideg, rq.item_degree, sizeof(uint32_t) * n_items, cudaMemcpyHostToDevice, h->stream));
    }

    // ---- 2.-4. degree sort, groups, maps ----
    std::vector<uint32_t> us2o, is2o, ucnt, icnt;
    if (h->sorted_space) {
        us2o.resize(n_users); ucnt.resize(n_users); is2o.resize(n_items); icnt.resize(n_items);
        if ((rc = sort_by_degree(h, d_udeg, n_users, d_sorted_deg, d_s2o, d_iota, temp, temp_bytes)) != MASCOT_OK) return rc;
        CU(h, cudaMemcpyAsync(us2o.data(), d_s2o, sizeof(uint32_t) * n_users, cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaMemcpyAsync(ucnt.data(), d_sorted_deg, sizeof(uint32_t) * n_users, cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaStreamSynchronize(h->stream));
        if ((rc = sort_by_degree(h, d_ideg, n_items, d_sorted_deg, d_s2o, d_iota, temp, temp_bytes)) != MASCOT_OK) return rc;
        CU(h, cudaMemcpyAsync(is2o.data(), d_s2o, sizeof(uint32_t) * n_items, cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaMemcpyAsync(icnt.data(), d_sorted_deg, sizeof(uint32_t) * n_items, cudaMemcpyDeviceToHost, h->stream));
    }
    CU(h, cudaStreamSynchronize(h->stream));
    h->timings.rating_histogram_us += now_us() - t_phase; t_phase = now_us();

    uint64_t n_local = n_all;
    if (sharded) {
        // the ratings of this rank's users: the sum of their degrees (users are pinned to one rank)
        n_local = 0;
        for (uint32_t s = 0; s < n_users; s++)
            if (part_of_row(h->ulay, arena_row(h->ulay, s)) == (uint32_t)rq.rank) n_local += ucnt[s];
    }
    h->n_train = n_local;          // the automatic worker count and the hot-user mark follow this engine's own stream
    if ((rc = build_side(h, true, us2o, ucnt, udeg_local, n_local)) != MASCOT_OK) return rc;

    h->timings.grouping_us += now_us() - t_phase; t_phase = now_us();
    // ---- 5. sharded: keep this rank's ratings, one segment per step of the block schedule ----
    const NodeAos* enc_src = aos;
    const uint32_t* src_through = nullptr;
    if (sharded) {
        // item rows are needed for the block of a rating: build the item map first (flags come later, with local degrees)
        if ((rc = build_side(h, false, is2o, icnt, ideg_local, std::max<uint64_t>(n_local, 1))) != MASCOT_OK) return rc;
        const int kb = bits_for((uint64_t)rq.blocks + 1);
        if (n_all) {
            select_key_kernel<<<grid_for(n_all, 256), 256, 0, h->stream>>>(aos, n_all, h->d_umap, h->d_imap, h->ulay, h->ilay, (uint32_t)rq.rank,
                                                                          rq.blocks_per_rank, rq.blocks, key16_a, idx_a);
            CU(h, cudaGetLastError());
            CU(h, cub::DeviceRadixSort::SortPairs(temp, temp_bytes, key16_a, key16_b, idx_a, idx_b, n_all, 0, kb, h->stream));
            gather_aos_kernel<<<grid_for(n_all, 256), 256, 0, h->stream>>>(idx_b, n_all, aos, aos2);
            CU(h, cudaGetLastError());
            CU(h, cudaMemsetAsync(d_first, 0xff, sizeof(unsigned long long) * (rq.blocks + 1), h->stream));
            key_first_kernel<<<grid_for(n_all, 256), 256, 0, h->stream>>>(key16_b, n_all, d_first);
            CU(h, cudaGetLastError());
        }
        std::vector<unsigned long long> first(rq.blocks + 1, ~0ull);
        if (n_all) CU(h, cudaMemcpyAsync(first.data(), d_first, sizeof(unsigned long long) * first.size(), cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaStreamSynchronize(h->stream));
        seg.assign(rq.blocks + 1, 0);
        uint64_t end_pos = first[rq.blocks] == ~0ull ? n_all : first[rq.blocks];      // where the discarded ratings begin
        seg[rq.blocks] = end_pos;
        for (int t = (int)rq.blocks - 1; t >= 0; t--) seg[t] = first[t] == ~0ull ? seg[t + 1] : first[t];
        if (end_pos != n_local) return fail(h, MASCOT_ERR_STATE, "internal: selected ratings do not add up to the users' degrees");
        enc_src = aos2;
        src_through = idx_b;
        // local item degrees of the kept ratings, for the byte accounting of the item groups
        CU(h, cudaMemsetAsync(d_ldeg, 0, sizeof(uint32_t) * n_items, h->stream));
        if (n_local) {
            check_hist_kernel<<<grid_for(n_local, 256), 256, 0, h->stream>>>(aos2, n_local, n_users, n_items, nullptr, d_ldeg, h->d_err_flag);
            CU(h, cudaGetLastError());
        }
        CU(h, cudaMemcpyAsync(ideg_local.data(), d_ldeg, sizeof(uint32_t) * n_items, cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaStreamSynchronize(h->stream));
        dev_free(h->d_igroup); dev_free(h->d_iprec_row); dev_free(h->d_imap);
    }
    { const double t_g = now_us();
      if ((rc = build_side(h, false, is2o, icnt, ideg_local, std::max<uint64_t>(n_local, 1))) != MASCOT_OK) return rc;
      h->timings.grouping_us += now_us() - t_g; t_phase += now_us() - t_g; }
    h->seg_off = seg;
    h->n_train_accounted = n_local;
    h->uerr.assign(h->uend.size(), 0.f); h->ierr.assign(h->iend.size(), 0.f);
    h->init_uerr.assign(h->uend.size(), 1.f); h->init_ierr.assign(h->iend.size(), 1.f);   // mf_methods.cu:150-151

    // ---- 6. the coded training stream ----
    CU(h, dev_alloc(&h->tr_r, n_local)); CU(h, dev_alloc(&h->tr_u, n_local)); CU(h, dev_alloc(&h->tr_i, n_local));
    CU(h, dev_alloc(&h->tr_src, n_local));
    if (n_local) {
        CU(h, encode_segments(h, reinterpret_cast<const mascot_rating*>(enc_src), seg, h->cfg.shuffle != 0, h->tr_r, h->tr_u, h->tr_i, h->tr_src));
        if (src_through) {          // positions in the caller's array, not in the selected copy
            compose_kernel<<<grid_for(n_local, 256), 256, 0, h->stream>>>(h->tr_src, n_local, src_through);
            CU(h, cudaGetLastError());
        }
    }

    // ---- 7. the test set ----
    uint64_t n_test = rq.n_test;
    if (rq.n_test) {
        CU(h, cudaStreamSynchronize(h->stream));          // aos / aos2 are reused
        CU(h, cudaMemcpyAsync(aos, rq.test, sizeof(NodeAos) * rq.n_test, cudaMemcpyHostToDevice, h->stream));
        check_hist_kernel<<<grid_for(rq.n_test, 256), 256, 0, h->stream>>>(aos, rq.n_test, n_users, n_items, nullptr, nullptr, h->d_err_flag);
        CU(h, cudaGetLastError());
        CU(h, cudaMemcpyAsync(&bad, h->d_err_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
        CU(h, cudaStreamSynchronize(h->stream));
        if (bad) return fail(h, MASCOT_ERR_BAD_ARG, "test rating with id out of range");
        NodeAos* cur = aos; NodeAos* other = aos2;
        if (sharded && rq.world > 1) {
            owner_key_kernel<<<grid_for(rq.n_test, 256), 256, 0, h->stream>>>(cur, rq.n_test, h->d_umap, h->ulay, (uint32_t)rq.rank, key16_a, idx_a);
            CU(h, cudaGetLastError());
            CU(h, cub::DeviceRadixSort::SortPairs(temp, temp_bytes, key16_a, key16_b, idx_a, idx_b, rq.n_test, 0, 1, h->stream));
            gather_aos_kernel<<<grid_for(rq.n_test, 256), 256, 0, h->stream>>>(idx_b, rq.n_test, cur, other);
            CU(h, cudaGetLastError());
            CU(h, cudaMemsetAsync(d_first, 0xff, sizeof(unsigned long long) * 2, h->stream));
            key_first_kernel<<<grid_for(rq.n_test, 256), 256, 0, h->stream>>>(key16_b, rq.n_test, d_first);
            CU(h, cudaGetLastError());
            unsigned long long first[2] = {~0ull, ~0ull};
            CU(h, cudaMemcpyAsync(first, d_first, sizeof(first), cudaMemcpyDeviceToHost, h->stream));
            CU(h, cudaStreamSynchronize(h->stream));
            n_test = first[1] == ~0ull ? rq.n_test : first[1];
            std::swap(cur, other);
        }
        if (n_test) {
            // test_set_preprocess (preprocess_utils.h:38-52) leaves the test set ordered by (user, item)
            pair_key_kernel<<<grid_for(n_test, 256), 256, 0, h->stream>>>(cur, n_test, key64_a, idx_a);
            CU(h, cudaGetLastError());
            CU(h, cub::DeviceRadixSort::SortPairs(temp, temp_bytes, key64_a, key64_b, idx_a, idx_b, n_test, 0, 64, h->stream));
            gather_aos_kernel<<<grid_for(n_test, 256), 256, 0, h->stream>>>(idx_b, n_test, cur, other);
            CU(h, cudaGetLastError());
            std::swap(cur, other);
        }
        CU(h, dev_alloc(&h->te_r, n_test)); CU(h, dev_alloc(&h->te_u, n_test)); CU(h, dev_alloc(&h->te_i, n_test));
        if (n_test) {
            const std::vector<uint64_t> whole = {0, n_test};
            CU(h, encode_segments(h, reinterpret_cast<const mascot_rating*>(cur), whole, false, h->te_r, h->te_u, h->te_i, nullptr));
        }
    } else {
        CU(h, dev_alloc(&h->te_r, 0)); CU(h, dev_alloc(&h->te_u, 0)); CU(h, dev_alloc(&h->te_i, 0));
    }
    h->n_test = n_test;
    CU(h, cudaStreamSynchronize(h->stream));
    h->timings.reconstruction_us += now_us() - t_phase; t_phase = now_us();

    // ---- factor arenas and statistics ----
    const size_t pu = (size_t)h->urows * h->K, qi = (size_t)h->irows * h->K;
    if (h->kind == KIND_MIXED || h->kind == KIND_MEMQUANT || h->kind == KIND_SWITCH) {
        CU(h, dev_alloc(&h->P.f16, pu)); CU(h, dev_alloc(&h->Q.f16, qi));
        CU(h, cudaMemsetAsync(h->P.f16, 0, sizeof(__half) * pu, h->stream)); CU(h, cudaMemsetAsync(h->Q.f16, 0, sizeof(__half) * qi, h->stream));
    }
    if (h->kind != KIND_MEMQUANT) {
        CU(h, dev_alloc(&h->P.f32, pu)); CU(h, dev_alloc(&h->Q.f32, qi));
        CU(h, cudaMemsetAsync(h->P.f32, 0, sizeof(float) * pu, h->stream)); CU(h, cudaMemsetAsync(h->Q.f32, 0, sizeof(float) * qi, h->stream));
    }
    h->stats_copies = h->cfg.deterministic ? 1 : kStatCopies;
    h->stats_stride = (stats_floats(h) + 63) / 64 * 64;
    CU(h, dev_alloc(&h->d_stats, h->stats_stride * h->stats_copies));
    CU(h, cudaMemsetAsync(h->d_stats, 0, sizeof(float) * h->stats_stride * h->stats_copies, h->stream));
    h->h_stats.assign(stats_floats(h), 0.f);
    const size_t blocks = (size_t)((n_test + 511) / 512);
    CU(h, dev_alloc(&h->d_block_err, blocks));
    h->h_block_err.assign(blocks, 0.f);
    CU(h, cudaStreamSynchronize(h->stream));
    // the set-up's own use of the scratch buffer is over: the sort below may re-carve it
    const int rc_sort = sort_run_windows(h);
    if (rc_sort != MASCOT_OK) return rc_sort;
    const int rc_warm = warm_kernels(h);
    if (rc_warm != MASCOT_OK) return rc_warm;
    h->timings.additional_init_us += now_us() - t_phase;
    h->have_ratings = true;
    return MASCOT_OK;
}

}  // namespace mascot
