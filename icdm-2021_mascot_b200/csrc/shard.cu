// Sharded (multi-GPU) training inside the library: one engine per GPU, one host thread or process per
// engine, NCCL between them.  No counterpart in the reference, which is single-GPU.
//
// SCHEME.  Users are pinned: they are dealt to the ranks by degree (layout.cuh, snake order), with their
// ratings and their rows of P.  Items are cut into B = world x blocks_per_gpu blocks (sorted index s
// belongs to block s mod B), each block one contiguous range of the item arena.  Step t of an epoch:
// rank g trains its ratings whose item lies in block (m g + t) mod B (m = blocks_per_gpu), then passes
// that block to rank g-1, which trains it m steps later.  At any time the ranks work on disjoint users
// and disjoint item blocks, so no update is ever lost between GPUs, and after B steps every block is
// back where it started.  With m = 1 a rank needs the block its neighbour has just finished: transfer
// and updates alternate.  With m = 2 a block travels while its receiver trains another one: the
// transfers run on their own stream under the update kernels.  The price of m = 2 is that the workers of
// a GPU crowd on half as many item rows at a time, which costs convergence per epoch (measured); the
// caller chooses.
//
// The sampled statistics of a check epoch are all-reduced on the device and every rank takes the same
// switching decisions; the test error is all-reduced after an all-gather of the item blocks.
//
// NCCL is loaded with dlopen when the first group is formed, so a process that trains on one GPU needs
// no NCCL at all.  Every host-side wait that depends on another rank is a bounded poll (bounded_wait.h):
// when the limit passes the communicator is aborted and the call returns MASCOT_ERR_TIMEOUT; an
// asynchronous NCCL error returns MASCOT_ERR_COMM.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>

#include "bounded_wait.h"
#include "handle.h"

namespace mascot {

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
};

std::mutex g_api_mutex;
NcclApi g_api;

// Loads NCCL once per process.  A copy that the process has loaded already (same soname) is reused.
const NcclApi* nccl_api(std::string* why) {
    std::lock_guard<std::mutex> lock(g_api_mutex);
    if (g_api.lib) return &g_api;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) { if (why) *why = std::string("cannot load NCCL: ") + dlerror(); return nullptr; }
    NcclApi a;
    a.lib = lib;
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(lib, name); if (!p) ok = false; return p; };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
    a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
    if (!ok) { if (why) *why = "the NCCL library lacks a required symbol"; dlclose(lib); return nullptr; }
    g_api = a;
    return &g_api;
}

}  // namespace

struct ShardCtx {
    const NcclApi* api = nullptr;
    ncclComm_t comm = nullptr;
    bool comm_dead = false;                 // aborted after a timeout or an error: every later call fails
    int rank = 0, world = 1;
    uint32_t m = 1, blocks = 1;             // blocks per GPU, blocks in all
    uint32_t timeout_ms = 60000;
    uint64_t n_global = 0;                  // training ratings of the whole group
    cudaStream_t comm_stream = nullptr;
    std::vector<cudaEvent_t> ev_trained;    // per step: the update kernel of the step has finished
    std::vector<cudaEvent_t> ev_arrived;    // per block: the last transfer into this block has finished
    std::vector<uint8_t> arrival_pending;   // per block: a transfer into it was queued since it was last trained
    double* d_pair = nullptr;               // device scratch: (sum of squared errors, count)
    uint64_t bytes_sent = 0;                // item-block bytes this rank has sent so far
};

namespace {

#define NC(h, S, call)                                                                              \
    do {                                                                                            \
        ncclResult_t r_ = (call);                                                                   \
        if (r_ != ncclSuccess) {                                                                    \
            char buf_[512];                                                                         \
            snprintf(buf_, sizeof buf_, "%s failed: %s (%s:%d)", #call, (S)->api->GetErrorString(r_), __FILE__, __LINE__); \
            return fail(h, MASCOT_ERR_COMM, buf_);                                                  \
        }                                                                                           \
    } while (0)

// Waits until everything queued on `stream` has run, for at most the group's limit.
int wait_stream(mascot_handle* h, cudaStream_t stream, const char* what) {
    ShardCtx* S = h->shard;
    cudaError_t cuda_error = cudaSuccess;
    ncclResult_t nccl_error = ncclSuccess;
    const int rc = bounded_wait([&]() -> int {
        const cudaError_t q = cudaStreamQuery(stream);
        if (q == cudaSuccess) return 1;
        if (q != cudaErrorNotReady) { cuda_error = q; return MASCOT_ERR_CUDA; }
        if (S && S->comm && !S->comm_dead) {
            ncclResult_t a = ncclSuccess;
            if (S->api->CommGetAsyncError(S->comm, &a) != ncclSuccess || (a != ncclSuccess && a != ncclInProgress)) { nccl_error = a; return MASCOT_ERR_COMM; }
        }
        return 0;
    }, S ? S->timeout_ms : 60000u);
    if (rc == MASCOT_OK) return MASCOT_OK;
    if (S && S->comm && !S->comm_dead && (rc == MASCOT_ERR_TIMEOUT || rc == MASCOT_ERR_COMM)) {
        S->api->CommAbort(S->comm);           // ends the communicator's kernels, so the streams drain
        S->comm = nullptr; S->comm_dead = true;
    }
    char buf[256];
    if (rc == MASCOT_ERR_TIMEOUT) snprintf(buf, sizeof buf, "%s: no progress within %u ms (another rank missing?); the group was dissolved", what, S ? S->timeout_ms : 0u);
    else if (rc == MASCOT_ERR_COMM) snprintf(buf, sizeof buf, "%s: NCCL reported %s; the group was dissolved", what, S->api->GetErrorString(nccl_error));
    else snprintf(buf, sizeof buf, "%s: %s", what, cudaGetErrorString(cuda_error));
    return fail(h, rc, buf);
}

int usable(mascot_handle* h) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->shard) return fail(h, MASCOT_ERR_STATE, "mascot_shard_init must come first");
    if (h->shard->comm_dead) return fail(h, MASCOT_ERR_COMM, "the group of this engine was dissolved after a communication failure");
    return MASCOT_OK;
}

// Which item arenas hold live rows: a row lives in exactly one of them, by its group's precision, so an
// arena without live rows need not travel.  Every rank reaches the same answer.
void live_item_arenas(const mascot_handle* h, bool* f16, bool* f32) {
    *f16 = false; *f32 = false;
    for (uint8_t p : h->iprec) { if (p) *f32 = true; else *f16 = true; }
    if (!h->Q.f16) *f16 = false;
    if (!h->Q.f32) *f32 = false;
}

// Queues, on the transfer stream, the hand-over that follows the training of `sent_block`: it goes to
// rank-1, and `recv_block` - which rank+1 has just trained - arrives.
int queue_exchange(mascot_handle* h, uint32_t sent_block, uint32_t recv_block) {
    ShardCtx* S = h->shard;
    const int to = (S->rank + S->world - 1) % S->world, from = (S->rank + 1) % S->world;
    const size_t rows = h->ilay.rows_per_part, elems = rows * (size_t)h->K;
    bool f16, f32;
    live_item_arenas(h, &f16, &f32);
    NC(h, S, S->api->GroupStart());
    if (f16) {
        NC(h, S, S->api->Send(h->Q.f16 + (size_t)sent_block * elems, elems, ncclHalf, to, S->comm, S->comm_stream));
        NC(h, S, S->api->Recv(h->Q.f16 + (size_t)recv_block * elems, elems, ncclHalf, from, S->comm, S->comm_stream));
        S->bytes_sent += elems * sizeof(__half);
    }
    if (f32) {
        NC(h, S, S->api->Send(h->Q.f32 + (size_t)sent_block * elems, elems, ncclFloat, to, S->comm, S->comm_stream));
        NC(h, S, S->api->Recv(h->Q.f32 + (size_t)recv_block * elems, elems, ncclFloat, from, S->comm, S->comm_stream));
        S->bytes_sent += elems * sizeof(float);
    }
    NC(h, S, S->api->GroupEnd());
    return MASCOT_OK;
}

// All-gather of the arenas of one side over the home ranges of the ranks (in place).
int gather_side(mascot_handle* h, Arena a, const RowLayout& L, uint32_t parts_per_rank, bool f16, bool f32, cudaStream_t st) {
    ShardCtx* S = h->shard;
    const size_t elems = (size_t)L.rows_per_part * parts_per_rank * h->K;
    if (f16 && a.f16) NC(h, S, S->api->AllGather(a.f16 + elems * S->rank, a.f16, elems, ncclHalf, S->comm, st));
    if (f32 && a.f32) NC(h, S, S->api->AllGather(a.f32 + elems * S->rank, a.f32, elems, ncclFloat, S->comm, st));
    return MASCOT_OK;
}

}  // namespace

unsigned shard_worker_count(const mascot_handle* h) {
    // What decides the convergence per epoch of these racy updates is how many workers touch one row at
    // the same time.  A rank puts all its workers on 1/world of the items (and of the users), so a row
    // sees `world` times the per-rank count: the total over all ranks has to stay bounded, not the
    // count per GPU - which also means that more GPUs shorten an epoch only as far as the total grows.
    // Measured on the 100M-rating configuration on four GPUs (total / updates per second / epoch and time at
    // which the reference's final RMSE is reached / RMSE after 50 epochs): 18.9k / 33.8e9 / 33, 99 ms / 0.5998;
    // 28.4k / 38.0e9 / 38, 100 ms / 0.6003; 37.9k / 38.9e9 / 47, 132 ms / 0.6011.  About 28k (n / 3584, 2.3 times
    // the single-GPU automatic choice n / 8192) is used: the largest total that costs no time to the target RMSE.
    const ShardCtx* S = h->shard;
    const uint64_t total = std::max<uint64_t>(S->n_global / 3584, 512);
    const uint64_t w = std::max<uint64_t>(total / (uint64_t)S->world, 64);
    return (unsigned)w;
}

void shard_destroy(mascot_handle* h) {
    ShardCtx* S = h->shard;
    if (!S) return;
    if (S->comm && !S->comm_dead) {
        // a communicator with work in flight is aborted, an idle one is destroyed
        if (S->comm_stream && cudaStreamQuery(S->comm_stream) == cudaSuccess && cudaStreamQuery(h->stream) == cudaSuccess) S->api->CommDestroy(S->comm);
        else S->api->CommAbort(S->comm);
    }
    for (cudaEvent_t e : S->ev_trained) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : S->ev_arrived) if (e) cudaEventDestroy(e);
    if (S->comm_stream) cudaStreamDestroy(S->comm_stream);
    if (S->d_pair) cudaFree(S->d_pair);
    delete S;
    h->shard = nullptr;
}

}  // namespace mascot

using namespace mascot;

extern "C" {

int mascot_shard_schedule(uint32_t world, uint32_t blocks_per_gpu, uint32_t rank, uint32_t step,
                          uint32_t* train_block, uint32_t* send_to, uint32_t* recv_block, uint32_t* recv_from) {
    if (!world || !blocks_per_gpu || rank >= world || step >= world * blocks_per_gpu) return MASCOT_ERR_BAD_ARG;
    const uint32_t B = world * blocks_per_gpu;
    const uint32_t b = (blocks_per_gpu * rank + step) % B;
    if (train_block) *train_block = b;
    if (send_to) *send_to = (rank + world - 1) % world;
    if (recv_block) *recv_block = (b + blocks_per_gpu) % B;
    if (recv_from) *recv_from = (rank + 1) % world;
    return MASCOT_OK;
}

int mascot_comm_unique_id(void* id_out) {
    if (!id_out) return MASCOT_ERR_BAD_ARG;
    std::string why;
    const NcclApi* api = nccl_api(&why);
    if (!api) return fail(nullptr, MASCOT_ERR_COMM, why);
    static_assert(sizeof(ncclUniqueId) == MASCOT_COMM_ID_BYTES, "the id is passed around as 128 opaque bytes");
    ncclUniqueId id;
    const ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) return fail(nullptr, MASCOT_ERR_COMM, std::string("ncclGetUniqueId failed: ") + api->GetErrorString(r));
    std::memcpy(id_out, &id, sizeof id);
    return MASCOT_OK;
}

int mascot_shard_init(mascot_handle* h, const void* id, uint32_t rank, uint32_t world, uint32_t blocks_per_gpu, uint32_t timeout_ms) {
    if (!h || !id) return MASCOT_ERR_BAD_ARG;
    if (h->shard) return fail(h, MASCOT_ERR_STATE, "this engine already belongs to a group");
    if (!world || rank >= world || blocks_per_gpu < 1 || blocks_per_gpu > 2) return fail(h, MASCOT_ERR_BAD_ARG, "bad rank / world / blocks_per_gpu (1 or 2)");
    if (h->kind == KIND_AFP) return fail(h, MASCOT_ERR_UNSUPPORTED, "the AFP trainer keeps per-worker state for a whole epoch and is not sharded");
    std::string why;
    const NcclApi* api = nccl_api(&why);
    if (!api) return fail(h, MASCOT_ERR_COMM, why);
    CU(h, cudaSetDevice(h->cfg.device));
    ShardCtx* S = new (std::nothrow) ShardCtx();
    if (!S) return fail(h, MASCOT_ERR_OOM, "host allocation failed");
    S->api = api; S->rank = (int)rank; S->world = (int)world; S->m = blocks_per_gpu; S->blocks = world * blocks_per_gpu;
    S->timeout_ms = timeout_ms ? timeout_ms : 60000;
    h->shard = S;
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof uid);
    const ncclResult_t r = api->CommInitRank(&S->comm, (int)world, uid, (int)rank);
    if (r != ncclSuccess) {
        const std::string msg = std::string("ncclCommInitRank failed: ") + api->GetErrorString(r);
        S->comm = nullptr; shard_destroy(h);
        return fail(h, MASCOT_ERR_COMM, msg);
    }
    cudaError_t e = cudaStreamCreateWithFlags(&S->comm_stream, cudaStreamNonBlocking);
    S->ev_trained.assign(S->blocks, nullptr); S->ev_arrived.assign(S->blocks, nullptr); S->arrival_pending.assign(S->blocks, 0);
    for (uint32_t b = 0; b < S->blocks && e == cudaSuccess; b++) {
        e = cudaEventCreateWithFlags(&S->ev_trained[b], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&S->ev_arrived[b], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaMalloc(&S->d_pair, 2 * sizeof(double));
    if (e != cudaSuccess) { shard_destroy(h); CU(h, e); }
    return MASCOT_OK;
}

int mascot_shard_set_ratings(mascot_handle* h, const mascot_rating* train, uint64_t n_train, const mascot_rating* test, uint64_t n_test,
                             uint32_t n_users, uint32_t n_items) {
    int rc = usable(h);
    if (rc != MASCOT_OK) return rc;
    ShardCtx* S = h->shard;
    S->n_global = n_train;
    SetupRequest rq;
    rq.train = train; rq.n_train = n_train; rq.test = test; rq.n_test = n_test; rq.n_users = n_users; rq.n_items = n_items;
    rq.rank = S->rank; rq.world = S->world; rq.blocks = S->blocks; rq.blocks_per_rank = S->m;
    rq.n_segments = 1;
    rc = setup_ratings(h, rq);
    std::fill(S->arrival_pending.begin(), S->arrival_pending.end(), 0);
    if (rc != MASCOT_OK || S->world == 1) return rc;
    // NCCL opens its connections at the first use of a peer: do that here (one value to the left neighbour, one
    // from the right one, as the block hand-over will; one sum over all ranks, as the check epochs and the
    // evaluation will), so that the first epoch does not pay for it (about a second on one node).
    const int to = (S->rank + S->world - 1) % S->world, from = (S->rank + 1) % S->world;
    CU(h, cudaMemsetAsync(S->d_pair, 0, 2 * sizeof(double), S->comm_stream));
    NC(h, S, S->api->GroupStart());
    NC(h, S, S->api->Send(S->d_pair, 1, ncclDouble, to, S->comm, S->comm_stream));
    NC(h, S, S->api->Recv(S->d_pair + 1, 1, ncclDouble, from, S->comm, S->comm_stream));
    NC(h, S, S->api->GroupEnd());
    if ((rc = wait_stream(h, S->comm_stream, "opening the connections to the neighbours")) != MASCOT_OK) return rc;
    NC(h, S, S->api->AllReduce(S->d_pair, S->d_pair, 2, ncclDouble, ncclSum, S->comm, h->stream));
    return wait_stream(h, h->stream, "opening the connections of the group");
}

int mascot_shard_train_epoch(mascot_handle* h, uint32_t epoch, mascot_epoch_stats* out) {
    int rc = usable(h);
    if (rc != MASCOT_OK) return rc;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before training");
    ShardCtx* S = h->shard;
    NvtxRange range("mascot_shard_train_epoch");
    CU(h, cudaSetDevice(h->cfg.device));
    const float lr = epoch < h->lr.size() ? h->lr[epoch] : lr_at(h->cfg, epoch);
    const bool check = h->grouped && is_check_epoch(h->cfg, epoch);
    const uint32_t B = S->blocks, m = S->m;
    uint32_t launches = 0, promoted_u = 0, promoted_i = 0;
    const uint64_t bytes_this_epoch = algorithmic_bytes(h);
    LaunchShape shape;
    CU(h, cudaEventRecord(h->ev[0], h->stream));
    if (check) CU(h, cudaMemsetAsync(h->d_stats, 0, sizeof(float) * h->stats_stride * h->stats_copies, h->stream));   // mf_methods.cu:178-182
    CU(h, cudaEventRecord(h->ev[1], h->stream));
    for (uint32_t t = 0; t < B; t++) {
        const uint32_t b = (m * (uint32_t)S->rank + t) % B;
        if (S->arrival_pending[b]) {               // the block must be here before its ratings are trained
            CU(h, cudaStreamWaitEvent(h->stream, S->ev_arrived[b], 0));
            S->arrival_pending[b] = 0;
        }
        if ((rc = train_range(h, lr, epoch, t, check, &shape, &launches, h->n_train)) != MASCOT_OK) return rc;
        if (S->world > 1) {
            const uint32_t incoming = (b + m) % B;
            CU(h, cudaEventRecord(S->ev_trained[t], h->stream));
            CU(h, cudaStreamWaitEvent(S->comm_stream, S->ev_trained[t], 0));
            if ((rc = queue_exchange(h, b, incoming)) != MASCOT_OK) return rc;
            CU(h, cudaEventRecord(S->ev_arrived[incoming], S->comm_stream));
            S->arrival_pending[incoming] = 1;
        }
    }
    // every block is on its way home: wait for the arrivals before anything reads or converts the item rows
    for (uint32_t b = 0; b < B; b++)
        if (S->arrival_pending[b]) { CU(h, cudaStreamWaitEvent(h->stream, S->ev_arrived[b], 0)); S->arrival_pending[b] = 0; }
    if (check) {
        if (h->stats_copies > 1) { CU(h, launch_reduce_stats(h->d_stats, h->stats_copies, h->stats_stride, stats_floats(h), h->stream)); launches++; }
        if (S->world > 1) NC(h, S, S->api->AllReduce(h->d_stats, h->d_stats, stats_floats(h), ncclFloat, ncclSum, S->comm, h->stream));
    }
    CU(h, cudaEventRecord(h->ev[2], h->stream));
    if ((rc = wait_stream(h, h->stream, "sharded epoch")) != MASCOT_OK) return rc;
    if (check) {
        const int saved = h->stats_copies;
        h->stats_copies = 1;                      // folded and summed over the ranks above
        rc = fetch_stats(h, nullptr);
        h->stats_copies = saved;
        if (rc != MASCOT_OK) return rc;
        if ((rc = apply_stats(h, epoch, &promoted_u, &promoted_i, &launches)) != MASCOT_OK) return rc;
    }
    CU(h, cudaEventRecord(h->ev[3], h->stream));
    CU(h, cudaEventSynchronize(h->ev[3]));
    if (out) {
        std::memset(out, 0, sizeof(*out));
        out->updates = h->n_train; out->lr = lr; out->error_check = check ? 1 : 0;
        out->promoted_user_groups = promoted_u; out->promoted_item_groups = promoted_i; out->kernel_launches = launches;
        out->algorithmic_bytes = bytes_this_epoch;
        out->workers = shape.workers;
        cudaEventElapsedTime(&out->kernel_ms, h->ev[1], h->ev[2]);
        cudaEventElapsedTime(&out->total_ms, h->ev[0], h->ev[3]);
    }
    { float kms = 0.f; if (cudaEventElapsedTime(&kms, h->ev[1], h->ev[2]) == cudaSuccess) h->timings.update_us += 1e3 * kms; }
    return MASCOT_OK;
}

int mascot_shard_eval_rmse(mascot_handle* h, double* rmse) {
    int rc = usable(h);
    if (rc != MASCOT_OK) return rc;
    if (!rmse) return MASCOT_ERR_BAD_ARG;
    if (!h->have_ratings || !h->have_factors) return fail(h, MASCOT_ERR_STATE, "ratings and factors must be set before evaluation");
    ShardCtx* S = h->shard;
    CU(h, cudaSetDevice(h->cfg.device));
    // after an epoch a rank holds only its home blocks fresh: make all of Q fresh everywhere
    bool f16, f32;
    live_item_arenas(h, &f16, &f32);
    if (S->world > 1 && (rc = gather_side(h, h->Q, h->ilay, S->m, f16, f32, h->stream)) != MASCOT_OK) return rc;
    double pair[2] = {0.0, (double)h->n_test};
    if (h->n_test) {
        Stream t; t.r = h->te_r; t.u = h->te_u; t.i = h->te_i; t.n = h->n_test;
        CU(h, launch_rmse(h->K, t, h->P, h->Q, h->d_block_err, h->stream));
        CU(h, cudaMemcpyAsync(h->h_block_err.data(), h->d_block_err, sizeof(float) * h->h_block_err.size(), cudaMemcpyDeviceToHost, h->stream));
        if ((rc = wait_stream(h, h->stream, "sharded evaluation")) != MASCOT_OK) return rc;
        for (float v : h->h_block_err) pair[0] += (double)v;
    }
    if (S->world > 1) {
        CU(h, cudaMemcpyAsync(S->d_pair, pair, sizeof pair, cudaMemcpyHostToDevice, h->stream));
        NC(h, S, S->api->AllReduce(S->d_pair, S->d_pair, 2, ncclDouble, ncclSum, S->comm, h->stream));
        CU(h, cudaMemcpyAsync(pair, S->d_pair, sizeof pair, cudaMemcpyDeviceToHost, h->stream));
        if ((rc = wait_stream(h, h->stream, "sharded evaluation")) != MASCOT_OK) return rc;
    }
    *rmse = pair[1] > 0 ? std::sqrt(pair[0] / pair[1]) : 0.0;
    return MASCOT_OK;
}

int mascot_shard_gather_factors(mascot_handle* h) {
    int rc = usable(h);
    if (rc != MASCOT_OK) return rc;
    if (!h->have_factors) return fail(h, MASCOT_ERR_STATE, "no factors yet");
    ShardCtx* S = h->shard;
    if (S->world == 1) return MASCOT_OK;
    CU(h, cudaSetDevice(h->cfg.device));
    bool f16, f32;
    live_item_arenas(h, &f16, &f32);
    if ((rc = gather_side(h, h->Q, h->ilay, S->m, f16, f32, h->stream)) != MASCOT_OK) return rc;
    bool uf16 = false, uf32 = false;
    for (uint8_t p : h->uprec) { if (p) uf32 = true; else uf16 = true; }
    if ((rc = gather_side(h, h->P, h->ulay, 1, uf16, uf32, h->stream)) != MASCOT_OK) return rc;
    return wait_stream(h, h->stream, "gathering the factors");
}

int mascot_shard_info(mascot_handle* h, uint32_t* rank, uint32_t* world, uint32_t* blocks, uint64_t* local_ratings,
                      uint64_t* local_test_ratings, uint64_t* bytes_sent) {
    if (!h) return MASCOT_ERR_BAD_ARG;
    if (!h->shard) return fail(h, MASCOT_ERR_STATE, "mascot_shard_init must come first");
    if (rank) *rank = (uint32_t)h->shard->rank;
    if (world) *world = (uint32_t)h->shard->world;
    if (blocks) *blocks = h->shard->blocks;
    if (local_ratings) *local_ratings = h->n_train;
    if (local_test_ratings) *local_test_ratings = h->n_test;
    if (bytes_sent) *bytes_sent = h->shard->bytes_sent;
    return MASCOT_OK;
}

}  // extern "C"
