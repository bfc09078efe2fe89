/* libmascot - C ABI of the B200-native MASCOT training engine.
 *
 * The reference (Yujaeseo/ICDM-2021_MASCOT) has no FFI: its hot path sits behind the eight
 * `void X_training_mf(Mf_info*, SGD*)` trainers (mf_methods.h:4-11), `init_model_*`
 * (model_init.h:5-10) and `gpu_test_rmse` (rmse.h:168).  This header is what a binding of that
 * path would call instead.  Conventions:
 *   - every function returns an int status (MASCOT_OK == 0, negative on failure) instead of the
 *     reference's print-and-exit `gpuErr` (common.h:3-11); nothing throws or exits;
 *   - plain pointers and sizes only; the caller owns every host buffer it passes, the library owns
 *     all device memory of a handle until mascot_destroy();
 *   - one host control thread per handle, as in the reference (one thread, synchronous epochs);
 *   - factor matrices cross this boundary as fp32, row-major, k consecutive elements per row, in the
 *     caller's id space - the internal storage precision and element order never leak out;
 *   - there is no CPU fallback: without a usable CUDA device every call fails with
 *     MASCOT_ERR_CUDA / MASCOT_ERR_NO_DEVICE.
 */
#ifndef MASCOT_H
#define MASCOT_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MASCOT_ABI_VERSION 1

#if defined(__GNUC__)
#define MASCOT_API __attribute__((visibility("default")))
#else
#define MASCOT_API
#endif

enum {
    MASCOT_OK = 0,
    MASCOT_ERR_BAD_ARG = -1,      /* null pointer, k not in {64,128}, unknown variant, id out of range ... */
    MASCOT_ERR_CUDA = -2,         /* a CUDA runtime call failed; see mascot_last_error() */
    MASCOT_ERR_OOM = -3,          /* host or device allocation failed */
    MASCOT_ERR_STATE = -4,        /* call order violated (e.g. training before ratings were set) */
    MASCOT_ERR_NO_DEVICE = -5,    /* no CUDA device / requested device absent */
    MASCOT_ERR_TIMEOUT = -6,      /* a bounded wait on another rank of a sharded group ran out */
    MASCOT_ERR_UNSUPPORTED = -7,  /* valid request the engine does not implement */
    MASCOT_ERR_COMM = -8          /* NCCL / peer communication failure */
};

/* Training variants, numbered like the reference's `-v` flag (main.cu:152-162). */
enum {
    MASCOT_V_MASCOT = 1,    /* mascot_training_mf            mf_methods.cu:36-434   */
    MASCOT_V_AFP = 2,       /* adaptive_fixed_point_training mf_methods.cu:436-527  */
    MASCOT_V_MUPPET = 3,    /* muppet_training_mf            mf_methods.cu:529-711  */
    MASCOT_V_MPT = 4,       /* mixed_precision_training_mf   mf_methods.cu:713-818  */
    MASCOT_V_SGD = 5,       /* training_single_mf            mf_methods.cu:820-924  */
    MASCOT_V_NAIVE = 6,     /* mascot_training_mf_naive      mf_methods.cu:926-1301: the same arithmetic as
                               variant 1 with a slower group lookup in the reference; runs as variant 1 here */
    MASCOT_V_MEMQUANT = 7,  /* training_mem_quant_mf         mf_methods.cu:1303-1394 */
    MASCOT_V_SWITCH_ONLY = 8 /* training_switching_only      mf_methods.cu:1396-1562: the whole model in
                               binary16 until one sampled error test switches all of it to fp32 */
};

/* One rating; same 12-byte record as the reference's `Node` (common_struct.h:8-12). */
typedef struct mascot_rating {
    float r;
    uint32_t u;
    uint32_t i;
} mascot_rating;

/* Mirrors `Parameter` (common_struct.h:19-35) plus `Mf_info::version` / `is_yahoo`
 * (common_struct.h:85-86); the trailing fields are additive extensions. */
typedef struct mascot_config {
    float lambda;                /* -b   regularisation            default 0.015 (main.cu:19)  */
    float learning_rate;         /* -a                             default 0.01                */
    float decay;                 /* -d                             default 0.1                 */
    float sample_ratio;          /* -s / -r  sampled tail          default 0.01                */
    float error_threshold;       /* -e   promote when error > e    default 0.001               */
    uint32_t interval;           /* -it  epochs between checks     default 1                   */
    uint32_t user_group_num;     /* -ug  requested user groups     default 10                  */
    uint32_t item_group_num;     /* -ig  requested item groups     default 10                  */
    uint32_t k;                  /* -k   64 or 128                 default 128                 */
    uint32_t num_workers;        /* -wg  number of concurrent sequential workers (the reference's warps):
                                       fewer workers lose fewer updates of popular rows to races and
                                       converge faster per epoch, more workers run faster; rounded up
                                       to fill every SM evenly; 0 = automatic (one per 8192 training
                                       ratings, at least 512, at most what the GPU keeps resident - or 16 warps
                                       per SM when the binary16 factors exceed the GPU's L2, where more workers
                                       run slower; sets under 1.5M ratings: one per 512 ratings, at most 1536)
                                                                                   default 2048        */
    uint32_t epoch;              /* -l   number of epochs          default 50                  */
    uint32_t thread_block_size;  /* -bl  accepted for CLI parity, not used (blocks are sized per SM) */
    uint32_t version;            /* -v   one of MASCOT_V_*         default 7 in the reference  */
    uint32_t is_yahoo;           /* MuPPET starts at 12 bits when set (mf_methods.cu:600-601)  */
    /* ---- extensions ---- */
    uint32_t deterministic;      /* 1: a single worker walks the stream in order; bit-exact against
                                       a sequential host replay of the same rule                  */
    uint32_t shuffle;            /* 1: seeded permutation of the training stream (the reference shuffles with
                                       srand(time(0)), mf_methods.cu:38-39), then item-sorted windows of
                                       4096 ratings; 0: the caller's order, untouched                  */
    uint64_t seed;               /* seeds the stream permutation and mascot_init_factors()      */
    int32_t device;              /* CUDA device ordinal                                         */
    uint32_t muppet_width;       /* extension: first pass width of MuPPET, 8/12/14/16/32; 0 = the reference's start
                                    (8, or 12 for Yahoo input; mf_methods.cu:597-601) */
    uint32_t plain_user_stores;  /* extension: 0 (default) = with more than one worker, user rows are written back as
                                    reductions of their change, so racing updates of one user are not lost.  A user
                                    with so many ratings that more than about 32 workers would hold its row at the
                                    same time has only every 2^s-th of its updates written back (the others are
                                    dropped, as a plain store drops all but one of the concurrent ones), with s chosen
                                    so that about 32 concurrent updates of the most popular user remain;
                                    1 = plain stores like the reference (racing updates overwrite each other) */
    uint32_t l2_item_window;     /* extension: 1 = ask the GPU to keep the item factors in L2 (a persisting access-policy
                                    window of the engine's stream over the item arena, sized to what the device allows;
                                    everything else the stream touches is then treated as streaming).  Off by default:
                                    measured on one B200 on the 252M-rating set it makes an epoch SLOWER (35.8 ms against
                                    21.5 ms) - the item rows are read once per run of equal items anyway, and the user
                                    rows lose their place in L2.  Sets this process's persisting-L2 limit on the device
                                    for the life of the engine; mascot_destroy puts the old limit back. */
    uint32_t no_class_partition; /* extension: 0 (default) = after a promotion the stream is re-ordered by precision class and
                                    every class runs the kernel instantiation made for it (see mascot_train_epoch);
                                    1 = never re-order: every launch reads each id's precision bit */
    uint32_t run_window_log2;    /* extension: the resident training stream is sorted by item inside windows of 2^run_window_log2
                                    positions (after the seeded permutation), so that a worker meets an item's ratings in
                                    one run and reads and writes the item's row once per run.  0 (default) = 20; 1..12 =
                                    only the 4096-position windows of the encoding step; up to 32.  The engine shortens
                                    the windows to what all workers of a launch hold at one time and, when statistics
                                    are sampled, to a quarter of the sampled tail of a segment.  Ignored with
                                    shuffle = 0 and in deterministic mode (the caller's order is kept) */
    uint32_t reserved[2];
} mascot_config;

typedef struct mascot_epoch_stats {
    uint64_t updates;            /* ratings processed by this epoch's update kernel             */
    float lr;                    /* learning rate used (schedule mf_methods.cu:94-97)           */
    float kernel_ms;             /* update kernel, CUDA-event time on the engine's stream       */
    float total_ms;              /* update + statistics + promotion, CUDA-event time            */
    uint32_t error_check;        /* 1 when group errors were computed this epoch                */
    uint32_t promoted_user_groups;
    uint32_t promoted_item_groups;
    uint32_t kernel_launches;    /* kernels launched by this call                               */
    uint32_t workers;            /* concurrent sequential workers the update kernel ran with    */
    uint32_t pass_bits;          /* MuPPET: width of this epoch's forward/backward pass (8, 12, 14, 16, 32); else 0 */
    uint64_t algorithmic_bytes;  /* factor bytes the update rule reads + writes this epoch:
                                    sum over ratings of 2*k*(bytes per user element + bytes per
                                    item element), 2 for fp16 storage and 4 for fp32            */
} mascot_epoch_stats;

/* The phases of the reference's timing report (mf_methods.cu:401-418), in microseconds: host clock
 * around phases that end with a synchronisation, CUDA events for the update kernels. */
typedef struct mascot_timings {
    double rating_histogram_us;    /* upload, id check, degree histogram and degree sort (user_item_rating_histogram) */
    double grouping_us;            /* grouping walk, group / map / flag tables (split_group_based_equal_size_...) */
    double reconstruction_us;      /* id remap, shuffle, coding of the stream and the test set (matrix_reconstruction) */
    double copy_to_grouped_us;     /* factors scattered into the arenas (cpy2grouped_parameters_gpu_...) */
    double additional_init_us;     /* arenas, statistics buffers (mf_methods.cu:93-166) */
    double precision_switching_us; /* total: widening of promoted groups, re-tagging and re-partition of the stream */
    double error_computation_us;   /* total: folding and read-back of the statistics, group errors */
    double update_us;              /* total time of the update kernels */
} mascot_timings;

typedef struct mascot_handle mascot_handle;

/* ABI self-description for bindings: version and the byte sizes of the two public structs. */
MASCOT_API int mascot_abi_info(uint32_t* abi_version, uint32_t* config_bytes, uint32_t* epoch_stats_bytes);

/* Fill `cfg` with the reference CLI defaults (main.cu:19-32); extensions: shuffle=1, seed=1. */
MASCOT_API int mascot_config_default(mascot_config* cfg);

/* Create an engine on cfg->device.  Replaces the argument plumbing of main.cu:134-148. */
MASCOT_API int mascot_create(const mascot_config* cfg, mascot_handle** out);
MASCOT_API int mascot_destroy(mascot_handle* h);

/* Message of the last failure on this handle (or of the last failed mascot_create when h is NULL). */
MASCOT_API const char* mascot_last_error(const mascot_handle* h);
MASCOT_API const char* mascot_status_string(int status);

/* Hand over the training and test ratings (host memory, ids already compact in [0,n_users) x
 * [0,n_items), the id space produced by read_training_dataset, io_utils.h:93-106).  Uploads them,
 * and for MASCOT_V_MASCOT runs the m-quantization set-up: degree histogram, ascending sort,
 * grouping, id -> sorted-index remap (user_item_rating_histogram / split_group_... /
 * matrix_reconstruction, preprocess_utils.h:54-255; host shuffle mf_methods.cu:38-42).  The whole
 * set-up runs on the device after one host->device copy of each array; the host only walks per-entity
 * tables.  At most 2^32 - 1 ratings per engine. */
MASCOT_API int mascot_set_ratings(mascot_handle* h, const mascot_rating* train, uint64_t n_train,
                       const mascot_rating* test, uint64_t n_test, uint32_t n_users, uint32_t n_items);

/* Extension: replace the training stream by `train` (host memory, same id space and same
 * n_users / n_items as the last mascot_set_ratings) without redoing the set-up: one host->device
 * copy plus the encode kernel.  This is the per-step input path of an out-of-core / end-to-end
 * epoch.  Ids are checked on the device while the stream is coded: an id out of range is never used as
 * an index and makes the call return MASCOT_ERR_BAD_ARG (the stream then holds zero ratings of row 0 in
 * its place and should be reloaded).  If groups have been promoted the new stream is partitioned by
 * precision class like the one it replaces. */
MASCOT_API int mascot_reload_train(mascot_handle* h, const mascot_rating* train, uint64_t n_train);

/* N(0, 0.01^2) factors from a counter-based generator seeded with cfg.seed (init_model_single /
 * init_model_half, model_init.cu:114-173; the reference seeds cuRAND with clock()). */
MASCOT_API int mascot_init_factors(mascot_handle* h);
/* Caller-provided factors, fp32 [n_users][k] and [n_items][k] in compact-id order.  For fp16-stored
 * variants they are converted with round-to-nearest-even (model_init.cu:51-54). */
MASCOT_API int mascot_set_factors(mascot_handle* h, const float* P, const float* Q);

/* One epoch = one pass of the update kernel over the training stream with lr_schedule[epoch]; for
 * MASCOT_V_MASCOT also the sampled group-error statistics on check epochs and the precision
 * switching that follows (epoch body of mf_methods.cu:168-397; precision_switching.h:8-51).
 * `stats` may be NULL.
 * Sampling rule: on a check epoch every launched range of the stream - a segment, or, once groups have
 * been promoted and several workers run, each precision class inside a segment - passes its last
 * sample_ratio through the statistics kernel.  With one segment and no promoted group this is the
 * reference's "last sample_ratio of the stream" (mf_methods.cu:102-103).  Segments are what the last
 * mascot_set_ratings_sharded / mascot_train_epoch_streamed left (one segment after mascot_set_ratings).
 * Per-worker state of the AFP trainer starts afresh with every launched range.
 * After a promotion, and with more than one worker, the stream is stably re-ordered inside each segment
 * by (user precision, item precision), so that every class runs a kernel instantiation without
 * per-rating precision tests (one launch per class, one after the other; models larger than the GPU's L2 keep
 * their order, see mascot_config.no_class_partition); mascot_stream_source_index / mascot_get_stream_order follow the new order.
 * The deterministic mode never re-orders. */
MASCOT_API int mascot_train_epoch(mascot_handle* h, uint32_t epoch, mascot_epoch_stats* stats);

/* Test RMSE of the current factors, reduced exactly like gpu_test_rmse (rmse.h:168-189): fp32 dot
 * products, 512-rating block trees, float sum of the block partials, sqrt(sum / n). */
MASCOT_API int mascot_eval_rmse(mascot_handle* h, double* rmse);

/* Copy the factors out as fp32.  order 0: compact-id rows (what save_trained_model writes,
 * io_utils.h:242-303); order 1: sorted-index rows (save_trained_model_reconst, io_utils.h:305-332;
 * identical to order 0 for variants without m-quantization). */
MASCOT_API int mascot_get_factors(mascot_handle* h, float* P, float* Q, int order);

/* Group tables of one side (0 users, 1 items): number of groups, inclusive end index of each group
 * in sorted-index space, storage precision (0 fp16, 1 fp32) and the last normalised group error
 * (-1 for groups already in fp32).  Any output pointer may be NULL.  Arrays need room for the
 * requested group count of the config. */
MASCOT_API int mascot_get_group_info(mascot_handle* h, int side, uint32_t* n_groups, uint32_t* end_idx,
                          uint8_t* precision, float* error);

/* Extension: switch one fp16 group of the MASCOT variant to fp32 storage now - the action
 * precision_switching_by_groups_grad_diversity (precision_switching.h:8-51) takes for a group whose
 * error exceeds the threshold.  One way; a no-op for a group that is already fp32. */
MASCOT_API int mascot_promote_group(mascot_handle* h, int side, uint32_t group);

/* id -> sorted-index maps built by the m-quantization set-up (matrix_reconstruction,
 * preprocess_utils.h:215-240); identity for other variants.  Either pointer may be NULL. */
MASCOT_API int mascot_get_index_maps(mascot_handle* h, uint32_t* user2sorted, uint32_t* item2sorted);

/* Sampled statistics of the last check epoch (grad_sum_norm_{p,q} [groups*k] and per-group sum of
 * squared gradient norms; mascot_sgd_kernel.h:240-277, 448-456).  Pointers may be NULL. */
MASCOT_API int mascot_get_sample_stats(mascot_handle* h, float* grad_sum_p, float* grad_sum_q,
                            float* norm_sum_p, float* norm_sum_q);

/* The test set in the id space of `order` (1: sorted-index, what save_reconst_testset writes,
 * io_utils.h:374-405), sorted like test_set_preprocess (preprocess_utils.h:38-52) leaves it. */
MASCOT_API int mascot_get_test_ratings(mascot_handle* h, mascot_rating* out, int order);

/* Position in the caller's training array of the rating that the engine processes at stream
 * position `pos` (identity when shuffle == 0).  With shuffle == 1 the stream is the seeded
 * permutation of the caller's array, cut into windows of 4096 positions that are each sorted by
 * item so that equal items are neighbours; the resident stream of a multi-worker engine is then sorted by item
 * inside larger windows (mascot_config.run_window_log2) and, after a promotion, re-ordered by precision class
 * (mascot_train_epoch).  Lets a host replay follow exactly the same order. */
MASCOT_API int mascot_stream_source_index(const mascot_handle* h, uint64_t pos, uint64_t* src);
/* The whole order at once: src_out[pos] for pos in [0, n_train). */
MASCOT_API int mascot_get_stream_order(mascot_handle* h, uint32_t* src_out);

/* ---- building blocks for sharded (multi-GPU) training; no counterpart in the reference, which is
 * single-GPU.  One engine per GPU holds the ratings of its own users, cut into segments by item
 * block; the host (one process per GPU) trains a segment, passes that item block on to the next
 * GPU and receives the following one, so that no two GPUs ever update the same row at once.  Every
 * engine keeps full-size arenas in the same global index space, so a block is the same row range
 * on every GPU and "passing it on" is a plain copy of that range. ---- */

/* Like mascot_set_ratings, with the training ratings already ordered into `n_segments` consecutive
 * segments (segment_offsets has n_segments + 1 entries, from 0 to n_train; NULL with n_segments == 1)
 * and, optionally, the degrees of every user and item in the WHOLE data set, so that all shards
 * build identical sorted-index spaces and groups.  The seeded permutation and the item-sorted
 * windows stay inside a segment. */
MASCOT_API int mascot_set_ratings_sharded(mascot_handle* h, const mascot_rating* train, uint64_t n_train,
                               const uint64_t* segment_offsets, uint32_t n_segments,
                               const mascot_rating* test, uint64_t n_test, uint32_t n_users, uint32_t n_items,
                               const uint32_t* user_degree, const uint32_t* item_degree);
/* One epoch over a rating array that is still in HOST memory (pinned memory for a real overlap):
 * the array is uploaded in pieces of 8Mi ratings on a copy stream while the piece before it is
 * encoded and trained, so the epoch costs max(upload, updates) instead of their sum.  The seeded
 * permutation and the item-sorted windows stay inside a piece; afterwards the pieces are the
 * segments of the resident stream, as after mascot_reload_train.  Ids must be those given to
 * mascot_set_ratings (same users/items; checked on the device, MASCOT_ERR_BAD_ARG as for
 * mascot_reload_train); on a check epoch every piece contributes its own sampled tail (see
 * mascot_train_epoch).  The pieces are never re-ordered by precision class (that would need a host wait
 * per piece); once groups have been promoted each piece runs the kernel that reads every id's precision bit.  No reference counterpart (the reference uploads once,
 * mf_methods.cu:41-42).  AFP is not supported here (its per-worker state spans a whole epoch). */
MASCOT_API int mascot_train_epoch_streamed(mascot_handle* h, uint32_t epoch, const mascot_rating* train, uint64_t n_train,
                                mascot_epoch_stats* stats);
/* 1 when `epoch` computes group errors (mf_methods.cu:168-175), else 0. */
MASCOT_API int mascot_is_check_epoch(const mascot_handle* h, uint32_t epoch);
/* Zero the statistic accumulators (start of a check epoch). */
MASCOT_API int mascot_stats_begin(mascot_handle* h);
/* Train one segment with lr_schedule[epoch]; with collect_stats != 0 the last sample_ratio of the
 * segment adds to the statistic accumulators.  With stats == NULL the call does not wait for the
 * kernel (use mascot_sync), so copies on other streams can overlap it. */
MASCOT_API int mascot_train_segment(mascot_handle* h, uint32_t epoch, uint32_t segment, uint32_t collect_stats,
                                    mascot_epoch_stats* stats);
/* The accumulated sums of this engine, layout as in mascot_get_sample_stats. */
MASCOT_API int mascot_stats_fetch(mascot_handle* h, float* grad_sum_p, float* grad_sum_q, float* norm_sum_p, float* norm_sum_q);
/* Group errors and precision switching from sums the caller provides (e.g. summed over all shards). */
MASCOT_API int mascot_stats_apply(mascot_handle* h, uint32_t epoch, const float* grad_sum_p, const float* grad_sum_q,
                       const float* norm_sum_p, const float* norm_sum_q,
                       uint32_t* promoted_user_groups, uint32_t* promoted_item_groups);
/* Device addresses and byte sizes of the item rows [row_begin, row_end) (sorted-index space) in the
 * binary16 and the fp32 arena (NULL / 0 for an arena the variant does not keep). */
MASCOT_API int mascot_item_rows(mascot_handle* h, uint32_t row_begin, uint32_t row_end, void** f16_ptr, uint64_t* f16_bytes,
                     void** f32_ptr, uint64_t* f32_bytes);
/* Wait for everything queued on the engine's stream. */
MASCOT_API int mascot_sync(mascot_handle* h);
/* The CUDA stream (a cudaStream_t) every kernel and copy of this engine is queued on, so that a
 * host program can order its own transfers and events against the engine's work on the device,
 * without host-side waits.  No reference counterpart (the reference uses the default stream). */
MASCOT_API int mascot_get_stream(mascot_handle* h, void** stream);
/* Sum of squared test errors and number of test ratings of this engine (for an RMSE over shards). */
MASCOT_API int mascot_eval_sq_error(mascot_handle* h, double* sum_sq, uint64_t* count);

/* Accumulated phase times of this engine since mascot_create. */
MASCOT_API int mascot_get_timings(mascot_handle* h, mascot_timings* out);
/* Number of concurrent sequential workers the update launches of this engine ask for (the value of -wg, or
 * the automatic choice for the current stream when cfg.num_workers == 0). */
MASCOT_API int mascot_get_worker_count(mascot_handle* h, uint32_t* workers);

/* Release the engine's grow-only device scratch (staging buffer of mascot_reload_train, sort buffers of
 * the set-up and of the stream partition).  It is allocated again when next needed. */
MASCOT_API int mascot_release_scratch(mascot_handle* h);

/* ---- sharded training inside the library: one engine per GPU, one host thread or process per engine,
 * NCCL between them.  No counterpart in the reference (single-GPU).  Users are pinned to a GPU with their
 * ratings and their rows of P; the item factors are cut into world x blocks_per_gpu blocks that travel
 * from GPU to GPU during an epoch, so that no two GPUs ever update the same row at once.  Every call of
 * this section is collective: all engines of the group make it, in the same order.  Waits on other
 * ranks are bounded by the group's timeout: MASCOT_ERR_TIMEOUT / MASCOT_ERR_COMM dissolve the group
 * (the engine can still be read out and destroyed).  AFP is not sharded. ---- */

#define MASCOT_COMM_ID_BYTES 128
/* 128 opaque bytes that identify a group (an NCCL unique id).  One rank makes them; the caller carries
 * them to the other ranks by any means it has (shared memory between threads, a file, a socket, MPI). */
MASCOT_API int mascot_comm_unique_id(void* id_out);
/* Join the engine (on its cfg.device) to the group `id` as rank `rank` of `world`.  blocks_per_gpu: 1 =
 * a block is passed on when its training ends and the receiver waits for it; 2 = a block travels while
 * its receiver trains another one (transfers hidden under the update kernels; the workers of a GPU then
 * share half as many item rows at a time, which costs some convergence per epoch).  timeout_ms bounds
 * every wait on another rank (0 = 60 s). */
MASCOT_API int mascot_shard_init(mascot_handle* h, const void* id, uint32_t rank, uint32_t world, uint32_t blocks_per_gpu,
                                 uint32_t timeout_ms);
/* Like mascot_set_ratings, called by every rank with the WHOLE data set (same arrays on all ranks): the
 * engine builds the common index space from the global degrees, keeps the ratings of the users dealt to
 * its rank and orders them by the step of the block schedule at which their item block is on this GPU. */
MASCOT_API int mascot_shard_set_ratings(mascot_handle* h, const mascot_rating* train, uint64_t n_train,
                                        const mascot_rating* test, uint64_t n_test, uint32_t n_users, uint32_t n_items);
/* One epoch over this rank's ratings: world x blocks_per_gpu update launches with the block hand-overs
 * between them (ncclSend / ncclRecv on a transfer stream), on check epochs the all-reduce of the sampled
 * statistics and the same precision switching on every rank.  `stats` reports this rank's share. */
MASCOT_API int mascot_shard_train_epoch(mascot_handle* h, uint32_t epoch, mascot_epoch_stats* stats);
/* Test RMSE over all ranks (double accumulation of the ranks' block sums): all-gathers the item blocks,
 * evaluates this rank's test ratings, all-reduces (sum of squared errors, count). */
MASCOT_API int mascot_shard_eval_rmse(mascot_handle* h, double* rmse);
/* All-gather both factor matrices, after which mascot_get_factors on any rank returns the whole model. */
MASCOT_API int mascot_shard_gather_factors(mascot_handle* h);
/* Rank, world size, number of item blocks, this rank's training and test ratings, item-block bytes sent
 * so far.  Any pointer may be NULL. */
MASCOT_API int mascot_shard_info(mascot_handle* h, uint32_t* rank, uint32_t* world, uint32_t* blocks,
                                 uint64_t* local_ratings, uint64_t* local_test_ratings, uint64_t* bytes_sent);
/* The block schedule as a pure function (no device needed): in step `step` (0 <= step < world x
 * blocks_per_gpu) rank `rank` trains block *train_block, then sends it to *send_to while *recv_block -
 * trained by *recv_from in the same step - arrives; the arriving block is trained blocks_per_gpu steps
 * later.  Any output pointer may be NULL. */
MASCOT_API int mascot_shard_schedule(uint32_t world, uint32_t blocks_per_gpu, uint32_t rank, uint32_t step,
                                     uint32_t* train_block, uint32_t* send_to, uint32_t* recv_block, uint32_t* recv_from);

/* Measurement utility (no counterpart in the reference): GB/s at which all SMs of `device` read a buffer
 * of `bytes` with 128-bit L2-only loads, `passes` times after a warm-up pass.  A buffer that fits in L2
 * gives the L2 -> SM bandwidth the update kernel is judged against while the factors are L2-resident,
 * one far larger than L2 the HBM read bandwidth.  Allocates and frees the buffer. */
MASCOT_API int mascot_probe_read_bandwidth(int device, uint64_t bytes, uint32_t passes, double* gb_per_s);

/* ---- handle-free evaluation: the `gpu_test_rmse` used by test_mf (test_mf/test.cu:56-72) ---- */

/* Host buffers in, RMSE out: fp32 P [n_users][k], Q [n_items][k], test ratings with plain row
 * indices.  Copies to the device, evaluates, frees. */
MASCOT_API int mascot_rmse_host(const float* P, uint32_t n_users, const float* Q, uint32_t n_items, uint32_t k,
                     const mascot_rating* test, uint64_t n_test, int device, double* rmse);
/* Same evaluation on buffers already on the current device (fp32 rows in the reference's element
 * order).  Allocates its block-partial scratch with cudaMalloc and frees it before returning. */
MASCOT_API int mascot_rmse_device(const float* d_P, const float* d_Q, uint32_t k, const mascot_rating* d_test,
                       uint64_t n_test, double* rmse);

/* No counterpart in the reference.  The same evaluation as mascot_rmse_device for callers that
 * must not allocate device memory when they call: it performs no cudaMalloc / cudaFree and calls no
 * allocating library routine; the block partials go to a fixed 256 KiB array in device memory that
 * every GPU loading libmascot holds until the process exits.
 *   - limit: at most 33,554,432 test ratings per call (65,536 blocks of 512); larger sets are
 *     rejected with MASCOT_ERR_BAD_ARG and a message naming the limit;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call before any stream capture begins.  "No allocation"
 *     holds from the second call on a device: the first one also makes the CUDA runtime load this
 *     kernel's module onto the device, which allocates driver-side memory once;
 *   - all calls share the one array (and one host staging buffer) and it keeps the previous call's
 *     contents; each call overwrites every entry it reads, so nothing needs clearing, but two calls
 *     that overlap in time - from different threads or on different streams of one GPU - race;
 *   - inputs and output exactly as mascot_rmse_device: device pointers on the current device, fp32
 *     rows in the reference element order, RMSE written to host memory. */
MASCOT_API int mascot_rmse_device_noalloc(const float* d_P, const float* d_Q, uint32_t k, const mascot_rating* d_test,
                                          uint64_t n_test, double* rmse);

#ifdef __cplusplus
}
#endif
#endif /* MASCOT_H */
