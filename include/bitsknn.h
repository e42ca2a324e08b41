/* bitsknn.h -- C ABI of the B200 (sm_100a) k-NN hot path.
 *
 * Drop-in boundary for the device work behind the reference's algorithm objects
 * (jiriklepl/bits-knn-jpdc2024).  Every entry point
 *   - takes plain pointers and sizes (DEVICE pointers unless the name says `host`),
 *   - is stream-ordered and does not synchronise unless documented,
 *   - never allocates result memory: outputs and workspaces are the caller's,
 *   - returns an int status (BITSKNN_OK == 0) and never throws; the text of the last
 *     failure on the calling thread is available from bitsknn_last_error_string().
 *
 * Result convention (the reference's `distance_pair` order, include/bits/knn.hpp:13-17):
 * per query the k smallest (distance, index) pairs in ascending distance, ties broken by
 * the lowest index, as two row-major arrays float32[q][k] and int32[q][k].
 */
#ifndef BITSKNN_H_
#define BITSKNN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A `cudaStream_t` passed through the C ABI (NULL = the legacy default stream, which is
 * what the reference uses everywhere: include/bits/cuda_stream.hpp:198). */
typedef void* bitsknn_stream_t;

enum bitsknn_status
{
    BITSKNN_OK = 0,
    BITSKNN_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, misaligned pointer */
    BITSKNN_ERR_UNSUPPORTED_K = 2,    /* the reference's "Unsupported k value" (bits_knn.cu:52-62) */
    BITSKNN_ERR_UNSUPPORTED_DIM = 3,
    BITSKNN_ERR_WORKSPACE = 4,        /* caller-provided workspace too small */
    BITSKNN_ERR_CUDA = 5,             /* a CUDA runtime call failed (the reference's "CUDA error.") */
    BITSKNN_ERR_DEVICE_TIMEOUT = 6,   /* a bounded device-side wait expired */
    BITSKNN_ERR_UNSUPPORTED_MODE = 7,
    BITSKNN_ERR_COMM = 8              /* NCCL is missing or one of its calls failed */
};

/* Largest k of the selection / merge kernels (the reference's limit,
 * src/topk/singlepass/detail/definitions_common.hpp:4). */
#define BITSKNN_MAX_K 2048
/* Largest k of the fused kernel (src/topk/singlepass/detail/definitions_common.hpp:6). */
#define BITSKNN_FUSED_MAX_K 256

/* Library version (major * 10000 + minor * 100 + patch). */
int bitsknn_version(void);

/* Text of the last error reported on the calling thread ("" if none). */
const char* bitsknn_last_error_string(void);

/* Reads (and clears) the device-side status word that kernels set when one of their bounded
 * waits gives up.  Synchronises `stream`.  Returns BITSKNN_OK or BITSKNN_ERR_DEVICE_TIMEOUT. */
int bitsknn_device_status(bitsknn_stream_t stream);

/* Diagnostic: launches a one-warp kernel that waits on a barrier nothing ever completes, with a
 * poll limit of about a thousand tries (well under a millisecond), and reports the expiry the way
 * the production kernels do.  After it, bitsknn_device_status() returns
 * BITSKNN_ERR_DEVICE_TIMEOUT once and the context stays usable.  The reference has no device-side
 * waits and no such check (its only failure path is the CUCH macro, include/bits/cuch.hpp:9-19). */
int bitsknn_selftest_bounded_wait(bitsknn_stream_t stream);

/* Tuning knobs (launch shapes).  Unknown keys return BITSKNN_ERR_INVALID_ARGUMENT.  With a knob at
 * its default the library takes the shape from its tuning table (csrc/tuning_table.inc, keyed by
 * k, the number of row slices and, for the fused kernels, the dimension; regenerated on a GPU by
 * bits-knn-jpdc2024_b200/tune.py), the role of the reference's scripts/optima.csv and its lookup
 * config_algorithm (scripts/config.sh:98-214).
 *   "select.stage_bytes"  bytes per shared-memory stage of the row stream (multiple of 4096;
 *                         0 = automatic, the default); stages x stage_bytes beyond the 227 KiB a
 *                         block may use makes the next selection return INVALID_ARGUMENT
 *   "select.stages"       stages in the ring (2..8; 0 = automatic, the default)
 *   "select.merge_at"     merge the candidate buffer when it holds at least this percentage
 *                         of the list length (1..100; 100 = like the reference; lists of 1024
 *                         pairs and more, which are folded by selection over a buffer of twice
 *                         the list length, take up to 187; 0 = automatic, the default: 50 for
 *                         lists of up to 256 pairs, 75 for longer ones, 140 from 1024 pairs)
 *   "select.unroll"       128-bit vectors per thread examined under one warp vote (0 = automatic,
 *                         2 or 4; other values are rejected)
 *   "select.threads" / "select.ipt"  block size (256, 512, 1024) and list pairs per thread (1, 2, 4)
 *                         of the selection kernel; both non-zero and threads x ipt >= k to apply
 *   "fused.variant"       FP32 fused kernel: 0 = 8 queries per block, 1 = tiled (needs the
 *                         workspace), 2 = automatic (default)
 *   "fused.parts"         blocks per query tile of the tiled fused kernels, i.e. ranges the database
 *                         is cut into (0 = automatic, the default)
 *   "fused.tc_cap"        candidate slots per query and consumer group of the fused TF32/BF16 kernels:
 *                         0 = automatic (32, or 16 when the operand ring needs the shared memory), 16, 32
 *   "fused.tc_fold_above" fold a candidate buffer of those kernels above this many candidates
 *                         (1 .. slots - 1; 0 = automatic)
 *   "fused.tc_tf32_plain" image of the fused TF32 kernel: 0 = automatic (plainly rounded from 32
 *                         dimensions on, hi/lo split below), 1 = always plain, 2 = always split
 *   "profile.kernel_events"  1 = record CUDA events around the main kernels (bitsknn_kernel_ms)
 *   "fused.tc_mma_n"      points per tensor-core MMA of the fused TF32/BF16 kernels: 0 = automatic
 *                         (256 for image rows of two or more 128-byte K blocks when the operand
 *                         ring fits shared memory, else 128), 128 = always 128, 256 = 256 whenever
 *                         the ring fits
 * The reference's `--block-size` / `--items-per-thread` flags tune the same things for its
 * kernels (src/topk/singlepass/bits_knn.cu:98-114); here they are hints. */
int bitsknn_set_tuning(const char* key, int value);
int bitsknn_get_tuning(const char* key, int* value);
/* The index-th registered tuning key (0, 1, ...), NULL past the last one. */
const char* bitsknn_tuning_key(int index);

/* Device time of the last launch of one of the library's main kernels, in milliseconds, taken
 * with CUDA events on the launching stream while the knob "profile.kernel_events" is 1 (the
 * role of the reference's cuda_event pairs, include/bits/cuda_event.hpp:63-68, moved from the
 * transfers to the kernels).  Names: "select_kernel", "merge_kernel", "rerank_kernel",
 * "l2_fp32_kernel", "l2_tc_kernel", "fused_kernel", "fused_tiled_kernel", "fused_tc_kernel".
 * Synchronises on that launch's end.  INVALID_ARGUMENT if no timed launch of that name exists. */
int bitsknn_kernel_ms(const char* kernel, float* ms);

/* ---------------------------------------------------------------------------------------
 * `bits` top-k selection over a precomputed distance matrix.
 * Replaces run_bits_kernel<...>() (include/bits/topk/singlepass/bits_kernel.hpp:22-27) and
 * its dispatcher bits::run (src/topk/singlepass/bits_knn.cu:29-65).
 *
 *   d_dist           float32[q][ld], row-major, ld >= n; 4-byte aligned (rows whose start
 *                    is 16-byte aligned stream entirely through bulk copies)
 *   d_labels         optional int32[q][ld_labels]: explicit label of every matrix element
 *                    (NULL = the column index), the reference's `in_label`
 *   d_label_offsets  optional int32[q]: added to the implicit column index of row i, the
 *                    reference's `label_offsets` (bits_kernel.cuh:235-243)
 *   k                1 <= k <= BITSKNN_MAX_K (any value, not only powers of two)
 *   d_out_dist/idx   float32[q][k], int32[q][k]
 * Rows with n < k are padded with (+inf, position) like the reference's first block load.
 * --------------------------------------------------------------------------------------- */
int bitsknn_select(const float* d_dist, int64_t ld, const int32_t* d_labels, int64_t ld_labels,
                   const int32_t* d_label_offsets, int64_t q, int64_t n, int k, float* d_out_dist,
                   int32_t* d_out_idx, bitsknn_stream_t stream);

/* Ablation variants of the selection, same arguments and result as bitsknn_select with implicit
 * labels.  Replace the reference's registry entries `partial-bitonic-regs`
 * (src/topk/singlepass/partial_bitonic.cu:217-294: no buffer, every value sorted and merged) and
 * `partial-bitonic-buffered-static` (src/topk/singlepass/partial_bitonic_buffered.cu:216-337:
 * filtered buffer, but the sorted list and every network step in shared memory), which it keeps to
 * show what the register-resident list and the buffer buy (scripts/run-bitonic-sort.sh:33-54,
 * scripts/run-buffer.sh:65-75). */
enum bitsknn_ablation
{
    BITSKNN_ABLATION_NO_BUFFER = 0,
    BITSKNN_ABLATION_SHARED_LIST = 1
};
int bitsknn_select_ablation(const float* d_dist, int64_t ld, int64_t q, int64_t n, int k, int variant,
                            float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream);

/* Split-row selection: every row is cut into `splits` slices scanned by separate thread
 * blocks, whose candidates (q * splits * k pairs in the caller's workspace) are merged by a
 * second kernel.  Replaces single_query_bits (src/topk/singlepass/bits_knn.cu:116-186, the
 * `bits-sq --deg` algorithm).  splits == 0 lets the library choose from q and the SM count.
 * Workspace size: bitsknn_select_split_workspace_bytes(q, k, splits). */
/* The number of slices per row the library would choose (what `splits == 0` resolves to on the
 * current device; 1 = whole rows are best).  The reference leaves this choice to its `--deg`
 * flag and tuning tables (scripts/run-bits-sq.sh:25-29). */
int bitsknn_select_auto_splits(int64_t q, int64_t n, int k);
size_t bitsknn_select_split_workspace_bytes(int64_t q, int k, int splits);
int bitsknn_select_split(const float* d_dist, int64_t ld, const int32_t* d_label_offsets, int64_t q,
                         int64_t n, int k, int splits, void* d_workspace, size_t workspace_bytes,
                         float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream);

/* Split-row selection that allocates nothing (no counterpart in the reference).
 * For callers that cannot obtain device memory when they need a search -- a plug-in inside an
 * engine that owns the whole device pool, code on a path where an allocation would stall the
 * device, a process with a memory budget fixed at start-up.  Same result as
 * bitsknn_select_split, but the q * splits * k candidate pairs are kept in a fixed array that
 * is part of the library's device image: BITSKNN_STATIC_SCRATCH_BYTES on every GPU that
 * loads the library, for the life of the process.  Limits and rules:
 *   - q * splits * k * 8 bytes must fit (BITSKNN_ERR_WORKSPACE otherwise); splits >= 1;
 *   - the first call on each device looks up the array's device address and, with the CUDA
 *     runtime's lazy loading, is also when the driver places the kernels and the array on that
 *     device: make it at start-up, while memory is still to be had, and before starting any
 *     stream capture on that device.  The address is remembered per device; after a
 *     cudaDeviceReset() it is stale and the process must not use this entry point again;
 *   - every call on a device uses the same array: calls that can overlap on the GPU (different
 *     streams, different host threads) race and must be serialised by the caller;
 *   - neither this function nor anything it calls allocates or frees memory. */
#define BITSKNN_STATIC_SCRATCH_BYTES (8u << 20)
int bitsknn_select_split_static(const float* d_dist, int64_t ld, const int32_t* d_label_offsets, int64_t q,
                                int64_t n, int k, int splits, float* d_out_dist, int32_t* d_out_idx,
                                bitsknn_stream_t stream);

/* Merge of `lists` candidate lists per query into the k smallest pairs (candidate j of
 * list l of query i is at [l * list_stride + i * query_stride + j], strides in elements).
 * Pass 2 of the reference's split-row scheme (bits_knn.cu:170-183) and the merge step of
 * the database-sharded search (lists = number of shards). lists * k <= 65536.
 * bitsknn_merge_lists with sorted_lists != 0 promises that every list is ascending in the pair
 * order (what the selection and fused entry points write, padding (+inf, INT32_MAX) at the end):
 * then only the merging phases of the sorting network run.  bitsknn_merge makes no assumption. */
int bitsknn_merge(const float* d_cand_dist, const int32_t* d_cand_idx, int64_t list_stride,
                  int64_t query_stride, int64_t q, int lists, int k, float* d_out_dist,
                  int32_t* d_out_idx, bitsknn_stream_t stream);
int bitsknn_merge_lists(const float* d_cand_dist, const int32_t* d_cand_idx, int64_t list_stride,
                        int64_t query_stride, int64_t q, int lists, int k, int sorted_lists,
                        float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream);

/* Exact re-ranking of candidates: for every query the squared distance to each of its
 * `candidates` candidate points is recomputed in FP32 exactly as BITSKNN_L2_EXACT does (one
 * FMA chain of (y - x)^2 over the coordinates in order, the reference's l2_ops,
 * include/bits/distance/abstract_gemm.cuh:79-93) and the k smallest (distance, index) pairs by
 * that distance are reported.  Meant for the candidates a reduced-precision search returns
 * (a selection with k + margin over a TF32 / BF16 distance matrix): the result then carries the
 * distances of the FP32 path, and a neighbour that the rounded distances ranked a few places too
 * low is put back in its place.  The tensor-core modes of bitsknn_fused run this step themselves.
 * The reference has no such step; its tensor-core kernels report their rounded distances
 * (include/bits/topk/singlepass/detail/fused_tc_kernel.cuh:346,440).
 *   d_cand_idx   int32[q][ld_cand]: candidate j of query i = index_base + row of d_points;
 *                distinct per query; entries outside [index_base, index_base + n) are skipped
 *   candidates   candidates per query taken from each row (1 ... 65536), k <= BITSKNN_MAX_K */
int bitsknn_refine(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim,
                   const int32_t* d_cand_idx, int64_t ld_cand, int candidates, int32_t index_base, int k,
                   float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Squared-L2 distance matrix, GEMM form.
 * Replaces magma_distance::compute / magma_partial_distance::compute
 * (src/distance/magma_distance.cu:73-103) and run_abstract_gemm<Ops>
 * (include/bits/distance/abstract_gemm.cuh:730-755).
 *
 *   d_points   float32[n][dim] row-major,  d_queries float32[q][dim] row-major
 *   d_dist     float32[q][ld] row-major, ld >= n
 *   mode       BITSKNN_L2_EXACT    sum_d fmaf(x-y, x-y, acc), dims ascending (l2_ops)
 *              BITSKNN_L2_PARTIAL  |x|^2 - 2 x.y, FMA chains in dim order (partial_l2_ops);
 *                                  the query norm is NOT added, as in the reference
 *              BITSKNN_L2_TF32 / BITSKNN_L2_BF16  tensor-core modes (tcgen05, TMEM
 *                                  accumulators): |x|^2 + |y|^2 - 2 x.y with the dot product in
 *                                  reduced input precision and FP32 accumulation
 * Tensor-core modes need a workspace of bitsknn_l2_workspace_bytes(n, q, dim, mode). */
enum bitsknn_l2_mode
{
    BITSKNN_L2_EXACT = 0,
    BITSKNN_L2_PARTIAL = 1,
    BITSKNN_L2_TF32 = 2,
    BITSKNN_L2_BF16 = 3
};
size_t bitsknn_l2_workspace_bytes(int64_t n, int64_t q, int dim, int mode);

/* d_dst[c][r] = d_src[r][c] for a row-major rows x cols float32 matrix (rows <= 2097120), on the
 * device.  For inputs that arrive coordinate-major (dim x n: rows = dim, cols = n): every entry
 * point above takes vectors row-major, and this replaces the host-side transposes the reference
 * runs before its uploads (src/distance/magma_distance.cu:32-50,
 * src/topk/singlepass/fused_cache_knn.cu:159-194, src/main.cpp:333-343). */
int bitsknn_transpose(const float* d_src, int64_t rows, int64_t cols, float* d_dst, bitsknn_stream_t stream);
int bitsknn_l2(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim, int mode,
               float* d_dist, int64_t ld, void* d_workspace, size_t workspace_bytes,
               bitsknn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * `bits-fused`: distances computed tile by tile on chip and fed straight into the top-k;
 * the q x n matrix is never written.  Replaces fused_cache_knn::selection /
 * fused_cache::run / launch_fused_cache (src/topk/singlepass/fused_cache_knn.cu:29-216,
 * include/bits/topk/singlepass/fused_cache_kernel.hpp:35-36).
 *
 *   mode        BITSKNN_L2_PARTIAL (FP32 FFMA, bit-exact with the reference's fused kernel:
 *               reported distances are |x|^2 - 2 x.y), BITSKNN_L2_EXACT (FP32, sum (x-y)^2), or
 *               BITSKNN_L2_TF32 / BITSKNN_L2_BF16: the distance tile is produced by tcgen05
 *               tensor-core MMAs in tensor memory and consumed from there; the pairs that survive
 *               the scan are re-ranked by their exact FP32 distance (see bitsknn_refine), which is
 *               what is reported: sum (x-y)^2 as in BITSKNN_L2_EXACT.  The rounded tensor-core
 *               distances only decide which pairs are candidates, so the result is checked against
 *               the FP32 path by recall@k and k-th distance error rather than bit for bit
 *   k           1 <= k <= BITSKNN_FUSED_MAX_K
 *   index_base  added to every reported index (shard base of a sharded database)
 *   d_workspace bitsknn_fused_workspace_bytes() bytes, 256-byte aligned.  Required by the
 *               tensor-core modes (input images, norms, partial lists).  Optional for the FP32
 *               modes: with it the tiled kernel (128 queries per block, lists in the workspace)
 *               runs, with NULL / 0 the 8-queries-per-block kernel; both give the same bits
 * --------------------------------------------------------------------------------------- */
size_t bitsknn_fused_workspace_bytes(int64_t n, int64_t q, int dim, int k, int mode);
int bitsknn_fused(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim, int k,
                  int mode, int32_t index_base, float* d_out_dist, int32_t* d_out_idx, void* d_workspace,
                  size_t workspace_bytes, bitsknn_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Database-sharded search over several GPUs (one handle per GPU; one process or host thread
 * per GPU).  The reference is single-GPU; this generalises its split-row two-pass scheme
 * (single_query_bits, src/topk/singlepass/bits_knn.cu:116-186: per-slice top-k with
 * label_offsets, then a pass over the slices' candidates) from slices of a row to shards of the
 * database, and plugs into the same registry (src/main.cpp:109-155) as the id `bits-sharded`.
 *
 * Rank r of `world` holds points / matrix columns [shard_begin, shard_begin + n_local) and ALL
 * queries.  A search = local top-k with global labels on the caller's stream, ONE NCCL all-gather
 * of every rank's q x k pairs and the merge kernel, both on a stream the handle owns; every rank
 * ends with the full result in its d_out arrays.  All ranks must issue the same sequence of
 * searches with the same q and k.
 *
 *   bitsknn_sharded_unique_id  fills BITSKNN_SHARDED_ID_BYTES bytes (an ncclUniqueId) on one
 *                              rank; the caller distributes them to the others
 *   bitsknn_sharded_create     makes the handle and its own NCCL communicator from that id
 *                              (collective: every rank calls it, with its device current)
 *   bitsknn_sharded_init       the same over a communicator the caller owns (an ncclComm_t);
 *                              world == 1 needs neither NCCL nor a communicator (NULL)
 *   bitsknn_sharded_workspace_bytes  exchange buffers the caller provides (0 for one shard)
 *   ..._search_select / ..._search_fused  one search; stream-ordered: the result is complete
 *                              for work queued on `stream` after the call
 *   ..._submit_select          the same search, but `stream` does not wait for the exchange and
 *                              the merge, so they overlap the next search's local kernel (two
 *                              buffer slots); bitsknn_sharded_drain makes `stream` wait for
 *                              everything submitted
 *   bitsknn_sharded_destroy    synchronises the handle's stream, frees its events, stream and
 *                              (if it made it) the communicator
 * NCCL is looked up at run time (libnccl.so.2); without it these calls return BITSKNN_ERR_COMM
 * for world > 1 and the rest of the library is unaffected.
 * --------------------------------------------------------------------------------------- */
#define BITSKNN_SHARDED_ID_BYTES 128
typedef struct bitsknn_sharded bitsknn_sharded_t;
int bitsknn_sharded_unique_id(void* id);
int bitsknn_sharded_create(bitsknn_sharded_t** handle, const void* id, int rank, int world);
int bitsknn_sharded_init(bitsknn_sharded_t** handle, void* nccl_comm, int rank, int world);
int bitsknn_sharded_destroy(bitsknn_sharded_t* handle);
size_t bitsknn_sharded_workspace_bytes(const bitsknn_sharded_t* handle, int64_t q, int k);
int bitsknn_sharded_search_select(bitsknn_sharded_t* handle, const float* d_dist, int64_t ld, int64_t q,
                                  int64_t n_local, int k, int32_t shard_begin, float* d_out_dist,
                                  int32_t* d_out_idx, void* d_workspace, size_t workspace_bytes,
                                  bitsknn_stream_t stream);
int bitsknn_sharded_submit_select(bitsknn_sharded_t* handle, const float* d_dist, int64_t ld, int64_t q,
                                  int64_t n_local, int k, int32_t shard_begin, float* d_out_dist,
                                  int32_t* d_out_idx, void* d_workspace, size_t workspace_bytes,
                                  bitsknn_stream_t stream);
int bitsknn_sharded_search_fused(bitsknn_sharded_t* handle, const float* d_points, const float* d_queries,
                                 int64_t n_local, int64_t q, int dim, int k, int mode, int32_t shard_begin,
                                 float* d_out_dist, int32_t* d_out_idx, void* d_fused_workspace,
                                 size_t fused_workspace_bytes, void* d_workspace, size_t workspace_bytes,
                                 bitsknn_stream_t stream);
int bitsknn_sharded_drain(bitsknn_sharded_t* handle, bitsknn_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* BITSKNN_H_ */
