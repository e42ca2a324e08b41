// Shared device/host helpers of the bitsknn kernels (sm_100a).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "bitsknn.h"

namespace bitsknn
{

// Label of a padding entry.  Padding pairs are (+inf, PAD_IDX): they sort after every real
// pair, including real +inf distances (whose labels are smaller).
constexpr int PAD_IDX = 0x7fffffff;
constexpr unsigned FULL_MASK = 0xffffffffU;

// The one total order of the engine: ascending distance, ties to the lowest index.
// The reference's compare_and_swap (include/bits/topk/bitonic_sort_regs.cuh:53-60) looks at
// the distance only; adding the index makes every network below deterministic.
__device__ __forceinline__ bool pair_lt(float ad, int ai, float bd, int bi)
{
    return ad < bd || (ad == bd && ai < bi);
}

// Records a failure on the calling host thread and returns `code`.
int fail(int code, const char* fmt, ...);
// Checks a CUDA runtime status; on failure records file:line and returns BITSKNN_ERR_CUDA.
int cuda_fail(cudaError_t err, const char* what, const char* file, int line);

#define BITSKNN_CUDA_TRY(expr)                                                                     \
    do                                                                                             \
    {                                                                                              \
        const cudaError_t bitsknn_err_ = (expr);                                                   \
        if (bitsknn_err_ != cudaSuccess)                                                           \
        {                                                                                          \
            return ::bitsknn::cuda_fail(bitsknn_err_, #expr, __FILE__, __LINE__);                  \
        }                                                                                          \
    } while (0)

// Device-side status word (0 = fine).  Kernels OR a bit into it when a bounded wait expires.
int* device_status_word();
constexpr int DEVICE_STATUS_TIMEOUT = 1;

int tuning_value(const char* key, int fallback);

// Optional device timing of the dominant kernels ("profile.kernel_events" = 1): the launch sites
// wrap their kernel in a kernel_scope, which records a CUDA event on the stream before and after
// it; bitsknn_kernel_ms() returns the elapsed time of the last launch recorded under a name.
// Off (the default) a scope does nothing.
struct kernel_scope
{
    kernel_scope(const char* name, cudaStream_t stream);
    ~kernel_scope();
    kernel_scope(const kernel_scope&) = delete;
    kernel_scope& operator=(const kernel_scope&) = delete;

private:
    void* slot_;
    cudaStream_t stream_;
};
// Blocks per query tile for kernels that may cut the database into ranges: the smallest count up
// to `max_parts` after which no larger one fills the last wave of `slots` concurrent blocks
// noticeably (2 %) better.
int balanced_parts(int64_t query_tiles, int slots, int64_t max_parts);

int device_sm_count();

// bitsknn_select with `label_base` added to every implicit label (the global index of the first
// column when the matrix is one shard of a wider one); `no_filter` switches the radius filter off
// (ablation).  Defined in select.cu.
int select_rows(const float* d_dist, int64_t ld, const int32_t* d_labels, int64_t ld_labels,
                const int32_t* d_label_offsets, int32_t label_base, int64_t q, int64_t n, int k, float* d_out_dist,
                int32_t* d_out_idx, cudaStream_t stream, bool no_filter = false);

// Merge of `lists` candidate lists of `kin` pairs per query (pair j of list l of query i at
// [l * list_stride + i * query_stride + j]) into the `k` smallest pairs; `bias` (nullable, one
// value per query) is added to the reported distances.  `input` says whether every list arrives
// ascending (then only the merging phases of the sorting network run).  Defined in merge.cu.
enum class merge_input
{
    unsorted,
    sorted,
    rerank
};
int merge_lists(const float* cand_dist, const int32_t* cand_idx, int64_t list_stride, int64_t query_stride, int64_t q,
                int lists, int kin, int k, const float* bias, float* out_dist, int32_t* out_idx, merge_input input,
                cudaStream_t stream);
// The same over candidate indices alone: every candidate's distance is recomputed from the vectors
// (FP32 chain of (y - x)^2 in coordinate order) and the k smallest pairs by that distance are
// reported.  Candidate index = index_base + row of `points`; PAD_IDX entries are skipped.
int rerank_lists(const int32_t* cand_idx, int64_t list_stride, int64_t query_stride, int64_t q, int lists, int kin,
                 int k, const float* points, const float* queries, int64_t n, int dim, int32_t index_base,
                 float* out_dist, int32_t* out_idx, cudaStream_t stream);

} // namespace bitsknn
