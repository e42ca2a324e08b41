// Ablation variants of the selection, kept selectable so that what the register-resident list
// and the filtered buffer buy can be measured on the same data (the reference keeps its
// ancestors of `bits` registered for the same reason, src/main.cpp:111-155, and sweeps them in
// scripts/run-bitonic-sort.sh:33-54 and scripts/run-buffer.sh:65-75):
//
//   BITSKNN_ABLATION_NO_BUFFER    `partial-bitonic-regs` (src/topk/singlepass/partial_bitonic.cu:217-294):
//                                 no radius filter -- every value is sorted and merged into the
//                                 register-resident list.  This is select_kernel with its filter off.
//   BITSKNN_ABLATION_SHARED_LIST  `partial-bitonic-buffered-static`
//                                 (src/topk/singlepass/partial_bitonic_buffered.cu:216-337): the
//                                 filtered buffer is there, but the sorted list lives in shared
//                                 memory and every network step goes through shared memory.
// Both give the same pairs as bitsknn_select (same pair order).
#include <cmath>
#include <cstdint>

#include "common.cuh"

namespace bitsknn
{

namespace
{

constexpr int SL_THREADS = 256;
constexpr int SL_BATCH = 2; // values per thread and iteration, like the reference's BATCH_SIZE (:397)

// One compare-exchange pass of the (size, stride) bitonic network over K pairs in shared memory;
// blocks of `size` elements alternate direction, flipped as a whole when `desc`.
__device__ __forceinline__ void shared_step(float* d, int* x, int K, int size, int stride, bool desc)
{
    for (int t = threadIdx.x; t < K / 2; t += SL_THREADS)
    {
        const int lo = 2 * t - (t & (stride - 1)); // index with bit `stride` clear
        const int hi = lo + stride;
        const bool asc = (((lo & size) == 0) != desc);
        const bool hi_lt_lo = pair_lt(d[hi], x[hi], d[lo], x[lo]);
        if (hi_lt_lo == asc)
        {
            const float td = d[lo];
            d[lo] = d[hi];
            d[hi] = td;
            const int tx = x[lo];
            x[lo] = x[hi];
            x[hi] = tx;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void shared_sort(float* d, int* x, int K, bool desc)
{
    for (int size = 2; size <= K; size <<= 1)
    {
        for (int stride = size >> 1; stride > 0; stride >>= 1)
        {
            // the last phase (size == K) sorts the whole array one way
            shared_step(d, x, K, size == K ? 2 * K : size, stride, desc);
        }
    }
}

// Merges the buffer into the list (both K pairs in shared memory): buffer sorted descending,
// element-wise minimum, bitonic merge of the list; the buffer is reset to padding.
__device__ __forceinline__ void shared_merge(float* list_d, int* list_x, float* buf_d, int* buf_x, int K)
{
    shared_sort(buf_d, buf_x, K, true);
    for (int i = threadIdx.x; i < K; i += SL_THREADS)
    {
        if (pair_lt(buf_d[i], buf_x[i], list_d[i], list_x[i]))
        {
            list_d[i] = buf_d[i];
            list_x[i] = buf_x[i];
        }
        buf_d[i] = INFINITY;
        buf_x[i] = PAD_IDX;
    }
    __syncthreads();
    for (int stride = K >> 1; stride > 0; stride >>= 1)
    {
        shared_step(list_d, list_x, K, 2 * K, stride, false);
    }
}

__global__ void __launch_bounds__(SL_THREADS)
    select_shared_list_kernel(const float* __restrict__ dist, int64_t ld, int64_t n, int k, int K,
                              float* __restrict__ out_dist, int32_t* __restrict__ out_idx)
{
    extern __shared__ unsigned char sl_smem[];
    float* list_d = reinterpret_cast<float*>(sl_smem);
    int* list_x = reinterpret_cast<int*>(list_d + K);
    float* buf_d = reinterpret_cast<float*>(list_x + K);
    int* buf_x = reinterpret_cast<int*>(buf_d + K);
    __shared__ int buffer_size;
    const int tid = threadIdx.x;
    const float* row = dist + static_cast<int64_t>(blockIdx.x) * ld;

    for (int i = tid; i < K; i += SL_THREADS)
    {
        list_d[i] = INFINITY;
        list_x[i] = PAD_IDX;
        buf_d[i] = INFINITY;
        buf_x[i] = PAD_IDX;
    }
    if (tid == 0)
    {
        buffer_size = 0;
    }
    __syncthreads();
    float r_d = INFINITY;
    int r_x = PAD_IDX;

    for (int64_t base = 0; base < n; base += SL_THREADS * SL_BATCH)
    {
        float d[SL_BATCH];
        int x[SL_BATCH];
        int pos[SL_BATCH];
#pragma unroll
        for (int j = 0; j < SL_BATCH; ++j)
        {
            const int64_t col = base + tid + j * SL_THREADS;
            x[j] = static_cast<int>(col);
            d[j] = col < n ? row[col] : INFINITY;
            pos[j] = (col < n && pair_lt(d[j], x[j], r_d, r_x)) ? atomicAdd(&buffer_size, 1) : -1;
        }
        while (true)
        {
            bool overflow = false;
#pragma unroll
            for (int j = 0; j < SL_BATCH; ++j)
            {
                if (pos[j] >= 0 && pos[j] < K)
                {
                    buf_d[pos[j]] = d[j];
                    buf_x[pos[j]] = x[j];
                    pos[j] = -1;
                }
                overflow = overflow || pos[j] >= K;
                pos[j] -= pos[j] >= K ? K : 0;
            }
            if (__syncthreads_or(overflow ? 1 : 0) == 0)
            {
                break;
            }
            // the buffer is full: merge it; what did not fit takes the first slots of the empty buffer
            shared_merge(list_d, list_x, buf_d, buf_x, K);
            if (tid == 0)
            {
                buffer_size -= K;
            }
            r_d = list_d[k - 1];
            r_x = list_x[k - 1];
            __syncthreads();
        }
    }
    shared_merge(list_d, list_x, buf_d, buf_x, K);
    for (int i = tid; i < k; i += SL_THREADS)
    {
        out_dist[static_cast<int64_t>(blockIdx.x) * k + i] = list_d[i];
        out_idx[static_cast<int64_t>(blockIdx.x) * k + i] = list_x[i] == PAD_IDX ? i : list_x[i];
    }
}

} // namespace

} // namespace bitsknn

using namespace bitsknn;

extern "C" int bitsknn_select_ablation(const float* d_dist, int64_t ld, int64_t q, int64_t n, int k, int variant,
                                       float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream)
{
    auto cs = static_cast<cudaStream_t>(stream);
    if (variant == BITSKNN_ABLATION_NO_BUFFER)
    {
        return select_rows(d_dist, ld, nullptr, 0, nullptr, 0, q, n, k, d_out_dist, d_out_idx, cs, /*no_filter*/ true);
    }
    if (variant != BITSKNN_ABLATION_SHARED_LIST)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "unknown ablation variant %d", variant);
    }
    if (d_dist == nullptr || d_out_dist == nullptr || d_out_idx == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (q < 0 || n <= 0 || ld < n || n >= 0x7fffffffLL || q > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: q=%lld n=%lld ld=%lld", static_cast<long long>(q),
                    static_cast<long long>(n), static_cast<long long>(ld));
    }
    if (k < 1 || k > BITSKNN_MAX_K)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_K, "Unsupported k value: %d", k);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    int K = 16; // the reference instantiates the list for powers of two from 16 (definitions_common.hpp:4)
    while (K < k)
    {
        K *= 2;
    }
    const size_t smem = static_cast<size_t>(K) * 16U;
    BITSKNN_CUDA_TRY(cudaFuncSetAttribute(select_shared_list_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    {
        kernel_scope timed{"select_shared_list_kernel", cs};
        select_shared_list_kernel<<<static_cast<unsigned>(q), SL_THREADS, smem, cs>>>(d_dist, ld, n, k, K, d_out_dist,
                                                                                       d_out_idx);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}
