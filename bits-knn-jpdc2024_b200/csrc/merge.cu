// Merge of candidate lists into the k smallest pairs per query, and the exact re-ranking of
// candidates.
//
// One block per query folds `lists * kin` candidates into a register-resident sorted list,
// L = 256 * IPT at a time, with the networks of sortnet.cuh.  Three ways to take the candidates:
//   * sorted runs (RUN > 0): every list arrives ascending (the output of the selection and fused
//     kernels), so a round of L candidates is L / RUN sorted runs.  Runs are loaded alternately
//     reversed / straight, which is the state the bitonic sort is in after its phase RUN: only the
//     phases 2 RUN ... L remain (none when RUN == L: the fold is a reversed load, an element-wise
//     minimum and one bitonic merge);
//   * unsorted (RUN == 0): full sort of every round;
//   * re-ranking (RERANK): the candidate's distance is not read but recomputed from the vectors
//     as the FP32 chain  acc = fmaf(y - x, y - x, acc)  over the coordinates in order -- the
//     reference's l2_ops (include/bits/distance/abstract_gemm.cuh:79-93) -- so the reported pairs
//     carry exactly the distances of the FP32 path and are ordered by them.
// Pass 2 of the reference's split-row scheme (src/topk/singlepass/bits_knn.cu:170-183, which runs
// the selection kernel again over the candidates with explicit labels) has this role.
#include <algorithm>
#include <cmath>
#include <cstdint>

#include "common.cuh"
#include "sortnet.cuh"

namespace bitsknn
{

namespace
{

constexpr int MERGE_THREADS = 256;

struct merge_params
{
    const float* cand_dist;
    const int32_t* cand_idx;
    int64_t list_stride;
    int64_t query_stride;
    int lists;
    int kin; // candidates per list
    int k;   // pairs reported
    const float* bias; // nullable: one value per query, added to every reported distance
    float* out_dist;
    int32_t* out_idx;
    // re-ranking only
    const float* points;  // [n][dim]
    const float* queries; // [q][dim]
    int64_t n;
    int dim;
    int32_t index_base; // candidate index = index_base + row of `points`
};

// Squared distance of query `qs` (shared memory) and point row `x`, coordinates in order.
__device__ __forceinline__ float exact_l2(const float* __restrict__ x, const float* qs, int dim, bool vec4)
{
    float acc = 0.0F;
    if (vec4)
    {
        const float4* xv = reinterpret_cast<const float4*>(x);
        for (int c = 0; c < dim / 4; ++c)
        {
            const float4 v = __ldg(xv + c);
            const float d0 = qs[4 * c] - v.x;
            acc = fmaf(d0, d0, acc);
            const float d1 = qs[4 * c + 1] - v.y;
            acc = fmaf(d1, d1, acc);
            const float d2 = qs[4 * c + 2] - v.z;
            acc = fmaf(d2, d2, acc);
            const float d3 = qs[4 * c + 3] - v.w;
            acc = fmaf(d3, d3, acc);
        }
    }
    else
    {
        for (int c = 0; c < dim; ++c)
        {
            const float d = qs[c] - __ldg(x + c);
            acc = fmaf(d, d, acc);
        }
    }
    return acc;
}

template <int IPT, int RUN, bool RERANK>
__global__ void __launch_bounds__(MERGE_THREADS) merge_kernel(const merge_params p)
{
    constexpr int THREADS = MERGE_THREADS;
    constexpr int L = THREADS * IPT;
    __shared__ float sd[L];
    __shared__ int sx[L];
    extern __shared__ float qs[]; // re-ranking: the query's coordinates
    const int tid = threadIdx.x;
    const int64_t query = blockIdx.x;

    bool vec4 = false;
    if constexpr (RERANK)
    {
        for (int c = tid; c < p.dim; c += THREADS)
        {
            qs[c] = p.queries[query * p.dim + c];
        }
        vec4 = (p.dim & 3) == 0 && (reinterpret_cast<uintptr_t>(p.points) & 15U) == 0;
        __syncthreads();
    }

    // candidate `j` of list `l`: its pair, with the distance recomputed when re-ranking
    auto fetch = [&](int l, int j, float& d, int& x) {
        const int64_t at = l * p.list_stride + query * p.query_stride + j;
        x = p.cand_idx[at];
        if constexpr (RERANK)
        {
            const int64_t row = static_cast<int64_t>(x) - p.index_base;
            if (x == PAD_IDX || row < 0 || row >= p.n)
            {
                d = INFINITY;
                x = PAD_IDX;
            }
            else
            {
                d = exact_l2(p.points + row * p.dim, qs, p.dim, vec4);
            }
        }
        else
        {
            d = p.cand_dist[at];
        }
    };

    float ld[IPT];
    int lx[IPT];
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        ld[r] = INFINITY;
        lx[r] = PAD_IDX;
    }

    if constexpr (RUN > 0)
    {
        static_assert(RUN <= L, "a run fills at most one round");
        constexpr int PER_ROUND = L / RUN; // lists per round
        for (int l0 = 0; l0 < p.lists; l0 += PER_ROUND)
        {
            float cd[IPT];
            int cx[IPT];
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                // element e of the round (blocked arrangement) is entry i of run j; even runs are
                // loaded reversed so that they descend (padding first), odd runs ascend
                const int e = tid * IPT + r;
                const int j = e / RUN;
                const int i = e - j * RUN;
                const int src = (j & 1) == 0 ? RUN - 1 - i : i;
                cd[r] = INFINITY;
                cx[r] = PAD_IDX;
                if (l0 + j < p.lists && src < p.kin)
                {
                    fetch(l0 + j, src, cd[r], cx[r]);
                }
            }
            sort_phases_from<THREADS, IPT, L, RUN>::run(cd, cx, true, sd, sx, tid);
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                if (pair_lt(cd[r], cx[r], ld[r], lx[r]))
                {
                    ld[r] = cd[r];
                    lx[r] = cx[r];
                }
            }
            block_merge_bitonic<THREADS, IPT>(ld, lx, sd, sx, tid);
        }
    }
    else
    {
        const int total = p.lists * p.kin;
        for (int round = 0; round < total; round += L)
        {
            float cd[IPT];
            int cx[IPT];
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                const int ci = round + r * THREADS + tid;
                cd[r] = INFINITY;
                cx[r] = PAD_IDX;
                if (ci < total)
                {
                    const int l = ci / p.kin;
                    fetch(l, ci - l * p.kin, cd[r], cx[r]);
                }
            }
            block_fold<THREADS, IPT>(ld, lx, cd, cx, sd, sx, tid);
        }
    }
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        const int e = tid * IPT + r;
        if (e < p.k)
        {
            p.out_dist[query * p.k + e] = p.bias != nullptr ? ld[r] + p.bias[query] : ld[r];
            p.out_idx[query * p.k + e] = lx[r] == PAD_IDX ? e : lx[r];
        }
    }
}

template <int IPT, int RUN, bool RERANK>
int launch_merge(const merge_params& p, int64_t q, cudaStream_t stream)
{
    const size_t dyn = RERANK ? static_cast<size_t>(p.dim) * sizeof(float) : 0;
    {
        kernel_scope timed{RERANK ? "rerank_kernel" : "merge_kernel", stream};
        merge_kernel<IPT, RUN, RERANK><<<static_cast<unsigned>(q), MERGE_THREADS, dyn, stream>>>(p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

// Sorted input: the run length is the list length rounded up to a power of two, at least 32
// (shorter lists count as padded) and at most the round.
template <int IPT>
int dispatch_sorted(const merge_params& p, int64_t q, cudaStream_t stream)
{
    constexpr int L = MERGE_THREADS * IPT;
    int run = 32;
    while (run < p.kin)
    {
        run *= 2;
    }
    if constexpr (L >= 2048)
    {
        if (run == 2048)
        {
            return launch_merge<IPT, 2048, false>(p, q, stream);
        }
    }
    if constexpr (L >= 1024)
    {
        if (run == 1024)
        {
            return launch_merge<IPT, 1024, false>(p, q, stream);
        }
    }
    if constexpr (L >= 512)
    {
        if (run == 512)
        {
            return launch_merge<IPT, 512, false>(p, q, stream);
        }
    }
    switch (run)
    {
    case 32:
        return launch_merge<IPT, 32, false>(p, q, stream);
    case 64:
        return launch_merge<IPT, 64, false>(p, q, stream);
    case 128:
        return launch_merge<IPT, 128, false>(p, q, stream);
    case 256:
        return launch_merge<IPT, 256, false>(p, q, stream);
    default:
        return launch_merge<IPT, 0, false>(p, q, stream); // a list longer than the round: plain sort
    }
}

template <int IPT>
int dispatch_kind(const merge_params& p, int64_t q, merge_input input, cudaStream_t stream)
{
    switch (input)
    {
    case merge_input::sorted:
        return dispatch_sorted<IPT>(p, q, stream);
    case merge_input::rerank:
        return launch_merge<IPT, 0, true>(p, q, stream);
    default:
        return launch_merge<IPT, 0, false>(p, q, stream);
    }
}

int dispatch_merge(const merge_params& p, int64_t q, merge_input input, cudaStream_t stream)
{
    if (p.k <= 256)
    {
        return dispatch_kind<1>(p, q, input, stream);
    }
    if (p.k <= 512)
    {
        return dispatch_kind<2>(p, q, input, stream);
    }
    if (p.k <= 1024)
    {
        return dispatch_kind<4>(p, q, input, stream);
    }
    return dispatch_kind<8>(p, q, input, stream);
}

} // namespace

int merge_lists(const float* cd, const int32_t* cx, int64_t list_stride, int64_t query_stride, int64_t q, int lists,
                int kin, int k, const float* bias, float* od, int32_t* ox, merge_input input, cudaStream_t stream)
{
    merge_params p{};
    p.cand_dist = cd;
    p.cand_idx = cx;
    p.list_stride = list_stride;
    p.query_stride = query_stride;
    p.lists = lists;
    p.kin = kin;
    p.k = k;
    p.bias = bias;
    p.out_dist = od;
    p.out_idx = ox;
    return dispatch_merge(p, q, input, stream);
}

int rerank_lists(const int32_t* cx, int64_t list_stride, int64_t query_stride, int64_t q, int lists, int kin, int k,
                 const float* points, const float* queries, int64_t n, int dim, int32_t index_base, float* od,
                 int32_t* ox, cudaStream_t stream)
{
    merge_params p{};
    p.cand_idx = cx;
    p.list_stride = list_stride;
    p.query_stride = query_stride;
    p.lists = lists;
    p.kin = kin;
    p.k = k;
    p.out_dist = od;
    p.out_idx = ox;
    p.points = points;
    p.queries = queries;
    p.n = n;
    p.dim = dim;
    p.index_base = index_base;
    return dispatch_merge(p, q, merge_input::rerank, stream);
}

} // namespace bitsknn

using namespace bitsknn;

extern "C" int bitsknn_merge(const float* d_cand_dist, const int32_t* d_cand_idx, int64_t list_stride,
                             int64_t query_stride, int64_t q, int lists, int k, float* d_out_dist,
                             int32_t* d_out_idx, bitsknn_stream_t stream)
{
    return bitsknn_merge_lists(d_cand_dist, d_cand_idx, list_stride, query_stride, q, lists, k, 0, d_out_dist,
                               d_out_idx, stream);
}

extern "C" int bitsknn_merge_lists(const float* d_cand_dist, const int32_t* d_cand_idx, int64_t list_stride,
                                   int64_t query_stride, int64_t q, int lists, int k, int sorted_lists,
                                   float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream)
{
    if (d_cand_dist == nullptr || d_cand_idx == nullptr || d_out_dist == nullptr || d_out_idx == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (q < 0 || lists < 1 || list_stride < 0 || query_stride < 0 || q > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: q=%lld lists=%d", static_cast<long long>(q), lists);
    }
    if (k < 1 || k > BITSKNN_MAX_K)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_K, "Unsupported k value: %d", k);
    }
    if (static_cast<int64_t>(lists) * k > 65536)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "lists * k = %lld exceeds 65536", static_cast<long long>(lists) * k);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    return merge_lists(d_cand_dist, d_cand_idx, list_stride, query_stride, q, lists, k, k, nullptr, d_out_dist,
                       d_out_idx, sorted_lists != 0 ? merge_input::sorted : merge_input::unsorted,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int bitsknn_refine(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim,
                              const int32_t* d_cand_idx, int64_t ld_cand, int candidates, int32_t index_base, int k,
                              float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream)
{
    if (d_points == nullptr || d_queries == nullptr || d_cand_idx == nullptr || d_out_dist == nullptr ||
        d_out_idx == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (n <= 0 || q < 0 || q > 0x7fffffffLL || candidates < 1 || ld_cand < candidates || candidates > 65536)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: n=%lld q=%lld candidates=%d ld=%lld",
                    static_cast<long long>(n), static_cast<long long>(q), candidates, static_cast<long long>(ld_cand));
    }
    if (dim < 1 || dim > 4096)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (re-ranking takes 1..4096)", dim);
    }
    if (k < 1 || k > BITSKNN_MAX_K)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_K, "Unsupported k value: %d", k);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    return rerank_lists(d_cand_idx, 0, ld_cand, q, 1, candidates, k, d_points, d_queries, n, dim, index_base, d_out_dist,
                        d_out_idx, static_cast<cudaStream_t>(stream));
}
