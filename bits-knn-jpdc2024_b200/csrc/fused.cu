// `bits-fused`: brute-force k-NN whose distance tiles never leave the chip (FP32 modes).
//
// One block of 256 threads owns 8 queries and scans the whole database (or database shard):
//   * a tile of 1024 points x 4 coordinates is staged in shared memory (transposed to
//     coordinate-major while it is stored), double buffered against the global loads;
//   * every thread accumulates the 8 x 4 distances of its 4 points to the 8 queries in
//     registers, one FMA chain per distance in increasing coordinate order -- bit-identical
//     to the reference's fused kernel, which reports |x|^2 - 2 x.y WITHOUT the query norm
//     (include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:496-519, 622-630);
//   * a distance below its query's radius (current k-th pair) takes a slot in that query's
//     shared-memory buffer; when a buffer overflows, every warp folds ITS query's buffer
//     into that query's sorted list, which lives in the warp's registers (32 * IPT pairs),
//     with shuffle-only bitonic networks -- no block-wide sort is ever needed because
//     query w belongs to warp w.
// Same algorithm as fused_cache_kernel::run + multi_buffer (structs.cuh:25-305, 716-799);
// differences: row-major inputs read directly (the reference transposes on the host,
// src/topk/singlepass/fused_cache_knn.cu:159-194), candidates that did not fit are filtered
// again by the tightened radius instead of being carried over, and pairs are ordered by
// (distance, index) so that ties resolve to the lowest index.
#include <cstdint>

#include "common.cuh"
#include "tuning_table.cuh"
#include "sortnet.cuh"

namespace bitsknn
{

// tensor-core modes live in fused_tc.cu
size_t fused_tc_workspace_bytes(int64_t n, int64_t q, int dim, int k, int mode);
int fused_tc_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int mode,
                    int32_t index_base, float* out_dist, int32_t* out_idx, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream);

// FP32 tiled variant (128 queries per block) lives in fused_tiled.cu
bool fused_tiled_supports(int dim);
size_t fused_tiled_workspace_bytes(int64_t n, int64_t q, int dim, int k);
int fused_tiled_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int mode,
                       int32_t index_base, float* out_dist, int32_t* out_idx, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream);

namespace
{

constexpr int FUSED_THREADS = 256;
constexpr int QT = 8;                  // queries per block = warps per block
constexpr int PPT = 4;                 // points per thread
constexpr int PT = FUSED_THREADS * PPT; // points per tile
constexpr int DT = 4;                  // coordinates per staged tile
// Automatic choice between the two FP32 kernels: the tuning table (tuning_table.inc, from a sweep at
// q = 2^14, n = 2^20 on B200) first.  The tiled kernel wins from dim 16 on, and below that for short
// lists (its folds go through L2, the 8-query kernel keeps its lists in registers): dim 4: 10.1 ms
// against 15.4 at k = 16, 16.5 against 16.5 at k = 128, 29.9 against 17.3 at k = 256.
inline bool fused_prefers_tiled(int dim, int k)
{
    if (const fused_shape* row = find_fused_shape(dim, k); row != nullptr)
    {
        return row->tiled != 0;
    }
    return dim >= 16 || k <= 64 || (k <= 128 && dim >= 8);
}

struct fused_params
{
    const float* points;  // [n][dim]
    const float* queries; // [q][dim]
    int64_t n;
    int64_t q;
    int dim;
    int dim_pad; // dim rounded up to a multiple of DT
    int k;
    int32_t index_base;
    float* out_dist;
    int32_t* out_idx;
    int vec; // 16-byte loads of the points are possible
};

template <int IPT, bool PARTIAL>
__global__ void __launch_bounds__(FUSED_THREADS, 2) fused_kernel(const fused_params p)
{
    constexpr int KL = 32 * IPT; // list length = buffer capacity per query

    extern __shared__ __align__(16) unsigned char smem[];
    float* As = reinterpret_cast<float*>(smem);                   // [dim_pad][QT] query tile
    float* Bs = As + static_cast<size_t>(p.dim_pad) * QT;         // [2][DT][PT]
    float* buf_d = Bs + 2 * DT * PT;                              // [QT][KL]
    int* buf_x = reinterpret_cast<int*>(buf_d + QT * KL);         // [QT][KL]
    int* cnt = buf_x + QT * KL;                                   // [QT]
    float* sr_d = reinterpret_cast<float*>(cnt + QT);             // [QT] radius distance
    int* sr_x = reinterpret_cast<int*>(sr_d + QT);                // [QT] radius index

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t q0 = static_cast<int64_t>(blockIdx.x) * QT;

    // query tile, coordinate-major, zero padded (extra coordinates and missing queries)
    for (int e = tid; e < p.dim_pad * QT; e += FUSED_THREADS)
    {
        const int d = e / QT;
        const int i = e - d * QT;
        As[e] = (d < p.dim && q0 + i < p.q) ? p.queries[(q0 + i) * p.dim + d] : 0.0F;
    }
    if (tid < QT)
    {
        cnt[tid] = 0;
        sr_d[tid] = INFINITY;
        sr_x[tid] = PAD_IDX;
    }

    // this warp's query list (ascending, blocked over the lanes)
    float ld[IPT];
    int lx[IPT];
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        ld[r] = INFINITY;
        lx[r] = PAD_IDX;
    }

    const int nkt = p.dim_pad / DT;
    const int64_t ntiles = (p.n + PT - 1) / PT;
    const int64_t total_it = ntiles * nkt;

    // global -> register staging of (tile, kt): thread loads DT coordinates of points
    // tile*PT + u*256 + tid, u = 0..3 (stored conflict-free as Bs[c][u*256 + tid])
    float4 pf[PPT];
    auto prefetch = [&](int64_t tile, int kt) {
#pragma unroll
        for (int u = 0; u < PPT; ++u)
        {
            const int64_t pt = tile * PT + u * FUSED_THREADS + tid;
            const int c0 = kt * DT;
            float4 v = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
            if (pt < p.n)
            {
                const float* src = p.points + pt * p.dim + c0;
                if (p.vec != 0)
                {
                    v = __ldg(reinterpret_cast<const float4*>(src));
                }
                else
                {
                    v.x = c0 + 0 < p.dim ? __ldg(src + 0) : 0.0F;
                    v.y = c0 + 1 < p.dim ? __ldg(src + 1) : 0.0F;
                    v.z = c0 + 2 < p.dim ? __ldg(src + 2) : 0.0F;
                    v.w = c0 + 3 < p.dim ? __ldg(src + 3) : 0.0F;
                }
            }
            pf[u] = v;
        }
    };

    float acc[QT][PPT];
    float nrm[PPT];
    auto reset_acc = [&]() {
#pragma unroll
        for (int j = 0; j < PPT; ++j)
        {
            nrm[j] = 0.0F;
#pragma unroll
            for (int i = 0; i < QT; ++i)
            {
                acc[i][j] = 0.0F;
            }
        }
    };
    reset_acc();

    // folds this warp's buffer into its list (whole warp, shuffle-only networks)
    auto fold_own = [&]() {
        const int have = cnt[warp];
        const int valid = have < KL ? have : KL;
        if (valid > 0)
        {
            float cd[IPT];
            int cx[IPT];
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                const int s = r * 32 + lane;
                cd[r] = s < valid ? buf_d[warp * KL + s] : INFINITY;
                cx[r] = s < valid ? buf_x[warp * KL + s] : PAD_IDX;
            }
            block_fold<32, IPT>(ld, lx, cd, cx, nullptr, nullptr, lane);
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                if (lane * IPT + r == p.k - 1)
                {
                    sr_d[warp] = ld[r];
                    sr_x[warp] = lx[r];
                }
            }
        }
        __syncwarp();
        if (lane == 0)
        {
            cnt[warp] = 0;
        }
    };

    // tries to place pair (d, idx) of query i; returns false if the buffer is full
    auto offer = [&](int i, float d, int idx) -> bool {
        const int pos = atomicAdd(&cnt[i], 1);
        if (pos < KL)
        {
            buf_d[i * KL + pos] = d;
            buf_x[i * KL + pos] = idx;
            return true;
        }
        return false;
    };

    prefetch(0, 0);
    int kt = 0;
    int64_t tile = 0;
    for (int64_t it = 0; it < total_it; ++it)
    {
        float* B = Bs + (it & 1) * (DT * PT);
#pragma unroll
        for (int u = 0; u < PPT; ++u)
        {
            B[0 * PT + u * FUSED_THREADS + tid] = pf[u].x;
            B[1 * PT + u * FUSED_THREADS + tid] = pf[u].y;
            B[2 * PT + u * FUSED_THREADS + tid] = pf[u].z;
            B[3 * PT + u * FUSED_THREADS + tid] = pf[u].w;
        }
        __syncthreads(); // tile visible; everyone is done with the other buffer's previous use
        if (it + 1 < total_it)
        {
            const bool wrap = kt + 1 == nkt;
            prefetch(wrap ? tile + 1 : tile, wrap ? 0 : kt + 1);
        }
#pragma unroll
        for (int c = 0; c < DT; ++c)
        {
            const float4 b4 = *reinterpret_cast<const float4*>(&B[c * PT + tid * PPT]);
            const float4 a0 = *reinterpret_cast<const float4*>(&As[(kt * DT + c) * QT]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[(kt * DT + c) * QT + 4]);
            const float a[QT] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[PPT] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int j = 0; j < PPT; ++j)
            {
                if constexpr (PARTIAL)
                {
                    nrm[j] = fmaf(b[j], b[j], nrm[j]);
                }
#pragma unroll
                for (int i = 0; i < QT; ++i)
                {
                    if constexpr (PARTIAL)
                    {
                        acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    }
                    else
                    {
                        const float diff = a[i] - b[j];
                        acc[i][j] = fmaf(diff, diff, acc[i][j]);
                    }
                }
            }
        }
        if (kt + 1 < nkt)
        {
            ++kt;
            continue;
        }

        // ---- all coordinates of this tile are in: filter the 8 x 4 distances -------------
        const int64_t pt0 = tile * PT + static_cast<int64_t>(tid) * PPT; // first point of this thread
        unsigned pending = 0;
#pragma unroll
        for (int i = 0; i < QT; ++i)
        {
            const float rd = sr_d[i];
#pragma unroll
            for (int j = 0; j < PPT; ++j)
            {
                const float d = PARTIAL ? (nrm[j] - 2.0F * acc[i][j]) : acc[i][j];
                acc[i][j] = d;
                if (d <= rd && pt0 + j < p.n)
                {
                    const int idx = p.index_base + static_cast<int>(pt0 + j);
                    if (pair_lt(d, idx, rd, sr_x[i]) && !offer(i, d, idx))
                    {
                        pending |= 1U << (i * PPT + j);
                    }
                }
            }
        }
        // some buffer overflowed: fold them all, tighten the radii, offer the rest again
        while (__syncthreads_or(pending != 0 ? 1 : 0) != 0)
        {
            fold_own();
            __syncthreads();
#pragma unroll
            for (int i = 0; i < QT; ++i)
            {
#pragma unroll
                for (int j = 0; j < PPT; ++j)
                {
                    const unsigned bit = 1U << (i * PPT + j);
                    if ((pending & bit) != 0)
                    {
                        const int idx = p.index_base + static_cast<int>(pt0 + j);
                        if (!pair_lt(acc[i][j], idx, sr_d[i], sr_x[i]) || offer(i, acc[i][j], idx))
                        {
                            pending &= ~bit;
                        }
                    }
                }
            }
        }
        reset_acc();
        kt = 0;
        ++tile;
    }

    __syncthreads();
    fold_own();
    if (q0 + warp < p.q)
    {
        float* od = p.out_dist + (q0 + warp) * p.k;
        int32_t* ox = p.out_idx + (q0 + warp) * p.k;
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = lane * IPT + r;
            if (e < p.k)
            {
                od[e] = ld[r];
                ox[e] = lx[r] == PAD_IDX ? e : lx[r];
            }
        }
    }
}

template <int IPT>
int launch_fused(const fused_params& p, int mode, cudaStream_t stream)
{
    constexpr int KL = 32 * IPT;
    const size_t smem = (static_cast<size_t>(p.dim_pad) * QT + 2 * DT * PT + 2 * QT * KL + 3 * QT) * 4;
    if (smem > 200 * 1024)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (query tile does not fit shared memory)",
                    p.dim);
    }
    const int64_t grid = (p.q + QT - 1) / QT;
    kernel_scope timed{"fused_kernel", stream};
    if (mode == BITSKNN_L2_PARTIAL)
    {
        auto kernel = fused_kernel<IPT, true>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FUSED_THREADS, smem, stream>>>(p);
    }
    else
    {
        auto kernel = fused_kernel<IPT, false>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FUSED_THREADS, smem, stream>>>(p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

} // namespace

} // namespace bitsknn

using namespace bitsknn;

extern "C" size_t bitsknn_fused_workspace_bytes(int64_t n, int64_t q, int dim, int k, int mode)
{
    if (mode == BITSKNN_L2_TF32 || mode == BITSKNN_L2_BF16)
    {
        return fused_tc_workspace_bytes(n, q, dim, k, mode);
    }
    if (mode == BITSKNN_L2_PARTIAL || mode == BITSKNN_L2_EXACT)
    {
        // optional for the FP32 modes: with it the tiled kernel (128 queries per block) can be used
        return fused_tiled_workspace_bytes(n, q, dim, k);
    }
    return 0;
}

extern "C" int bitsknn_fused(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim, int k,
                             int mode, int32_t index_base, float* d_out_dist, int32_t* d_out_idx, void* d_workspace,
                             size_t workspace_bytes, bitsknn_stream_t stream)
{
    if (d_points == nullptr || d_queries == nullptr || d_out_dist == nullptr || d_out_idx == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (n <= 0 || q < 0 || n > 0x7fffffffLL - PT || q > 0x7fffffffLL * QT / 2)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: n=%lld q=%lld", static_cast<long long>(n),
                    static_cast<long long>(q));
    }
    if (static_cast<int64_t>(index_base) + n > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "index_base + n exceeds the int32 label range");
    }
    if (dim < 1)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d", dim);
    }
    if (k < 1 || k > BITSKNN_FUSED_MAX_K)
    {
        // the reference's fused dispatcher rejects k the same way (fused_cache_knn.cu:76-80)
        return fail(BITSKNN_ERR_UNSUPPORTED_K, "Unsupported k value: %d", k);
    }
    if (mode != BITSKNN_L2_PARTIAL && mode != BITSKNN_L2_EXACT && mode != BITSKNN_L2_TF32 && mode != BITSKNN_L2_BF16)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "fused mode %d is not available", mode);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    if (mode == BITSKNN_L2_TF32 || mode == BITSKNN_L2_BF16)
    {
        return fused_tc_launch(d_points, d_queries, n, q, dim, k, mode, index_base, d_out_dist, d_out_idx, d_workspace,
                               workspace_bytes, static_cast<cudaStream_t>(stream));
    }
    // FP32: the tiled kernel needs its list workspace; without one (or when asked through the
    // "fused.variant" knob: 0 = 8-query blocks, 1 = tiled, 2 = automatic) the 8-query kernel runs
    const int variant = tuning_value("fused.variant", 2);
    const bool have_ws = fused_tiled_supports(dim) && d_workspace != nullptr &&
                         workspace_bytes >= fused_tiled_workspace_bytes(n, q, dim, k) &&
                         (reinterpret_cast<uintptr_t>(d_workspace) & 255U) == 0;
    if (have_ws && (variant == 1 || (variant == 2 && fused_prefers_tiled(dim, k))))
    {
        return fused_tiled_launch(d_points, d_queries, n, q, dim, k, mode, index_base, d_out_dist, d_out_idx,
                                  d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    }
    fused_params p{};
    p.points = d_points;
    p.queries = d_queries;
    p.n = n;
    p.q = q;
    p.dim = dim;
    p.dim_pad = ((dim + DT - 1) / DT) * DT;
    p.k = k;
    p.index_base = index_base;
    p.out_dist = d_out_dist;
    p.out_idx = d_out_idx;
    p.vec = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15U) == 0);
    auto cs = static_cast<cudaStream_t>(stream);
    if (k <= 32)
    {
        return launch_fused<1>(p, mode, cs);
    }
    if (k <= 64)
    {
        return launch_fused<2>(p, mode, cs);
    }
    if (k <= 128)
    {
        return launch_fused<4>(p, mode, cs);
    }
    return launch_fused<8>(p, mode, cs);
}
