// `bits-fused`, FP32, tiled variant: the distance tile of the GEMM-form kernel (128 queries x 128
// points per block, 8 x 8 per thread, one FMA chain per distance in coordinate order -- the same
// arithmetic as l2.cu, hence bit-identical with the reference's fused kernel and its
// abstract_gemm) is filtered in registers instead of being stored.
//
// Against the 8-queries-per-block kernel of fused.cu every database coordinate fetched from L2
// now feeds 128 queries instead of 8, and the inner loop is the distance kernel's (64 FMAs per
// four 128-bit shared-memory loads).  Per query the block keeps a 32-slot candidate buffer in
// shared memory (slots handed out by shared atomics) and the radius; the sorted lists
// (32 * IPT pairs) live in the workspace and are only touched by folds, which the warps do with
// the shuffle networks of warpfold.cuh (warp w folds queries w, w + 8, ...).  A fold round runs
// when some buffer is at least half full or a candidate found no slot; candidates left over are
// filtered again by the tightened radius.  The database may be cut into `parts` ranges scanned by
// different blocks (small q); merge_lists() merges the per-part lists.
// Reference counterpart: fused_cache_kernel::run + multi_buffer
// (include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:25-305,716-799).
#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "sortnet.cuh"
#include "warpfold.cuh"

namespace bitsknn
{

namespace
{

constexpr int FT_BM = 128;
constexpr int FT_BN = 128;
constexpr int FT_BK = 16;
constexpr int FT_PAD = FT_BM + 4;
constexpr int FT_THREADS = 256;
constexpr int FT_CAP = 32;

struct tiled_params
{
    const float* points;
    const float* queries;
    int64_t n;
    int64_t q;
    int dim;
    int k;
    int32_t index_base;
    int parts;
    int64_t tiles; // point tiles of 128
    float* list_d; // [parts][q][KL]
    int32_t* list_x;
    int vec_in;
};

__device__ __forceinline__ void ft_load8(const float* __restrict__ base, int64_t rows, int dim, int64_t row, int k0,
                                         bool vec, float (&v)[8])
{
    if (row < rows && vec && k0 + 8 <= dim)
    {
        const float4* p = reinterpret_cast<const float4*>(base + row * dim + k0);
        const float4 a = __ldg(p);
        const float4 b = __ldg(p + 1);
        v[0] = a.x;
        v[1] = a.y;
        v[2] = a.z;
        v[3] = a.w;
        v[4] = b.x;
        v[5] = b.y;
        v[6] = b.z;
        v[7] = b.w;
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        v[j] = (row < rows && k0 + j < dim) ? __ldg(base + row * dim + k0 + j) : 0.0F;
    }
}

template <int IPT, bool PARTIAL>
__global__ void __launch_bounds__(FT_THREADS, 2) fused_tiled_kernel(const tiled_params p)
{
    constexpr int KL = 32 * IPT;
    extern __shared__ __align__(16) unsigned char ft_smem[];
    auto As = reinterpret_cast<float(*)[FT_BK][FT_PAD]>(ft_smem);                        // [2][16][132]
    auto Bs = reinterpret_cast<float(*)[FT_BK][FT_PAD]>(ft_smem + sizeof(float) * 2 * FT_BK * FT_PAD);
    auto buf_d = reinterpret_cast<float(*)[FT_CAP]>(ft_smem + sizeof(float) * 4 * FT_BK * FT_PAD); // [128][32]
    auto buf_x = reinterpret_cast<int(*)[FT_CAP]>(ft_smem + sizeof(float) * (4 * FT_BK * FT_PAD + FT_BM * FT_CAP));
    __shared__ int cnt[FT_BM];
    __shared__ float sr_d[FT_BM];
    __shared__ int sr_x[FT_BM];
    __shared__ int has_list[FT_BM];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const int64_t qb = blockIdx.x / p.parts;
    const int part = static_cast<int>(blockIdx.x - qb * p.parts);
    const int64_t m0 = qb * FT_BM;
    const int64_t per = (p.tiles + p.parts - 1) / p.parts;
    const int64_t t_begin = part * per;
    const int64_t t_end = t_begin + per < p.tiles ? t_begin + per : p.tiles;

    const int lrow = tid >> 1;
    const int lk = (tid & 1) * 8;
    const int ntk = (p.dim + FT_BK - 1) / FT_BK;

    if (tid < FT_BM)
    {
        cnt[tid] = 0;
        has_list[tid] = 0;
        // a query row beyond q never accepts a candidate
        sr_d[tid] = m0 + tid < p.q ? INFINITY : -INFINITY;
        sr_x[tid] = PAD_IDX;
    }
    __syncthreads();

    // folds the buffers of this warp's queries (w, w + 8, ...) that hold candidates
    auto fold_round = [&]() {
        for (int qi = warp; qi < FT_BM; qi += FT_THREADS / 32)
        {
            // a fold costs a round trip to the list whatever the buffer holds, so nearly empty
            // buffers wait for a later round (the final flush takes whatever is left)
            const int have = cnt[qi];
            const bool flush = have >= FT_CAP / 4;
            if (flush && m0 + qi < p.q)
            {
                const int valid = have < FT_CAP ? have : FT_CAP;
                const float cd = lane < valid ? buf_d[qi][lane] : INFINITY;
                const int cx = lane < valid ? buf_x[qi][lane] : PAD_IDX;
                float* gl_d = p.list_d + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
                int32_t* gl_x = p.list_x + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
                float nd;
                int nx;
                warp_fold_global<IPT>(cd, cx, has_list[qi] != 0, gl_d, gl_x, p.k, lane, nd, nx);
                if (lane == 0)
                {
                    sr_d[qi] = nd;
                    sr_x[qi] = nx;
                    has_list[qi] = 1;
                    cnt[qi] = 0;
                }
            }
            __syncwarp();
        }
    };

    for (int64_t t = t_begin; t < t_end; ++t)
    {
        const int64_t n0 = t * FT_BN;
        float acc[8][8];
        float nrm[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            nrm[i] = 0.0F;
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                acc[i][j] = 0.0F;
            }
        }
        float ra[8];
        float rb[8];
        ft_load8(p.queries, p.q, p.dim, m0 + lrow, lk, p.vec_in != 0, ra);
        ft_load8(p.points, p.n, p.dim, n0 + lrow, lk, p.vec_in != 0, rb);
        __syncthreads(); // the previous tile's readers of buffer 0 are done
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            As[0][lk + j][lrow] = ra[j];
            Bs[0][lk + j][lrow] = rb[j];
        }
        __syncthreads();
        int buf = 0;
        for (int kt = 0; kt < ntk; ++kt)
        {
            if (kt + 1 < ntk)
            {
                ft_load8(p.queries, p.q, p.dim, m0 + lrow, (kt + 1) * FT_BK + lk, p.vec_in != 0, ra);
                ft_load8(p.points, p.n, p.dim, n0 + lrow, (kt + 1) * FT_BK + lk, p.vec_in != 0, rb);
            }
#pragma unroll
            for (int kk = 0; kk < FT_BK; ++kk)
            {
                const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
                const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
                const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
                const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
                const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                if constexpr (PARTIAL)
                {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                    {
                        nrm[j] = fmaf(b[j], b[j], nrm[j]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
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
            if (kt + 1 < ntk)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    As[buf ^ 1][lk + j][lrow] = ra[j];
                    Bs[buf ^ 1][lk + j][lrow] = rb[j];
                }
            }
            __syncthreads();
            buf ^= 1;
        }

        // ---- filter the 8 x 8 distances of this thread -------------------------------------
        unsigned long long pending = 0;
        const int ncols = p.n - n0 < FT_BN ? static_cast<int>(p.n - n0) : FT_BN; // valid columns of this tile
        const int c_lo = tx * 4;       // this thread's columns: c_lo .. c_lo + 3 and 64 + c_lo .. + 3
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const int row = i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4);
            const float rd = sr_d[row];
            // finish the 8 distances of this row and look at their minimum first: once the radius
            // has settled almost every row is rejected by this one comparison
            float mn = INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                const float d = PARTIAL ? (nrm[j] - 2.0F * acc[i][j]) : acc[i][j];
                acc[i][j] = d;
                mn = fminf(mn, d);
            }
            if (mn <= rd)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const float d = acc[i][j];
                    const int c = j < 4 ? c_lo + j : 64 + c_lo + (j - 4);
                    if (d <= rd && c < ncols)
                    {
                        const int idx = p.index_base + static_cast<int>(n0) + c;
                        if (pair_lt(d, idx, rd, sr_x[row]))
                        {
                            const int pos = atomicAdd(&cnt[row], 1);
                            if (pos < FT_CAP)
                            {
                                buf_d[row][pos] = d;
                                buf_x[row][pos] = idx;
                            }
                            else
                            {
                                pending |= 1ULL << (i * 8 + j);
                            }
                        }
                    }
                }
            }
        }
        // a fold round when a candidate found no slot or some buffer is at least half full
        bool trigger = pending != 0 || (tid < FT_BM && cnt[tid] >= FT_CAP / 2);
        while (__syncthreads_or(trigger ? 1 : 0) != 0)
        {
            fold_round();
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                const int row = i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const unsigned long long bit = 1ULL << (i * 8 + j);
                    if ((pending & bit) != 0)
                    {
                        const int64_t col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                        const int idx = p.index_base + static_cast<int>(col);
                        bool done = true;
                        if (pair_lt(acc[i][j], idx, sr_d[row], sr_x[row]))
                        {
                            const int pos = atomicAdd(&cnt[row], 1);
                            if (pos < FT_CAP)
                            {
                                buf_d[row][pos] = acc[i][j];
                                buf_x[row][pos] = idx;
                            }
                            else
                            {
                                done = false;
                            }
                        }
                        if (done)
                        {
                            pending &= ~bit;
                        }
                    }
                }
            }
            trigger = pending != 0;
        }
    }

    // flush what is left and make sure every live query of this part has a complete list
    __syncthreads();
    if (tid < FT_BM && has_list[tid] == 0 && cnt[tid] == 0)
    {
        cnt[tid] = -1; // marks "write an all-padding list"
    }
    __syncthreads();
    for (int qi = warp; qi < FT_BM; qi += FT_THREADS / 32)
    {
        const int have = cnt[qi];
        if (have != 0 && m0 + qi < p.q)
        {
            const int valid = have < 0 ? 0 : (have < FT_CAP ? have : FT_CAP);
            const float cd = lane < valid ? buf_d[qi][lane] : INFINITY;
            const int cx = lane < valid ? buf_x[qi][lane] : PAD_IDX;
            float* gl_d = p.list_d + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
            int32_t* gl_x = p.list_x + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
            float nd;
            int nx;
            warp_fold_global<IPT>(cd, cx, has_list[qi] != 0, gl_d, gl_x, p.k, lane, nd, nx);
        }
        __syncwarp();
    }
}

struct tiled_layout
{
    int kl;
    int parts;
    size_t off_ld, off_lx, total;
};

tiled_layout tiled_layout_of(int64_t n, int64_t q, int k)
{
    tiled_layout l{};
    l.kl = k <= 32 ? 32 : (k <= 64 ? 64 : (k <= 128 ? 128 : 256));
    const int64_t nqb = (q + FT_BM - 1) / FT_BM;
    const int64_t tiles = (n + FT_BN - 1) / FT_BN;
    // two blocks fit an SM; split the database only when the query tiles cannot fill them
    const int slots = 2 * device_sm_count();
    const int64_t want = 4 * nqb >= 3 * slots ? 1 : (slots + nqb - 1) / nqb;
    l.parts = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, std::max<int64_t>(1, tiles / 32))));
    const size_t lists = static_cast<size_t>(l.parts) * static_cast<size_t>(q) * l.kl;
    l.off_ld = 0;
    l.off_lx = (lists * 4 + 255) & ~static_cast<size_t>(255);
    l.total = l.off_lx + ((lists * 4 + 255) & ~static_cast<size_t>(255));
    return l;
}

template <int IPT>
int launch_tiled(const tiled_params& p, int mode, int64_t grid, cudaStream_t stream)
{
    constexpr size_t smem = sizeof(float) * (4 * FT_BK * FT_PAD + 2 * FT_BM * FT_CAP);
    if (mode == BITSKNN_L2_PARTIAL)
    {
        auto kernel = fused_tiled_kernel<IPT, true>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FT_THREADS, smem, stream>>>(p);
    }
    else
    {
        auto kernel = fused_tiled_kernel<IPT, false>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FT_THREADS, smem, stream>>>(p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

} // namespace

size_t fused_tiled_workspace_bytes(int64_t n, int64_t q, int k)
{
    if (n <= 0 || q <= 0 || k <= 0)
    {
        return 0;
    }
    return tiled_layout_of(n, q, k).total;
}

int fused_tiled_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int mode,
                       int32_t index_base, float* out_dist, int32_t* out_idx, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream)
{
    const tiled_layout l = tiled_layout_of(n, q, k);
    if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255U) != 0)
    {
        return fail(BITSKNN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) needed, %zu given", l.total,
                    workspace_bytes);
    }
    auto* ws = static_cast<unsigned char*>(workspace);
    tiled_params p{};
    p.points = points;
    p.queries = queries;
    p.n = n;
    p.q = q;
    p.dim = dim;
    p.k = k;
    p.index_base = index_base;
    p.parts = l.parts;
    p.tiles = (n + FT_BN - 1) / FT_BN;
    p.list_d = reinterpret_cast<float*>(ws + l.off_ld);
    p.list_x = reinterpret_cast<int32_t*>(ws + l.off_lx);
    p.vec_in = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(points) & 15U) == 0) &&
               ((reinterpret_cast<uintptr_t>(queries) & 15U) == 0);
    const int64_t grid = ((q + FT_BM - 1) / FT_BM) * l.parts;
    int rc;
    switch (l.kl)
    {
    case 32:
        rc = launch_tiled<1>(p, mode, grid, stream);
        break;
    case 64:
        rc = launch_tiled<2>(p, mode, grid, stream);
        break;
    case 128:
        rc = launch_tiled<4>(p, mode, grid, stream);
        break;
    default:
        rc = launch_tiled<8>(p, mode, grid, stream);
        break;
    }
    if (rc != BITSKNN_OK)
    {
        return rc;
    }
    return merge_lists(p.list_d, p.list_x, static_cast<int64_t>(q) * l.kl, l.kl, q, l.parts, l.kl, k, nullptr, out_dist,
                       out_idx, stream);
}

} // namespace bitsknn
