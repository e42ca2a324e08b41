// Squared-L2 distance matrix in GEMM form, FP32 exact modes (CUDA cores).
//
// dist[i][j] for query i and point j, both row-major with `dim` coordinates:
//   BITSKNN_L2_EXACT    acc = fmaf(q - x, q - x, acc) over the coordinates in increasing order
//                       (the reference's l2_ops, include/bits/distance/abstract_gemm.cuh:79-93)
//   BITSKNN_L2_PARTIAL  dot = fmaf(q, x, dot), nrm = fmaf(x, x, nrm), result nrm - 2 dot
//                       (partial_l2_ops, abstract_gemm.cuh:139-169; query norm not added)
// Every output has ONE accumulator that sees the coordinates in order -- no split-K, no tree
// reduction -- so the bits equal the reference kernel's (abstract_gemm.cuh:494-714), whose
// tiling (96x96 tile, 6x6 per thread, K tile 16) is replaced by a 128x128 tile with 8x8 per
// thread, 128-bit shared-memory fragments and row-major inputs read directly (the reference
// transposes both inputs on the host first: src/distance/magma_distance.cu:32-50).
// Coordinates beyond `dim` in the last K tile are zero on both sides, which leaves every
// accumulator unchanged (fmaf(0, 0, acc) == acc), like the reference's guarded loads.
#include <cstdint>

#include "common.cuh"

namespace bitsknn
{

// tensor-core modes live in l2_tc.cu
size_t l2_tc_workspace_bytes(int64_t n, int64_t q, int dim, int mode);
int l2_tc_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int mode, float* dist,
                 int64_t ld, void* workspace, size_t workspace_bytes, cudaStream_t stream);

namespace
{

constexpr int BM = 128; // queries per block
constexpr int BN = 128; // points per block
constexpr int BK = 16;  // coordinates per shared-memory tile
constexpr int PADDED = BM + 4;
constexpr int L2_THREADS = 256;

// Loads 8 consecutive coordinates [k0, k0+8) of row `row` (zero outside the matrix).
__device__ __forceinline__ void load8(const float* __restrict__ base, int64_t rows, int dim, int64_t row, int k0,
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

template <bool PARTIAL>
__global__ void __launch_bounds__(L2_THREADS, 2)
    l2_fp32_kernel(const float* __restrict__ points, const float* __restrict__ queries, int64_t n, int64_t q, int dim,
                   float* __restrict__ out, int64_t ld, int vec_in, int vec_out)
{
    __shared__ __align__(16) float As[2][BK][PADDED];
    __shared__ __align__(16) float Bs[2][BK][PADDED];

    const int tid = threadIdx.x;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * BN;

    // loader role: row tid/2 of the tile, coordinates (tid&1)*8 .. +7 of the K tile
    const int lrow = tid >> 1;
    const int lk = (tid & 1) * 8;

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

    const int ntiles = (dim + BK - 1) / BK;
    float ra[8];
    float rb[8];
    load8(queries, q, dim, m0 + lrow, lk, vec_in != 0, ra);
    load8(points, n, dim, n0 + lrow, lk, vec_in != 0, rb);
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        As[0][lk + j][lrow] = ra[j];
        Bs[0][lk + j][lrow] = rb[j];
    }
    __syncthreads();

    int buf = 0;
    for (int t = 0; t < ntiles; ++t)
    {
        if (t + 1 < ntiles)
        {
            load8(queries, q, dim, m0 + lrow, (t + 1) * BK + lk, vec_in != 0, ra);
            load8(points, n, dim, n0 + lrow, (t + 1) * BK + lk, vec_in != 0, rb);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk)
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
        if (t + 1 < ntiles)
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

    // epilogue: rows m0 + {ty*4+i, 64+ty*4+i}, columns n0 + {tx*4+j, 64+tx*4+j}
#pragma unroll
    for (int i = 0; i < 8; ++i)
    {
        const int64_t row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= q)
        {
            continue;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half)
        {
            const int64_t col = n0 + half * 64 + tx * 4;
            float r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const float v = acc[i][half * 4 + j];
                r[j] = PARTIAL ? (nrm[half * 4 + j] - 2.0F * v) : v;
            }
            float* dst = out + row * ld + col;
            if (vec_out != 0 && col + 3 < n)
            {
                __stcs(reinterpret_cast<float4*>(dst), make_float4(r[0], r[1], r[2], r[3]));
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    if (col + j < n)
                    {
                        __stcs(dst + j, r[j]);
                    }
                }
            }
        }
    }
}

} // namespace

} // namespace bitsknn

using namespace bitsknn;

namespace bitsknn
{

namespace
{

// dst[c][r] = src[r][c] for a rows x cols matrix: 32 x 32 tiles through a padded shared-memory
// tile so that both the loads and the stores are coalesced.
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ src, int64_t rows, int64_t cols,
                                                        float* __restrict__ dst)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31;
    const int ty = threadIdx.x >> 5; // 0..7
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32;
#pragma unroll
    for (int i = 0; i < 32; i += 8)
    {
        const int64_t r = r0 + ty + i;
        const int64_t c = c0 + tx;
        tile[ty + i][tx] = (r < rows && c < cols) ? src[r * cols + c] : 0.0F;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 32; i += 8)
    {
        const int64_t c = c0 + ty + i;
        const int64_t r = r0 + tx;
        if (c < cols && r < rows)
        {
            dst[c * rows + r] = tile[tx][ty + i];
        }
    }
}

} // namespace

} // namespace bitsknn

extern "C" int bitsknn_transpose(const float* d_src, int64_t rows, int64_t cols, float* d_dst, bitsknn_stream_t stream)
{
    using namespace bitsknn;
    if (d_src == nullptr || d_dst == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (rows < 0 || cols < 0 || (rows + 31) / 32 > 65535 || (cols + 31) / 32 > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: rows=%lld cols=%lld (at most 2097120 rows)",
                    static_cast<long long>(rows), static_cast<long long>(cols));
    }
    if (rows == 0 || cols == 0)
    {
        return BITSKNN_OK;
    }
    const dim3 grid(static_cast<unsigned>((cols + 31) / 32), static_cast<unsigned>((rows + 31) / 32));
    transpose_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_src, rows, cols, d_dst);
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

extern "C" size_t bitsknn_l2_workspace_bytes(int64_t n, int64_t q, int dim, int mode)
{
    if (mode == BITSKNN_L2_TF32 || mode == BITSKNN_L2_BF16)
    {
        return l2_tc_workspace_bytes(n, q, dim, mode);
    }
    return 0;
}

extern "C" int bitsknn_l2(const float* d_points, const float* d_queries, int64_t n, int64_t q, int dim, int mode,
                          float* d_dist, int64_t ld, void* d_workspace, size_t workspace_bytes,
                          bitsknn_stream_t stream)
{
    if (d_points == nullptr || d_queries == nullptr || d_dist == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (n <= 0 || q < 0 || ld < n)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: n=%lld q=%lld ld=%lld", static_cast<long long>(n),
                    static_cast<long long>(q), static_cast<long long>(ld));
    }
    if (dim < 1 || dim > 65536)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d", dim);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    auto cs = static_cast<cudaStream_t>(stream);
    if (mode == BITSKNN_L2_TF32 || mode == BITSKNN_L2_BF16)
    {
        return l2_tc_launch(d_points, d_queries, n, q, dim, mode, d_dist, ld, d_workspace, workspace_bytes, cs);
    }
    if (mode != BITSKNN_L2_EXACT && mode != BITSKNN_L2_PARTIAL)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "unknown distance mode %d", mode);
    }
    const int64_t gx = (n + BM - 1) / BN;
    const int64_t gy = (q + BM - 1) / BM;
    if (gy > 65535 || gx > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "too many queries for one launch: %lld", static_cast<long long>(q));
    }
    const int vec_in = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15U) == 0) &&
                       ((reinterpret_cast<uintptr_t>(d_queries) & 15U) == 0);
    const int vec_out = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_dist) & 15U) == 0);
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    kernel_scope timed{"l2_fp32_kernel", cs};
    if (mode == BITSKNN_L2_PARTIAL)
    {
        l2_fp32_kernel<true><<<grid, L2_THREADS, 0, cs>>>(d_points, d_queries, n, q, dim, d_dist, ld, vec_in, vec_out);
    }
    else
    {
        l2_fp32_kernel<false><<<grid, L2_THREADS, 0, cs>>>(d_points, d_queries, n, q, dim, d_dist, ld, vec_in, vec_out);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}
