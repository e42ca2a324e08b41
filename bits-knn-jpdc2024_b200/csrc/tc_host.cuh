// Host-side helpers and the input pre-pass shared by the tensor-core kernels
// (distance matrix in l2_tc.cu, fused search in fused_tc.cu).
#pragma once

#include <cstdint>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace bitsknn
{

namespace
{

constexpr int TILE_M = 128;        // queries per block tile (TMEM lanes)
constexpr int TILE_N = 128;        // points per MMA tile (TMEM columns per accumulator)
constexpr int STAGE_BYTES = 16384; // 128 rows x 128 bytes
constexpr int MAX_KB = 8;          // K blocks of 128 bytes in the resident query tile

// Pre-pass, one warp per row: writes the FP32 norm of the row and its MMA-input image.
//
// Plain image: the row rounded to nearest in the input type, zero padded to `ext_pad`.
// Split image (`split` != 0): every coordinate v is written as hi = rn(v) and lo = rn(v - hi),
// and the row is laid out along K as
//     queries  [hi | hi | lo]      points  [hi | lo | hi]
// so that ONE contraction over 3 * dim yields hi.hi + hi.lo + lo.hi -- the product with the
// rounding error of both inputs compensated to first order (only lo.lo is dropped).
// Compact split image (`split` == 2): hi and lo are stored once each, both zero padded to a
// whole number of MMA K steps (dp = dim rounded up to 16 BF16 / 8 TF32 elements):
//     [hi (dp) | lo (dp) | norm columns]
// and the kernel that reads it pairs the steps itself (hi.hi, lo.hi, hi.lo), which saves the
// memory traffic of the duplicated hi part.
//
// With `norm_cols` != 0 three more coordinates follow the vector part: for points the three-way
// split of -|x|^2 / 2 in the input type (together exact to FP32), for queries 1, 1, 1.  The
// contraction then yields  x.y - |x|^2 / 2, i.e. -(|x|^2 - 2 x.y) / 2: the partial distance
// comes out of the tensor core and the consumer only has to compare.
template <bool BF16>
__global__ void tc_prepare_kernel(const float* __restrict__ src, int64_t rows, int dim, int ext_pad, int split,
                                  int is_points, int norm_cols, void* __restrict__ dst, float* __restrict__ norms,
                                  float* __restrict__ max_norm = nullptr)
{
    const int lane = threadIdx.x & 31;
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows)
    {
        return;
    }
    auto round_in = [](float v) -> float {
        if constexpr (BF16)
        {
            return __bfloat162float(__float2bfloat16_rn(v));
        }
        else
        {
            uint32_t t;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(v));
            return __uint_as_float(t);
        }
    };
    auto store = [&](int c, float v) {
        if constexpr (BF16)
        {
            static_cast<__nv_bfloat16*>(dst)[row * ext_pad + c] = __float2bfloat16_rn(v);
        }
        else
        {
            static_cast<float*>(dst)[row * ext_pad + c] = v;
        }
    };
    const float* in = src + row * dim;
    float nrm = 0.0F;
    constexpr int STEP = BF16 ? 16 : 8;
    const int dp = (dim + STEP - 1) / STEP * STEP;
    if (split == 2)
    {
        for (int d = lane; d < dp; d += 32)
        {
            const float v = d < dim ? in[d] : 0.0F;
            nrm = fmaf(v, v, nrm);
            const float hi = round_in(v);
            store(d, hi);
            store(dp + d, round_in(v - hi));
        }
    }
    for (int d = lane; d < dim && split != 2; d += 32)
    {
        const float v = in[d];
        nrm = fmaf(v, v, nrm);
        const float hi = round_in(v);
        if (split != 0)
        {
            const float lo = round_in(v - hi);
            store(d, hi);
            store(dim + d, is_points != 0 ? lo : hi);
            store(2 * dim + d, is_points != 0 ? hi : lo);
        }
        else
        {
            store(d, hi);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        nrm += __shfl_xor_sync(FULL_MASK, nrm, o);
    }
    int tail = split == 2 ? 2 * dp : (split != 0 ? 3 : 1) * dim;
    if (norm_cols != 0)
    {
        if (lane == 0)
        {
            if (is_points != 0)
            {
                const float h = -0.5F * nrm;
                const float p0 = round_in(h);
                const float p1 = round_in(h - p0);
                const float p2 = round_in(h - p0 - p1);
                store(tail, p0);
                store(tail + 1, p1);
                store(tail + 2, p2);
            }
            else
            {
                store(tail, 1.0F);
                store(tail + 1, 1.0F);
                store(tail + 2, 1.0F);
            }
        }
        tail += 3;
    }
    for (int c = tail + lane; c < ext_pad; c += 32)
    {
        store(c, 0.0F);
    }
    if (lane == 0)
    {
        norms[row] = nrm;
        if (max_norm != nullptr)
        {
            // largest squared norm of all rows (non-negative floats order like their bit patterns);
            // the plain read first keeps all but a few rows away from the atomic
            if (nrm > *reinterpret_cast<volatile float*>(max_norm))
            {
                atomicMax(reinterpret_cast<int*>(max_norm), __float_as_int(nrm));
            }
        }
    }
}

using encode_fn_t = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t tensor_map_encoder()
{
    static std::once_flag once;
    static encode_fn_t fn = nullptr;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
        {
            fn = reinterpret_cast<encode_fn_t>(ptr);
        }
    });
    return fn;
}

// rows x dim_pad matrix of 4-byte (TF32) or 2-byte (BF16) elements, box = 128 bytes x `box_rows` rows
// (a row pitch that is not a whole number of boxes is fine: the last box is zero filled past the
// row's end); the pitch in bytes must be a multiple of 16
int make_map(CUtensorMap* map, void* base, int64_t rows, int dim_pad, bool bf16, unsigned box_rows = 128U)
{
    encode_fn_t encode = tensor_map_encoder();
    if (encode == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cuTensorMapEncodeTiled is not available from this driver");
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(dim_pad), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(dim_pad) * (bf16 ? 2U : 4U)};
    const cuuint32_t box[2] = {bf16 ? 64U : 32U, box_rows};
    const cuuint32_t elem[2] = {1U, 1U};
    const CUresult rc = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base,
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cuTensorMapEncodeTiled failed with code %d", static_cast<int>(rc));
    }
    return BITSKNN_OK;
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

} // namespace

} // namespace bitsknn
