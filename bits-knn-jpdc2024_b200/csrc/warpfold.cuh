// Warp-level fold of up to 32 candidate pairs into a sorted list of 32 * IPT pairs that lives
// in global memory (L2-resident workspace), shared by the fused kernels.
#pragma once

#include "common.cuh"
#include "sortnet.cuh"

namespace bitsknn
{

// Sorts a bitonic array of 32 * IPT pairs ascending; entry e lives in lane e % 32, register
// e / 32.  Strides of 32 and more are exchanges between registers of one lane (M = stride / 32,
// a compile-time constant so that the arrays stay in registers), smaller ones are shuffles.
template <int IPT, int M>
struct striped_reg_steps
{
    static __device__ __forceinline__ void run(float (&d)[IPT], int (&x)[IPT])
    {
        if constexpr (M >= 1)
        {
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                if ((r & M) == 0)
                {
                    if (pair_lt(d[r | M], x[r | M], d[r], x[r]))
                    {
                        const float td = d[r];
                        d[r] = d[r | M];
                        d[r | M] = td;
                        const int tx = x[r];
                        x[r] = x[r | M];
                        x[r | M] = tx;
                    }
                }
            }
            striped_reg_steps<IPT, M / 2>::run(d, x);
        }
    }
};

template <int IPT>
__device__ __forceinline__ void merge_striped(float (&d)[IPT], int (&x)[IPT], int lane)
{
    striped_reg_steps<IPT, IPT / 2>::run(d, x);
#pragma unroll
    for (int J = 16; J >= 1; J >>= 1)
    {
        const bool keep_min = (lane & J) == 0;
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const float pd = __shfl_xor_sync(FULL_MASK, d[r], J);
            const int px = __shfl_xor_sync(FULL_MASK, x[r], J);
            if (pair_lt(pd, px, d[r], x[r]) == keep_min)
            {
                d[r] = pd;
                x[r] = px;
            }
        }
    }
}

// Entry `pos` of a striped list (register pos / 32 of lane pos % 32), delivered to every lane.
// (Opaque selects: a plain ?: chain is turned into an indexed load from a stack copy of the
// list, which costs a local store per list update.)
template <int IPT>
__device__ __forceinline__ float striped_entry_d(const float (&ld)[IPT], int pos)
{
    float nd = ld[0];
#pragma unroll
    for (int r = 1; r < IPT; ++r)
    {
        const int pick = r == pos / 32 ? 1 : 0;
        asm("{\n.reg .pred p;\nsetp.ne.s32 p, %2, 0;\nselp.f32 %0, %1, %0, p;\n}" : "+f"(nd) : "f"(ld[r]), "r"(pick));
    }
    return __shfl_sync(FULL_MASK, nd, pos & 31);
}

template <int IPT>
__device__ __forceinline__ int striped_entry_x(const int (&lx)[IPT], int pos)
{
    int nx = lx[0];
#pragma unroll
    for (int r = 1; r < IPT; ++r)
    {
        const int pick = r == pos / 32 ? 1 : 0;
        asm("{\n.reg .pred p;\nsetp.ne.s32 p, %2, 0;\nselp.s32 %0, %1, %0, p;\n}" : "+r"(nx) : "r"(lx[r]), "r"(pick));
    }
    return __shfl_sync(FULL_MASK, nx, pos & 31);
}

// Folds the candidates (one pair per lane, padding = (+inf, PAD_IDX)) into the list at
// gl_d / gl_x (striped: entry e in lane e % 32, register e / 32; `has_list` false = the list is
// still empty and is not read).  The candidates are sorted descending with shuffles, the
// element-wise minimum against the list's last 32 entries leaves the 32 * IPT smallest pairs as
// a bitonic array (the candidates count as padded with +inf in front), the striped merge sorts
// it, and the list is written back.  Every lane returns the new radius pair (entry k - 1) and,
// when `half_d` is given, the distance of entry ceil(k / 2) - 1.
template <int IPT>
__device__ __forceinline__ void warp_fold_global(float cand_d, int cand_x, bool has_list, float* gl_d, int32_t* gl_x,
                                                 int k, int lane, float& radius_d, int& radius_x,
                                                 float* half_d = nullptr)
{
    float cd[1] = {cand_d};
    int cx[1] = {cand_x};
    block_sort<32, 1>(cd, cx, true, nullptr, nullptr, lane);
    float ld[IPT];
    int lx[IPT];
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        ld[r] = has_list ? gl_d[r * 32 + lane] : INFINITY;
        lx[r] = has_list ? gl_x[r * 32 + lane] : PAD_IDX;
    }
    if (pair_lt(cd[0], cx[0], ld[IPT - 1], lx[IPT - 1]))
    {
        ld[IPT - 1] = cd[0];
        lx[IPT - 1] = cx[0];
    }
    merge_striped<IPT>(ld, lx, lane);
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        gl_d[r * 32 + lane] = ld[r];
        gl_x[r * 32 + lane] = lx[r];
    }
    radius_d = striped_entry_d<IPT>(ld, k - 1);
    radius_x = striped_entry_x<IPT>(lx, k - 1);
    if (half_d != nullptr)
    {
        // entry ceil(k / 2) - 1: with a second list over other points, the larger of the two
        // lists' entries at this position has at least k pairs below or at it
        *half_d = striped_entry_d<IPT>(ld, (k + 1) / 2 - 1);
    }
    __syncwarp(); // the list stores are ordered before any later load by this warp
}

// The same fold as a real function call: the kernels that fold from several places in their
// scan loops keep ONE copy of the sorting networks in their instruction stream this way.
struct radius_pair
{
    float d;
    int x;
    float half_d; // distance of entry ceil(k / 2) - 1
};

template <int IPT>
__device__ __noinline__ radius_pair warp_fold_global_call(float cand_d, int cand_x, bool has_list, float* gl_d,
                                                          int32_t* gl_x, int k, int lane)
{
    radius_pair r;
    warp_fold_global<IPT>(cand_d, cand_x, has_list, gl_d, gl_x, k, lane, r.d, r.x, &r.half_d);
    return r;
}

} // namespace bitsknn
