// Block-wide bitonic networks over a register-resident array of (distance, index) pairs.
//
// Data arrangement: a group of THREADS threads (a whole block, or one warp when THREADS == 32;
// `tid` is the thread's rank in the group) holds IPT pairs each; pair r of thread t is element
// e = t * IPT + r of a block-wide array of N = THREADS * IPT elements ("blocked"
// arrangement, the one the reference keeps its sorted lists in:
// include/bits/topk/bitonic_sort_regs.cuh:411).  A compare-exchange with partner e ^ J is
//   * register-to-register inside a thread when J < IPT,
//   * a warp shuffle when the partner lies in the same warp (J < 32 * IPT),
//   * an exchange through shared memory otherwise.
// This is the role of block_sort / block_sort_bitonic / reversed_bitonic_stage of the
// reference (bitonic_sort_regs.cuh:86-460, bitonic_sort_warp.cuh:22-119), re-derived here on
// the classic (k, j) formulation of the network with the pair order of common.cuh, so the
// result does not depend on the network: all real keys are distinct.
#pragma once

#include "common.cuh"

namespace bitsknn
{

// One compare-exchange step of the (K, J) bitonic network.  Elements whose index has bit K
// clear sort ascending (descending when `desc`), the others the opposite way; with K == N
// no element has the bit, so the whole array goes one way.
// `sd`/`sx` are shared-memory scratch arrays of N floats / ints (used only when J >= 32*IPT).
template <int THREADS, int IPT, int K, int J>
__device__ __forceinline__ void cx_step(float (&d)[IPT], int (&x)[IPT], bool desc, float* sd, int* sx, int tid)
{
    if constexpr (J < IPT)
    {
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            if ((r & J) == 0)
            {
                const int e = tid * IPT + r;
                const bool asc = (((e & K) == 0) != desc);
                // all real keys are distinct, so "not (upper < lower)" means "lower < upper" except
                // for identical padding pairs, whose exchange changes nothing
                const bool upper_lt_lower = pair_lt(d[r | J], x[r | J], d[r], x[r]);
                const bool swap = (upper_lt_lower == asc);
                if (swap)
                {
                    const float td = d[r];
                    d[r] = d[r | J];
                    d[r | J] = td;
                    const int tx = x[r];
                    x[r] = x[r | J];
                    x[r | J] = tx;
                }
            }
        }
    }
    else
    {
        constexpr int TJ = J / IPT; // partner thread = tid ^ TJ, same register r
        float pd[IPT];
        int px[IPT];
        if constexpr (TJ < 32)
        {
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                pd[r] = __shfl_xor_sync(FULL_MASK, d[r], TJ);
                px[r] = __shfl_xor_sync(FULL_MASK, x[r], TJ);
            }
        }
        else
        {
            // slot r * THREADS + tid: conflict-free for every IPT
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                sd[r * THREADS + tid] = d[r];
                sx[r * THREADS + tid] = x[r];
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < IPT; ++r)
            {
                pd[r] = sd[r * THREADS + (tid ^ TJ)];
                px[r] = sx[r * THREADS + (tid ^ TJ)];
            }
            __syncthreads();
        }
        const bool lower = (tid & TJ) == 0;
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = tid * IPT + r;
            const bool asc = (((e & K) == 0) != desc);
            const bool keep_min = (lower == asc);
            // one comparison serves both directions (see above: equal pairs are identical pairs)
            const bool take = (pair_lt(pd[r], px[r], d[r], x[r]) == keep_min);
            if (take)
            {
                d[r] = pd[r];
                x[r] = px[r];
            }
        }
    }
}

// Steps J, J/2, ..., 1 of phase K: turns bitonic runs of length 2J into sorted runs.
template <int THREADS, int IPT, int K, int J>
struct merge_steps
{
    static __device__ __forceinline__ void run(float (&d)[IPT], int (&x)[IPT], bool desc, float* sd, int* sx,
                                               int tid)
    {
        cx_step<THREADS, IPT, K, J>(d, x, desc, sd, sx, tid);
        if constexpr (J > 1)
        {
            merge_steps<THREADS, IPT, K, J / 2>::run(d, x, desc, sd, sx, tid);
        }
    }
};

// Phases 2, 4, ..., K of the full sort.
template <int THREADS, int IPT, int K>
struct sort_phases
{
    static __device__ __forceinline__ void run(float (&d)[IPT], int (&x)[IPT], bool desc, float* sd, int* sx,
                                               int tid)
    {
        if constexpr (K > 2)
        {
            sort_phases<THREADS, IPT, K / 2>::run(d, x, desc, sd, sx, tid);
        }
        merge_steps<THREADS, IPT, K, K / 2>::run(d, x, desc, sd, sx, tid);
    }
};

// Phases 2 * KMIN, ..., K of the full sort: what is left to do when the array already consists of
// sorted runs of KMIN elements whose directions are those the phase KMIN would have left (run j
// ascending when j is even, descending when odd; all flipped when `desc`).
template <int THREADS, int IPT, int K, int KMIN>
struct sort_phases_from
{
    static __device__ __forceinline__ void run(float (&d)[IPT], int (&x)[IPT], bool desc, float* sd, int* sx,
                                               int tid)
    {
        if constexpr (K >= 2 * KMIN)
        {
            sort_phases_from<THREADS, IPT, K / 2, KMIN>::run(d, x, desc, sd, sx, tid);
            merge_steps<THREADS, IPT, K, K / 2>::run(d, x, desc, sd, sx, tid);
        }
    }
};

// Sorts the block-wide array (ascending, or descending when `desc`).
template <int THREADS, int IPT>
__device__ __forceinline__ void block_sort(float (&d)[IPT], int (&x)[IPT], bool desc, float* sd, int* sx, int tid)
{
    sort_phases<THREADS, IPT, THREADS * IPT>::run(d, x, desc, sd, sx, tid);
}

// Sorts a block-wide BITONIC array ascending (the last phase of the sort alone).
template <int THREADS, int IPT>
__device__ __forceinline__ void block_merge_bitonic(float (&d)[IPT], int (&x)[IPT], float* sd, int* sx, int tid)
{
    merge_steps<THREADS, IPT, THREADS * IPT, THREADS * IPT / 2>::run(d, x, false, sd, sx, tid);
}

// Folds N unsorted candidates (cd, cx) into the ascending list (ld, lx): sorts the candidates
// descending, keeps the element-wise smaller pair (which leaves the N smallest of the 2N
// as a bitonic array) and sorts that.  Same three moves as the reference's
// shared_buffer::merge (include/bits/topk/singlepass/detail/bits_kernel.cuh:145-199).
template <int THREADS, int IPT>
__device__ __forceinline__ void block_fold(float (&ld)[IPT], int (&lx)[IPT], float (&cd)[IPT], int (&cx)[IPT],
                                           float* sd, int* sx, int tid)
{
    block_sort<THREADS, IPT>(cd, cx, true, sd, sx, tid);
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

} // namespace bitsknn
