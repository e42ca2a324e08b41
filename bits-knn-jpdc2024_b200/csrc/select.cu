// `bits` top-k selection over a precomputed distance matrix (the candidate-list merge of the
// split-row form is in merge.cu).
//
// One thread block scans one row (or one slice of a row).  The row is streamed from HBM by
// 1-D bulk asynchronous copies (TMA engine, no tensor map) into a ring of shared-memory
// stages guarded by mbarriers; the threads read the stages with 128-bit loads, keep only the
// values below the running k-th pair ("radius"), append the survivors to a shared-memory
// candidate buffer by warp-aggregated slot allocation, and fold the buffer into a sorted,
// register-resident list of L = 256 * IPT pairs with bitonic networks when it fills up.
//
// The algorithm is the reference's buffered partial bitonic sort
// (include/bits/topk/singlepass/detail/bits_kernel.cuh:317-408: filter by radius :117-126,
// buffer merge :145-199, overflow loop :383-391); the implementation differs where B200
// wants it to:
//   * bulk-copy ring instead of per-thread 4-byte loads + prefetch.global.L2 (:221-259);
//   * an optimistic pass per stage with ONE barrier (survivors are rare once the radius has
//     settled) that falls back to the reference's barrier-per-batch loop only when the
//     buffer would overflow;
//   * one ballot-free warp scan + one shared atomic per warp instead of one atomic per
//     survivor;
//   * every comparison is on the (distance, index) pair, so the output is the unique
//     lowest-index answer whatever the arrival order of candidates.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "sortnet.cuh"

namespace bitsknn
{

namespace
{

constexpr int SELECT_THREADS = 256;
constexpr int MAX_STAGES = 8;

struct select_params
{
    const float* dist;
    int64_t ld;
    const int32_t* labels;
    int64_t ld_labels;
    const int32_t* label_offsets;
    int32_t label_base; // added to every implicit label (the first column's global index)
    int64_t n;
    int k;
    int splits;       // slices per row (1 = whole rows)
    int64_t slice;    // elements per slice, a multiple of 4
    float* out_dist;  // [rows * splits][k]
    int32_t* out_idx; // [rows * splits][k]
    int raw_pad;      // 1: leave padding as (+inf, PAD_IDX) (candidate lists for a later merge)
    int no_filter;    // 1: never tighten the radius: every value is buffered, sorted and merged (ablation)
    int stage_floats; // floats per stage, a multiple of 4 * SELECT_THREADS
    int stages;
    int merge_at;     // fold the buffer as soon as it holds this many candidates (<= L)
    int* status;
};

struct select_ctrl
{
    int count;  // slow path: allocated slots (may exceed L)
    int inc[3]; // fast path: slots allocated during stage c, in inc[c % 3]
    float r_d;  // radius pair, written by the owner of list element k-1
    int r_x;
};

template <int THREADS, int IPT>
struct select_block
{
    static constexpr int L = THREADS * IPT;

    float ld[IPT]; // the sorted list (ascending), blocked arrangement
    int lx[IPT];
    float r_d; // radius = k-th smallest pair seen so far
    int r_x;
    float* buf_d;
    int* buf_x;
    select_ctrl* ctrl;
    const int32_t* labp; // explicit labels of this slice or nullptr
    int lab0;            // implicit label of slice element 0
    int k;
    bool keep_radius;    // the un-buffered ablation: the filter radius stays at +inf

    __device__ __forceinline__ int label_of(int e) const { return labp != nullptr ? labp[e] : lab0 + e; }

    // Folds the first `valid` buffer entries into the list and refreshes the radius.
    // Entered and left with all threads; leaves the buffer empty (ctrl->count = 0).
    __device__ __forceinline__ void fold(int valid)
    {
        const int tid = threadIdx.x;
        float cd[IPT];
        int cx[IPT];
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int s = r * THREADS + tid;
            const bool in = s < valid;
            cd[r] = in ? buf_d[s] : INFINITY;
            cx[r] = in ? buf_x[s] : PAD_IDX;
        }
        __syncthreads(); // the buffer now doubles as exchange scratch of the networks
        block_fold<THREADS, IPT>(ld, lx, cd, cx, buf_d, buf_x, tid);
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            if (tid * IPT + r == k - 1)
            {
                ctrl->r_d = ld[r];
                ctrl->r_x = lx[r];
            }
        }
        if (tid == 0)
        {
            ctrl->count = 0;
        }
        __syncthreads();
        if (!keep_radius)
        {
            r_d = ctrl->r_d;
            r_x = ctrl->r_x;
        }
    }

    // Evaluates the filter on one 4-vector; returns the number of survivors of this lane.
    __device__ __forceinline__ int filter4(const float4& val, bool live, int e0, float (&dv)[4], int (&lab)[4],
                                           bool (&pr)[4]) const
    {
        dv[0] = val.x;
        dv[1] = val.y;
        dv[2] = val.z;
        dv[3] = val.w;
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            pr[j] = false;
            lab[j] = 0;
            if (live && dv[j] <= r_d)
            {
                lab[j] = label_of(e0 + j);
                pr[j] = pair_lt(dv[j], lab[j], r_d, r_x);
            }
            cnt += pr[j] ? 1 : 0;
        }
        return cnt;
    }

    // Slot offsets of this lane's survivors inside the warp's allocation: one ballot per vector
    // component, no dependent shuffle chain.  Returns the warp's total.
    static __device__ __forceinline__ int warp_slots(const bool (&pr)[4], int (&off)[4])
    {
        const unsigned below = (1U << (threadIdx.x & 31)) - 1U;
        int total = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const unsigned b = __ballot_sync(FULL_MASK, pr[j]);
            off[j] = total + __popc(b & below);
            total += __popc(b);
        }
        return total;
    }

    // Optimistic insertion of one 4-vector (whole warp): survivors beyond the capacity are
    // dropped; the caller detects that from the stage's slot count and redoes the stage.
    __device__ __forceinline__ void insert_fast(const float4& val, bool live, int e0, int count0, int* inc)
    {
        float dv[4];
        int lab[4];
        bool pr[4];
        int off[4];
        filter4(val, live, e0, dv, lab, pr);
        const int total = warp_slots(pr, off);
        if (total == 0)
        {
            return;
        }
        int base = 0;
        if ((threadIdx.x & 31) == 0)
        {
            base = atomicAdd(inc, total);
        }
        base = count0 + __shfl_sync(FULL_MASK, base, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const int pos = base + off[j];
            if (pr[j] && pos < L)
            {
                buf_d[pos] = dv[j];
                buf_x[pos] = lab[j];
            }
        }
    }

    // Optimistic insertion by a single lane (no warp cooperation): used when hits are sparse.
    __device__ __forceinline__ void insert_lane(const float4& val, int e0, int count0, int* inc)
    {
        const float dv[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            if (dv[j] <= r_d)
            {
                const int lab = label_of(e0 + j);
                if (pair_lt(dv[j], lab, r_d, r_x))
                {
                    const int pos = count0 + atomicAdd(inc, 1);
                    if (pos < L)
                    {
                        buf_d[pos] = dv[j];
                        buf_x[pos] = lab;
                    }
                }
            }
        }
    }

    // Guaranteed insertion of one stage: the reference's scheme (bits_kernel.cuh:277-302,
    // 383-391) -- allocate slots for a batch of THREADS*4 values, write those that fit, fold
    // the full buffer and retry the rest.  Returns the number of folds it needed.
    __device__ __forceinline__ int stage_slow(const float4* sv, int nv, int e_base, int count0)
    {
        const int tid = threadIdx.x;
        const int lane = tid & 31;
        int folds = 0;
        if (tid == 0)
        {
            ctrl->count = count0;
        }
        __syncthreads();
        for (int vb = 0; vb < nv; vb += THREADS)
        {
            const int v = vb + tid;
            const bool live = v < nv;
            const float4 val = live ? sv[v] : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
            float dv[4];
            int lab[4];
            bool pr[4];
            filter4(val, live, e_base + 4 * v, dv, lab, pr);
            while (true)
            {
                // allocate slots for what is still pending, write what fits
                int off[4];
                const int total = warp_slots(pr, off);
                int base = 0;
                if (lane == 0 && total > 0)
                {
                    base = atomicAdd(&ctrl->count, total);
                }
                base = __shfl_sync(FULL_MASK, base, 0);
                bool overflow = false;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    if (pr[j])
                    {
                        const int pos = base + off[j];
                        if (pos < L)
                        {
                            buf_d[pos] = dv[j];
                            buf_x[pos] = lab[j];
                            pr[j] = false;
                        }
                        else
                        {
                            overflow = true;
                        }
                    }
                }
                if (__syncthreads_or(overflow ? 1 : 0) == 0)
                {
                    break;
                }
                // the buffer is full: fold it, then offer the rest again under the tighter radius
                // (unlike the reference, which carries every allocated slot over)
                fold(L);
                ++folds;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    pr[j] = pr[j] && pair_lt(dv[j], lab[j], r_d, r_x);
                }
            }
        }
        return folds;
    }
};

template <int THREADS, int IPT, int UNROLL>
__global__ void __launch_bounds__(THREADS) select_kernel(const select_params p)
{
    using block_t = select_block<THREADS, IPT>;
    constexpr int L = block_t::L;
    constexpr int SPARSE_LANES = 6; // up to this many lanes with a candidate: per-lane insertion

    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int CH = p.stage_floats;
    const int NST = p.stages;

    float* stage_base = reinterpret_cast<float*>(smem);
    block_t blk;
    blk.buf_d = stage_base + static_cast<size_t>(NST) * CH;
    blk.buf_x = reinterpret_cast<int*>(blk.buf_d + L);
    uint64_t* bars = reinterpret_cast<uint64_t*>(blk.buf_x + L);
    blk.ctrl = reinterpret_cast<select_ctrl*>(bars + MAX_STAGES);
    blk.k = p.k;
    blk.keep_radius = p.no_filter != 0;

    // which slice of which row
    const int64_t vrow = blockIdx.x;
    const int64_t row = vrow / p.splits;
    const int64_t begin = (vrow - row * p.splits) * p.slice;
    int64_t m64 = (p.n < begin + p.slice ? p.n : begin + p.slice) - begin;
    const int m = m64 > 0 ? static_cast<int>(m64) : 0;
    const float* rowp = p.dist + row * p.ld + begin;
    blk.labp = p.labels != nullptr ? p.labels + row * p.ld_labels + begin : nullptr;
    blk.lab0 = static_cast<int>(begin) + p.label_base + (p.label_offsets != nullptr ? p.label_offsets[row] : 0);

    // [0,h): scalar head up to the first 16-byte boundary, [h,h+mid): streamed, then a tail < 4
    int h = static_cast<int>(((16U - (reinterpret_cast<uintptr_t>(rowp) & 15U)) & 15U) >> 2);
    h = h < m ? h : m;
    const int mid = ((m - h) >> 2) << 2;
    const int tail = m - h - mid;
    const int nchunks = (mid + CH - 1) / CH;

#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        blk.ld[r] = INFINITY;
        blk.lx[r] = PAD_IDX;
    }
    blk.r_d = INFINITY;
    blk.r_x = PAD_IDX;

    auto issue = [&](int c, int st) {
        const int floats = (mid - c * CH) < CH ? (mid - c * CH) : CH;
        ptx::mbar_expect_tx(&bars[st], static_cast<uint32_t>(floats) * 4U);
        ptx::bulk_g2s(stage_base + static_cast<size_t>(st) * CH, rowp + h + static_cast<int64_t>(c) * CH,
                      static_cast<uint32_t>(floats) * 4U, &bars[st]);
    };

    if (tid == 0)
    {
        for (int s = 0; s < NST; ++s)
        {
            ptx::mbar_init(&bars[s], 1);
        }
        blk.ctrl->count = 0;
        blk.ctrl->inc[0] = 0;
        blk.ctrl->inc[1] = 0;
        blk.ctrl->inc[2] = 0;
        ptx::mbar_init_fence();
    }
    __syncthreads();
    if (tid == 0)
    {
        for (int c = 0; c < NST && c < nchunks; ++c)
        {
            issue(c, c);
        }
    }

    // head and tail elements go straight into the buffer (at most 6 of them)
    if (tid < h + tail)
    {
        const int e = tid < h ? tid : mid + tid;
        const float d = rowp[e];
        const int lab = blk.label_of(e);
        if (pair_lt(d, lab, blk.r_d, blk.r_x))
        {
            const int pos = atomicAdd(&blk.ctrl->count, 1);
            blk.buf_d[pos] = d;
            blk.buf_x[pos] = lab;
        }
    }
    __syncthreads();
    int count0 = blk.ctrl->count; // candidates in the buffer; identical in every thread
    bool go_slow = true;          // the first stage always overflows (radius = +inf)
    bool timed_out = false;
    int c = 0;

    int st = 0;          // stage of chunk c            (c % NST without a division)
    uint32_t phase = 0;  // parity of that stage's use  ((c / NST) & 1)
    int i3 = 0;          // c % 3

    for (; c < nchunks; ++c)
    {
        const float4* sv = reinterpret_cast<const float4*>(stage_base + static_cast<size_t>(st) * CH);
        const int floats = (mid - c * CH) < CH ? (mid - c * CH) : CH;
        const int nv = floats >> 2;
        const int e_base = h + c * CH;
        int* inc = &blk.ctrl->inc[i3];

        if (!ptx::mbar_wait_bounded(&bars[st], phase))
        {
            timed_out = true;
        }

        bool redo = go_slow;
        if (!go_slow)
        {
            int vb = 0;
            // groups of UNROLL vectors per thread, no bounds checks; one vote per group
            for (; vb + THREADS * UNROLL <= nv; vb += THREADS * UNROLL)
            {
                float4 val[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                {
                    val[u] = sv[vb + u * THREADS + tid];
                }
                float mn[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                {
                    mn[u] = fminf(fminf(val[u].x, val[u].y), fminf(val[u].z, val[u].w));
                }
                float mall = mn[0];
#pragma unroll
                for (int u = 1; u < UNROLL; ++u)
                {
                    mall = fminf(mall, mn[u]);
                }
                const unsigned hitters = __ballot_sync(FULL_MASK, mall <= blk.r_d);
                if (hitters == 0)
                {
                    continue;
                }
                if (__popc(hitters) <= SPARSE_LANES)
                {
                    // few lanes saw a candidate: they take slots one by one, the others idle
                    if (mall <= blk.r_d)
                    {
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u)
                        {
                            if (mn[u] <= blk.r_d)
                            {
                                blk.insert_lane(val[u], e_base + 4 * (vb + u * THREADS + tid), count0, inc);
                            }
                        }
                    }
                }
                else
                {
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u)
                    {
                        const bool hit = mn[u] <= blk.r_d;
                        if (__any_sync(FULL_MASK, hit))
                        {
                            blk.insert_fast(val[u], hit, e_base + 4 * (vb + u * THREADS + tid), count0, inc);
                        }
                    }
                }
            }
            // ragged end of the last stage
            for (; vb < nv; vb += THREADS)
            {
                const int v = vb + tid;
                const bool live = v < nv;
                const float4 val = live ? sv[v] : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
                const bool hit = live && fminf(fminf(val.x, val.y), fminf(val.z, val.w)) <= blk.r_d;
                if (__any_sync(FULL_MASK, hit))
                {
                    blk.insert_fast(val, hit, e_base + 4 * v, count0, inc);
                }
            }
        }
        // one barrier per stage: every thread is done reading the stage and adding to `inc`
        if (__syncthreads_or(timed_out ? 1 : 0) != 0)
        {
            timed_out = true;
            break;
        }
        if (!go_slow)
        {
            const int added = *inc;
            if (count0 + added > L)
            {
                redo = true; // some survivors were dropped: forget this pass, redo the stage
            }
            else
            {
                count0 += added;
            }
        }
        if (tid == 0)
        {
            blk.ctrl->inc[i3 == 0 ? 2 : i3 - 1] = 0; // slot of stage c+2: last read before this barrier
        }
        if (redo)
        {
            const int folds = blk.stage_slow(sv, nv, e_base, count0);
            count0 = blk.ctrl->count;
            go_slow = folds > 1;
        }
        if (count0 >= p.merge_at)
        {
            blk.fold(count0);
            count0 = 0;
        }
        // every thread has passed a barrier after its last read of this stage
        if (tid == 0 && c + NST < nchunks)
        {
            issue(c + NST, st);
        }
        i3 = i3 == 2 ? 0 : i3 + 1;
        if (++st == NST)
        {
            st = 0;
            phase ^= 1U;
        }
    }

    if (timed_out)
    {
        // report, let the copies still in flight land (bounded), and leave
        for (int cc = c + 1; cc < nchunks && cc < c + NST; ++cc)
        {
            ptx::mbar_wait_bounded(&bars[cc % NST], static_cast<uint32_t>((cc / NST) & 1), 1U << 16);
        }
        if (tid == 0)
        {
            atomicOr(p.status, DEVICE_STATUS_TIMEOUT);
        }
        return;
    }

    if (count0 > 0)
    {
        blk.fold(count0);
    }

    float* od = p.out_dist + vrow * p.k;
    int32_t* ox = p.out_idx + vrow * p.k;
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        const int e = tid * IPT + r;
        if (e < p.k)
        {
            int x = blk.lx[r];
            if (p.raw_pad == 0 && x == PAD_IDX)
            {
                x = e; // the reference pads short rows with (+inf, position): bits_kernel.cuh:340-358
            }
            od[e] = blk.ld[r];
            ox[e] = x;
        }
    }
}

size_t select_smem_bytes(int L, int stage_floats, int stages)
{
    return static_cast<size_t>(stages) * stage_floats * 4 + static_cast<size_t>(L) * 8 + MAX_STAGES * 8 +
           sizeof(select_ctrl);
}

template <int THREADS, int IPT>
int launch_select(select_params p, int64_t vrows, cudaStream_t stream)
{
    constexpr int L = THREADS * IPT;
    // 0 = automatic: half-full buffers for lists of up to 256 pairs, three-quarter-full ones for
    // longer lists, whose folds cost more against what an earlier tightening of the radius saves
    int merge_pct = tuning_value("select.merge_at", 0);
    if (merge_pct <= 0)
    {
        merge_pct = L <= 256 ? 50 : 75;
    }
    p.merge_at = std::max(1, (L * merge_pct) / 100);
    // a stage is a whole number of 4-vectors per thread
    p.stage_floats = std::max(4 * THREADS, (p.stage_floats / (4 * THREADS)) * (4 * THREADS));
    const size_t smem = select_smem_bytes(L, p.stage_floats, p.stages);
    // 128-bit vectors per thread examined under one warp vote
    // (0 = automatic: 2, which measured a little ahead of 4 for every block size: 0.83 ms against
    // 0.85 at k = 512, 1.70 against 1.74 at k = 2048, no register spills at 4 blocks per SM for k <= 256)
    int unroll = tuning_value("select.unroll", 0);
    unroll = unroll != 0 ? unroll : 2;
    auto kernel = unroll == 2 ? select_kernel<THREADS, IPT, 2> : select_kernel<THREADS, IPT, 4>;
    if (smem > 227U * 1024U)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT,
                    "select.stage_bytes x select.stages = %d x %d needs %zu bytes of shared memory per block; "
                    "the limit is %u", p.stage_floats * 4, p.stages, smem, 227U * 1024U);
    }
    BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    {
        kernel_scope timed{"select_kernel", stream};
        kernel<<<static_cast<unsigned>(vrows), THREADS, smem, stream>>>(p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

int dispatch_select(const select_params& p, int64_t vrows, cudaStream_t stream)
{
    // smallest list that holds k: the reference's dynamic_switch_le over K
    // (src/topk/singlepass/bits_knn.cu:44), with the list never shorter than the block
    // Long lists take larger blocks (the reference's tuned shapes use 512 threads for k = 2048,
    // scripts/optima.csv:1282): more threads fold a list of the same length with fewer pairs, and
    // registers, per thread.
    const int wide = tuning_value("select.wide_block", 1);
    if (p.k <= 256)
    {
        return launch_select<256, 1>(p, vrows, stream);
    }
    if (p.k <= 512)
    {
        return wide != 0 ? launch_select<512, 1>(p, vrows, stream) : launch_select<256, 2>(p, vrows, stream);
    }
    if (p.k <= 1024)
    {
        return wide != 0 ? launch_select<512, 2>(p, vrows, stream) : launch_select<256, 4>(p, vrows, stream);
    }
    // the longest lists: 1024 threads with two pairs each (measured against 512 x 4 at q = 1024,
    // n = 2^20, k = 2048: 1.74 ms against 2.00 on uniform rows, 4.5 against 5.5 per 128 descending rows;
    // at k = 1024 the 512-thread block stays ahead on uniform rows, 1.09 ms against 1.25)
    return wide != 0 ? launch_select<1024, 2>(p, vrows, stream) : launch_select<256, 8>(p, vrows, stream);
}

int dispatch_merge(const float* cd, const int32_t* cx, int64_t list_stride, int64_t query_stride, int64_t q, int lists,
                   int k, float* od, int32_t* ox, cudaStream_t stream)
{
    // the slices' lists arrive ascending
    return merge_lists(cd, cx, list_stride, query_stride, q, lists, k, k, nullptr, od, ox, merge_input::sorted, stream);
}

} // namespace

namespace
{

int check_select_args(const float* d_dist, int64_t ld, int64_t q, int64_t n, int k, const float* od, const int32_t* ox)
{
    if (d_dist == nullptr || od == nullptr || ox == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (q < 0 || n <= 0 || ld < n)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: q=%lld n=%lld ld=%lld", static_cast<long long>(q),
                    static_cast<long long>(n), static_cast<long long>(ld));
    }
    if (n >= std::numeric_limits<int32_t>::max() - 4 || q > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "row length or row count beyond int32 labels");
    }
    if (k < 1 || k > BITSKNN_MAX_K)
    {
        // same wording as the reference's dispatcher (src/topk/singlepass/bits_knn.cu:52-55)
        return fail(BITSKNN_ERR_UNSUPPORTED_K, "Unsupported k value: %d", k);
    }
    if ((reinterpret_cast<uintptr_t>(d_dist) & 3U) != 0)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "distance matrix is not 4-byte aligned");
    }
    return BITSKNN_OK;
}

void fill_stream_config(select_params& p)
{
    // 0 = automatic: the shapes measured best on B200 -- 3 x 16 KiB for 256-thread blocks
    // (4 blocks per SM), 3 x 32 KiB for 512-thread blocks, 2 x 64 KiB for the longest lists
    int stage_bytes = tuning_value("select.stage_bytes", 0);
    int stages = tuning_value("select.stages", 0);
    const bool wide = p.k > 256 && tuning_value("select.wide_block", 1) != 0;
    if (stage_bytes <= 0)
    {
        stage_bytes = !wide ? 16384 : (p.k > 1024 ? 65536 : 32768);
    }
    if (stages <= 0)
    {
        stages = wide && p.k > 1024 ? 2 : 3;
    }
    stage_bytes = std::max((stage_bytes / 4096) * 4096, 4096);
    p.stage_floats = stage_bytes / 4;
    p.stages = std::min(std::max(stages, 2), MAX_STAGES);
}

} // namespace

} // namespace bitsknn

using namespace bitsknn;

namespace bitsknn
{

int select_rows(const float* d_dist, int64_t ld, const int32_t* d_labels, int64_t ld_labels,
                const int32_t* d_label_offsets, int32_t label_base, int64_t q, int64_t n, int k, float* d_out_dist,
                int32_t* d_out_idx, cudaStream_t stream)
{
    if (const int rc = check_select_args(d_dist, ld, q, n, k, d_out_dist, d_out_idx); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (d_labels != nullptr && ld_labels < n)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "label matrix stride %lld shorter than n", static_cast<long long>(ld_labels));
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    select_params p{};
    p.dist = d_dist;
    p.ld = ld;
    p.labels = d_labels;
    p.ld_labels = ld_labels;
    p.label_offsets = d_label_offsets;
    p.label_base = label_base;
    p.n = n;
    p.k = k;
    p.splits = 1;
    p.slice = (n + 3) & ~static_cast<int64_t>(3);
    p.out_dist = d_out_dist;
    p.out_idx = d_out_idx;
    p.raw_pad = 0;
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    // "select.filter" = 0 turns the radius filter off: the un-buffered partial bitonic sort the
    // reference keeps as an ablation (partial-bitonic-regs, src/topk/singlepass/partial_bitonic.cu:217-294)
    p.no_filter = tuning_value("select.filter", 1) == 0 ? 1 : 0;
    fill_stream_config(p);
    return dispatch_select(p, q, stream);
}

} // namespace bitsknn

extern "C" int bitsknn_select(const float* d_dist, int64_t ld, const int32_t* d_labels, int64_t ld_labels,
                              const int32_t* d_label_offsets, int64_t q, int64_t n, int k, float* d_out_dist,
                              int32_t* d_out_idx, bitsknn_stream_t stream)
{
    return select_rows(d_dist, ld, d_labels, ld_labels, d_label_offsets, 0, q, n, k, d_out_dist, d_out_idx,
                       static_cast<cudaStream_t>(stream));
}

namespace
{

int resolve_splits(int64_t q, int64_t n, int k, int splits)
{
    if (splits > 0)
    {
        return splits;
    }
    // Blocks the device wants in flight, measured on B200 for q = 1 ... 4096 at 4 GiB: short lists
    // run 4 blocks of 256 threads per SM, the longest one block of 512 threads; more slices than
    // that only add warm-up (every slice finds its own radius) and merge work.
    const int sms = device_sm_count();
    const int64_t want = static_cast<int64_t>(sms) * (k <= 64 ? 600 : (k <= 256 ? 400 : (k <= 1024 ? 200 : 130))) / 148;
    int64_t s = (want + q / 2) / std::max<int64_t>(q, 1);
    // a slice should be long against the list it has to fill
    const int64_t list = k <= 256 ? 256 : (k <= 512 ? 512 : (k <= 1024 ? 1024 : 2048));
    s = std::min(s, std::max<int64_t>(1, n / (32 * list)));
    s = std::min<int64_t>(std::max<int64_t>(s, 1), 64);
    s = std::min<int64_t>(s, std::max(1, 65536 / k)); // the merge pass takes at most 65536 candidates per query
    return static_cast<int>(s);
}

} // namespace

extern "C" int bitsknn_select_auto_splits(int64_t q, int64_t n, int k)
{
    if (q <= 0 || n <= 0 || k <= 0 || k > BITSKNN_MAX_K)
    {
        return 1;
    }
    return resolve_splits(q, n, k, 0);
}

extern "C" size_t bitsknn_select_split_workspace_bytes(int64_t q, int k, int splits)
{
    if (q <= 0 || k <= 0)
    {
        return 0;
    }
    const int s = splits > 0 ? splits : 64; // upper bound of the automatic choice
    return static_cast<size_t>(q) * static_cast<size_t>(s) * static_cast<size_t>(k) * 8U;
}

extern "C" int bitsknn_select_split(const float* d_dist, int64_t ld, const int32_t* d_label_offsets, int64_t q,
                                    int64_t n, int k, int splits, void* d_workspace, size_t workspace_bytes,
                                    float* d_out_dist, int32_t* d_out_idx, bitsknn_stream_t stream)
{
    if (const int rc = check_select_args(d_dist, ld, q, n, k, d_out_dist, d_out_idx); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (splits < 0 || splits > 4096)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid number of slices per row: %d", splits);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    const int s = resolve_splits(q, n, k, splits);
    if (static_cast<int64_t>(s) * k > 65536)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "slices * k = %lld exceeds 65536", static_cast<long long>(s) * k);
    }
    if (q * s > 0x7fffffffLL)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "q * slices = %lld row slices exceed the grid limit of 2^31 - 1",
                    static_cast<long long>(q) * s);
    }
    const size_t need = static_cast<size_t>(q) * s * k * 8U;
    if (d_workspace == nullptr || workspace_bytes < need)
    {
        return fail(BITSKNN_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    }
    auto* cand_dist = static_cast<float*>(d_workspace);
    auto* cand_idx = reinterpret_cast<int32_t*>(cand_dist + static_cast<size_t>(q) * s * k);

    select_params p{};
    p.dist = d_dist;
    p.ld = ld;
    p.labels = nullptr;
    p.ld_labels = 0;
    p.label_offsets = d_label_offsets;
    p.n = n;
    p.k = k;
    p.splits = s;
    p.slice = (((n + s - 1) / s) + 3) & ~static_cast<int64_t>(3);
    p.out_dist = cand_dist;
    p.out_idx = cand_idx;
    p.raw_pad = 1;
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    fill_stream_config(p);
    auto cs = static_cast<cudaStream_t>(stream);
    if (const int rc = dispatch_select(p, q * s, cs); rc != BITSKNN_OK)
    {
        return rc;
    }
    return dispatch_merge(cand_dist, cand_idx, k, static_cast<int64_t>(s) * k, q, s, k, d_out_dist, d_out_idx, cs);
}

// ---------------------------------------------------------------------------------------
// Split-row selection for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a search:
// a plug-in running inside an engine that reserved the whole device for its own pool, code
// between two latency-critical launches where an allocation would serialise the device, or
// a process whose memory budget was fixed at start-up.  For them the candidate lists of the
// two-pass scheme live in a file-scope device array of fixed size that is part of the loaded
// library image (each GPU that loads the library holds these bytes until the process exits).
//
// In host code `g_static_candidates` is only a host-side handle of the symbol, NOT a device
// address: handing it to a kernel would fault or, on systems where the GPU can reach host
// memory, silently read and write the wrong bytes.  The device address is looked up once per
// device with cudaGetSymbolAddress while that device is current, and that pointer is what
// the kernels get.
constexpr size_t STATIC_CANDIDATE_BYTES = static_cast<size_t>(BITSKNN_STATIC_SCRATCH_BYTES);
static __device__ __align__(256) unsigned char g_static_candidates[STATIC_CANDIDATE_BYTES];

namespace
{

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
void* g_static_ptr[MAX_DEVICES] = {};

// Device address of the static candidate array on the current device (looked up on the first
// call per device; that first call should therefore happen outside any stream capture).
int static_candidates(void** out)
{
    int device = 0;
    BITSKNN_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= MAX_DEVICES)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "device ordinal %d beyond the %d supported", device, MAX_DEVICES);
    }
    std::lock_guard<std::mutex> lock{g_static_mutex};
    if (g_static_ptr[device] == nullptr)
    {
        void* ptr = nullptr;
        BITSKNN_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_candidates));
        g_static_ptr[device] = ptr;
    }
    *out = g_static_ptr[device];
    return BITSKNN_OK;
}

} // namespace

extern "C" int bitsknn_select_split_static(const float* d_dist, int64_t ld, const int32_t* d_label_offsets,
                                           int64_t q, int64_t n, int k, int splits, float* d_out_dist,
                                           int32_t* d_out_idx, bitsknn_stream_t stream)
{
    if (const int rc = check_select_args(d_dist, ld, q, n, k, d_out_dist, d_out_idx); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (splits < 1 || splits > 4096)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid number of slices per row: %d", splits);
    }
    if (static_cast<int64_t>(splits) * k > 65536)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "slices * k = %lld exceeds 65536", static_cast<long long>(splits) * k);
    }
    const size_t need = static_cast<size_t>(q) * static_cast<size_t>(splits) * static_cast<size_t>(k) * 8U;
    if (need > STATIC_CANDIDATE_BYTES)
    {
        return fail(BITSKNN_ERR_WORKSPACE,
                    "q * splits * k = %lld candidate pairs need %zu bytes; the built-in scratch holds %zu bytes "
                    "(use bitsknn_select_split with your own workspace for larger problems)",
                    static_cast<long long>(q) * splits * k, need, STATIC_CANDIDATE_BYTES);
    }
    if (q == 0)
    {
        return BITSKNN_OK;
    }
    void* scratch = nullptr;
    if (const int rc = static_candidates(&scratch); rc != BITSKNN_OK)
    {
        return rc;
    }
    // pass 1 overwrites every candidate slot that pass 2 reads (each block stores all k pairs of
    // its slice, padding included), so nothing in the array has to be cleared between calls
    auto* cand_dist = static_cast<float*>(scratch);
    auto* cand_idx = reinterpret_cast<int32_t*>(cand_dist + static_cast<size_t>(q) * splits * k);

    select_params p{};
    p.dist = d_dist;
    p.ld = ld;
    p.labels = nullptr;
    p.ld_labels = 0;
    p.label_offsets = d_label_offsets;
    p.n = n;
    p.k = k;
    p.splits = splits;
    p.slice = (((n + splits - 1) / splits) + 3) & ~static_cast<int64_t>(3);
    p.out_dist = cand_dist;
    p.out_idx = cand_idx;
    p.raw_pad = 1;
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    fill_stream_config(p);
    auto cs = static_cast<cudaStream_t>(stream);
    if (const int rc = dispatch_select(p, q * splits, cs); rc != BITSKNN_OK)
    {
        return rc;
    }
    return dispatch_merge(cand_dist, cand_idx, k, static_cast<int64_t>(splits) * k, q, splits, k, d_out_dist,
                          d_out_idx, cs);
}
