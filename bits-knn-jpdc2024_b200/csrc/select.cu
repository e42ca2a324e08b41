// `bits` top-k selection over a precomputed distance matrix (the candidate-list merge of the
// split-row form is in merge.cu).
//
// One thread block scans one row (or one slice of a row).  The row is streamed from HBM by
// 1-D bulk asynchronous copies (TMA engine, no tensor map) into a ring of shared-memory
// stages guarded by mbarriers; the threads read the stages with 128-bit loads, keep only the
// values below the running k-th pair ("radius"), append the survivors to a shared-memory
// candidate buffer by warp-aggregated slot allocation, and fold the buffer into a sorted,
// register-resident list of L = THREADS * IPT pairs with bitonic networks when it fills up.
//
// The algorithm is the reference's buffered partial bitonic sort
// (include/bits/topk/singlepass/detail/bits_kernel.cuh:317-408: filter by radius :117-126,
// buffer merge :145-199, overflow loop :383-391); the implementation differs where B200
// wants it to:
//   * bulk-copy ring instead of per-thread 4-byte loads + prefetch.global.L2 (:221-259);
//   * an optimistic pass per stage with ONE barrier (survivors are rare once the radius has
//     settled), redone only when the buffer (2 L slots) would overflow;
//   * a DENSE stage -- more survivors than the buffer has room for: the first stage of a row, or
//     rows that arrive in descending order, where every value passes the filter -- is not pushed
//     through the buffer batch by batch (the reference sorts and merges every buffered value,
//     :145-199, 383-391, which makes its adversarial case seven times slower than its random
//     case).  The stage already sits in shared memory, so it is cut down first: a sorted sample
//     of L of its values proposes a pivot with at least L and at most `room` survivors at or
//     below it; only those enter the buffer and are sorted and merged -- everything above the
//     pivot cannot be among the L smallest.  The reference's batch loop stays as the last resort;
//   * warp ballots + one shared atomic per warp instead of one atomic per survivor;
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
#include "tuning_table.cuh"

namespace bitsknn
{

namespace
{

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
    int stage_floats; // floats per stage, a multiple of 4 * THREADS
    int stages;
    int merge_at;     // fold the buffer as soon as it holds this many candidates (<= L; < 2 L for folds by selection)
    int* status;
};

struct select_ctrl
{
    int count;         // guaranteed path / head and tail / after a fold: entries in the buffer
    int inc[3];        // optimistic path: slots allocated during stage c, in inc[c % 3]
    int warp_sums[32]; // block-wide counts
    float r_d;         // radius pair, written by the owner of list element k-1 (fold) or the pivot (plan)
    int r_x;
    int dense;         // plan: the stage was dense
    // fold by selection (long lists): range of keys that holds the k-th, counters
    unsigned long long key_lo;
    unsigned long long key_hi;
    int sel_bin;       // bucket that holds the wanted rank
    int sel_before;    // keys in the buckets before it
    int sel_count;     // keys in it
    int sel_real;      // real (non-padding) keys
    int sel_kept;      // survivors written so far
    int sel_ties;      // keys equal to the pivot taken so far
};

// What a block knows about its row besides the list: passed by value to the out-of-line parts.
struct row_ctx
{
    float* buf_d; // candidate buffer, 2 L slots
    int* buf_x;
    select_ctrl* ctrl;
    const int32_t* labp; // explicit labels of this slice or nullptr
    int lab0;            // implicit label of slice element 0
    int k;
    float r_d; // radius = k-th smallest pair seen so far
    int r_x;
    bool keep_radius; // the un-buffered ablation: the filter radius stays at +inf
};

__device__ __forceinline__ int label_of(const row_ctx& s, int e) { return s.labp != nullptr ? s.labp[e] : s.lab0 + e; }

// Evaluates the filter on one 4-vector; returns the number of survivors of this lane.
__device__ __forceinline__ int filter4(const row_ctx& s, const float4& val, bool live, int e0, float (&dv)[4],
                                       int (&lab)[4], bool (&pr)[4])
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
        if (live && dv[j] <= s.r_d)
        {
            lab[j] = label_of(s, e0 + j);
            pr[j] = pair_lt(dv[j], lab[j], s.r_d, s.r_x);
        }
        cnt += pr[j] ? 1 : 0;
    }
    return cnt;
}

// Slot offsets of this lane's survivors inside the warp's allocation: one ballot per vector
// component, no dependent shuffle chain.  Returns the warp's total.
__device__ __forceinline__ int warp_slots(const bool (&pr)[4], int (&off)[4])
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

// Optimistic insertion of one 4-vector (whole warp): survivors beyond the capacity `cap` are
// dropped; the caller detects that from the stage's slot count and redoes the stage.
__device__ __forceinline__ void insert_fast(const row_ctx& s, int cap, const float4& val, bool live, int e0, int count0,
                                            int* inc)
{
    float dv[4];
    int lab[4];
    bool pr[4];
    int off[4];
    filter4(s, val, live, e0, dv, lab, pr);
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
        if (pr[j] && pos < cap)
        {
            s.buf_d[pos] = dv[j];
            s.buf_x[pos] = lab[j];
        }
    }
}

// Optimistic insertion by a single lane (no warp cooperation): used when hits are sparse.
__device__ __forceinline__ void insert_lane(const row_ctx& s, int cap, const float4& val, int e0, int count0, int* inc)
{
    const float dv[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        if (dv[j] <= s.r_d)
        {
            const int lab = label_of(s, e0 + j);
            if (pair_lt(dv[j], lab, s.r_d, s.r_x))
            {
                const int pos = count0 + atomicAdd(inc, 1);
                if (pos < cap)
                {
                    s.buf_d[pos] = dv[j];
                    s.buf_x[pos] = lab;
                }
            }
        }
    }
}

// One pass over a stage with the current radius: every survivor takes a slot of `inc`
// (optimistic: slots beyond the capacity are dropped).  UNROLL vectors per thread are examined
// under one warp vote.
template <int THREADS, int UNROLL>
__device__ __forceinline__ void scan_stage(const row_ctx& s, int cap, const float4* sv, int nv, int e_base, int count0,
                                           int* inc)
{
    constexpr int SPARSE_LANES = 6; // up to this many lanes with a candidate: per-lane insertion
    const int tid = threadIdx.x;
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
        const unsigned hitters = __ballot_sync(FULL_MASK, mall <= s.r_d);
        if (hitters == 0)
        {
            continue;
        }
        if (__popc(hitters) <= SPARSE_LANES)
        {
            // few lanes saw a candidate: they take slots one by one, the others idle
            if (mall <= s.r_d)
            {
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                {
                    if (mn[u] <= s.r_d)
                    {
                        insert_lane(s, cap, val[u], e_base + 4 * (vb + u * THREADS + tid), count0, inc);
                    }
                }
            }
        }
        else
        {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
            {
                const bool hit = mn[u] <= s.r_d;
                if (__any_sync(FULL_MASK, hit))
                {
                    insert_fast(s, cap, val[u], hit, e_base + 4 * (vb + u * THREADS + tid), count0, inc);
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
        const bool hit = live && fminf(fminf(val.x, val.y), fminf(val.z, val.w)) <= s.r_d;
        if (__any_sync(FULL_MASK, hit))
        {
            insert_fast(s, cap, val, hit, e_base + 4 * v, count0, inc);
        }
    }
}

// ---- the parts that run a few times per row ---------------------------------------------------

// The pair order as one unsigned 64-bit key: distance (sign-magnitude floats made monotone; the
// two zeros coincide, as they do under <) above the label (signed order).
__device__ __forceinline__ unsigned long long pair_key(float d, int x)
{
    uint32_t u = __float_as_uint(d + 0.0F);
    u = (u & 0x80000000U) != 0 ? ~u : (u | 0x80000000U);
    return (static_cast<unsigned long long>(u) << 32) | (static_cast<uint32_t>(x) ^ 0x80000000U);
}

constexpr unsigned long long PAD_KEY = 0xFF800000FFFFFFFFULL; // key of the padding pair (+inf, PAD_IDX)

// Fold for long lists (L >= 1024): the list is kept as an UNSORTED set of the k smallest pairs and a
// fold is a selection, not a sort -- the k-th smallest key of list + buffer is found by bucketing
// (256 buckets over the range that still holds it, narrowed level by level, then a ranking of the
// last 32 or fewer keys inside one warp), everything below it is compacted into the list and the
// pivot is the new radius.  A fold of a 2048-pair list is about a tenth of the instructions of the
// sorting networks (77 compare-exchange steps, 20 of them through shared memory); the list is
// sorted once, when the row ends.  Takes the whole buffer; returns 0 (nothing stays buffered).
template <int THREADS, int IPT>
__device__ __forceinline__ int fold_select(float (&ld)[IPT], int (&lx)[IPT], row_ctx s, int valid)
{
    constexpr int E = 3 * IPT; // pairs a thread holds: its share of the list and of the 2 L buffer slots
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    select_ctrl* ctrl = s.ctrl;
    float pd[E];
    int px[E];
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        pd[r] = ld[r];
        px[r] = lx[r];
    }
#pragma unroll
    for (int r = 0; r < 2 * IPT; ++r)
    {
        const int e = r * THREADS + tid;
        const bool in = e < valid;
        pd[IPT + r] = in ? s.buf_d[e] : INFINITY;
        px[IPT + r] = in ? s.buf_x[e] : PAD_IDX;
    }
    // range and number of the real keys
    unsigned long long kmin = PAD_KEY;
    unsigned long long kmax = 0;
    int real = 0;
#pragma unroll
    for (int i = 0; i < E; ++i)
    {
        const unsigned long long key = pair_key(pd[i], px[i]);
        if (key != PAD_KEY)
        {
            kmin = key < kmin ? key : kmin;
            kmax = key > kmax ? key : kmax;
            ++real;
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
    {
        const unsigned long long a = __shfl_xor_sync(FULL_MASK, kmin, o);
        const unsigned long long b = __shfl_xor_sync(FULL_MASK, kmax, o);
        kmin = a < kmin ? a : kmin;
        kmax = b > kmax ? b : kmax;
        real += __shfl_xor_sync(FULL_MASK, real, o);
    }
    if (tid == 0)
    {
        ctrl->key_lo = PAD_KEY;
        ctrl->key_hi = 0;
        ctrl->sel_real = 0;
        ctrl->sel_kept = 0;
        ctrl->sel_ties = 0;
    }
    __syncthreads(); // every thread holds its buffer entries: the buffer is scratch from here on
    uint32_t* hist = reinterpret_cast<uint32_t*>(s.buf_d);                           // 256 buckets
    unsigned long long* last = reinterpret_cast<unsigned long long*>(s.buf_d + 256); // the last <= 32 keys
    if (lane == 0 && real > 0)
    {
        atomicMin(&ctrl->key_lo, kmin);
        atomicMax(&ctrl->key_hi, kmax);
        atomicAdd(&ctrl->sel_real, real);
    }
    __syncthreads();
    const int total_real = ctrl->sel_real;
    const int k = s.k;
    unsigned long long pivot = PAD_KEY; // keys below the pivot stay, and `ties` keys equal to it
    int ties = 0;
    if (total_real >= k)
    {
        unsigned long long lo = ctrl->key_lo;
        unsigned long long hi = ctrl->key_hi;
        int want = k; // rank (1-based) of the pivot among the keys in [lo, hi]
        while (true)
        {
            const unsigned long long range = hi - lo;
            const int shift = range < 256ULL ? 0 : (64 - __clzll(static_cast<long long>(range))) - 8;
            if (tid < 256)
            {
                hist[tid] = 0;
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < E; ++i)
            {
                const unsigned long long key = pair_key(pd[i], px[i]);
                if (key >= lo && key <= hi)
                {
                    atomicAdd(&hist[static_cast<uint32_t>((key - lo) >> shift)], 1U);
                }
            }
            __syncthreads();
            if (tid < 32)
            {
                // lane l sums buckets 8 l .. 8 l + 7; the bucket in which the running count reaches `want`
                uint32_t h[8];
                uint32_t sum = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    h[j] = hist[lane * 8 + j];
                    sum += h[j];
                }
                uint32_t incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1)
                {
                    const uint32_t t = __shfl_up_sync(FULL_MASK, incl, o);
                    incl += lane >= o ? t : 0U;
                }
                uint32_t before = incl - sum;
                if (before < static_cast<uint32_t>(want) && static_cast<uint32_t>(want) <= incl)
                {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                    {
                        if (before < static_cast<uint32_t>(want) && static_cast<uint32_t>(want) <= before + h[j])
                        {
                            ctrl->sel_bin = lane * 8 + j;
                            ctrl->sel_before = static_cast<int>(before);
                            ctrl->sel_count = static_cast<int>(h[j]);
                        }
                        before += h[j];
                    }
                }
            }
            __syncthreads();
            const int bin = ctrl->sel_bin;
            const int count = ctrl->sel_count;
            want -= ctrl->sel_before;
            lo += static_cast<unsigned long long>(bin) << shift;
            const unsigned long long top = lo + ((1ULL << shift) - 1ULL); // (wraps when the bucket reaches the top)
            hi = top >= lo && top < hi ? top : hi;
            if (shift == 0)
            {
                // one key value per bucket: it is the pivot, `want` of its copies stay
                pivot = lo;
                ties = want;
                break;
            }
            if (count <= 32)
            {
                // rank the bucket's keys inside one warp
                if (tid == 0)
                {
                    ctrl->sel_count = 0;
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < E; ++i)
                {
                    const unsigned long long key = pair_key(pd[i], px[i]);
                    if (key >= lo && key <= hi)
                    {
                        last[atomicAdd(&ctrl->sel_count, 1)] = key;
                    }
                }
                __syncthreads();
                if (tid < 32)
                {
                    const unsigned long long mine = lane < count ? last[lane] : PAD_KEY;
                    int less = 0;
                    int same = 0;
                    for (int j = 0; j < count; ++j)
                    {
                        const unsigned long long other = __shfl_sync(FULL_MASK, mine, j);
                        less += other < mine ? 1 : 0;
                        same += other == mine ? 1 : 0;
                    }
                    if (lane < count && less < want && want <= less + same)
                    {
                        // (copies of one key all get here and write the same words)
                        ctrl->key_lo = mine;
                        ctrl->sel_before = want - less;
                    }
                }
                __syncthreads();
                pivot = ctrl->key_lo;
                ties = ctrl->sel_before;
                break;
            }
            // (the barrier after the scan also keeps the next level's clearing of the buckets behind
            // every thread's read of the scan's result)
            __syncthreads();
        }
    }
    else
    {
        __syncthreads();
    }
    // compaction: survivors into the front of the buffer area, any order
    float* out_d = s.buf_d;
    int* out_x = s.buf_x;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < E; ++i)
    {
        const unsigned long long key = pair_key(pd[i], px[i]);
        bool keep = key < pivot;
        if (key == pivot && key != PAD_KEY)
        {
            keep = atomicAdd(&ctrl->sel_ties, 1) < ties;
        }
        const unsigned b = __ballot_sync(FULL_MASK, keep);
        if (b != 0)
        {
            int base = 0;
            if (lane == 0)
            {
                base = atomicAdd(&ctrl->sel_kept, __popc(b));
            }
            base = __shfl_sync(FULL_MASK, base, 0);
            if (keep)
            {
                const int pos = base + __popc(b & ((1U << lane) - 1U));
                out_d[pos] = pd[i];
                out_x[pos] = px[i];
            }
        }
    }
    __syncthreads();
    const int kept = ctrl->sel_kept;
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        const int e = tid * IPT + r;
        ld[r] = e < kept ? out_d[e] : INFINITY;
        lx[r] = e < kept ? out_x[e] : PAD_IDX;
    }
    if (tid == 0)
    {
        // the pivot is the k-th smallest pair seen so far
        float rd = INFINITY;
        int rx = PAD_IDX;
        if (pivot != PAD_KEY)
        {
            uint32_t u = static_cast<uint32_t>(pivot >> 32);
            u = (u & 0x80000000U) != 0 ? (u ^ 0x80000000U) : ~u;
            rd = __uint_as_float(u);
            rx = static_cast<int>(static_cast<uint32_t>(pivot) ^ 0x80000000U);
        }
        ctrl->r_d = rd;
        ctrl->r_x = rx;
        ctrl->count = 0;
    }
    __syncthreads();
    return 0;
}

// Lists of this many pairs and more are folded by selection.
constexpr int SELECT_FOLD_FROM = 1024;

// Folds buffer entries into the list, L at a time, and publishes the new radius in ctrl->r_d/r_x.
// Whole chunks of L are always folded; a remainder is folded too (padded) when it holds at least
// `keep_below` entries, else it is moved to the front of the buffer and stays a candidate.
// Returns the number of entries left in the buffer.  Entered and left with all threads.
template <int THREADS, int IPT>
__device__ __forceinline__ int fold_buffer(float (&ld)[IPT], int (&lx)[IPT], row_ctx s, int valid, int keep_below)
{
    constexpr int L = THREADS * IPT;
    if constexpr (L >= SELECT_FOLD_FROM)
    {
        return fold_select<THREADS, IPT>(ld, lx, s, valid);
    }
    const int tid = threadIdx.x;
    int base = 0;
    for (; base < valid; base += L)
    {
        const int here = valid - base < L ? valid - base : L;
        if (here < L && here < keep_below)
        {
            break;
        }
        float cd[IPT];
        int cx[IPT];
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = r * THREADS + tid;
            const bool in = e < here;
            cd[r] = in ? s.buf_d[base + e] : INFINITY;
            cx[r] = in ? s.buf_x[base + e] : PAD_IDX;
        }
        __syncthreads(); // these L slots now double as exchange scratch of the networks
        block_fold<THREADS, IPT>(ld, lx, cd, cx, s.buf_d + base, s.buf_x + base, tid);
    }
    const int left = base < valid ? valid - base : 0;
    float md[IPT];
    int mx[IPT];
    if (left > 0 && base > 0)
    {
        // the remainder moves to the front (it is shorter than a chunk: one read, barrier, write)
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = r * THREADS + tid;
            md[r] = e < left ? s.buf_d[base + e] : 0.0F;
            mx[r] = e < left ? s.buf_x[base + e] : 0;
        }
    }
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        if (tid * IPT + r == s.k - 1)
        {
            s.ctrl->r_d = ld[r];
            s.ctrl->r_x = lx[r];
        }
    }
    if (tid == 0)
    {
        s.ctrl->count = left;
    }
    __syncthreads();
    if (left > 0 && base > 0)
    {
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = r * THREADS + tid;
            if (e < left)
            {
                s.buf_d[e] = md[r];
                s.buf_x[e] = mx[r];
            }
        }
    }
    return left;
}

// Guaranteed insertion of one stage: the reference's scheme (bits_kernel.cuh:277-302,
// 383-391) -- allocate slots for a batch of THREADS*4 values, write those that fit, fold
// the full buffer and retry the rest.  Leaves the number of buffered entries in ctrl->count and
// the radius in ctrl->r_d/r_x.
template <int THREADS, int IPT>
__device__ __forceinline__ bool stage_slow(float (&ld)[IPT], int (&lx)[IPT], row_ctx s, const float4* sv, int nv, int e_base,
                                        int count0)
{
    constexpr int B = 2 * THREADS * IPT;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    bool folded = false; // the stage's survivors did not fit beside what the buffer held
    if (tid == 0)
    {
        s.ctrl->count = count0;
        s.ctrl->r_d = s.r_d;
        s.ctrl->r_x = s.r_x;
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
        filter4(s, val, live, e_base + 4 * v, dv, lab, pr);
        while (true)
        {
            // allocate slots for what is still pending, write what fits
            int off[4];
            const int total = warp_slots(pr, off);
            int base = 0;
            if (lane == 0 && total > 0)
            {
                base = atomicAdd(&s.ctrl->count, total);
            }
            base = __shfl_sync(FULL_MASK, base, 0);
            bool overflow = false;
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                if (pr[j])
                {
                    const int pos = base + off[j];
                    if (pos < B)
                    {
                        s.buf_d[pos] = dv[j];
                        s.buf_x[pos] = lab[j];
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
            folded = true;
            fold_buffer<THREADS, IPT>(ld, lx, s, B, 0);
            if (!s.keep_radius)
            {
                s.r_d = s.ctrl->r_d;
                s.r_x = s.ctrl->r_x;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                pr[j] = pr[j] && pair_lt(dv[j], lab[j], s.r_d, s.r_x);
            }
        }
    }
    return folded;
}

// Number of values of the stage that pass the radius filter and are not above the pivot pair
// (block-wide; two barriers).  A pivot that is itself a survivor is below the radius, so
// everything at or below it passes the filter too and only the pivot is compared (BELOW_RADIUS).
template <int THREADS, bool BELOW_RADIUS>
__device__ __forceinline__ int count_stage(const row_ctx& s, const float4* sv, int nv, int e_base, float pd, int px)
{
    const int tid = threadIdx.x;
    int c = 0;
    for (int v = tid; v < nv; v += THREADS)
    {
        const float4 val = sv[v];
        const float dv[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            if constexpr (BELOW_RADIUS)
            {
                c += dv[j] < pd ? 1 : 0;
                if (dv[j] == pd)
                {
                    c += label_of(s, e_base + 4 * v + j) <= px ? 1 : 0;
                }
            }
            else
            {
                if (dv[j] <= s.r_d)
                {
                    c += pair_lt(dv[j], label_of(s, e_base + 4 * v + j), s.r_d, s.r_x) ? 1 : 0;
                }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        c += __shfl_xor_sync(FULL_MASK, c, o);
    }
    if ((tid & 31) == 0)
    {
        s.ctrl->warp_sums[tid >> 5] = c;
    }
    __syncthreads();
    int total = 0;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w)
    {
        total += s.ctrl->warp_sums[w];
    }
    __syncthreads();
    return total;
}

// Decides how the survivors of a stage that the optimistic pass could not place (or that is
// expected to be dense) reach the buffer.  Returns the number of values the next pass over the
// stage will insert, or -1 when no pivot was found (the caller falls back to stage_slow).
//   * no more survivors than the buffer has room for: the radius stays, all of them go in
//     (ctrl->dense = 0);
//   * a dense stage (ctrl->dense = 1): a sorted sample of L of its values proposes pivots until
//     one has at least k and at most `room` survivors at or below it (preferably no more than fit
//     one chunk of L, or little more than k when k is close to L).  That pivot, published in
//     ctrl->r_d/r_x as an inclusive bound, becomes the radius of the pass (the fold that follows
//     replaces it by the list's own radius, which is not above it); everything above the pivot
//     cannot be among the k smallest pairs.
// `expect_dense` skips the count of all survivors.  The buffer holds count0 < L candidates in
// its first half; the second half is scratch here (sample sort, sorted samples).
template <int THREADS, int IPT>
__device__ __forceinline__ int plan_stage(row_ctx s, const float4* sv, int nv, int e_base, int count0, bool expect_dense)
{
    constexpr int L = THREADS * IPT;
    constexpr int B = 2 * L;
    const int tid = threadIdx.x;
    const int total = 4 * nv;
    const int room = B - count0;
    if (!expect_dense)
    {
        const int survivors = count_stage<THREADS, false>(s, sv, nv, e_base, 0.0F, 0);
        if (survivors <= room)
        {
            if (tid == 0)
            {
                s.ctrl->dense = 0;
            }
            __syncthreads();
            return survivors;
        }
    }
    float* scr_d = s.buf_d + L;
    int* scr_x = s.buf_x + L;
    // sorted sample of L values of the stage (values that fail the filter count as padding)
    {
        float sd[IPT];
        int sx[IPT];
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            const int e = tid * IPT + r;
            sd[r] = INFINITY;
            sx[r] = PAD_IDX;
            if (total >= L || e < total)
            {
                const int at = total >= L ? static_cast<int>((static_cast<int64_t>(e) * total) / L) : e;
                const float v = reinterpret_cast<const float*>(sv)[at];
                const int lab = label_of(s, e_base + at);
                if (pair_lt(v, lab, s.r_d, s.r_x))
                {
                    sd[r] = v;
                    sx[r] = lab;
                }
            }
        }
        block_sort<THREADS, IPT>(sd, sx, false, scr_d, scr_x, tid);
#pragma unroll
        for (int r = 0; r < IPT; ++r)
        {
            scr_d[tid * IPT + r] = sd[r];
            scr_x[tid * IPT + r] = sx[r];
        }
        __syncthreads();
    }
    // Acceptable: k <= c <= room.  Preferred: one chunk (c <= L) when k leaves space for that,
    // else at most a quarter chunk beyond k (what is beyond a chunk stays in the buffer).
    const int k = s.k;
    const bool one_chunk = 4 * k <= 3 * L;
    const int want_hi = one_chunk ? L : (k + L / 4 < room ? k + L / 4 : room);
    const int target = (k + want_hi) / 2;
    int lo = -1; // largest sample rank known to have fewer than k survivors at or below it
    int hi = L;  // smallest sample rank known to have more than want_hi
    int best_j = -1; // a sample inside [k, room] but above want_hi, in case nothing better turns up
    int best_c = 0;
    // the j-th smallest sample has about (j + 1) * total / L survivors at or below it
    int j = static_cast<int>((static_cast<int64_t>(target) * L) / (total > 0 ? total : 1)) - 1;
    j = j < 0 ? 0 : (j > L - 1 ? L - 1 : j);
    int chosen = -1;
    int chosen_c = 0;
    for (int it = 0; it < 8; ++it)
    {
        const float pd = scr_d[j];
        const int px = scr_x[j];
        int c = room + 1; // a padding sample is at or above every survivor
        if (px != PAD_IDX)
        {
            c = count_stage<THREADS, true>(s, sv, nv, e_base, pd, px);
        }
        if (c >= k && c <= want_hi)
        {
            chosen = j;
            chosen_c = c;
            break;
        }
        if (c < k)
        {
            lo = j;
        }
        else
        {
            hi = j;
            if (c <= room && (best_j < 0 || c < best_c))
            {
                best_j = j;
                best_c = c;
            }
        }
        if (hi - lo <= 1)
        {
            break;
        }
        int64_t next = (c > 0 && c <= room) ? (static_cast<int64_t>(j + 1) * target) / c - 1 : (lo + hi) / 2;
        if (next <= lo || next >= hi)
        {
            next = (lo + hi) / 2;
        }
        j = static_cast<int>(next);
    }
    if (chosen < 0)
    {
        chosen = best_j;
        chosen_c = best_c;
    }
    if (chosen < 0)
    {
        if (expect_dense)
        {
            // the stage was not dense after all: if all its survivors fit, they simply go in
            const int survivors = count_stage<THREADS, false>(s, sv, nv, e_base, 0.0F, 0);
            if (survivors <= room)
            {
                if (tid == 0)
                {
                    s.ctrl->dense = 0;
                }
                __syncthreads();
                return survivors;
            }
        }
        return -1;
    }
    if (tid == 0)
    {
        // inclusive bound for the strict filter: labels are integers
        s.ctrl->r_d = scr_d[chosen];
        s.ctrl->r_x = scr_x[chosen] + 1;
        s.ctrl->dense = 1;
    }
    __syncthreads(); // the bound is published; every thread is done with the scratch half
    return chosen_c;
}

// Position of a block in its row: which chunk comes next, where the ring and the rotating
// counters stand, how many candidates wait in the buffer, the radius.  Lives in local memory and
// is only read and written when stream_row() is entered and left.
struct stream_state
{
    int c;          // next chunk
    int st;         // its stage                      (c % stages)
    uint32_t phase; // parity of that stage's use     ((c / stages) & 1)
    int i3;         // c % 3
    int count0;     // candidates in the buffer; identical in every thread
    int dense_run;  // dense stages in a row
    float r_d;      // radius = k-th smallest pair seen so far
    int r_x;
};

// What does not change while a row is scanned.
struct row_layout
{
    float* stage_base;
    uint64_t* bars;
    const float* stream; // first streamed element of the row (16-byte aligned)
    int h;               // elements before it (labels of the stream start at h)
    int mid;             // streamed elements
    int nchunks;
    int CH;
    int NST;
    int merge_at;
};

enum stream_event
{
    EV_DONE = 0,     // the row is finished
    EV_PLAN = 1,     // chunk c has arrived and is expected to be dense: nothing was done with it
    EV_OVERFLOW = 2, // the optimistic pass over chunk c did not fit: it is to be forgotten
    EV_FOLD = 3,     // the pass over chunk c went in and the buffer wants folding
    EV_TIMEOUT = 4
};

__device__ __forceinline__ void issue_chunk(const row_layout& g, int c, int st)
{
    const int floats = (g.mid - c * g.CH) < g.CH ? (g.mid - c * g.CH) : g.CH;
    ptx::mbar_expect_tx(&g.bars[st], static_cast<uint32_t>(floats) * 4U);
    ptx::bulk_g2s(g.stage_base + static_cast<size_t>(st) * g.CH, g.stream + static_cast<int64_t>(c) * g.CH,
                  static_cast<uint32_t>(floats) * 4U, &g.bars[st]);
}

// The streaming loop: stage after stage, one optimistic pass and one barrier each, for as long as
// the survivors fit and the buffer does not want folding.  Everything else is reported to the
// caller as an event, with the chunk in question still in its stage.  The caller runs it as the
// inner loop of its event loop, so the compiler treats this loop, and not the sorting networks
// of the event handlers, as the place where registers matter (64 per thread at four blocks per SM).
template <int THREADS, int IPT, int UNROLL>
__device__ __forceinline__ int stream_row(stream_state* state, row_ctx s, const row_layout& g)
{
    constexpr int B = 2 * THREADS * IPT;
    const int tid = threadIdx.x;
    int c = state->c;
    int st = state->st;
    uint32_t phase = state->phase;
    int i3 = state->i3;
    int count0 = state->count0;
    const int dense_run = state->dense_run;
    s.r_d = state->r_d;
    s.r_x = state->r_x;
    int event = EV_DONE;
    for (; c < g.nchunks; ++c)
    {
        const float4* sv = reinterpret_cast<const float4*>(g.stage_base + static_cast<size_t>(st) * g.CH);
        const int floats = (g.mid - c * g.CH) < g.CH ? (g.mid - c * g.CH) : g.CH;
        const int nv = floats >> 2;
        const int e_base = g.h + c * g.CH;
        int* inc = &s.ctrl->inc[i3];

        const bool arrived = ptx::mbar_wait_bounded(&g.bars[st], phase);
        // no optimistic pass where it is bound to fail: the first stage (radius +inf), or after
        // two dense stages in a row (the same decision in every thread)
        const bool plan = (c == 0 || dense_run >= 2) && 4 * nv > B - count0 && !s.keep_radius;
        if (arrived && !plan)
        {
            scan_stage<THREADS, UNROLL>(s, B, sv, nv, e_base, count0, inc);
        }
        // one barrier per stage: every thread is done reading the stage and adding to `inc`; a
        // thread whose wait expired takes the whole block out with it
        if (__syncthreads_or(arrived ? 0 : 1) != 0)
        {
            event = EV_TIMEOUT;
            break;
        }
        if (plan)
        {
            event = EV_PLAN;
            break;
        }
        const int added = *inc;
        if (count0 + added > B)
        {
            event = EV_OVERFLOW; // some survivors were dropped
            break;
        }
        count0 += added;
        if (count0 >= g.merge_at)
        {
            event = EV_FOLD;
            break;
        }
        if (tid == 0)
        {
            s.ctrl->inc[i3 == 0 ? 2 : i3 - 1] = 0; // slot of stage c+2: last read before this barrier
            // every thread has passed a barrier after its last read of this stage
            if (c + g.NST < g.nchunks)
            {
                issue_chunk(g, c + g.NST, st);
            }
        }
        i3 = i3 == 2 ? 0 : i3 + 1;
        if (++st == g.NST)
        {
            st = 0;
            phase ^= 1U;
        }
    }
    state->c = c;
    state->st = st;
    state->phase = phase;
    state->i3 = i3;
    state->count0 = count0;
    return event;
}

// 64 registers per thread at most: four blocks of 256 threads (two of 512, one of 1024) per SM
#ifndef BITSKNN_SELECT_MINBLOCKS
#define BITSKNN_SELECT_MINBLOCKS (1024 / THREADS)
#endif
template <int THREADS, int IPT, int UNROLL>
__global__ void __launch_bounds__(THREADS, BITSKNN_SELECT_MINBLOCKS) select_kernel(const select_params p)
{
    constexpr int L = THREADS * IPT;
    constexpr int B = 2 * L;

    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;

    row_layout g;
    g.CH = p.stage_floats;
    g.NST = p.stages;
    g.merge_at = p.merge_at;
    g.stage_base = reinterpret_cast<float*>(smem);
    row_ctx s;
    s.buf_d = g.stage_base + static_cast<size_t>(g.NST) * g.CH;
    s.buf_x = reinterpret_cast<int*>(s.buf_d + B);
    g.bars = reinterpret_cast<uint64_t*>(s.buf_x + B);
    s.ctrl = reinterpret_cast<select_ctrl*>(g.bars + MAX_STAGES);
    s.k = p.k;
    s.keep_radius = p.no_filter != 0;

    // which slice of which row
    const int64_t vrow = blockIdx.x;
    const int64_t row = vrow / p.splits;
    const int64_t begin = (vrow - row * p.splits) * p.slice;
    int64_t m64 = (p.n < begin + p.slice ? p.n : begin + p.slice) - begin;
    const int m = m64 > 0 ? static_cast<int>(m64) : 0;
    const float* rowp = p.dist + row * p.ld + begin;
    s.labp = p.labels != nullptr ? p.labels + row * p.ld_labels + begin : nullptr;
    s.lab0 = static_cast<int>(begin) + p.label_base + (p.label_offsets != nullptr ? p.label_offsets[row] : 0);

    // [0,h): scalar head up to the first 16-byte boundary, [h,h+mid): streamed, then a tail < 4
    int h = static_cast<int>(((16U - (reinterpret_cast<uintptr_t>(rowp) & 15U)) & 15U) >> 2);
    h = h < m ? h : m;
    g.h = h;
    g.mid = ((m - h) >> 2) << 2;
    const int tail = m - h - g.mid;
    g.nchunks = (g.mid + g.CH - 1) / g.CH;
    g.stream = rowp + h;

    // the sorted list (ascending), blocked arrangement
    float ld[IPT];
    int lx[IPT];
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        ld[r] = INFINITY;
        lx[r] = PAD_IDX;
    }
    s.r_d = INFINITY;
    s.r_x = PAD_IDX;

    if (tid == 0)
    {
        for (int i = 0; i < g.NST; ++i)
        {
            ptx::mbar_init(&g.bars[i], 1);
        }
        s.ctrl->count = 0;
        s.ctrl->inc[0] = 0;
        s.ctrl->inc[1] = 0;
        s.ctrl->inc[2] = 0;
        ptx::mbar_init_fence();
    }
    __syncthreads();
    if (tid == 0)
    {
        for (int c = 0; c < g.NST && c < g.nchunks; ++c)
        {
            issue_chunk(g, c, c);
        }
    }

    // head and tail elements go straight into the buffer (at most 6 of them)
    if (tid < h + tail)
    {
        const int e = tid < h ? tid : g.mid + tid;
        const float d = rowp[e];
        const int lab = label_of(s, e);
        if (pair_lt(d, lab, s.r_d, s.r_x))
        {
            const int pos = atomicAdd(&s.ctrl->count, 1);
            s.buf_d[pos] = d;
            s.buf_x[pos] = lab;
        }
    }
    __syncthreads();

    stream_state state;
    state.c = 0;
    state.st = 0;
    state.phase = 0;
    state.i3 = 0;
    state.count0 = s.ctrl->count;
    state.dense_run = 0;
    state.r_d = s.r_d;
    state.r_x = s.r_x;

    while (true)
    {
        const int event = stream_row<THREADS, IPT, UNROLL>(&state, s, g);
        if (event == EV_DONE)
        {
            break;
        }
        if (event == EV_TIMEOUT)
        {
            // report, let the copies still in flight land (bounded), and leave
            for (int cc = state.c + 1; cc < g.nchunks && cc < state.c + g.NST; ++cc)
            {
                ptx::mbar_wait_bounded(&g.bars[cc % g.NST], static_cast<uint32_t>((cc / g.NST) & 1), 1U << 16);
            }
            if (tid == 0)
            {
                atomicOr(p.status, DEVICE_STATUS_TIMEOUT);
            }
            return;
        }
        // chunk state.c sits in its stage and wants more than an optimistic pass
        const int c = state.c;
        const float4* sv = reinterpret_cast<const float4*>(g.stage_base + static_cast<size_t>(state.st) * g.CH);
        const int floats = (g.mid - c * g.CH) < g.CH ? (g.mid - c * g.CH) : g.CH;
        const int nv = floats >> 2;
        const int e_base = g.h + c * g.CH;
        int* inc = &s.ctrl->inc[state.i3];
        int count0 = state.count0;
        bool dense = false;
        if (event == EV_PLAN || event == EV_OVERFLOW)
        {
            // the un-buffered ablation sorts and merges every value; with folds by selection the first
            // stage (radius +inf: everything goes in) is cheaper taken as it is than planned: its three
            // or four folds cost less than the plan's sorted sample and counting passes
            const bool first_unplanned = L >= SELECT_FOLD_FROM && event == EV_PLAN && c == 0;
            bool slow = s.keep_radius || first_unplanned;
            if (L >= SELECT_FOLD_FROM && count0 >= L && !slow)
            {
                // the plan sorts its sample in the upper half of the buffer; with folds by selection
                // the buffer may hold more than a list's worth by now: those go into the list first
                count0 = fold_buffer<THREADS, IPT>(ld, lx, s, count0, 0);
                s.r_d = s.ctrl->r_d;
                s.r_x = s.ctrl->r_x;
            }
            if (!slow)
            {
                if (event == EV_OVERFLOW)
                {
                    // the pass is forgotten; the barrier keeps the reset behind every thread's read of
                    // the pass's count (a thread that read 0 instead would carry on alone)
                    __syncthreads();
                    if (tid == 0)
                    {
                        *inc = 0;
                    }
                }
                // which of the stage's survivors go in, and under which radius
                const int planned = plan_stage<THREADS, IPT>(s, sv, nv, e_base, count0, event == EV_PLAN);
                if (planned < 0)
                {
                    slow = true;
                }
                else
                {
                    dense = s.ctrl->dense != 0;
                    if (dense)
                    {
                        s.r_d = s.ctrl->r_d;
                        s.r_x = s.ctrl->r_x;
                    }
                    scan_stage<THREADS, UNROLL>(s, B, sv, nv, e_base, count0, inc);
                    __syncthreads();
                    count0 += planned;
                }
            }
            if (slow)
            {
                const bool folded = stage_slow<THREADS, IPT>(ld, lx, s, sv, nv, e_base, count0);
                dense = first_unplanned && folded;
                count0 = s.ctrl->count;
                if (!s.keep_radius)
                {
                    s.r_d = s.ctrl->r_d;
                    s.r_x = s.ctrl->r_x;
                }
            }
        }
        state.dense_run = dense ? state.dense_run + 1 : 0;
        // The stage is done (every thread has passed a barrier after its last read of it): its memory
        // is refilled now, before the fold, so that the copy runs while the block folds.
        if (tid == 0 && c + g.NST < g.nchunks)
        {
            issue_chunk(g, c + g.NST, state.st);
        }
        if (count0 >= g.merge_at)
        {
            count0 = fold_buffer<THREADS, IPT>(ld, lx, s, count0, g.merge_at);
            if (!s.keep_radius)
            {
                s.r_d = s.ctrl->r_d;
                s.r_x = s.ctrl->r_x;
            }
        }
        // its counter slot of two stages on is cleared
        if (tid == 0)
        {
            s.ctrl->inc[state.i3 == 0 ? 2 : state.i3 - 1] = 0;
        }
        state.c = c + 1;
        state.i3 = state.i3 == 2 ? 0 : state.i3 + 1;
        if (++state.st == g.NST)
        {
            state.st = 0;
            state.phase ^= 1U;
        }
        state.count0 = count0;
        state.r_d = s.r_d;
        state.r_x = s.r_x;
    }

    if (state.count0 > 0)
    {
        fold_buffer<THREADS, IPT>(ld, lx, s, state.count0, 0);
    }
    if constexpr (L >= SELECT_FOLD_FROM)
    {
        // the list was kept as a set: sorted once, here
        __syncthreads();
        block_sort<THREADS, IPT>(ld, lx, false, s.buf_d, s.buf_x, tid);
    }

    float* od = p.out_dist + vrow * p.k;
    int32_t* ox = p.out_idx + vrow * p.k;
#pragma unroll
    for (int r = 0; r < IPT; ++r)
    {
        const int e = tid * IPT + r;
        if (e < p.k)
        {
            int x = lx[r];
            if (p.raw_pad == 0 && x == PAD_IDX)
            {
                x = e; // the reference pads short rows with (+inf, position): bits_kernel.cuh:340-358
            }
            od[e] = ld[r];
            ox[e] = x;
        }
    }
}

size_t select_smem_bytes(int L, int stage_floats, int stages)
{
    // stages + candidate buffer (2 L pairs) + barriers + control
    return static_cast<size_t>(stages) * stage_floats * 4 + static_cast<size_t>(2 * L) * 8 + MAX_STAGES * 8 +
           sizeof(select_ctrl);
}

// The launch shape of one selection: block size, pairs per thread, stage ring, fold threshold.
// Knobs set by the caller win, then the tuning table (keyed by k and the number of row slices),
// then the built-in rule.
struct launch_shape
{
    int threads;
    int ipt;
    int stage_bytes;
    int stages;
    int merge_pct;
    int unroll;
};

launch_shape resolve_shape(int k, int64_t vrows)
{
    // built-in rule: the smallest list that holds k (the reference's dynamic_switch_le over K,
    // src/topk/singlepass/bits_knn.cu:44), with the list never shorter than the block.  Long lists
    // take larger blocks (the reference's tuned shapes use 512 threads for k = 2048,
    // scripts/optima.csv:1282): more threads fold a list of the same length with fewer pairs, and
    // registers, per thread.  3 x 16 KiB stages for 256-thread blocks (4 blocks per SM), 3 x 32 KiB
    // for 512-thread blocks, 2 x 64 KiB for 1024-thread blocks; half-full buffers are folded for
    // lists of up to 256 pairs, three-quarter-full ones for longer lists, whose folds cost more
    // against what an earlier tightening of the radius saves.
    launch_shape shape{};
    if (k <= 256)
    {
        shape = {256, 1, 16384, 3, 50, 2};
    }
    else if (k <= 512)
    {
        shape = {512, 1, 32768, 3, 75, 2};
    }
    else if (k <= 1024)
    {
        shape = {512, 2, 32768, 3, 75, 2};
    }
    else
    {
        shape = {1024, 2, 65536, 2, 75, 2};
    }
    if (const select_shape* row = find_select_shape(k, vrows); row != nullptr)
    {
        shape = {row->threads, row->ipt, row->stage_bytes, row->stages, row->merge_pct, row->unroll};
    }
    const int threads = tuning_value("select.threads", 0);
    const int ipt = tuning_value("select.ipt", 0);
    if (threads > 0 && ipt > 0 && threads * ipt >= k)
    {
        shape.threads = threads;
        shape.ipt = ipt;
    }
    if (const int v = tuning_value("select.stage_bytes", 0); v > 0)
    {
        shape.stage_bytes = v;
    }
    if (const int v = tuning_value("select.stages", 0); v > 0)
    {
        shape.stages = v;
    }
    if (const int v = tuning_value("select.merge_at", 0); v > 0)
    {
        shape.merge_pct = v;
    }
    if (const int v = tuning_value("select.unroll", 0); v > 0)
    {
        shape.unroll = v;
    }
    return shape;
}

template <int THREADS, int IPT>
int launch_select(select_params p, const launch_shape& shape, int64_t vrows, cudaStream_t stream)
{
    constexpr int L = THREADS * IPT;
    // (folds by selection take the whole buffer of 2 L slots whatever it holds, so they may wait longer)
    p.merge_at = std::min(L >= SELECT_FOLD_FROM ? 2 * L - L / 8 : L, std::max(1, (L * shape.merge_pct) / 100));
    // a stage is a whole number of 4-vectors per thread
    const int stage_bytes = std::max((shape.stage_bytes / 4096) * 4096, 4096);
    p.stage_floats = std::max(4 * THREADS, (stage_bytes / 4 / (4 * THREADS)) * (4 * THREADS));
    p.stages = std::min(std::max(shape.stages, 2), MAX_STAGES);
    const size_t smem = select_smem_bytes(L, p.stage_floats, p.stages);
    // 128-bit vectors per thread examined under one warp vote
    auto kernel = shape.unroll == 4 ? select_kernel<THREADS, IPT, 4> : select_kernel<THREADS, IPT, 2>;
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
    const launch_shape shape = resolve_shape(p.k, vrows);
    switch (shape.threads * 16 + shape.ipt)
    {
    case 256 * 16 + 1:
        return launch_select<256, 1>(p, shape, vrows, stream);
    case 256 * 16 + 2:
        return launch_select<256, 2>(p, shape, vrows, stream);
    case 256 * 16 + 4:
        return launch_select<256, 4>(p, shape, vrows, stream);
    case 512 * 16 + 1:
        return launch_select<512, 1>(p, shape, vrows, stream);
    case 512 * 16 + 2:
        return launch_select<512, 2>(p, shape, vrows, stream);
    case 512 * 16 + 4:
        return launch_select<512, 4>(p, shape, vrows, stream);
    case 1024 * 16 + 1:
        return launch_select<1024, 1>(p, shape, vrows, stream);
    case 1024 * 16 + 2:
        return launch_select<1024, 2>(p, shape, vrows, stream);
    default:
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "no selection kernel for %d threads x %d pairs per thread",
                    shape.threads, shape.ipt);
    }
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

} // namespace

} // namespace bitsknn

using namespace bitsknn;

namespace bitsknn
{

int select_rows(const float* d_dist, int64_t ld, const int32_t* d_labels, int64_t ld_labels,
                const int32_t* d_label_offsets, int32_t label_base, int64_t q, int64_t n, int k, float* d_out_dist,
                int32_t* d_out_idx, cudaStream_t stream, bool no_filter)
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
    // without the radius filter this is the un-buffered partial bitonic sort the reference keeps as
    // an ablation (partial-bitonic-regs, src/topk/singlepass/partial_bitonic.cu:217-294)
    p.no_filter = no_filter ? 1 : 0;
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
    int wanted = k <= 64 ? 600 : (k <= 256 ? 400 : (k <= 1024 ? 200 : 130));
    if (const select_shape* row = find_select_shape(k, q); row != nullptr && row->blocks_wanted > 0)
    {
        wanted = row->blocks_wanted;
    }
    const int64_t want = static_cast<int64_t>(sms) * wanted / 148;
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
    auto cs = static_cast<cudaStream_t>(stream);
    if (const int rc = dispatch_select(p, q * splits, cs); rc != BITSKNN_OK)
    {
        return rc;
    }
    return dispatch_merge(cand_dist, cand_idx, k, static_cast<int64_t>(splits) * k, q, splits, k, d_out_dist,
                          d_out_idx, cs);
}
