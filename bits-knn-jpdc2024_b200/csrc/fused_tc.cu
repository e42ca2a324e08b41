// `bits-fused` on the tensor cores: the partial distance tile is produced by tcgen05.mma in
// tensor memory and consumed from there by the top-k -- no distance ever reaches HBM.
//
// The contraction runs over the compact split image of tc_host.cuh ([hi | lo | norm columns]; the
// MMA warp pairs the K steps: points.hi with queries.hi and queries.lo, points.lo with
// queries.hi, norm step with norm step), so an accumulator holds  s = x.y - |x|^2 / 2  and the
// partial distance is d = -2 s (= |x|^2 - 2 x.y, the quantity the reference's fused kernel ranks by,
// include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:622-630).  The consumer compares
// raw accumulators against  -bound / 2: one max-tree and one vote per 16 columns.
//
// Block = 352 threads on one SM, 128 queries (the TMEM lanes):
//   warp 8   TMA producer (query image once, point image K blocks through a ring of stages)
//   warps 9, 10  tcgen05.mma issue, the two taking MMAs in turn (tc_pipeline.cuh; warp 9 also
//            allocates the tensor memory: 4 accumulators of 128 columns).  Whenever the ring fits,
//            an MMA covers 256 points and fills two neighbouring accumulators, one per consumer
//            group (NMMA = 256); long vectors fall back to 128 points per MMA.
//   warps 0-7  consumers, two groups of four.  Group g takes every other 128-point tile (each
//            group alternates between two accumulators, so the MMAs run ahead of it);
//            thread t of a group is query 32 * (warp % 4) + t and reads its row with
//            tcgen05.ld.  Each (group, query) has a private 32-slot candidate buffer in shared
//            memory (no atomics: one writer) and a sorted list of KL = 32 * IPT pairs in the
//            workspace (HBM/L2), touched only when the buffer is folded: the warp sorts the 32
//            candidates with shuffles, takes the element-wise minimum against the list's last 32
//            entries and finishes with a bitonic merge (striped arrangement: entry e in lane
//            e % 32).  The acceptance bound of a query is the smallest of: its group's radius,
//            the partner group's radius, and the larger of the two lists' entries
//            ceil(k / 2) - 1 (the lists cover different points, so k pairs lie at or below it).
// After the scan the 2 * parts lists of every query hold its candidates by tensor-core distance;
// rerank_lists() recomputes every candidate's distance as the exact FP32 chain of (y - x)^2 and
// reports the k smallest pairs by that, so the rounding of the tensor-core inputs only decides
// which pairs are looked at (with an allowance in the acceptance bound), not what is reported.
// Role of the reference's fused_tc_kernel (detail/fused_tc_kernel.cuh:177-445, wmma based and
// "suboptimal" by its authors' note in src/gen.py:45), rebuilt on tcgen05 / TMEM / TMA.
#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "ptx.cuh"
#include "sortnet.cuh"
#include "tc.cuh"
#include "tc_host.cuh"
#include "tc_pipeline.cuh"
#include "warpfold.cuh"

namespace bitsknn
{

namespace
{

constexpr int FT_THREADS = 352;
constexpr int FT_PRODUCER_WARP = 8;
constexpr int FT_MMA_WARP = 9;
constexpr int FT_ACCS = tcpipe::ACCS; // four 128-column accumulators: each consumer group owns two
constexpr int CAP = 32; // candidate slots per (group, query); 16 when the operand ring needs the room

struct ftc_params
{
    float* list_d;   // [parts * 2][q][KL]
    int32_t* list_x; // [parts * 2][q][KL]
    int64_t n;
    int64_t q;
    int nkb;    // 128-byte K blocks per row of the images
    int nsteps; // MMA K steps (32 bytes) per row that hold data
    int hs;     // steps of the hi part of a compact split image (0: plain image)
    int stages;
    int parts;
    int64_t tiles;
    int cap;          // candidate slots per (group, query): 32 or 16
    int fold_above;   // a buffer is folded when it holds more than this many candidates (cap - 16 or cap - 8)
    int k;            // list entry k - 1 is a list's radius (the reported k plus a margin)
    int32_t index_base;
    const float* qnorm;    // [q] squared norms of the queries
    const float* max_norm; // largest squared norm of a point
    float slack;           // relative error bound of the tensor-core distance (of |x|^2 + |y|^2)
    int* status;
};

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <bool BF16, int IPT, int NMMA>
__global__ void __launch_bounds__(FT_THREADS, 1)
    fused_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_p, const ftc_params p)
{
    constexpr int KL = 32 * IPT;
    constexpr int NT = NMMA / TILE_N;            // 128-column tiles per MMA (1 or 2)
    constexpr int STAGE_B = NT * STAGE_BYTES;    // one K block of NMMA points

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint2 a_tab_both[2][MAX_KB * 4]; // one descriptor table per MMA-issuing thread
    tcpipe::state pipe;
    pipe.a_tiles = smem;
    pipe.b_ring = pipe.a_tiles + static_cast<size_t>(p.nkb) * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pipe.b_ring + static_cast<size_t>(p.stages) * STAGE_B);
    pipe.a_full = bars;
    pipe.full_b = bars + 1;
    pipe.empty_b = pipe.full_b + 16;
    pipe.acc_full = pipe.empty_b + 16;
    pipe.acc_empty = pipe.acc_full + FT_ACCS;
    pipe.a_tab = &a_tab_both[0][0];
    uint64_t* acc_full = pipe.acc_full;
    uint64_t* acc_empty = pipe.acc_empty;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pipe.acc_empty + FT_ACCS);
    float* rad = reinterpret_cast<float*>(bars + 64);     // [2][128] radius distance per group and query
    float* hlf = rad + 2 * TILE_M;                        // [2][128] distance of list entry ceil(k / 2) - 1
    const int cap = p.cap;
    float* buf_d = hlf + 2 * TILE_M;                      // [8 warps][cap][32 lanes]
    int* buf_x = reinterpret_cast<int*>(buf_d + 8 * cap * 32);
    const tcpipe::shape shape{p.nkb, p.nsteps, p.hs, p.stages};

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int64_t qb = blockIdx.x / p.parts;
    const int part = static_cast<int>(blockIdx.x - qb * p.parts);
    // tiles of 128 points; a part is a whole number of MMAs (a tile beyond n holds no valid column)
    const int64_t per = ((p.tiles + p.parts - 1) / p.parts + NT - 1) / NT * NT;
    const int64_t tiles_up = (p.tiles + NT - 1) / NT * NT;
    const int64_t t_begin = part * per;
    const int64_t t_end = t_begin + per < tiles_up ? t_begin + per : tiles_up;

    if (tid == 0)
    {
        tcpipe::init_barriers(pipe, p.stages);
    }
    if (tid < 2 * TILE_M)
    {
        rad[tid] = INFINITY;
        hlf[tid] = INFINITY;
    }
    if (warp == FT_MMA_WARP)
    {
        tc::tmem_alloc(tmem_slot, tcpipe::TMEM_COLS);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == FT_PRODUCER_WARP)
    {
        if (lane == 0 && t_begin < t_end)
        {
            ok = tcpipe::producer<BF16, NMMA>(pipe, shape, &map_q, &map_p, qb * TILE_M, t_begin, t_end);
        }
    }
    else if (warp == FT_MMA_WARP || warp == FT_MMA_WARP + 1)
    {
        if (lane == 0 && t_begin < t_end)
        {
            ok = tcpipe::mma_issuer<BF16, NMMA>(pipe, shape, tmem_base, warp - FT_MMA_WARP, t_begin, t_end);
        }
    }
    else
    {
        const int group = warp >> 2;
        const int w4 = warp & 3;
        const int qrow = w4 * 32 + lane;              // query of this thread inside the tile
        const int64_t gq = qb * TILE_M + qrow;        // global query
        const bool live = gq < p.q;
        float* my_buf_d = buf_d + warp * (cap * 32);  // slot s of lane l at [s * 32 + (l + s) % 32]
        int* my_buf_x = buf_x + warp * (cap * 32);
        const int64_t list_id = static_cast<int64_t>(part) * 2 + group;
        const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;

        // radius pair of this (group, query); a dead row (query beyond q) never accepts anything
        float r_d = live ? INFINITY : -INFINITY;
        int r_x = PAD_IDX;
        float thr = live ? -INFINITY : INFINITY; // accumulators >= thr are candidates
        float h_d = INFINITY; // distance of entry ceil(k / 2) - 1 of this (group, query)'s list
        int cnt = 0;
        bool has_list = false;
        // What a tensor-core distance may be off by (the rounding of the split images and of the
        // accumulation grow with the norms, not with the distance): candidates are kept up to this
        // far beyond the k-th distance found so far, and the exact re-ranking after the scan decides.
        const float slack_d = live ? p.slack * (p.qnorm[gq] + *p.max_norm) : 0.0F;

        // Upper bound of the query's true k-th distance: each group's own radius, and the larger
        // of the two groups' entries ceil(k / 2) - 1 (the two lists cover different points, so at
        // least k pairs lie at or below it) plus the error allowance.
        auto bound = [&]() {
            const int other = (group ^ 1) * TILE_M + qrow;
            return fminf(fminf(r_d, rad[other]), fmaxf(h_d, hlf[other]) + slack_d);
        };

        // Folds the buffers of the queries whose lanes are set in `mask` into their lists.
        auto fold_queries = [&](unsigned mask) {
            while (mask != 0)
            {
                const int L = __ffs(static_cast<int>(mask)) - 1;
                mask &= mask - 1;
                const int cnt_l = __shfl_sync(FULL_MASK, cnt, L);
                const bool has_l = __shfl_sync(FULL_MASK, has_list ? 1 : 0, L) != 0;
                const int64_t gq_l = qb * TILE_M + w4 * 32 + L;
                float* gl_d = p.list_d + (list_id * p.q + gq_l) * KL;
                int32_t* gl_x = p.list_x + (list_id * p.q + gq_l) * KL;
                // candidates: slot `lane` of query L's buffer
                // (slot s of query L sits in bank (L + s) % 32: the 32 slots come from 32 banks)
                const float cd = lane < cnt_l ? my_buf_d[lane * 32 + ((L + lane) & 31)] : INFINITY;
                const int cx = lane < cnt_l ? my_buf_x[lane * 32 + ((L + lane) & 31)] : PAD_IDX;
                const radius_pair nr = warp_fold_global_call<IPT>(cd, cx, has_l, gl_d, gl_x, p.k, lane);
                const float nd = nr.d;
                const int nx = nr.x;
                if (lane == L)
                {
                    r_d = nd;
                    r_x = nx;
                    cnt = 0;
                    has_list = true;
                    h_d = nr.half_d;
                    rad[group * TILE_M + qrow] = nd;
                    hlf[group * TILE_M + qrow] = nr.half_d;
                }
                __syncwarp(); // the list stores are ordered before any later load by this warp
            }
        };

        // Maxima of the four groups of four columns of a half chunk.
        auto group_maxima = [](const uint32_t(&v)[16], float(&g)[4]) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                g[i] = fmaxf(max3(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2])),
                             __uint_as_float(v[4 * i + 3]));
            }
        };

        // Folds every buffer that is more than half full and tightens the bound.
        auto fold_full = [&]() {
            const unsigned need = __ballot_sync(FULL_MASK, cnt > p.fold_above);
            if (need != 0)
            {
                __syncwarp();
                fold_queries(need);
                if (live)
                {
                    thr = fmaxf(thr, -0.5F * bound());
                }
            }
        };

        // The candidates of one half chunk (16 columns) of this thread's row go to its buffer; full
        // buffers are folded.  A buffer holds at most fold_above candidates when a run of
        // cap - fold_above columns (16 or 8) starts, so the pushes of the run always fit.
        auto push_half = [&](const uint32_t(&v)[16], const float(&g)[4], int64_t col0) {
            const int ncols = p.n - col0 < 16 ? static_cast<int>(p.n - col0) : 16; // valid columns
            const float r_part = -2.0F * thr; // the bound as a distance
            // warp votes per group of four, then per column
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                if (__any_sync(FULL_MASK, g[i] >= thr))
                {
#pragma unroll
                    for (int j = 4 * i; j < 4 * i + 4; ++j)
                    {
                        const float s = __uint_as_float(v[j]);
                        if (s >= thr && j < ncols)
                        {
                            const float d = -2.0F * s;
                            const int idx = p.index_base + static_cast<int>(col0 + j);
                            if (d <= r_part && pair_lt(d, idx, r_d, r_x))
                            {
                                my_buf_d[cnt * 32 + ((lane + cnt) & 31)] = d;
                                my_buf_x[cnt * 32 + ((lane + cnt) & 31)] = idx;
                                ++cnt;
                            }
                        }
                    }
                }
                if (i == 1 && cap - p.fold_above < 16)
                {
                    fold_full();
                }
            }
            fold_full();
        };

        // this group's tiles are the local tiles lt = group, group + 2, ...; tile lt sits in
        // accumulator lt % 4, so the group alternates between its two accumulators
        int64_t lt = group;
        for (int64_t t = t_begin + group; t < t_end && ok; t += 2, lt += 2)
        {
            if (live)
            {
                thr = -0.5F * bound();
            }
            const int a = static_cast<int>(lt & (FT_ACCS - 1));
            // (made warp-uniform: the lanes poll independently)
            if (!__all_sync(FULL_MASK, ptx::mbar_wait_bounded_spin(&acc_full[tcpipe::acc_full_index<NMMA>(a)], static_cast<uint32_t>((lt >> 2) & 1))))
            {
                ok = false;
                break;
            }
            tc::fence_after_sync();
            const uint32_t acc_addr = tmem_base + lane_base + static_cast<uint32_t>(a * TILE_N);
            // 32 columns per step: both halves' max-trees run side by side and one vote rejects the
            // step; the registers are free for the next load as soon as the step is decided (the
            // other warp of this scheduler covers the load's latency)
            uint32_t lo[16];
            uint32_t hi[16];
            tc::tmem_ld_32x32_halves(acc_addr, lo, hi);
#pragma unroll 1
            for (int c = 0; c < TILE_N / 32; ++c)
            {
                float g_lo[4];
                float g_hi[4];
                tc::tmem_ld_wait();
                group_maxima(lo, g_lo);
                group_maxima(hi, g_hi);
                const float mx = max3(max3(g_lo[0], g_lo[1], g_lo[2]), max3(g_hi[0], g_hi[1], g_hi[2]),
                                      fmaxf(g_lo[3], g_hi[3]));
                if (__any_sync(FULL_MASK, mx >= thr))
                {
                    const int64_t col0 = t * TILE_N + c * 32;
                    push_half(lo, g_lo, col0);
                    push_half(hi, g_hi, col0 + 16);
                }
                if (c + 1 < TILE_N / 32)
                {
                    tc::tmem_ld_32x32_halves(acc_addr + static_cast<uint32_t>(c * 32 + 32), lo, hi);
                }
                else
                {
                    // every accumulator of this thread has been looked at: the buffer may be reused
                    tc::fence_before_sync();
                    tc::mbar_arrive(&acc_empty[a]);
                }
            }
        }
        // flush: every live (group, query) leaves a complete list behind, padding included
        __syncwarp();
        fold_queries(__ballot_sync(FULL_MASK, live && ok));
    }

    if (!ok)
    {
        atomicOr(p.status, DEVICE_STATUS_TIMEOUT);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == FT_MMA_WARP)
    {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, tcpipe::TMEM_COLS);
    }
}

struct ftc_layout
{
    int dim_pad; // row pitch of the images in elements
    int split;   // image kind for the pre-pass (2: compact split, 0: plain)
    int hs;      // K steps of the hi part (0: plain image)
    int nsteps;  // K steps that hold data
    int nkb;     // 128-byte K blocks per row
    int kl;
    int parts;
    int k_scan;  // list position of the radius during the scan: k plus a margin, at most kl
    size_t off_pn, off_qn, off_max, off_p, off_q, off_ld, off_lx, total;
};

ftc_layout ftc_layout_of(int64_t n, int64_t q, int dim, int k, bool bf16)
{
    ftc_layout l{};
    const tcpipe::image_shape img = tcpipe::image_shape_of(dim, bf16, true);
    l.dim_pad = img.dim_pad;
    l.split = img.split;
    l.hs = img.hs;
    l.nsteps = img.nsteps;
    l.nkb = img.nkb;
    l.kl = k <= 32 ? 32 : (k <= 64 ? 64 : (k <= 128 ? 128 : 256));
    // The lists are longer than k anyway; the scan keeps a few more pairs than asked for inside
    // them (a quarter more, at least four) so that a neighbour whose tensor-core distance came out
    // a little too large is still a candidate when the exact re-ranking decides.
    l.k_scan = std::min(l.kl, k + std::max(4, k / 4));
    const int64_t nqb = (q + TILE_M - 1) / TILE_M;
    const int64_t tiles = (n + TILE_N - 1) / TILE_N;
    // every extra part is one more pair of lists per query that has to find its own radius, so
    // the database is only split when the query tiles alone cannot occupy the SMs (parts of at
    // least 64 tiles)
    const int sms = device_sm_count();
    const int64_t want = 4 * nqb >= 3 * sms ? 1 : (sms + nqb - 1) / nqb;
    l.parts = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, std::max<int64_t>(1, tiles / 64))));
    if (const int forced = tuning_value("fused.parts", 0); forced > 0)
    {
        l.parts = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(forced, std::max<int64_t>(1, tiles / 64))));
    }
    const size_t esz = bf16 ? 2 : 4;
    l.off_pn = 0;
    l.off_qn = align256(static_cast<size_t>(n) * 4);
    l.off_max = l.off_qn + align256(static_cast<size_t>(q) * 4);
    l.off_p = l.off_max + 256;
    l.off_q = l.off_p + align256(static_cast<size_t>(n) * l.dim_pad * esz);
    l.off_ld = l.off_q + align256(static_cast<size_t>(q) * l.dim_pad * esz);
    const size_t lists = static_cast<size_t>(l.parts) * 2 * static_cast<size_t>(q) * l.kl;
    l.off_lx = l.off_ld + align256(lists * 4);
    l.total = l.off_lx + align256(lists * 4);
    return l;
}

template <bool BF16, int IPT, int NMMA>
int launch_ftc(const CUtensorMap& map_q, const CUtensorMap& map_p, const ftc_params& p, size_t smem, int64_t grid,
               cudaStream_t stream)
{
    auto kernel = fused_tc_kernel<BF16, IPT, NMMA>;
    BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    {
        kernel_scope timed{"fused_tc_kernel", stream};
        kernel<<<static_cast<unsigned>(grid), FT_THREADS, smem, stream>>>(map_q, map_p, p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

template <bool BF16>
int run_ftc(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int32_t index_base,
            float* out_dist, int32_t* out_idx, unsigned char* ws, cudaStream_t stream)
{
    const ftc_layout l = ftc_layout_of(n, q, dim, k, BF16);
    float* pn = reinterpret_cast<float*>(ws + l.off_pn);
    float* qn = reinterpret_cast<float*>(ws + l.off_qn);
    float* pmax = reinterpret_cast<float*>(ws + l.off_max);
    void* cp = ws + l.off_p;
    void* cq = ws + l.off_q;
    BITSKNN_CUDA_TRY(cudaMemsetAsync(pmax, 0, sizeof(float), stream));
    tc_prepare_kernel<BF16>
        <<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(points, n, dim, l.dim_pad, l.split, 1, 1, cp, pn, pmax);
    tc_prepare_kernel<BF16>
        <<<static_cast<unsigned>((q + 7) / 8), 256, 0, stream>>>(queries, q, dim, l.dim_pad, l.split, 0, 1, cq, qn);
    BITSKNN_CUDA_TRY(cudaGetLastError());

    ftc_params p{};
    p.list_d = reinterpret_cast<float*>(ws + l.off_ld);
    p.list_x = reinterpret_cast<int32_t*>(ws + l.off_lx);
    p.n = n;
    p.q = q;
    p.nkb = l.nkb;
    p.nsteps = l.nsteps;
    p.hs = l.hs;
    p.parts = l.parts;
    p.tiles = (n + TILE_N - 1) / TILE_N;
    p.k = l.k_scan;
    p.index_base = index_base;
    p.qnorm = qn;
    p.max_norm = pmax;
    // split images: the dropped lo.lo products and the accumulation stay below 2^-16 (BF16) /
    // 2^-21 (TF32) of |x|^2 + |y|^2 in every measured case; four times that is allowed.  Plainly
    // rounded images (long vectors) carry the rounding of both inputs.
    p.slack = l.split != 0 ? (BF16 ? 0x1p-14F : 0x1p-19F) : (BF16 ? 0x1p-8F : 0x1p-11F);
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    // shared memory: query image + ring + barriers + radii + candidate buffers.  The MMA covers 256
    // points (two tiles, one per consumer group) when at least two of its 32 KiB stages fit beside
    // the query image, else 128 points.
    // 32 candidate slots per (group, query); 16 for long image rows (five or more 128-byte K blocks:
    // TF32 from dim 57, BF16 from dim 121), where the 32 KiB that frees -- two more 16 KiB stages --
    // buy more than the extra folds cost (q = 2^14, n = 2^20: TF32 dim 64 k = 16 14.6 -> 11.7 ms,
    // BF16 dim 128 k = 64 15.2 -> 13.0 ms; for shorter rows the ring is deep enough and the smaller
    // buffers only add folds: BF16 dim 64 k = 128 11.4 -> 13.1 ms)
    auto fixed_bytes = [](int cap) { return static_cast<size_t>(1024 + 64 * 8 + 4 * TILE_M * 4) + 2U * (8U * cap * 32U * 4U); };
    auto room_for = [&](int cap) { return static_cast<int>((227 * 1024 - fixed_bytes(cap)) / STAGE_BYTES) - p.nkb; };
    p.cap = CAP;
    if (const int forced = tuning_value("fused.tc_cap", 0); forced == 16 || forced == 32)
    {
        p.cap = forced;
    }
    else if (p.nkb >= 5)
    {
        p.cap = 16;
    }
    // folding fuller buffers means fewer folds (each sorts 32 slots whatever they hold) but a check of
    // the fill every 8 columns instead of every 16: worth it for the longer lists only (k = 128:
    // 11.5 -> 11.3 ms at dim 64, q = 2^14, n = 2^20; k = 16: 7.9 -> 8.0)
    p.fold_above = p.cap == 32 ? (k > 32 ? 24 : 16) : 8;
    if (const int forced = tuning_value("fused.tc_fold_above", 0); forced > 0 && (p.cap - forced == 8 || p.cap - forced == 16))
    {
        p.fold_above = forced;
    }
    const size_t fixed = fixed_bytes(p.cap);
    const int room128 = room_for(p.cap);
    if (room128 < 2)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (query image does not fit shared memory)", dim);
    }
    const int want_n = tuning_value("fused.tc_mma_n", 0);
    const bool wide = want_n == 128 ? false : room128 >= 4;
    const int nt = wide ? 2 : 1;
    p.stages = std::min(wide ? 4 : 8, room128 / nt);
    const size_t smem = fixed + (static_cast<size_t>(p.nkb) + static_cast<size_t>(p.stages) * nt) * STAGE_BYTES;

    CUtensorMap map_q;
    CUtensorMap map_p;
    if (const int rc = make_map(&map_q, cq, q, l.dim_pad, BF16); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (const int rc = make_map(&map_p, cp, n, l.dim_pad, BF16, wide ? 256U : 128U); rc != BITSKNN_OK)
    {
        return rc;
    }

    const int64_t nqb = (q + TILE_M - 1) / TILE_M;
    const int64_t grid = nqb * p.parts;
    int rc;
    switch (l.kl * nt)
    {
    case 32:
        rc = launch_ftc<BF16, 1, 128>(map_q, map_p, p, smem, grid, stream);
        break;
    case 64:
        rc = wide ? launch_ftc<BF16, 1, 256>(map_q, map_p, p, smem, grid, stream)
                  : launch_ftc<BF16, 2, 128>(map_q, map_p, p, smem, grid, stream);
        break;
    case 128:
        rc = wide ? launch_ftc<BF16, 2, 256>(map_q, map_p, p, smem, grid, stream)
                  : launch_ftc<BF16, 4, 128>(map_q, map_p, p, smem, grid, stream);
        break;
    case 256:
        rc = wide ? launch_ftc<BF16, 4, 256>(map_q, map_p, p, smem, grid, stream)
                  : launch_ftc<BF16, 8, 128>(map_q, map_p, p, smem, grid, stream);
        break;
    default:
        rc = launch_ftc<BF16, 8, 256>(map_q, map_p, p, smem, grid, stream);
        break;
    }
    if (rc != BITSKNN_OK)
    {
        return rc;
    }
    // The 2 * parts lists of every query hold its candidates ranked by tensor-core distances.  The
    // result is decided by the exact FP32 distance of every candidate (one FMA chain of (y - x)^2
    // per pair, as the FP32 path computes it), which is also the distance reported.
    return rerank_lists(p.list_x, static_cast<int64_t>(q) * l.kl, l.kl, q, 2 * l.parts, l.kl, k, points, queries, n, dim,
                        index_base, out_dist, out_idx, stream);
}

} // namespace

size_t fused_tc_workspace_bytes(int64_t n, int64_t q, int dim, int k, int mode)
{
    if (n <= 0 || q <= 0 || dim <= 0 || k <= 0)
    {
        return 0;
    }
    return ftc_layout_of(n, q, dim, k, mode == BITSKNN_L2_BF16).total;
}

int fused_tc_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int mode,
                    int32_t index_base, float* out_dist, int32_t* out_idx, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream)
{
    const bool bf16 = mode == BITSKNN_L2_BF16;
    const int max_dim = MAX_KB * (bf16 ? 64 : 32) - 3;
    if (dim > max_dim)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (fused tensor-core modes take up to %d)", dim,
                    max_dim);
    }
    const size_t need = fused_tc_workspace_bytes(n, q, dim, k, mode);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255U) != 0)
    {
        return fail(BITSKNN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) needed, %zu given", need,
                    workspace_bytes);
    }
    auto* ws = static_cast<unsigned char*>(workspace);
    return bf16 ? run_ftc<true>(points, queries, n, q, dim, k, index_base, out_dist, out_idx, ws, stream)
                : run_ftc<false>(points, queries, n, q, dim, k, index_base, out_dist, out_idx, ws, stream);
}

} // namespace bitsknn
