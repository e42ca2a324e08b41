// `bits-fused` on the tensor cores: the partial distance tile is produced by tcgen05.mma in
// tensor memory and consumed from there by the top-k -- no distance ever reaches HBM.
//
// The contraction runs over the compact split image of tc_host.cuh ([hi | lo | norm columns]; the
// MMA warp pairs the K steps: points.hi with queries.hi and queries.lo, points.lo with
// queries.hi, norm step with norm step), so an accumulator holds  s = x.y - |x|^2 / 2  and the
// partial distance is d = -2 s (= |x|^2 - 2 x.y, the quantity the reference's fused kernel ranks by,
// include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:622-630).  The consumer compares
// raw accumulators against  -bound / 2: one max-tree and one vote per 32 columns.
//
// Block = 608 threads on one SM, 128 queries (the TMEM lanes):
//   warp 16  TMA producer (query image once, point image K blocks through a ring of stages)
//   warps 17, 18  tcgen05.mma issue, each with its own accumulators (tc_pipeline.cuh; warp 17 also
//            allocates the tensor memory: 4 accumulators of 128 columns).  For image rows of two
//            or more K blocks an MMA covers 256 points and fills two neighbouring accumulators, one
//            per scanner group (NMMA = 256), whenever the ring fits; one-K-block rows and long
//            vectors take 128 points per MMA.
//   warps 0-7  scanners, two groups of four.  Group g takes every other 128-point tile (each
//            group alternates between two accumulators, so the MMAs run ahead of it); thread t of
//            a group is query 32 * (warp % 4) + t and reads its row with tcgen05.ld, 64 columns
//            per step.  A scanner only compares: a tree of maxima and one vote per 32 columns
//            against the query's threshold (-bound / 2).  It releases the accumulator when it has
//            looked at it and mails the chunks (32 columns) in which some lane saw something to
//            its helper, one message per tile (a ring of mailbox slots guarded by mbarriers).
//   warps 8-15  helpers, one per scanner, on the same tensor-memory lanes (same queries).  A
//            helper takes the flagged chunks out of tensor memory again, releases the accumulator
//            as soon as the last of them is in its registers, pushes every accumulator that passes
//            the current bound into the query's candidate buffer and folds full buffers into the
//            query's list.  Each (group, query) has a private 32-slot candidate buffer in shared
//            memory (no atomics: one writer) and a sorted list of KL = 32 * IPT pairs in the
//            workspace (HBM/L2), touched only when the buffer is folded: the warp sorts the 32
//            candidates with shuffles, takes the element-wise minimum against the list's last 32
//            entries and finishes with a bitonic merge (striped arrangement: entry e in lane
//            e % 32).  The acceptance bound of a query is the smallest of: its group's radius,
//            the partner group's radius, and the larger of the two lists' entries
//            ceil(k / 2) - 1 (the lists cover different points, so k pairs lie at or below it).
//            The helper publishes the threshold in shared memory; a scanner reads it once per
//            tile, and a stale value only costs a needless message.
//   Why two kinds of warps: with the pushes and folds inside the scanning warps, every tile waited
//   for the slowest of the eight warps (a push costs about a thousand clocks, a fold two to
//   three thousand, and nine tiles in ten had at least one), and the MMAs waited with it.
// After the scan the lists of every query (two, or 2 * parts where the database was cut into
// ranges) hold its candidates by tensor-core distance;
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

constexpr int FT_THREADS = 608;
constexpr int FT_HELPER_WARP = 8;    // warps 8-15: helper of scanner warp (warp - 8)
constexpr int FT_PRODUCER_WARP = 16;
constexpr int FT_MMA_WARP = 17;
constexpr int FT_MAIL_SLOTS = 16;    // chunks a scanner may be ahead of its helper
// mail from a scanner to its helper: (local tile << 4) | mask of the tile's four chunks to look at
constexpr uint32_t FT_MAIL_SCAN_DONE = 0xFFFFFFFFU;
constexpr int FT_ACCS = tcpipe::ACCS; // four 128-column accumulators: each scanner group owns two
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
    int parts;       // database ranges of the query tiles from full_blocks on
    int full_blocks; // leading query tiles that are scanned whole, one block each
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
    __shared__ uint64_t mail_full[8][FT_MAIL_SLOTS];  // scanner -> helper: slot holds a message
    __shared__ uint64_t mail_empty[8][FT_MAIL_SLOTS]; // helper -> scanner: slot may be reused
    __shared__ uint32_t mail_code[8][FT_MAIL_SLOTS];
    __shared__ float thr_s[2 * TILE_M];               // acceptance threshold per (group, query), kept by the helpers
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

    // the first full_blocks blocks scan the whole database for one query tile each; the others
    // share the remaining query tiles, `parts` database ranges per tile
    const bool whole = static_cast<int64_t>(blockIdx.x) < p.full_blocks;
    const int64_t tail_block = static_cast<int64_t>(blockIdx.x) - p.full_blocks;
    const int nparts = whole ? 1 : p.parts;
    const int64_t qb = whole ? static_cast<int64_t>(blockIdx.x) : p.full_blocks + tail_block / p.parts;
    const int part = whole ? 0 : static_cast<int>(tail_block % p.parts);
    // tiles of 128 points; a part is a whole number of MMAs (a tile beyond n holds no valid column)
    const int64_t per = ((p.tiles + nparts - 1) / nparts + NT - 1) / NT * NT;
    const int64_t tiles_up = (p.tiles + NT - 1) / NT * NT;
    const int64_t t_begin = part * per;
    const int64_t t_end = t_begin + per < tiles_up ? t_begin + per : tiles_up;

    if (tid == 0)
    {
        tcpipe::init_barriers(pipe, p.stages, 2 * TILE_M); // scanners and helpers both release an accumulator
    }
    if (tid < 8 * FT_MAIL_SLOTS)
    {
        ptx::mbar_init(&mail_full[0][0] + tid, 1);
        ptx::mbar_init(&mail_empty[0][0] + tid, 1);
    }
    if (tid < 2 * TILE_M)
    {
        rad[tid] = INFINITY;
        hlf[tid] = INFINITY;
        // a dead row (query beyond q) never accepts anything
        thr_s[tid] = qb * TILE_M + (tid & (TILE_M - 1)) < p.q ? -INFINITY : INFINITY;
    }
    ptx::mbar_init_fence();
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
    else if (warp < FT_HELPER_WARP)
    {
        // ---- scanner: looks at every accumulator once and tells its helper which chunks (32
        // columns) hold something at or above some lane's threshold.  It touches neither the
        // candidate buffers nor the lists, so its loop is short and its pace even.
        const int group = warp >> 2;
        const int w4 = warp & 3;
        const int qrow = w4 * 32 + lane; // query of this thread inside the tile
        const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
        uint64_t* my_full = mail_full[warp];
        uint64_t* my_empty = mail_empty[warp];
        uint32_t* my_code = mail_code[warp];
        int slot = 0;
        uint32_t mph = 0;
        // (lane 0 alone posts; a fresh barrier passes a wait on the opposite parity at once)
        auto post = [&](uint32_t code) {
            bool sent = true;
            if (lane == 0)
            {
                sent = ptx::mbar_wait_bounded_spin(&my_empty[slot], mph ^ 1U);
                my_code[slot] = code;
                tc::mbar_arrive(&my_full[slot]);
            }
            if (++slot == FT_MAIL_SLOTS)
            {
                slot = 0;
                mph ^= 1U;
            }
            return sent;
        };

        auto group_maxima = [](const uint32_t(&v)[16], float(&g)[4]) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                g[i] = fmaxf(max3(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2])),
                             __uint_as_float(v[4 * i + 3]));
            }
        };

        // this group's tiles are the local tiles lt = group, group + 2, ...; tile lt sits in
        // accumulator lt % 4, so the group alternates between its two accumulators
        int64_t lt = group;
        for (int64_t t = t_begin + group; t < t_end && ok; t += 2, lt += 2)
        {
            // the helper tightens the threshold as the lists fill; a stale one only sends it a
            // chunk it would not have needed
            const float thr = *reinterpret_cast<volatile float*>(&thr_s[group * TILE_M + qrow]);
            const int a = static_cast<int>(lt & (FT_ACCS - 1));
            // (made warp-uniform: the lanes poll independently)
            if (!__all_sync(FULL_MASK, ptx::mbar_wait_bounded_spin(&acc_full[tcpipe::acc_full_index<NMMA>(a)],
                                                                   static_cast<uint32_t>((lt >> 2) & 1))))
            {
                ok = false;
                break;
            }
            tc::fence_after_sync();
            const uint32_t acc_addr = tmem_base + lane_base + static_cast<uint32_t>(a * TILE_N);
            // 64 columns per step (two loads in flight, two independent trees of maxima, one vote per
            // 32 columns); the next step's loads are issued as soon as the maxima are taken
            uint32_t lo0[16];
            uint32_t hi0[16];
            uint32_t lo1[16];
            uint32_t hi1[16];
            uint32_t flagged = 0; // chunks of this tile that hold something for some lane
            tc::tmem_ld_32x32_halves(acc_addr, lo0, hi0);
            tc::tmem_ld_32x32_halves(acc_addr + 32U, lo1, hi1);
#pragma unroll 1
            for (int c = 0; c < TILE_N / 32; c += 2)
            {
                float g0_lo[4];
                float g0_hi[4];
                float g1_lo[4];
                float g1_hi[4];
                tc::tmem_ld_wait();
                group_maxima(lo0, g0_lo);
                group_maxima(hi0, g0_hi);
                group_maxima(lo1, g1_lo);
                group_maxima(hi1, g1_hi);
                const float mx0 = max3(max3(g0_lo[0], g0_lo[1], g0_lo[2]), max3(g0_hi[0], g0_hi[1], g0_hi[2]),
                                       fmaxf(g0_lo[3], g0_hi[3]));
                const float mx1 = max3(max3(g1_lo[0], g1_lo[1], g1_lo[2]), max3(g1_hi[0], g1_hi[1], g1_hi[2]),
                                       fmaxf(g1_lo[3], g1_hi[3]));
                if (c + 2 < TILE_N / 32)
                {
                    tc::tmem_ld_32x32_halves(acc_addr + static_cast<uint32_t>(c * 32 + 64), lo0, hi0);
                    tc::tmem_ld_32x32_halves(acc_addr + static_cast<uint32_t>(c * 32 + 96), lo1, hi1);
                }
                const bool any0 = __any_sync(FULL_MASK, mx0 >= thr);
                const bool any1 = __any_sync(FULL_MASK, mx1 >= thr);
                flagged |= (any0 ? 1U : 0U) << c;
                flagged |= (any1 ? 2U : 0U) << c;
            }
            // This thread's reads of the accumulator are over.  The helper releases it too, once it
            // has the last flagged chunk in registers; with nothing flagged it is not told about the
            // tile at all and the scanner arrives in its place.
            tc::fence_before_sync();
            if (flagged == 0)
            {
                tc::mbar_arrive(&acc_empty[a], 2U);
            }
            else
            {
                tc::mbar_arrive(&acc_empty[a]);
                const bool sent = post((static_cast<uint32_t>(lt) << 4) | flagged);
                if (!__shfl_sync(FULL_MASK, sent ? 1 : 0, 0))
                {
                    ok = false;
                }
            }
        }
        post(FT_MAIL_SCAN_DONE);
    }
    else if (warp < FT_PRODUCER_WARP)
    {
        // ---- helper of scanner warp (warp - 8): same queries (tensor-memory lanes), owns their
        // candidate buffers and lists.  Takes the chunks its scanner points at out of tensor memory
        // again, pushes what passes the current bound, folds full buffers, publishes the threshold.
        const int hw = warp - FT_HELPER_WARP;
        const int group = hw >> 2;
        const int w4 = hw & 3;
        const int qrow = w4 * 32 + lane;              // query of this thread inside the tile
        const int64_t gq = qb * TILE_M + qrow;        // global query
        const bool live = gq < p.q;
        float* my_buf_d = buf_d + hw * (cap * 32);    // slot s of lane l at [s * 32 + (l + s) % 32]
        int* my_buf_x = buf_x + hw * (cap * 32);
        const int64_t list_id = static_cast<int64_t>(part) * 2 + group;
        const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
        uint64_t* my_full = mail_full[hw];
        uint64_t* my_empty = mail_empty[hw];
        const uint32_t* my_code = mail_code[hw];

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

        // Column j (0..31) of the chunk held in lo / hi: a tree of bitwise selects on the bits of j
        // (registers cannot be indexed, and a copy of the chunk in local memory would cost more).
        auto column = [](const uint32_t(&lo)[16], const uint32_t(&hi)[16], int j) {
            auto pick = [](uint32_t a, uint32_t b, uint32_t mk) { return (a & mk) | (b & ~mk); };
            const uint32_t m4 = 0U - ((static_cast<uint32_t>(j) >> 4) & 1U);
            const uint32_t m3 = 0U - ((static_cast<uint32_t>(j) >> 3) & 1U);
            const uint32_t m2 = 0U - ((static_cast<uint32_t>(j) >> 2) & 1U);
            const uint32_t m1 = 0U - ((static_cast<uint32_t>(j) >> 1) & 1U);
            const uint32_t m0 = 0U - (static_cast<uint32_t>(j) & 1U);
            uint32_t v8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                v8[i] = pick(pick(hi[i + 8], lo[i + 8], m4), pick(hi[i], lo[i], m4), m3);
            }
            uint32_t v2[2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
            {
                v2[i] = pick(pick(v8[i + 6], v8[i + 2], m2), pick(v8[i + 4], v8[i], m2), m1);
            }
            return __uint_as_float(pick(v2[1], v2[0], m0));
        };

        // One chunk: 32 columns of this thread's row, starting at point col0.  Every lane marks its
        // columns at or above the threshold in a bit mask and pushes them one by one (the lanes
        // diverge).  A lane whose buffer is full waits for the fold that follows and goes on under
        // the tightened bound.
        auto take_chunk = [&](const uint32_t(&lo)[16], const uint32_t(&hi)[16], int64_t col0) {
            unsigned m = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j)
            {
                m |= (__uint_as_float(lo[j]) >= thr ? 1U : 0U) << j;
                m |= (__uint_as_float(hi[j]) >= thr ? 1U : 0U) << (16 + j);
            }
            if (p.n - col0 < 32)
            {
                // ragged end: the columns from n on hold no point
                m &= p.n <= col0 ? 0U : (1U << static_cast<int>(p.n - col0)) - 1U;
            }
            while (__any_sync(FULL_MASK, m != 0))
            {
                while (m != 0 && cnt < cap)
                {
                    const int j = __ffs(static_cast<int>(m)) - 1;
                    m &= m - 1;
                    const float s = column(lo, hi, j);
                    const float d = -2.0F * s;
                    const int idx = p.index_base + static_cast<int>(col0 + j);
                    if (s >= thr && pair_lt(d, idx, r_d, r_x))
                    {
                        my_buf_d[cnt * 32 + ((lane + cnt) & 31)] = d;
                        my_buf_x[cnt * 32 + ((lane + cnt) & 31)] = idx;
                        ++cnt;
                    }
                }
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
            }
        };

        int slot = 0;
        uint32_t mph = 0;
        while (ok)
        {
            if (!__all_sync(FULL_MASK, ptx::mbar_wait_bounded_spin(&my_full[slot], mph)))
            {
                ok = false;
                break;
            }
            const uint32_t code = my_code[slot];
            __syncwarp();
            if (lane == 0)
            {
                tc::mbar_arrive(&my_empty[slot]);
            }
            if (++slot == FT_MAIL_SLOTS)
            {
                slot = 0;
                mph ^= 1U;
            }
            if (code == FT_MAIL_SCAN_DONE)
            {
                break;
            }
            const int64_t lt = code >> 4;
            const int a = static_cast<int>(lt & (FT_ACCS - 1));
            uint32_t todo = code & 15U;
            tc::fence_after_sync();
            while (todo != 0)
            {
                const int c = __ffs(static_cast<int>(todo)) - 1;
                todo &= todo - 1;
                uint32_t lo[16];
                uint32_t hi[16];
                tc::tmem_ld_32x32_halves(tmem_base + lane_base + static_cast<uint32_t>(a * TILE_N + c * 32), lo, hi);
                if (live)
                {
                    thr = fmaxf(thr, -0.5F * bound()); // the partner group may have tightened it
                }
                tc::tmem_ld_wait();
                if (todo == 0)
                {
                    // the last chunk wanted from this accumulator is in registers
                    tc::fence_before_sync();
                    tc::mbar_arrive(&acc_empty[a]);
                }
                take_chunk(lo, hi, (t_begin + lt) * TILE_N + c * 32);
            }
            thr_s[group * TILE_M + qrow] = thr;
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
    int parts;       // database ranges per query tile from full_blocks on
    int full_blocks; // leading query tiles scanned whole
    int k_scan;  // list position of the radius during the scan: k plus a margin, at most kl
    size_t off_pn, off_qn, off_max, off_p, off_q, off_ld, off_lx, total;
};

ftc_layout ftc_layout_of(int64_t n, int64_t q, int dim, int k, bool bf16)
{
    ftc_layout l{};
    // TF32 from 32 dimensions on: the plainly rounded image (one product per K step instead of the
    // split image's three).  Its distances are off by up to 2^-11 of |x|^2 + |y|^2; the acceptance
    // bound allows for that, the lists keep a margin and the exact re-ranking decides, and at these
    // dimensions few enough points lie that close to the k-th distance: recall 1.0 and no error of
    // the k-th distance in the quality tests at dim 32 and 64, uniform and clustered (q = 2^14,
    // n = 2^20: dim 64, k = 16 11.3 -> 7.7 ms; dim 32 7.7 -> 6.5 ms).  At lower dimensions too many
    // points lie within the allowance (dim 16, tight clusters: the stated bounds are missed; dim 4:
    // k-th distance off by 4 %), and a BF16 image rounded plainly (2^-8) is too coarse at every
    // dimension: both keep the split.
    const int want_plain = tuning_value("fused.tc_tf32_plain", 0);
    const bool plain = !bf16 && (want_plain == 1 || (want_plain == 0 && dim >= 32));
    const tcpipe::image_shape img = tcpipe::image_shape_of(dim, bf16, true, plain);
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
    // Blocks run in waves of one per SM.  A block's time is its share of the scan plus the work of
    // bringing its lists' radii down, which hardly shrinks with the range it scans (measured at
    // q = 2^16, n = 2^20 with one and two ranges: that work is about 0.3 of a full scan for k <= 32
    // and 0.45 above).  So: as many whole waves of query tiles as there are scan the database whole,
    // one block per tile, and the query tiles that are left over -- all of them when there are fewer
    // tiles than SMs -- are cut into database ranges (of at least 64 tiles), as many as make
    // waves x block time smallest (q = 8192: 64 tiles, two ranges, one wave of 128 blocks: 5.3 ms at
    // dim 32, k = 64, against 7.8 ms with three ranges; q = 2^16: 444 tiles whole in three waves and
    // 68 tiles in two ranges in a fourth, shorter one).
    const int sms = device_sm_count();
    const double fixed_work = k > 32 ? 0.45 : 0.3;
    const int64_t max_parts = std::max<int64_t>(1, std::min<int64_t>(tiles / 64, 4 * sms));
    l.full_blocks = static_cast<int>(nqb / sms * sms);
    const int64_t rest = nqb - l.full_blocks;
    l.parts = 1;
    if (rest > 0)
    {
        double best = 0.0;
        for (int64_t parts = 1; parts <= max_parts; ++parts)
        {
            const double waves = static_cast<double>((rest * parts + sms - 1) / sms);
            const double cost = waves * (1.0 / static_cast<double>(parts) + fixed_work);
            if (parts == 1 || cost < best * 0.98)
            {
                best = cost;
                l.parts = static_cast<int>(parts);
            }
            if (rest * parts >= 4 * static_cast<int64_t>(sms))
            {
                break;
            }
        }
    }
    if (const int forced = tuning_value("fused.parts", 0); forced > 0)
    {
        // a forced count applies to every query tile
        l.full_blocks = 0;
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
    p.full_blocks = l.full_blocks;
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
    // points (two tiles, one per scanner group) when at least two of its 32 KiB stages fit beside
    // the query image, else 128 points.
    // 32 candidate slots per (group, query); 16 for long image rows (five or more 128-byte K blocks:
    // TF32 from dim 57, BF16 from dim 121), where the 32 KiB that frees -- two more 16 KiB stages --
    // buy more than the extra folds cost (q = 2^14, n = 2^20: TF32 dim 64 k = 16 14.6 -> 11.7 ms,
    // BF16 dim 128 k = 64 15.2 -> 13.0 ms; for shorter rows the ring is deep enough and the smaller
    // buffers only add folds: BF16 dim 64 k = 128 11.4 -> 13.1 ms)
    auto fixed_bytes = [](int cap) { return static_cast<size_t>(1024 + 64 * 8 + 4 * TILE_M * 4) + 2U * (8U * cap * 32U * 4U); };
    // (the kernel's static shared memory -- descriptor tables, mailboxes, thresholds -- is 4.5 KiB)
    auto room_for = [&](int cap) { return static_cast<int>((227 * 1024 - 4608 - fixed_bytes(cap)) / STAGE_BYTES) - p.nkb; };
    p.cap = CAP;
    if (const int forced = tuning_value("fused.tc_cap", 0); forced == 16 || forced == 32)
    {
        p.cap = forced;
    }
    else if (p.nkb >= 5)
    {
        p.cap = 16;
    }
    // folding fuller buffers means fewer folds (each sorts 32 slots whatever they hold) but a later
    // radius: worth it for the longer lists only (q = 2^14, n = 2^20, dim 64: k = 128 folds above
    // 16 / 24 / 28: 11.96 / 11.52 / 11.40 ms; k = 16: 7.66 / 7.71 / 7.74)
    p.fold_above = p.cap == 32 ? (k > 64 ? 28 : (k > 32 ? 24 : 16)) : 8;
    if (const int forced = tuning_value("fused.tc_fold_above", 0); forced > 0 && forced < p.cap)
    {
        p.fold_above = forced;
    }
    const size_t fixed = fixed_bytes(p.cap);
    const int room128 = room_for(p.cap);
    if (room128 < 2)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (query image does not fit shared memory)", dim);
    }
    // One-K-block rows (BF16 up to dim 16, TF32 up to dim 8) are bound by the round trip of an
    // accumulator, not by the MMAs: there 128-point MMAs, which hand every accumulator over by
    // itself and sooner, are 2-4 % faster (q = 2^14, n = 2^20, dim 16: k = 16 5.39 -> 5.18 ms, k = 128
    // 9.17 -> 8.77 ms); from two K blocks on the 256-point MMAs win (dim 32: 6.50 against 6.79 ms).
    const int want_n = tuning_value("fused.tc_mma_n", 0);
    const bool wide = want_n == 128 ? false : (want_n == 256 || p.nkb >= 2) && room128 >= 4;
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
    const int64_t grid = l.full_blocks + (nqb - l.full_blocks) * p.parts;
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
    // (the queries of the tiles scanned whole have two lists each, the others 2 * parts)
    const int64_t q_whole = std::min<int64_t>(q, static_cast<int64_t>(l.full_blocks) * TILE_M);
    const int64_t list_stride = static_cast<int64_t>(q) * l.kl;
    if (q_whole > 0)
    {
        if (const int rc2 = rerank_lists(p.list_x, list_stride, l.kl, q_whole, 2, l.kl, k, points, queries, n, dim, index_base,
                                         out_dist, out_idx, stream);
            rc2 != BITSKNN_OK)
        {
            return rc2;
        }
    }
    if (q_whole < q)
    {
        return rerank_lists(p.list_x + q_whole * l.kl, list_stride, l.kl, q - q_whole, 2 * l.parts, l.kl, k, points,
                            queries + q_whole * dim, n, dim, index_base, out_dist + q_whole * k, out_idx + q_whole * k, stream);
    }
    return BITSKNN_OK;
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
