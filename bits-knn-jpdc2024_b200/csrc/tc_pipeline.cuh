// The operand pipeline shared by the tensor-core kernels (distance matrix in l2_tc.cu, fused
// search in fused_tc.cu): one TMA producer thread and two MMA-issuing threads around
//   * the query image of the block, resident in shared memory (nkb K blocks of 16 KiB),
//   * a ring of stages, each one K block of NMMA points (128-byte rows, 128-byte swizzle),
//   * four 128-column accumulators in tensor memory.  Tile lt (128 points) of the block's range
//     goes to accumulator lt % 4, used for the (lt / 4)-th time; the readers of the accumulators
//     arrive on acc_empty (128 arrivals, or as many as the kernel says) when they have taken a tile out.
// One MMA covers NMMA = 128 or 256 points; a 256-point MMA fills two neighbouring accumulators
// and reports both on the barrier of the first (acc_full_index).
//
// The tensor pipe runs a 128 x 256 x 16 MMA in 128 clocks (128 x 128 x 16: 73), and it holds the
// issuing thread for that long: whatever the thread does between two MMAs -- barrier waits,
// commits (about 95 clocks each), descriptor arithmetic -- is added to the MMA time instead of
// being covered by it (4096 back-to-back MMAs: 128 clocks each; with a commit after every fourth:
// 258; the same from two threads that issue side by side: 129).  So two threads issue, and
// nothing makes one wait for the other: unit u (one MMA's worth of points) belongs to thread
// u % 2, which has its own accumulators ((2 u) % 4 and the next for 256-point MMAs, u % 4 for
// 128-point ones) and its own "stage full" barriers.  The ring itself is shared and filled in
// unit order; a stage has one full barrier per issuing thread (the producer signals the one of
// the unit's thread), so that each thread sees every phase of the barriers it waits on -- a
// parity wait on a barrier whose earlier phases the thread has not watched could pass early.
//
// Images (tc_host.cuh): plain (hs == 0: step st of the points meets step st of the queries) or
// compact split ([hi (hs steps) | lo (hs steps) | optional norm step]: a hi step of the points
// meets the queries' hi and lo steps, a lo step the queries' hi step, the norm step its twin).
// Every wait is bounded; a role that gives up returns false and the kernel reports it.
#pragma once

#include <cstdint>

#include "common.cuh"
#include "ptx.cuh"
#include "tc.cuh"
#include "tc_host.cuh"

namespace bitsknn::tcpipe
{

constexpr int ACCS = 4;           // 128-column accumulators in tensor memory
constexpr int TMEM_COLS = 512;
constexpr int K_STEP_BYTES = 32;  // one MMA consumes 32 bytes of K (8 TF32 / 16 BF16)
constexpr int MAX_STAGES = 8;

struct shape
{
    int nkb;    // 128-byte K blocks per row of the images
    int nsteps; // MMA K steps (32 bytes) per row that hold data
    int hs;     // steps of the hi part of a compact split image (0: plain image)
    int stages; // ring stages (at most MAX_STAGES)
};

// Barriers and buffers of one block, all in shared memory.
struct state
{
    unsigned char* a_tiles; // nkb x 16 KiB, 1024-byte aligned
    unsigned char* b_ring;  // stages x (NMMA / 128) x 16 KiB
    uint64_t* a_full;
    uint64_t* full_b;       // [2][MAX_STAGES]: per issuing thread
    uint64_t* empty_b;      // [stages]
    uint64_t* acc_full;     // [ACCS]
    uint64_t* acc_empty;    // [ACCS]
    uint2* a_tab;           // [2][MAX_KB * 4]: descriptor table of each issuing thread
};

// Barrier that reports tile accumulator `a` full: a 256-point MMA reports its two accumulators on
// the barrier of the first.
template <int NMMA>
__device__ __forceinline__ int acc_full_index(int a)
{
    return NMMA == 2 * TILE_N ? (a & ~1) : a;
}

// Number of 64-bit barrier words `carve` lays out (a_full, 16 full, 16 empty, 2 x ACCS).
constexpr int BARRIER_WORDS = 1 + 16 + 16 + 2 * ACCS;

__device__ __forceinline__ void init_barriers(const state& st, int stages, int acc_readers = 128)
{
    ptx::mbar_init(st.a_full, 1);
    for (int s = 0; s < stages; ++s)
    {
        ptx::mbar_init(&st.full_b[s], 1);
        ptx::mbar_init(&st.full_b[MAX_STAGES + s], 1);
        ptx::mbar_init(&st.empty_b[s], 1);
    }
    for (int a = 0; a < ACCS; ++a)
    {
        ptx::mbar_init(&st.acc_full[a], 1);
        ptx::mbar_init(&st.acc_empty[a], acc_readers);
    }
    ptx::mbar_init_fence();
}

// TMA producer (one thread): the query tile once, then the K blocks of the point tiles
// [t_begin, t_end) in order (t in units of 128 points, NMMA points per load).
template <bool BF16, int NMMA>
__device__ __forceinline__ bool producer(const state& st, const shape& sh, const CUtensorMap* map_q,
                                         const CUtensorMap* map_p, int64_t query_row, int64_t t_begin, int64_t t_end)
{
    constexpr int KB_ELEMS = BF16 ? 64 : 32;
    constexpr int NT = NMMA / TILE_N;
    constexpr int STAGE_B = NT * STAGE_BYTES;
    ptx::mbar_expect_tx(st.a_full, static_cast<uint32_t>(sh.nkb) * STAGE_BYTES);
    for (int kb = 0; kb < sh.nkb; ++kb)
    {
        tc::tma_load_2d(st.a_tiles + static_cast<size_t>(kb) * STAGE_BYTES, map_q, kb * KB_ELEMS,
                        static_cast<int>(query_row), st.a_full);
    }
    int s = 0;
    uint32_t ph = 0;
    int issuer = 0;
    for (int64_t t = t_begin; t < t_end; t += NT, issuer ^= 1)
    {
        for (int kb = 0; kb < sh.nkb; ++kb)
        {
            // a fresh barrier passes a wait on the opposite parity at once
            if (!ptx::mbar_wait_bounded_spin(&st.empty_b[s], ph ^ 1U))
            {
                return false;
            }
            uint64_t* full = &st.full_b[issuer * MAX_STAGES + s];
            ptx::mbar_expect_tx(full, STAGE_B);
            tc::tma_load_2d(st.b_ring + static_cast<size_t>(s) * STAGE_B, map_p, kb * KB_ELEMS, static_cast<int>(t * TILE_N),
                            full);
            if (++s == sh.stages)
            {
                s = 0;
                ph ^= 1U;
            }
        }
    }
    return true;
}

// One of the two MMA-issuing threads (issuer = 0 or 1): takes every other unit of the block's
// range, waits for its accumulators and its stages, issues, commits.
template <bool BF16, int NMMA>
__device__ __forceinline__ bool mma_issuer(const state& st, const shape& sh, uint32_t tmem_base, int issuer,
                                           int64_t t_begin, int64_t t_end)
{
    constexpr int NT = NMMA / TILE_N;
    constexpr int STAGE_B = NT * STAGE_BYTES;
    constexpr uint32_t idesc = tc::instr_desc(BF16 ? 1U : 2U, TILE_M, NMMA);
    uint2* a_tab = st.a_tab + issuer * (MAX_KB * 4);
    // Low descriptor words of the query steps that meet step s of the point image (0: none).
    const uint64_t a_desc0 = tc::smem_desc_sw128(st.a_tiles);
    const uint32_t desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
    auto a_step = [&](int s) {
        return static_cast<uint32_t>(a_desc0) + static_cast<uint32_t>(s >> 2) * (STAGE_BYTES >> 4) +
               static_cast<uint32_t>((s & 3) * (K_STEP_BYTES >> 4));
    };
    for (int s = 0; s < MAX_KB * 4; ++s)
    {
        uint2 e = make_uint2(0U, 0U);
        if (s < sh.nsteps)
        {
            if (sh.hs == 0 || s >= 2 * sh.hs)
            {
                e.x = a_step(s);
            }
            else if (s < sh.hs)
            {
                e.x = a_step(s);
                e.y = a_step(sh.hs + s);
            }
            else
            {
                e.x = a_step(s - sh.hs);
            }
        }
        a_tab[s] = e;
    }
    if (!ptx::mbar_wait_bounded_spin(st.a_full, 0))
    {
        return false;
    }
    const uint32_t b_lo0 = static_cast<uint32_t>(tc::smem_desc_sw128(st.b_ring));
    uint64_t* full_b = st.full_b + issuer * MAX_STAGES;
    // ring position of this thread's first unit; `seen` holds, per stage, the parity of the next
    // phase of this thread's full barrier
    int s = (issuer * sh.nkb) % sh.stages;
    uint32_t seen = 0;
    int64_t lt = static_cast<int64_t>(issuer) * NT;
    for (int64_t t = t_begin + issuer * NT; t < t_end; t += 2 * NT, lt += 2 * NT)
    {
        const int a = static_cast<int>(lt & (ACCS - 1));
        const uint32_t aph = static_cast<uint32_t>((lt >> 2) & 1);
        if (!ptx::mbar_wait_bounded_spin(&st.acc_empty[a], aph ^ 1U) ||
            (NT == 2 && !ptx::mbar_wait_bounded_spin(&st.acc_empty[a + 1], aph ^ 1U)))
        {
            return false;
        }
        tc::fence_after_sync();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(a * TILE_N);
        for (int kb = 0; kb < sh.nkb; ++kb)
        {
            // the one or two query steps that meet each of the four steps of this K block
            // (read before the wait: the MMA statements below order memory accesses)
            uint2 a_words[4];
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
            {
                a_words[ks] = a_tab[kb * 4 + ks];
            }
            if (!ptx::mbar_wait_bounded_spin(&full_b[s], (seen >> s) & 1U))
            {
                return false;
            }
            seen ^= 1U << s;
            tc::fence_after_sync();
            const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(s) * (STAGE_B >> 4);
#pragma unroll
            for (int ks = 0; ks < 128 / K_STEP_BYTES; ++ks)
            {
                const uint2 a_lo = a_words[ks];
                const uint32_t b_st = b_lo + static_cast<uint32_t>(ks * (K_STEP_BYTES >> 4));
                tc::mma_words<BF16>(acc, a_lo.x, b_st, desc_hi, idesc, (kb | ks) != 0 ? 1U : 0U, a_lo.x);
                tc::mma_words<BF16>(acc, a_lo.y, b_st, desc_hi, idesc, 1U, a_lo.y);
            }
            tc::mma_commit(&st.empty_b[s]); // the stage is free once these MMAs have read it
            if (++s == sh.stages)
            {
                s = 0;
            }
        }
        tc::mma_commit(&st.acc_full[a]);
        // step over the other thread's unit
        s = (s + sh.nkb) % sh.stages;
    }
    return true;
}

// Image shape for a row of `dim` coordinates: compact split when it fits the resident query
// tile, else the plainly rounded row.  `norm_cols`: three more columns (tc_host.cuh).
struct image_shape
{
    int dim_pad; // row pitch of the images in elements
    int split;   // image kind for the pre-pass (2: compact split, 0: plain)
    int hs;
    int nsteps;
    int nkb;
};

inline image_shape image_shape_of(int dim, bool bf16, bool norm_cols, bool plain = false)
{
    image_shape l{};
    const int unit = bf16 ? 64 : 32; // elements per 128-byte K block
    const int step = unit / 4;       // elements per MMA K step
    const int dp = (dim + step - 1) / step * step;
    const int extra = norm_cols ? 1 : 0;
    if (!plain && 2 * (dp / step) + extra <= MAX_KB * 4)
    {
        // compact split image: [hi (dp) | lo (dp) | norm columns, padded to one step]
        l.split = 2;
        l.hs = dp / step;
        l.nsteps = 2 * l.hs + extra;
        l.dim_pad = 2 * dp + extra * step;
    }
    else
    {
        // plain image: [row | norm columns], padded to whole K steps (the part of the last K block
        // beyond the row is filled with zeros by the TMA unit and costs neither traffic nor MMAs)
        l.split = 0;
        l.hs = 0;
        l.nsteps = (dim + 3 * extra + step - 1) / step;
        l.dim_pad = l.nsteps * step;
    }
    l.nkb = (l.nsteps + 3) / 4;
    return l;
}

} // namespace bitsknn::tcpipe
