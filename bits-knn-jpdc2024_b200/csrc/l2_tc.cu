// Squared-L2 distance matrix on the 5th-generation tensor cores (tcgen05), TF32 / BF16 inputs,
// FP32 accumulation in tensor memory:  dist = |x|^2 + |y|^2 - 2 x.y.
//
// This is the only dense contraction of the engine (the role of the reference's
// abstract_gemm<partial_l2_ops>, include/bits/distance/abstract_gemm.cuh:139-169,494-714, and
// of its tensor-core experiment fused_tc_kernel.cuh:109-158,346,440: a pre-pass that converts
// the inputs and computes the norms, then `fmaf(-2, dot, |x|^2) + |y|^2`).
//
//   pre-pass   rounds the inputs to the MMA input type (round-to-nearest) into an image in the
//              caller's workspace and writes the FP32 norms of the ORIGINAL vectors; whenever it
//              fits the resident query tile (dim <= 128 TF32 / 256 BF16) the image is the compact
//              hi/lo split of tc_host.cuh, which compensates the input rounding and is what keeps
//              recall@k >= 0.999 against the FP32 path
//   main       352 threads per block, one block per SM:
//              warp 8      TMA producer: query tile once, then point tiles through a ring
//              warps 9, 10 tcgen05.mma issue, each with its own accumulators (tc_pipeline.cuh), M = 128 queries,
//                          N = 256 points (two accumulators at once) or 128, K = 8 TF32 / 16 BF16
//                          per instruction; warp 9 allocates the 512 TMEM columns
//              warps 0-7   epilogue, two groups of four: group g drains every other 128-point
//                      tile with tcgen05.ld 32 lanes x 32 columns, transposes
//                      through a shared-memory staging tile so that every 128-byte row segment
//                      is written by 8 lanes, adds the norms, streaming 128-bit stores; each group
//                      alternates between two accumulators, so the MMAs run ahead of it
// Every mbarrier wait is bounded; on expiry the role stops, the block reaches its final barrier,
// frees its TMEM and sets the device status word.
#include <algorithm>
#include <cstdint>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tc.cuh"
#include "tc_host.cuh"
#include "tc_pipeline.cuh"

namespace bitsknn
{

namespace
{

constexpr int TC_THREADS = 352;     // 8 epilogue warps + TMA producer warp + two MMA warps
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int ACCS = tcpipe::ACCS;  // four 128-column accumulators: each epilogue group owns two
constexpr int STAGE_LD = 36;       // row stride (floats) of the epilogue staging tiles

struct tc_params
{
    const float* qn; // [q] query norms
    const float* pn; // [n] point norms
    float* out;
    int64_t ld;
    int64_t n;
    int64_t q;
    int nkb;      // K blocks per tile
    int nsteps;   // MMA K steps per row that hold data
    int hs;       // steps of the hi part of the compact split image (0: plain image)
    int stages;   // ring stages
    int parts;    // blocks per query tile
    int64_t tiles; // point tiles
    int* status;
};

template <bool BF16, int NMMA>
__global__ void __launch_bounds__(TC_THREADS, 1)
    l2_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_p, const tc_params p)
{
    constexpr int NT = NMMA / TILE_N;            // 128-column tiles per MMA (1 or 2)
    constexpr int STAGE_B = NT * STAGE_BYTES;    // one K block of NMMA points
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint2 a_tab_both[2][MAX_KB * 4]; // one descriptor table per MMA-issuing thread
    tcpipe::state pipe;
    pipe.a_tiles = smem;                                                            // nkb x 16 KiB
    pipe.b_ring = pipe.a_tiles + static_cast<size_t>(p.nkb) * STAGE_BYTES;          // stages x STAGE_B
    uint64_t* bars = reinterpret_cast<uint64_t*>(pipe.b_ring + static_cast<size_t>(p.stages) * STAGE_B);
    pipe.a_full = bars;
    pipe.full_b = bars + 1;
    pipe.empty_b = pipe.full_b + 16;
    pipe.acc_full = pipe.empty_b + 16;
    pipe.acc_empty = pipe.acc_full + ACCS;
    pipe.a_tab = &a_tab_both[0][0];
    uint64_t* acc_full = pipe.acc_full;
    uint64_t* acc_empty = pipe.acc_empty;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pipe.acc_empty + ACCS);
    float* staging = reinterpret_cast<float*>(bars + 64); // 8 warps x 32 rows x STAGE_LD floats
    const tcpipe::shape shape{p.nkb, p.nsteps, p.hs, p.stages};

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int64_t qb = blockIdx.x / p.parts;
    const int part = static_cast<int>(blockIdx.x - qb * p.parts);
    // tiles of 128 points; a part is a whole number of MMAs (a tile beyond n stores nothing)
    const int64_t per = ((p.tiles + p.parts - 1) / p.parts + NT - 1) / NT * NT;
    const int64_t tiles_up = (p.tiles + NT - 1) / NT * NT;
    const int64_t t_begin = part * per;
    const int64_t t_end = t_begin + per < tiles_up ? t_begin + per : tiles_up;

    if (tid == 0)
    {
        tcpipe::init_barriers(pipe, p.stages);
    }
    if (warp == MMA_WARP)
    {
        tc::tmem_alloc(tmem_slot, tcpipe::TMEM_COLS);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == PRODUCER_WARP)
    {
        if (lane == 0 && t_begin < t_end)
        {
            ok = tcpipe::producer<BF16, NMMA>(pipe, shape, &map_q, &map_p, qb * TILE_M, t_begin, t_end);
        }
    }
    else if (warp == MMA_WARP || warp == MMA_WARP + 1)
    {
        if (lane == 0 && t_begin < t_end)
        {
            ok = tcpipe::mma_issuer<BF16, NMMA>(pipe, shape, tmem_base, warp - MMA_WARP, t_begin, t_end);
        }
    }
    else
    {
        // epilogue: two groups of four warps; group g drains accumulator buffer g, i.e. every
        // other tile.  Warp w of a group owns TMEM lanes 32 * w .. + 31 = 32 query rows.
        const int group = warp >> 2;
        const int w4 = warp & 3;
        const bool vec_out = (p.ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15U) == 0);
        float* stage = staging + warp * (32 * STAGE_LD);
        // after the transposition through `stage`, lane l writes the column quad (l & 7) * 4 of
        // rows 4 * i + (l >> 3), i = 0..7: their query norms stay in registers
        const int sub = lane >> 3;
        const int cq4 = (lane & 7) * 4;
        float qn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const int64_t r = qb * TILE_M + w4 * 32 + i * 4 + sub;
            qn[i] = r < p.q ? __ldg(p.qn + r) : 0.0F;
        }
        const uint32_t lane_row = static_cast<uint32_t>(w4 * 32) << 16;
        int64_t lt = group; // this group's tiles are the local tiles group, group + 2, ...
        for (int64_t t = t_begin + group; t < t_end && ok; t += 2, lt += 2)
        {
            // point norms of this lane's four column quads, fetched before the wait so that their
            // latency hides behind it
            float pn_all[TILE_N / 32][4];
#pragma unroll
            for (int c = 0; c < TILE_N / 32; ++c)
            {
                const int64_t col = t * TILE_N + c * 32 + cq4;
                if (col + 3 < p.n)
                {
                    const float4 t4 = __ldg(reinterpret_cast<const float4*>(p.pn + col));
                    pn_all[c][0] = t4.x;
                    pn_all[c][1] = t4.y;
                    pn_all[c][2] = t4.z;
                    pn_all[c][3] = t4.w;
                }
                else
                {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                    {
                        pn_all[c][e] = col + e < p.n ? __ldg(p.pn + col + e) : 0.0F;
                    }
                }
            }
            // (made warp-uniform: the lanes poll independently)
            const int a = static_cast<int>(lt & (ACCS - 1));
            const uint32_t lane_base = lane_row + static_cast<uint32_t>(a * TILE_N);
            if (!__all_sync(FULL_MASK, ptx::mbar_wait_bounded_spin(&acc_full[tcpipe::acc_full_index<NMMA>(a)], static_cast<uint32_t>((lt >> 2) & 1))))
            {
                ok = false;
                break;
            }
            tc::fence_after_sync();
            uint32_t v[32];
            tc::tmem_ld_32x32(tmem_base + lane_base, v);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < TILE_N / 32; ++c)
            {
                // raw accumulators of this thread's row -> staging tile (row stride 36 floats:
                // conflict-free 128-bit writes and reads)
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                {
                    *reinterpret_cast<uint4*>(stage + lane * STAGE_LD + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
                // the next 32 columns travel from TMEM while this chunk is finished and stored
                if (c + 1 < TILE_N / 32)
                {
                    tc::tmem_ld_32x32(tmem_base + lane_base + static_cast<uint32_t>((c + 1) * 32), v);
                }
                __syncwarp();
                const int64_t col = t * TILE_N + c * 32 + cq4;
                const float(&pn4)[4] = pn_all[c];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    const int rr = i * 4 + sub;
                    const int64_t orow = qb * TILE_M + w4 * 32 + rr;
                    const float4 acc = *reinterpret_cast<const float4*>(stage + rr * STAGE_LD + cq4);
                    float4 r;
                    r.x = fmaf(-2.0F, acc.x, pn4[0]) + qn[i];
                    r.y = fmaf(-2.0F, acc.y, pn4[1]) + qn[i];
                    r.z = fmaf(-2.0F, acc.z, pn4[2]) + qn[i];
                    r.w = fmaf(-2.0F, acc.w, pn4[3]) + qn[i];
                    if (orow < p.q)
                    {
                        float* dst = p.out + orow * p.ld + col;
                        if (vec_out && col + 3 < p.n)
                        {
                            __stcs(reinterpret_cast<float4*>(dst), r);
                        }
                        else
                        {
                            const float e4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                            {
                                if (col + e < p.n)
                                {
                                    __stcs(dst + e, e4[e]);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (c + 1 < TILE_N / 32)
                {
                    tc::tmem_ld_wait();
                }
                else
                {
                    // every accumulator of this thread has been read: the MMA warp may reuse the buffer
                    tc::fence_before_sync();
                    tc::mbar_arrive(&acc_empty[a]);
                }
            }
        }
    }

    if (!ok)
    {
        atomicOr(p.status, DEVICE_STATUS_TIMEOUT);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP)
    {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, tcpipe::TMEM_COLS);
    }
}

struct tc_layout
{
    tcpipe::image_shape img;
    size_t off_pn, off_qn, off_p, off_q, total;
};

tc_layout layout_of(int64_t n, int64_t q, int dim, bool bf16)
{
    tc_layout l{};
    l.img = tcpipe::image_shape_of(dim, bf16, false);
    const size_t esz = bf16 ? 2 : 4;
    l.off_pn = 0;
    l.off_qn = align256(static_cast<size_t>(n) * 4);
    l.off_p = l.off_qn + align256(static_cast<size_t>(q) * 4);
    l.off_q = l.off_p + align256(static_cast<size_t>(n) * l.img.dim_pad * esz);
    l.total = l.off_q + align256(static_cast<size_t>(q) * l.img.dim_pad * esz);
    return l;
}

template <bool BF16, int NMMA>
int launch_tc(const CUtensorMap& map_q, const CUtensorMap& map_p, const tc_params& p, size_t smem, int64_t grid,
              cudaStream_t stream)
{
    auto kernel = l2_tc_kernel<BF16, NMMA>;
    BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    {
        kernel_scope timed{"l2_tc_kernel", stream};
        kernel<<<static_cast<unsigned>(grid), TC_THREADS, smem, stream>>>(map_q, map_p, p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

template <bool BF16>
int run_tc(const float* points, const float* queries, int64_t n, int64_t q, int dim, float* dist, int64_t ld,
           unsigned char* ws, cudaStream_t stream)
{
    const tc_layout l = layout_of(n, q, dim, BF16);
    float* pn = reinterpret_cast<float*>(ws + l.off_pn);
    float* qn = reinterpret_cast<float*>(ws + l.off_qn);
    void* cp = ws + l.off_p;
    void* cq = ws + l.off_q;
    tc_prepare_kernel<BF16>
        <<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(points, n, dim, l.img.dim_pad, l.img.split, 1, 0, cp, pn);
    tc_prepare_kernel<BF16>
        <<<static_cast<unsigned>((q + 7) / 8), 256, 0, stream>>>(queries, q, dim, l.img.dim_pad, l.img.split, 0, 0, cq, qn);
    BITSKNN_CUDA_TRY(cudaGetLastError());

    tc_params p{};
    p.qn = qn;
    p.pn = pn;
    p.out = dist;
    p.ld = ld;
    p.n = n;
    p.q = q;
    p.nkb = l.img.nkb;
    p.nsteps = l.img.nsteps;
    p.hs = l.img.hs;
    p.tiles = (n + TILE_N - 1) / TILE_N;
    const int64_t nqb = (q + TILE_M - 1) / TILE_M;
    const int sms = device_sm_count();
    // blocks per query tile: ranges of at least 64 point tiles, last wave of blocks (one per SM) nearly full
    p.parts = balanced_parts(nqb, sms, std::min<int64_t>(p.tiles / 64, 64));
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    // shared memory: query image + ring + barriers + staging tiles.  An MMA covers 256 points when
    // at least two of its 32 KiB stages fit beside the query image, else 128 points.
    const size_t fixed = 1024 + 64 * 8 + 8 * 32 * STAGE_LD * 4;
    const int room128 = static_cast<int>((227 * 1024 - fixed) / STAGE_BYTES) - p.nkb;
    if (room128 < 2)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (query image does not fit shared memory)", dim);
    }
    const bool wide = tuning_value("fused.tc_mma_n", 0) == 128 ? false : room128 >= 4;
    const int nt = wide ? 2 : 1;
    p.stages = std::min(wide ? 4 : 8, room128 / nt);
    const size_t smem = fixed + (static_cast<size_t>(p.nkb) + static_cast<size_t>(p.stages) * nt) * STAGE_BYTES;

    CUtensorMap map_q;
    CUtensorMap map_p;
    if (const int rc = make_map(&map_q, cq, q, l.img.dim_pad, BF16); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (const int rc = make_map(&map_p, cp, n, l.img.dim_pad, BF16, wide ? 256U : 128U); rc != BITSKNN_OK)
    {
        return rc;
    }
    const int64_t grid = nqb * p.parts;
    return wide ? launch_tc<BF16, 256>(map_q, map_p, p, smem, grid, stream)
                : launch_tc<BF16, 128>(map_q, map_p, p, smem, grid, stream);
}

} // namespace

size_t l2_tc_workspace_bytes(int64_t n, int64_t q, int dim, int mode)
{
    if (n <= 0 || q <= 0 || dim <= 0)
    {
        return 0;
    }
    return layout_of(n, q, dim, mode == BITSKNN_L2_BF16).total;
}

int l2_tc_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int mode, float* dist,
                 int64_t ld, void* workspace, size_t workspace_bytes, cudaStream_t stream)
{
    const bool bf16 = mode == BITSKNN_L2_BF16;
    const int max_dim = MAX_KB * (bf16 ? 64 : 32);
    if (dim > max_dim)
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (tensor-core modes take up to %d)", dim, max_dim);
    }
    if (n > 0x7fffffffLL - TILE_N || q > 0x7fffffffLL - TILE_M)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "sizes beyond the 32-bit tensor-map coordinates");
    }
    const size_t need = l2_tc_workspace_bytes(n, q, dim, mode);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255U) != 0)
    {
        return fail(BITSKNN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) needed, %zu given", need,
                    workspace_bytes);
    }
    auto* ws = static_cast<unsigned char*>(workspace);
    return bf16 ? run_tc<true>(points, queries, n, q, dim, dist, ld, ws, stream)
                : run_tc<false>(points, queries, n, q, dim, dist, ld, ws, stream);
}

} // namespace bitsknn
