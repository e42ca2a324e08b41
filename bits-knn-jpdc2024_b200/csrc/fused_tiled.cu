// `bits-fused`, FP32, tiled variant: the distance tile of the GEMM-form kernel (128 queries x 128
// points per block, 8 x 8 per thread, one FMA chain per distance in coordinate order -- the same
// arithmetic as l2.cu, hence bit-identical with the reference's fused kernel and its
// abstract_gemm) is filtered in registers instead of being stored.
//
// A pre-pass writes both inputs as tile images: for every 128 rows the coordinates transposed,
// [coordinate][row] (coordinates zero padded to a multiple of four, which changes no FP32 sum),
// followed by one row of squared norms (accumulated in coordinate order like the reference does).
// The block keeps its query image resident in shared memory and streams the point image through a
// ring of 32-coordinate slabs with 1-D bulk copies (cp.async.bulk + mbarrier): the compute warps
// issue no global loads at all, their inner loop is four 128-bit shared-memory loads per 64 FMAs.
//
// Per query the block keeps a 32-slot candidate buffer in shared memory (slots handed out by
// shared atomics) and the radius; the sorted lists (32 * IPT pairs) live in the workspace and are
// only touched by folds, which the warps do with the shuffle networks of warpfold.cuh (warp w folds
// queries w, w + 8, ...).  A fold round runs when some buffer is at least half full or a candidate
// found no slot; candidates left over are filtered again by the tightened radius.  The database
// may be cut into `parts` ranges scanned by different blocks (small q); merge_lists() merges the
// per-part lists.
// Reference counterpart: fused_cache_kernel::run + multi_buffer
// (include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:25-305,716-799).
#include <algorithm>
#include <cstdint>

#include "common.cuh"
#include "ptx.cuh"
#include "sortnet.cuh"
#include "warpfold.cuh"

namespace bitsknn
{

namespace
{

constexpr int FT_BM = 128;
constexpr int FT_BN = 128;
// (measured at q = 2^14, n = 2^20: slabs of 32 coordinates with two in flight take one block barrier per
// 32 coordinates and the same shared memory as four slabs of 16: dim 64 60.9 -> 58.7 ms, dim 32 33.1 -> 32.0;
// three slabs of 32 no longer leave room for two blocks per SM at dim 64: 70.9 ms)
constexpr int FT_BK = 32;      // coordinates per slab
constexpr int FT_STAGES = 2;   // slabs in flight
constexpr int FT_THREADS = 256;
constexpr int FT_CAP = 32;
constexpr int FT_SLAB_FLOATS = (FT_BK + 1) * FT_BN; // the coordinate rows + room for the norm row
constexpr int FT_MAX_DIM = 320;                     // query image + ring + buffers within 227 KiB

struct tiled_params
{
    const float* pimg; // [tiles][dp + 1][128]: point coordinates transposed per tile, then |x|^2
    const float* qimg; // [query tiles][dp + 1][128]
    int64_t n;
    int64_t q;
    int dp; // coordinates padded to a multiple of 4
    int k;
    int32_t index_base;
    int parts;
    int64_t tiles; // point tiles of 128
    float* list_d; // [parts][q][KL]
    int32_t* list_x;
    int* status;
};

// Pre-pass: one block per 128 rows, thread r owns row r of the tile.
__global__ void __launch_bounds__(FT_BN) ft_image_kernel(const float* __restrict__ src, int64_t rows, int dim, int dp,
                                                         float* __restrict__ dst)
{
    const int r = threadIdx.x;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * FT_BN + r;
    float* out = dst + static_cast<int64_t>(blockIdx.x) * (dp + 1) * FT_BN;
    const float* in = src + row * dim;
    float nrm = 0.0F;
    for (int d = 0; d < dp; ++d)
    {
        const float v = (row < rows && d < dim) ? __ldg(in + d) : 0.0F;
        nrm = fmaf(v, v, nrm);
        out[d * FT_BN + r] = v;
    }
    out[dp * FT_BN + r] = nrm;
}

template <int IPT, bool PARTIAL>
__global__ void __launch_bounds__(FT_THREADS, 2) fused_tiled_kernel(const tiled_params p)
{
    constexpr int KL = 32 * IPT;
    // ring [FT_STAGES][FT_BK + 1][128] | query image [dp][128] | candidate buffers [128][32] x 2
    extern __shared__ __align__(128) unsigned char ft_smem[];
    float* Bs = reinterpret_cast<float*>(ft_smem);
    float* As = Bs + FT_STAGES * FT_SLAB_FLOATS;
    auto buf_d = reinterpret_cast<float(*)[FT_CAP]>(As + p.dp * FT_BM);
    auto buf_x = reinterpret_cast<int(*)[FT_CAP]>(As + p.dp * FT_BM + FT_BM * FT_CAP);
    __shared__ uint64_t full[FT_STAGES];
    __shared__ uint64_t a_full;
    __shared__ int cnt[FT_BM];
    __shared__ float sr_d[FT_BM];
    __shared__ int sr_x[FT_BM];
    __shared__ int has_list[FT_BM];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    // (32-bit tile and slab counters: fewer registers; the host checks that they fit)
    const int qb = static_cast<int>(blockIdx.x) / p.parts;
    const int part = static_cast<int>(blockIdx.x) - qb * p.parts;
    const int64_t m0 = static_cast<int64_t>(qb) * FT_BM;
    const int tiles = static_cast<int>(p.tiles);
    const int per = (tiles + p.parts - 1) / p.parts;
    const int t_begin = part * per;
    const int t_end = t_begin + per < tiles ? t_begin + per : tiles;
    const int nslab = (p.dp + FT_BK - 1) / FT_BK;
    const int total = (t_end > t_begin ? t_end - t_begin : 0) * nslab; // slabs this block consumes

    if (tid < FT_BM)
    {
        cnt[tid] = 0;
        has_list[tid] = 0;
        // a query row beyond q never accepts a candidate
        sr_d[tid] = m0 + tid < p.q ? INFINITY : -INFINITY;
        sr_x[tid] = PAD_IDX;
    }
    if (tid == 0)
    {
        ptx::mbar_init(&a_full, 1);
        for (int s = 0; s < FT_STAGES; ++s)
        {
            ptx::mbar_init(&full[s], 1);
        }
        ptx::mbar_init_fence();
    }
    __syncthreads();

    // Producer state (thread 0 alone): the next slab to request, as (tile, slab) and as a count.
    int issue_t = t_begin;
    int issue_s = 0;
    int issued = 0;
    auto issue_slab = [&](int stage) {
        const int rows = p.dp - issue_s * FT_BK < FT_BK ? p.dp - issue_s * FT_BK : FT_BK;
        // the norm row follows the last coordinate row and travels with the last slab
        const uint32_t bytes = static_cast<uint32_t>(rows + (issue_s == nslab - 1 ? 1 : 0)) * FT_BN * 4U;
        const float* src = p.pimg + (static_cast<int64_t>(issue_t) * (p.dp + 1) + issue_s * FT_BK) * FT_BN;
        ptx::mbar_expect_tx(&full[stage], bytes);
        ptx::bulk_g2s(Bs + stage * FT_SLAB_FLOATS, src, bytes, &full[stage]);
        ++issued;
        if (++issue_s == nslab)
        {
            issue_s = 0;
            ++issue_t;
        }
    };
    if (tid == 0 && total > 0)
    {
        const uint32_t a_bytes = static_cast<uint32_t>(p.dp) * FT_BM * 4U;
        ptx::mbar_expect_tx(&a_full, a_bytes);
        const float* qsrc = p.qimg + static_cast<int64_t>(qb) * (p.dp + 1) * FT_BM;
        for (int s = 0; s < nslab; ++s)
        {
            const int rows = p.dp - s * FT_BK < FT_BK ? p.dp - s * FT_BK : FT_BK;
            ptx::bulk_g2s(As + s * FT_BK * FT_BM, qsrc + s * FT_BK * FT_BM, static_cast<uint32_t>(rows) * FT_BM * 4U,
                          &a_full);
        }
        for (int s = 0; s < FT_STAGES && issued < total; ++s)
        {
            issue_slab(s);
        }
    }
    bool ok = true;
    if (total > 0)
    {
        ok = ptx::mbar_wait_bounded(&a_full, 0);
    }

    // folds the buffers of this warp's queries (w, w + 8, ...) that hold candidates
    auto fold_round = [&]() {
        for (int qi = warp; qi < FT_BM; qi += FT_THREADS / 32)
        {
            // a fold costs a round trip to the list whatever the buffer holds, so nearly empty
            // buffers wait for a later round (the final flush takes whatever is left)
            const int have = cnt[qi];
            const bool flush = have >= FT_CAP / 4;
            if (flush && m0 + qi < p.q)
            {
                const int valid = have < FT_CAP ? have : FT_CAP;
                const float cd = lane < valid ? buf_d[qi][lane] : INFINITY;
                const int cx = lane < valid ? buf_x[qi][lane] : PAD_IDX;
                float* gl_d = p.list_d + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
                int32_t* gl_x = p.list_x + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
                const radius_pair nr = warp_fold_global_call<IPT>(cd, cx, has_list[qi] != 0, gl_d, gl_x, p.k, lane);
                if (lane == 0)
                {
                    sr_d[qi] = nr.d;
                    sr_x[qi] = nr.x;
                    has_list[qi] = 1;
                    cnt[qi] = 0;
                }
            }
            __syncwarp();
        }
    };

    int stage = 0;
    uint32_t parity = 0;
    for (int t = t_begin; t < t_end; ++t)
    {
        const int64_t n0 = static_cast<int64_t>(t) * FT_BN;
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
        for (int s = 0; s < nslab; ++s)
        {
            // (a wait that runs out is reported through the status word; the block carries on
            // so that every thread still reaches every barrier)
            ok = ptx::mbar_wait_bounded(&full[stage], parity) && ok;
            const float* Bsl = Bs + stage * FT_SLAB_FLOATS;
            const float* Asl = As + s * FT_BK * FT_BM;
            const int rows = p.dp - s * FT_BK < FT_BK ? p.dp - s * FT_BK : FT_BK;
            for (int k4 = 0; k4 < rows; k4 += 4)
            {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                {
                    const float* ar = Asl + (k4 + kk) * FT_BM;
                    const float* br = Bsl + (k4 + kk) * FT_BN;
                    const float4 a0 = *reinterpret_cast<const float4*>(ar + ty * 4);
                    const float4 a1 = *reinterpret_cast<const float4*>(ar + 64 + ty * 4);
                    const float4 b0 = *reinterpret_cast<const float4*>(br + tx * 4);
                    const float4 b1 = *reinterpret_cast<const float4*>(br + 64 + tx * 4);
                    const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
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
            }
            if (PARTIAL && s == nslab - 1)
            {
                // squared norms of this thread's eight points: the row after the coordinates
                const float* nr = Bsl + rows * FT_BN;
                const float4 n0v = *reinterpret_cast<const float4*>(nr + tx * 4);
                const float4 n1v = *reinterpret_cast<const float4*>(nr + 64 + tx * 4);
                nrm[0] = n0v.x;
                nrm[1] = n0v.y;
                nrm[2] = n0v.z;
                nrm[3] = n0v.w;
                nrm[4] = n1v.x;
                nrm[5] = n1v.y;
                nrm[6] = n1v.z;
                nrm[7] = n1v.w;
            }
            __syncthreads(); // every thread is done with this stage: it can be refilled
            if (tid == 0 && issued < total)
            {
                issue_slab(stage);
            }
            if (++stage == FT_STAGES)
            {
                stage = 0;
                parity ^= 1U;
            }
        }

    // ---- filter the 8 x 8 distances of this thread -------------------------------------
        unsigned long long pending = 0;
        const int ncols = p.n - n0 < FT_BN ? static_cast<int>(p.n - n0) : FT_BN; // valid columns of this tile
        const int c_lo = tx * 4;       // this thread's columns: c_lo .. c_lo + 3 and 64 + c_lo .. + 3
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const int row = i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4);
            const float rd = sr_d[row];
            // finish the 8 distances of this row and look at their minimum first: once the radius
            // has settled almost every row is rejected by this one comparison
            float mn = INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                const float d = PARTIAL ? (nrm[j] - 2.0F * acc[i][j]) : acc[i][j];
                acc[i][j] = d;
                mn = fminf(mn, d);
            }
            if (mn <= rd)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const float d = acc[i][j];
                    const int c = j < 4 ? c_lo + j : 64 + c_lo + (j - 4);
                    if (d <= rd && c < ncols)
                    {
                        const int idx = p.index_base + static_cast<int>(n0) + c;
                        if (pair_lt(d, idx, rd, sr_x[row]))
                        {
                            const int pos = atomicAdd(&cnt[row], 1);
                            if (pos < FT_CAP)
                            {
                                buf_d[row][pos] = d;
                                buf_x[row][pos] = idx;
                            }
                            else
                            {
                                pending |= 1ULL << (i * 8 + j);
                            }
                        }
                    }
                }
            }
        }
        // a fold round when a candidate found no slot or some buffer is at least half full
        bool trigger = pending != 0 || (tid < FT_BM && cnt[tid] >= FT_CAP / 2);
        while (__syncthreads_or(trigger ? 1 : 0) != 0)
        {
            fold_round();
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                const int row = i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const unsigned long long bit = 1ULL << (i * 8 + j);
                    if ((pending & bit) != 0)
                    {
                        const int64_t col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                        const int idx = p.index_base + static_cast<int>(col);
                        bool done = true;
                        if (pair_lt(acc[i][j], idx, sr_d[row], sr_x[row]))
                        {
                            const int pos = atomicAdd(&cnt[row], 1);
                            if (pos < FT_CAP)
                            {
                                buf_d[row][pos] = acc[i][j];
                                buf_x[row][pos] = idx;
                            }
                            else
                            {
                                done = false;
                            }
                        }
                        if (done)
                        {
                            pending &= ~bit;
                        }
                    }
                }
            }
            trigger = pending != 0;
        }
    }

    // flush what is left and make sure every live query of this part has a complete list
    __syncthreads();
    if (tid < FT_BM && has_list[tid] == 0 && cnt[tid] == 0)
    {
        cnt[tid] = -1; // marks "write an all-padding list"
    }
    __syncthreads();
    for (int qi = warp; qi < FT_BM; qi += FT_THREADS / 32)
    {
        const int have = cnt[qi];
        if (have != 0 && m0 + qi < p.q)
        {
            const int valid = have < 0 ? 0 : (have < FT_CAP ? have : FT_CAP);
            const float cd = lane < valid ? buf_d[qi][lane] : INFINITY;
            const int cx = lane < valid ? buf_x[qi][lane] : PAD_IDX;
            float* gl_d = p.list_d + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
            int32_t* gl_x = p.list_x + (static_cast<int64_t>(part) * p.q + m0 + qi) * KL;
            warp_fold_global_call<IPT>(cd, cx, has_list[qi] != 0, gl_d, gl_x, p.k, lane);
        }
        __syncwarp();
    }
    if (!ok)
    {
        atomicOr(p.status, DEVICE_STATUS_TIMEOUT);
    }
}


struct tiled_layout
{
    int kl;
    int parts;       // database ranges per query tile from full_blocks on
    int full_blocks; // leading query tiles scanned whole
    int dp;
    size_t off_pimg, off_qimg, off_ld, off_lx, total;
};

tiled_layout tiled_layout_of(int64_t n, int64_t q, int dim, int k)
{
    tiled_layout l{};
    l.kl = k <= 32 ? 32 : (k <= 64 ? 64 : (k <= 128 ? 128 : 256));
    l.dp = (dim + 3) / 4 * 4;
    const int64_t nqb = (q + FT_BM - 1) / FT_BM;
    const int64_t tiles = (n + FT_BN - 1) / FT_BN;
    // two blocks fit an SM.  As many whole waves of query tiles as there are scan the database whole;
    // for the tiles left over (all of them when there are fewer than block slots) the database is
    // split as far as those blocks still run at once (measured: q = 2^14 on 148 SMs takes 19.3 ms
    // with 2 ranges, 21.8 with 3, 20.5 with 4)
    const int slots = 2 * device_sm_count();
    l.full_blocks = static_cast<int>(nqb / slots * slots);
    const int64_t rest = nqb - l.full_blocks;
    const int64_t want = rest > 0 ? std::max<int64_t>(1, slots / rest) : 1;
    l.parts = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, std::max<int64_t>(1, tiles / 32))));
    if (const int forced = tuning_value("fused.parts", 0); forced > 0)
    {
        // a forced count applies to every query tile
        l.full_blocks = 0;
        l.parts = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(forced, std::max<int64_t>(1, tiles / 32))));
    }
    const size_t lists = static_cast<size_t>(l.parts) * static_cast<size_t>(q) * l.kl;
    auto align256 = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    l.off_pimg = 0;
    l.off_qimg = align256(static_cast<size_t>(tiles) * (l.dp + 1) * FT_BN * 4);
    l.off_ld = l.off_qimg + align256(static_cast<size_t>(nqb) * (l.dp + 1) * FT_BM * 4);
    l.off_lx = l.off_ld + align256(lists * 4);
    l.total = l.off_lx + align256(lists * 4);
    return l;
}

size_t tiled_smem_bytes(int dp)
{
    return sizeof(float) * (static_cast<size_t>(FT_STAGES) * FT_SLAB_FLOATS + static_cast<size_t>(dp) * FT_BM +
                            2 * FT_BM * FT_CAP);
}

template <int IPT>
int launch_tiled(const tiled_params& p, int mode, int64_t grid, cudaStream_t stream)
{
    const size_t smem = tiled_smem_bytes(p.dp);
    kernel_scope timed{"fused_tiled_kernel", stream};
    if (mode == BITSKNN_L2_PARTIAL)
    {
        auto kernel = fused_tiled_kernel<IPT, true>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FT_THREADS, smem, stream>>>(p);
    }
    else
    {
        auto kernel = fused_tiled_kernel<IPT, false>;
        BITSKNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(grid), FT_THREADS, smem, stream>>>(p);
    }
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

} // namespace

bool fused_tiled_supports(int dim) { return dim >= 1 && dim <= FT_MAX_DIM; }

size_t fused_tiled_workspace_bytes(int64_t n, int64_t q, int dim, int k)
{
    if (n <= 0 || q <= 0 || k <= 0 || !fused_tiled_supports(dim))
    {
        return 0;
    }
    return tiled_layout_of(n, q, dim, k).total;
}

int fused_tiled_launch(const float* points, const float* queries, int64_t n, int64_t q, int dim, int k, int mode,
                       int32_t index_base, float* out_dist, int32_t* out_idx, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream)
{
    if (!fused_tiled_supports(dim))
    {
        return fail(BITSKNN_ERR_UNSUPPORTED_DIM, "Unsupported dimension: %d (the tiled fused kernel takes up to %d)", dim,
                    FT_MAX_DIM);
    }
    if (n / FT_BN * ((dim + FT_BK - 1) / FT_BK) >= (int64_t{1} << 31) - FT_BN)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "the tiled fused kernel counts up to 2^31 slabs of coordinates x 128 points");
    }
    const tiled_layout l = tiled_layout_of(n, q, dim, k);
    if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255U) != 0)
    {
        return fail(BITSKNN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) needed, %zu given", l.total,
                    workspace_bytes);
    }
    auto* ws = static_cast<unsigned char*>(workspace);
    float* pimg = reinterpret_cast<float*>(ws + l.off_pimg);
    float* qimg = reinterpret_cast<float*>(ws + l.off_qimg);
    const int64_t tiles = (n + FT_BN - 1) / FT_BN;
    const int64_t nqb = (q + FT_BM - 1) / FT_BM;
    ft_image_kernel<<<static_cast<unsigned>(tiles), FT_BN, 0, stream>>>(points, n, dim, l.dp, pimg);
    ft_image_kernel<<<static_cast<unsigned>(nqb), FT_BM, 0, stream>>>(queries, q, dim, l.dp, qimg);
    BITSKNN_CUDA_TRY(cudaGetLastError());

    tiled_params p{};
    p.pimg = pimg;
    p.qimg = qimg;
    p.n = n;
    p.q = q;
    p.dp = l.dp;
    p.k = k;
    p.index_base = index_base;
    p.tiles = tiles;
    p.status = device_status_word();
    if (p.status == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    // Two launches of the same kernel: the query tiles that scan the database whole (one block each,
    // whole waves of them), then the tiles left over with `parts` database ranges each.  Each has its
    // own region of lists: [q_whole][KL], then [parts][q - q_whole][KL].
    float* list_d = reinterpret_cast<float*>(ws + l.off_ld);
    int32_t* list_x = reinterpret_cast<int32_t*>(ws + l.off_lx);
    // (tiles left over that are not cut: everything is one launch)
    const int64_t q_whole = l.parts == 1 ? 0 : std::min<int64_t>(q, static_cast<int64_t>(l.full_blocks) * FT_BM);
    const int64_t whole_blocks = l.parts == 1 ? 0 : l.full_blocks;
    auto launch = [&](int64_t q0, int64_t rows, int parts, int64_t grid) {
        tiled_params r = p;
        r.q = rows;
        r.parts = parts;
        r.qimg = qimg + (q0 / FT_BM) * static_cast<int64_t>(l.dp + 1) * FT_BM;
        r.list_d = list_d + q0 * l.kl;
        r.list_x = list_x + q0 * l.kl;
        switch (l.kl)
        {
        case 32:
            return launch_tiled<1>(r, mode, grid, stream);
        case 64:
            return launch_tiled<2>(r, mode, grid, stream);
        case 128:
            return launch_tiled<4>(r, mode, grid, stream);
        default:
            return launch_tiled<8>(r, mode, grid, stream);
        }
    };
    if (q_whole > 0)
    {
        if (const int rc = launch(0, q_whole, 1, whole_blocks); rc != BITSKNN_OK)
        {
            return rc;
        }
        if (const int rc = merge_lists(list_d, list_x, q_whole * l.kl, l.kl, q_whole, 1, l.kl, k, nullptr, out_dist, out_idx,
                                       merge_input::sorted, stream);
            rc != BITSKNN_OK)
        {
            return rc;
        }
    }
    if (q_whole < q)
    {
        const int64_t rows = q - q_whole;
        if (const int rc = launch(q_whole, rows, l.parts, (nqb - whole_blocks) * l.parts); rc != BITSKNN_OK)
        {
            return rc;
        }
        return merge_lists(list_d + q_whole * l.kl, list_x + q_whole * l.kl, rows * l.kl, l.kl, rows, l.parts, l.kl, k, nullptr,
                           out_dist + q_whole * k, out_idx + q_whole * k, merge_input::sorted, stream);
    }
    return BITSKNN_OK;
}

} // namespace bitsknn
