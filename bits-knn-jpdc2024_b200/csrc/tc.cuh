// Inline-PTX wrappers for the Blackwell tensor-core path: TMA tensor-map loads, tcgen05 MMA
// with shared-memory operand descriptors, tensor-memory (TMEM) allocation and loads.
// No multicast is used anywhere (every load names only this CTA's shared memory and barrier).
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace bitsknn::tc
{

// ---- TMA: 2-D tiled load global -> shared, completion on an mbarrier ---------------------
// x = innermost coordinate (elements; x * element size must be a multiple of 16 bytes),
// y = row.  Out-of-range parts of the box are filled with zeros and still counted in the
// transaction bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(ptx::smem_addr(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(ptx::smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ptx::smem_addr(bar)) : "memory");
}

// The same, counted as `count` arrivals.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(ptx::smem_addr(bar)), "r"(count) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------
// Allocates `cols` (power of two >= 32) TMEM columns; the base address lands in *slot (shared
// memory).  Executed by one whole warp; the same warp frees the columns before the kernel ends.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_addr(slot)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp gets lane (lane base + t),
// columns [col, col + 32).  The lane base of a warp is 32 * (warp id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                   "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                   "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                   "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr)
                 : "memory");
}

// 32 columns delivered into two 16-register halves (columns [col, col+16) and [col+16, col+32)).
__device__ __forceinline__ void tmem_ld_32x32_halves(uint32_t taddr, uint32_t (&a)[16], uint32_t (&b)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
                   "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]),
                   "=r"(a[15]), "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]),
                   "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]),
                   "=r"(b[14]), "=r"(b[15])
                 : "r"(taddr)
                 : "memory");
}

// Same, 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                   "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- MMA ----------------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B and a 128-byte inner box
// writes): 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is
// unused for swizzled K-major tiles (1), descriptor version 1 (sm_100), layout type 2.
// The tile must start on a 1024-byte boundary.  Stepping along K inside the 128-byte row is an
// addition of (bytes >> 4) to the start-address field.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* tile)
{
    const uint64_t addr = (ptx::smem_addr(tile) & 0x3FFFFU) >> 4;
    uint64_t desc = addr;                       // bits [0,14): start address >> 4
    desc |= static_cast<uint64_t>(1) << 16;     // bits [16,30): leading byte offset >> 4
    desc |= static_cast<uint64_t>(1024 >> 4) << 32; // bits [32,46): stride byte offset >> 4
    desc |= static_cast<uint64_t>(1) << 46;     // bits [46,48): descriptor version
    desc |= static_cast<uint64_t>(2) << 61;     // bits [61,64): SWIZZLE_128B
    return desc;
}

// Instruction descriptor for kind::tf32 / kind::f16 with FP32 accumulation, both operands
// K-major, M x N output tile.  format: 1 = BF16, 2 = TF32.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t format, uint32_t m, uint32_t n)
{
    return (1U << 4)           // D format F32
           | (format << 7)     // A format
           | (format << 10)    // B format
           | ((n >> 3) << 17)  // N / 8
           | ((m >> 4) << 24); // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
template <bool BF16>
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    const uint32_t acc = accumulate ? 1U : 0U;
    if constexpr (BF16)
    {
        asm volatile("{\n"
                     ".reg .pred p;\n"
                     "setp.ne.b32 p, %4, 0;\n"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
                     "}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
                     : "memory");
    }
    else
    {
        asm volatile("{\n"
                     ".reg .pred p;\n"
                     "setp.ne.b32 p, %4, 0;\n"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
                     "}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
                     : "memory");
    }
}

// The same with the descriptors given as their low words (start address and leading byte offset:
// the part that differs between tiles and K steps) plus the shared high word; `enable` == 0
// skips the instruction.  Keeps the issuing thread's 64-bit arithmetic out of its loop.
template <bool BF16>
__device__ __forceinline__ void mma_words(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                          uint32_t accumulate, uint32_t enable)
{
    if constexpr (BF16)
    {
        asm volatile("{\n"
                     ".reg .pred p, q;\n"
                     ".reg .b64 da, db;\n"
                     "setp.ne.b32 p, %5, 0;\n"
                     "setp.ne.b32 q, %6, 0;\n"
                     "mov.b64 da, {%1, %3};\n"
                     "mov.b64 db, {%2, %3};\n"
                     "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
                     "}\n" ::"r"(d_tmem),
                     "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(enable)
                     : "memory");
    }
    else
    {
        asm volatile("{\n"
                     ".reg .pred p, q;\n"
                     ".reg .b64 da, db;\n"
                     "setp.ne.b32 p, %5, 0;\n"
                     "setp.ne.b32 q, %6, 0;\n"
                     "mov.b64 da, {%1, %3};\n"
                     "mov.b64 db, {%2, %3};\n"
                     "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n"
                     "}\n" ::"r"(d_tmem),
                     "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(enable)
                     : "memory");
    }
}

// Makes `bar` complete one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     ptx::smem_addr(bar))
                 : "memory");
}

} // namespace bitsknn::tc
