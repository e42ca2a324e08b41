// Thin inline-PTX wrappers: mbarrier, 1-D bulk async copies (TMA without a tensor map).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace bitsknn::ptx
{

__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy before any copy uses them.
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` polls or after about two seconds of SM clocks, whichever
// comes first (each poll may itself suspend for a hardware-defined time, so the poll count alone
// would not bound the time).  Returns false on expiry; the caller reports it and leaves.
constexpr long long WAIT_CLOCK_LIMIT = 1LL << 32;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1U << 22))
{
    if (mbar_try_wait(bar, parity))
    {
        return true;
    }
    const long long deadline = clock64() + WAIT_CLOCK_LIMIT;
    for (uint32_t i = 1; i < limit; ++i)
    {
        if (mbar_try_wait(bar, parity))
        {
            return true;
        }
        if (i > 64)
        {
            __nanosleep(64);
            if ((i & 63U) == 0 && clock64() > deadline)
            {
                return false;
            }
        }
    }
    return false;
}

// The same without the sleeping back-off, for waits on a pipeline's critical path (a sleeping
// waiter notices a completed phase late, which a short ring cannot absorb).  The poll carries a
// suspend-time hint instead: the hardware parks the thread until the phase completes or the hint
// runs out, so a waiting thread does not compete for issue slots with the warps it waits for.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns)
                 : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_bounded_spin(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity))
    {
        return true;
    }
    const long long deadline = clock64() + WAIT_CLOCK_LIMIT;
    while (true)
    {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
        {
            if (mbar_try_wait_hint(bar, parity, 2000U))
            {
                return true;
            }
        }
        if (clock64() > deadline)
        {
            return false;
        }
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

} // namespace bitsknn::ptx
