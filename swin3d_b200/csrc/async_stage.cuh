// Asynchronous staging primitives (sm_90+/sm_100a): mbarrier objects in shared memory and the bulk
// asynchronous copy engine (cp.async.bulk, global -> this block's shared memory, completion counted
// in bytes on an mbarrier).  Every copy here reads the launching GPU's own global memory and lands in
// the issuing block's shared memory; none addresses another block or another GPU.
//
// Every wait is bounded: mbar_wait gives up after MBAR_WAIT_TRIES polls and returns false, and the
// kernels then leave their loops through a block-uniform flag and record the event in an error word.
#pragma once
#include <stdint.h>

namespace s3d {

constexpr int MBAR_WAIT_TRIES = 1 << 22;

__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

// Makes the initialised barriers visible to the asynchronous proxy.
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later asynchronous copies.
__device__ __forceinline__ void async_proxy_fence()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// true once the phase with the given parity has completed, false if it did not within the bound.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity)
{
    for (int i = 0; i < MBAR_WAIT_TRIES; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// bytes: a multiple of 16; dst and src 16-byte aligned.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// Barrier among the first `count` threads of the block (a multiple of 32), id 1; the producer warp,
// which runs ahead, does not take part.
template <int COUNT>
__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(COUNT) : "memory");
}

}  // namespace s3d
