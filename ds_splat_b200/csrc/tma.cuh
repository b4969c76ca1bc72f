// Thin wrappers over the sm_90+/sm_100 bulk asynchronous copy engine (TMA, untiled form) and the
// shared-memory mbarrier that tracks its completion.  Only copies from THIS GPU's global memory into the
// issuing block's own shared memory are used; nothing here multicasts.
//
// Rules the callers must keep: source and destination 16-byte aligned, size a multiple of 16 bytes.
// Waiting is bounded: mbar_wait_bounded() gives up after a fixed number of polls and returns false; the
// caller then reads its data with ordinary loads into buffers the copies do not write, and waits again
// (bounded) before its block exits, so a kernel can neither hang on a copy nor retire with one in flight.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace dsb {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, const uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival that also announces how many bytes the bulk copies of this phase will deliver.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, const uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, const uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Polls at most `limit` times; false means the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, const uint32_t parity, const uint32_t limit = 1u << 20) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// global -> shared bulk copy of `bytes` (multiple of 16), completion counted on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, const uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

}  // namespace dsb
