// Bulk asynchronous copies (the TMA unit's 1-D form) and mbarrier helpers for sm_100a.
//
// Only CTA-local copies are used: global memory of this GPU -> this CTA's shared memory, completion
// signalled on an mbarrier in the same CTA.  Both addresses are 16-byte aligned and the size is a
// multiple of 16 bytes (checked on the host before a kernel that uses these is chosen).
// Every wait is bounded: after kSpinLimit unsuccessful polls the waiter gives up, so a protocol bug
// cannot hang the GPU; the kernel then records the failure in g_async_error and leaves.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dl {

constexpr uint32_t kSpinLimit = 1u << 24;  // polls of ~20 ns each: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// One arrival that also announces `bytes` of asynchronous copies still to land on this barrier.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t spin = 0; spin < limit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// global -> shared bulk copy of `bytes` (multiple of 16), completion counted on `bar`.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

}  // namespace dl
