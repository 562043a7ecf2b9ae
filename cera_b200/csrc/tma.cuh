// mbarrier, bulk-copy (TMA unit) and asynchronous-copy helpers for kernels that stage global memory through a
// ring of shared-memory stages.  Every wait is bounded: when the limit runs out the waiter raises the CTA's
// abort flag (so the CTA's other waits give up at once) and ORs `who` into a status word in device
// memory that the host reads through cera_cuda_kernel_status.  No copy is addressed to another CTA.
#pragma once

#include "common.cuh"

namespace cera {
namespace tma {

constexpr uint32_t SPIN_LIMIT = 1u << 22;  // polls of ~50-100 ns: a fraction of a second at most

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false when the limit ran out or another warp of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned int *status,
                                          unsigned int who) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (i > 64) __nanosleep(40);
    }
    *abort_flag = 1;
    atomicOr(status, who);
    return false;
}
// The same with mbarrier.try_wait, which suspends the thread in hardware for a bounded time instead of spinning on
// test_wait: far fewer issued instructions while a copy is in flight.  Bounded like mbar_wait.
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_blocking(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned int *status,
                                                   unsigned int who) {
    for (uint32_t i = 0; i < (SPIN_LIMIT >> 4); ++i) {  // each try may block for microseconds: keep the total bound comparable
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(status, who);
    return false;
}
// One contiguous global range (16-byte aligned, a multiple of 16 bytes) -> this CTA's shared memory; the bytes are
// counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 16 bytes global -> shared through the LSU's asynchronous copy path (L1-bypassing).
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// Arrive on `bar` once every cp.async this thread has issued so far has landed (the arrival is one of the
// barrier's expected count).
__device__ __forceinline__ void cp_async_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

}  // namespace tma
}  // namespace cera
