// Device side of the tensor-parallel exchange, for kernels that carry it themselves: a producer
// mirrors the stores of its slice into every peer's exchange region (tp_push), and the consumer of
// the gathered vector signals and waits in its prologue (tp_arrive_wait).  See tp.cu for the
// protocol; size < 2 turns every helper into a no-op.
#pragma once

#include "common.cuh"

namespace cera {

constexpr uint32_t TP_MAX_RANKS = 8;
constexpr uint32_t TP_NO_SLOT = 0xFFFFFFFFu;

struct TpCtx {
    char *peer[TP_MAX_RANKS];  // every rank's exchange region as mapped on this device; peer[rank] is its own
    uint32_t rank, size;
    uint32_t flags_off;        // byte offset of flags[n_slots][TP_MAX_RANKS] (u32) inside a region
    uint32_t pairs_off;        // byte offset of the greedy pairs[TP_MAX_RANKS] {f32 bits, index}
    const uint32_t *seq;       // device: sequence number of the running step
    uint32_t *status;          // device: 0, or 0x80000000 | peer << 24 | slot + 1 after a wait ran out
    uint64_t timeout_ns;
};

// What a kernel of the decode step does for the exchange.
struct TpHook {
    TpCtx ctx;
    uint32_t wait_slot = TP_NO_SLOT;  // exchange whose arrival this kernel's input needs
    int push = 0;                     // mirror this kernel's output stores to the peers
};

__device__ __forceinline__ uint64_t tp_global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void tp_st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t tp_ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// True once *flag has reached seq (wrap-safe); false when the budget ran out first.
__device__ inline bool tp_wait_flag(const uint32_t *flag, uint32_t seq, uint64_t timeout_ns) {
    const uint64_t t0 = tp_global_ns();
    for (uint32_t it = 0;; ++it) {
        if ((int32_t)(tp_ld_acquire_sys(flag) - seq) >= 0) return true;
        if ((it & 15) == 15) {
            if (tp_global_ns() - t0 > timeout_ns) return false;
            if (it > 4096) __nanosleep(200);
        }
    }
}

__device__ __forceinline__ void tp_record_timeout(uint32_t *status, uint32_t slot, uint32_t peer) {
    atomicCAS(status, 0u, 0x80000000u | (peer << 24) | ((slot + 1) & 0xFFFFFFu));
}

__device__ __forceinline__ uint32_t *tp_flag(const TpCtx &c, uint32_t at_rank, uint32_t slot, uint32_t src) {
    return (uint32_t *)(c.peer[at_rank] + c.flags_off) + (size_t)slot * TP_MAX_RANKS + src;
}

// Prologue of the kernel that consumes exchange `slot`.  Call from every thread of every CTA (1-D
// blocks of at least `size` threads), after griddepcontrol.wait: at that point the producing grid of
// this rank has completed, so its mirrored stores are performed and the first CTA may tell the peers;
// then every CTA waits until all peers have said the same.
__device__ __forceinline__ void tp_arrive_wait(const TpCtx &c, uint32_t slot) {
    if (c.size < 2 || slot == TP_NO_SLOT) return;
    const uint32_t t = threadIdx.x;
    if (t < c.size && t != c.rank) {
        const uint32_t seq = *(volatile const uint32_t *)c.seq;
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
            __threadfence_system();
            tp_st_release_sys(tp_flag(c, t, slot, c.rank), seq);
        }
        if (*(volatile uint32_t *)c.status == 0 && !tp_wait_flag(tp_flag(c, c.rank, slot, t), seq, c.timeout_ns))
            tp_record_timeout(c.status, slot, t);
    }
    __syncthreads();
}

// Store v at the same offset of every peer's region as `local` has in this rank's.
template <typename V>
__device__ __forceinline__ void tp_push(const TpCtx &c, V *local, V v) {
    const size_t off = (size_t)((char *)local - c.peer[c.rank]);
    for (uint32_t p = 0; p < c.size; ++p)
        if (p != c.rank) *(V *)(c.peer[p] + off) = v;
}

}  // namespace cera
