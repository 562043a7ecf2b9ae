// Tensor-parallel exchange over NVLink peer memory: the all-gather that follows a row-split
// GEMV, written as stores into every peer's copy of the gathered vector plus a flag per
// (exchange slot, source rank).
//
// cera's only parallelism on this path is over output rows (cera/src/backend/cpu.rs:380-391);
// splitting every matrix by rows keeps each per-row dot product identical to the single-GPU
// one, so logits and the greedy stream do not depend on the number of ranks.  After each
// row-split product a rank owns a slice of a vector every rank needs in full (the Q8_0
// attention output, the residual stream, the Q8_0 SwiGLU activations, the logits).  Each
// rank keeps those vectors in one "exchange region" at the same offsets, maps every peer's
// region (CUDA IPC between the one-process-per-GPU ranks), and pushes its slice with plain
// peer stores; no load ever crosses the link.
//
// Ordering: data stores, __threadfence_system(), then a release store of the step sequence
// number into flags[slot][my rank] of the peer.  The same kernel then waits until the
// peer's flag for this slot carries the sequence number, so "exchange kernel complete" means
// "every peer's slice has landed here" and the consumers need no change.  The wait is bounded
// by the global nanosecond timer: on expiry it records (slot, peer) in the model's status
// word and returns; once the word is set no later exchange waits, and the host turns the word
// into CERA_CUDA_ERR_TIMEOUT at its next synchronisation.
#include "ops.h"

namespace cera {

namespace {

__device__ void push_range(char *dst, const char *src, TpRange r) {
    if (((r.off | r.bytes) & 15) == 0) {
        const uint4 *s = (const uint4 *)(src + r.off);
        uint4 *d = (uint4 *)(dst + r.off);
        for (uint32_t i = threadIdx.x; i < r.bytes / 16; i += blockDim.x) d[i] = s[i];
    } else {
        const uint32_t *s = (const uint32_t *)(src + r.off);
        uint32_t *d = (uint32_t *)(dst + r.off);
        for (uint32_t i = threadIdx.x; i < r.bytes / 4; i += blockDim.x) d[i] = s[i];
    }
}

// One CTA per peer: copy up to three byte ranges of the local region to the same offsets of the
// peer's region, signal the peer, wait for the peer's signal.
__global__ void __launch_bounds__(512) tp_exchange_kernel(TpCtx c, TpRange r0, TpRange r1, TpRange r2, uint32_t slot) {
    pdl_trigger();
    pdl_wait();
    const uint32_t p = blockIdx.x + (blockIdx.x >= c.rank ? 1u : 0u);
    const uint32_t seq = *c.seq;
    char *dst = c.peer[p];
    const char *src = c.peer[c.rank];
    if (r0.bytes) push_range(dst, src, r0);
    if (r1.bytes) push_range(dst, src, r1);
    if (r2.bytes) push_range(dst, src, r2);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        tp_st_release_sys((uint32_t *)(dst + c.flags_off) + (size_t)slot * TP_MAX_RANKS + c.rank, seq);
        if (*(volatile uint32_t *)c.status == 0) {
            const uint32_t *mine = (const uint32_t *)(src + c.flags_off) + (size_t)slot * TP_MAX_RANKS + p;
            if (!tp_wait_flag(mine, seq, c.timeout_ns)) tp_record_timeout(c.status, slot, p);
        }
    }
}

// Greedy pick across ranks: every rank publishes (value, global index) of its local first maximum,
// then every rank takes the first strict maximum in rank order, which is the first strict maximum
// in index order because rank r owns indices [r * local_n, (r + 1) * local_n)
// (cera/src/sampler.rs:20-30).
__global__ void __launch_bounds__(32) tp_argmax_kernel(TpCtx c, const float *logits_local, uint32_t local_n,
                                                       const uint32_t *local_idx, uint32_t *tok_out, uint32_t slot) {
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = *c.seq;
    const uint32_t t = threadIdx.x;
    const uint32_t li = *local_idx;
    const float lv = logits_local[li < local_n ? li : 0];
    const unsigned long long pair = (unsigned long long)__float_as_uint(lv) | ((unsigned long long)(c.rank * local_n + li) << 32);
    char *own = c.peer[c.rank];
    if (t < c.size) {
        *((volatile unsigned long long *)(c.peer[t] + c.pairs_off) + c.rank) = pair;
        if (t != c.rank) {
            __threadfence_system();
            tp_st_release_sys((uint32_t *)(c.peer[t] + c.flags_off) + (size_t)slot * TP_MAX_RANKS + c.rank, seq);
            if (*(volatile uint32_t *)c.status == 0) {
                const uint32_t *mine = (const uint32_t *)(own + c.flags_off) + (size_t)slot * TP_MAX_RANKS + t;
                if (!tp_wait_flag(mine, seq, c.timeout_ns)) tp_record_timeout(c.status, slot, t);
            }
        }
    }
    __syncwarp();
    if (t == 0) {
        const volatile unsigned long long *pairs = (const volatile unsigned long long *)(own + c.pairs_off);
        unsigned long long w = pairs[0];
        float best = __uint_as_float((uint32_t)w);
        uint32_t best_i = (uint32_t)(w >> 32);
        for (uint32_t r = 1; r < c.size; ++r) {
            w = pairs[r];
            const float v = __uint_as_float((uint32_t)w);
            if (v > best) {
                best = v;
                best_i = (uint32_t)(w >> 32);
            }
        }
        *tok_out = best_i;
    }
}

__global__ void tp_tick_kernel(uint32_t *seq) {
    pdl_trigger();
    pdl_wait();
    *seq += 1;
}

}  // namespace

int32_t launch_tp_tick(uint32_t *seq, cudaStream_t st) {
    CERA_CUDA_TRY(launch_k(tp_tick_kernel, dim3(1), dim3(1), 0, st, seq));
    count_launch();
    return CERA_CUDA_OK;
}

int32_t launch_tp_exchange(const TpCtx &ctx, const TpRange *ranges, int n_ranges, uint32_t slot, cudaStream_t st) {
    if (ctx.size < 2) return CERA_CUDA_OK;
    if (n_ranges < 0 || n_ranges > 3) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_exchange: 0..3 ranges, got %d", n_ranges);
    TpRange r[3] = {{0, 0}, {0, 0}, {0, 0}};
    uint32_t most = 0;
    for (int i = 0; i < n_ranges && ranges; ++i) {
        if ((ranges[i].off | ranges[i].bytes) & 3)
            return fail(CERA_CUDA_ERR_BAD_ARG, "tp_exchange: range %d (offset %u, %u bytes) is not 4-byte aligned", i,
                        ranges[i].off, ranges[i].bytes);
        r[i] = ranges[i];
        most = ranges[i].bytes > most ? ranges[i].bytes : most;
    }
    const int threads = most >= 512 * 16 ? 512 : (most >= 128 * 16 ? 256 : 128);
    CERA_CUDA_TRY(launch_k(tp_exchange_kernel, dim3(ctx.size - 1), dim3(threads), 0, st, ctx, r[0], r[1], r[2], slot));
    count_launch();
    return CERA_CUDA_OK;
}

int32_t launch_tp_argmax(const TpCtx &ctx, const float *logits_local, uint32_t local_n, const uint32_t *local_idx,
                         uint32_t *tok_out, uint32_t slot, cudaStream_t st) {
    CERA_CUDA_TRY(launch_k(tp_argmax_kernel, dim3(1), dim3(32), 0, st, ctx, logits_local, local_n, local_idx, tok_out, slot));
    count_launch();
    return CERA_CUDA_OK;
}

}  // namespace cera

using namespace cera;

extern "C" {

// Runs one exchange whose peer is a second buffer on the same device that nothing ever signals, with a
// short wait budget, and reports the status word the kernel leaves behind: the bounded-wait path on one GPU.
int32_t cera_cuda_tp_wait_selftest(uint32_t timeout_ms, uint32_t *status_out, float *elapsed_ms) {
    if (!status_out) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_wait_selftest: null argument");
    if (timeout_ms == 0 || timeout_ms > 2000) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_wait_selftest: timeout_ms must be 1..2000");
    const size_t region = 4096;
    char *buf = nullptr;
    CERA_CUDA_TRY(cudaMalloc((void **)&buf, 2 * region + 256));
    cudaError_t e = cudaMemset(buf, 0, 2 * region + 256);
    TpCtx c{};
    c.peer[0] = buf;
    c.peer[1] = buf + region;
    c.rank = 0;
    c.size = 2;
    c.flags_off = 1024;
    c.pairs_off = 2048;
    c.seq = (const uint32_t *)(buf + 2 * region);
    c.status = (uint32_t *)(buf + 2 * region + 64);
    c.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    const uint32_t one = 1;
    if (e == cudaSuccess) e = cudaMemcpy((void *)c.seq, &one, 4, cudaMemcpyHostToDevice);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    int32_t st = check_cuda(e, "tp_wait_selftest setup");
    if (st == CERA_CUDA_OK) {
        TpRange r{0, 256};
        cudaEventRecord(e0, nullptr);
        st = launch_tp_exchange(c, &r, 1, 3, nullptr);
        cudaEventRecord(e1, nullptr);
        if (st == CERA_CUDA_OK) st = check_cuda(cudaDeviceSynchronize(), "tp_wait_selftest");
        if (st == CERA_CUDA_OK) st = check_cuda(cudaMemcpy(status_out, c.status, 4, cudaMemcpyDeviceToHost), "tp_wait_selftest");
        float ms = 0.0f;
        if (st == CERA_CUDA_OK && elapsed_ms && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *elapsed_ms = ms;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(buf);
    return st;
}

}  // extern "C"
