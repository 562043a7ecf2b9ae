// Decode GEMV with the weight stream staged by the TMA unit (bulk asynchronous copies).
//
// Same lane-task arithmetic as gemv_rows.cu (gemv_task.cuh); what changes is how weight bytes reach
// the lanes.  One CTA per SM runs 8 consumer warps and 1 producer warp.  The producer's elected lane
// walks the CTA's row tiles and, per tile, issues one cp.async.bulk per weight plane (each plane of a
// tile is one contiguous byte range in the planar layout) into a ring of shared-memory stages, arming
// the stage's `full` mbarrier with the byte count.  Consumers wait on `full`, pull their lane tasks out
// of shared memory (piece-major planes: conflict-free 128-bit reads), release the stage on its `empty`
// mbarrier and do the dp4a work from registers.  Up to STAGES-1 tiles (100-190 KB per SM) stay in flight
// with no register cost, so the HBM stream no longer stalls on the consumers' arithmetic.
//
// Every copy targets the issuing CTA alone; no thread-block cluster is used.  Every mbarrier wait is bounded: a wait that runs out
// raises a flag in device memory (cera_cuda_kernel_status reports it), makes the CTA's other waits give
// up at once, and the kernel returns after a bounded drain of the copies it still has in flight.
#include <cstdlib>
#include <cstring>

#include "gemv_task.cuh"

namespace cera {

namespace {

constexpr int TM_CONSUMER_WARPS = 8;
constexpr int TM_THREADS = (TM_CONSUMER_WARPS + 1) * 32;
constexpr int TM_UNR = 2;
constexpr int TM_MAX_STAGES = 6;
constexpr int TM_MAX_SEGS = 3;
constexpr uint32_t TM_SPIN_LIMIT = 1u << 22;  // polls of ~50-100 ns: a fraction of a second at most
constexpr size_t TM_HEADER_BYTES = 256;
constexpr size_t TM_SMEM_BUDGET = 200 * 1024;

__device__ unsigned int g_tma_status = 0;  // bit 0: a consumer wait ran out, bit 1: a producer wait ran out

struct TmaParams {
    WeightView w[TM_MAX_SEGS];
    float *y[TM_MAX_SEGS];
    uint32_t row_end[TM_MAX_SEGS];
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k, t128;
    int wpr, epilogue, stages;
    uint32_t plane_b[4];  // bytes per row of the q, qh, hdr, d planes
    uint32_t stage_bytes;
    GemvFusion f;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
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
// Bounded wait.  Returns false when the limit ran out or another warp of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned int who) {
    for (uint32_t i = 0; i < TM_SPIN_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (i > 64) __nanosleep(40);
    }
    *abort_flag = 1;
    atomicOr(&g_tma_status, who);
    return false;
}
// One contiguous global range -> shared memory, completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(TM_CONSUMER_WARPS * 32) : "memory"); }

template <int T>
__global__ void __launch_bounds__(TM_THREADS, 1) gemv_tma_kernel(const TmaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float partial[TM_CONSUMER_WARPS][TM_UNR];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + TM_MAX_STAGES;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + 128);
    uint8_t *ring = smem + TM_HEADER_BYTES;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int S = p.stages, wpr = p.wpr;
    const uint32_t RP = (TM_CONSUMER_WARPS / wpr) * TM_UNR;  // rows per tile
    const uint32_t n_tiles = p.total_rows / RP;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, TM_CONSUMER_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const uint32_t off_qh = RP * p.plane_b[0], off_h = off_qh + RP * p.plane_b[1], off_d = off_h + RP * p.plane_b[2];

    if (warp == TM_CONSUMER_WARPS) {
        // ---------------- producer: weights are immutable, so it starts before the dependency wait
        if (lane == 0) {
            pdl_trigger();
            uint32_t i = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
                const int s = (int)(i % (uint32_t)S);
                if (i >= (uint32_t)S && !mbar_wait(empty + s, ((i / S) - 1) & 1, abort_flag, 2u)) {
                    ok = false;
                    break;
                }
                const uint32_t row = tile * RP;
                int sg = 0;
                while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
                const size_t local = row - (sg ? p.row_end[sg - 1] : 0);
                const WeightView &w = p.w[sg];
                uint8_t *st = ring + (size_t)s * p.stage_bytes;
                mbar_expect_tx(full + s, RP * (p.plane_b[0] + p.plane_b[1] + p.plane_b[2] + p.plane_b[3]));
                bulk_g2s(st, w.q + local * p.plane_b[0], RP * p.plane_b[0], full + s);
                if (p.plane_b[1]) bulk_g2s(st + off_qh, w.qh + local * p.plane_b[1], RP * p.plane_b[1], full + s);
                bulk_g2s(st + off_h, w.hdr + local * p.plane_b[2], RP * p.plane_b[2], full + s);
                if (p.plane_b[3]) bulk_g2s(st + off_d, w.d + local * p.plane_b[3], RP * p.plane_b[3], full + s);
            }
            if (!ok || *abort_flag) {
                // bounded drain: let the copies already issued land before the CTA's shared memory goes away
                const uint32_t issued = i;
                for (uint32_t j = issued > (uint32_t)S ? issued - S : 0; j < issued; ++j) {
                    uint64_t *bar = full + (j % S);
                    for (uint32_t t = 0; t < (1u << 16) && !mbar_test(bar, (j / S) & 1); ++t) __nanosleep(100);
                }
            }
        }
        return;
    }

    // ---------------- consumers
    const int wj = warp % wpr, wr = warp / wpr;
    const uint32_t tau = (uint32_t)wj * 32 + lane;
    const bool active = tau < p.t128;
    pdl_trigger();
    pdl_wait();
    ActRegs<T> act;
    if (active) load_act<T>(p.x, tau, act);

    uint32_t i = 0;
    bool dead = false;  // a wait ran out: keep walking the tiles (the named barriers below must still be met by
                        // every consumer warp) but touch nothing
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
        const int s = (int)(i % (uint32_t)S);
        if (!dead && !mbar_wait(full + s, (i / S) & 1, abort_flag, 1u)) dead = true;
        if (dead) {
            if (wpr > 1) {
                consumer_bar();
                consumer_bar();
            }
            continue;
        }
        const uint8_t *st = ring + (size_t)s * p.stage_bytes;
        WeightView sv;
        sv.type = T;
        sv.m = RP;
        sv.k = p.k;
        sv.nb = p.w[0].nb;
        sv.t128 = p.t128;
        sv.ilv = 0;
        sv.q = st;
        sv.qh = st + off_qh;
        sv.hdr = st + off_h;
        sv.d = st + off_d;
        Raw<T> raw[TM_UNR];
        if (active) {
#pragma unroll
            for (int u = 0; u < TM_UNR; ++u) load_raw<T, false>(sv, (size_t)(wr * TM_UNR + u), tau, raw[u]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);  // the bytes are in registers: the stage may be refilled

        const uint32_t row0 = tile * RP + wr * TM_UNR;
        int sg = 0;
        while (sg + 1 < p.n_segs && row0 >= p.row_end[sg]) ++sg;
        const uint32_t l0 = row0 - (sg ? p.row_end[sg - 1] : 0);
        float acc[TM_UNR];
#pragma unroll
        for (int u = 0; u < TM_UNR; ++u) {
            acc[u] = active ? task_dot<T>(raw[u], act, tau) : 0.0f;
            acc[u] = warp_sum(acc[u]);
        }
        if (wpr > 1) {
            if (lane == 0) {
#pragma unroll
                for (int u = 0; u < TM_UNR; ++u) partial[warp][u] = acc[u];
            }
            consumer_bar();
            if (wj == 0) {
#pragma unroll
                for (int u = 0; u < TM_UNR; ++u) {
                    float v = 0.0f;
                    for (int j = 0; j < wpr; ++j) v += partial[wr * wpr + j][u];
                    acc[u] = v;
                }
            }
            consumer_bar();
        }
        if (wj == 0 && lane == 0) {
            if (p.epilogue == EPI_ROPE_KV) {
                // rows (2i, 2i+1) of one head: a NORM rotation pair (cera/src/backend/cpu.rs:5161-5180)
                const uint32_t pos = *p.f.pos_dev;
                if (sg == 2) {
                    store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0, acc[0]);
                    store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0 + 1, acc[1]);
                } else {
                    const uint32_t pi = (l0 % p.f.head_dim) >> 1;
                    const float cs = p.f.rope_cs[2 * pi], sn = p.f.rope_cs[2 * pi + 1];
                    const float r0 = __fsub_rn(__fmul_rn(acc[0], cs), __fmul_rn(acc[1], sn));
                    const float r1 = __fadd_rn(__fmul_rn(acc[0], sn), __fmul_rn(acc[1], cs));
                    if (sg == 0) {
                        p.y[0][l0] = r0;
                        p.y[0][l0 + 1] = r1;
                    } else {
                        store_kv(p.f.k_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0, r0);
                        store_kv(p.f.k_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0 + 1, r1);
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < TM_UNR; ++u) {
                    float *y = p.y[sg] + l0 + u;
                    *y = p.epilogue == EPI_ADD ? __fadd_rn(*y, acc[u]) : acc[u];
                }
            }
        }
    }
}

// Measured on B200 this kernel ties or trails the register-streaming kernel (8 consumer warps per SM
// cannot issue the dp4a work fast enough to drain the ring), so it is opt-in: CERA_CUDA_GEMV=tma.
bool tma_enabled() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_GEMV");
        return e && strcmp(e, "tma") == 0;
    }();
    return v;
}

template <int T>
int32_t launch_tma_typed(const TmaParams &p, size_t smem, uint32_t n_tiles, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemv_tma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(TM_HEADER_BYTES + TM_SMEM_BUDGET)));
        configured_dev = dev;
    }
    const uint32_t cap = (uint32_t)sm_count();
    count_launch();
    return check_cuda(launch_k(gemv_tma_kernel<T>, dim3(n_tiles < cap ? n_tiles : cap), dim3(TM_THREADS), smem, st, p),
                      "gemv (tma) launch");
}

}  // namespace

// Single-column GEMV through the TMA-staged kernel.  *taken = false: the shape is outside its rules
// (k not a multiple of 128, a row count that is not a whole number of tiles, plane ranges that are not
// multiples of 16 bytes, or a tile too large for two stages); nothing was launched.
int32_t launch_gemv_tma(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                        cudaStream_t st, bool *taken) {
    *taken = false;
    if (!tma_enabled() || n_segs < 1 || n_segs > TM_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    const uint32_t k = segs[0].w.k, t128 = segs[0].w.t128;
    if (!is_block_type(type) || t128 == 0 || t128 > 32 * TM_CONSUMER_WARPS) return CERA_CUDA_OK;
    for (int i = 0; i < n_segs; ++i)
        if (segs[i].w.ilv) return CERA_CUDA_OK;  // rows are copied whole: not for the interleaved K-quant planes
    if ((uintptr_t)x.quants % 16 || (uintptr_t)x.scales % 16 || (uintptr_t)x.sums % 16) return CERA_CUDA_OK;
    TmaParams p{};
    if (fusion) p.f = *fusion;
    int wpr = 1;
    while (wpr * 32u < t128) wpr <<= 1;
    const uint32_t RP = (TM_CONSUMER_WARPS / wpr) * TM_UNR;
    const TypeInfo ti = type_info(type);
    const uint32_t nb = segs[0].w.nb;
    p.plane_b[0] = nb * ti.q_b;
    p.plane_b[1] = nb * ti.qh_b;
    p.plane_b[2] = nb * ti.hdr_b;
    p.plane_b[3] = nb * ti.d_b;
    uint32_t tile_bytes = 0;
    for (int i = 0; i < 4; ++i) {
        if ((RP * p.plane_b[i]) % 16) return CERA_CUDA_OK;
        tile_bytes += RP * p.plane_b[i];
    }
    const int stages = (int)(TM_SMEM_BUDGET / tile_bytes) < TM_MAX_STAGES ? (int)(TM_SMEM_BUDGET / tile_bytes) : TM_MAX_STAGES;
    if (stages < 2) return CERA_CUDA_OK;
    uint32_t rows = 0;
    for (int i = 0; i < n_segs; ++i) {
        if (segs[i].w.type != type || segs[i].w.k != k || segs[i].w.m % RP) return CERA_CUDA_OK;
        p.w[i] = segs[i].w;
        p.y[i] = segs[i].y;
        rows += segs[i].w.m;
        p.row_end[i] = rows;
    }
    if (epilogue == EPI_ROPE_KV) {
        if (n_segs != 3 || wpr != 1 || !p.f.rope_cs || !p.f.pos_dev || !p.f.k_cache || !p.f.v_cache || p.f.head_dim % 2)
            return CERA_CUDA_OK;
    }
    p.n_segs = n_segs;
    p.total_rows = rows;
    p.x = x;
    p.k = k;
    p.t128 = t128;
    p.wpr = wpr;
    p.epilogue = epilogue;
    p.stages = stages;
    p.stage_bytes = tile_bytes;
    *taken = true;
    const size_t smem = TM_HEADER_BYTES + (size_t)stages * tile_bytes;
    CERA_DISPATCH_BLOCK_TYPE(type, return (launch_tma_typed<TT>(p, smem, rows / RP, st)));
    return CERA_CUDA_OK;
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_kernel_status(uint32_t *status_out) {
    if (!status_out) return fail(CERA_CUDA_ERR_BAD_ARG, "kernel_status: null argument");
    unsigned int v = 0;
    CERA_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_tma_status, sizeof(v)));
    v |= gemm_tc_status() << 8;      // bits 8..12: roles of the tcgen05 GEMM
    v |= gemv_exact_status() << 16;  // bit 16: a copy of the reference-order GEMV never arrived
    *status_out = v;
    if (v) return fail(CERA_CUDA_ERR_TIMEOUT, "a bounded device-side wait ran out (status word %u)", v);
    return CERA_CUDA_OK;
}

}  // extern "C"
