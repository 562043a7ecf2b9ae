// Decode GEMV (one activation column), the kernel the decode step runs on.
//
// HBM-bound, and on B200 (about 23 bytes per SM clock) close to instruction-bound
// as well, so the design minimises instructions per weight:
//   * the unit of work is a LANE TASK of 128 weights whose position in k is fixed
//     per lane, so the 128 activation quants, their block scales and the
//     scale-premultiplied block sums are loaded into registers ONCE per kernel;
//   * the low-quant plane is stored piece-major (see WeightView), so lane t's
//     c-th 128-bit load is contiguous with its neighbours': each warp load
//     instruction streams 512 contiguous bytes, L1-bypassing;
//   * UNR rows per warp are fetched before any is consumed (10-20 independent
//     128-bit loads in flight per lane);
//   * K-quant scales are decoded for four sub-blocks at once with word-wide
//     masks (no per-sub-block branches), and each task's result is factored as
//     d * sum_j sc_j * (xs_j * U_j) - dmin * sum_j mn_j * (xs_j * A_j).
// Integer sums U_j (dp4a) are exact.  The f32 combination order is this
// kernel's own: per lane over its task, xor-shuffle tree over the warp, then
// the warps sharing a row in index order.
//
// Arithmetic contract: cera/src/backend/simd.rs:4593-4637 (Q4_0/Q8_0),
// 5693-5878 (Q4_K), 5893-5976 (Q4_1), 5988-6195 (Q6_K).
#include "gemv_task.cuh"

namespace cera {

namespace {

constexpr int RW_WARPS = 8;
constexpr int RW_THREADS = RW_WARPS * 32;
constexpr int RW_MAX_SEGS = 3;

struct RowsParams {
    WeightView w[RW_MAX_SEGS];
    float *y[RW_MAX_SEGS];
    uint32_t row_end[RW_MAX_SEGS];
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k, t128;
    int wpr;  // warps sharing one row: 1, 2, 4 or 8
    int epilogue;
    GemvFusion f;
    TpHook tp;
};

template <int T, int UNR>
__global__ void __launch_bounds__(RW_THREADS) gemv_rows_kernel(const RowsParams p) {
    __shared__ float partial[RW_WARPS][UNR];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpr = p.wpr, rows_per_pass = (RW_WARPS / wpr) * UNR;
    const int wj = warp % wpr, wr = warp / wpr;
    const uint32_t tau = (uint32_t)wj * 32 + lane;
    const bool active = tau < p.t128;

    ActRegs<T> act;
    bool first = true;

    for (uint32_t base = blockIdx.x * rows_per_pass; base < p.total_rows; base += gridDim.x * rows_per_pass) {
        Raw<T> raw[UNR];
        uint32_t local[UNR];
        int seg[UNR];
        bool valid[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t row = base + wr * UNR + u;
            valid[u] = row < p.total_rows;
            int s = 0;
            while (s + 1 < p.n_segs && row >= p.row_end[s]) ++s;
            seg[u] = s;
            local[u] = row - (s ? p.row_end[s - 1] : 0);
            if (valid[u] && active) load_raw<T>(p.w[s], local[u], tau, raw[u]);
        }
        if (first) {
            // the first rows' weight loads are in flight; only now wait for the producer of the activations
            pdl_trigger();
            pdl_wait();
            tp_arrive_wait(p.tp.ctx, p.tp.wait_slot);
            if (active) load_act<T>(p.x, tau, act);
            first = false;
        }
        float acc[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            acc[u] = (valid[u] && active) ? task_dot<T>(raw[u], act, tau) : 0.0f;
            acc[u] = warp_sum(acc[u]);
        }
        if (wpr == 1) {
            if (lane == 0) {
                if (p.epilogue == EPI_ROPE_KV && UNR == 2) {
                    // rows (2i, 2i+1) of one head: a NORM rotation pair (cera/src/backend/cpu.rs:5161-5180)
                    if (valid[0]) {
                        const uint32_t pos = *p.f.pos_dev, l0 = local[0];
                        if (seg[0] == 2) {
                            store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0, acc[0]);
                            store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0 + 1, acc[1]);
                        } else {
                            const uint32_t pi = (l0 % p.f.head_dim) >> 1;
                            const float cs = p.f.rope_cs[2 * pi], sn = p.f.rope_cs[2 * pi + 1];
                            const float r0 = __fsub_rn(__fmul_rn(acc[0], cs), __fmul_rn(acc[1], sn));
                            const float r1 = __fadd_rn(__fmul_rn(acc[0], sn), __fmul_rn(acc[1], cs));
                            if (seg[0] == 0) {
                                p.y[0][l0] = r0;
                                p.y[0][l0 + 1] = r1;
                            } else {
                                store_kv(p.f.k_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0, r0);
                                store_kv(p.f.k_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + l0 + 1, r1);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < UNR; ++u)
                        if (valid[u]) {
                            float *y = p.y[seg[u]] + local[u];
                            const float r = p.epilogue == EPI_ADD ? __fadd_rn(*y, acc[u]) : acc[u];
                            *y = r;
                            if (p.tp.push) tp_push(p.tp.ctx, y, r);
                        }
                }
            }
        } else {
            if (lane == 0) {
#pragma unroll
                for (int u = 0; u < UNR; ++u) partial[warp][u] = acc[u];
            }
            __syncthreads();
            if (wj == 0 && lane < UNR) {
                // lane u of the row's first warp finishes row u of this warp group
                float v = 0.0f;
                for (int j = 0; j < wpr; ++j) v += partial[wr * wpr + j][lane];
                bool ok = false;
                uint32_t loc = 0;
                int sg = 0;
#pragma unroll
                for (int u = 0; u < UNR; ++u)
                    if (u == lane) {
                        ok = valid[u];
                        loc = local[u];
                        sg = seg[u];
                    }
                if (ok) {
                    float *y = p.y[sg] + loc;
                    const float r = p.epilogue == EPI_ADD ? __fadd_rn(*y, v) : v;
                    *y = r;
                    if (p.tp.push) tp_push(p.tp.ctx, y, r);
                }
            }
            __syncthreads();
        }
    }
}

__global__ void rope_table_kernel(const uint32_t *__restrict__ pos_dev, uint32_t half, float ts, const float *__restrict__ ff,
                                  float *__restrict__ table, const float *__restrict__ full) {
    pdl_trigger();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    if (full) {  // host-computed cos / sin of every position: copy this position's row
        const size_t at = ((size_t)*pos_dev * half + i) * 2;
        table[2 * i] = full[at];
        table[2 * i + 1] = full[at + 1];
        return;
    }
    float theta = (float)*pos_dev;
    for (uint32_t s = 0; s < i; ++s) theta = __fmul_rn(theta, ts);
    if (ff) theta = __fdiv_rn(theta, ff[i]);
    float sn, cs;
    sincosf(theta, &sn, &cs);
    table[2 * i] = cs;
    table[2 * i + 1] = sn;
}

template <int T>
int32_t launch_rows_typed(const RowsParams &p, cudaStream_t st) {
    constexpr int UNR = 2;
    const uint32_t cap = (uint32_t)sm_count() * 2;
    const uint32_t rows_per_pass = (RW_WARPS / p.wpr) * UNR;
    const uint32_t passes = (p.total_rows + rows_per_pass - 1) / rows_per_pass;
    count_launch();
    return check_cuda(launch_k(gemv_rows_kernel<T, UNR>, dim3(passes < cap ? passes : cap), dim3(RW_THREADS), 0, st, p),
                      "gemv launch");
}

}  // namespace

// Single-column GEMV over up to three same-typed weight matrices.  *taken = false: the shape is
// outside this kernel's rules (k not a multiple of 128, wider than 8 warps of lane tasks, or a
// fused epilogue whose alignment rules do not hold); nothing was launched and the caller falls back.
int32_t launch_gemv_rows(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                         cudaStream_t st, bool *taken, const TpHook *tp) {
    *taken = false;
    if (n_segs < 1 || n_segs > RW_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    const uint32_t k = segs[0].w.k, t128 = segs[0].w.t128;
    if (!is_block_type(type) || t128 == 0 || t128 > 32 * RW_WARPS) return CERA_CUDA_OK;
    RowsParams p{};
    if (fusion) p.f = *fusion;
    if (tp) p.tp = *tp;
    if ((uintptr_t)x.quants % 16 || (uintptr_t)x.scales % 16 || (uintptr_t)x.sums % 16) return CERA_CUDA_OK;
    uint32_t rows = 0;
    for (int i = 0; i < n_segs; ++i) {
        if (segs[i].w.type != type || segs[i].w.k != k) return CERA_CUDA_OK;
        p.w[i] = segs[i].w;
        p.y[i] = segs[i].y;
        rows += segs[i].w.m;
        p.row_end[i] = rows;
    }
    int wpr = 1;
    while (wpr * 32u < t128) wpr <<= 1;
    if (epilogue == EPI_ROPE_KV) {
        if (n_segs != 3 || wpr != 1 || !p.f.rope_cs || !p.f.pos_dev || !p.f.k_cache || !p.f.v_cache || p.f.head_dim % 2 ||
            segs[0].w.m % 2 || segs[1].w.m % 2 || segs[2].w.m % 2)
            return CERA_CUDA_OK;
    }
    p.n_segs = n_segs;
    p.total_rows = rows;
    p.x = x;
    p.k = k;
    p.t128 = t128;
    p.wpr = wpr;
    p.epilogue = epilogue;
    *taken = true;
    CERA_DISPATCH_BLOCK_TYPE(type, return (launch_rows_typed<TT>(p, st)));
    return CERA_CUDA_OK;
}

int32_t launch_rope_table(const uint32_t *pos_dev, size_t head_dim, float theta_scale, const float *freq_factors,
                          float *table, cudaStream_t st, const float *full_table) {
    const uint32_t half = (uint32_t)(head_dim / 2);
    count_launch();
    return check_cuda(launch_k(rope_table_kernel, dim3((half + 63) / 64), dim3(64), 0, st, pos_dev, half, theta_scale,
                               freq_factors, table, full_table),
                      "rope table launch");
}

}  // namespace cera
