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
#include "formats.cuh"
#include "ops.h"

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
};

// signed x signed and unsigned x signed byte dot products
__device__ __forceinline__ int dp_ss(int w, int a, int c) { return __dp4a(w, a, c); }
__device__ __forceinline__ int dp_us(uint32_t w, int a, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(a), "r"(c));
    return d;
}
__device__ __forceinline__ int dot_lo(const uint4 v, const int4 a) {  // low nibbles
    int s = dp_ss(v.x & 0x0F0F0F0F, a.x, 0);
    s = dp_ss(v.y & 0x0F0F0F0F, a.y, s);
    s = dp_ss(v.z & 0x0F0F0F0F, a.z, s);
    return dp_ss(v.w & 0x0F0F0F0F, a.w, s);
}
// High nibbles without shifting them down: bytes hold 16*nibble (as unsigned), the sum is an
// exact multiple of 16; the caller shifts the accumulated sum once.
__device__ __forceinline__ int dot_hi16(const uint4 v, const int4 a, int s) {
    s = dp_us(v.x & 0xF0F0F0F0u, a.x, s);
    s = dp_us(v.y & 0xF0F0F0F0u, a.y, s);
    s = dp_us(v.z & 0xF0F0F0F0u, a.z, s);
    return dp_us(v.w & 0xF0F0F0F0u, a.w, s);
}
__device__ __forceinline__ int dot_w(const uint32_t w[4], const int4 a, int s) {
    s = dp_ss((int)w[0], a.x, s);
    s = dp_ss((int)w[1], a.y, s);
    s = dp_ss((int)w[2], a.z, s);
    return dp_ss((int)w[3], a.w, s);
}
__device__ __forceinline__ float byte_f(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xFFu); }

// Activations of one lane task, resident in registers for the whole kernel.
template <int T>
struct ActRegs {
    int4 a[8];     // 128 quants: block j = a[2j], a[2j+1]
    float xs[4];   // block scales
    float xb[8];   // Q6_K: -32 * xs_j * (sum of 16 quants) per half; others: xb[j] = xs_j * (sum of 32 quants)
};

template <int T>
__device__ __forceinline__ void load_act(const ActView &x, uint32_t tau, ActRegs<T> &r) {
    const int4 *q = reinterpret_cast<const int4 *>(x.quants + (size_t)tau * 128);
#pragma unroll
    for (int i = 0; i < 8; ++i) r.a[i] = q[i];
    const float4 s = *reinterpret_cast<const float4 *>(x.scales + (size_t)tau * 4);
    r.xs[0] = s.x; r.xs[1] = s.y; r.xs[2] = s.z; r.xs[3] = s.w;
    const int4 sm = *reinterpret_cast<const int4 *>(x.sums + (size_t)tau * 8);  // 8 int16 half sums
    const int h[8] = {(int16_t)(sm.x & 0xFFFF), sm.x >> 16, (int16_t)(sm.y & 0xFFFF), sm.y >> 16,
                      (int16_t)(sm.z & 0xFFFF), sm.z >> 16, (int16_t)(sm.w & 0xFFFF), sm.w >> 16};
    if (T == CERA_TYPE_Q6_K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) r.xb[i] = -32.0f * (r.xs[i >> 1] * (float)h[i]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) r.xb[j] = r.xs[j] * (float)(h[2 * j] + h[2 * j + 1]);
    }
}

// Weight bytes of one lane task.
template <int T>
struct Raw {
    uint4 p[T == CERA_TYPE_Q8_0 ? 8 : 4];  // low-quant pieces
    uint4 hi[(T == CERA_TYPE_Q5_K || T == CERA_TYPE_Q6_K) ? 2 : 1];
    uint4 hd;                               // header words (format specific, see load_raw)
};

template <int T>
__device__ __forceinline__ void load_raw(const WeightView &w, size_t row, uint32_t tau, Raw<T> &r) {
    constexpr int NP = T == CERA_TYPE_Q8_0 ? 8 : 4;
    const TypeInfo ti = type_info(T);
    const uint8_t *q = w.q + row * ((size_t)w.nb * ti.q_b) + (size_t)tau * 16;
#pragma unroll
    for (int c = 0; c < NP; ++c) r.p[c] = ld_stream(q + (size_t)c * w.t128 * 16);
    if (T == CERA_TYPE_Q4_0 || T == CERA_TYPE_Q8_0) {  // 4 half scales
        const uint2 d = __ldg(reinterpret_cast<const uint2 *>(w.hdr + (row * w.nb + 4 * (size_t)tau) * 2));
        r.hd = make_uint4(d.x, d.y, 0, 0);
    } else if (T == CERA_TYPE_Q4_1) {  // 4 x (d, m)
        r.hd = __ldg(reinterpret_cast<const uint4 *>(w.hdr + (row * w.nb + 4 * (size_t)tau) * 4));
    } else if (T == CERA_TYPE_Q4_K || T == CERA_TYPE_Q5_K) {  // d, dmin, scales[12] of super-block tau/2
        const size_t sb = row * w.nb + (tau >> 1);
        r.hd = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb);
        if (T == CERA_TYPE_Q5_K) {
            const uint4 *h = reinterpret_cast<const uint4 *>(w.qh + sb * 32);
            r.hi[0] = __ldg(h);
            r.hi[1] = __ldg(h + 1);
        }
    } else {  // Q6_K: 8 int8 scales of half nh, d in .z
        const size_t sb = row * w.nb + (tau >> 1);
        const uint32_t nh = tau & 1;
        const uint2 sc = __ldg(reinterpret_cast<const uint2 *>(w.hdr + sb * 16 + nh * 8));
        const uint16_t d = __ldg(reinterpret_cast<const uint16_t *>(w.d) + sb);
        r.hd = make_uint4(sc.x, sc.y, d, 0);
        const uint4 *h = reinterpret_cast<const uint4 *>(w.qh + sb * 64 + nh * 32);
        r.hi[0] = __ldg(h);
        r.hi[1] = __ldg(h + 1);
    }
}

// Six-bit scales and mins of sub-blocks 4hf .. 4hf+3, one per byte (cera/src/quant.rs:591-605,
// evaluated for four sub-blocks at once).  y, z, w = scales[0..3], [4..7], [8..11].
__device__ __forceinline__ void kq_quad(const uint4 &h, uint32_t hf, uint32_t &scp, uint32_t &mnp) {
    const uint32_t lo_sc = h.y & 0x3F3F3F3Fu, lo_mn = h.z & 0x3F3F3F3Fu;
    const uint32_t hi_sc = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    const uint32_t hi_mn = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    scp = hf ? hi_sc : lo_sc;
    mnp = hf ? hi_mn : lo_mn;
}

template <int T>
__device__ __forceinline__ float task_dot(const Raw<T> &r, const ActRegs<T> &x, uint32_t tau) {
    if (T == CERA_TYPE_Q4_0 || T == CERA_TYPE_Q4_1) {
        // piece c = block c of the task: low nibbles = elements 0-15, high nibbles = 16-31
        float acc = 0.0f;
        const uint32_t hw[4] = {r.hd.x, r.hd.y, r.hd.z, r.hd.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int U = dot_lo(r.p[c], x.a[2 * c]) + (dot_hi16(r.p[c], x.a[2 * c + 1], 0) >> 4);
            const float t = x.xs[c] * (float)U;
            if (T == CERA_TYPE_Q4_0) {
                const float d = h2f((uint16_t)(hw[c >> 1] >> (16 * (c & 1))));
                acc = fmaf(d, fmaf(-8.0f, x.xb[c], t), acc);  // sum (q-8)*a = U - 8*A
            } else {
                const float d = h2f((uint16_t)(hw[c] & 0xFFFF)), m = h2f((uint16_t)(hw[c] >> 16));
                acc = fmaf(d, t, fmaf(m, x.xb[c], acc));
            }
        }
        return acc;
    }
    if (T == CERA_TYPE_Q8_0) {
        float acc = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t w0[4] = {r.p[2 * c].x, r.p[2 * c].y, r.p[2 * c].z, r.p[2 * c].w};
            const uint32_t w1[4] = {r.p[2 * c + 1].x, r.p[2 * c + 1].y, r.p[2 * c + 1].z, r.p[2 * c + 1].w};
            const int U = dot_w(w1, x.a[2 * c + 1], dot_w(w0, x.a[2 * c], 0));
            const float d = h2f((uint16_t)((c < 2 ? r.hd.x : r.hd.y) >> (16 * (c & 1))));
            acc = fmaf(d, x.xs[c] * (float)U, acc);
        }
        return acc;
    }
    if (T == CERA_TYPE_Q4_K || T == CERA_TYPE_Q5_K) {
        // tau = 2*bi + hf; piece c = (gg = c/2, half = c%2): low nibbles = sub-block 4hf+2gg,
        // high nibbles = sub-block 4hf+2gg+1, elements [16*half, 16*half+16)
        const uint32_t hf = tau & 1;
        int U[4];
        if (T == CERA_TYPE_Q4_K) {
#pragma unroll
            for (int gg = 0; gg < 2; ++gg) {
                U[2 * gg] = dot_lo(r.p[2 * gg], x.a[4 * gg]) + dot_lo(r.p[2 * gg + 1], x.a[4 * gg + 1]);
                U[2 * gg + 1] = dot_hi16(r.p[2 * gg + 1], x.a[4 * gg + 3], dot_hi16(r.p[2 * gg], x.a[4 * gg + 2], 0)) >> 4;
            }
        } else {
#pragma unroll
            for (int gg = 0; gg < 2; ++gg) {
                int ul = 0, uh = 0;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint4 v = r.p[2 * gg + half], b = r.hi[half];
                    const uint32_t vv[4] = {v.x, v.y, v.z, v.w}, bb[4] = {b.x, b.y, b.z, b.w};
                    uint32_t lo[4], hi[4];
                    const int sh = 4 * hf + 2 * gg;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo[i] = (vv[i] & 0x0F0F0F0Fu) | (((bb[i] >> sh) & 0x01010101u) << 4);
                        hi[i] = ((vv[i] >> 4) & 0x0F0F0F0Fu) | (((bb[i] >> (sh + 1)) & 0x01010101u) << 4);
                    }
                    ul = dot_w(lo, x.a[4 * gg + half], ul);
                    uh = dot_w(hi, x.a[4 * gg + 2 + half], uh);
                }
                U[2 * gg] = ul;
                U[2 * gg + 1] = uh;
            }
        }
        uint32_t scp, mnp;
        kq_quad(r.hd, hf, scp, mnp);
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s1 = fmaf(byte_f(scp, j), x.xs[j] * (float)U[j], s1);
            s2 = fmaf(byte_f(mnp, j), x.xb[j], s2);
        }
        const float d = h2f((uint16_t)(r.hd.x & 0xFFFF)), dmin = h2f((uint16_t)(r.hd.x >> 16));
        return fmaf(d, s1, -(dmin * s2));
    }
    // Q6_K: tau = 2*bi + nh; piece c = (gl = c/2, half = c%2): low nibbles = group gl, high nibbles =
    // group gl+2, elements [16*half, +16); qh piece `half` carries bits 2gl (group gl) and 2gl+4 (group gl+2).
    {
        float acc = 0.0f;
#pragma unroll
        for (int gl = 0; gl < 2; ++gl)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint4 v = r.p[2 * gl + half], b = r.hi[half];
                const uint32_t vv[4] = {v.x, v.y, v.z, v.w}, bb[4] = {b.x, b.y, b.z, b.w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    lo[i] = (vv[i] & 0x0F0F0F0Fu) | (((bb[i] >> (2 * gl)) & 0x03030303u) << 4);
                    hi[i] = ((vv[i] >> 4) & 0x0F0F0F0Fu) | (((bb[i] >> (2 * gl + 4)) & 0x03030303u) << 4);
                }
                const int Ul = dot_w(lo, x.a[2 * gl + half], 0), Uh = dot_w(hi, x.a[2 * (gl + 2) + half], 0);
                // scales[8nh + 2j + half]: byte 2j+half of the 8 loaded bytes, j = gl and gl+2
                const float scl = (float)(int8_t)(r.hd.x >> (8 * (2 * gl + half)));
                const float sch = (float)(int8_t)(r.hd.y >> (8 * (2 * gl + half)));
                acc = fmaf(scl, fmaf(x.xs[gl], (float)Ul, x.xb[2 * gl + half]), acc);
                acc = fmaf(sch, fmaf(x.xs[gl + 2], (float)Uh, x.xb[2 * (gl + 2) + half]), acc);
            }
        return h2f((uint16_t)r.hd.z) * acc;
    }
}

__device__ __forceinline__ void store_kv(void *cache, int f16, size_t idx, float v) {
    if (f16) reinterpret_cast<__half *>(cache)[idx] = __float2half_rn(v);
    else reinterpret_cast<float *>(cache)[idx] = v;
}

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
                            *y = p.epilogue == EPI_ADD ? __fadd_rn(*y, acc[u]) : acc[u];
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
                    *y = p.epilogue == EPI_ADD ? __fadd_rn(*y, v) : v;
                }
            }
            __syncthreads();
        }
    }
}

__global__ void rope_table_kernel(const uint32_t *__restrict__ pos_dev, uint32_t half, float ts, const float *__restrict__ ff,
                                  float *__restrict__ table) {
    pdl_trigger();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
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
                         cudaStream_t st, bool *taken) {
    *taken = false;
    if (n_segs < 1 || n_segs > RW_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    const uint32_t k = segs[0].w.k, t128 = segs[0].w.t128;
    if (!is_block_type(type) || t128 == 0 || t128 > 32 * RW_WARPS) return CERA_CUDA_OK;
    RowsParams p{};
    if (fusion) p.f = *fusion;
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
                          float *table, cudaStream_t st) {
    const uint32_t half = (uint32_t)(head_dim / 2);
    count_launch();
    return check_cuda(launch_k(rope_table_kernel, dim3((half + 63) / 64), dim3(64), 0, st, pos_dev, half, theta_scale,
                               freq_factors, table),
                      "rope table launch");
}

}  // namespace cera
