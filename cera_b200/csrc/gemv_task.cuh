// Lane-task arithmetic shared by the single-column GEMV kernels: one lane owns 128 weights whose
// position in k is fixed, keeps the matching 128 activation quants, block scales and premultiplied
// block sums in registers, and turns the task's weight bytes into one f32 contribution.
// Integer sums (dp4a) are exact.  Arithmetic contract: cera/src/backend/simd.rs:4593-4637
// (Q4_0/Q8_0), 5693-5878 (Q4_K), 5893-5976 (Q4_1), 5988-6195 (Q6_K).
#pragma once

#include "formats.cuh"
#include "ops.h"

namespace cera {

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

// Loads of weight bytes: GLOBAL = streaming / read-only global loads, otherwise plain loads (the
// view then points at a shared-memory copy of the same planes).
template <bool GLOBAL>
__device__ __forceinline__ uint4 ldw16(const void *p) {
    if (GLOBAL) return ld_stream(p);
    return *reinterpret_cast<const uint4 *>(p);
}
template <bool GLOBAL, typename V>
__device__ __forceinline__ V ldh(const void *p) {
    if (GLOBAL) return __ldg(reinterpret_cast<const V *>(p));
    return *reinterpret_cast<const V *>(p);
}

template <int T, bool GLOBAL = true>
__device__ __forceinline__ void load_raw(const WeightView &w, size_t row, uint32_t tau, Raw<T> &r) {
    constexpr int NP = T == CERA_TYPE_Q8_0 ? 8 : 4;
    const TypeInfo ti = type_info(T);
#pragma unroll
    for (int c = 0; c < NP; ++c) r.p[c] = ldw16<GLOBAL>(q_piece_ptr(w, row, NP, tau * NP + c));
    if (T == CERA_TYPE_Q4_0 || T == CERA_TYPE_Q8_0) {  // 4 half scales
        const uint2 d = ldh<GLOBAL, uint2>(w.hdr + (row * w.nb + 4 * (size_t)tau) * 2);
        r.hd = make_uint4(d.x, d.y, 0, 0);
    } else if (T == CERA_TYPE_Q4_1) {  // 4 x (d, m)
        r.hd = ldh<GLOBAL, uint4>(w.hdr + (row * w.nb + 4 * (size_t)tau) * 4);
    } else if (T == CERA_TYPE_Q4_K || T == CERA_TYPE_Q5_K) {  // d, dmin, scales[12] of super-block tau/2
        const size_t sb = sb_index(w, row, tau >> 1);
        r.hd = ldh<GLOBAL, uint4>(w.hdr + sb * 16);
        if (T == CERA_TYPE_Q5_K) {
            r.hi[0] = ldh<GLOBAL, uint4>(w.qh + sb * 32);
            r.hi[1] = ldh<GLOBAL, uint4>(w.qh + sb * 32 + 16);
        }
    } else {  // Q6_K: 8 int8 scales of half nh, d in .z
        const size_t sb = sb_index(w, row, tau >> 1);
        const uint32_t nh = tau & 1;
        const uint2 sc = ldh<GLOBAL, uint2>(w.hdr + sb * 16 + nh * 8);
        const uint16_t d = ldh<GLOBAL, uint16_t>(w.d + sb * 2);
        r.hd = make_uint4(sc.x, sc.y, d, 0);
        r.hi[0] = ldh<GLOBAL, uint4>(w.qh + sb * 64 + nh * 32);
        r.hi[1] = ldh<GLOBAL, uint4>(w.qh + sb * 64 + nh * 32 + 16);
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

}  // namespace cera
