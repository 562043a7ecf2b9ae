// Per-format decode of the planar weight layout into dp4a-ready words.
//
// The unit of work is an ITEM: 32 weights fetched with one 128-bit load of the
// low-quant plane (two for Q8_0) and handled by one lane.  An item always
// splits into two 16-element HALVES, each aligned with 16 consecutive Q8_0
// activation quants, so every integer sum a kernel forms is one of the
// half-block sums the CPU kernels' per-block sums are made of:
//   Q4_0/Q4_1/Q8_0  item b      : halves = elements [0,16) and [16,32) of block b
//   Q4_K/Q5_K       item 8*bi+c : g=c/2, h=c%2; low nibbles = sub-block 2g,
//                                 high nibbles = sub-block 2g+1, elements [16h,16h+16)
//   Q6_K            item 8*bi+c : nh=c/4, gl=(c/2)%2, h=c%2; low nibbles = group gl,
//                                 high nibbles = group gl+2 of half nh, elements [16h,16h+16)
// (block geometry: cera/src/quant.rs:173-293; lane pairing with activations:
// cera/src/backend/simd.rs:5818-5827 and 6042-6061).
#pragma once

#include "common.cuh"

namespace cera {

struct HalfRef {
    int off;      // element offset of the half inside the row (multiple of 16)
    float scale;  // weight-side factor multiplying (float)u * xs
    float mscale; // weight-side factor multiplying xs * (float)a in the correction term
};

template <int T>
struct Fmt;

// Dot of 16 weight bytes (4 words, each byte a small non-negative or signed
// int8) with 16 activation quants.
__device__ __forceinline__ int dot16(const int w[4], const int8_t *a16) {
    const int4 a = __ldg(reinterpret_cast<const int4 *>(a16));
    int s = __dp4a(w[0], a.x, 0);
    s = __dp4a(w[1], a.y, s);
    s = __dp4a(w[2], a.z, s);
    return __dp4a(w[3], a.w, s);
}

// ------------------------------------------------------------------ Q4_0 ----
template <>
struct Fmt<CERA_TYPE_Q4_0> {
    static constexpr int SIGN = 0;  // the -8 recentring is folded into view()
    struct Raw {
        uint4 q;
        uint16_t d;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t b = row * w.nb + item;
        Raw r;
        r.q = ld_stream(w.q + row * ((size_t)w.nb * 16) + q_piece_off(w.t128, 4, (uint32_t)item));
        r.d = __ldg(reinterpret_cast<const uint16_t *>(w.hdr) + b);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        const uint32_t v[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = v[i] & 0x0F0F0F0F;
            hi[i] = (v[i] >> 4) & 0x0F0F0F0F;
        }
        const float d = h2f(r.d);
        h0 = {32 * item, d, 0.0f};
        h1 = {32 * item + 16, d, 0.0f};
    }
    // kernel-view integer sum (what the CPU kernels' dot32 returns): u - 8a
    __device__ static int view(int u, int a) { return u - 8 * a; }
    static constexpr bool WHOLE_BLOCK = true;  // both halves share one block scale
    // cera/src/quant.rs:370-373
    __device__ static float deq(int q, const HalfRef &h) { return __fmul_rn((float)(q - 8), h.scale); }
};

// ------------------------------------------------------------------ Q4_1 ----
template <>
struct Fmt<CERA_TYPE_Q4_1> {
    static constexpr int SIGN = +1;
    struct Raw {
        uint4 q;
        uint32_t dm;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t b = row * w.nb + item;
        Raw r;
        r.q = ld_stream(w.q + row * ((size_t)w.nb * 16) + q_piece_off(w.t128, 4, (uint32_t)item));
        r.dm = __ldg(reinterpret_cast<const uint32_t *>(w.hdr) + b);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        const uint32_t v[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = v[i] & 0x0F0F0F0F;
            hi[i] = (v[i] >> 4) & 0x0F0F0F0F;
        }
        const float d = h2f((uint16_t)(r.dm & 0xFFFF)), m = h2f((uint16_t)(r.dm >> 16));
        h0 = {32 * item, d, m};
        h1 = {32 * item + 16, d, m};
    }
    __device__ static int view(int u, int) { return u; }
    static constexpr bool WHOLE_BLOCK = true;
    // cera/src/quant.rs:431-432: multiply, then add (two roundings)
    __device__ static float deq(int q, const HalfRef &h) {
        return __fadd_rn(__fmul_rn((float)q, h.scale), h.mscale);
    }
};

// ------------------------------------------------------------------ Q8_0 ----
template <>
struct Fmt<CERA_TYPE_Q8_0> {
    static constexpr int SIGN = 0;  // no correction term
    struct Raw {
        uint4 q0, q1;
        uint16_t d;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t b = row * w.nb + item;
        Raw r;
        const uint8_t *rq = w.q + row * ((size_t)w.nb * 32);
        r.q0 = ld_stream(rq + q_piece_off(w.t128, 8, 2u * item));
        r.q1 = ld_stream(rq + q_piece_off(w.t128, 8, 2u * item + 1));
        r.d = __ldg(reinterpret_cast<const uint16_t *>(w.hdr) + b);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        lo[0] = r.q0.x; lo[1] = r.q0.y; lo[2] = r.q0.z; lo[3] = r.q0.w;
        hi[0] = r.q1.x; hi[1] = r.q1.y; hi[2] = r.q1.z; hi[3] = r.q1.w;
        const float d = h2f(r.d);
        h0 = {32 * item, d, 0.0f};
        h1 = {32 * item + 16, d, 0.0f};
    }
    __device__ static int view(int u, int) { return u; }
    static constexpr bool WHOLE_BLOCK = true;
    static constexpr bool SIGNED_BYTES = true;
    // cera/src/quant.rs:498
    __device__ static float deq(int q, const HalfRef &h) { return __fmul_rn((float)q, h.scale); }
};

// 6-bit scale and min of sub-blocks 2g and 2g+1 from the header words
// (y = scales[0..3], z = scales[4..7], w = scales[8..11]).
__device__ __forceinline__ void kq_pair(const uint4 &h, int g, int &sc0, int &mn0, int &sc1, int &mn1) {
    if (g < 2) {
        const int s = 16 * g;  // bit offset of byte 2g
        sc0 = (h.y >> s) & 63;
        mn0 = (h.z >> s) & 63;
        sc1 = (h.y >> (s + 8)) & 63;
        mn1 = (h.z >> (s + 8)) & 63;
    } else {
        const int s = 16 * (g - 2);
        sc0 = ((h.w >> s) & 0xF) | (((h.y >> (s + 6)) & 3) << 4);
        mn0 = ((h.w >> (s + 4)) & 0xF) | (((h.z >> (s + 6)) & 3) << 4);
        sc1 = ((h.w >> (s + 8)) & 0xF) | (((h.y >> (s + 14)) & 3) << 4);
        mn1 = ((h.w >> (s + 12)) & 0xF) | (((h.z >> (s + 14)) & 3) << 4);
    }
}

// ------------------------------------------------------------------ Q4_K ----
template <>
struct Fmt<CERA_TYPE_Q4_K> {
    static constexpr int SIGN = -1;
    struct Raw {
        uint4 q, h;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t sb = sb_index(w, row, item >> 3);
        Raw r;
        r.q = ld_stream(q_piece_ptr(w, row, 4, (uint32_t)item));
        r.h = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        const uint32_t v[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = v[i] & 0x0F0F0F0F;
            hi[i] = (v[i] >> 4) & 0x0F0F0F0F;
        }
        const int c = item & 7, g = c >> 1, half = c & 1;
        int sc0, mn0, sc1, mn1;
        kq_pair(r.h, g, sc0, mn0, sc1, mn1);
        const float d = h2f((uint16_t)(r.h.x & 0xFFFF)), dmin = h2f((uint16_t)(r.h.x >> 16));
        const int base = (item >> 3) * 256 + 64 * g + 16 * half;
        h0 = {base, __fmul_rn(d, (float)sc0), __fmul_rn(dmin, (float)mn0)};
        h1 = {base + 32, __fmul_rn(d, (float)sc1), __fmul_rn(dmin, (float)mn1)};
    }
    __device__ static int view(int u, int) { return u; }
    static constexpr bool WHOLE_BLOCK = false;
    // cera/src/quant.rs:655-663 and 850-861: (d*sc)*q - (dmin*mn)
    __device__ static float deq(int q, const HalfRef &h) {
        return __fsub_rn(__fmul_rn(h.scale, (float)q), h.mscale);
    }
};

// ------------------------------------------------------------------ Q5_K ----
template <>
struct Fmt<CERA_TYPE_Q5_K> {
    static constexpr int SIGN = -1;
    struct Raw {
        uint4 q, h, qh;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t sb = sb_index(w, row, item >> 3);
        Raw r;
        r.q = ld_stream(q_piece_ptr(w, row, 4, (uint32_t)item));
        r.qh = __ldg(reinterpret_cast<const uint4 *>(w.qh + sb * 32 + (item & 1) * 16));
        r.h = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        const int c = item & 7, g = c >> 1, half = c & 1;
        const uint32_t v[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
        const uint32_t b[4] = {r.qh.x, r.qh.y, r.qh.z, r.qh.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = (v[i] & 0x0F0F0F0F) | (((b[i] >> (2 * g)) & 0x01010101) << 4);
            hi[i] = ((v[i] >> 4) & 0x0F0F0F0F) | (((b[i] >> (2 * g + 1)) & 0x01010101) << 4);
        }
        int sc0, mn0, sc1, mn1;
        kq_pair(r.h, g, sc0, mn0, sc1, mn1);
        const float d = h2f((uint16_t)(r.h.x & 0xFFFF)), dmin = h2f((uint16_t)(r.h.x >> 16));
        const int base = (item >> 3) * 256 + 64 * g + 16 * half;
        h0 = {base, __fmul_rn(d, (float)sc0), __fmul_rn(dmin, (float)mn0)};
        h1 = {base + 32, __fmul_rn(d, (float)sc1), __fmul_rn(dmin, (float)mn1)};
    }
    __device__ static int view(int u, int) { return u; }
    static constexpr bool WHOLE_BLOCK = false;
    // cera/src/quant.rs:655-663 and 850-861: (d*sc)*q - (dmin*mn)
    __device__ static float deq(int q, const HalfRef &h) {
        return __fsub_rn(__fmul_rn(h.scale, (float)q), h.mscale);
    }
};

// ------------------------------------------------------------------ Q6_K ----
template <>
struct Fmt<CERA_TYPE_Q6_K> {
    static constexpr int SIGN = -1;
    struct Raw {
        uint4 q, qh, sc;
        uint16_t d;
    };
    __device__ static Raw load(const WeightView &w, size_t row, int item) {
        const size_t sb = sb_index(w, row, item >> 3);
        const int c = item & 7;
        Raw r;
        r.q = ld_stream(q_piece_ptr(w, row, 4, (uint32_t)item));
        r.qh = __ldg(reinterpret_cast<const uint4 *>(w.qh + sb * 64 + (c >> 2) * 32 + (c & 1) * 16));
        r.sc = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb);
        r.d = __ldg(reinterpret_cast<const uint16_t *>(w.d) + sb);
        return r;
    }
    __device__ static void decode(const Raw &r, int item, int lo[4], int hi[4], HalfRef &h0, HalfRef &h1) {
        const int c = item & 7, nh = c >> 2, gl = (c >> 1) & 1, half = c & 1;
        const uint32_t v[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
        const uint32_t b[4] = {r.qh.x, r.qh.y, r.qh.z, r.qh.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = (v[i] & 0x0F0F0F0F) | (((b[i] >> (2 * gl)) & 0x03030303) << 4);
            hi[i] = ((v[i] >> 4) & 0x0F0F0F0F) | (((b[i] >> (2 * gl + 4)) & 0x03030303) << 4);
        }
        // scales[8nh + 2gl + half] and the same +4: words (2nh) and (2nh+1), byte 2gl+half
        const uint32_t w0 = nh ? r.sc.z : r.sc.x, w1 = nh ? r.sc.w : r.sc.y;
        const int sh = 8 * (2 * gl + half);
        const float sc0 = (float)(int8_t)((w0 >> sh) & 0xFF), sc1 = (float)(int8_t)((w1 >> sh) & 0xFF);
        const float d = h2f(r.d), d32 = __fmul_rn(d, 32.0f);
        const int base = (item >> 3) * 256 + 128 * nh + 32 * gl + 16 * half;
        h0 = {base, __fmul_rn(sc0, d), __fmul_rn(d32, sc0)};
        h1 = {base + 64, __fmul_rn(sc1, d), __fmul_rn(d32, sc1)};
    }
    __device__ static int view(int u, int) { return u; }
    static constexpr bool WHOLE_BLOCK = false;
    // cera/src/quant.rs:751-758: (d*sc)*(q-32)
    __device__ static float deq(int q, const HalfRef &h) { return __fmul_rn(h.scale, (float)(q - 32)); }
};

#define CERA_DISPATCH_BLOCK_TYPE(T, ...)                                  \
    switch (T) {                                                          \
        case CERA_TYPE_Q4_0: { constexpr int TT = CERA_TYPE_Q4_0; __VA_ARGS__; } break; \
        case CERA_TYPE_Q4_1: { constexpr int TT = CERA_TYPE_Q4_1; __VA_ARGS__; } break; \
        case CERA_TYPE_Q8_0: { constexpr int TT = CERA_TYPE_Q8_0; __VA_ARGS__; } break; \
        case CERA_TYPE_Q4_K: { constexpr int TT = CERA_TYPE_Q4_K; __VA_ARGS__; } break; \
        case CERA_TYPE_Q5_K: { constexpr int TT = CERA_TYPE_Q5_K; __VA_ARGS__; } break; \
        case CERA_TYPE_Q6_K: { constexpr int TT = CERA_TYPE_Q6_K; __VA_ARGS__; } break; \
        default: return ::cera::fail(CERA_CUDA_ERR_UNSUPPORTED, "no int8 kernel for ggml type %d", (int)(T)); \
    }

}  // namespace cera
