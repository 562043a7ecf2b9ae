// CPU oracle: scalar restatement of cera's quantized-matmul hot path.
// TEST INFRASTRUCTURE ONLY - see cera_oracle.h for the scope note and the pins.
//
// Compile with -ffp-contract=off: the Rust originals never contract a*b+c, and
// the places where the reference issues a fused multiply-add are spelled
// std::fmaf here.

#include "cera_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

inline uint32_t f2u(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
inline float u2f(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// ---- half conversions (cera/src/quant.rs:48-73, 117-164, 91-100) ----------

float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu;
    const uint32_t mant = h & 0x3FFu;
    uint32_t rest;
    if (e == 0) {
        if (mant == 0) {
            rest = 0;
        } else {
            // renormalise a subnormal half into a normal single
            const uint32_t shift = (uint32_t)__builtin_clz(mant) - 21u;
            rest = ((113u - shift) << 23) | ((mant << (shift + 13u)) & 0x007FFFFFu);
        }
    } else if (e == 0x1F) {
        rest = mant == 0 ? 0x7F800000u : (0x7FC00000u | (mant << 13));
    } else {
        rest = ((e + 112u) << 23) | (mant << 13);
    }
    return u2f(sign | rest);
}

uint16_t f2h(float v) {
    const uint32_t b = f2u(v);
    const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    const int32_t ex = (int32_t)((b >> 23) & 0xFFu);
    const uint32_t mant = b & 0x007FFFFFu;
    if (ex == 0xFF) {
        if (mant == 0) return sign | 0x7C00u;
        return (uint16_t)(sign | 0x7E00u | ((mant >> 13) & 0x3FFu));
    }
    int32_t e = ex - 127 + 15;
    if (e >= 0x1F) return sign | 0x7C00u;
    if (e <= 0) {
        if (e < -10) return sign;
        const uint32_t m = mant | 0x00800000u;
        const uint32_t shift = (uint32_t)(14 - e);
        const uint32_t halfbit = (m >> (shift - 1)) & 1u;
        const uint32_t sticky = (m & ((1u << (shift - 1)) - 1u)) != 0 ? 1u : 0u;
        const uint32_t odd = (m >> shift) & 1u;
        const uint32_t round = halfbit & (sticky | odd);
        return (uint16_t)(sign | ((m >> shift) + round));
    }
    const uint32_t lsb = (mant >> 13) & 1u;
    const uint32_t rounded = mant + 0x0FFFu + lsb;
    const uint32_t carry = rounded >> 23;
    const uint32_t e2 = (uint32_t)e + carry;
    if (e2 >= 0x1F) return sign | 0x7C00u;
    return (uint16_t)(sign | (e2 << 10) | ((rounded >> 13) & 0x3FFu));
}

float bf2f(uint16_t bits) {
    const uint32_t quiet = ((bits & 0x7FFFu) > 0x7F80u) ? 0x00400000u : 0u;
    return u2f(((uint32_t)bits << 16) | quiet);
}

// ---- block geometry (cera/src/tensor.rs:3-62) -----------------------------

int blk_elems(int t) {
    switch (t) {
        case CERA_T_F32: case CERA_T_F16: case CERA_T_BF16: return 1;
        case CERA_T_Q4_0: case CERA_T_Q4_1: case CERA_T_Q8_0: return 32;
        case CERA_T_Q4_K: case CERA_T_Q5_K: case CERA_T_Q6_K: return 256;
        default: return 0;
    }
}
int blk_bytes(int t) {
    switch (t) {
        case CERA_T_F32: return 4;
        case CERA_T_F16: case CERA_T_BF16: return 2;
        case CERA_T_Q4_0: return 18;
        case CERA_T_Q4_1: return 20;
        case CERA_T_Q8_0: return 34;
        case CERA_T_Q4_K: return 144;
        case CERA_T_Q5_K: return 176;
        case CERA_T_Q6_K: return 210;
        default: return 0;
    }
}

// 6-bit scale/min unpacking shared by Q4_K and Q5_K (cera/src/quant.rs:591-605).
void kscales(const uint8_t *s, uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 4; ++j) {
        sc[j] = s[j] & 63;
        mn[j] = s[j + 4] & 63;
    }
    for (int j = 4; j < 8; ++j) {
        sc[j] = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        mn[j] = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// Quants of one 32-element activation-aligned group of a weight row, as the
// int8 kernels see them.  `g32` counts 32-element groups from the row start.
// Q4_0: q-8; Q8_0: signed; Q4_1/Q4_K/Q5_K: unsigned; Q6_K: unsigned 0..63.
void group_quants(int type, const uint8_t *row, size_t g32, int32_t q[32]) {
    switch (type) {
        case CERA_T_Q4_0: {
            const uint8_t *b = row + g32 * 18 + 2;
            for (int t = 0; t < 16; ++t) {
                q[t] = (b[t] & 15) - 8;
                q[t + 16] = (b[t] >> 4) - 8;
            }
        } break;
        case CERA_T_Q4_1: {
            const uint8_t *b = row + g32 * 20 + 4;
            for (int t = 0; t < 16; ++t) {
                q[t] = b[t] & 15;
                q[t + 16] = b[t] >> 4;
            }
        } break;
        case CERA_T_Q8_0: {
            const int8_t *b = (const int8_t *)(row + g32 * 34 + 2);
            for (int t = 0; t < 32; ++t) q[t] = b[t];
        } break;
        case CERA_T_Q4_K: {
            const uint8_t *blk = row + (g32 / 8) * 144;
            const size_t s = g32 % 8;
            const uint8_t *qs = blk + 16 + (s / 2) * 32;
            for (int l = 0; l < 32; ++l) q[l] = (s & 1) ? (qs[l] >> 4) : (qs[l] & 15);
        } break;
        case CERA_T_Q5_K: {
            const uint8_t *blk = row + (g32 / 8) * 176;
            const size_t s = g32 % 8;
            const uint8_t *qh = blk + 16;
            const uint8_t *qs = blk + 48 + (s / 2) * 32;
            for (int l = 0; l < 32; ++l) {
                const int lo = (s & 1) ? (qs[l] >> 4) : (qs[l] & 15);
                q[l] = lo + 16 * ((qh[l] >> s) & 1);
            }
        } break;
        case CERA_T_Q6_K: {
            const uint8_t *blk = row + (g32 / 8) * 210;
            const size_t r = g32 % 8, nh = r / 4, g = r % 4;
            const uint8_t *ql = blk + nh * 64 + (g & 1) * 32;
            const uint8_t *qh = blk + 128 + nh * 32;
            for (int l = 0; l < 32; ++l) {
                const int lo = (g < 2) ? (ql[l] & 15) : (ql[l] >> 4);
                q[l] = lo | (((qh[l] >> (2 * g)) & 3) << 4);
            }
        } break;
        default:
            for (int t = 0; t < 32; ++t) q[t] = 0;
    }
}

// ---- dequantizers ---------------------------------------------------------

void dq_q4_0(const uint8_t *b, float *o) {  // quant.rs:364-376
    const float d = h2f(rd16(b));
    for (int i = 0; i < 16; ++i) {
        o[i] = (float)((b[2 + i] & 15) - 8) * d;
        o[i + 16] = (float)((b[2 + i] >> 4) - 8) * d;
    }
}
void dq_q4_1(const uint8_t *b, float *o) {  // quant.rs:422-435
    const float d = h2f(rd16(b)), m = h2f(rd16(b + 2));
    for (int i = 0; i < 16; ++i) {
        o[i] = (float)(b[4 + i] & 15) * d + m;
        o[i + 16] = (float)(b[4 + i] >> 4) * d + m;
    }
}
void dq_q8_0(const uint8_t *b, float *o) {  // quant.rs:494-501
    const float d = h2f(rd16(b));
    for (int i = 0; i < 32; ++i) o[i] = (float)(int8_t)b[2 + i] * d;
}
void dq_q4_k(const uint8_t *b, float *o) {  // quant.rs:610-670
    const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
    uint8_t sc[8], mn[8];
    kscales(b + 4, sc, mn);
    const uint8_t *qs = b + 16;
    for (int j = 0; j < 4; ++j) {
        const float d1 = d * (float)sc[2 * j], m1 = dmin * (float)mn[2 * j];
        const float d2 = d * (float)sc[2 * j + 1], m2 = dmin * (float)mn[2 * j + 1];
        for (int l = 0; l < 32; ++l) {
            o[64 * j + l] = d1 * (float)(qs[32 * j + l] & 15) - m1;
            o[64 * j + 32 + l] = d2 * (float)(qs[32 * j + l] >> 4) - m2;
        }
    }
}
void dq_q5_k(const uint8_t *b, float *o) {  // quant.rs:836-870
    const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
    uint8_t sc[8], mn[8];
    kscales(b + 4, sc, mn);
    const uint8_t *qh = b + 16, *qs = b + 48;
    for (int j = 0; j < 4; ++j) {
        const float d1 = d * (float)sc[2 * j], m1 = dmin * (float)mn[2 * j];
        const float d2 = d * (float)sc[2 * j + 1], m2 = dmin * (float)mn[2 * j + 1];
        for (int l = 0; l < 32; ++l) {
            const float h1 = ((qh[l] >> (2 * j)) & 1) ? 16.0f : 0.0f;
            const float h2 = ((qh[l] >> (2 * j + 1)) & 1) ? 16.0f : 0.0f;
            o[64 * j + l] = d1 * ((float)(qs[32 * j + l] & 15) + h1) - m1;
            o[64 * j + 32 + l] = d2 * ((float)(qs[32 * j + l] >> 4) + h2) - m2;
        }
    }
}
void dq_q6_k(const uint8_t *b, float *o) {  // quant.rs:735-767
    const float d = h2f(rd16(b + 208));
    const int8_t *sc = (const int8_t *)(b + 192);
    for (int nh = 0; nh < 2; ++nh) {
        const uint8_t *ql = b + 64 * nh, *qh = b + 128 + 32 * nh;
        const int8_t *s = sc + 8 * nh;
        float *y = o + 128 * nh;
        for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int8_t q1 = (int8_t)(((ql[l] & 15) | ((qh[l] & 3) << 4)) - 32);
            const int8_t q2 = (int8_t)(((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32);
            const int8_t q3 = (int8_t)(((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            const int8_t q4 = (int8_t)(((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
            y[l] = d * (float)s[is] * (float)q1;
            y[l + 32] = d * (float)s[is + 2] * (float)q2;
            y[l + 64] = d * (float)s[is + 4] * (float)q3;
            y[l + 96] = d * (float)s[is + 6] * (float)q4;
        }
    }
}

// ---- weight quantizers (cera/src/convert/quantize.rs) ---------------------

inline float sclamp(float v, float lo, float hi) {  // quantize.rs:12-20
    if (std::isnan(v) || v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

void wq_q8_0(const float *in, uint8_t *out) {  // quantize.rs:344-387
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = std::fabs(in[i]) > amax ? std::fabs(in[i]) : amax;
    const uint16_t dh = f2h(amax / 127.0f);
    out[0] = dh & 0xFF;
    out[1] = dh >> 8;
    const float d = h2f(dh);
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 32; ++i)
        out[2 + i] = (uint8_t)(int8_t)sclamp(std::round(in[i] * id), -127.0f, 127.0f);
}
void wq_q4_0(const float *in, uint8_t *out) {  // quantize.rs:523-570
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = std::fabs(in[i]) > amax ? std::fabs(in[i]) : amax;
    const uint16_t dh = f2h(amax / 8.0f);
    out[0] = dh & 0xFF;
    out[1] = dh >> 8;
    const float d = h2f(dh);
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 16; ++i) {
        const uint8_t q0 = (uint8_t)sclamp(std::floor(in[i] * id + 8.5f), 0.0f, 15.0f);
        const uint8_t q1 = (uint8_t)sclamp(std::floor(in[i + 16] * id + 8.5f), 0.0f, 15.0f);
        out[2 + i] = (uint8_t)(q0 | (q1 << 4));
    }
}
// ggml quantize_row_q4_1_ref (published algorithm; no counterpart in cera).
void wq_q4_1(const float *in, uint8_t *out) {
    float mn = in[0], mx = in[0];
    for (int i = 1; i < 32; ++i) {
        mn = in[i] < mn ? in[i] : mn;
        mx = in[i] > mx ? in[i] : mx;
    }
    const float d = (mx - mn) / 15.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    const uint16_t dh = f2h(d), mh = f2h(mn);
    out[0] = dh & 0xFF;
    out[1] = dh >> 8;
    out[2] = mh & 0xFF;
    out[3] = mh >> 8;
    for (int i = 0; i < 16; ++i) {
        const uint8_t q0 = (uint8_t)sclamp(std::floor((in[i] - mn) * id + 0.5f), 0.0f, 15.0f);
        const uint8_t q1 = (uint8_t)sclamp(std::floor((in[i + 16] - mn) * id + 0.5f), 0.0f, 15.0f);
        out[4 + i] = (uint8_t)(q0 | (q1 << 4));
    }
}

// Shared front half of the Q4_K / Q5_K quantizers (quantize.rs:738-816, 870-948):
// per-sub-block extrema, the two super-scales, 6-bit scales/mins and their packing.
void kq_header(const float *in, float qmax, uint8_t *out, float &ad, float &admin, uint8_t qsc[8],
               uint8_t qmn[8]) {
    float smin[8], smax[8];
    for (int s = 0; s < 8; ++s) {
        float lo = in[32 * s], hi = in[32 * s];
        for (int l = 1; l < 32; ++l) {
            const float x = in[32 * s + l];
            if (x < lo) lo = x;
            if (x > hi) hi = x;
        }
        smin[s] = lo;
        smax[s] = hi;
    }
    float max_range = 0.0f, max_min_abs = 0.0f;
    for (int s = 0; s < 8; ++s) {
        const float eff = std::fmin(smin[s], 0.0f);
        const float range = smax[s] - eff;
        if (range > max_range) max_range = range;
        if (-eff > max_min_abs) max_min_abs = -eff;
    }
    const uint16_t dh = f2h((max_range / 63.0f) / qmax), mh = f2h(max_min_abs / 63.0f);
    out[0] = dh & 0xFF;
    out[1] = dh >> 8;
    out[2] = mh & 0xFF;
    out[3] = mh >> 8;
    ad = h2f(dh);
    admin = h2f(mh);
    for (int s = 0; s < 8; ++s) {
        const float eff = std::fmin(smin[s], 0.0f);
        const float range = smax[s] - eff;
        qsc[s] = ad > 0.0f ? (uint8_t)sclamp(std::round((range / qmax) / ad), 0.0f, 63.0f) : 0;
        qmn[s] = admin > 0.0f ? (uint8_t)sclamp(std::round((-eff) / admin), 0.0f, 63.0f) : 0;
    }
    for (int j = 0; j < 4; ++j) {
        out[4 + j] = (uint8_t)((qsc[j] & 0x3F) | (((qsc[j + 4] & 0x30) >> 4) << 6));
        out[8 + j] = (uint8_t)((qmn[j] & 0x3F) | (((qmn[j + 4] & 0x30) >> 4) << 6));
        out[12 + j] = (uint8_t)((qsc[j + 4] & 0x0F) | ((qmn[j + 4] & 0x0F) << 4));
    }
}
void wq_q4_k(const float *in, uint8_t *out) {  // quantize.rs:719-846
    float ad, admin;
    uint8_t qsc[8], qmn[8];
    kq_header(in, 15.0f, out, ad, admin, qsc, qmn);
    for (int j = 0; j < 4; ++j) {
        const float sc0 = (float)qsc[2 * j] * ad, sc1 = (float)qsc[2 * j + 1] * ad;
        const float m0 = (float)qmn[2 * j] * admin, m1 = (float)qmn[2 * j + 1] * admin;
        for (int l = 0; l < 32; ++l) {
            const uint8_t q0 =
                sc0 > 0.0f ? (uint8_t)sclamp(std::round((in[64 * j + l] + m0) / sc0), 0.0f, 15.0f) : 0;
            const uint8_t q1 =
                sc1 > 0.0f ? (uint8_t)sclamp(std::round((in[64 * j + 32 + l] + m1) / sc1), 0.0f, 15.0f)
                           : 0;
            out[16 + 32 * j + l] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}
void wq_q5_k(const float *in, uint8_t *out) {  // quantize.rs:851-988
    float ad, admin;
    uint8_t qsc[8], qmn[8];
    kq_header(in, 31.0f, out, ad, admin, qsc, qmn);
    uint8_t *qh = out + 16, *qs = out + 48;
    std::memset(qh, 0, 32);
    for (int j = 0; j < 4; ++j) {
        const float sc0 = (float)qsc[2 * j] * ad, sc1 = (float)qsc[2 * j + 1] * ad;
        const float m0 = (float)qmn[2 * j] * admin, m1 = (float)qmn[2 * j + 1] * admin;
        for (int l = 0; l < 32; ++l) {
            const uint8_t q0 =
                sc0 > 0.0f ? (uint8_t)sclamp(std::round((in[64 * j + l] + m0) / sc0), 0.0f, 31.0f) : 0;
            const uint8_t q1 =
                sc1 > 0.0f ? (uint8_t)sclamp(std::round((in[64 * j + 32 + l] + m1) / sc1), 0.0f, 31.0f)
                           : 0;
            qs[32 * j + l] = (uint8_t)((q0 & 15) | ((q1 & 15) << 4));
            qh[l] |= (uint8_t)((((q0 >> 4) & 1) << (2 * j)) | (((q1 >> 4) & 1) << (2 * j + 1)));
        }
    }
}
void wq_q6_k(const float *in, uint8_t *out) {  // quantize.rs:993-1094
    float smax[16];
    float max_all = 0.0f;
    for (int s = 0; s < 16; ++s) {
        float amax = 0.0f;
        for (int l = 0; l < 16; ++l) {
            const float a = std::fabs(in[16 * s + l]);
            if (a > amax) amax = a;
        }
        smax[s] = amax;
        if (amax > max_all) max_all = amax;
    }
    const uint16_t dh = f2h(max_all / (128.0f * 32.0f));
    out[208] = dh & 0xFF;
    out[209] = dh >> 8;
    const float ad = h2f(dh);
    const float id = ad != 0.0f ? 1.0f / ad : 0.0f;
    int8_t qsc[16];
    for (int s = 0; s < 16; ++s) {
        qsc[s] = (int8_t)sclamp(std::round(smax[s] * id / 32.0f), -128.0f, 127.0f);
        out[192 + s] = (uint8_t)qsc[s];
    }
    for (int nh = 0; nh < 2; ++nh) {
        uint8_t *ql = out + 64 * nh, *qh = out + 128 + 32 * nh;
        for (int l = 0; l < 32; ++l) {
            uint8_t q[4];
            for (int g = 0; g < 4; ++g) {
                const float sc = (float)qsc[8 * nh + l / 16 + 2 * g] * ad;
                const float isc = sc != 0.0f ? 1.0f / sc : 0.0f;
                q[g] = (uint8_t)sclamp(std::floor(in[128 * nh + 32 * g + l] * isc + 32.5f), 0.0f, 63.0f);
            }
            ql[l] = (uint8_t)((q[0] & 15) | ((q[2] & 15) << 4));
            ql[l + 32] = (uint8_t)((q[1] & 15) | ((q[3] & 15) << 4));
            qh[l] = (uint8_t)(((q[0] >> 4) & 3) | (((q[1] >> 4) & 3) << 2) | (((q[2] >> 4) & 3) << 4) |
                              (((q[3] >> 4) & 3) << 6));
        }
    }
}

// ---- x86 int8 tier, lane for lane -----------------------------------------
// One 256-bit dot (cera/src/backend/simd.rs:6319-6341): lane L holds the exact
// integer sum of products of elements 4L..4L+3.
inline void dot_lanes(const int32_t q[32], const int8_t *a, float lanes[8]) {
    for (int L = 0; L < 8; ++L) {
        int32_t s = 0;
        for (int t = 0; t < 4; ++t) s += q[4 * L + t] * (int32_t)a[4 * L + t];
        lanes[L] = (float)s;
    }
}
inline float hsum8(const float v[8]) {  // simd.rs:4545-4553
    const float s0 = v[4] + v[0], s1 = v[5] + v[1], s2 = v[6] + v[2], s3 = v[7] + v[3];
    const float t0 = s0 + s2, t1 = s1 + s3;
    return t0 + t1;
}
inline int32_t isum(const int8_t *a, int n) {
    int32_t s = 0;
    for (int i = 0; i < n; ++i) s += a[i];
    return s;
}

// Q4_0 / Q8_0: one 8-lane accumulator per (row, column) (simd.rs:4593-4637,
// 4777-4905 - the tiled GEMM keeps the same per-cell chain).
float cell_q40_q80(int type, const uint8_t *row, const float *xs, const int8_t *xq, size_t nb) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int bsz = type == CERA_T_Q4_0 ? 18 : 34;
    for (size_t b = 0; b < nb; ++b) {
        int32_t q[32];
        float lanes[8];
        group_quants(type, row, b, q);
        dot_lanes(q, xq + 32 * b, lanes);
        const float scale = h2f(rd16(row + b * bsz)) * xs[b];
        for (int L = 0; L < 8; ++L) acc[L] = std::fmaf(lanes[L], scale, acc[L]);
    }
    return hsum8(acc);
}

// Q4_1 (simd.rs:5893-5976): single chain, block-sum term added.
float cell_q4_1(const uint8_t *row, const float *xs, const int8_t *xq, size_t nb) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float macc = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        int32_t q[32];
        float lanes[8];
        group_quants(CERA_T_Q4_1, row, b, q);
        dot_lanes(q, xq + 32 * b, lanes);
        const float d = h2f(rd16(row + 20 * b)), mm = h2f(rd16(row + 20 * b + 2));
        const float scale = xs[b] * d;
        for (int L = 0; L < 8; ++L) acc[L] = std::fmaf(lanes[L], scale, acc[L]);
        macc += xs[b] * mm * (float)isum(xq + 32 * b, 32);
    }
    return hsum8(acc) + macc;
}

// Q4_K / Q5_K (simd.rs:5693-5878).  fast == the n==1 decode path: four
// round-robin accumulators tree-added at the end.
float cell_q45_k(int type, const uint8_t *row, const float *xs, const int8_t *xq, size_t sb,
                 bool fast) {
    const int bsz = type == CERA_T_Q4_K ? 144 : 176;
    float facc[4][8] = {};
    float macc = 0.0f;
    int slot = 0;
    for (size_t bi = 0; bi < sb; ++bi) {
        const uint8_t *blk = row + bi * bsz;
        const float d = h2f(rd16(blk)), dmin = h2f(rd16(blk + 2));
        uint8_t sc[8], mn[8];
        kscales(blk + 4, sc, mn);
        for (int s = 0; s < 8; ++s) {
            const size_t xb = bi * 8 + s;
            int32_t q[32];
            float lanes[8];
            group_quants(type, row, xb, q);
            dot_lanes(q, xq + 32 * xb, lanes);
            const float dsc = d * (float)sc[s], dmn = dmin * (float)mn[s];
            const float scale = xs[xb] * dsc;
            float *acc = facc[fast ? slot : 0];
            for (int L = 0; L < 8; ++L) acc[L] = std::fmaf(lanes[L], scale, acc[L]);
            macc += xs[xb] * dmn * (float)isum(xq + 32 * xb, 32);
            slot = (slot + 1) & 3;
        }
    }
    if (!fast) return hsum8(facc[0]) - macc;
    float f[8];
    for (int L = 0; L < 8; ++L) f[L] = (facc[0][L] + facc[1][L]) + (facc[2][L] + facc[3][L]);
    return hsum8(f) - macc;
}

// Q6_K (simd.rs:5988-6195): lanes 0-3 carry scale sc0, lanes 4-7 sc1.
float cell_q6_k(const uint8_t *row, const float *xs, const int8_t *xq, size_t sb, bool fast) {
    float facc[4][8] = {};
    float macc = 0.0f;
    int slot = 0;
    for (size_t bi = 0; bi < sb; ++bi) {
        const uint8_t *blk = row + bi * 210;
        const int8_t *scales = (const int8_t *)(blk + 192);
        const float d = h2f(rd16(blk + 208));
        const float d32 = d * 32.0f;
        for (int nh = 0; nh < 2; ++nh) {
            for (int g = 0; g < 4; ++g) {
                const size_t xb = bi * 8 + nh * 4 + g;
                int32_t q[32];
                float lanes[8];
                group_quants(CERA_T_Q6_K, row, xb, q);
                dot_lanes(q, xq + 32 * xb, lanes);
                const float sc0 = (float)scales[nh * 8 + 2 * g], sc1 = (float)scales[nh * 8 + 2 * g + 1];
                const float s0 = (sc0 * d) * xs[xb], s1 = (sc1 * d) * xs[xb];
                float *acc = facc[fast ? slot : 0];
                for (int L = 0; L < 4; ++L) acc[L] = std::fmaf(lanes[L], s0, acc[L]);
                for (int L = 4; L < 8; ++L) acc[L] = std::fmaf(lanes[L], s1, acc[L]);
                const float sx0 = (float)isum(xq + 32 * xb, 16), sx1 = (float)isum(xq + 32 * xb + 16, 16);
                macc += xs[xb] * d32 * (sc0 * sx0 + sc1 * sx1);
                slot = (slot + 1) & 3;
            }
        }
    }
    if (!fast) return hsum8(facc[0]) - macc;
    float f[8];
    for (int L = 0; L < 8; ++L) f[L] = (facc[0][L] + facc[1][L]) + (facc[2][L] + facc[3][L]);
    return hsum8(f) - macc;
}

float cell(int type, const uint8_t *row, const float *xs, const int8_t *xq, size_t k, bool fast) {
    switch (type) {
        case CERA_T_Q4_0: case CERA_T_Q8_0: return cell_q40_q80(type, row, xs, xq, k / 32);
        case CERA_T_Q4_1: return cell_q4_1(row, xs, xq, k / 32);
        case CERA_T_Q4_K: case CERA_T_Q5_K: return cell_q45_k(type, row, xs, xq, k / 256, fast);
        case CERA_T_Q6_K: return cell_q6_k(row, xs, xq, k / 256, fast);
        default: return std::numeric_limits<float>::quiet_NaN();
    }
}

bool int8_type(int t) {
    return t == CERA_T_Q4_0 || t == CERA_T_Q4_1 || t == CERA_T_Q8_0 || t == CERA_T_Q4_K ||
           t == CERA_T_Q5_K || t == CERA_T_Q6_K;
}

// Q5_K against f32 activations (quant.rs:892-937).
float q5k_dot_f32(const uint8_t *b, const float *y) {
    const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
    uint8_t sc[8], mn[8];
    kscales(b + 4, sc, mn);
    const uint8_t *qh = b + 16, *qs = b + 48;
    float sumf = 0.0f;
    for (int j = 0; j < 4; ++j) {
        const float sc1 = sc[2 * j], mn1 = mn[2 * j], sc2 = sc[2 * j + 1], mn2 = mn[2 * j + 1];
        float sum1 = 0, sum2 = 0, smn1 = 0, smn2 = 0;
        for (int l = 0; l < 32; ++l) {
            const float h1 = ((qh[l] >> (2 * j)) & 1) ? 16.0f : 0.0f;
            const float h2 = ((qh[l] >> (2 * j + 1)) & 1) ? 16.0f : 0.0f;
            const float q1 = (float)(qs[32 * j + l] & 15) + h1;
            const float q2 = (float)(qs[32 * j + l] >> 4) + h2;
            sum1 += q1 * y[64 * j + l];
            sum2 += q2 * y[64 * j + 32 + l];
            smn1 += y[64 * j + l];
            smn2 += y[64 * j + 32 + l];
        }
        sumf += d * (sc1 * sum1 + sc2 * sum2) - dmin * (mn1 * smn1 + mn2 * smn2);
    }
    return sumf;
}

template <class F>
void par_rows(size_t m, int n_threads, F f) {
    if (n_threads <= 1 || m < 64) {
        for (size_t i = 0; i < m; ++i) f(i);
        return;
    }
    std::vector<std::thread> th;
    const size_t per = (m + n_threads - 1) / n_threads;
    for (int t = 0; t < n_threads; ++t) {
        const size_t lo = t * per, hi = std::min(m, lo + per);
        if (lo >= hi) break;
        th.emplace_back([=] {
            for (size_t i = lo; i < hi; ++i) f(i);
        });
    }
    for (auto &t : th) t.join();
}

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

}  // namespace

// ===========================================================================
extern "C" {

int cera_oracle_block_elems(int t) { return blk_elems(t); }
int cera_oracle_block_bytes(int t) { return blk_bytes(t); }
size_t cera_oracle_row_bytes(int t, size_t k) {
    const int e = blk_elems(t);
    return e ? (k / e) * (size_t)blk_bytes(t) : 0;
}
float cera_oracle_f16_to_f32(uint16_t b) { return h2f(b); }
uint16_t cera_oracle_f32_to_f16(float v) { return f2h(v); }
float cera_oracle_bf16_to_f32(uint16_t b) { return bf2f(b); }

int cera_oracle_dequantize_row(int type, const uint8_t *src, size_t k, float *dst) {
    const int e = blk_elems(type), bb = blk_bytes(type);
    if (!e || k % e) return -1;
    for (size_t b = 0; b < k / e; ++b) {
        const uint8_t *p = src + b * bb;
        float *o = dst + b * e;
        switch (type) {
            case CERA_T_F32: std::memcpy(o, p, 4); break;
            case CERA_T_F16: *o = h2f(rd16(p)); break;
            case CERA_T_BF16: *o = bf2f(rd16(p)); break;
            case CERA_T_Q4_0: dq_q4_0(p, o); break;
            case CERA_T_Q4_1: dq_q4_1(p, o); break;
            case CERA_T_Q8_0: dq_q8_0(p, o); break;
            case CERA_T_Q4_K: dq_q4_k(p, o); break;
            case CERA_T_Q5_K: dq_q5_k(p, o); break;
            case CERA_T_Q6_K: dq_q6_k(p, o); break;
            default: return -1;
        }
    }
    return 0;
}

int cera_oracle_quantize_weights(int type, const float *in, size_t n, uint8_t *out) {
    const int e = blk_elems(type), bb = blk_bytes(type);
    if (!e || e == 1 || n % e) return -1;
    for (size_t b = 0; b < n / e; ++b) {
        const float *i = in + b * e;
        uint8_t *o = out + b * bb;
        switch (type) {
            case CERA_T_Q8_0: wq_q8_0(i, o); break;
            case CERA_T_Q4_0: wq_q4_0(i, o); break;
            case CERA_T_Q4_1: wq_q4_1(i, o); break;
            case CERA_T_Q4_K: wq_q4_k(i, o); break;
            case CERA_T_Q5_K: wq_q5_k(i, o); break;
            case CERA_T_Q6_K: wq_q6_k(i, o); break;
            default: return -1;
        }
    }
    return 0;
}

void cera_oracle_quantize_q8_0(const float *x, size_t k, float *scales, int8_t *quants) {
    for (size_t b = 0; b < k / 32; ++b) {
        const float *v = x + 32 * b;
        float amax = 0.0f;
        for (int t = 0; t < 32; ++t) {
            const float a = std::fabs(v[t]);
            // f32::max semantics: a NaN operand is ignored.
            if (!(a != a)) amax = a > amax ? a : amax;
        }
        const float d = amax / 127.0f;
        const float r = 1.0f / d;
        const float id = (d != 0.0f && std::isfinite(r)) ? r : 0.0f;
        scales[b] = h2f(f2h(d));
        for (int t = 0; t < 32; ++t) {
            float p = std::nearbyintf(v[t] * id);  // round-half-even in the default mode
            int8_t q;
            if (p != p) q = 0;
            else q = (int8_t)(p < -128.0f ? -128.0f : (p > 127.0f ? 127.0f : p));
            quants[32 * b + t] = q;
        }
    }
}

void cera_oracle_quantize_columns(const float *mat, size_t dim, size_t n, float *scales,
                                  int8_t *quants) {
    std::vector<float> col(dim);
    for (size_t j = 0; j < n; ++j) {
        for (size_t i = 0; i < dim; ++i) col[i] = mat[i * n + j];
        cera_oracle_quantize_q8_0(col.data(), dim, scales + j * (dim / 32), quants + j * dim);
    }
}

int cera_oracle_block_sums(int type, const uint8_t *row, size_t k, const int8_t *aq, int32_t *u,
                           int32_t *a) {
    if (!int8_type(type) || k % blk_elems(type)) return -1;
    for (size_t b = 0; b < k / 32; ++b) {
        int32_t q[32];
        group_quants(type, row, b, q);
        for (int h = 0; h < 2; ++h) {
            int32_t su = 0, sa = 0;
            for (int t = 0; t < 16; ++t) {
                su += q[16 * h + t] * (int32_t)aq[32 * b + 16 * h + t];
                sa += aq[32 * b + 16 * h + t];
            }
            u[2 * b + h] = su;
            a[2 * b + h] = sa;
        }
    }
    return 0;
}

int cera_oracle_gemm_preq(int type, const uint8_t *w, const float *bs, const int8_t *bq, float *out,
                          size_t m, size_t n, size_t k) {
    if (!int8_type(type) || k % blk_elems(type)) return -1;
    const size_t rb = cera_oracle_row_bytes(type, k), nb = k / 32;
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j)
            out[i * n + j] = cell(type, w + i * rb, bs + j * nb, bq + j * k, k, n == 1);
    return 0;
}

static int gemv_impl(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k,
                     int n_threads) {
    const int e = blk_elems(type);
    if (!e || k % e) return -1;
    const size_t rb = cera_oracle_row_bytes(type, k);
    if (type == CERA_T_Q5_K) {
        par_rows(m, n_threads, [&](size_t i) {
            float sum = 0.0f;
            for (size_t bi = 0; bi < k / 256; ++bi) sum += q5k_dot_f32(w + i * rb + bi * 176, x + 256 * bi);
            y[i] = sum;
        });
        return 0;
    }
    if (!int8_type(type)) {
        par_rows(m, n_threads, [&](size_t i) {
            float s = 0.0f;
            for (size_t c = 0; c < k; ++c) {
                float wv;
                const uint8_t *p = w + i * rb + c * blk_bytes(type);
                if (type == CERA_T_F32) std::memcpy(&wv, p, 4);
                else wv = type == CERA_T_F16 ? h2f(rd16(p)) : bf2f(rd16(p));
                s += wv * x[c];
            }
            y[i] = s;
        });
        return 0;
    }
    if (k % 32) return -1;
    std::vector<float> xs(k / 32);
    std::vector<int8_t> xq(k);
    cera_oracle_quantize_q8_0(x, k, xs.data(), xq.data());
    par_rows(m, n_threads,
             [&](size_t i) { y[i] = cell(type, w + i * rb, xs.data(), xq.data(), k, true); });
    return 0;
}

int cera_oracle_gemv(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k) {
    return gemv_impl(type, w, x, y, m, k, 1);
}

void cera_oracle_rmsnorm(float *x, const float *weight, size_t n, float eps) {
    double ss = 0.0;
    for (size_t i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
    const double mean = ss / (double)n;
    const float inv = (float)(1.0 / std::sqrt(mean + (double)eps));
    for (size_t i = 0; i < n; ++i) x[i] = x[i] * inv * weight[i];
}

float cera_oracle_expf(float x) {
    const float R = u2f(0x4B400000u), LOG2E = u2f(0x3FB8AA3Bu), LN2_HI = u2f(0x3F317200u),
                LN2_LO = u2f(0x35BFBE8Eu), C1 = u2f(0x3F7FFFF6u), C2 = u2f(0x3EFFFEDBu),
                C3 = u2f(0x3E2AAF33u), C4 = u2f(0x3D2B9F17u), C5 = u2f(0x3C072010u);
    const float z = R + x * LOG2E;
    const float n = z - R;
    const float b = x - n * LN2_HI - n * LN2_LO;
    const uint32_t e = f2u(z) << 23;
    const float k = u2f(e + 0x3F800000u);
    const float u = b * b;
    const float j = C1 * b + (C2 + C3 * b + (C4 + C5 * b) * u) * u;
    const float abs_n = u2f(f2u(n) & 0x7FFFFFFFu);
    if (abs_n <= 126.0f) return k + j * k;
    if (abs_n > 192.0f) return n > 0.0f ? std::numeric_limits<float>::infinity() : 0.0f;
    const uint32_t d = n <= 0.0f ? 0x82000000u : 0u;
    const float s1 = u2f(d + 0x7F000000u);
    const float s2 = u2f(e - d);
    return (s2 + s2 * j) * s1;
}

void cera_oracle_silu_mul(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; ++i) gate[i] = gate[i] / (1.0f + cera_oracle_expf(-gate[i])) * up[i];
}

void cera_oracle_softmax(float *x, size_t n) {
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t i = 0; i < n; ++i)
        if (!(x[i] != x[i])) mx = x[i] > mx ? x[i] : mx;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        x[i] = cera_oracle_expf(x[i] - mx);
        sum += (double)x[i];
    }
    const float inv = (float)(1.0 / sum);
    for (size_t i = 0; i < n; ++i) x[i] *= inv;
}

static void rope_head(float *h, float pos, size_t hd, float base, const float *ff, int neox) {
    const float ts = std::pow(base, -2.0f / (float)hd);
    float theta = pos;
    const size_t half = hd / 2;
    for (size_t i = 0; i < half; ++i) {
        const float t = neox ? theta : theta / (ff ? ff[i] : 1.0f);
        const float s = std::sin(t), c = std::cos(t);
        float &a = neox ? h[i] : h[2 * i];
        float &b = neox ? h[i + half] : h[2 * i + 1];
        const float x0 = a, x1 = b;
        a = x0 * c - x1 * s;
        b = x0 * s + x1 * c;
        theta *= ts;
    }
}

void cera_oracle_rope(float *q, float *k, size_t pos, size_t nh, size_t nkv, size_t hd, float base,
                      const float *ff, int rope_type) {
    for (size_t h = 0; h < nh; ++h) rope_head(q + h * hd, (float)pos, hd, base, ff, rope_type);
    for (size_t h = 0; h < nkv; ++h) rope_head(k + h * hd, (float)pos, hd, base, ff, rope_type);
}

// Decode attention of one token (cera/src/model/transformer.rs:1166-1305).  The score and value loops
// follow what the reference runs on an x86 host with AVX2+FMA(+F16C) - the host class whose int8 tier the
// GEMV restatement above follows - whenever head_dim is a multiple of 8 and at most 256
// (cera/src/backend/cpu.rs:3264-3290, 3330-3352): scores are two 8-lane FMA accumulators over alternating
// 8-wide slices of the head, added, then hsum256 (cpu.rs:3522-3585, 3489-3497); the value sum is one FMA per
// output element per position, in position order (cpu.rs:3587-3625).  f16 caches widen each element first
// (vcvtph2ps is exact; cpu.rs attn_scores_f16_avx2 / attn_values_f16_avx2).  Other head sizes take the
// reference's scalar loops (cpu.rs:3292-3300, 3354-3362).
void cera_oracle_decode_attention(const float *q, const void *kc, const void *vc, int kv_f16,
                                  size_t nh, size_t nkv, size_t hd, size_t seq, float scale,
                                  float *out, float *scores) {
    const size_t kv_dim = nkv * hd, group = nh / nkv;
    const float *kf = (const float *)kc, *vf = (const float *)vc;
    const uint16_t *kh = (const uint16_t *)kc, *vh = (const uint16_t *)vc;
    const bool vec = hd % 8 == 0 && hd <= 256;
    for (size_t h = 0; h < nh; ++h) {
        const float *qh = q + h * hd;
        const size_t off = (h / group) * hd;
        for (size_t t = 0; t < seq; ++t) {
            const size_t base = t * kv_dim + off;
            auto kat = [&](size_t d) { return kv_f16 ? h2f(kh[base + d]) : kf[base + d]; };
            if (vec) {
                float s0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, s1[8] = {0, 0, 0, 0, 0, 0, 0, 0}, s[8];
                const size_t nv = hd / 8;
                size_t i = 0;
                for (; i + 2 <= nv; i += 2)
                    for (int L = 0; L < 8; ++L) {
                        s0[L] = std::fmaf(qh[8 * i + L], kat(8 * i + L), s0[L]);
                        s1[L] = std::fmaf(qh[8 * (i + 1) + L], kat(8 * (i + 1) + L), s1[L]);
                    }
                if (i < nv)
                    for (int L = 0; L < 8; ++L) s0[L] = std::fmaf(qh[8 * i + L], kat(8 * i + L), s0[L]);
                for (int L = 0; L < 8; ++L) s[L] = s0[L] + s1[L];
                scores[t] = hsum8(s) * scale;
            } else {
                float dot = 0.0f;
                for (size_t d = 0; d < hd; ++d) dot += qh[d] * kat(d);
                scores[t] = dot * scale;
            }
        }
        cera_oracle_softmax(scores, seq);
        float *o = out + h * hd;
        for (size_t d = 0; d < hd; ++d) o[d] = 0.0f;
        for (size_t t = 0; t < seq; ++t) {
            const float s = scores[t];
            const size_t base = t * kv_dim + off;
            for (size_t d = 0; d < hd; ++d) {
                const float v = kv_f16 ? h2f(vh[base + d]) : vf[base + d];
                o[d] = vec ? std::fmaf(s, v, o[d]) : o[d] + s * v;
            }
        }
    }
}

void cera_oracle_flash_attention_gqa(const float *q, const float *kc, const float *vc, size_t nh,
                                     size_t nkv, size_t hd, size_t n, size_t start_pos, float scale,
                                     float *out) {
    const size_t kv_dim = nkv * hd, group = nh / nkv, TILE = 32;
    std::vector<float> ql(hd), acc(hd);
    float ts[32];
    for (size_t h = 0; h < nh; ++h) {
        const size_t off = (h / group) * hd;
        for (size_t j = 0; j < n; ++j) {
            const size_t max_kv = start_pos + j + 1;
            for (size_t d = 0; d < hd; ++d) ql[d] = q[(h * hd + d) * n + j];
            float rmax = -std::numeric_limits<float>::infinity();
            double rsum = 0.0;
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (size_t s0 = 0; s0 < max_kv; s0 += TILE) {
                const size_t len = std::min(TILE, max_kv - s0);
                float tmax = -std::numeric_limits<float>::infinity();
                for (size_t ti = 0; ti < len; ++ti) {
                    float dot = 0.0f;
                    for (size_t d = 0; d < hd; ++d) dot += ql[d] * kc[(s0 + ti) * kv_dim + off + d];
                    ts[ti] = dot * scale;
                    tmax = ts[ti] > tmax ? ts[ti] : tmax;
                }
                const float nmax = rmax > tmax ? rmax : tmax;
                const float resc = rmax > -std::numeric_limits<float>::infinity()
                                       ? cera_oracle_expf(rmax - nmax) : 0.0f;
                double tsum = 0.0;
                for (size_t ti = 0; ti < len; ++ti) {
                    ts[ti] = cera_oracle_expf(ts[ti] - nmax);
                    tsum += (double)ts[ti];
                }
                for (size_t d = 0; d < hd; ++d) acc[d] *= resc;
                for (size_t ti = 0; ti < len; ++ti)
                    for (size_t d = 0; d < hd; ++d) acc[d] += ts[ti] * vc[(s0 + ti) * kv_dim + off + d];
                rsum = rsum * (double)resc + tsum;
                rmax = nmax;
            }
            const float inv = (float)(1.0 / rsum);
            for (size_t d = 0; d < hd; ++d) out[(h * n + j) * hd + d] = acc[d] * inv;
        }
    }
}

uint32_t cera_oracle_argmax(const float *l, size_t n) {
    uint32_t bi = 0;
    float bv = -std::numeric_limits<float>::infinity();
    for (size_t i = 0; i < n; ++i)
        if (l[i] > bv) {
            bv = l[i];
            bi = (uint32_t)i;
        }
    return bi;
}

// IEEE total order key for f32 (Rust f32::total_cmp).
static inline int32_t total_key(float f) {
    int32_t b = (int32_t)f2u(f);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

void cera_oracle_select_experts(const float *probs, const float *bias, size_t ne, size_t n_used,
                                uint32_t *ids, float *weights) {
    std::vector<char> taken(ne, 0);
    const size_t cnt = std::min(n_used, ne);
    for (size_t r = 0; r < cnt; ++r) {
        long best = -1;
        int32_t bk = 0;
        for (size_t e = 0; e < ne; ++e) {
            if (taken[e]) continue;
            const int32_t key = total_key(probs[e] + (bias ? bias[e] : 0.0f));
            if (best < 0 || key > bk) {  // strict: ties keep the lower index
                best = (long)e;
                bk = key;
            }
        }
        taken[best] = 1;
        ids[r] = (uint32_t)best;
        weights[r] = probs[best];
    }
    float denom = 0.0f;
    for (size_t r = 0; r < cnt; ++r) denom += weights[r];
    denom = std::fmax(denom, 1.0f / 16384.0f);
    for (size_t r = 0; r < cnt; ++r) weights[r] /= denom;
}

void cera_oracle_synth_normal(float *out, size_t n, uint64_t seed, uint64_t offset, float sigma) {
    const float scale = sigma * (1.0f / 65536.0f);
    for (size_t i = 0; i < n; ++i) {
        const uint64_t c = (offset + i) * 3ull;
        const uint64_t key = splitmix64(seed);
        int32_t sum = 0;
        for (int r = 0; r < 3; ++r) {
            const uint64_t h = splitmix64(key ^ (c + (uint64_t)r));
            sum += (int32_t)(h & 0xFFFF) + (int32_t)((h >> 16) & 0xFFFF) +
                   (int32_t)((h >> 32) & 0xFFFF) + (int32_t)((h >> 48) & 0xFFFF);
        }
        out[i] = (float)(sum - 393210) * scale;
    }
}

// ---- dense llama model ----------------------------------------------------

struct TensorRef {
    int type = -1;
    size_t rows = 0, cols = 0;
    const uint8_t *bytes = nullptr;
};

// One LoRA pair of a projection: y += B (scale * (A x))  (cera/src/lora.rs:794-821).
struct LoraPair {
    size_t rank = 0, k = 0, d = 0;
    float scale = 0.0f;
    std::vector<float> a, b;  // A [rank x k], B [d x rank], row-major
};

// lora.rs:799-821 apply_decode, operation for operation: each dot product is summed from zero in index order, the
// scale is folded into the rank-sized vector, and the finished B row dot is added to y once.
static void lora_apply(const LoraPair &t, const float *x, float *y) {
    if (t.rank == 0 || t.scale == 0.0f) return;
    std::vector<float> tmp(t.rank);
    for (size_t r = 0; r < t.rank; ++r) {
        float acc = 0.0f;
        for (size_t i = 0; i < t.k; ++i) acc += t.a[r * t.k + i] * x[i];
        tmp[r] = acc * t.scale;
    }
    for (size_t o = 0; o < t.d; ++o) {
        float acc = 0.0f;
        for (size_t r = 0; r < t.rank; ++r) acc += t.b[o * t.rank + r] * tmp[r];
        y[o] += acc;
    }
}

struct cera_oracle_model {
    cera_oracle_config cfg;
    std::vector<LoraPair> lora;  // [layer * 7 + target], targets in the order of cera/src/lora.rs:63-70 (q, k, v, o, gate, up, down)
    TensorRef embd, out_norm, output, rope_freqs;
    std::vector<TensorRef> attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down;
    std::vector<std::vector<uint8_t>> kcache, vcache;  // f32 or f16 bytes, time-major
    size_t seq_len = 0;
    std::vector<float> last_hidden;
};

cera_oracle_model *cera_oracle_model_create(const cera_oracle_config *cfg) {
    auto *m = new cera_oracle_model();
    m->cfg = *cfg;
    const size_t L = cfg->n_layers;
    for (auto *v : {&m->attn_norm, &m->wq, &m->wk, &m->wv, &m->wo, &m->ffn_norm, &m->gate, &m->up,
                    &m->down})
        v->resize(L);
    m->kcache.resize(L);
    m->vcache.resize(L);
    return m;
}

int cera_oracle_model_set_tensor(cera_oracle_model *m, int role, int layer, int type, size_t rows,
                                 size_t cols, const void *bytes) {
    TensorRef t{type, rows, cols, (const uint8_t *)bytes};
    auto at = [&](std::vector<TensorRef> &v) -> int {
        if (layer < 0 || (size_t)layer >= v.size()) return -1;
        v[layer] = t;
        return 0;
    };
    switch (role) {
        case CERA_ROLE_TOKEN_EMBD: m->embd = t; return 0;
        case CERA_ROLE_OUTPUT_NORM: m->out_norm = t; return 0;
        case CERA_ROLE_OUTPUT: m->output = t; return 0;
        case CERA_ROLE_ROPE_FREQS: m->rope_freqs = t; return 0;
        case CERA_ROLE_ATTN_NORM: return at(m->attn_norm);
        case CERA_ROLE_ATTN_Q: return at(m->wq);
        case CERA_ROLE_ATTN_K: return at(m->wk);
        case CERA_ROLE_ATTN_V: return at(m->wv);
        case CERA_ROLE_ATTN_OUTPUT: return at(m->wo);
        case CERA_ROLE_FFN_NORM: return at(m->ffn_norm);
        case CERA_ROLE_FFN_GATE: return at(m->gate);
        case CERA_ROLE_FFN_UP: return at(m->up);
        case CERA_ROLE_FFN_DOWN: return at(m->down);
        default: return -1;
    }
}

int cera_cpu_gemv(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k, int nt);
int cera_cpu_gemv_vnni(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k, int nt);
int cera_cpu_has_avx2_vnni(void);

// Which build of the x86 int8 kernels the model forward uses: 0 = the scalar restatement, 1 = AVX2 (default when the host
// has it), 2 = AVX-512 VNNI.  All three give identical bits (tests); the choice only changes the wall time.
static int g_cpu_tier = 1;
void cera_oracle_set_cpu_tier(int tier) { g_cpu_tier = tier; }

int cera_oracle_model_forward(cera_oracle_model *M, uint32_t token, size_t pos, float *logits) {
    const auto &c = M->cfg;
    if (token >= c.vocab_size || pos != M->seq_len || pos >= c.max_seq_len) return -1;
    const size_t hs = c.hidden_size, hd = c.head_dim, qd = (size_t)c.n_heads * hd,
                 kvd = (size_t)c.n_kv_heads * hd, ff = c.intermediate_size;
    const int nt = c.n_threads > 0 ? c.n_threads : 1;
    auto gemv = [&](const TensorRef &t, const float *x, float *y) {
        // The AVX2 build is bit-identical to the scalar restatement (tested), so
        // use it when present; it only changes the wall time.
        if (int8_type(t.type) && t.type != CERA_T_Q5_K) {
            if (g_cpu_tier == 2 && cera_cpu_has_avx2_vnni()) return cera_cpu_gemv_vnni(t.type, t.bytes, x, y, t.rows, t.cols, nt);
            if (g_cpu_tier >= 1 && cera_cpu_has_avx2()) return cera_cpu_gemv(t.type, t.bytes, x, y, t.rows, t.cols, nt);
        }
        return gemv_impl(t.type, t.bytes, x, y, t.rows, t.cols, nt);
    };
    std::vector<float> hidden(hs), normed(hs), q(qd), k(kvd), v(kvd), attn(qd), out(hs), g(ff), u(ff),
        scores(pos + 1);
    // embedding row (transformer.rs:949-1018)
    cera_oracle_dequantize_row(M->embd.type,
                               M->embd.bytes + (size_t)token * cera_oracle_row_bytes(M->embd.type, hs),
                               hs, hidden.data());
    // Granite scalar multipliers, applied where cera/src/model/llama.rs applies them (1544-1546, 515-521, 543-549, 591-594)
    if (c.embedding_scale != 0.0f && c.embedding_scale != 1.0f)
        for (size_t i = 0; i < hs; ++i) hidden[i] *= c.embedding_scale;
    const float res_scale = c.residual_scale != 0.0f ? c.residual_scale : 1.0f;
    const float att_scale = c.attention_scale != 0.0f ? c.attention_scale : 1.0f / std::sqrt((float)hd);
    const float *ffreq = M->rope_freqs.bytes ? (const float *)M->rope_freqs.bytes : nullptr;
    const size_t esz = c.kv_f16 ? 2 : 4;
    for (size_t l = 0; l < c.n_layers; ++l) {
        normed = hidden;
        cera_oracle_rmsnorm(normed.data(), (const float *)M->attn_norm[l].bytes, hs, c.rms_norm_eps);
        gemv(M->wq[l], normed.data(), q.data());
        gemv(M->wk[l], normed.data(), k.data());
        gemv(M->wv[l], normed.data(), v.data());
        if (!M->lora.empty()) {  // before RoPE, input = the normed hidden (cera/src/model/transformer.rs:1383-1387)
            lora_apply(M->lora[l * 7 + 0], normed.data(), q.data());
            lora_apply(M->lora[l * 7 + 1], normed.data(), k.data());
            lora_apply(M->lora[l * 7 + 2], normed.data(), v.data());
        }
        cera_oracle_rope(q.data(), k.data(), pos, c.n_heads, c.n_kv_heads, hd, c.rope_theta, ffreq,
                         c.rope_type);
        auto &kc = M->kcache[l];
        auto &vc = M->vcache[l];
        kc.resize((pos + 1) * kvd * esz);
        vc.resize((pos + 1) * kvd * esz);
        if (c.kv_f16) {
            uint16_t *kp = (uint16_t *)kc.data() + pos * kvd, *vp = (uint16_t *)vc.data() + pos * kvd;
            for (size_t i = 0; i < kvd; ++i) {
                kp[i] = f2h(k[i]);
                vp[i] = f2h(v[i]);
            }
        } else {
            std::memcpy(kc.data() + pos * kvd * 4, k.data(), kvd * 4);
            std::memcpy(vc.data() + pos * kvd * 4, v.data(), kvd * 4);
        }
        cera_oracle_decode_attention(q.data(), kc.data(), vc.data(), c.kv_f16, c.n_heads, c.n_kv_heads,
                                     hd, pos + 1, att_scale, attn.data(),
                                     scores.data());
        gemv(M->wo[l], attn.data(), out.data());
        if (!M->lora.empty()) lora_apply(M->lora[l * 7 + 3], attn.data(), out.data());  // transformer.rs:1519-1528
        if (res_scale != 1.0f)
            for (size_t i = 0; i < hs; ++i) out[i] *= res_scale;
        for (size_t i = 0; i < hs; ++i) hidden[i] += out[i];
        normed = hidden;
        cera_oracle_rmsnorm(normed.data(), (const float *)M->ffn_norm[l].bytes, hs, c.rms_norm_eps);
        gemv(M->gate[l], normed.data(), g.data());
        gemv(M->up[l], normed.data(), u.data());
        if (!M->lora.empty()) {  // before the SwiGLU product (transformer.rs:1588-1605)
            lora_apply(M->lora[l * 7 + 4], normed.data(), g.data());
            lora_apply(M->lora[l * 7 + 5], normed.data(), u.data());
        }
        cera_oracle_silu_mul(g.data(), u.data(), ff);
        gemv(M->down[l], g.data(), out.data());
        if (!M->lora.empty()) lora_apply(M->lora[l * 7 + 6], g.data(), out.data());  // transformer.rs:1642-1651
        if (res_scale != 1.0f)
            for (size_t i = 0; i < hs; ++i) out[i] *= res_scale;
        for (size_t i = 0; i < hs; ++i) hidden[i] += out[i];
    }
    cera_oracle_rmsnorm(hidden.data(), (const float *)M->out_norm.bytes, hs, c.rms_norm_eps);
    M->last_hidden = hidden;
    M->seq_len += 1;
    if (logits) {
        const TensorRef &o = M->output.bytes ? M->output : M->embd;
        gemv(o, hidden.data(), logits);
        if (c.logit_scale != 0.0f && c.logit_scale != 1.0f) {
            const float inv = 1.0f / c.logit_scale;
            const size_t vocab = c.vocab_size;
            for (size_t i = 0; i < vocab; ++i) logits[i] *= inv;
        }
    }
    return 0;
}

void cera_oracle_lora_apply(size_t rank, size_t k, size_t d, float scale, const float *a, const float *b, const float *x,
                            float *y) {
    LoraPair t;
    t.rank = rank;
    t.k = k;
    t.d = d;
    t.scale = scale;
    t.a.assign(a, a + rank * k);
    t.b.assign(b, b + d * rank);
    lora_apply(t, x, y);
}

int cera_oracle_model_set_lora(cera_oracle_model *M, int target, int layer, size_t rank, size_t k, size_t d, float scale,
                               const float *a, const float *b) {
    if (target < 0 || target > 6 || layer < 0 || (uint32_t)layer >= M->cfg.n_layers || !a || !b || rank == 0) return -1;
    if (M->lora.empty()) M->lora.resize((size_t)M->cfg.n_layers * 7);
    LoraPair &t = M->lora[(size_t)layer * 7 + target];
    t.rank = rank;
    t.k = k;
    t.d = d;
    t.scale = scale;
    t.a.assign(a, a + rank * k);
    t.b.assign(b, b + d * rank);
    return 0;
}

void cera_oracle_model_truncate_kv(cera_oracle_model *m, size_t len) {
    if (len < m->seq_len) m->seq_len = len;
}
// InferenceState::shift_kv_with_rope (cera/src/kv_cache.rs:1091-1320): drain rows [n_keep, n_keep+shift) of every
// layer's K and V, then rotate each K head now at [n_keep, new_len) by R(-shift) with the forward pass's RoPE
// helper (theta_0 = -shift; f16 caches are widened, rotated and narrowed again).
int cera_oracle_model_shift_kv(cera_oracle_model *M, size_t n_keep, size_t shift) {
    const auto &c = M->cfg;
    if (shift == 0 || n_keep + shift > M->seq_len) return -1;
    const size_t kvd = (size_t)c.n_kv_heads * c.head_dim, esz = c.kv_f16 ? 2 : 4, row = kvd * esz;
    const size_t new_len = M->seq_len - shift;
    const float *ffreq = M->rope_freqs.bytes ? (const float *)M->rope_freqs.bytes : nullptr;
    std::vector<float> buf(c.head_dim);
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        auto &kc = M->kcache[l];
        auto &vc = M->vcache[l];
        if (kc.size() < M->seq_len * row) return -1;
        kc.erase(kc.begin() + n_keep * row, kc.begin() + (n_keep + shift) * row);
        vc.erase(vc.begin() + n_keep * row, vc.begin() + (n_keep + shift) * row);
        for (size_t t = n_keep; t < new_len; ++t)
            for (size_t h = 0; h < c.n_kv_heads; ++h) {
                if (c.kv_f16) {
                    uint16_t *p = (uint16_t *)kc.data() + t * kvd + h * c.head_dim;
                    for (size_t d = 0; d < c.head_dim; ++d) buf[d] = h2f(p[d]);
                    rope_head(buf.data(), -(float)shift, c.head_dim, c.rope_theta, ffreq, c.rope_type);
                    for (size_t d = 0; d < c.head_dim; ++d) p[d] = f2h(buf[d]);
                } else {
                    rope_head((float *)kc.data() + t * kvd + h * c.head_dim, -(float)shift, c.head_dim, c.rope_theta, ffreq, c.rope_type);
                }
            }
    }
    M->seq_len = new_len;
    return 0;
}
size_t cera_oracle_model_seq_len(const cera_oracle_model *m) { return m->seq_len; }
void cera_oracle_model_set_threads(cera_oracle_model *m, int n) { m->cfg.n_threads = n; }
int cera_oracle_model_last_hidden(const cera_oracle_model *m, float *out) {
    if (m->last_hidden.empty()) return -1;
    std::memcpy(out, m->last_hidden.data(), m->last_hidden.size() * 4);
    return 0;
}
size_t cera_oracle_model_kv(const cera_oracle_model *m, size_t layer, int which, void *out, size_t cap) {
    if (layer >= m->kcache.size()) return 0;
    const auto &c = which ? m->vcache[layer] : m->kcache[layer];
    const size_t kvd = (size_t)m->cfg.n_kv_heads * m->cfg.head_dim;
    const size_t n = m->seq_len * kvd * (m->cfg.kv_f16 ? 2 : 4);
    if (out) std::memcpy(out, c.data(), n < cap ? n : cap);
    return n;
}
void cera_oracle_model_free(cera_oracle_model *m) { delete m; }

}  // extern "C"
