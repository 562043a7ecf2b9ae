// Decode attention in the reference's own arithmetic order, so that its output is bit-identical to
// what cera computes on an x86 host with AVX2+FMA (cera/src/model/transformer.rs:1166-1305 calling
// cera/src/backend/cpu.rs:3522-3625 and softmax_inplace, cpu.rs:2617-2633), for head sizes that are a
// multiple of 32 up to 256 and up to 8 query heads per KV head.
//
// The reference computes, per query head: every score as two 8-lane FMA accumulators over alternating
// 8-wide slices of the head (16 chains of head_dim/16 FMAs), added lane-wise, reduced in the hsum256
// order and multiplied by the scale; then a plain softmax over ALL positions (maximum, ggml_expf,
// f64 sum, one multiplication by (float)(1/sum)); then out[d] = fma(p[t], V[t][d], out[d]) for t in
// position order.  The last step is a serial chain per output element that an online-softmax
// (flash-decode) kernel cannot reproduce, so the work is split differently here:
//
//   scores kernel : one thread per (position, query head); the G heads of a KV head sit in adjacent
//                   threads and share the K row.  Scores go to a workspace [n_heads][ld].
//   values kernel : one CTA per (KV head, 32 output dims).  All threads first turn the scores of the
//                   group's heads into probabilities (block maximum, ggml_expf, f64 sum by a fixed
//                   tree, scaling); then 8 threads per head - four output dims each - walk the
//                   positions in order with one FMA per dim per position, and finally emit the f32
//                   outputs and their Q8_0 form (a 32-dim slice of a head is one Q8_0 block).
//
// The f64 sum of the exponentials is a tree, the reference's a left-to-right loop: the two can differ
// in the last bits of the f64 sum, which survive the narrowing to f32 only in about one softmax in
// 10^7 (and not at all while every partial sum is exactly representable, which holds whenever the
// probabilities span fewer than ~29 binary orders of magnitude).
#include <cstdlib>
#include <cstring>

#include "act.cuh"
#include "ops.h"

namespace cera {

namespace {

constexpr int AX_TILE = 32;        // positions per CTA pass of the scores kernel
constexpr int AX_VTHREADS = 256;   // threads of the values kernel
constexpr uint32_t AX_SMEM_POS = 4096;  // probabilities of up to this many positions stay in shared memory

__device__ __forceinline__ void load8(const void *base, size_t elem, bool f16, float (&v)[8]) {
    if (f16) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(base) + elem));
        const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(base) + elem));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(base) + elem + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// blockDim.x = AX_TILE * G.  Dynamic shared memory: G * (hd + 4) floats.
__global__ void attn_scores_exact_kernel(const float *__restrict__ q, const void *__restrict__ kc, int kv_f16, uint32_t seq_len,
                                         const uint32_t *__restrict__ seq_dev, uint32_t n_kv, uint32_t G, uint32_t hd, float scale,
                                         float *__restrict__ ws, uint32_t ld) {
    extern __shared__ __align__(16) float ax_q[];
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = seq_dev ? *seq_dev : seq_len;
    const uint32_t kvh = blockIdx.y, qstride = hd + 4;
    for (uint32_t i = threadIdx.x; i < G * hd; i += blockDim.x) ax_q[(i / hd) * qstride + i % hd] = q[(size_t)kvh * G * hd + i];
    __syncthreads();
    const uint32_t h = threadIdx.x % G, pt = threadIdx.x / G;
    const float *qh = ax_q + h * qstride;
    const size_t kv_dim = (size_t)n_kv * hd;
    const uint32_t nv = hd / 8;
    for (uint32_t tile = blockIdx.x; tile * AX_TILE < seq; tile += gridDim.x) {
        const uint32_t t = tile * AX_TILE + pt;
        if (t >= seq) continue;
        const size_t row = (size_t)t * kv_dim + (size_t)kvh * hd;
        float s0[8], s1[8];
#pragma unroll
        for (int L = 0; L < 8; ++L) s0[L] = s1[L] = 0.0f;
        uint32_t i = 0;
        for (; i + 2 <= nv; i += 2) {
            float k0[8], k1[8];
            load8(kc, row + 8 * i, kv_f16, k0);
            load8(kc, row + 8 * i + 8, kv_f16, k1);
            const float4 qa = *reinterpret_cast<const float4 *>(qh + 8 * i), qb = *reinterpret_cast<const float4 *>(qh + 8 * i + 4);
            const float4 qc = *reinterpret_cast<const float4 *>(qh + 8 * i + 8), qd = *reinterpret_cast<const float4 *>(qh + 8 * i + 12);
            const float q0[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const float q1[8] = {qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
            for (int L = 0; L < 8; ++L) {
                s0[L] = fmaf(q0[L], k0[L], s0[L]);
                s1[L] = fmaf(q1[L], k1[L], s1[L]);
            }
        }
        if (i < nv) {
            float k0[8];
            load8(kc, row + 8 * i, kv_f16, k0);
#pragma unroll
            for (int L = 0; L < 8; ++L) s0[L] = fmaf(qh[8 * i + L], k0[L], s0[L]);
        }
        float s[8];
#pragma unroll
        for (int L = 0; L < 8; ++L) s[L] = __fadd_rn(s0[L], s1[L]);
        // hsum256: lanes i and i+4, then (0,2) and (1,3), then the two (cera/src/backend/cpu.rs:3489-3497)
        const float a0 = __fadd_rn(s[0], s[4]), a1 = __fadd_rn(s[1], s[5]), a2 = __fadd_rn(s[2], s[6]), a3 = __fadd_rn(s[3], s[7]);
        const float dot = __fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a1, a3));
        ws[(size_t)(kvh * G + h) * ld + t] = __fmul_rn(dot, scale);
    }
}

// grid (hd / 32, n_kv), AX_VTHREADS threads.  ws: scores [n_heads][ld]; pw: probabilities [n_heads][ld] in global
// memory, used when the positions do not fit shared memory (every CTA of a KV head writes the same values there).
// Dynamic shared memory: min(seq bucket, AX_SMEM_POS) * G floats.
__global__ void __launch_bounds__(AX_VTHREADS)
attn_values_exact_kernel(const float *__restrict__ ws, float *__restrict__ pw, uint32_t ld, const void *__restrict__ vc, int kv_f16,
                         uint32_t seq_len, const uint32_t *__restrict__ seq_dev, uint32_t n_kv, uint32_t G, uint32_t hd,
                         uint32_t smem_pos, float *__restrict__ out, float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    extern __shared__ __align__(16) float ax_p[];  // [position][G]
    __shared__ double red_d[AX_VTHREADS / 32];
    __shared__ float red_f[AX_VTHREADS / 32];
    __shared__ float bc_f;
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = seq_dev ? *seq_dev : seq_len;
    const uint32_t kvh = blockIdx.y, d0 = blockIdx.x * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool in_smem = seq <= smem_pos;
    for (uint32_t h = 0; h < G; ++h) {
        const float *s = ws + (size_t)(kvh * G + h) * ld;
        float *pg = pw + (size_t)(kvh * G + h) * ld;
        // maximum (f32::max fold: NaN scores are ignored)
        float mx = -INFINITY;
        for (uint32_t t = tid; t < seq; t += AX_VTHREADS) mx = fmaxf(mx, s[t]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red_f[warp] = mx;
        __syncthreads();
        if (tid == 0) {
            float m = red_f[0];
            for (int w = 1; w < AX_VTHREADS / 32; ++w) m = fmaxf(m, red_f[w]);
            bc_f = m;
        }
        __syncthreads();
        mx = bc_f;
        // exponentials and their f64 sum (fixed tree: thread-strided partials, xor shuffles, warps in index order)
        double sum = 0.0;
        for (uint32_t t = tid; t < seq; t += AX_VTHREADS) {
            const float e = ggml_expf(__fsub_rn(s[t], mx));
            if (in_smem) ax_p[(size_t)t * G + h] = e;
            sum += (double)e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) red_d[warp] = sum;
        __syncthreads();
        if (tid == 0) {
            double tot = red_d[0];
            for (int w = 1; w < AX_VTHREADS / 32; ++w) tot += red_d[w];
            bc_f = (float)(1.0 / tot);
        }
        __syncthreads();
        const float inv = bc_f;
        for (uint32_t t = tid; t < seq; t += AX_VTHREADS) {
            if (in_smem) ax_p[(size_t)t * G + h] = __fmul_rn(ax_p[(size_t)t * G + h], inv);
            else pg[t] = __fmul_rn(ggml_expf(__fsub_rn(s[t], mx)), inv);  // recomputed: the CTAs of a KV head all store the same final value
        }
        __syncthreads();
    }
    // every CTA of the KV head wrote the same probabilities to pw; this CTA's own writes are visible to it after the barrier
    if (tid >= (int)(G * 8)) return;
    const uint32_t h = tid >> 3, dq = tid & 7;
    const size_t kv_dim = (size_t)n_kv * hd;
    const size_t col = (size_t)kvh * hd + d0 + 4 * dq;
    const float *pg = pw + (size_t)(kvh * G + h) * ld;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    auto load_v = [&](uint32_t t, float (&v)[4]) {
        if (kv_f16) {
            const uint2 r = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(vc) + (size_t)t * kv_dim + col));
            const __half2 *hh = reinterpret_cast<const __half2 *>(&r);
            const float2 a = __half22float2(hh[0]), b = __half22float2(hh[1]);
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
            const float4 r = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(vc) + (size_t)t * kv_dim + col));
            v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
        }
    };
    uint32_t t0 = 0;
    for (; t0 + 8 <= seq; t0 += 8) {
        float v[8][4], p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            load_v(t0 + i, v[i]);
            p[i] = in_smem ? ax_p[(size_t)(t0 + i) * G + h] : pg[t0 + i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(p[i], v[i][j], acc[j]);
    }
    for (; t0 < seq; ++t0) {
        float v[4];
        load_v(t0, v);
        const float p = in_smem ? ax_p[(size_t)t0 * G + h] : pg[t0];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = fmaf(p, v[j], acc[j]);
    }
    const size_t o = (size_t)(kvh * G + h) * hd + d0 + 4 * dq;
    *reinterpret_cast<float4 *>(out + o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (quants) {
        // Q8_0 of the 32-dim block the eight threads of this head hold (cera/src/backend/cpu.rs:942-958)
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = fabsf(acc[j]);
            amax = fmaxf(amax, a == a ? a : 0.0f);
        }
        const unsigned grp = 0xFFu << (lane & 24);
#pragma unroll
        for (int s = 4; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(grp, amax, s));
        const float d = __fdiv_rn(amax, 127.0f);
        const float r = __fdiv_rn(1.0f, d);
        const float id = (d != 0.0f && isfinite(r)) ? r : 0.0f;
        int qv[4], s4 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float pq = rintf(__fmul_rn(acc[j], id));
            qv[j] = pq != pq ? 0 : (int)fminf(fmaxf(pq, -128.0f), 127.0f);
            s4 += qv[j];
        }
        s4 += __shfl_xor_sync(grp, s4, 1);
        s4 += __shfl_xor_sync(grp, s4, 2);
        const uint32_t packed = (uint32_t)(uint8_t)qv[0] | ((uint32_t)(uint8_t)qv[1] << 8) | ((uint32_t)(uint8_t)qv[2] << 16) |
                                ((uint32_t)(uint8_t)qv[3] << 24);
        const float sc = __half2float(__float2half_rn(d));
        uint32_t *qw = reinterpret_cast<uint32_t *>(quants + o);
        *qw = packed;
        if (dq == 0) scales[o / 32] = sc;
        if ((dq & 3) == 0) sums[o / 16] = (int16_t)s4;
        if (tp.push) {
            tp_push(tp.ctx, qw, packed);
            if (dq == 0) tp_push(tp.ctx, scales + o / 32, sc);
            if ((dq & 3) == 0) tp_push(tp.ctx, sums + o / 16, (int16_t)s4);
        }
    }
}

// CERA_CUDA_ATTN=flash (or any of the split-kernel selectors) keeps decode attention on the online-softmax kernels.
bool exact_off() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_ATTN");
        return e && e[0] != 0;
    }();
    return v;
}

}  // namespace

bool attn_exact_supports(size_t n_heads, size_t n_kv_heads, size_t head_dim) {
    if (exact_off() || n_kv_heads == 0 || n_heads % n_kv_heads) return false;
    const size_t G = n_heads / n_kv_heads;
    return G >= 1 && G <= 8 && head_dim % 32 == 0 && head_dim >= 32 && head_dim <= 256;
}

// Plan word of the reference-order kernels: ATT_EXACT_FLAG | b, b = 1..4: probabilities of up to b * 1024 positions
// stay in shared memory; b = 5: they go through global memory.
constexpr uint32_t ATT_EXACT_FLAG = 0x200;

uint32_t attn_exact_plan(size_t seq_len_hint) {
    const size_t b = (seq_len_hint + 1023) / 1024;
    return ATT_EXACT_FLAG | (uint32_t)(b < 1 ? 1 : b > 4 ? 5 : b);
}

size_t attn_exact_workspace_bytes(size_t n_heads, size_t seq_len) {
    return 2 * n_heads * ((seq_len + 63) / 64 * 64) * sizeof(float);
}

// The workspace's capacity fixes the row stride of the score matrix, so launches captured once (length read from
// seq_len_dev) serve every length the workspace can hold.
int32_t launch_decode_attention_exact(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads, size_t n_kv_heads,
                                      size_t head_dim, size_t seq_len, const uint32_t *seq_len_dev, uint32_t plan, float scale,
                                      float *out, void *workspace, size_t workspace_bytes, float *scales, int8_t *quants,
                                      int16_t *sums, cudaStream_t st, const TpHook *tp) {
    if (!q || !kc || !vc || !out || !workspace) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: null argument");
    const size_t cap = workspace_bytes / (2 * n_heads * sizeof(float)) / 64 * 64;  // positions the workspace holds
    if (cap == 0 || seq_len > cap)
        return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: workspace of %zu bytes holds %zu positions, %zu needed", workspace_bytes, cap, seq_len);
    if (seq_len == 0 && !seq_len_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: empty KV cache");
    const uint32_t G = (uint32_t)(n_heads / n_kv_heads), hd = (uint32_t)head_dim, nkv = (uint32_t)n_kv_heads;
    const uint32_t ld = (uint32_t)cap;
    const uint32_t b = plan & 0xFF;
    size_t reach = b >= 5 ? cap : (size_t)b * 1024;  // longest length this launch may meet
    if (reach > cap) reach = cap;
    if (seq_len > reach) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: plan 0x%x does not cover %zu positions", plan, seq_len);
    float *ws = (float *)workspace, *pw = ws + n_heads * (size_t)ld;
    // scores: a fixed number of CTAs per KV head walks the position tiles, so one captured launch serves every length
    const uint32_t tiles = (uint32_t)((reach + AX_TILE - 1) / AX_TILE);
    uint32_t per_head = (uint32_t)(2 * sm_count() / (int)nkv);
    if (per_head < 1) per_head = 1;
    if (per_head > tiles) per_head = tiles;
    count_launch();
    CERA_CUDA_TRY(launch_k(attn_scores_exact_kernel, dim3(per_head, nkv), dim3(AX_TILE * G), (size_t)G * (hd + 4) * sizeof(float), st, q,
                           kc, kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, hd, scale, ws, ld));
    const uint32_t smem_pos = b >= 5 ? 0u : (uint32_t)reach;
    const size_t smem = (size_t)smem_pos * G * sizeof(float);
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            CERA_CUDA_TRY(cudaFuncSetAttribute(attn_values_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)(AX_SMEM_POS * 8 * sizeof(float))));
            raised = true;
        }
    }
    count_launch();
    return check_cuda(launch_k(attn_values_exact_kernel, dim3(hd / 32, nkv), dim3(AX_VTHREADS), smem, st, (const float *)ws, pw, ld, vc,
                               kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, hd, smem_pos, out, scales, quants, sums,
                               tp ? *tp : TpHook{}),
                      "attention (values) launch");
}

}  // namespace cera
