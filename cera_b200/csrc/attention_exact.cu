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
//   scores kernel : one half-warp per (position, query head): its sixteen lanes are the sixteen chains, and
//                   four shuffle steps add them in the reference's order.  Scores go to a workspace
//                   [n_heads][ld].
//   values kernel : one CTA per (KV head, 32 output dims).  Its warps first turn the scores of the
//                   group's heads into probabilities (maximum, ggml_expf, f64 sum by a fixed tree,
//                   scaling; the heads side by side), while all threads stage the V slice through
//                   shared memory with asynchronous copies, in tiles of 256 positions, two tiles
//                   ahead (a context of up to 768 positions is requested whole before the softmax
//                   starts); then one warp per head - a lane per output dim - walks the positions
//                   in order with one FMA per position, and finally emits the f32 outputs and their
//                   Q8_0 form (a 32-dim slice of a head is one Q8_0 block: one warp).
//
// The f64 sum of the exponentials is a tree, the reference's a left-to-right loop: the two can differ
// in the last bits of the f64 sum, which survive the narrowing to f32 only in about one softmax in
// 10^7 (and not at all while every partial sum is exactly representable, which holds whenever the
// probabilities span fewer than ~29 binary orders of magnitude).
#include <cooperative_groups.h>

#include <cstdlib>
#include <cstring>

#include "act.cuh"
#include "ops.h"

namespace cg = cooperative_groups;

namespace cera {

namespace {

constexpr int AX_VTHREADS = 512;   // threads of the values and fused kernels

// One HALF-WARP per (position, query head): its sixteen lanes are the reference's sixteen FMA chains (accumulator a,
// lane L) - lane c = 8a + L multiplies elements 16j + c of the head for j = 0, 1, ... - and four xor-shuffle steps add
// them in the reference's order (the two accumulators, then hsum256: lanes L and L+4, then (0,2) and (1,3), then the
// two).  The two half-warps of a warp take two heads of the same position, so they read the same K row; the heads of
// a group iterate over the warp pairs.  blockDim.x = 256 (eight warps = eight positions per pass); dynamic shared
// memory: G * hd floats of q.
constexpr int AX_SWARPS = 8;
template <int HD>  // head size known at compile time (0: read it from the argument)
__global__ void __launch_bounds__(AX_SWARPS * 32)
attn_scores_exact_kernel(const float *__restrict__ q, const void *__restrict__ kc, int kv_f16, uint32_t seq_len,
                         const uint32_t *__restrict__ seq_dev, uint32_t n_kv, uint32_t G, uint32_t hd_arg, float scale,
                         float *__restrict__ ws, uint32_t ld) {
    extern __shared__ __align__(16) float ax_q[];
    const uint32_t hd = HD ? (uint32_t)HD : hd_arg;
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = seq_dev ? *seq_dev : seq_len;
    const uint32_t kvh = blockIdx.y;
    for (uint32_t i = threadIdx.x; i < G * hd; i += blockDim.x) ax_q[i] = q[(size_t)kvh * G * hd + i];
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c = lane & 15, hsel = lane >> 4;
    const size_t kv_dim = (size_t)n_kv * hd;
    const uint32_t nv = hd / 8, a = c >> 3, steps = (nv + 1) / 2;
    for (uint32_t t = blockIdx.x * AX_SWARPS + warp; t < seq; t += gridDim.x * AX_SWARPS) {
        const size_t row = (size_t)t * kv_dim + (size_t)kvh * hd;
        // this lane's elements of the K row: 16j + c while chunk 2j + a exists (at most 16 of them: hd <= 256)
        float kv[16];
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j) {
            kv[j] = 0.0f;
            if (j < steps && 2 * j + a < nv) {
                const size_t e = row + 16 * j + c;
                kv[j] = kv_f16 ? __half2float(__ldg(reinterpret_cast<const __half *>(kc) + e)) : __ldg(reinterpret_cast<const float *>(kc) + e);
            }
        }
        for (uint32_t h0 = 0; h0 < G; h0 += 2) {
            const uint32_t h = h0 + hsel;
            const bool live = h < G;
            const float *qh = ax_q + (live ? h : 0) * hd;
            float acc = 0.0f;
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j)
                if (j < steps && 2 * j + a < nv) acc = fmaf(qh[16 * j + c], kv[j], acc);
            // accumulators 0 and 1 of the same lane L, then hsum256
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
            if (live && c == 0) ws[(size_t)(kvh * G + h) * ld + t] = __fmul_rn(acc, scale);
        }
    }
}

__device__ __forceinline__ void ax_cp16(void *smem, const void *gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void ax_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ax_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int AX_VT = 256;     // positions per staged V tile
constexpr int AX_VSTAGES = 3;  // tiles in the ring (two in flight while one is walked)
constexpr int AX_VTHREADS_C = AX_VTHREADS;

// AX_VT positions (or fewer) of one lane's chain: out = fma(p[t], V[t][d], out) in position order.  `base`: the tile,
// one row of 32 dims per position; pp: the head's probabilities from this tile's first position on, 16-byte aligned.
template <bool F16>
__device__ __forceinline__ float ax_chain_tile(const char *base, const float *__restrict__ pp, uint32_t cnt, uint32_t d, float inv, float acc) {
    auto v_at = [&](uint32_t i) -> float {
        if (F16) return __half2float(*reinterpret_cast<const __half *>(base + (size_t)i * 64 + d * 2));
        return *reinterpret_cast<const float *>(base + (size_t)i * 128 + d * 4);
    };
    uint32_t i = 0;
    // eight positions per step (two 128-bit loads of probabilities, eight values), fetched one step ahead of their FMAs:
    // the chain is a dependent FMA per position, the loads must never be what it waits for
    if (cnt >= 8) {
        float4 pa = *reinterpret_cast<const float4 *>(pp), pb = *reinterpret_cast<const float4 *>(pp + 4);
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v_at(j);
        for (; i + 16 <= cnt; i += 8) {
            const float4 na = *reinterpret_cast<const float4 *>(pp + i + 8), nb = *reinterpret_cast<const float4 *>(pp + i + 12);
            float nv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) nv[j] = v_at(i + 8 + j);
            acc = fmaf(__fmul_rn(pa.x, inv), v[0], acc);
            acc = fmaf(__fmul_rn(pa.y, inv), v[1], acc);
            acc = fmaf(__fmul_rn(pa.z, inv), v[2], acc);
            acc = fmaf(__fmul_rn(pa.w, inv), v[3], acc);
            acc = fmaf(__fmul_rn(pb.x, inv), v[4], acc);
            acc = fmaf(__fmul_rn(pb.y, inv), v[5], acc);
            acc = fmaf(__fmul_rn(pb.z, inv), v[6], acc);
            acc = fmaf(__fmul_rn(pb.w, inv), v[7], acc);
            pa = na;
            pb = nb;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = nv[j];
        }
        acc = fmaf(__fmul_rn(pa.x, inv), v[0], acc);
        acc = fmaf(__fmul_rn(pa.y, inv), v[1], acc);
        acc = fmaf(__fmul_rn(pa.z, inv), v[2], acc);
        acc = fmaf(__fmul_rn(pa.w, inv), v[3], acc);
        acc = fmaf(__fmul_rn(pb.x, inv), v[4], acc);
        acc = fmaf(__fmul_rn(pb.y, inv), v[5], acc);
        acc = fmaf(__fmul_rn(pb.z, inv), v[6], acc);
        acc = fmaf(__fmul_rn(pb.w, inv), v[7], acc);
        i += 8;
    }
    for (; i < cnt; ++i) acc = fmaf(__fmul_rn(pp[i], inv), v_at(i), acc);
    return acc;
}

// Requests V tile `tile` (AX_VT positions x 32 dims of one KV head) into its ring slot; every thread commits one group
// per call, empty or not, so the wait counts stay uniform.
__device__ __forceinline__ void ax_stage_tile(uint32_t tile, uint32_t n_tiles, uint32_t seq, uint32_t per_pos, float *vt, const void *vc,
                                              size_t kv_dim, size_t col0, int kv_f16, int tid) {
    if (tile < n_tiles) {
        char *dst = reinterpret_cast<char *>(vt + (size_t)(tile % AX_VSTAGES) * AX_VT * 32);
        const uint32_t t0 = tile * AX_VT, cnt = min((uint32_t)AX_VT, seq - t0) * per_pos;
        const uint32_t sh = kv_f16 ? 2 : 3;  // per_pos = 4 or 8 pieces of 16 bytes
        const char *src0 = reinterpret_cast<const char *>(vc) + ((size_t)t0 * kv_dim + col0) * (kv_f16 ? 2 : 4);
        const size_t row_bytes = kv_dim * (kv_f16 ? 2 : 4);
        for (uint32_t i = tid; i < cnt; i += AX_VTHREADS_C) {
            const uint32_t pl = i >> sh, pc = i & (per_pos - 1);
            ax_cp16(dst + (size_t)i * 16, src0 + (size_t)pl * row_bytes + pc * 16);
        }
    }
    ax_commit();
}

// grid (hd / 32, n_kv), AX_VTHREADS threads.  ws: scores [n_heads][ld]; pw: probabilities [n_heads][ld] in global
// memory, used when the positions do not fit shared memory (every CTA of a KV head writes the same values there).
// Dynamic shared memory: AX_VSTAGES V tiles of AX_VT x 32 floats, then smem_pos * G floats of probabilities.
// Softmax of the group's heads, the position-ordered value chains of one 32-dim slice, and the outputs (f32 + Q8_0).
// The first V tiles have been requested by the caller.  scores_in_smem: ax_p already holds the scores (the fused
// kernel); otherwise they are read from ws.
__device__ __forceinline__ void ax_softmax_chain_emit(const float *__restrict__ ws, float *__restrict__ pw, uint32_t ld, const void *__restrict__ vc,
                                                      int kv_f16, uint32_t seq, uint32_t n_kv, uint32_t G, uint32_t hd, uint32_t smem_pos,
                                                      uint32_t kvh, uint32_t d0, float *vt, float *ax_p, double *red_d, float *red_f, float *inv_h,
                                                      bool scores_in_smem, float *__restrict__ out, float *scales, int8_t *quants,
                                                      int16_t *sums, const TpHook &tp) {
    const uint32_t pstride = smem_pos + 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t kv_dim = (size_t)n_kv * hd;
    const bool in_smem = seq <= smem_pos;
    const uint32_t n_tiles = (seq + AX_VT - 1) / AX_VT;
    const uint32_t per_pos = kv_f16 ? 4 : 8;  // 16-byte pieces per position

    // ---- probabilities of the group's heads.  Head h is handled by warps [h * nwh, (h + 1) * nwh).
    const uint32_t nwh = (AX_VTHREADS / 32) / G, h_mine = warp / nwh, wl = warp % nwh;  // warps past G * nwh idle here
    const bool has_head = h_mine < G;
    const uint32_t hth = nwh * 32, hti = wl * 32 + lane;  // threads of my head, my index among them
    const float *s_row = ws + (size_t)(kvh * G + (has_head ? h_mine : 0)) * ld;
    float *p_row = pw + (size_t)(kvh * G + (has_head ? h_mine : 0)) * ld;
    float mx = -INFINITY;
    if (has_head) {
#pragma unroll 4
        for (uint32_t t = hti; t < seq; t += hth) {  // (unrolled: the loads of four steps are in flight together)
            const float v = scores_in_smem ? ax_p[(size_t)h_mine * pstride + t] : s_row[t];
            if (in_smem && !scores_in_smem) ax_p[(size_t)h_mine * pstride + t] = v;
            mx = fmaxf(mx, v);  // f32::max fold: NaN scores are ignored
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    if (has_head) {
        mx = red_f[h_mine * nwh];
        for (uint32_t w = 1; w < nwh; ++w) mx = fmaxf(mx, red_f[h_mine * nwh + w]);
    }
    // exponentials and their f64 sum (fixed tree: thread-strided partials, xor shuffles, the head's warps in index order)
    double sum = 0.0;
    if (has_head) {
#pragma unroll 4
        for (uint32_t t = hti; t < seq; t += hth) {
            const float e = ggml_expf(__fsub_rn(in_smem ? ax_p[(size_t)h_mine * pstride + t] : s_row[t], mx));
            if (in_smem) ax_p[(size_t)h_mine * pstride + t] = e;
            else p_row[t] = e;  // every CTA of the KV head stores the same value; the chain multiplies by 1 / sum
            sum += (double)e;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red_d[warp] = sum;
    __syncthreads();
    if (has_head) {
        double tot = red_d[h_mine * nwh];
        for (uint32_t w = 1; w < nwh; ++w) tot += red_d[h_mine * nwh + w];
        const float inv = (float)(1.0 / tot);
        if (wl == 0 && lane == 0) inv_h[h_mine] = inv;
        if (in_smem) {
#pragma unroll 4
            for (uint32_t t = hti; t < seq; t += hth) ax_p[(size_t)h_mine * pstride + t] = __fmul_rn(ax_p[(size_t)h_mine * pstride + t], inv);
        }
    }
    // (the first barrier of the tile loop below also publishes the probabilities)
    // Probabilities that went through global memory come back tile by tile, by asynchronous copies into a ring beside
    // the V tiles (a chain that read them with global loads spent its time on their latency): tiles 0-2 as groups of
    // their own here, later ones in the group of the V tile they belong to.
    float *pt = ax_p;  // [AX_VSTAGES][G][AX_VT], in place of the (unused) probability table
    auto stage_p = [&](uint32_t tile) {
        if (tile < n_tiles) {
            const uint32_t t0 = tile * AX_VT, pieces = (min((uint32_t)AX_VT, seq - t0) + 3) / 4;
            float *dst = pt + (size_t)(tile % AX_VSTAGES) * G * AX_VT;
            for (uint32_t i = tid; i < G * (AX_VT / 4); i += AX_VTHREADS_C) {
                const uint32_t hh = i / (AX_VT / 4), pc = i % (AX_VT / 4);
                if (pc < pieces) ax_cp16(dst + (size_t)hh * AX_VT + pc * 4, pw + (size_t)(kvh * G + hh) * ld + t0 + pc * 4);
            }
        }
    };
    if (!in_smem) {
        __syncthreads();  // every thread's probabilities are written
#pragma unroll
        for (int i = 0; i < AX_VSTAGES; ++i) {
            stage_p(i);
            ax_commit();
        }
    }

    // ---- out[d] = fma(p[t], V[t][d], out[d]) in position order: warp h walks head h, a lane per output dim
    const bool chain = (uint32_t)warp < G;
    const uint32_t h = warp, d = lane;
    float acc = 0.0f;
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        // this thread's copies of tile `tile` have landed: tiles 0-2 were committed up front, tile j + 2 in iteration j,
        // so at most two younger groups (iteration 0) or one (later) may still be in flight
        if (tile == 0) ax_wait<2>();
        else ax_wait<1>();
        __syncthreads();  // everyone's have; and every chain warp is done with the slot restaged below
        if (tile > 0) {
            if (!in_smem) stage_p(tile - 1 + AX_VSTAGES);  // joins the commit group of the V tile below
            ax_stage_tile(tile - 1 + AX_VSTAGES, n_tiles, seq, per_pos, vt, vc, kv_dim, (size_t)kvh * hd + d0, kv_f16, tid);
        }
        if (chain) {
            const uint32_t t0 = tile * AX_VT, cnt = min((uint32_t)AX_VT, seq - t0);
            const char *base = reinterpret_cast<const char *>(vt + (size_t)(tile % AX_VSTAGES) * AX_VT * 32);
            // separate instantiations so that shared-memory probabilities are read with shared loads, not generic ones
            if (in_smem) acc = kv_f16 ? ax_chain_tile<true>(base, ax_p + (size_t)h * pstride + t0, cnt, d, 1.0f, acc)
                                      : ax_chain_tile<false>(base, ax_p + (size_t)h * pstride + t0, cnt, d, 1.0f, acc);
            else {
                const float *pp = pt + (size_t)(tile % AX_VSTAGES) * G * AX_VT + (size_t)h * AX_VT;
                const float inv = inv_h[h];  // the staged values are the exponentials: p = e * (1 / sum), rounded, as the reference stores it
                acc = kv_f16 ? ax_chain_tile<true>(base, pp, cnt, d, inv, acc) : ax_chain_tile<false>(base, pp, cnt, d, inv, acc);
            }
        }
    }
    ax_wait<0>();
    if (!chain) return;
    const size_t o = (size_t)(kvh * G + h) * hd + d0 + d;
    out[o] = acc;
    if (quants) {
        // Q8_0 of the 32-dim block this warp holds (cera/src/backend/cpu.rs:942-958)
        const float av = fabsf(acc);
        float amax = av == av ? av : 0.0f;
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sft));
        const float dd = __fdiv_rn(amax, 127.0f);
        const float r = __fdiv_rn(1.0f, dd);
        const float id = (dd != 0.0f && isfinite(r)) ? r : 0.0f;
        const float pq = rintf(__fmul_rn(acc, id));
        const int qv = pq != pq ? 0 : (int)fminf(fmaxf(pq, -128.0f), 127.0f);
        int s16 = qv;  // sums of the two 16-element halves
#pragma unroll
        for (int sft = 8; sft > 0; sft >>= 1) s16 += __shfl_xor_sync(0xffffffffu, s16, sft);
        const float sc = __half2float(__float2half_rn(dd));
        quants[o] = (int8_t)qv;
        if (d == 0) scales[o / 32] = sc;
        if ((d & 15) == 0) sums[o / 16] = (int16_t)s16;
        if (tp.push) {
            // peers receive whole 32-bit words: lanes 0, 4, 8, ... gather their four quants
            uint32_t packed = (uint32_t)(uint8_t)qv;
            packed |= (uint32_t)(uint8_t)__shfl_down_sync(0xffffffffu, qv, 1) << 8;
            packed |= (uint32_t)(uint8_t)__shfl_down_sync(0xffffffffu, qv, 2) << 16;
            packed |= (uint32_t)(uint8_t)__shfl_down_sync(0xffffffffu, qv, 3) << 24;
            if ((d & 3) == 0) tp_push(tp.ctx, reinterpret_cast<uint32_t *>(quants + o), packed);
            if (d == 0) tp_push(tp.ctx, scales + o / 32, sc);
            if ((d & 15) == 0) tp_push(tp.ctx, sums + o / 16, (int16_t)s16);
        }
    }
}

// grid (hd / 32, n_kv), AX_VTHREADS threads.  ws: scores [n_heads][ld]; pw: probabilities [n_heads][ld] in global
// memory, used when the positions do not fit shared memory (every CTA of a KV head writes the same values there).
// Dynamic shared memory: AX_VSTAGES V tiles of AX_VT x 32 floats, then smem_pos * G floats of probabilities.
__global__ void __launch_bounds__(AX_VTHREADS)
attn_values_exact_kernel(const float *__restrict__ ws, float *__restrict__ pw, uint32_t ld, const void *__restrict__ vc, int kv_f16,
                         uint32_t seq_len, const uint32_t *__restrict__ seq_dev, uint32_t n_kv, uint32_t G, uint32_t hd,
                         uint32_t smem_pos, float *__restrict__ out, float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    extern __shared__ __align__(16) float ax_dyn[];
    float *vt = ax_dyn;                                  // [AX_VSTAGES][AX_VT][32] (f16 caches use half of each tile)
    float *ax_p = ax_dyn + AX_VSTAGES * AX_VT * 32;      // [G][smem_pos + 4]: a head's probabilities are contiguous, heads four banks apart
    __shared__ double red_d[AX_VTHREADS / 32];
    __shared__ float red_f[AX_VTHREADS / 32];
    __shared__ float inv_h[8];  // 1 / sum of every head of the group
    pdl_trigger();
    const uint32_t kvh = blockIdx.y, d0 = blockIdx.x * 32;
    pdl_wait();
    uint32_t seq = seq_dev ? *seq_dev : seq_len;
    // a launch planned with a probability table serves lengths up to the table (the host checks this for lengths it knows
    // and plans captured launches from the length they will meet); never index past it
    if (smem_pos && seq > smem_pos) seq = smem_pos;
    const uint32_t n_tiles = (seq + AX_VT - 1) / AX_VT;
    // V tiles: a position's 32-dim slice is 128 contiguous bytes (64 for an f16 cache): 16-byte asynchronous copies,
    // the first tiles are requested before the softmax so that they land while it runs
#pragma unroll
    for (int i = 0; i < AX_VSTAGES; ++i)
        ax_stage_tile(i, n_tiles, seq, kv_f16 ? 4 : 8, vt, vc, (size_t)n_kv * hd, (size_t)kvh * hd + d0, kv_f16, threadIdx.x);
    ax_softmax_chain_emit(ws, pw, ld, vc, kv_f16, seq, n_kv, G, hd, smem_pos, kvh, d0, vt, ax_p, red_d, red_f, inv_h, false, out, scales, quants,
                          sums, tp);
}

// ONE launch for contexts whose scores fit shared memory: the hd / 32 CTAs of a KV head are a thread-block cluster.
// CTA r computes the scores of the r-th share of the positions (a half-warp per (position, head) as above, four
// positions in flight per warp) and stores each into the score table of EVERY CTA of the cluster (distributed shared
// memory); after one cluster barrier each CTA runs the softmax on its own copy and the value chains of its 32 dims.
// grid = n_kv * CL CTAs (CL = hd / 32), AX_VTHREADS threads; dynamic shared memory: V tiles, score table, G * hd floats of q.
template <int HD>
__global__ void __launch_bounds__(AX_VTHREADS)
attn_fused_exact_kernel(const float *__restrict__ q, const void *__restrict__ kc, const void *__restrict__ vc, int kv_f16, uint32_t seq_len,
                        const uint32_t *__restrict__ seq_dev, uint32_t n_kv, uint32_t G, float scale, uint32_t smem_pos,
                        float *__restrict__ out, float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    extern __shared__ __align__(16) float ax_dyn[];
    constexpr uint32_t CL = HD / 32, NK = HD / 16;       // cluster size; K elements per lane of a half-warp
    float *vt = ax_dyn;
    float *ax_p = ax_dyn + AX_VSTAGES * AX_VT * 32;      // [G][smem_pos + 4]
    const uint32_t pstride = smem_pos + 4;
    float *ax_q = ax_p + (size_t)G * pstride;            // [G][HD]
    __shared__ double red_d[AX_VTHREADS / 32];
    __shared__ float red_f[AX_VTHREADS / 32];
    __shared__ float inv_h[8];  // 1 / sum of every head of the group
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t r = cluster.block_rank(), kvh = blockIdx.x / CL, d0 = r * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // a CTA's shared memory may be written by its peers only once it runs: every CTA arrives here, and waits for the
    // others just before its first remote store
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    pdl_trigger();
    pdl_wait();
    uint32_t seq = seq_dev ? *seq_dev : seq_len;
    if (seq > smem_pos) seq = smem_pos;  // the score tables hold smem_pos positions (see the values kernel)
    const uint32_t n_tiles = (seq + AX_VT - 1) / AX_VT;
#pragma unroll
    for (int i = 0; i < AX_VSTAGES; ++i)
        ax_stage_tile(i, n_tiles, seq, kv_f16 ? 4 : 8, vt, vc, (size_t)n_kv * HD, (size_t)kvh * HD + d0, kv_f16, tid);
    for (uint32_t i = tid; i < G * HD; i += AX_VTHREADS) ax_q[i] = q[(size_t)kvh * G * HD + i];
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    // ---- scores of this CTA's share of the positions, into every CTA's table
    {
        const uint32_t share = (seq + CL - 1) / CL, t_begin = r * share, t_end = min(seq, t_begin + share);
        const uint32_t c16 = lane & 15, hsel = lane >> 4;
        float *peer_p = cluster.map_shared_rank(ax_p, c16 < CL ? c16 : 0);  // lane c of a half-warp stores into CTA c's table
        const size_t kv_dim = (size_t)n_kv * HD;
        constexpr uint32_t UN = 4;  // positions in flight per warp
        for (uint32_t t0 = t_begin + warp * UN; t0 < t_end; t0 += (AX_VTHREADS / 32) * UN) {
            // lane c16 = 8a + L holds elements 16j + c16 of each K row (chunk 2j + a of the reference's alternating accumulators)
            float kv[UN][NK];
#pragma unroll
            for (uint32_t u = 0; u < UN; ++u) {
                const uint32_t t = min(t0 + u, t_end - 1);
                const size_t row = (size_t)t * kv_dim + (size_t)kvh * HD;
#pragma unroll
                for (uint32_t j = 0; j < NK; ++j) {
                    const size_t e = row + 16 * j + c16;
                    kv[u][j] = kv_f16 ? __half2float(__ldg(reinterpret_cast<const __half *>(kc) + e)) : __ldg(reinterpret_cast<const float *>(kc) + e);
                }
            }
            for (uint32_t h0 = 0; h0 < G; h0 += 2) {
                const uint32_t h = h0 + hsel;
                const bool live = h < G;
                const float *qh = ax_q + (live ? h : 0) * HD;
                float qv[NK];
#pragma unroll
                for (uint32_t j = 0; j < NK; ++j) qv[j] = qh[16 * j + c16];
#pragma unroll
                for (uint32_t u = 0; u < UN; ++u) {
                    float acc = 0.0f;
#pragma unroll
                    for (uint32_t j = 0; j < NK; ++j) acc = fmaf(qv[j], kv[u][j], acc);
                    // accumulators 0 and 1 of the same lane L, then hsum256
                    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
                    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
                    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
                    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
                    const float sc = __fmul_rn(acc, scale);
                    if (live && c16 < CL && t0 + u < t_end) peer_p[(size_t)h * pstride + t0 + u] = sc;
                }
            }
        }
    }
    cluster.sync();  // every CTA's table is complete; nothing remote is touched after this point
    ax_softmax_chain_emit(nullptr, nullptr, 0, vc, kv_f16, seq, n_kv, G, HD, smem_pos, kvh, d0, vt, ax_p, red_d, red_f, inv_h, true, out, scales,
                          quants, sums, tp);
}

constexpr size_t AX_SMEM_MAX = 226 * 1024;  // dynamic shared memory the values / fused kernels may ask for

template <int HD>
int32_t launch_fused(uint32_t cl, size_t smem, cudaStream_t st, const float *q, const void *kc, const void *vc, int kv_f16, uint32_t seq_len,
                     const uint32_t *seq_dev, uint32_t nkv, uint32_t G, float scale, uint32_t fpos, float *out, float *scales,
                     int8_t *quants, int16_t *sums, const TpHook &tp) {
    static thread_local int raised_dev = -1;  // per head size: opt in to more than 48 KB once per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (raised_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(attn_fused_exact_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AX_SMEM_MAX));
        raised_dev = dev;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nkv * cl);
    cfg.blockDim = dim3(AX_VTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    count_launch();
    return check_cuda(cudaLaunchKernelEx(&cfg, attn_fused_exact_kernel<HD>, q, kc, vc, kv_f16, seq_len, seq_dev, nkv, G, scale, fpos, out, scales,
                                         quants, sums, tp),
                      "attention (fused) launch");
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
    // ---- one launch when the scores fit shared memory (CERA_CUDA_ATTN_EXACT=split keeps the two-kernel form)
    static const bool no_fused = [] { const char *e = getenv("CERA_CUDA_ATTN_EXACT"); return e && strcmp(e, "split") == 0; }();
    if (!no_fused && b == 1 && (hd == 64 || hd == 128 || hd == 256)) {  // up to 1024 positions (measured: 12.7 against 14.3 us at 512, slower than the pair at 4096)
        const uint32_t fpos = (uint32_t)reach;
        const size_t fsmem = ((size_t)AX_VSTAGES * AX_VT * 32 + ((size_t)fpos + 4) * G + (size_t)G * hd) * sizeof(float);
        if (fsmem <= AX_SMEM_MAX) {
            const uint32_t cl = hd / 32;
            const TpHook hook = tp ? *tp : TpHook{};
            if (hd == 64)
                return launch_fused<64>(cl, fsmem, st, q, kc, vc, kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, scale, fpos, out, scales, quants, sums, hook);
            if (hd == 128)
                return launch_fused<128>(cl, fsmem, st, q, kc, vc, kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, scale, fpos, out, scales, quants, sums, hook);
            return launch_fused<256>(cl, fsmem, st, q, kc, vc, kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, scale, fpos, out, scales, quants, sums, hook);
        }
    }
    // scores: a fixed number of CTAs per KV head walks the position tiles, so one captured launch serves every length
    const uint32_t tiles = (uint32_t)((reach + AX_SWARPS - 1) / AX_SWARPS);
    uint32_t per_head = (uint32_t)(4 * sm_count() / (int)nkv);
    if (per_head < 1) per_head = 1;
    if (per_head > tiles) per_head = tiles;
    count_launch();
    const dim3 sgrid(per_head, nkv), sblock(AX_SWARPS * 32);
    const size_t sq = (size_t)G * hd * sizeof(float);
    const uint32_t sl32 = (uint32_t)seq_len;
    if (hd == 128) CERA_CUDA_TRY(launch_k(attn_scores_exact_kernel<128>, sgrid, sblock, sq, st, q, kc, kv_f16, sl32, seq_len_dev, nkv, G, hd, scale, ws, ld));
    else if (hd == 64) CERA_CUDA_TRY(launch_k(attn_scores_exact_kernel<64>, sgrid, sblock, sq, st, q, kc, kv_f16, sl32, seq_len_dev, nkv, G, hd, scale, ws, ld));
    else CERA_CUDA_TRY(launch_k(attn_scores_exact_kernel<0>, sgrid, sblock, sq, st, q, kc, kv_f16, sl32, seq_len_dev, nkv, G, hd, scale, ws, ld));
    uint32_t smem_pos = b >= 5 ? 0u : (uint32_t)reach;
    if (((size_t)AX_VSTAGES * AX_VT * 32 + ((size_t)smem_pos + 4) * G) * sizeof(float) > AX_SMEM_MAX) smem_pos = 0;  // probabilities through global memory
    // probability table [G][smem_pos + 4], or - probabilities through global memory - a ring of probability tiles [stages][G][AX_VT]
    const size_t smem = ((size_t)AX_VSTAGES * AX_VT * 32 + (smem_pos ? ((size_t)smem_pos + 4) * G : (size_t)AX_VSTAGES * G * AX_VT)) * sizeof(float);
    {
        // static + dynamic shared memory can pass the 48 KB default even at the shortest contexts: opt in once per device
        static thread_local int raised_dev = -1;
        int dev = 0;
        cudaGetDevice(&dev);
        if (raised_dev != dev) {
            CERA_CUDA_TRY(cudaFuncSetAttribute(attn_values_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AX_SMEM_MAX));
            raised_dev = dev;
        }
    }
    count_launch();
    return check_cuda(launch_k(attn_values_exact_kernel, dim3(hd / 32, nkv), dim3(AX_VTHREADS), smem, st, (const float *)ws, pw, ld, vc,
                               kv_f16, (uint32_t)seq_len, seq_len_dev, nkv, G, hd, smem_pos, out, scales, quants, sums,
                               tp ? *tp : TpHook{}),
                      "attention (values) launch");
}

}  // namespace cera
