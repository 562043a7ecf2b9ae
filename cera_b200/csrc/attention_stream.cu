// Long-context flash-decode attention: the KV stream staged through a shared-memory ring by asynchronous copies.
//
// Same split-KV contract as attention.cu (one CTA per (KV head, split) serves all G query heads and leaves
// an (out, max, sum) record per head for attn_merge_kernel), built for contexts of thousands of positions,
// where the register-resident kernel runs out of loads in flight.  One CTA of 8 warps per SM walks its
// positions in tiles of 64.  A tile's K and V rows (a head's slice of a cache row is one contiguous 128-512
// byte range, rows are a cache-row pitch apart) are copied into one stage of a shared-memory ring with
// 16-byte cp.async operations, 16-32 per thread; the copies of the next STAGES-1 tiles (up to 200 KB per SM)
// are in flight while a tile is consumed, at no register cost, in the classic multistage form: wait for the
// oldest commit group, one CTA barrier, issue the tile that reuses the stage everybody just left, compute.
// (Two TMA forms were measured first and dropped: one cp.async.bulk per row keeps the TMA unit busy with
// 128 requests of 512 bytes per tile, 1.9 TB/s; a single producer warp issuing the 16-byte copies cannot
// issue them fast enough, 3.2 TB/s.)
//
// Arithmetic per tile, in two phases with a CTA barrier between them.
//   Scores: warp w takes positions [32*(w/4), +32) and dims [HD/4*(w%4), +HD/4); lane = position.  A lane reads its
//   K row piece once (a quarter warp reads eight different rows: 128 useful bytes per shared-memory wavefront) and
//   uses it for all G heads, whose q values are broadcast reads; no cross-lane reduction.  The four quarter sums of
//   a (position, head) go to shared memory.  (With lane = (position, head) each K element was read G times and the
//   kernel was bound by shared-memory wavefronts: 85 us at 32 768 positions against 45 us.)
//   Softmax and P x V: warp w takes positions [8w, 8w+8); lane = (position, head) adds the quarter sums, keeps the
//   running max / sum of its head online with the polynomial expf; the probabilities go through a 128-byte per-warp
//   buffer, and for the P x V product every lane owns head_dim/32 output dims of all G heads.
//
// Arithmetic contract: cera/src/model/transformer.rs:1166-1305 with cera/src/backend/cpu.rs:3222-3363
// (scores = q.K * scale, softmax with ggml's expf, weighted V sum); the online, split form agrees within
// f32 rounding.  The kernel has no spin waits: cp.async.wait_group and CTA barriers only.
#include <cstdlib>
#include <cstring>

#include "ops.h"
#include "tma.cuh"

namespace cera {

namespace {

constexpr int AS_CW = 8;                       // warps per CTA
constexpr int AS_THREADS = AS_CW * 32;
constexpr int AS_TILE = 64;                    // positions per stage, 8 per warp
constexpr size_t AS_SMEM_BUDGET = 226 * 1024;  // of the 227 KB a CTA may opt into
constexpr size_t AS_HEADER = 128;

template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int HD, bool F16>
__device__ __forceinline__ float4 ld4(const uint8_t *row, int d) {
    if (F16) {
        const uint2 u = *reinterpret_cast<const uint2 *>(row + d * 2);
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return *reinterpret_cast<const float4 *>(row + d * 4);
}

template <int HD, int G, bool F16, int S>
__global__ void __launch_bounds__(AS_THREADS, 1)
attn_stream_kernel(const float *__restrict__ q, const uint8_t *__restrict__ kc, const uint8_t *__restrict__ vc,
                   uint32_t seq_len_imm, const uint32_t *__restrict__ seq_len_dev, uint32_t n_kv_heads, float scale,
                   float *__restrict__ ws) {
    constexpr int VEC = HD / 32;               // output dims per lane
    constexpr int PPS = 32 / G;                // positions per warp step
    constexpr int STEPS = 8 / PPS;
    constexpr int ESZ = F16 ? 2 : 4;
    constexpr int RB = HD * ESZ;               // bytes of a head's slice of a cache row
    constexpr int RS = RB + 16;                // stage row stride: 8 rows start in 8 different bank groups
    constexpr int STAGE = 2 * AS_TILE * RS;    // K rows then V rows
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int QS = HD + 4;  // q row stride: the G heads read by a quarter warp start in different bank groups
    float *qs = reinterpret_cast<float *>(smem + AS_HEADER);               // [G][QS]
    float *pbuf = qs + G * QS;                                             // [AS_CW][32]
    float *cbuf = pbuf + AS_CW * 32;                                       // [AS_CW][G]
    float *s_m = cbuf + AS_CW * G, *s_l = s_m + AS_CW * G;                 // [AS_CW][G] each
    float *s_acc = s_l + AS_CW * G;                                        // [AS_CW][G][HD]
    float *spart = s_acc + AS_CW * G * HD;                                 // [4 dim quarters][AS_TILE][G] partial scores
    uint8_t *ring = reinterpret_cast<uint8_t *>(spart + 4 * AS_TILE * G);
    ring = reinterpret_cast<uint8_t *>(((uintptr_t)ring + 127) & ~(uintptr_t)127);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    pdl_trigger();
    pdl_wait();  // the newest cache row and q come from the previous kernels
    const uint32_t seq_len = seq_len_dev ? *seq_len_dev : seq_len_imm;
    uint32_t chunk = (seq_len + n_splits - 1) / n_splits;
    chunk = (chunk + AS_TILE - 1) / AS_TILE * AS_TILE;
    const uint32_t t_begin = min(seq_len, split * chunk), t_end = min(seq_len, t_begin + chunk);
    const uint32_t n_tiles = (t_end - t_begin + AS_TILE - 1) / AS_TILE;
    for (int i = threadIdx.x; i < G * HD; i += AS_THREADS) qs[(i / HD) * QS + i % HD] = q[(size_t)kvh * G * HD + i];

    const size_t row_pitch = (size_t)n_kv_heads * RB;  // bytes between consecutive positions
    // every thread copies its share of tile `i` into stage i % S and closes a commit group (also when the tile does
    // not exist, so that "all but the newest S-2 groups" always means "tile i has landed")
    auto issue = [&](uint32_t i) {
        if (i < n_tiles) {
            constexpr uint32_t CPR = RB / 16;  // 16-byte pieces per row
            const uint32_t t0 = t_begin + i * AS_TILE, rows = min((uint32_t)AS_TILE, t_end - t0);
            uint8_t *st = ring + (size_t)(i % S) * STAGE;
            // thread t copies piece t % CPR of rows t / CPR, t / CPR + RSTEP, ...: pointers advance by constants
            constexpr uint32_t RSTEP = AS_THREADS / CPR;
            const uint32_t c16 = (threadIdx.x % CPR) * 16;
            uint32_t r = threadIdx.x / CPR;
            size_t src = (size_t)(t0 + r) * row_pitch + (size_t)kvh * RB + c16;
            uint8_t *dk = st + r * RS + c16;
            for (; r < rows; r += RSTEP, src += (size_t)RSTEP * row_pitch, dk += RSTEP * RS) {
                tma::cp_async16(dk, kc + src);
                tma::cp_async16(dk + AS_TILE * RS, vc + src);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < S - 1; ++i) issue((uint32_t)i);

    // ---------------- consumers
    float acc[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[g][v] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // state of head lane % G, replicated over the lanes that share it
    const int head = lane % G, pin = lane / G;
    float *pw = pbuf + warp * 32, *cw = cbuf + warp * G;
    for (uint32_t i = 0; i < n_tiles; ++i) {
        cp_async_wait_group<S - 2>();  // this thread's copies of tile i have landed
        __syncthreads();               // ... everybody's have, q is in place, everybody has left tile i-1's stage and scores
        issue(i + S - 1);              // which is the stage tile i+S-1 goes into
        const uint8_t *kst = ring + (size_t)(i % S) * STAGE, *vst = kst + AS_TILE * RS;
        const uint32_t t0 = t_begin + i * AS_TILE;
        {
            // ---- scores: lane = position, this warp's quarter of the dims, all G heads
            constexpr int QD = HD / 4;
            const uint32_t pos = 32 * (warp >> 2) + lane;
            const int c = warp & 3;
            if (t0 + 32 * (warp >> 2) < t_end) {  // warp-uniform
                const uint8_t *krow = kst + min(pos, (uint32_t)(AS_TILE - 1)) * RS;
                float sa[G], sb[G];
#pragma unroll
                for (int g = 0; g < G; ++g) sa[g] = sb[g] = 0.0f;
#pragma unroll
                for (int d = c * QD; d < (c + 1) * QD; d += 4) {
                    const float4 k4 = ld4<HD, F16>(krow, d);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 q4 = *reinterpret_cast<const float4 *>(qs + g * QS + d);  // same address on every lane
                        sa[g] = fmaf(q4.x, k4.x, sa[g]);
                        sb[g] = fmaf(q4.y, k4.y, sb[g]);
                        sa[g] = fmaf(q4.z, k4.z, sa[g]);
                        sb[g] = fmaf(q4.w, k4.w, sb[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) spart[(c * AS_TILE + pos) * G + g] = sa[g] + sb[g];
            }
        }
        __syncthreads();
#pragma unroll
        for (int step = 0; step < STEPS; ++step) {
            const uint32_t first = 8 * warp + step * PPS;  // first position of this step inside the tile
            if (t0 + first >= t_end) break;                // warp-uniform: nothing of this step is cached
            const uint32_t mine = first + pin;
            const bool valid = t0 + mine < t_end;
            float sc = -INFINITY;
            if (valid) {
                const float *sp = spart + mine * G + head;
                sc = __fmul_rn((sp[0] + sp[AS_TILE * G]) + (sp[2 * AS_TILE * G] + sp[3 * AS_TILE * G]), scale);
            }
            float tmax = sc;
#pragma unroll
            for (int o = G; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            const float m_new = fmaxf(m_run, tmax);  // finite: the step's first position is cached
            const float p = valid ? ggml_expf(__fsub_rn(sc, m_new)) : 0.0f;
            const float corr = m_run == -INFINITY ? 0.0f : ggml_expf(__fsub_rn(m_run, m_new));
            float psum = p;
#pragma unroll
            for (int o = G; o < 32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l_run = fmaf(l_run, corr, psum);
            m_run = m_new;
            pw[lane] = p;                    // [position in step][head]
            if (lane < G) cw[lane] = corr;   // lane < G has head == lane
            __syncwarp();
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float cg = cw[g];
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[g][v] *= cg;
            }
#pragma unroll
            for (int j = 0; j < PPS; ++j) {
                if (t0 + first + j >= t_end) break;  // warp-uniform
                const uint8_t *vrow = vst + (first + j) * RS;
                float vv[VEC];
                if constexpr (VEC == 4) {
                    const float4 v4 = ld4<HD, F16>(vrow, lane * 4);
                    vv[0] = v4.x; vv[1] = v4.y; vv[2] = v4.z; vv[3] = v4.w;
                } else {
#pragma unroll
                    for (int v = 0; v < VEC; ++v)
                        vv[v] = F16 ? __half2float(reinterpret_cast<const __half *>(vrow)[lane * VEC + v])
                                    : reinterpret_cast<const float *>(vrow)[lane * VEC + v];
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pg = pw[j * G + g];
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[g][v] = fmaf(pg, vv[v], acc[g][v]);
                }
            }
            __syncwarp();  // pw / cw are rewritten by the next step
        }
    }
    cp_async_wait_group<0>();

    // merge the consumer warps of this CTA (same arithmetic as attn_split_kernel)
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) s_acc[(warp * G + g) * HD + lane * VEC + v] = acc[g][v];
    if (lane < G) {
        s_m[warp * G + lane] = m_run;
        s_l[warp * G + lane] = l_run;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += AS_CW * 32) {
        const int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AS_CW; ++w) M = fmaxf(M, s_m[w * G + g]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < AS_CW; ++w) {
            const float f = s_m[w * G + g] == -INFINITY ? 0.0f : ggml_expf(s_m[w * G + g] - M);
            L = fmaf(s_l[w * G + g], f, L);
            O = fmaf(s_acc[(w * G + g) * HD + d], f, O);
        }
        float *rec = ws + ((size_t)(kvh * G + g) * n_splits + split) * (HD + 2);
        rec[d] = O;
        if (d == 0) {
            rec[HD] = M;
            rec[HD + 1] = L;
        }
    }
}

template <int HD, int G, bool F16, int S>
int32_t launch_stream_staged(dim3 grid, size_t smem, cudaStream_t st, const float *q, const void *kc, const void *vc, uint32_t seq_len,
                             const uint32_t *seq_dev, uint32_t n_kv, float scale, float *ws) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(attn_stream_kernel<HD, G, F16, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AS_SMEM_BUDGET));
        configured_dev = dev;
    }
    return check_cuda(launch_k(attn_stream_kernel<HD, G, F16, S>, grid, dim3(AS_THREADS), smem, st, q, (const uint8_t *)kc,
                               (const uint8_t *)vc, seq_len, seq_dev, n_kv, scale, ws),
                      "attention (stream) launch");
}

template <int HD, int G, bool F16>
int32_t launch_stream_typed(dim3 grid, cudaStream_t st, const float *q, const void *kc, const void *vc, uint32_t seq_len,
                            const uint32_t *seq_dev, uint32_t n_kv, float scale, float *ws) {
    constexpr size_t RS = HD * (F16 ? 2 : 4) + 16, STAGE = 2 * AS_TILE * RS;
    constexpr size_t FIXED =
        AS_HEADER + (size_t)(G * (HD + 4) + AS_CW * 32 + 3 * AS_CW * G + AS_CW * G * HD + 4 * AS_TILE * G) * 4 + 128;
    constexpr int FIT = (int)((AS_SMEM_BUDGET - FIXED) / STAGE);
    constexpr int S = FIT >= 4 ? 4 : FIT;  // 2, 3 or 4 stages
    static_assert(S >= 2, "no room for two stages");
    return launch_stream_staged<HD, G, F16, S>(grid, FIXED + (size_t)S * STAGE, st, q, kc, vc, seq_len, seq_dev, n_kv, scale, ws);
}

}  // namespace

// The split pass of a long-context decode attention through the cp.async-staged kernel; the caller runs the merge
// pass over the same workspace.  *taken = false: shape without an instantiation (head_dim 64 / 128, group 4 / 8).
int32_t launch_attention_stream(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_kv_heads, size_t group,
                                size_t head_dim, uint32_t seq_len, const uint32_t *seq_len_dev, uint32_t n_splits, float scale,
                                float *ws, cudaStream_t st, bool *taken) {
    *taken = true;
    const dim3 grid((unsigned)n_kv_heads, n_splits);
    const uint32_t nkv = (uint32_t)n_kv_heads;
    const bool f16 = kv_f16 != 0;
#define CERA_AS(HDV, GV)                                                                                              \
    return f16 ? launch_stream_typed<HDV, GV, true>(grid, st, q, kc, vc, seq_len, seq_len_dev, nkv, scale, ws)        \
               : launch_stream_typed<HDV, GV, false>(grid, st, q, kc, vc, seq_len, seq_len_dev, nkv, scale, ws)
    if (head_dim == 128 && group == 4) CERA_AS(128, 4);
    if (head_dim == 128 && group == 8) CERA_AS(128, 8);
    if (head_dim == 64 && group == 4) CERA_AS(64, 4);
    if (head_dim == 64 && group == 8) CERA_AS(64, 8);
#undef CERA_AS
    *taken = false;
    return CERA_CUDA_OK;
}

}  // namespace cera
