// Causal attention of a chunk of prompt tokens (prefill), tiled through shared memory.
//
// A CTA owns one KV head and PA_BQ consecutive query tokens; warp w owns query w of the block with all G query heads of
// the group, so every staged K / V row serves PA_BQ * G (query, head) pairs.  Keys go by in tiles of 32, double-buffered
// with cp.async:
//   scores : lane = key.  The lane keeps 32 dims of its K row in registers at a time and reads the queries as
//            shared-memory broadcasts: no shuffle per key, four FMAs per broadcast load.
//   softmax: one running maximum / sum per (query, head), updated once per tile (two warp reductions and ONE expf per
//            key, against a reduction and two expf per key in the one-warp-per-row kernel).
//   P.V    : lane = four output dims.  The tile's probabilities sit in shared memory, V rows are read as float4 and
//            shared by the G heads.
// Rows are padded to 132 floats (f16 caches: staged as stored, 272 bytes per row, widened on the way to the registers),
// so the lane = key reads (stride one row) hit all 32 banks.
//
// Arithmetic contract: cera/src/backend/cpu.rs:4028-4241 (scaled dot, causal limit start_pos + j, online softmax);
// the f32 summation order is this kernel's own.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "act.cuh"
#include "ops.h"
#include "tma.cuh"

namespace cera {

namespace {

constexpr int PA_WARPS = 8, PA_THREADS = PA_WARPS * 32, PA_BQ = PA_WARPS;
constexpr int PA_TK = 32;        // keys per tile
constexpr int PA_HD = 128;       // head dim
constexpr int PA_ROW_F32 = 528, PA_ROW_F16 = 272;   // bytes per staged row (512 / 256 of data + padding)

template <int G, bool F16>
constexpr size_t pa_smem_bytes() {
    return (size_t)2 * 2 * PA_TK * (F16 ? PA_ROW_F16 : PA_ROW_F32) + (size_t)(PA_BQ * G * PA_HD + PA_WARPS * G * PA_TK) * sizeof(float);
}

// Eight consecutive elements of a staged row as two float4.
template <bool F16>
__device__ __forceinline__ void pa_load8(const uint8_t *row, int first, float4 &a, float4 &b) {
    if (F16) {
        const uint4 r = *reinterpret_cast<const uint4 *>(row + first * 2);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&r.z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2 *>(&r.w));
        a = make_float4(f0.x, f0.y, f1.x, f1.y);
        b = make_float4(f2.x, f2.y, f3.x, f3.y);
    } else {
        a = *reinterpret_cast<const float4 *>(row + first * 4);
        b = *reinterpret_cast<const float4 *>(row + first * 4 + 16);
    }
}
template <bool F16>
__device__ __forceinline__ float4 pa_load4(const uint8_t *row, int first) {
    if (F16) {
        const uint2 r = *reinterpret_cast<const uint2 *>(row + first * 2);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
        return make_float4(f0.x, f0.y, f1.x, f1.y);
    }
    return *reinterpret_cast<const float4 *>(row + first * 4);
}

__device__ __forceinline__ float pa_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

template <int G, bool F16>
__global__ void __launch_bounds__(PA_THREADS) attn_prefill_tiled_kernel(const float *__restrict__ q, const uint8_t *__restrict__ kc,
                                                                        const uint8_t *__restrict__ vc, uint32_t n_heads,
                                                                        uint32_t n_kv_heads, uint32_t n, uint32_t start_pos,
                                                                        float scale, float *__restrict__ out) {
    extern __shared__ __align__(16) uint8_t pa_smem[];
    constexpr int ROWB = F16 ? PA_ROW_F16 : PA_ROW_F32, ESZ = F16 ? 2 : 4, STAGE = PA_TK * ROWB;
    constexpr int PIECES = PA_HD * ESZ / 16;          // 16-byte pieces per cache row
    uint8_t *ks = pa_smem;                            // [2][32][ROWB]
    uint8_t *vs = ks + 2 * STAGE;                     // [2][32][ROWB]
    float *qs = reinterpret_cast<float *>(vs + 2 * STAGE);   // [PA_BQ * G][128]
    float *ps = qs + PA_BQ * G * PA_HD;               // [warps][G][32]

    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t kvh = blockIdx.x;
    const uint32_t qb = gridDim.y - 1 - blockIdx.y;   // the longest rows start first
    const uint32_t q0 = qb * PA_BQ, j = q0 + warp;
    const size_t kv_dim = (size_t)n_kv_heads * PA_HD, q_dim = (size_t)n_heads * PA_HD;
    const uint32_t q_last = min(q0 + PA_BQ, n) - 1;
    const uint32_t cta_kv = start_pos + q_last + 1;   // keys the block's last query sees
    const uint32_t n_tiles = (cta_kv + PA_TK - 1) / PA_TK;
    const bool live = j < n;
    const uint32_t my_kv = live ? start_pos + j + 1 : 0;

    auto issue = [&](uint32_t t, int stage) {
        uint8_t *kd = ks + stage * STAGE, *vd = vs + stage * STAGE;
        for (int i = tid; i < PA_TK * PIECES; i += PA_THREADS) {
            const int r = i / PIECES, pc = i % PIECES;
            const uint32_t key = min(t * PA_TK + r, cta_kv - 1);   // rows past the limit are masked; keep the read in range
            const size_t src = ((size_t)key * kv_dim + (size_t)kvh * PA_HD) * ESZ + pc * 16;
            tma::cp_async16(kd + r * ROWB + pc * 16, kc + src);
            tma::cp_async16(vd + r * ROWB + pc * 16, vc + src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    issue(0, 0);
    // queries of the block: pair (w, g) at qs[(w * G + g) * 128]
    for (int i = tid; i < PA_BQ * G * 32; i += PA_THREADS) {
        const int pair = i >> 5, pc = i & 31;
        const uint32_t jq = q0 + pair / G;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (jq < n) v = *reinterpret_cast<const float4 *>(q + jq * q_dim + ((size_t)kvh * G + pair % G) * PA_HD + pc * 4);
        *reinterpret_cast<float4 *>(qs + pair * PA_HD + pc * 4) = v;
    }

    float m_run[G], l_run[G];
    float4 acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.0f;
        acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float *qw = qs + warp * G * PA_HD;
    float *pw = ps + warp * G * PA_TK;

    for (uint32_t t = 0; t < n_tiles; ++t) {
        const int stage = t & 1;
        if (t + 1 < n_tiles) {
            issue(t + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (t * PA_TK < my_kv) {
            const uint8_t *kt = ks + stage * STAGE + lane * ROWB;
            const uint8_t *vt = vs + stage * STAGE;
            float2 s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int dc = 0; dc < PA_HD / 32; ++dc) {
                float4 kr[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) pa_load8<F16>(kt, dc * 32 + 8 * i, kr[2 * i], kr[2 * i + 1]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 qq = *reinterpret_cast<const float4 *>(qw + g * PA_HD + dc * 32 + 4 * i);
                        // packed f32 pairs (FFMA2): even dims accumulate in .x, odd dims in .y
                        s[g] = __ffma2_rn(make_float2(qq.x, qq.y), make_float2(kr[i].x, kr[i].y), s[g]);
                        s[g] = __ffma2_rn(make_float2(qq.z, qq.w), make_float2(kr[i].z, kr[i].w), s[g]);
                    }
                }
            }
            const bool valid = t * PA_TK + lane < my_kv;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float sv = valid ? __fmul_rn(__fadd_rn(s[g].x, s[g].y), scale) : -INFINITY;
                const float m_new = fmaxf(m_run[g], pa_warp_max(sv));   // finite: key t * 32 is valid for this query
                const float corr = m_run[g] == -INFINITY ? 0.0f : ggml_expf(__fsub_rn(m_run[g], m_new));
                const float p = valid ? ggml_expf(__fsub_rn(sv, m_new)) : 0.0f;
                l_run[g] = fmaf(l_run[g], corr, warp_sum(p));
                acc[g].x *= corr;
                acc[g].y *= corr;
                acc[g].z *= corr;
                acc[g].w *= corr;
                m_run[g] = m_new;
                pw[g * PA_TK + lane] = p;
            }
            __syncwarp();
#pragma unroll
            for (int k4 = 0; k4 < PA_TK / 4; ++k4) {
                const float4 v0 = pa_load4<F16>(vt + (4 * k4 + 0) * ROWB, 4 * lane);
                const float4 v1 = pa_load4<F16>(vt + (4 * k4 + 1) * ROWB, 4 * lane);
                const float4 v2 = pa_load4<F16>(vt + (4 * k4 + 2) * ROWB, 4 * lane);
                const float4 v3 = pa_load4<F16>(vt + (4 * k4 + 3) * ROWB, 4 * lane);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float4 pp = *reinterpret_cast<const float4 *>(pw + g * PA_TK + 4 * k4);
                    const float2 p0 = make_float2(pp.x, pp.x), p1 = make_float2(pp.y, pp.y), p2 = make_float2(pp.z, pp.z),
                                 p3 = make_float2(pp.w, pp.w);
                    float2 lo = make_float2(acc[g].x, acc[g].y), hi = make_float2(acc[g].z, acc[g].w);
                    lo = __ffma2_rn(p3, make_float2(v3.x, v3.y), __ffma2_rn(p2, make_float2(v2.x, v2.y),
                         __ffma2_rn(p1, make_float2(v1.x, v1.y), __ffma2_rn(p0, make_float2(v0.x, v0.y), lo))));
                    hi = __ffma2_rn(p3, make_float2(v3.z, v3.w), __ffma2_rn(p2, make_float2(v2.z, v2.w),
                         __ffma2_rn(p1, make_float2(v1.z, v1.w), __ffma2_rn(p0, make_float2(v0.z, v0.w), hi))));
                    acc[g] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
            __syncwarp();   // the probabilities are rewritten by the next tile
        }
        __syncthreads();    // the stage is refilled by the copy issued in the next iteration
    }

    if (live) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float inv = 1.0f / l_run[g];
            float4 o = make_float4(acc[g].x * inv, acc[g].y * inv, acc[g].z * inv, acc[g].w * inv);
            *reinterpret_cast<float4 *>(out + j * q_dim + ((size_t)kvh * G + g) * PA_HD + 4 * lane) = o;
        }
    }
}

template <int G, bool F16>
int32_t launch_tiled(const float *q, const uint8_t *kc, const uint8_t *vc, uint32_t nh, uint32_t nkv, uint32_t n, uint32_t sp,
                     float scale, float *out, cudaStream_t st) {
    constexpr size_t smem = pa_smem_bytes<G, F16>();
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_tiled_kernel<G, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_dev = dev;
    }
    const dim3 grid(nkv, (n + PA_BQ - 1) / PA_BQ);
    count_launch();
    return check_cuda(launch_k(attn_prefill_tiled_kernel<G, F16>, grid, dim3(PA_THREADS), smem, st, q, kc, vc, nh, nkv, n, sp, scale, out),
                      "prefill attention (tiled) launch");
}

}  // namespace

// f32 or f16 cache, head_dim 128, group size 1, 2, 4 or 8, 16-byte aligned operands; anything else: *taken = false and the
// caller runs the one-warp-per-row kernel.  CERA_CUDA_PREFILL_ATTN=rows turns this kernel off.
int32_t launch_prefill_attention_tiled(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                       size_t n_kv_heads, size_t head_dim, size_t n, size_t start_pos, float scale, float *out,
                                       cudaStream_t st, bool *taken) {
    *taken = false;
    static const bool off = [] {
        const char *e = getenv("CERA_CUDA_PREFILL_ATTN");
        return e && strcmp(e, "rows") == 0;
    }();
    if (off || head_dim != PA_HD || n == 0) return CERA_CUDA_OK;
    if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) % 16) return CERA_CUDA_OK;
    const size_t g = n_heads / n_kv_heads;
    const uint32_t nh = (uint32_t)n_heads, nkv = (uint32_t)n_kv_heads, nn = (uint32_t)n, sp = (uint32_t)start_pos;
    const uint8_t *kf = (const uint8_t *)kc, *vf = (const uint8_t *)vc;
    *taken = true;
#define CERA_PA_CASE(GG)                                                                              \
    case GG:                                                                                          \
        return kv_f16 ? launch_tiled<GG, true>(q, kf, vf, nh, nkv, nn, sp, scale, out, st)            \
                      : launch_tiled<GG, false>(q, kf, vf, nh, nkv, nn, sp, scale, out, st)
    switch (g) {
        CERA_PA_CASE(1);
        CERA_PA_CASE(2);
        CERA_PA_CASE(4);
        CERA_PA_CASE(8);
        default: *taken = false; return CERA_CUDA_OK;
    }
#undef CERA_PA_CASE
}

}  // namespace cera
