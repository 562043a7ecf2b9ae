// Flash-decode GQA attention: split-KV partial pass + merge pass.
//
// HBM-bound on the KV stream.  Grid = (n_kv_heads, n_splits): one CTA owns one
// KV head and one contiguous range of cached positions and serves all G = n_heads /
// n_kv_heads query heads of that KV head, so every K and V row is read from
// HBM exactly once.  Inside a CTA each warp walks tiles of P = 32/G positions:
//   * lane L holds head_dim/32 consecutive dims of every row (coalesced 128-bit loads),
//   * the P*G partial dot products are reduced with a 31-shuffle butterfly transpose,
//     leaving score (position L/G, head L%G) on lane L,
//   * running max / sum per head are kept online (one exp per lane per tile),
//   * probabilities are broadcast back by shuffle for the P x V accumulation.
// Warps merge through shared memory, splits merge in a second kernel that also
// emits the Q8_0 form of the output for the o-projection.
//
// Arithmetic contract: cera/src/model/transformer.rs:1166-1305 with
// cera/src/backend/cpu.rs:3222-3363 (scores = q.K * scale, softmax with the
// polynomial expf, weighted V sum); the online form agrees within f32 rounding.
#include <cooperative_groups.h>

#include <cstdlib>
#include <cstring>

#include "ops.h"

namespace cg = cooperative_groups;

namespace cera {

namespace {

constexpr int ATT_WARPS = 8;
constexpr int MAX_SPLITS = 64;
constexpr uint32_t ATT_CLUSTER_FLAG = 0x80;
constexpr uint32_t ATT_STREAM_FLAG = 0x100;  // long contexts: the split kernel that stages K/V through shared memory with cp.async, low bits = splits
constexpr size_t ATT_CLUSTER_MAX_SEQ = 4096;

template <int VEC, bool F16>
__device__ __forceinline__ void load_row(const void *base, size_t elem_off, float (&v)[VEC]) {
    if (F16) {
        const __half *p = reinterpret_cast<const __half *>(base) + elem_off;
        if (VEC == 4) {
            const uint2 u = *reinterpret_cast<const uint2 *>(p);
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
#pragma unroll
            for (int i = 0; i < VEC; i += 2) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(p + i));
                v[i] = a.x;
                v[i + 1] = a.y;
            }
        }
    } else {
        const float *p = reinterpret_cast<const float *>(base) + elem_off;
        if (VEC % 4 == 0) {
#pragma unroll
            for (int i = 0; i < VEC; i += 4) {
                const float4 a = *reinterpret_cast<const float4 *>(p + i);
                v[i] = a.x; v[i + 1] = a.y; v[i + 2] = a.z; v[i + 3] = a.w;
            }
        } else {
            const float2 a = *reinterpret_cast<const float2 *>(p);
            v[0] = a.x;
            v[1] = a.y;
        }
    }
}

// The scan of one CTA over cached positions [t_begin, t_end) of KV head kvh for its G query heads: on return
// acc / m_run / l_run hold this warp's unnormalised output, running maximum and running sum (the state of head
// lane % G, replicated over its P lanes).
template <int VEC, int G, bool F16, int W>
__device__ __forceinline__ void attn_scan(const float *__restrict__ q, const void *__restrict__ kc, const void *__restrict__ vc,
                                          uint32_t kvh, uint32_t t_begin, uint32_t t_end, size_t kv_dim, float scale,
                                          float (&acc)[G][VEC], float &m_run, float &l_run) {
    constexpr int HD = VEC * 32;
    constexpr int P = 32 / G;  // positions per warp tile
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // q slices of the G heads this CTA serves
    float qv[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) qv[g][v] = q[(size_t)(kvh * G + g) * HD + lane * VEC + v];

#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[g][v] = 0.0f;
    m_run = -INFINITY;
    l_run = 0.0f;

    const size_t head_off = (size_t)kvh * HD + lane * VEC;
    for (uint32_t t0 = t_begin + warp * P; t0 < t_end; t0 += W * P) {
        float kr[P][VEC], vr[P][VEC];
#pragma unroll
        for (int i = 0; i < P; ++i) {
            const uint32_t t = t0 + i;
            if (t < t_end) {
                load_row<VEC, F16>(kc, t * kv_dim + head_off, kr[i]);
                load_row<VEC, F16>(vc, t * kv_dim + head_off, vr[i]);
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) kr[i][v] = vr[i][v] = 0.0f;
            }
        }
        float val[32];
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float s = 0.0f;
#pragma unroll
                for (int v = 0; v < VEC; ++v) s = fmaf(qv[g][v], kr[i][v], s);
                val[i * G + g] = s;
            }
        // butterfly transpose-reduce: afterwards lane L holds the full sum of val[L]
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int j = 0; j < o; ++j) {
                const float send = up ? val[j] : val[j + o];
                const float keep = up ? val[j + o] : val[j];
                val[j] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        const uint32_t my_t = t0 + lane / G;
        const float s = my_t < t_end ? __fmul_rn(val[0], scale) : -INFINITY;
        float tmax = s;
#pragma unroll
        for (int o = G; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m_run, tmax);  // finite: the tile holds at least one valid position
        const float p = my_t < t_end ? ggml_expf(__fsub_rn(s, m_new)) : 0.0f;
        const float corr = m_run == -INFINITY ? 0.0f : ggml_expf(__fsub_rn(m_run, m_new));
        float psum = p;
#pragma unroll
        for (int o = G; o < 32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l_run = fmaf(l_run, corr, psum);
        m_run = m_new;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float cg = __shfl_sync(0xffffffffu, corr, g);
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[g][v] *= cg;
        }
#pragma unroll
        for (int i = 0; i < P; ++i)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pg = __shfl_sync(0xffffffffu, p, i * G + g);
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[g][v] = fmaf(pg, vr[i][v], acc[g][v]);
            }
    }
}

// Workspace record per (query head, split): out[head_dim], max, sum.
template <int VEC, int G, bool F16>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_split_kernel(const float *__restrict__ q, const void *__restrict__ kc, const void *__restrict__ vc,
                  uint32_t seq_len_imm, const uint32_t *__restrict__ seq_len_dev, uint32_t n_kv_heads, float scale,
                  float *__restrict__ ws) {
    constexpr int HD = VEC * 32;
    constexpr int P = 32 / G;  // positions per warp tile
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const uint32_t seq_len = seq_len_dev ? *seq_len_dev : seq_len_imm;
    const size_t kv_dim = (size_t)n_kv_heads * HD;

    uint32_t chunk = (seq_len + n_splits - 1) / n_splits;
    chunk = (chunk + P - 1) / P * P;
    const uint32_t t_begin = min(seq_len, split * chunk), t_end = min(seq_len, t_begin + chunk);

    float acc[G][VEC];
    float m_run, l_run;
    attn_scan<VEC, G, F16, ATT_WARPS>(q, kc, vc, kvh, t_begin, t_end, kv_dim, scale, acc, m_run, l_run);

    // merge the warps of this CTA
    __shared__ float s_acc[ATT_WARPS][G][HD];
    __shared__ float s_m[ATT_WARPS][G], s_l[ATT_WARPS][G];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) s_acc[warp][g][lane * VEC + v] = acc[g][v];
    if (lane < G) {
        s_m[warp][lane] = m_run;
        s_l[warp][lane] = l_run;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, s_m[w][g]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float f = s_m[w][g] == -INFINITY ? 0.0f : ggml_expf(s_m[w][g] - M);
            L = fmaf(s_l[w][g], f, L);
            O = fmaf(s_acc[w][g][d], f, O);
        }
        float *rec = ws + ((size_t)(kvh * G + g) * n_splits + split) * (HD + 2);
        rec[d] = O;
        if (d == 0) {
            rec[HD] = M;
            rec[HD + 1] = L;
        }
    }
}

// One CTA per query head, one thread per output dim.
__global__ void attn_merge_kernel(const float *__restrict__ ws, uint32_t n_splits, uint32_t hd, float *__restrict__ out,
                                  float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    pdl_trigger();
    pdl_wait();
    const uint32_t h = blockIdx.x, d = threadIdx.x;
    const float *base = ws + (size_t)h * n_splits * (hd + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * (hd + 2) + hd]);
    double L = 0.0;
    float O = 0.0f;
    for (uint32_t s = 0; s < n_splits; ++s) {
        const float *rec = base + s * (hd + 2);
        const float m = rec[hd];
        const float f = m == -INFINITY ? 0.0f : ggml_expf(m - M);
        L += (double)(rec[hd + 1] * f);
        O = fmaf(rec[d], f, O);
    }
    const float v = O * (float)(1.0 / L);
    const size_t o = (size_t)h * hd + d;
    out[o] = v;
    if (quants) {
        float scale;
        int hs;
        const int qv = quantize_lane(v, scale, hs);
        quants[o] = (int8_t)qv;
        if ((d & 31) == 0) scales[o / 32] = scale;
        if ((d & 15) == 0) sums[o / 16] = (int16_t)hs;
        if (tp.push) {
            tp_push(tp.ctx, quants + o, (int8_t)qv);
            if ((d & 31) == 0) tp_push(tp.ctx, scales + o / 32, scale);
            if ((d & 15) == 0) tp_push(tp.ctx, sums + o / 16, (int16_t)hs);
        }
    }
}

// Short contexts (up to ATT_CLUSTER_MAX_SEQ positions): the splits of one KV head form a thread-block
// cluster and merge through distributed shared memory, so one launch does what the split and merge
// kernels do and the partial results never leave the SMs.  Grid = n_kv_heads * CL CTAs in clusters of
// CL; CTA r of a cluster scans the r-th share of the positions, leaves its (out, max, sum) per query
// head in its own shared memory, and after a cluster barrier combines G*HD/CL of the outputs from all
// CL shares (same arithmetic as attn_merge_kernel), emitting f32 and Q8_0.
template <int VEC, int G, bool F16, int W>
__global__ void __launch_bounds__(W * 32)
attn_cluster_kernel(const float *__restrict__ q, const void *__restrict__ kc, const void *__restrict__ vc,
                    uint32_t seq_len_imm, const uint32_t *__restrict__ seq_len_dev, uint32_t n_kv_heads, float scale,
                    float *__restrict__ out, float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    constexpr int HD = VEC * 32;
    constexpr int P = 32 / G;
    __shared__ float s_acc[W][G][HD];
    __shared__ float s_m[W][G], s_l[W][G];
    __shared__ float part[G][HD];      // this CTA's share, read by the whole cluster
    __shared__ float part_m[G], part_l[G];
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t CL = cluster.num_blocks(), split = cluster.block_rank();
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kvh = blockIdx.x / CL;
    const uint32_t seq_len = seq_len_dev ? *seq_len_dev : seq_len_imm;
    const size_t kv_dim = (size_t)n_kv_heads * HD;
    uint32_t chunk = (seq_len + CL - 1) / CL;
    chunk = (chunk + P - 1) / P * P;
    const uint32_t t_begin = min(seq_len, split * chunk), t_end = min(seq_len, t_begin + chunk);

    float acc[G][VEC];
    float m_run, l_run;
    attn_scan<VEC, G, F16, W>(q, kc, vc, kvh, t_begin, t_end, kv_dim, scale, acc, m_run, l_run);

#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int v = 0; v < VEC; ++v) s_acc[warp][g][lane * VEC + v] = acc[g][v];
    if (lane < G) {
        s_m[warp][lane] = m_run;
        s_l[warp][lane] = l_run;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < W; ++w) M = fmaxf(M, s_m[w][g]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const float f = s_m[w][g] == -INFINITY ? 0.0f : ggml_expf(s_m[w][g] - M);
            L = fmaf(s_l[w][g], f, L);
            O = fmaf(s_acc[w][g][d], f, O);
        }
        part[g][d] = O;
        if (d == 0) {
            part_m[g] = M;
            part_l[g] = L;
        }
    }
    cluster.sync();
    // outputs [split * per, (split + 1) * per) of this KV head's G*HD; per is a multiple of 32, so every warp
    // that enters the loop is whole and quantizes one Q8_0 block
    const int per = G * HD / (int)CL;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int idx = (int)split * per + i, g = idx / HD, d = idx % HD;
        // remote reads in batches of eight, issued together (they are independent: one round trip through the cluster
        // network per batch, not one per share); pass 1 finds the maximum, pass 2 accumulates
        float M = -INFINITY;
        for (uint32_t r0 = 0; r0 < CL; r0 += 8) {
            float mv[8];
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) mv[r] = r0 + r < CL ? cluster.map_shared_rank(&part_m[0], r0 + r)[g] : -INFINITY;
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) M = fmaxf(M, mv[r]);
        }
        double L = 0.0;
        float O = 0.0f;
        for (uint32_t r0 = 0; r0 < CL; r0 += 8) {
            float mv[8], lv[8], ov[8];
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) {
                const bool in = r0 + r < CL;
                mv[r] = in ? cluster.map_shared_rank(&part_m[0], r0 + r)[g] : -INFINITY;
                lv[r] = in ? cluster.map_shared_rank(&part_l[0], r0 + r)[g] : 0.0f;
                ov[r] = in ? cluster.map_shared_rank(&part[0][0], r0 + r)[g * HD + d] : 0.0f;
            }
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) {
                const float f = mv[r] == -INFINITY ? 0.0f : ggml_expf(mv[r] - M);
                L += (double)(lv[r] * f);
                O = fmaf(ov[r], f, O);
            }
        }
        const float v = O * (float)(1.0 / L);
        const size_t o = (size_t)(kvh * G + g) * HD + d;
        out[o] = v;
        if (quants) {
            float qs;
            int hs;
            const int qv = quantize_lane(v, qs, hs);
            quants[o] = (int8_t)qv;
            if ((d & 31) == 0) scales[o / 32] = qs;
            if ((d & 15) == 0) sums[o / 16] = (int16_t)hs;
            if (tp.push) {
                tp_push(tp.ctx, quants + o, (int8_t)qv);
                if ((d & 31) == 0) tp_push(tp.ctx, scales + o / 32, qs);
                if ((d & 15) == 0) tp_push(tp.ctx, sums + o / 16, (int16_t)hs);
            }
        }
    }
    cluster.sync();  // peers may still be reading this CTA's share
}

// Causal attention for a batch of prompt tokens: one warp per (query head, query token), online softmax
// over cache rows [0, start_pos + j] with the polynomial expf (cera/src/backend/cpu.rs:4146-4241; the tile
// width there is 32, here 1, which only changes f32 rounding).  q / out are token-major.
template <int VEC, bool F16>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_prefill_kernel(const float *__restrict__ q, const void *__restrict__ kc, const void *__restrict__ vc, uint32_t n_heads,
                    uint32_t n_kv_heads, uint32_t n, uint32_t start_pos, float scale, float *__restrict__ out) {
    constexpr int HD = VEC * 32;
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t h = blockIdx.x, j = blockIdx.y * ATT_WARPS + warp;
    if (j >= n) return;
    const uint32_t kvh = h / (n_heads / n_kv_heads);
    const size_t kv_dim = (size_t)n_kv_heads * HD, q_dim = (size_t)n_heads * HD;
    const size_t head_off = (size_t)kvh * HD + lane * VEC;
    float qv[VEC], acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        qv[v] = q[j * q_dim + (size_t)h * HD + lane * VEC + v];
        acc[v] = 0.0f;
    }
    float m_run = -INFINITY, l_run = 0.0f;
    const uint32_t max_kv = start_pos + j + 1;
    for (uint32_t t0 = 0; t0 < max_kv; t0 += 4) {
        float kr[4][VEC], vr[4][VEC], sc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (t0 + i < max_kv) {
                load_row<VEC, F16>(kc, (t0 + i) * kv_dim + head_off, kr[i]);
                load_row<VEC, F16>(vc, (t0 + i) * kv_dim + head_off, vr[i]);
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) kr[i][v] = vr[i][v] = 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float s = 0.0f;
#pragma unroll
            for (int v = 0; v < VEC; ++v) s = fmaf(qv[v], kr[i][v], s);
            sc[i] = s;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (t0 + i >= max_kv) break;
            const float s = __fmul_rn(sc[i], scale);
            const float m_new = fmaxf(m_run, s);
            const float corr = m_run == -INFINITY ? 0.0f : ggml_expf(__fsub_rn(m_run, m_new));
            const float pexp = ggml_expf(__fsub_rn(s, m_new));
            l_run = fmaf(l_run, corr, pexp);
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(pexp, vr[i][v], acc[v] * corr);
            m_run = m_new;
        }
    }
    const float inv = 1.0f / l_run;
#pragma unroll
    for (int v = 0; v < VEC; ++v) out[j * q_dim + (size_t)h * HD + lane * VEC + v] = acc[v] * inv;
}

template <int VEC, int G>
int32_t launch_split(bool f16, dim3 grid, cudaStream_t st, const float *q, const void *kc, const void *vc,
                     uint32_t seq_len, const uint32_t *seq_dev, uint32_t n_kv, float scale, float *ws) {
    if (f16)
        return check_cuda(launch_k(attn_split_kernel<VEC, G, true>, grid, dim3(ATT_WARPS * 32), 0, st, q, kc, vc, seq_len,
                                   seq_dev, n_kv, scale, ws), "attention launch");
    return check_cuda(launch_k(attn_split_kernel<VEC, G, false>, grid, dim3(ATT_WARPS * 32), 0, st, q, kc, vc, seq_len,
                               seq_dev, n_kv, scale, ws), "attention launch");
}

template <int VEC, int G, int W>
int32_t launch_cluster(bool f16, uint32_t cl, cudaStream_t st, const float *q, const void *kc, const void *vc, uint32_t seq_len,
                       const uint32_t *seq_dev, uint32_t n_kv, float scale, float *out, float *scales, int8_t *quants,
                       int16_t *sums, const TpHook &tp) {
    if (cl > 8) {
        static thread_local int configured_dev = -1;
        int dev = 0;
        cudaGetDevice(&dev);
        if (configured_dev != dev) {
            CERA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<VEC, G, true, W>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
            CERA_CUDA_TRY(cudaFuncSetAttribute(attn_cluster_kernel<VEC, G, false, W>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
            configured_dev = dev;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_kv * cl);
    cfg.blockDim = dim3(W * 32);
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
    if (f16)
        return check_cuda(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<VEC, G, true, W>, q, kc, vc, seq_len, seq_dev, n_kv, scale, out,
                                             scales, quants, sums, tp), "attention (cluster) launch");
    return check_cuda(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<VEC, G, false, W>, q, kc, vc, seq_len, seq_dev, n_kv, scale, out,
                                         scales, quants, sums, tp), "attention (cluster) launch");
}

}  // namespace

constexpr uint32_t ATT_EXACT_FLAG = 0x200;  // plan word of the reference-order kernels (attention_exact.cu)

// Enough for either decode path: per-split partial records (split kernels) or the score and probability rows of every
// head (reference-order kernels).
size_t attn_workspace_bytes(size_t n_heads, size_t head_dim, size_t seq_len) {
    const size_t split = n_heads * MAX_SPLITS * (head_dim + 2) * sizeof(float);
    const size_t exact = attn_exact_workspace_bytes(n_heads, seq_len);
    return split > exact ? split : exact;
}

uint32_t attn_plan(size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t seq_len_hint) {
    if (attn_exact_supports(n_heads, n_kv_heads, head_dim)) return attn_exact_plan(seq_len_hint);
    return attn_pick_splits(n_kv_heads, seq_len_hint);
}

// Plan for a decode attention over seq_len_hint positions.  Up to ATT_CLUSTER_MAX_SEQ positions: the one-launch
// cluster kernel, returned as ATT_CLUSTER_FLAG | cluster size (1, 2, 4, 8 or 16; about 64 positions per CTA, more
// once the cluster is full).  Beyond: the number of splits of the two-kernel path.
// CERA_CUDA_ATTN=split keeps every length on the two-kernel path.
uint32_t attn_pick_splits(size_t n_kv_heads, size_t seq_len_hint) {
    static const bool no_cluster = [] {
        const char *e = getenv("CERA_CUDA_ATTN");
        return e && strcmp(e, "split") == 0;
    }();
    if (!no_cluster && seq_len_hint <= ATT_CLUSTER_MAX_SEQ) {
        // about 128 positions per CTA (one pass of its 16 warps at a group size of 4) up to the portable cluster of 8
        // (measured faster than 16 up to 1024 positions); longer contexts take 16 CTAs per cluster, which the kernel
        // opts into
        uint32_t cl = 1;
        while (cl < 8 && (size_t)cl * 128 < seq_len_hint) cl <<= 1;
        if (seq_len_hint > 1024) cl = 16;
        return ATT_CLUSTER_FLAG | cl;
    }
    static const bool no_stream = [] {
        const char *e = getenv("CERA_CUDA_ATTN");
        return e && (strcmp(e, "split") == 0 || strcmp(e, "registers") == 0);
    }();
    if (!no_stream) {
        // one CTA per SM, every split a whole number of 64-position tiles
        size_t ns = (size_t)sm_count() / (n_kv_heads ? n_kv_heads : 1);
        const size_t tiles = (seq_len_hint + 63) / 64;
        if (ns > tiles) ns = tiles;
        if (ns > 63) ns = 63;
        if (ns < 1) ns = 1;
        return ATT_STREAM_FLAG | (uint32_t)ns;
    }
    // Fill the machine about twice over, but never give a split fewer than 64 positions.
    size_t want = (size_t)(2 * sm_count() + n_kv_heads - 1) / n_kv_heads;
    const size_t by_len = (seq_len_hint + 63) / 64;
    if (want > by_len) want = by_len;
    if (want < 1) want = 1;
    if (want > MAX_SPLITS) want = MAX_SPLITS;
    return (uint32_t)want;
}

int32_t launch_decode_attention_ex(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                   size_t n_kv_heads, size_t head_dim, size_t seq_len, const uint32_t *seq_len_dev,
                                   uint32_t n_splits, float scale, float *out, void *workspace, size_t workspace_bytes,
                                   float *scales, int8_t *quants, int16_t *sums, cudaStream_t st, const TpHook *tp) {
    if (!q || !kc || !vc || !out || !workspace) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: null argument");
    if (n_kv_heads == 0 || n_heads % n_kv_heads)
        return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: n_heads (%zu) must be a positive multiple of n_kv_heads (%zu)",
                    n_heads, n_kv_heads);
    const size_t G = n_heads / n_kv_heads;
    if (seq_len == 0 && !seq_len_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: empty KV cache");
    if (n_splits & ATT_EXACT_FLAG)
        return launch_decode_attention_exact(q, kc, vc, kv_f16, n_heads, n_kv_heads, head_dim, seq_len, seq_len_dev, n_splits, scale,
                                             out, workspace, workspace_bytes, scales, quants, sums, st, tp);
    if (workspace_bytes < attn_workspace_bytes(n_heads, head_dim, 0))
        return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: workspace of %zu bytes is too small", workspace_bytes);
    const bool streamed = (n_splits & ATT_STREAM_FLAG) != 0;
    if (streamed) n_splits &= ~ATT_STREAM_FLAG;
    const bool clustered = (n_splits & ATT_CLUSTER_FLAG) != 0;
    uint32_t cl = n_splits & ~ATT_CLUSTER_FLAG;
    if (clustered ? (cl != 1 && cl != 2 && cl != 4 && cl != 8 && cl != 16) : (n_splits < 1 || n_splits > MAX_SPLITS))
        return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention: split plan 0x%x", n_splits);
    // every CTA of a cluster finishes whole 32-wide Q8_0 blocks of the G*head_dim outputs of its KV head
    while (clustered && cl > 1 && (G * head_dim / cl) % 32) cl >>= 1;
    const dim3 grid((unsigned)n_kv_heads, clustered ? 1 : n_splits);
    float *ws = (float *)workspace;
    const bool f16 = kv_f16 != 0;
    const uint32_t sl = (uint32_t)seq_len, nkv = (uint32_t)n_kv_heads;
    const TpHook hook = tp ? *tp : TpHook{};
    // Cluster kernel: 16 warps per CTA for groups of 4 up to 1024 positions (128 positions per pass, 32 KB of merge
    // buffers), 8 warps otherwise (measured faster in clusters of 16; groups of 8 would not fit static shared memory).
#define CERA_ATT(VEC, GG)                                                                                                  \
    att_status = !clustered ? launch_split<VEC, GG>(f16, grid, st, q, kc, vc, sl, seq_len_dev, nkv, scale, ws)               \
                 : (GG == 4 && cl <= 8)                                                                                     \
                     ? launch_cluster<VEC, GG, (GG == 4 ? 16 : 8)>(f16, cl, st, q, kc, vc, sl, seq_len_dev, nkv, scale, out, scales,   \
                                                                  quants, sums, hook)                                       \
                     : launch_cluster<VEC, GG, 8>(f16, cl, st, q, kc, vc, sl, seq_len_dev, nkv, scale, out, scales, quants, sums, hook)
    bool ok = true;
    int32_t att_status = CERA_CUDA_OK;
    bool stream_taken = false;
    if (streamed) {
        CERA_TRY(launch_attention_stream(q, kc, vc, kv_f16, n_kv_heads, G, head_dim, sl, seq_len_dev, n_splits, scale, ws, st,
                                         &stream_taken));
    }
    if (stream_taken) {
    } else if (head_dim == 128) {
        switch (G) {
            case 4: CERA_ATT(4, 4); break;
            case 8: CERA_ATT(4, 8); break;
            default: ok = false;
        }
    } else if (head_dim == 64) {
        switch (G) {
            case 4: CERA_ATT(2, 4); break;
            case 8: CERA_ATT(2, 8); break;
            default: ok = false;
        }
    } else {
        ok = false;
    }
#undef CERA_ATT
    if (!ok)
        return fail(CERA_CUDA_ERR_UNSUPPORTED, "decode_attention: head_dim %zu with group size %zu has no kernel "
                    "(head_dim 64 or 128, group 4 or 8)", head_dim, G);
    count_launch();
    CERA_TRY(att_status);
    if (clustered) return CERA_CUDA_OK;
    count_launch();
    return check_cuda(launch_k(attn_merge_kernel, dim3((unsigned)n_heads), dim3((unsigned)head_dim), 0, st,
                               (const float *)ws, n_splits, (uint32_t)head_dim, out, scales, quants, sums,
                               tp ? *tp : TpHook{}),
                      "attention merge launch");
}

int32_t launch_prefill_attention(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                 size_t n_kv_heads, size_t head_dim, size_t n, size_t start_pos, float scale, float *out,
                                 cudaStream_t st) {
    if (!q || !kc || !vc || !out) return fail(CERA_CUDA_ERR_BAD_ARG, "prefill_attention: null argument");
    if (n_kv_heads == 0 || n_heads % n_kv_heads) return fail(CERA_CUDA_ERR_BAD_ARG, "prefill_attention: bad head counts");
    if (n == 0) return CERA_CUDA_OK;
    bool tiled = false;
    CERA_TRY(launch_prefill_attention_tiled(q, kc, vc, kv_f16, n_heads, n_kv_heads, head_dim, n, start_pos, scale, out, st, &tiled));
    if (tiled) return CERA_CUDA_OK;
    const dim3 grid((unsigned)n_heads, (unsigned)((n + ATT_WARPS - 1) / ATT_WARPS));
    const dim3 block(ATT_WARPS * 32);
    const uint32_t nh = (uint32_t)n_heads, nkv = (uint32_t)n_kv_heads, nn = (uint32_t)n, sp = (uint32_t)start_pos;
    count_launch();
    if (head_dim == 128) {
        if (kv_f16) return check_cuda(launch_k(attn_prefill_kernel<4, true>, grid, block, 0, st, q, kc, vc, nh, nkv, nn, sp, scale, out), "prefill attention launch");
        return check_cuda(launch_k(attn_prefill_kernel<4, false>, grid, block, 0, st, q, kc, vc, nh, nkv, nn, sp, scale, out), "prefill attention launch");
    }
    if (head_dim == 64) {
        if (kv_f16) return check_cuda(launch_k(attn_prefill_kernel<2, true>, grid, block, 0, st, q, kc, vc, nh, nkv, nn, sp, scale, out), "prefill attention launch");
        return check_cuda(launch_k(attn_prefill_kernel<2, false>, grid, block, 0, st, q, kc, vc, nh, nkv, nn, sp, scale, out), "prefill attention launch");
    }
    return fail(CERA_CUDA_ERR_UNSUPPORTED, "prefill_attention: head_dim %zu has no kernel (64 or 128)", head_dim);
}

int32_t launch_decode_attention(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                size_t n_kv_heads, size_t head_dim, size_t seq_len, float scale, float *out,
                                void *workspace, size_t workspace_bytes, float *scales, int8_t *quants, int16_t *sums,
                                cudaStream_t st) {
    return launch_decode_attention_ex(q, kc, vc, kv_f16, n_heads, n_kv_heads, head_dim, seq_len, nullptr,
                                      attn_plan(n_heads, n_kv_heads, head_dim, seq_len), scale, out, workspace, workspace_bytes,
                                      scales, quants, sums, st);
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_prefill_attention(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev, int32_t kv_f16,
                                    size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t n, size_t start_pos,
                                    float scale, float *out_dev, void *stream) {
    return launch_prefill_attention(q_dev, k_cache_dev, v_cache_dev, kv_f16, n_heads, n_kv_heads, head_dim, n, start_pos,
                                    scale, out_dev, (cudaStream_t)stream);
}

size_t cera_cuda_decode_attention_workspace_bytes(size_t n_heads, size_t head_dim, size_t seq_len) {
    return attn_workspace_bytes(n_heads, head_dim, seq_len);
}

int32_t cera_cuda_decode_attention(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev, int32_t kv_f16,
                                   size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t seq_len, float scale,
                                   float *out_dev, void *workspace_dev, size_t workspace_bytes, void *stream) {
    return launch_decode_attention(q_dev, k_cache_dev, v_cache_dev, kv_f16, n_heads, n_kv_heads, head_dim, seq_len,
                                   scale, out_dev, workspace_dev, workspace_bytes, nullptr, nullptr, nullptr,
                                   (cudaStream_t)stream);
}

}  // extern "C"
