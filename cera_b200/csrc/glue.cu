// Small kernels around the matmuls on the decode path: RoPE (+KV append),
// embedding row lookup, argmax.
#include <cmath>

#include "formats.cuh"
#include "ops.h"

namespace cera {

namespace {

// One thread per rotation pair.  theta_i = pos * ts^i built by repeated f32
// multiplication exactly as the CPU loop does (cera/src/backend/cpu.rs:5161-5180,
// 5041-5054), so the angle fed to sincos is bit-identical; sincosf itself is
// CUDA's full-range implementation (last-ulp differences from libm are inside
// the path's f32 tolerance).
__global__ void rope_kernel(float *q, float *k, const float *__restrict__ v, uint32_t pos_imm,
                            const uint32_t *__restrict__ pos_dev, uint32_t n_heads, uint32_t n_kv_heads, uint32_t hd,
                            float ts, const float *__restrict__ ff, int neox, void *k_cache, void *v_cache, int kv_f16,
                            const float *__restrict__ table) {
    pdl_trigger();
    pdl_wait();
    const uint32_t half = hd / 2;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t total = (n_heads + n_kv_heads) * half;
    // blockIdx.y walks a batch of tokens at consecutive positions (token-major q / k / v)
    const uint32_t pos = (pos_dev ? *pos_dev : pos_imm) + blockIdx.y;
    const size_t kv_dim = (size_t)n_kv_heads * hd;
    q += (size_t)blockIdx.y * n_heads * hd;
    k += (size_t)blockIdx.y * kv_dim;
    if (v) v += (size_t)blockIdx.y * kv_dim;
    if (idx < total) {
        const uint32_t h = idx / half, i = idx % half;
        float sn, cs;
        if (table) {  // cos / sin of every (position, pair), computed on the host with the C library the reference's host uses
            cs = table[((size_t)pos * half + i) * 2];
            sn = table[((size_t)pos * half + i) * 2 + 1];
        } else {
            float theta = (float)pos;
            for (uint32_t s = 0; s < i; ++s) theta = __fmul_rn(theta, ts);
            if (!neox && ff) theta = __fdiv_rn(theta, ff[i]);
            sincosf(theta, &sn, &cs);
        }
        float *head = h < n_heads ? q + (size_t)h * hd : k + (size_t)(h - n_heads) * hd;
        const uint32_t i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
        const float x0 = head[i0], x1 = head[i1];
        const float r0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        const float r1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        head[i0] = r0;
        head[i1] = r1;
        if (k_cache && h >= n_heads) {
            const size_t o = (size_t)pos * kv_dim + (size_t)(h - n_heads) * hd;
            if (kv_f16) {
                __half *kc = (__half *)k_cache;
                kc[o + i0] = __float2half_rn(r0);
                kc[o + i1] = __float2half_rn(r1);
            } else {
                float *kc = (float *)k_cache;
                kc[o + i0] = r0;
                kc[o + i1] = r1;
            }
        }
    }
    // v rows ride along: threads beyond the rotation pairs are not needed, reuse the same grid
    if (v_cache) {
        for (size_t e = idx; e < kv_dim; e += (size_t)gridDim.x * blockDim.x) {  // gridDim.x spans one token
            const size_t o = (size_t)pos * kv_dim + e;
            if (kv_f16) ((__half *)v_cache)[o] = __float2half_rn(v[e]);
            else ((float *)v_cache)[o] = v[e];
        }
    }
}

// LoRA delta of one projection for one token: y += B (scale * (A x))  (cera/src/lora.rs:794-821 apply_decode; A is
// [rank x k], B is [d x rank], row-major, f32).  Every CTA recomputes the rank-sized vector (A is small and stays in
// L2) and then finishes 256 outputs; each B-row dot product is summed from zero and added to y once, as the
// reference requires for its decode and prefill forms to agree.
constexpr int LORA_MAX_RANK = 256;
__global__ void __launch_bounds__(256) lora_kernel(const float *__restrict__ x, const float *__restrict__ a,
                                                   const float *__restrict__ b, uint32_t rank, uint32_t k, uint32_t d, float scale,
                                                   float *y) {
    __shared__ float tmp[LORA_MAX_RANK];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t r = warp; r < rank; r += 8) {
        const float *row = a + (size_t)r * k;
        float acc = 0.0f;
        for (uint32_t i = lane; i < k; i += 32) acc = fmaf(row[i], x[i], acc);
        acc = warp_sum(acc);
        if (lane == 0) tmp[r] = __fmul_rn(acc, scale);
    }
    __syncthreads();
    const uint32_t o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= d) return;
    const float *row = b + (size_t)o * rank;
    float acc = 0.0f;
    for (uint32_t r = 0; r < rank; ++r) acc = __fadd_rn(acc, __fmul_rn(row[r], tmp[r]));
    y[o] = __fadd_rn(y[o], acc);
}

// Context shift of one layer's cache (cera/src/kv_cache.rs:1091-1320, shift_kv_with_rope): rows
// [n_keep + shift, seq_len) move down by `shift`; every moved K head is rotated once more by R(-shift)
// (cera/src/backend/cpu.rs:5056-5083 split halves, 5145-5180 adjacent pairs, same iterated theta with
// theta_0 = -shift), V rows move unchanged.  The tail is read from a copy (`k_src` / `v_src` hold rows
// [n_keep + shift, seq_len) as they were), so rows can be written in any order.  One thread per
// rotation pair of a K row; the V row rides along.
__global__ void kv_shift_kernel(const void *__restrict__ k_src, const void *__restrict__ v_src, void *k_cache, void *v_cache,
                                uint32_t n_keep, uint32_t shift, uint32_t n_rows, uint32_t n_kv_heads, uint32_t hd, float ts,
                                const float *__restrict__ ff, int neox, int kv_f16) {
    const uint32_t half = hd / 2, row = blockIdx.y;
    if (row >= n_rows) return;
    const size_t kv_dim = (size_t)n_kv_heads * hd;
    const size_t src = (size_t)row * kv_dim, dst = (size_t)(n_keep + row) * kv_dim;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n_kv_heads * half) {
        const uint32_t h = idx / half, i = idx % half;
        float theta = -(float)shift;
        for (uint32_t s = 0; s < i; ++s) theta = __fmul_rn(theta, ts);
        if (!neox && ff) theta = __fdiv_rn(theta, ff[i]);
        float sn, cs;
        sincosf(theta, &sn, &cs);
        const uint32_t i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
        const size_t o = (size_t)h * hd;
        float x0, x1;
        if (kv_f16) {
            x0 = __half2float(((const __half *)k_src)[src + o + i0]);
            x1 = __half2float(((const __half *)k_src)[src + o + i1]);
        } else {
            x0 = ((const float *)k_src)[src + o + i0];
            x1 = ((const float *)k_src)[src + o + i1];
        }
        const float r0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        const float r1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        if (kv_f16) {
            ((__half *)k_cache)[dst + o + i0] = __float2half_rn(r0);
            ((__half *)k_cache)[dst + o + i1] = __float2half_rn(r1);
        } else {
            ((float *)k_cache)[dst + o + i0] = r0;
            ((float *)k_cache)[dst + o + i1] = r1;
        }
    }
    for (size_t e = idx; e < kv_dim; e += (size_t)gridDim.x * blockDim.x) {
        if (kv_f16) ((__half *)v_cache)[dst + e] = ((const __half *)v_src)[src + e];
        else ((float *)v_cache)[dst + e] = ((const float *)v_src)[src + e];
    }
}

template <int T>
__global__ void embed_kernel(WeightView w, uint32_t token_imm, const uint32_t *__restrict__ token_dev, float *out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t token = token_dev ? token_dev[blockIdx.y] : token_imm;  // blockIdx.y walks a batch of tokens
    out += (size_t)blockIdx.y * w.k;
    const int items = w.k / 32;
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= items || token >= w.m) return;
    const typename Fmt<T>::Raw raw = Fmt<T>::load(w, token, item);
    int lo[4], hi[4];
    HalfRef h0, h1;
    Fmt<T>::decode(raw, item, lo, hi, h0, h1);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int q0 = (lo[i] >> (8 * t)) & 0xFF, q1 = (hi[i] >> (8 * t)) & 0xFF;
            if (T == CERA_TYPE_Q8_0) {
                q0 = (int8_t)q0;
                q1 = (int8_t)q1;
            }
            out[h0.off + 4 * i + t] = Fmt<T>::deq(q0, h0);
            out[h1.off + 4 * i + t] = Fmt<T>::deq(q1, h1);
        }
}

constexpr int ARGMAX_BLOCKS = 128, ARGMAX_THREADS = 256;

// Order: greater value wins; on equal values the lower index wins, which is
// what a left-to-right strict `>` scan returns.
__device__ __forceinline__ void amax_merge(float &bv, uint32_t &bi, float v, uint32_t i) {
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

__global__ void argmax_stage1(const float *__restrict__ x, uint32_t n, uint32_t *scratch) {
    pdl_trigger();
    pdl_wait();
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = x[i];
        if (v > bv) {  // ascending i within a thread: strict > keeps the first
            bv = v;
            bi = i;
        }
    }
    __shared__ float sv[ARGMAX_THREADS];
    __shared__ uint32_t si[ARGMAX_THREADS];
    sv[threadIdx.x] = bv;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) amax_merge(sv[threadIdx.x], si[threadIdx.x], sv[threadIdx.x + s], si[threadIdx.x + s]);
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        scratch[2 * blockIdx.x] = __float_as_uint(sv[0]);
        scratch[2 * blockIdx.x + 1] = si[0];
    }
}

__global__ void argmax_stage2(const uint32_t *__restrict__ scratch, int blocks, uint32_t *out) {
    pdl_trigger();
    pdl_wait();
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (int b = threadIdx.x; b < blocks; b += 32) amax_merge(bv, bi, __uint_as_float(scratch[2 * b]), scratch[2 * b + 1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        amax_merge(bv, bi, ov, oi);
    }
    // no finite / non-NaN winner -> index 0, as the reference returns
    if (threadIdx.x == 0) *out = bi == 0xFFFFFFFFu ? 0u : bi;
}

}  // namespace

int32_t launch_rope(float *q, float *k, const float *v, size_t pos, const uint32_t *pos_dev, size_t n_heads,
                    size_t n_kv_heads, size_t head_dim, float theta_scale, const float *freq_factors, int rope_type,
                    void *k_cache, void *v_cache, int kv_f16, cudaStream_t st, const float *table) {
    if (!q || !k) return fail(CERA_CUDA_ERR_BAD_ARG, "rope: null argument");
    if (head_dim == 0 || head_dim % 2) return fail(CERA_CUDA_ERR_BAD_ARG, "rope: head_dim %zu must be even", head_dim);
    if (v_cache && !v) return fail(CERA_CUDA_ERR_BAD_ARG, "rope: v_cache without v");
    const uint32_t total = (uint32_t)((n_heads + n_kv_heads) * (head_dim / 2));
    const int threads = 128;
    count_launch();
    return check_cuda(launch_k(rope_kernel, dim3((total + threads - 1) / threads), dim3(threads), 0, st, q, k, v, (uint32_t)pos,
                               pos_dev, (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)head_dim, theta_scale, freq_factors,
                               rope_type == 1 ? 1 : 0, k_cache, v_cache, kv_f16, table),
                      "rope launch");
}

// cos / sin of every (position, rotation pair) on the host, operation for operation as the reference's loop
// (cera/src/backend/cpu.rs:5041-5054, 5161-5180): theta starts at the position and is multiplied by
// base^(-2/head_dim) per pair in f32, NORM pairs divide by their frequency factor, and sin / cos come from the C
// library - the one a CPU build of the reference on the same host calls, whereas the device's sincosf may differ
// from it in the last bit.  out: [n_pos][head_dim/2][2] = {cos, sin}.
void rope_table_host(size_t n_pos, size_t head_dim, float rope_theta, const float *freq_factors, int rope_type, float *out) {
    const size_t half = head_dim / 2;
    const float ts = std::pow(rope_theta, -2.0f / (float)head_dim);
    const bool neox = rope_type == 1;
    for (size_t pos = 0; pos < n_pos; ++pos) {
        float theta = (float)pos;
        for (size_t i = 0; i < half; ++i) {
            const float t = neox ? theta : theta / (freq_factors ? freq_factors[i] : 1.0f);
            out[(pos * half + i) * 2] = std::cos(t);
            out[(pos * half + i) * 2 + 1] = std::sin(t);
            theta *= ts;
        }
    }
}

int32_t launch_embed(const WeightView &w, uint32_t token, const uint32_t *token_dev, float *out, cudaStream_t st) {
    const int items = w.k / 32, threads = 128;
    count_launch();
    CERA_DISPATCH_BLOCK_TYPE(w.type, return check_cuda(launch_k(embed_kernel<TT>, dim3((items + threads - 1) / threads), dim3(threads),
                                                                0, st, w, token, token_dev, out), "embed launch"));
    return CERA_CUDA_OK;
}

int32_t launch_rope_batch(float *q, float *k, const float *v, size_t start_pos, size_t n, size_t n_heads, size_t n_kv_heads,
                          size_t head_dim, float theta_scale, const float *freq_factors, int rope_type, void *k_cache,
                          void *v_cache, int kv_f16, cudaStream_t st, const float *table) {
    if (!q || !k) return fail(CERA_CUDA_ERR_BAD_ARG, "rope: null argument");
    if (head_dim == 0 || head_dim % 2) return fail(CERA_CUDA_ERR_BAD_ARG, "rope: head_dim %zu must be even", head_dim);
    if (n == 0) return CERA_CUDA_OK;
    const uint32_t total = (uint32_t)((n_heads + n_kv_heads) * (head_dim / 2));
    const int threads = 128;
    count_launch();
    return check_cuda(launch_k(rope_kernel, dim3((total + threads - 1) / threads, (unsigned)n), dim3(threads), 0, st, q, k, v,
                               (uint32_t)start_pos, (const uint32_t *)nullptr, (uint32_t)n_heads, (uint32_t)n_kv_heads,
                               (uint32_t)head_dim, theta_scale, freq_factors, rope_type == 1 ? 1 : 0, k_cache, v_cache, kv_f16, table),
                      "rope launch");
}

int32_t launch_embed_batch(const WeightView &w, const uint32_t *tokens_dev, size_t n, float *out, cudaStream_t st) {
    if (n == 0) return CERA_CUDA_OK;
    const int items = w.k / 32, threads = 128;
    count_launch();
    CERA_DISPATCH_BLOCK_TYPE(w.type, return check_cuda(launch_k(embed_kernel<TT>, dim3((items + threads - 1) / threads, (unsigned)n),
                                                                dim3(threads), 0, st, w, 0u, tokens_dev, out), "embed launch"));
    return CERA_CUDA_OK;
}

size_t argmax_scratch_words() { return 2 * ARGMAX_BLOCKS; }

namespace {
__global__ void scale_kernel(float *__restrict__ x, size_t n, float s) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] = __fmul_rn(x[i], s);
}
__global__ void scaled_add_kernel(float *__restrict__ y, const float *__restrict__ x, size_t n, float s) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __fadd_rn(y[i], __fmul_rn(x[i], s));
}
}  // namespace

int32_t launch_scale(float *x, size_t n, float s, cudaStream_t st) {
    if (n == 0) return CERA_CUDA_OK;
    const unsigned grid = (unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    count_launch();
    return check_cuda(launch_k(scale_kernel, dim3(grid), dim3(256), 0, st, x, n, s), "scale launch");
}
int32_t launch_scaled_add(float *y, const float *x, size_t n, float s, cudaStream_t st) {
    if (n == 0) return CERA_CUDA_OK;
    const unsigned grid = (unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    count_launch();
    return check_cuda(launch_k(scaled_add_kernel, dim3(grid), dim3(256), 0, st, y, x, n, s), "scaled add launch");
}

int32_t launch_argmax(const float *x, size_t n, uint32_t *out, uint32_t *scratch, cudaStream_t st) {
    if (!x || !out || !scratch) return fail(CERA_CUDA_ERR_BAD_ARG, "argmax: null argument");
    count_launch(2);
    CERA_CUDA_TRY(launch_k(argmax_stage1, dim3(ARGMAX_BLOCKS), dim3(ARGMAX_THREADS), 0, st, x, (uint32_t)n, scratch));
    return check_cuda(launch_k(argmax_stage2, dim3(1), dim3(32), 0, st, (const uint32_t *)scratch, (int)ARGMAX_BLOCKS, out),
                      "argmax launch");
}

int32_t launch_lora(const float *x, const float *a, const float *b, size_t rank, size_t k, size_t d, float scale, float *y,
                    cudaStream_t st) {
    if (rank == 0 || rank > LORA_MAX_RANK) return fail(CERA_CUDA_ERR_BAD_ARG, "lora: rank %zu outside 1..%d", rank, LORA_MAX_RANK);
    CERA_CUDA_TRY(launch_k(lora_kernel, dim3((unsigned)((d + 255) / 256)), dim3(256), 0, st, x, a, b, (uint32_t)rank, (uint32_t)k,
                           (uint32_t)d, scale, y));
    count_launch();
    return CERA_CUDA_OK;
}

int32_t launch_kv_shift(const void *k_src, const void *v_src, void *k_cache, void *v_cache, size_t n_keep, size_t shift,
                        size_t n_rows, size_t n_kv_heads, size_t head_dim, float theta_scale, const float *freq_factors,
                        int rope_type, int kv_f16, cudaStream_t st) {
    if (n_rows == 0) return CERA_CUDA_OK;
    const uint32_t pairs = (uint32_t)(n_kv_heads * head_dim / 2);
    const dim3 grid((pairs + 127) / 128, (unsigned)n_rows);
    kv_shift_kernel<<<grid, 128, 0, st>>>(k_src, v_src, k_cache, v_cache, (uint32_t)n_keep, (uint32_t)shift, (uint32_t)n_rows,
                                         (uint32_t)n_kv_heads, (uint32_t)head_dim, theta_scale, freq_factors, rope_type != 0 ? 1 : 0,
                                         kv_f16);
    count_launch();
    return check_cuda(cudaGetLastError(), "kv shift launch");
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_rope(float *q_dev, float *k_dev, size_t pos, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                       float freq_base, const float *freq_factors_dev, int32_t rope_type, void *stream) {
    const float ts = powf(freq_base, -2.0f / (float)head_dim);
    return launch_rope(q_dev, k_dev, nullptr, pos, nullptr, n_heads, n_kv_heads, head_dim, ts, freq_factors_dev,
                       rope_type, nullptr, nullptr, 0, (cudaStream_t)stream, nullptr);
}

}  // extern "C"
