// Q8_0 activation quantizer kernels, alone and fused behind RMSNorm / SiLU*mul.
#include "act.cuh"
#include "ops.h"

namespace cera {

namespace {

// One warp per (column, block).  strided != 0: x is [k x n] with row stride n.
__global__ void quantize_kernel(const float *__restrict__ x, size_t k, size_t n, int strided, float *scales,
                                int8_t *quants, int16_t *sums) {
    pdl_trigger();
    pdl_wait();
    const size_t nb = k / 32;
    const size_t wid = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= nb * n) return;
    const size_t j = wid / nb, b = wid % nb;
    const size_t e = b * 32 + lane;
    const float v = strided ? x[e * n + j] : x[j * k + e];
    float scale;
    int hs;
    const int q = quantize_lane(v, scale, hs);
    quants[j * k + e] = (int8_t)q;
    if (lane == 0) scales[j * nb + b] = scale;
    if (sums && (lane & 15) == 0) sums[j * (k / 16) + b * 2 + (lane >> 4)] = (int16_t)hs;
}

// RMSNorm of one column per CTA (cera/src/backend/cpu.rs:2479-2496: f64 sum of
// squares, inv = (float)(1/sqrt(mean+eps)), x*inv*w left to right), then
// optionally the Q8_0 quantizer on the normed values.  Latency-bound and on the critical path of
// every projection: 32 warps, every thread's x and w values fetched once with all loads issued
// before the reduction, and at most four 32-element blocks quantized per warp one after another
// (up to 4096 elements; longer columns loop).
constexpr int RN_WARPS = 32, RN_THREADS = RN_WARPS * 32, RN_CH = 4;

__global__ void __launch_bounds__(RN_THREADS) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ weight,
                                                              size_t n_elem, double inv_n, float eps, float *out_f32,
                                                              float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    __shared__ double red[RN_WARPS];
    __shared__ float inv_s;
    pdl_trigger();
    const size_t col = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nblk = (uint32_t)((n_elem + 31) >> 5);
    const bool single = nblk <= RN_WARPS * RN_CH;  // up to 4096 elements stay in registers
    // lane `lane` of warp `warp` owns element `lane` of 32-blocks warp, warp+32, ...
    float wv[RN_CH], xv[RN_CH];
    if (single) {
#pragma unroll
        for (int j = 0; j < RN_CH; ++j) {
            const size_t i = (size_t)(warp + RN_WARPS * j) * 32 + lane;
            wv[j] = i < n_elem ? weight[i] : 0.0f;  // weights do not depend on the previous kernel
        }
    }
    pdl_wait();
    tp_arrive_wait(tp.ctx, tp.wait_slot);
    const float *xc = x + col * n_elem;
    double ss = 0.0;
    for (uint32_t c0 = 0; c0 < nblk; c0 += RN_WARPS * RN_CH) {
#pragma unroll
        for (int j = 0; j < RN_CH; ++j) {
            const size_t i = (size_t)(c0 + warp + RN_WARPS * j) * 32 + lane;
            xv[j] = i < n_elem ? xc[i] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < RN_CH; ++j) ss += (double)xv[j] * (double)xv[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        double t = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) inv_s = (float)(1.0 / sqrt(t / (double)n_elem + (double)eps));  // the reference's f64 expression, IEEE division and square root
    }
    __syncthreads();
    const float inv = inv_s;
    for (uint32_t c0 = 0; c0 < nblk; c0 += RN_WARPS * RN_CH) {
#pragma unroll
        for (int j = 0; j < RN_CH; ++j) {
            const uint32_t b = c0 + warp + RN_WARPS * j;
            if (b >= nblk) continue;  // warp-uniform
            const size_t i = (size_t)b * 32 + lane;
            const bool in = i < n_elem;  // only the f32-only path may see a ragged last block
            const float xi = single ? xv[j] : (in ? xc[i] : 0.0f);
            const float wi = single ? wv[j] : (in ? weight[i] : 0.0f);
            const float v = __fmul_rn(__fmul_rn(xi, inv), wi);
            if (out_f32 && in) out_f32[col * n_elem + i] = v;
            if (quants) {
                float scale;
                int hs;
                const int q = quantize_lane(v, scale, hs);
                quants[col * n_elem + i] = (int8_t)q;
                if (lane == 0) scales[col * (n_elem / 32) + b] = scale;
                if ((lane & 15) == 0) sums[col * (n_elem / 16) + 2 * b + (lane >> 4)] = (int16_t)hs;
            }
        }
    }
}

// The same operation for columns whose length is a multiple of 32, laid out for latency: every thread owns FOUR
// consecutive elements (one 128-bit load of x and of the weights), so a 32-element Q8_0 block is eight neighbouring
// lanes: its amax takes three shuffle steps, its two 16-element sums two, and all blocks of the column are quantized
// at the same time instead of four per warp one after another.  Up to 4096 elements stay in registers between the
// sum of squares and the scaling; longer columns re-read x.
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_q8_kernel(const float *__restrict__ x, const float *__restrict__ weight,
                                                                 size_t n_elem, double inv_n, float eps, float *out_f32,
                                                                 float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    __shared__ double red[RN_WARPS];
    __shared__ float inv_s;
    pdl_trigger();
    const size_t col = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nvec = (uint32_t)(n_elem >> 2);
    const bool single = nvec <= RN_THREADS;
    float4 wv = make_float4(0.f, 0.f, 0.f, 0.f), xv = wv;
    if (single && threadIdx.x < nvec) wv = reinterpret_cast<const float4 *>(weight)[threadIdx.x];  // independent of the previous kernel
    pdl_wait();
    tp_arrive_wait(tp.ctx, tp.wait_slot);
    const float4 *xc = reinterpret_cast<const float4 *>(x + col * n_elem);
    double ss = 0.0;
    for (uint32_t v = threadIdx.x; v < nvec; v += RN_THREADS) {
        xv = xc[v];
        ss += (double)xv.x * (double)xv.x;
        ss += (double)xv.y * (double)xv.y;
        ss += (double)xv.z * (double)xv.z;
        ss += (double)xv.w * (double)xv.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        double t = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) inv_s = (float)(1.0 / sqrt(t / (double)n_elem + (double)eps));  // the reference's f64 expression, IEEE division and square root
    }
    __syncthreads();
    const float inv = inv_s;
    // whole warps iterate together: nvec is a multiple of 8, so a block's eight lanes are all in or all out
    for (uint32_t v0 = 0; v0 < nvec; v0 += RN_THREADS) {
        const uint32_t v = v0 + threadIdx.x;
        const bool in = v < nvec;
        if (!single) {
            xv = in ? xc[v] : make_float4(0.f, 0.f, 0.f, 0.f);
            wv = in ? reinterpret_cast<const float4 *>(weight)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float e[4] = {__fmul_rn(__fmul_rn(xv.x, inv), wv.x), __fmul_rn(__fmul_rn(xv.y, inv), wv.y),
                      __fmul_rn(__fmul_rn(xv.z, inv), wv.z), __fmul_rn(__fmul_rn(xv.w, inv), wv.w)};
        if (out_f32 && in) reinterpret_cast<float4 *>(out_f32 + col * n_elem)[v] = make_float4(e[0], e[1], e[2], e[3]);
        // Q8_0 of the block these eight lanes share (cera/src/backend/cpu.rs:942-958)
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = fabsf(e[i]);
            amax = fmaxf(amax, a == a ? a : 0.0f);  // f32::max ignores NaN
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 127.0f);
        const float r = __fdiv_rn(1.0f, d);
        const float id = (d != 0.0f && isfinite(r)) ? r : 0.0f;
        int q[4], s4 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float pq = rintf(__fmul_rn(e[i], id));
            q[i] = pq != pq ? 0 : (int)fminf(fmaxf(pq, -128.0f), 127.0f);
            s4 += q[i];
        }
        s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 2);  // sum of the 16 elements of lanes 4j .. 4j+3
        if (in) {
            const uint32_t packed = (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) | ((uint32_t)(uint8_t)q[2] << 16) |
                                    ((uint32_t)(uint8_t)q[3] << 24);
            reinterpret_cast<uint32_t *>(quants + col * n_elem)[v] = packed;
            if ((lane & 7) == 0) scales[col * (n_elem / 32) + (v >> 3)] = __half2float(__float2half_rn(d));
            if ((lane & 3) == 0) sums[col * (n_elem / 16) + (v >> 2)] = (int16_t)s4;
        }
    }
}

__global__ void silu_mul_kernel(float *gate, const float *__restrict__ up, size_t n_elem, size_t n_cols,
                                float *scales, int8_t *quants, int16_t *sums, const TpHook tp) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elem * n_cols) return;
    const float v = silu_mul(gate[i], up[i]);
    gate[i] = v;
    if (quants) {
        float scale;
        int hs;
        const int q = quantize_lane(v, scale, hs);
        const int lane = threadIdx.x & 31;
        quants[i] = (int8_t)q;
        if (lane == 0) scales[i / 32] = scale;
        if ((lane & 15) == 0) sums[i / 16] = (int16_t)hs;
        if (tp.push) {
            tp_push(tp.ctx, quants + i, (int8_t)q);
            if (lane == 0) tp_push(tp.ctx, scales + i / 32, scale);
            if ((lane & 15) == 0) tp_push(tp.ctx, sums + i / 16, (int16_t)hs);
        }
    }
}

// SiLU*mul with the Q8_0 quantizer, four consecutive elements per thread (one 128-bit load of gate and of up): a
// 32-element block is eight neighbouring lanes, so its amax takes three shuffle steps and its 16-element sums two.
__global__ void __launch_bounds__(256) silu_mul_q8_kernel(float *gate, const float *__restrict__ up, size_t n_vec, float *scales,
                                                          int8_t *quants, int16_t *sums, const TpHook tp) {
    pdl_trigger();
    pdl_wait();
    const size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool in = v < n_vec;  // n_vec is a multiple of 8: a block's eight lanes are all in or all out
    const int lane = threadIdx.x & 31;
    float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f), u4 = g4;
    if (in) {
        g4 = reinterpret_cast<const float4 *>(gate)[v];
        u4 = reinterpret_cast<const float4 *>(up)[v];
    }
    const float e[4] = {silu_mul(g4.x, u4.x), silu_mul(g4.y, u4.y), silu_mul(g4.z, u4.z), silu_mul(g4.w, u4.w)};
    if (in) reinterpret_cast<float4 *>(gate)[v] = make_float4(e[0], e[1], e[2], e[3]);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = fabsf(e[i]);
        amax = fmaxf(amax, a == a ? a : 0.0f);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float r = __fdiv_rn(1.0f, d);
    const float id = (d != 0.0f && isfinite(r)) ? r : 0.0f;
    int q[4], s4 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float pq = rintf(__fmul_rn(e[i], id));
        q[i] = pq != pq ? 0 : (int)fminf(fmaxf(pq, -128.0f), 127.0f);
        s4 += q[i];
    }
    s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
    s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
    if (!in) return;
    const uint32_t packed = (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) | ((uint32_t)(uint8_t)q[2] << 16) |
                            ((uint32_t)(uint8_t)q[3] << 24);
    const float scale = __half2float(__float2half_rn(d));
    reinterpret_cast<uint32_t *>(quants)[v] = packed;
    if ((lane & 7) == 0) scales[v >> 3] = scale;
    if ((lane & 3) == 0) sums[v >> 2] = (int16_t)s4;
    if (tp.push) {
        tp_push(tp.ctx, reinterpret_cast<uint32_t *>(quants) + v, packed);
        if ((lane & 7) == 0) tp_push(tp.ctx, scales + (v >> 3), scale);
        if ((lane & 3) == 0) tp_push(tp.ctx, sums + (v >> 2), (int16_t)s4);
    }
}

}  // namespace

int32_t launch_quantize(const float *x, size_t k, size_t n, bool strided, float *scales, int8_t *quants,
                        int16_t *sums, cudaStream_t st) {
    if (!x || !scales || !quants) return fail(CERA_CUDA_ERR_BAD_ARG, "quantize_q8_0: null argument");
    if (k == 0 || k % 32) return fail(CERA_CUDA_ERR_BAD_ARG, "quantize_q8_0: k=%zu must be a positive multiple of 32", k);
    if (n == 0) return CERA_CUDA_OK;
    const size_t warps = (k / 32) * n;
    const int threads = 256;
    const size_t grid = (warps * 32 + threads - 1) / threads;
    CERA_CUDA_TRY(launch_k(quantize_kernel, dim3((unsigned)grid), dim3(threads), 0, st, x, k, n, strided ? 1 : 0, scales, quants, sums));
    count_launch();
    return check_cuda(cudaGetLastError(), "quantize launch");
}

int32_t launch_rmsnorm(const float *x, const float *weight, size_t n_elem, size_t n_cols, float eps, float *out_f32,
                       float *scales, int8_t *quants, int16_t *sums, cudaStream_t st, const TpHook *tp) {
    if (!x || !weight) return fail(CERA_CUDA_ERR_BAD_ARG, "rmsnorm: null argument");
    if (quants && (n_elem % 32 || !scales || !sums))
        return fail(CERA_CUDA_ERR_BAD_ARG, "rmsnorm+quantize: n=%zu must be a multiple of 32", n_elem);
    if (n_elem == 0 || n_cols == 0) return CERA_CUDA_OK;
    const int threads = RN_THREADS;
    if (quants && ((uintptr_t)x % 16 == 0) && ((uintptr_t)weight % 16 == 0) && (!out_f32 || (uintptr_t)out_f32 % 16 == 0) &&
        (uintptr_t)quants % 4 == 0) {
        CERA_CUDA_TRY(launch_k(rmsnorm_q8_kernel, dim3((unsigned)n_cols), dim3(threads), 0, st, x, weight, n_elem, 1.0 / (double)n_elem, eps,
                               out_f32, scales, quants, sums, tp ? *tp : TpHook{}));
        count_launch();
        return check_cuda(cudaGetLastError(), "rmsnorm launch");
    }
    CERA_CUDA_TRY(launch_k(rmsnorm_kernel, dim3((unsigned)n_cols), dim3(threads), 0, st, x, weight, n_elem, 1.0 / (double)n_elem, eps, out_f32, scales,
                           quants, sums, tp ? *tp : TpHook{}));
    count_launch();
    return check_cuda(cudaGetLastError(), "rmsnorm launch");
}

int32_t launch_silu_mul(float *gate, const float *up, size_t n_elem, size_t n_cols, float *scales, int8_t *quants,
                        int16_t *sums, cudaStream_t st, const TpHook *tp) {
    if (!gate || !up) return fail(CERA_CUDA_ERR_BAD_ARG, "silu_mul: null argument");
    if (quants && n_elem % 32) return fail(CERA_CUDA_ERR_BAD_ARG, "silu_mul+quantize: n=%zu must be a multiple of 32", n_elem);
    const size_t total = n_elem * n_cols;
    if (total == 0) return CERA_CUDA_OK;
    const int threads = 256;
    if (quants && (uintptr_t)gate % 16 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)quants % 4 == 0) {
        const size_t n_vec = total / 4;
        CERA_CUDA_TRY(launch_k(silu_mul_q8_kernel, dim3((unsigned)((n_vec + threads - 1) / threads)), dim3(threads), 0, st, gate, up, n_vec,
                               scales, quants, sums, tp ? *tp : TpHook{}));
        count_launch();
        return check_cuda(cudaGetLastError(), "silu_mul launch");
    }
    CERA_CUDA_TRY(launch_k(silu_mul_kernel, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, st, gate, up,
                           n_elem, n_cols, scales, quants, sums, tp ? *tp : TpHook{}));
    count_launch();
    return check_cuda(cudaGetLastError(), "silu_mul launch");
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_quantize_q8_0(const float *x_dev, size_t k, size_t n, float *scales_dev, int8_t *quants_dev,
                                int16_t *sums_dev, void *stream) {
    return launch_quantize(x_dev, k, n, false, scales_dev, quants_dev, sums_dev, (cudaStream_t)stream);
}

int32_t cera_cuda_quantize_columns(const float *mat_dev, size_t dim, size_t n, float *scales_dev, int8_t *quants_dev,
                                   int16_t *sums_dev, void *stream) {
    return launch_quantize(mat_dev, dim, n, true, scales_dev, quants_dev, sums_dev, (cudaStream_t)stream);
}

int32_t cera_cuda_rmsnorm(const float *x_dev, const float *weight_dev, size_t n, float eps, float *out_dev,
                          void *stream) {
    if (!out_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "rmsnorm: null output");
    return launch_rmsnorm(x_dev, weight_dev, n, 1, eps, out_dev, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

int32_t cera_cuda_rmsnorm_q8_0(const float *x_dev, const float *weight_dev, size_t n, float eps, float *out_dev,
                               float *scales_dev, int8_t *quants_dev, int16_t *sums_dev, void *stream) {
    if (!scales_dev || !quants_dev || !sums_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "rmsnorm_q8_0: null output");
    return launch_rmsnorm(x_dev, weight_dev, n, 1, eps, out_dev, scales_dev, quants_dev, sums_dev, (cudaStream_t)stream);
}

int32_t cera_cuda_silu_mul(float *gate_dev, const float *up_dev, size_t n, void *stream) {
    return launch_silu_mul(gate_dev, up_dev, n, 1, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

}  // extern "C"
