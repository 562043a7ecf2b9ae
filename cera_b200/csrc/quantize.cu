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
        // 1/sqrt(mean + eps) in f64, narrowed once: the reciprocal square root and the multiplication by 1/n are each
        // within an f64 ulp of the reference's sqrt and divisions, far below the f32 rounding that follows
        if (lane == 0) inv_s = (float)rsqrt(t * inv_n + (double)eps);
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
