// Synthetic tensors and f32 -> GGML block quantizers on the device.
//
// Built with -fmad=false: every expression below is evaluated with one IEEE
// rounding per operation, in the order written, so the bytes are identical to
// the CPU restatement of the same rules (cera/src/convert/quantize.rs:344-387
// Q8_0, 523-570 Q4_0, 719-846 Q4_K, 851-988 Q5_K, 993-1094 Q6_K; Q4_1 follows
// ggml's published quantize_row_q4_1_ref, the reference has no Q4_1 quantizer).
#include "common.cuh"

namespace cera {

namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Irwin-Hall(12) over 16-bit uniforms: mean 393210, standard deviation ~65536.
__global__ void synth_kernel(float *out, size_t n, uint64_t seed, uint64_t offset, float sigma) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t key = splitmix64(seed), c = (offset + i) * 3ull;
    int sum = 0;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
        const uint64_t h = splitmix64(key ^ (c + (uint64_t)r));
        sum += (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)((h >> 48) & 0xFFFF);
    }
    out[i] = (float)(sum - 393210) * (sigma * (1.0f / 65536.0f));
}

__device__ __forceinline__ uint16_t f2h(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float h2fl(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ float sclamp(float v, float lo, float hi) {
    if (v != v || v < lo) return lo;
    if (v > hi) return hi;
    return v;
}
// Every block size and every f16 field offset is even, so the field is 2-byte aligned.
__device__ __forceinline__ void put16(uint8_t *p, uint16_t v) { *reinterpret_cast<uint16_t *>(p) = v; }

__device__ void wq_q8_0(const float *in, uint8_t *out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = fabsf(in[i]) > amax ? fabsf(in[i]) : amax;
    const uint16_t dh = f2h(amax / 127.0f);
    put16(out, dh);
    const float d = h2fl(dh);
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 32; ++i) out[2 + i] = (uint8_t)(int8_t)sclamp(roundf(in[i] * id), -127.0f, 127.0f);
}

__device__ void wq_q4_0(const float *in, uint8_t *out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = fabsf(in[i]) > amax ? fabsf(in[i]) : amax;
    const uint16_t dh = f2h(amax / 8.0f);
    put16(out, dh);
    const float d = h2fl(dh);
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 16; ++i) {
        const uint8_t q0 = (uint8_t)sclamp(floorf(in[i] * id + 8.5f), 0.0f, 15.0f);
        const uint8_t q1 = (uint8_t)sclamp(floorf(in[i + 16] * id + 8.5f), 0.0f, 15.0f);
        out[2 + i] = (uint8_t)(q0 | (q1 << 4));
    }
}

__device__ void wq_q4_1(const float *in, uint8_t *out) {
    float mn = in[0], mx = in[0];
    for (int i = 1; i < 32; ++i) {
        mn = in[i] < mn ? in[i] : mn;
        mx = in[i] > mx ? in[i] : mx;
    }
    const float d = (mx - mn) / 15.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    put16(out, f2h(d));
    put16(out + 2, f2h(mn));
    for (int i = 0; i < 16; ++i) {
        const uint8_t q0 = (uint8_t)sclamp(floorf((in[i] - mn) * id + 0.5f), 0.0f, 15.0f);
        const uint8_t q1 = (uint8_t)sclamp(floorf((in[i + 16] - mn) * id + 0.5f), 0.0f, 15.0f);
        out[4 + i] = (uint8_t)(q0 | (q1 << 4));
    }
}

__device__ void kq_header(const float *in, float qmax, uint8_t *out, float &ad, float &admin, uint8_t qsc[8],
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
        const float eff = fminf(smin[s], 0.0f);
        const float range = smax[s] - eff;
        if (range > max_range) max_range = range;
        if (-eff > max_min_abs) max_min_abs = -eff;
    }
    const uint16_t dh = f2h((max_range / 63.0f) / qmax), mh = f2h(max_min_abs / 63.0f);
    put16(out, dh);
    put16(out + 2, mh);
    ad = h2fl(dh);
    admin = h2fl(mh);
    for (int s = 0; s < 8; ++s) {
        const float eff = fminf(smin[s], 0.0f);
        const float range = smax[s] - eff;
        qsc[s] = ad > 0.0f ? (uint8_t)sclamp(roundf((range / qmax) / ad), 0.0f, 63.0f) : 0;
        qmn[s] = admin > 0.0f ? (uint8_t)sclamp(roundf((-eff) / admin), 0.0f, 63.0f) : 0;
    }
    for (int j = 0; j < 4; ++j) {
        out[4 + j] = (uint8_t)((qsc[j] & 0x3F) | (((qsc[j + 4] & 0x30) >> 4) << 6));
        out[8 + j] = (uint8_t)((qmn[j] & 0x3F) | (((qmn[j + 4] & 0x30) >> 4) << 6));
        out[12 + j] = (uint8_t)((qsc[j + 4] & 0x0F) | ((qmn[j + 4] & 0x0F) << 4));
    }
}

__device__ void wq_q4_k(const float *in, uint8_t *out) {
    float ad, admin;
    uint8_t qsc[8], qmn[8];
    kq_header(in, 15.0f, out, ad, admin, qsc, qmn);
    for (int j = 0; j < 4; ++j) {
        const float sc0 = (float)qsc[2 * j] * ad, sc1 = (float)qsc[2 * j + 1] * ad;
        const float m0 = (float)qmn[2 * j] * admin, m1 = (float)qmn[2 * j + 1] * admin;
        for (int l = 0; l < 32; ++l) {
            const uint8_t q0 = sc0 > 0.0f ? (uint8_t)sclamp(roundf((in[64 * j + l] + m0) / sc0), 0.0f, 15.0f) : 0;
            const uint8_t q1 = sc1 > 0.0f ? (uint8_t)sclamp(roundf((in[64 * j + 32 + l] + m1) / sc1), 0.0f, 15.0f) : 0;
            out[16 + 32 * j + l] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

__device__ void wq_q5_k(const float *in, uint8_t *out) {
    float ad, admin;
    uint8_t qsc[8], qmn[8];
    kq_header(in, 31.0f, out, ad, admin, qsc, qmn);
    uint8_t *qh = out + 16, *qs = out + 48;
    for (int l = 0; l < 32; ++l) qh[l] = 0;
    for (int j = 0; j < 4; ++j) {
        const float sc0 = (float)qsc[2 * j] * ad, sc1 = (float)qsc[2 * j + 1] * ad;
        const float m0 = (float)qmn[2 * j] * admin, m1 = (float)qmn[2 * j + 1] * admin;
        for (int l = 0; l < 32; ++l) {
            const uint8_t q0 = sc0 > 0.0f ? (uint8_t)sclamp(roundf((in[64 * j + l] + m0) / sc0), 0.0f, 31.0f) : 0;
            const uint8_t q1 = sc1 > 0.0f ? (uint8_t)sclamp(roundf((in[64 * j + 32 + l] + m1) / sc1), 0.0f, 31.0f) : 0;
            qs[32 * j + l] = (uint8_t)((q0 & 15) | ((q1 & 15) << 4));
            qh[l] |= (uint8_t)((((q0 >> 4) & 1) << (2 * j)) | (((q1 >> 4) & 1) << (2 * j + 1)));
        }
    }
}

__device__ void wq_q6_k(const float *in, uint8_t *out) {
    float smax[16];
    float max_all = 0.0f;
    for (int s = 0; s < 16; ++s) {
        float amax = 0.0f;
        for (int l = 0; l < 16; ++l) {
            const float a = fabsf(in[16 * s + l]);
            if (a > amax) amax = a;
        }
        smax[s] = amax;
        if (amax > max_all) max_all = amax;
    }
    const uint16_t dh = f2h(max_all / (128.0f * 32.0f));
    put16(out + 208, dh);
    const float ad = h2fl(dh);
    const float id = ad != 0.0f ? 1.0f / ad : 0.0f;
    int8_t qsc[16];
    for (int s = 0; s < 16; ++s) {
        qsc[s] = (int8_t)sclamp(roundf(smax[s] * id / 32.0f), -128.0f, 127.0f);
        out[192 + s] = (uint8_t)qsc[s];
    }
    for (int nh = 0; nh < 2; ++nh) {
        uint8_t *ql = out + 64 * nh, *qh = out + 128 + 32 * nh;
        for (int l = 0; l < 32; ++l) {
            uint8_t q[4];
            for (int g = 0; g < 4; ++g) {
                const float sc = (float)qsc[8 * nh + l / 16 + 2 * g] * ad;
                const float isc = sc != 0.0f ? 1.0f / sc : 0.0f;
                q[g] = (uint8_t)sclamp(floorf(in[128 * nh + 32 * g + l] * isc + 32.5f), 0.0f, 63.0f);
            }
            ql[l] = (uint8_t)((q[0] & 15) | ((q[2] & 15) << 4));
            ql[l + 32] = (uint8_t)((q[1] & 15) | ((q[3] & 15) << 4));
            qh[l] = (uint8_t)(((q[0] >> 4) & 3) | (((q[1] >> 4) & 3) << 2) | (((q[2] >> 4) & 3) << 4) |
                              (((q[3] >> 4) & 3) << 6));
        }
    }
}

__global__ void quantize_weights_kernel(int type, const float *__restrict__ in, size_t n_blocks, uint8_t *out) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const TypeInfo ti = type_info(type);
    const float *i = in + b * ti.elems;
    uint8_t *o = out + b * ti.bytes;
    switch (type) {
        case CERA_TYPE_Q8_0: wq_q8_0(i, o); break;
        case CERA_TYPE_Q4_0: wq_q4_0(i, o); break;
        case CERA_TYPE_Q4_1: wq_q4_1(i, o); break;
        case CERA_TYPE_Q4_K: wq_q4_k(i, o); break;
        case CERA_TYPE_Q5_K: wq_q5_k(i, o); break;
        case CERA_TYPE_Q6_K: wq_q6_k(i, o); break;
    }
}

}  // namespace
}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_synth_normal(float *out_dev, size_t n, uint64_t seed, uint64_t offset, float sigma, void *stream) {
    if (!out_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "synth_normal: null output");
    if (n == 0) return CERA_CUDA_OK;
    const int threads = 256;
    synth_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, (cudaStream_t)stream>>>(out_dev, n, seed, offset,
                                                                                               sigma);
    count_launch();
    return check_cuda(cudaGetLastError(), "synth launch");
}

int32_t cera_cuda_quantize_weights(int32_t type, const float *in_dev, size_t n, void *out_dev, void *stream) {
    if (!in_dev || !out_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "quantize_weights: null argument");
    if (!is_block_type(type)) return fail(CERA_CUDA_ERR_UNSUPPORTED, "quantize_weights: ggml type %d", type);
    const TypeInfo ti = type_info(type);
    if (n % ti.elems) return fail(CERA_CUDA_ERR_BAD_ARG, "quantize_weights: n=%zu is not a multiple of %d", n, ti.elems);
    const size_t n_blocks = n / ti.elems;
    if (n_blocks == 0) return CERA_CUDA_OK;
    const int threads = 64;
    quantize_weights_kernel<<<(unsigned)((n_blocks + threads - 1) / threads), threads, 0, (cudaStream_t)stream>>>(
        type, in_dev, n_blocks, (uint8_t *)out_dev);
    count_launch();
    return check_cuda(cudaGetLastError(), "quantize_weights launch");
}

}  // extern "C"
