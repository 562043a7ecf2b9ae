// Device-side Q8_0 activation quantizer and the glue math it is fused with.
#pragma once

#include "common.cuh"

namespace cera {

// Q8_0-quantized activations as the kernels consume them (column j at j*k).
struct ActView {
    const float *scales;    // [n][k/32]
    const int8_t *quants;   // [n][k]
    const int16_t *sums;    // [n][k/16] sums of 16 consecutive quants
};

// ggml's polynomial expf, operation for operation (cera/src/backend/cpu.rs:2504-2544);
// every step individually rounded so the result is bit-identical to the CPU's.
__device__ __forceinline__ float ggml_expf(float x) {
    const float R = __uint_as_float(0x4B400000u), LOG2E = __uint_as_float(0x3FB8AA3Bu),
                LN2_HI = __uint_as_float(0x3F317200u), LN2_LO = __uint_as_float(0x35BFBE8Eu),
                C1 = __uint_as_float(0x3F7FFFF6u), C2 = __uint_as_float(0x3EFFFEDBu),
                C3 = __uint_as_float(0x3E2AAF33u), C4 = __uint_as_float(0x3D2B9F17u),
                C5 = __uint_as_float(0x3C072010u);
    const float z = __fadd_rn(R, __fmul_rn(x, LOG2E));
    const float n = __fsub_rn(z, R);
    const float b = __fsub_rn(__fsub_rn(x, __fmul_rn(n, LN2_HI)), __fmul_rn(n, LN2_LO));
    const uint32_t e = __float_as_uint(z) << 23;
    const float k = __uint_as_float(e + 0x3F800000u);
    const float u = __fmul_rn(b, b);
    const float p45 = __fadd_rn(C4, __fmul_rn(C5, b));
    const float p23 = __fadd_rn(__fadd_rn(C2, __fmul_rn(C3, b)), __fmul_rn(p45, u));
    const float j = __fadd_rn(__fmul_rn(C1, b), __fmul_rn(p23, u));
    const float abs_n = fabsf(n);
    if (abs_n <= 126.0f) return __fadd_rn(k, __fmul_rn(j, k));
    if (abs_n > 192.0f) return n > 0.0f ? __int_as_float(0x7F800000) : 0.0f;
    const uint32_t d = n <= 0.0f ? 0x82000000u : 0u;
    const float s1 = __uint_as_float(d + 0x7F000000u);
    const float s2 = __uint_as_float(e - d);
    return __fmul_rn(__fadd_rn(s2, __fmul_rn(s2, j)), s1);
}

// cera/src/backend/cpu.rs:2573: g / (1 + expf(-g)) * u
__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, ggml_expf(-g))), u);
}

// One warp quantizes one 32-element block: lane t holds v (cera/src/backend/cpu.rs:942-958).
// Returns the int8 quant of this lane; lane 0 of each 16-lane half gets the half sum in
// `half_sum`; `scale` is the f16-rounded block scale (same on every lane).
__device__ __forceinline__ int quantize_lane(float v, float &scale, int &half_sum) {
    float amax = fabsf(v);
    if (amax != amax) amax = 0.0f;  // f32::max ignores NaN
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float r = __fdiv_rn(1.0f, d);
    const float id = (d != 0.0f && isfinite(r)) ? r : 0.0f;
    scale = __half2float(__float2half_rn(d));
    float p = rintf(__fmul_rn(v, id));
    int q;
    if (p != p) q = 0;
    else q = (int)fminf(fmaxf(p, -128.0f), 127.0f);
    int s = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    half_sum = s;
    return q;
}

}  // namespace cera
