// One 32-weight item against NC contiguous Q8_0 activation columns: the inner step shared by the
// item-wise GEMV / small-batch GEMM and the expert-grouped GEMM.
#pragma once

#include "act.cuh"
#include "formats.cuh"

namespace cera {

template <int T, int NC>
__device__ __forceinline__ void accumulate_item(const typename Fmt<T>::Raw &raw, int item, const ActView &x, uint32_t k,
                                                float (&acc)[NC]) {
    using F = Fmt<T>;
    int lo[4], hi[4];
    HalfRef h0, h1;
    F::decode(raw, item, lo, hi, h0, h1);
    const uint32_t nb32 = k >> 5, nb16 = k >> 4;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const int8_t *q = x.quants + (size_t)c * k;
        const int u0 = dot16(lo, q + h0.off), u1 = dot16(hi, q + h1.off);
        if (F::WHOLE_BLOCK) {
            const float xs = __ldg(x.scales + (size_t)c * nb32 + (h0.off >> 5));
            int a0 = 0, a1 = 0;
            if (T != CERA_TYPE_Q8_0) {
                const int s2 = __ldg(reinterpret_cast<const int *>(x.sums + (size_t)c * nb16 + (h0.off >> 4)));
                a0 = (int)(int16_t)(s2 & 0xFFFF);
                a1 = s2 >> 16;
            }
            const int U = F::view(u0, a0) + F::view(u1, a1);
            acc[c] = fmaf((float)U, __fmul_rn(h0.scale, xs), acc[c]);
            if (F::SIGN != 0) acc[c] = fmaf(__fmul_rn(xs, h0.mscale), (float)(F::SIGN * (a0 + a1)), acc[c]);
        } else {
            const float xs0 = __ldg(x.scales + (size_t)c * nb32 + (h0.off >> 5));
            const float xs1 = __ldg(x.scales + (size_t)c * nb32 + (h1.off >> 5));
            const int a0 = __ldg(x.sums + (size_t)c * nb16 + (h0.off >> 4));
            const int a1 = __ldg(x.sums + (size_t)c * nb16 + (h1.off >> 4));
            acc[c] = fmaf((float)u0, __fmul_rn(h0.scale, xs0), acc[c]);
            acc[c] = fmaf((float)u1, __fmul_rn(h1.scale, xs1), acc[c]);
            acc[c] = fmaf(__fmul_rn(xs0, h0.mscale), (float)(F::SIGN * a0), acc[c]);
            acc[c] = fmaf(__fmul_rn(xs1, h1.mscale), (float)(F::SIGN * a1), acc[c]);
        }
    }
}

}  // namespace cera
