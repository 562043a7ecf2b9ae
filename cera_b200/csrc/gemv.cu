// Decode GEMV / small-batch GEMM: quantized weights x Q8_0 activations.
//
// HBM-bound.  One warp owns one weight row at a time (grid-stride over rows);
// each lane streams 16-byte items of the low-quant plane with L1-bypassing
// 128-bit loads, unpacks nibbles / high bits in registers, forms exact int32
// half-block sums with dp4a against the Q8_0 activation quants (read through
// L1, they are shared by every row), scales them in f32 and the warp reduces
// with shuffles.  NC activation columns reuse the unpacked weights.
//
// Arithmetic contract: cera/src/backend/simd.rs:4593-4637 (Q4_0/Q8_0),
// 5693-5878 (Q4_K), 5893-5976 (Q4_1), 5988-6195 (Q6_K).  Integer sums are
// exact; the f32 combination order is this kernel's own (per-lane sequential
// fma over the lane's items, then an xor-shuffle tree), within the path's f32
// tolerance of any of the reference's three orders.
#include <cstdlib>
#include <cstring>

#include "formats.cuh"
#include "gemv_item.cuh"
#include "ops.h"
#include "weight.h"

namespace cera {

namespace {

constexpr int MAX_SEGS = 3;
constexpr int WARPS = 8;

struct GemvParams {
    WeightView w[MAX_SEGS];
    float *y[MAX_SEGS];
    uint32_t row_end[MAX_SEGS];  // cumulative row counts
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k;
    uint32_t ldy;  // row stride of y in floats
    uint32_t ldc;  // column stride of y in floats
    int epilogue;
    TpHook tp;
};

template <int T, int NC, int UNROLL>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(const GemvParams p) {
    using F = Fmt<T>;
    pdl_trigger();
    pdl_wait();
    tp_arrive_wait(p.tp.ctx, p.tp.wait_slot);
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * WARPS + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * WARPS;
    const int items = p.k >> 5;

    for (uint32_t row = warp; row < p.total_rows; row += n_warps) {
        int s = 0;
        while (s + 1 < p.n_segs && row >= p.row_end[s]) ++s;
        const uint32_t local = row - (s ? p.row_end[s - 1] : 0);
        const WeightView &w = p.w[s];

        float acc[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] = 0.0f;

        for (int base = 0; base < items; base += 32 * UNROLL) {
            typename F::Raw raw[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int item = base + u * 32 + lane;
                if (item < items) raw[u] = F::load(w, local, item);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int item = base + u * 32 + lane;
                if (item < items) accumulate_item<T, NC>(raw[u], item, p.x, p.k, acc);
            }
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] = warp_sum(acc[c]);
        if (lane == 0) {
            float *y = p.y[s] + (size_t)local * p.ldy;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float *yc = y + (size_t)c * p.ldc;
                const float r = p.epilogue == EPI_ADD ? __fadd_rn(*yc, acc[c]) : acc[c];
                *yc = r;
                if (p.tp.push) tp_push(p.tp.ctx, yc, r);
            }
        }
    }
}

// Q5_K against f32 activations (cera/src/quant.rs:892-937, cpu.rs:1830-1854):
// per 64-element pair d*(sc1*S1 + sc2*S2) - dmin*(mn1*Y1 + mn2*Y2).  One warp per row;
// each lane owns whole items so the element sums inside an item stay sequential.
__global__ void __launch_bounds__(WARPS * 32) gemv_q5k_f32_kernel(const WeightView w, const float *__restrict__ x,
                                                                float *__restrict__ y) {
    using F = Fmt<CERA_TYPE_Q5_K>;
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * WARPS + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * WARPS;
    const int items = w.k >> 5;
    for (uint32_t row = warp; row < w.m; row += n_warps) {
        float acc = 0.0f;
        for (int item = lane; item < items; item += 32) {
            const F::Raw raw = F::load(w, row, item);
            int lo[4], hi[4];
            HalfRef h0, h1;
            F::decode(raw, item, lo, hi, h0, h1);
            float s0 = 0.0f, s1 = 0.0f, y0 = 0.0f, y1 = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float xa = __ldg(x + h0.off + 4 * i + t), xb = __ldg(x + h1.off + 4 * i + t);
                    s0 = fmaf((float)((lo[i] >> (8 * t)) & 0xFF), xa, s0);
                    s1 = fmaf((float)((hi[i] >> (8 * t)) & 0xFF), xb, s1);
                    y0 += xa;
                    y1 += xb;
                }
            acc += h0.scale * s0 + h1.scale * s1 - (h0.mscale * y0 + h1.mscale * y1);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}

template <int T, int NC>
int32_t launch_typed(const GemvParams &p, cudaStream_t st) {
    const uint32_t ctas_needed = (p.total_rows + WARPS - 1) / WARPS;
    const uint32_t cap = (uint32_t)sm_count() * 8;
    const uint32_t grid = ctas_needed < cap ? ctas_needed : cap;
    count_launch();
    if (p.k >= 4096) return check_cuda(launch_k(gemv_kernel<T, NC, 4>, dim3(grid), dim3(WARPS * 32), 0, st, p), "gemv launch");
    return check_cuda(launch_k(gemv_kernel<T, NC, 1>, dim3(grid), dim3(WARPS * 32), 0, st, p), "gemv launch");
}

template <int T>
int32_t launch_cols(const GemvParams &p, size_t n_cols, cudaStream_t st) {
    switch (n_cols) {
        case 1: return launch_typed<T, 1>(p, st);
        case 2: return launch_typed<T, 2>(p, st);
        case 4: return launch_typed<T, 4>(p, st);
        case 8: return launch_typed<T, 8>(p, st);
        default: return fail(CERA_CUDA_ERR_BAD_ARG, "gemv: column tile %zu not instantiated", n_cols);
    }
}

}  // namespace

// CERA_CUDA_GEMV=direct keeps every GEMV on the item-wise kernel (A/B runs); read once.
static bool force_direct() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_GEMV");
        return e && strcmp(e, "direct") == 0;
    }();
    return v;
}

int32_t launch_gemv_fused(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp) {
    const bool hooked = tp && (tp->push || tp->wait_slot != TP_NO_SLOT);  // the TMA-staged variant carries no exchange hooks
    if (!hooked) {
        CERA_TRY(launch_gemv_tma(segs, n_segs, x, epilogue, fusion, st, taken));
        if (*taken) return CERA_CUDA_OK;
    }
    return launch_gemv_rows(segs, n_segs, x, epilogue, fusion, st, taken, tp);
}

// All segments must share the type and k.  n_cols in {1,2,4,8}.
int32_t launch_gemv(const GemvSeg *segs, int n_segs, const ActView &x, size_t n_cols, size_t ldy, int epilogue,
                    cudaStream_t st, size_t ldc, bool batch_tile, const TpHook *tp) {
    if (n_segs < 1 || n_segs > MAX_SEGS) return fail(CERA_CUDA_ERR_BAD_ARG, "gemv: %d segments", n_segs);
    if (n_cols == 1 && ldy == 1 && !batch_tile && !force_direct()) {
        bool taken = false;
        // K-quants: the kernel whose f32 order is the reference's (bit-identical results), else the streaming kernels
        CERA_TRY(launch_gemv_exact(segs, n_segs, x, epilogue, nullptr, st, &taken, tp));
        if (taken) return CERA_CUDA_OK;
        CERA_TRY(launch_gemv_fused(segs, n_segs, x, epilogue, nullptr, st, &taken, tp));
        if (taken) return CERA_CUDA_OK;
    }
    GemvParams p{};
    uint32_t rows = 0;
    for (int i = 0; i < n_segs; ++i) {
        if (segs[i].w.type != segs[0].w.type || segs[i].w.k != segs[0].w.k)
            return fail(CERA_CUDA_ERR_BAD_ARG, "gemv: fused segments must share type and k");
        p.w[i] = segs[i].w;
        p.y[i] = segs[i].y;
        rows += segs[i].w.m;
        p.row_end[i] = rows;
    }
    p.n_segs = n_segs;
    p.total_rows = rows;
    p.x = x;
    p.k = segs[0].w.k;
    p.epilogue = epilogue;
    p.ldy = (uint32_t)ldy;
    p.ldc = (uint32_t)ldc;
    if (tp) p.tp = *tp;
    if ((uintptr_t)x.quants % 16 || (uintptr_t)x.sums % 4 || (p.k % 32))
        return fail(CERA_CUDA_ERR_BAD_ARG, "gemv: activation quants must be 16-byte aligned and k a multiple of 32");
    CERA_DISPATCH_BLOCK_TYPE(segs[0].w.type, return (launch_cols<TT>(p, n_cols, st)));
    return CERA_CUDA_OK;
}

// Any n: column tiles of 8/4/2/1 through the multi-column GEMV.  Weights are
// re-streamed once per tile, so this is the small-batch path; large batches
// belong to the tensor-core GEMM.  Cell (row i, column j) goes to out[i*ldy + j*ldc]:
// (ldy, ldc) = (n, 1) is the reference's row-major [m x n]; (1, m) is token-major.
int32_t launch_gemm_ex(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                       cudaStream_t st) {
    const size_t k = w.k;
    {
        bool taken = false;
        CERA_TRY(launch_gemm_tc(w, x, n, out, ldy, ldc, epilogue, st, &taken));  // tcgen05 / TMEM
        if (taken) return CERA_CUDA_OK;
        CERA_TRY(launch_gemm_mma(w, x, n, out, ldy, ldc, epilogue, st, &taken));  // warp-level mma.sync
        if (taken) return CERA_CUDA_OK;
    }
    size_t j = 0;
    while (j < n) {
        const size_t left = n - j;
        const size_t nc = left >= 8 ? 8 : left >= 4 ? 4 : left >= 2 ? 2 : 1;
        GemvSeg seg{w, out + j * ldc};
        ActView xv{x.scales + j * (k / 32), x.quants + j * k, x.sums + j * (k / 16)};
        // Every tile of a batch runs the item-wise kernel, so a cell's arithmetic does not depend on how the
        // columns were tiled; only the reference-layout single column (n == 1) takes the decode kernel.
        CERA_TRY(launch_gemv(&seg, 1, xv, nc, ldy, epilogue, st, ldc, /*batch_tile=*/n > 1));
        j += nc;
    }
    return CERA_CUDA_OK;
}

int32_t launch_gemm(const WeightView &w, const ActView &x, size_t n, float *out, cudaStream_t st) {
    return launch_gemm_ex(w, x, n, out, n, 1, EPI_STORE, st);
}

int32_t launch_gemv_q5k_f32(const WeightView &w, const float *x, float *y, cudaStream_t st) {
    const uint32_t ctas_needed = (w.m + WARPS - 1) / WARPS, cap = (uint32_t)sm_count() * 8;
    gemv_q5k_f32_kernel<<<ctas_needed < cap ? ctas_needed : cap, WARPS * 32, 0, st>>>(w, x, y);
    count_launch();
    return check_cuda(cudaGetLastError(), "gemv_q5k_f32 launch");
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_gemv(const cera_cuda_weight *w, const float *x_dev, float *y_dev, void *stream) {
    if (!w || !x_dev || !y_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "gemv: null argument");
    if (!w->xq) return fail(CERA_CUDA_ERR_STATE, "gemv: weight was created without activation scratch");
    cudaStream_t st = (cudaStream_t)stream;
    CERA_TRY(launch_quantize(x_dev, w->v.k, 1, false, w->xs, w->xq, w->xsum, st));
    GemvSeg seg{w->v, y_dev};
    ActView x{w->xs, w->xq, w->xsum};
    return launch_gemv(&seg, 1, x, 1, 1, EPI_STORE, st);
}

int32_t cera_cuda_gemv_q5k_f32(const cera_cuda_weight *w, const float *x_dev, float *y_dev, void *stream) {
    if (!w || !x_dev || !y_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "gemv_q5k_f32: null argument");
    if (w->v.type != CERA_TYPE_Q5_K) return fail(CERA_CUDA_ERR_UNSUPPORTED, "gemv_q5k_f32: weight is ggml type %d", w->v.type);
    return launch_gemv_q5k_f32(w->v, x_dev, y_dev, (cudaStream_t)stream);
}

int32_t cera_cuda_gemm_preq(const cera_cuda_weight *w, const float *scales_dev, const int8_t *quants_dev,
                            const int16_t *sums_dev, float *out_dev, size_t m, size_t n, size_t k, void *stream) {
    if (!w || !scales_dev || !quants_dev || !sums_dev || !out_dev)
        return fail(CERA_CUDA_ERR_BAD_ARG, "gemm_preq: null argument");
    // A declined GEMM must be loud: callers reuse output buffers (cera/src/model/transformer.rs:790-820).
    if (m != w->v.m || k != w->v.k)
        return fail(CERA_CUDA_ERR_BAD_ARG, "gemm_preq: shape [%zu x %zu] does not match the weight [%u x %u]", m, k,
                    w->v.m, w->v.k);
    if (n == 0) return CERA_CUDA_OK;
    return launch_gemm(w->v, ActView{scales_dev, quants_dev, sums_dev}, n, out_dev, (cudaStream_t)stream);
}

}  // extern "C"
