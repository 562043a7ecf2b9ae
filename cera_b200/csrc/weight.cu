// Weight upload (GGUF blocks -> 16-byte aligned planes), bit-exact dequantize,
// and the integer block-sum probe used by the parity tests.
#include <new>

#include "formats.cuh"
#include "weight.h"

namespace cera {

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// One thread per GGUF block: scatter its fields into the planes.
__global__ void repack_kernel(const WeightView w, const uint8_t *__restrict__ raw, size_t n_blocks) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const int type = w.type;
    const uint32_t nb = w.nb;
    uint8_t *qh = const_cast<uint8_t *>(w.qh), *hdr = const_cast<uint8_t *>(w.hdr), *d = const_cast<uint8_t *>(w.d);
    const TypeInfo ti = type_info(type);
    const uint8_t *src = raw + b * ti.bytes;
    auto cp = [](uint8_t *dst, const uint8_t *s, int n) {
        for (int i = 0; i < n; ++i) dst[i] = s[i];
    };
    // low-quant plane: the block's 16-byte pieces go to their (possibly piece-major) slots in the row
    const size_t row = b / nb;
    const uint32_t blk = (uint32_t)(b - row * nb);
    const uint32_t ppb = ti.q_b / 16, np = type == CERA_TYPE_Q8_0 ? 8u : 4u;
    auto cpq = [&](const uint8_t *s) {
        for (uint32_t j = 0; j < ppb; ++j) cp(const_cast<uint8_t *>(q_piece_ptr(w, row, np, blk * ppb + j)), s + 16 * j, 16);
    };
    const size_t sbi = sb_index(w, row, blk);  // slot of this block in the per-block planes (== b unless rows are interleaved)
    switch (type) {
        case CERA_TYPE_Q4_0:  // d(2) qs(16)
            cp(hdr + b * 2, src, 2);
            cpq(src + 2);
            break;
        case CERA_TYPE_Q4_1:  // d(2) m(2) qs(16)
            cp(hdr + b * 4, src, 4);
            cpq(src + 4);
            break;
        case CERA_TYPE_Q8_0:  // d(2) qs(32)
            cp(hdr + b * 2, src, 2);
            cpq(src + 2);
            break;
        case CERA_TYPE_Q4_K:  // d(2) dmin(2) scales(12) qs(128)
            cp(hdr + sbi * 16, src, 16);
            cpq(src + 16);
            break;
        case CERA_TYPE_Q5_K:  // d(2) dmin(2) scales(12) qh(32) qs(128)
            cp(hdr + sbi * 16, src, 16);
            cp(qh + sbi * 32, src + 16, 32);
            cpq(src + 48);
            break;
        case CERA_TYPE_Q6_K:  // ql(128) qh(64) scales(16) d(2)
            cpq(src);
            cp(qh + sbi * 64, src + 128, 64);
            cp(hdr + sbi * 16, src + 192, 16);
            cp(d + sbi * 2, src + 208, 2);
            break;
    }
}

// One lane per item; out is [nrows x k] f32.
template <int T>
__global__ void dequant_kernel(WeightView w, size_t row0, size_t nrows, float *__restrict__ out) {
    const size_t items_per_row = w.k / 32;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nrows * items_per_row) return;
    const size_t r = idx / items_per_row;
    const int item = (int)(idx % items_per_row);
    const typename Fmt<T>::Raw raw = Fmt<T>::load(w, row0 + r, item);
    int lo[4], hi[4];
    HalfRef h0, h1;
    Fmt<T>::decode(raw, item, lo, hi, h0, h1);
    float *o0 = out + r * w.k + h0.off, *o1 = out + r * w.k + h1.off;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int q0 = (lo[i] >> (8 * t)) & 0xFF, q1 = (hi[i] >> (8 * t)) & 0xFF;
            if (T == CERA_TYPE_Q8_0) {
                q0 = (int8_t)q0;
                q1 = (int8_t)q1;
            }
            o0[4 * i + t] = Fmt<T>::deq(q0, h0);
            o1[4 * i + t] = Fmt<T>::deq(q1, h1);
        }
}

// Integer half-block sums of one row against one activation column.
template <int T>
__global__ void block_sums_kernel(WeightView w, size_t row, const int8_t *__restrict__ xq, int32_t *u, int32_t *a) {
    const int items = w.k / 32;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const typename Fmt<T>::Raw raw = Fmt<T>::load(w, row, item);
        int lo[4], hi[4];
        HalfRef h0, h1;
        Fmt<T>::decode(raw, item, lo, hi, h0, h1);
        const int one[4] = {0x01010101, 0x01010101, 0x01010101, 0x01010101};
        const int a0 = dot16(one, xq + h0.off), a1 = dot16(one, xq + h1.off);
        u[h0.off / 16] = Fmt<T>::view(dot16(lo, xq + h0.off), a0);
        u[h1.off / 16] = Fmt<T>::view(dot16(hi, xq + h1.off), a1);
        a[h0.off / 16] = a0;
        a[h1.off / 16] = a1;
    }
}

}  // namespace

int32_t weight_upload(int32_t type, size_t m, size_t k, const void *bytes, size_t nbytes, bool with_scratch,
                      cera_cuda_weight **out) {
    if (!out || !bytes) return fail(CERA_CUDA_ERR_BAD_ARG, "weight_create: null argument");
    if (!is_block_type(type))
        return fail(CERA_CUDA_ERR_UNSUPPORTED, "weight_create: ggml type %d has no quantized-matmul kernel", type);
    const TypeInfo ti = type_info(type);
    if (m == 0 || k == 0 || k % ti.elems)
        return fail(CERA_CUDA_ERR_BAD_ARG, "weight_create: k=%zu is not a positive multiple of the block width %d", k,
                    ti.elems);
    const size_t nb = k / ti.elems, n_blocks = m * nb;
    if (nbytes != n_blocks * ti.bytes)
        return fail(CERA_CUDA_ERR_BAD_ARG, "weight_create: %zu bytes given, [%zu x %zu] of type %d needs %zu", nbytes,
                    m, k, type, n_blocks * (size_t)ti.bytes);
    if (m > 0xFFFFFFFFull || k > 0x7FFFFFFFull) return fail(CERA_CUDA_ERR_BAD_ARG, "weight_create: shape too large");

    auto *w = new (std::nothrow) cera_cuda_weight();
    if (!w) return fail(CERA_CUDA_ERR_OOM, "weight_create: host allocation failed");
    cudaGetDevice(&w->device);
    // K-quants with whole 128-weight lane tasks: groups of eight rows interleaved (common.cuh), rows padded with zeros
    const bool kq = type == CERA_TYPE_Q4_K || type == CERA_TYPE_Q5_K || type == CERA_TYPE_Q6_K;
    const uint32_t ilv = (kq && k % 128 == 0) ? 8u : 0u;
    const size_t plane_blocks = ilv ? (m + 7) / 8 * 8 * nb : n_blocks;
    const size_t q_sz = align_up(plane_blocks * ti.q_b, 256), qh_sz = align_up(plane_blocks * ti.qh_b, 256),
                 hdr_sz = align_up(plane_blocks * ti.hdr_b, 256), d_sz = align_up(plane_blocks * ti.d_b, 256);
    const size_t xs_sz = with_scratch ? align_up(k / 32 * 4, 256) : 0, xq_sz = with_scratch ? align_up(k, 256) : 0,
                 xsum_sz = with_scratch ? align_up(k / 16 * 2, 256) : 0;
    w->bytes = q_sz + qh_sz + hdr_sz + d_sz + xs_sz + xq_sz + xsum_sz;
    int32_t st = check_cuda(cudaMalloc(&w->base, w->bytes), "cudaMalloc(weight planes)");
    if (st != CERA_CUDA_OK) {
        delete w;
        return st;
    }
    uint8_t *p = (uint8_t *)w->base;
    uint8_t *q = p;
    uint8_t *qh = q + q_sz;
    uint8_t *hdr = qh + qh_sz;
    uint8_t *d = hdr + hdr_sz;
    if (with_scratch) {
        w->xs = (float *)(d + d_sz);
        w->xq = (int8_t *)((uint8_t *)w->xs + xs_sz);
        w->xsum = (int16_t *)((uint8_t *)w->xq + xq_sz);
    }
    const uint32_t t128 = k % 128 == 0 ? (uint32_t)(k / 128) : 0u;
    w->v = WeightView{type, (uint32_t)m, (uint32_t)k, (uint32_t)nb, t128, ilv, q, ti.qh_b ? qh : nullptr, hdr,
                      ti.d_b ? d : nullptr, nullptr};
    if (ilv && plane_blocks != n_blocks) {  // the padding rows of the last group read as zero weights
        st = check_cuda(cudaMemset(w->base, 0, q_sz + qh_sz + hdr_sz + d_sz), "cudaMemset(weight planes)");
        if (st != CERA_CUDA_OK) {
            cudaFree(w->base);
            delete w;
            return st;
        }
    }

    // Stage the raw blocks on the device, scatter, release the staging copy.
    void *raw = nullptr;
    st = check_cuda(cudaMalloc(&raw, nbytes), "cudaMalloc(weight staging)");
    if (st == CERA_CUDA_OK) st = check_cuda(cudaMemcpy(raw, bytes, nbytes, cudaMemcpyDefault), "cudaMemcpy(weight)");
    if (st == CERA_CUDA_OK) {
        const int threads = 128;
        const size_t grid = (n_blocks + threads - 1) / threads;
        repack_kernel<<<(unsigned)grid, threads>>>(w->v, (const uint8_t *)raw, n_blocks);
        count_launch();
        st = check_cuda(cudaGetLastError(), "repack launch");
        if (st == CERA_CUDA_OK) st = check_cuda(cudaDeviceSynchronize(), "repack");
    }
    if (raw) cudaFree(raw);
    if (st != CERA_CUDA_OK) {
        cudaFree(w->base);
        delete w;
        return st;
    }
    *out = w;
    return CERA_CUDA_OK;
}

}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_weight_create(int32_t type, size_t m, size_t k, const void *bytes, size_t nbytes,
                                cera_cuda_weight **out) {
    return weight_upload(type, m, k, bytes, nbytes, true, out);
}

void cera_cuda_weight_free(cera_cuda_weight *w) {
    if (!w) return;
    if (w->base) cudaFree(w->base);
    if (w->tc_image) cudaFree(w->tc_image);
    delete w;
}

int32_t cera_cuda_weight_prepare_gemm(cera_cuda_weight *w, int32_t *has_image) {
    bool built = false;
    const int32_t rc = weight_prepare_tc(w, &built);
    if (has_image) *has_image = built ? 1 : 0;
    return rc;
}

int32_t cera_cuda_weight_info(const cera_cuda_weight *w, int32_t *type, size_t *m, size_t *k, size_t *device_bytes) {
    if (!w) return fail(CERA_CUDA_ERR_BAD_ARG, "weight_info: null weight");
    if (type) *type = w->v.type;
    if (m) *m = w->v.m;
    if (k) *k = w->v.k;
    if (device_bytes) *device_bytes = w->bytes + w->tc_bytes;
    return CERA_CUDA_OK;
}

int32_t cera_cuda_dequantize_rows(const cera_cuda_weight *w, size_t row0, size_t nrows, float *out_dev, void *stream) {
    if (!w || !out_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "dequantize_rows: null argument");
    if (row0 + nrows > w->v.m) return fail(CERA_CUDA_ERR_BAD_ARG, "dequantize_rows: rows [%zu,%zu) exceed m=%u", row0, row0 + nrows, w->v.m);
    if (nrows == 0) return CERA_CUDA_OK;
    const size_t total = nrows * (w->v.k / 32);
    const int threads = 128;
    const unsigned grid = (unsigned)((total + threads - 1) / threads);
    CERA_DISPATCH_BLOCK_TYPE(w->v.type, (dequant_kernel<TT><<<grid, threads, 0, (cudaStream_t)stream>>>(w->v, row0, nrows, out_dev)));
    count_launch();
    return check_cuda(cudaGetLastError(), "dequantize launch");
}

int32_t cera_cuda_block_sums(const cera_cuda_weight *w, size_t row, const int8_t *quants_dev, int32_t *u_dev,
                             int32_t *a_dev, void *stream) {
    if (!w || !quants_dev || !u_dev || !a_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "block_sums: null argument");
    if (row >= w->v.m) return fail(CERA_CUDA_ERR_BAD_ARG, "block_sums: row %zu out of range", row);
    if ((uintptr_t)quants_dev % 16) return fail(CERA_CUDA_ERR_BAD_ARG, "block_sums: quants must be 16-byte aligned");
    CERA_DISPATCH_BLOCK_TYPE(w->v.type, (block_sums_kernel<TT><<<1, 128, 0, (cudaStream_t)stream>>>(w->v, row, quants_dev, u_dev, a_dev)));
    count_launch();
    return check_cuda(cudaGetLastError(), "block_sums launch");
}

}  // extern "C"
