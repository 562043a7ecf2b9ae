// Shared declarations for the sm_100a kernels: status plumbing, the device
// layout of a quantized weight, and the per-format decode helpers every kernel
// (GEMV, GEMM, dequantize, block-sum probe) goes through.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cera_cuda.h"

namespace cera {

// ---- status ---------------------------------------------------------------
int32_t fail(int32_t code, const char *fmt, ...);
int32_t check_cuda(cudaError_t e, const char *what);
void count_launch(int n = 1);      // bumps the library-wide kernel launch counter
uint64_t launches_so_far();

#define CERA_CUDA_TRY(expr)                                          \
    do {                                                             \
        int32_t _st = ::cera::check_cuda((expr), #expr);             \
        if (_st != CERA_CUDA_OK) return _st;                         \
    } while (0)
#define CERA_TRY(expr)                                               \
    do {                                                             \
        int32_t _st = (expr);                                        \
        if (_st != CERA_CUDA_OK) return _st;                         \
    } while (0)

// ---- device layout of a weight matrix --------------------------------------
// GGUF stores a row as packed blocks (18/20/34/144/176/210 bytes) whose fields
// are at best 2-byte aligned.  On load each tensor is split into planes whose
// per-row extents are multiples of 16 bytes, so a warp streams a row with
// 128-bit loads; the byte total is unchanged.  `nb` counts the format's blocks
// per row (32-element blocks, or 256-element super-blocks for K-quants).
//
//   Q4_0 : q[m][nb][16]                     d[m][nb] (half)
//   Q4_1 : q[m][nb][16]                     dm[m][nb] (half2: d, m)
//   Q8_0 : q[m][nb][32]                     d[m][nb] (half)
//   Q4_K : q[m][nb][128]                    hdr[m][nb][16] (d, dmin, scales[12])
//   Q5_K : q[m][nb][128]  qh[m][nb][32]     hdr[m][nb][16]
//   Q6_K : q[m][nb][128]  qh[m][nb][64]     sc[m][nb][16]   d[m][nb] (half)
//
// Inside a row the low-quant plane is stored PIECE-MAJOR when k is a multiple of 128
// (t128 = k/128 != 0): the row is cut into 128-weight lane tasks of NP 16-byte pieces
// (NP = 4, or 8 for Q8_0), and piece c of task t sits at 16*(c*t128 + t).  A warp whose
// lane t fetches piece c of its own task then reads 512 contiguous bytes per load.
struct WeightView {
    int32_t type;
    uint32_t m, k, nb;
    uint32_t t128;       // lane tasks per row, 0 = pieces in GGUF order
    uint32_t ilv;        // 8: K-quant planes interleave groups of eight rows (see below), 0: rows one after another
    const uint8_t *q;    // low quant plane
    const uint8_t *qh;   // high-bit plane (Q5_K, Q6_K)
    const uint8_t *hdr;  // scale plane (see table)
    const uint8_t *d;    // Q6_K super-scale plane
    const uint8_t *tc;   // optional: f16 operand image for the tcgen05 GEMM (Q4_K / Q5_K), null without one
};

struct TypeInfo {
    int elems, bytes;    // GGUF block
    int q_b, qh_b, hdr_b, d_b;  // plane bytes per block
};

__host__ __device__ inline TypeInfo type_info(int t) {
    switch (t) {
        case CERA_TYPE_Q4_0: return {32, 18, 16, 0, 2, 0};
        case CERA_TYPE_Q4_1: return {32, 20, 16, 0, 4, 0};
        case CERA_TYPE_Q8_0: return {32, 34, 32, 0, 2, 0};
        case CERA_TYPE_Q4_K: return {256, 144, 128, 0, 16, 0};
        case CERA_TYPE_Q5_K: return {256, 176, 128, 32, 16, 0};
        case CERA_TYPE_Q6_K: return {256, 210, 128, 64, 16, 2};
        case CERA_TYPE_F32: return {1, 4, 4, 0, 0, 0};
        case CERA_TYPE_F16: return {1, 2, 2, 0, 0, 0};
        case CERA_TYPE_BF16: return {1, 2, 2, 0, 0, 0};
        default: return {0, 0, 0, 0, 0, 0};
    }
}

// K-quants with k a multiple of 128 are stored with groups of EIGHT ROWS INTERLEAVED (ilv = 8; the row count is
// padded to a multiple of eight with zero rows): in the low-quant plane piece c of task t of row r sits at
//   (r/8) * 8 * row_bytes + ((t*8 + r%8) * 4 + c) * 16,
// so that the 32 lanes (row%8, c) of a warp that walk their strips in task order read 512 contiguous bytes per
// load; the header, high-bit and super-scale planes are indexed by sb_index() = ((r/8)*nb + sb)*8 + r%8.
// Byte offset inside a row's low-quant plane of its i-th 16-byte piece (GGUF order).
__host__ __device__ inline size_t q_piece_off(uint32_t t128, uint32_t np, uint32_t i) {
    if (!t128) return (size_t)i * 16;
    const uint32_t t = i / np, c = i - t * np;
    return ((size_t)c * t128 + t) * 16;
}

// Index of (row, super-block) in the per-super-block planes (hdr, qh, d).
__host__ __device__ inline size_t sb_index(const WeightView &w, size_t row, size_t sb) {
    return w.ilv ? ((row >> 3) * w.nb + sb) * 8 + (row & 7) : row * w.nb + sb;
}
// Address of the i-th 16-byte piece (GGUF order) of a row's low-quant plane; np = pieces per lane task (4, Q8_0: 8).
__host__ __device__ inline const uint8_t *q_piece_ptr(const WeightView &w, size_t row, uint32_t np, uint32_t i) {
    const TypeInfo ti = type_info(w.type);
    const size_t row_bytes = (size_t)w.nb * ti.q_b;
    if (w.ilv) {
        const uint32_t t = i >> 2, c = i & 3;
        return w.q + (row >> 3) * 8 * row_bytes + (((size_t)t * 8 + (row & 7)) * 4 + c) * 16;
    }
    return w.q + row * row_bytes + q_piece_off(w.t128, np, i);
}

inline bool is_block_type(int t) {
    return t == CERA_TYPE_Q4_0 || t == CERA_TYPE_Q4_1 || t == CERA_TYPE_Q8_0 || t == CERA_TYPE_Q4_K ||
           t == CERA_TYPE_Q5_K || t == CERA_TYPE_Q6_K;
}

// ---- small device helpers ---------------------------------------------------
__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

// 6-bit scale / min of sub-block s from the 12 packed bytes
// (cera/src/quant.rs:591-605).
__device__ __forceinline__ void kscale(const uint8_t *s12, int s, int &sc, int &mn) {
    if (s < 4) {
        sc = s12[s] & 63;
        mn = s12[s + 4] & 63;
    } else {
        sc = (s12[s + 4] & 0x0F) | ((s12[s - 4] >> 6) << 4);
        mn = (s12[s + 4] >> 4) | ((s12[s] >> 6) << 4);
    }
}

// 128-bit streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- programmatic dependent launch ----------------------------------------------
// Every kernel of the decode step begins with pdl_trigger() (the next kernel in the stream may be
// scheduled and run the part of its code that precedes its own pdl_wait()) and calls pdl_wait()
// before it first touches anything an earlier kernel wrote, and before its own first write.  Weight
// bytes are immutable, so a GEMV prefetches its first rows ahead of the wait.  Both are no-ops when
// the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool pdl_enabled();  // CERA_CUDA_PDL=0 turns the launch attribute off (read once)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- launch geometry ----------------------------------------------------------
int sm_count();  // SMs of the current device (148 on B200), cached

}  // namespace cera
