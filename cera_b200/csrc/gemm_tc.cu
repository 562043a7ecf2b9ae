// Prefill GEMM on the fifth-generation tensor cores: out[m x n] = W (Q4_K / Q5_K / Q6_K) x X (Q8_0 columns) with
// tcgen05.mma, accumulators in tensor memory (TMEM), for n >= 33 columns (Q6_K: n >= 129) and k a multiple of 256.
//
// The arithmetic contract (cera/src/backend/simd.rs:5248-5371, 5693-5878) scales every 32-element block's integer sum
// by (weight block scale) x (activation block scale).  A kernel that rescales each block's sum on the CUDA cores is
// bound by that work, not by the tensor pipe (measured: 11 300 issued instructions per 128-k stage around 512 cycles
// of MMA).  Here BOTH block scales ride inside the operands, so the tensor cores accumulate a whole 256-element
// super-block and the CUDA cores touch the accumulators once per super-block:
//
//  * Weight operand: sc * q, the six-bit sub-block scale times the 4/5-bit quant (at most 63 * 31 = 1953 < 2048):
//    an exact small integer in f16.
//  * Activation operand: v = (g * xs_b) * a for the int8 quant a of block b - the activation block scale folded in, g a
//    power of two per token that brings every v below 2^15 - as TWO f16 operands: the top 11 bits of v and the
//    f16-rounded remainder.  Each MMA step runs twice (high and low part) into the same accumulator; 22 significant
//    bits of every activation survive, the products are exact, the f32 accumulation is the tensor core's.
//  * The min term sum_b dmin * mn_b * (xs_b * A_b) (A_b = the block's sum of quants) is one more 16-column MMA per
//    super-block: the eight six-bit mins (each twice) times the high / low parts of g * xs_b * A_b, into a third
//    accumulator.
//  * Per super-block the epilogue folds out[row] += (d[row] * D - dmin[row] * Dm) / g into a TMEM region.
//
// The results agree with the reference within its f32 tolerance (1e-3 relative; measured ~1e-6), not bit for bit: the
// bit-exact block sums are the decode path's and cera_cuda_block_sums' business.
//
// The activation operands are converted ONCE per GEMM by two small kernels (a per-token range search for g, then the
// high / low operand tiles written to a stream-ordered scratch buffer in the shared-memory layout of the GEMM kernels,
// so that a stage's 32 KB arrive by one bulk asynchronous copy).  The weight operand comes from a RESIDENT IMAGE of the
// weight (weight_prepare_tc: sc * q as f16 in the same tile layout, about 2.3 bytes per weight, built when a model sees
// its first batched prompt or a caller asks for it), so a stage is a few bulk copies and 8-16 MMAs; a weight without an
// image has its operand built in shared memory by producer warps straight from the quantized bytes (nibble -> 0x6400|q
// -> one HFMA2 with the sub-block scale), same results.  Tiles use the canonical K-major no-swizzle layout (8-row x
// 16-byte core matrices), 64 k-elements per stage.
//
// Three kernels:
//  * gemm_tcw_kernel ("wide", image only): 128 tokens x 256 rows per CTA when those tiles alone fill the device.  TMEM
//    holds two double-buffered 256-column accumulators; the running output lives in the epilogue threads' registers;
//    the min term is one more GEMM over the k / 32 blocks after the k loop.
//  * gemm_tc_kernel<T, IMG>: 128 x 128 per CTA.  IMG: the loader thread fetches all three operands, the min term is the
//    16-column MMA above into its own double-buffered accumulator, output in registers.  !IMG: 18 warps - warp 0
//    issues the MMAs from one thread, warps 1-8 build the weight operand (thread = weight row x half of the stage's
//    bytes), one thread of warp 9 requests the activation operands, warps 10-17 are the epilogue (thread = token lane x
//    64 rows) with the running output in a fourth TMEM region.
//  * gemm_tc6_kernel (Q6_K, image only): sc * (q - 32) needs 13 bits, so the image holds it as two exact f16 operands
//    and a k-step is three MMAs; no min term.
// Stages and accumulator buffers are handed over through mbarriers (tcgen05.commit arrives on them when the MMAs have
// finished).  Every wait is bounded: when a limit runs out the CTA raises an abort flag, its roles leave their loops,
// TMEM is freed and a status word reports it (cera_cuda_kernel_status).
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "gemv_task.cuh"
#include "tma.cuh"
#include "weight.h"

namespace cera {

__device__ unsigned int g_tc_status = 0;  // nonzero: a bounded wait of gemm_tc_kernel ran out (bits name the role)

namespace {

constexpr int TC_BM = 128;      // tokens per tile (TMEM lanes)
constexpr int TC_BN = 128;      // weight rows per tile (TMEM columns)
constexpr int TC_KS = 64;       // k elements per stage: two 32-element blocks, half a 128-weight task
constexpr int TC_STAGES = 4;    // = stages per 256-element super-block
constexpr int TC_W_WARPS = 8, TC_EPI_WARPS = 8;
constexpr int TC_THREADS = (2 + TC_W_WARPS + TC_EPI_WARPS) * 32;  // 576: MMA issue, weight producers, operand loader, epilogue
constexpr int TC_THREADS_IMG = (2 + TC_EPI_WARPS) * 32;            // 320: with a resident weight image there are no weight producers
constexpr int TC_IMG_THREADS = 256;                                   // the activation-image kernel: (token, block of the stage)
constexpr uint32_t TC_OP_BYTES = TC_BM * TC_KS * 2;                      // one operand tile of a stage: 16 KB
constexpr uint32_t TC_STAGE_BYTES = 3 * TC_OP_BYTES;                     // activations high, activations low, weights
// per super-block, two slots: the min-term operands (16 k-columns each) and the row-side tables
constexpr uint32_t TC_MINOP_BYTES = TC_BM * 16 * 2;                      // 4 KB: [2 k chunks][128 rows][8 f16]
constexpr uint32_t TC_SLOT_BYTES = 2 * TC_MINOP_BYTES + 2 * TC_BN * 4;   // A, B, dval[128], dmin[128]
// resident weight image (tc_weight_image_kernel): per (row tile, stage) one operand tile; per (row tile, super-block) the
// row side of the min operand followed by dval[128], dmin[128] - the tail of a slot, one copy
constexpr uint32_t TC_SIDE_BYTES = TC_MINOP_BYTES + 2 * TC_BN * 4;        // 5 KB
constexpr uint32_t TC_TAIL_OFF = TC_STAGES * TC_STAGE_BYTES + 2 * TC_SLOT_BYTES;  // barriers, TMEM address, abort flag
constexpr uint32_t TC_SMEM_BYTES = TC_TAIL_OFF + 256;
constexpr uint32_t TC_TMEM_COLS = 512;  // D0 [0,128) D1 [128,256), then Dm [256,384) OUT [384,512) or, with the weight image, Dm0 Dm1
constexpr uint32_t TC_KC_STRIDE = TC_BM * 16;                            // bytes between 8-element k chunks: 2048

// The wide variant (a CTA owns 128 tokens x 256 weight rows, weight image only): stages of the two activation operand
// tiles and the operand tiles of two 128-row image tiles; the min term is one more GEMM at the end of the k loop (see
// gemm_tcw_kernel), whose stages of 32 activation blocks reuse the ring.
constexpr int TCW_STAGES = 3;
constexpr uint32_t TCW_STAGE_BYTES = 4 * TC_OP_BYTES;                     // A high, A low, B rows [0,128), B rows [128,256): 64 KB
constexpr uint32_t TCW_MIN_J = 32;                                        // activation blocks (k / 32 columns) per min stage
constexpr uint32_t TCW_MINT_BYTES = TC_BM * TCW_MIN_J * 2;                // one min-GEMM operand tile: 8 KB
constexpr uint32_t TCW_DVAL_OFF = TCW_STAGES * TCW_STAGE_BYTES;           // two slots of d[256]
constexpr uint32_t TCW_RS_OFF = TCW_DVAL_OFF + 2 * 2 * TC_BN * 4;         // 2^-s[256] of the min GEMM's weight rows
constexpr uint32_t TCW_TAIL_OFF = TCW_RS_OFF + 2 * TC_BN * 4;
constexpr uint32_t TCW_SMEM_BYTES = TCW_TAIL_OFF + 256;
constexpr int TCW_THREADS = (2 + TC_EPI_WARPS) * 32;

// Regions of a weight's resident image (byte offsets): the operand tile of every (128-row tile, stage); per (tile,
// super-block) the row side of the min operand, d[128] and dmin[128]; per (tile, min stage) the high and the low part of
// dmin * min * 2^s; per tile 2^-s[128].
struct TcImage {
    uint32_t tiles, n_it, n_sb, n_mit;
    size_t side, wmin, rscale, total;
};
__host__ __device__ inline TcImage tc_image_layout(uint32_t m, uint32_t k) {
    TcImage L;
    L.tiles = (m + TC_BN - 1) / TC_BN;
    L.n_it = k / TC_KS;
    L.n_sb = k / 256;
    L.n_mit = (k / 32 + TCW_MIN_J - 1) / TCW_MIN_J;
    L.side = (size_t)L.tiles * L.n_it * TC_OP_BYTES;
    L.wmin = L.side + (size_t)L.tiles * L.n_sb * TC_SIDE_BYTES;
    L.rscale = L.wmin + (size_t)L.tiles * L.n_mit * 2 * TCW_MINT_BYTES;
    L.total = L.rscale + (size_t)L.tiles * TC_BN * 4;
    return L;
}

struct TcParams {
    WeightView w;
    float *out;
    uint32_t m, n, k;
    uint32_t ldy, ldc;
    int epilogue;
    // the activation operands of this GEMM, converted once (tc_token_image_kernel): per (token tile, stage) the high and
    // the low operand tile, per (token tile, super-block) the token side of the min operand, per token 1 / g
    const uint8_t *img, *img_min;
    const float *ginv;
    const uint8_t *xm;  // per (token tile, min stage) the high and the low part of g * xs_b * A_b (the wide variant's min GEMM)
    // Up to two more weights that take the same activations (q / k / v, gate / up), with images, in the same launch: the
    // grid's y tiles [y_end[i - 1], y_end[i]) belong to weight i (0 = the fields above).
    uint32_t n_w;
    uint32_t y_end[3];
    const uint8_t *tc_x[2];
    float *out_x[2];
    uint32_t m_x[2], ldc_x[2];
};

// The weight a CTA works for and its y tile inside that weight.
struct TcSub {
    const uint8_t *tc;
    float *out;
    uint32_t m, ldc, by;
};
__device__ __forceinline__ TcSub tc_select(const TcParams &p) {
    TcSub s{p.w.tc, p.out, p.m, p.ldc, blockIdx.y};
    if (p.n_w > 1 && blockIdx.y >= p.y_end[0]) {
        const int i = (p.n_w > 2 && blockIdx.y >= p.y_end[1]) ? 1 : 0;
        s.tc = p.tc_x[i];
        s.out = p.out_x[i];
        s.m = p.m_x[i];
        s.ldc = p.ldc_x[i];
        s.by = blockIdx.y - p.y_end[i];
    }
    return s;
}

// ---- PTX wrappers -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tma::smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16, issued by one thread.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;  // disable-output-lane mask: none
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero)
        : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tma::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; `lbo` = bytes between the
// two 8-element k chunks of one MMA, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
           (1ull << 46);
}
// Instruction descriptor: f16 x f16 -> f32, both operands K-major, M x N.
__host__ __device__ constexpr uint32_t tc_idesc(uint32_t M, uint32_t N) { return (1u << 4) | ((N >> 3) << 17) | ((M >> 4) << 24); }

// Eight f16 values of a k chunk for row `r`: offset of the 16-byte slot in an operand tile.
__device__ __forceinline__ uint32_t op_off(uint32_t kc, uint32_t r) { return kc * TC_KC_STRIDE + r * 16; }

// Four unsigned bytes -> two half2 holding 1024 + byte (the exponent 0x64 puts the byte into the mantissa's low bits).
__device__ __forceinline__ void bytes_to_h1024(uint32_t v, __half2 &lo, __half2 &hi) {
    const uint32_t a = __byte_perm(v, 0x64646464u, 0x5140), b = __byte_perm(v, 0x64646464u, 0x7362);
    lo = *reinterpret_cast<const __half2 *>(&a);
    hi = *reinterpret_cast<const __half2 *>(&b);
}

// g[token]: a power of two that brings every |xs_b * a| of the token below 2^15 (|a| <= 127, and |A_b| <= 4064 for the
// min operand: 2^15 / 32 keeps both in range).  One warp per token (tokens past n repeat the last one).
__global__ void tc_token_range_kernel(const ActView x, uint32_t n, uint32_t k, uint32_t n_pad, float *__restrict__ g_out, float *__restrict__ ginv_out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_pad) return;
    const uint32_t token = min(t, n - 1), nb32 = k >> 5;
    float mx = 0.0f;
    for (uint32_t b = lane; b < nb32; b += 32) {
        const float v = fabsf(__ldg(x.scales + (size_t)token * nb32 + b));
        mx = fmaxf(mx, v == v && v < 1.0e30f ? v : 0.0f);  // (scales beyond 1e30 are not activations: left out of the range search)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float g = 1.0f;
    if (mx > 0.0f) {
        int e;
        frexpf(mx * 4064.0f, &e);  // |xs_b * A_b| <= mx * 4064 < 2^e
        g = ldexpf(1.0f, 15 - e);
    }
    if (lane == 0) {
        g_out[t] = g;
        ginv_out[t] = 1.0f / g;
    }
}

// The activation operands of one (token tile, stage): v = (g * xs_b) * a for the 64 quants of the stage, as the top 11
// significant bits of v (high operand) and the f16-rounded remainder (low operand), written in the shared-memory
// layout of the GEMM kernel (chunk kc of token c at kc * 2048 + c * 16) so that a stage is one contiguous 32 KB copy;
// and g * xs_b * A_b, high and low, into the token side of the super-block's min operand.  grid (token tiles, stages),
// 256 threads: thread = (token, block of the stage).
__global__ void __launch_bounds__(TC_IMG_THREADS) tc_token_image_kernel(const ActView x, uint32_t n, uint32_t k, const float *__restrict__ g_tab,
                                                                         uint8_t *__restrict__ img, uint8_t *__restrict__ img_min, uint8_t *__restrict__ xm) {
    pdl_trigger();
    pdl_wait();
    const uint32_t c = threadIdx.x >> 1, blk = threadIdx.x & 1, it = blockIdx.y, st = it % TC_STAGES, sb = it / TC_STAGES;
    const uint32_t n_it = k / TC_KS, n_sb = k / 256, nb32 = k >> 5, nb16 = k >> 4;
    const uint32_t token = min(blockIdx.x * TC_BM + c, n - 1);
    const float g = g_tab[blockIdx.x * TC_BM + c];
    const uint32_t xb = it * 2 + blk;  // this thread's 32-element activation block
    const int8_t *src = x.quants + (size_t)token * k + (size_t)xb * 32;
    const uint4 r0 = __ldg(reinterpret_cast<const uint4 *>(src)), r1 = __ldg(reinterpret_cast<const uint4 *>(src) + 1);
    const float sg = __ldg(x.scales + (size_t)token * nb32 + xb) * g;
    const int16_t *sm = reinterpret_cast<const int16_t *>(x.sums) + (size_t)token * nb16 + 2 * xb;
    const float asum = (float)((int)__ldg(sm) + (int)__ldg(sm + 1));
    uint8_t *op_hi = img + ((size_t)blockIdx.x * n_it + it) * (2 * TC_OP_BYTES), *op_lo = op_hi + TC_OP_BYTES;
    const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    const float2 sg2 = make_float2(sg, sg);
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {  // eight elements = one 16-byte k chunk of each operand
        __half2 hi2[4], lo2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t w = words[2 * ch + (q >> 1)];
            const int e0 = (int)(int8_t)(w >> (16 * (q & 1))), e1 = (int)(int8_t)(w >> (16 * (q & 1) + 8));
            const float2 v = __fmul2_rn(make_float2((float)e0, (float)e1), sg2);
            // high part: the top 11 significant bits (exactly an f16 while v is in the normal range); low: the rest, rounded
            const float2 vh = make_float2(__uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u), __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u));
            const float2 vl = __fadd2_rn(v, make_float2(-vh.x, -vh.y));
            hi2[q] = __float22half2_rn(vh);
            lo2[q] = __float22half2_rn(vl);
        }
        *reinterpret_cast<uint4 *>(op_hi + op_off(4 * blk + ch, c)) = *reinterpret_cast<const uint4 *>(&hi2[0]);
        *reinterpret_cast<uint4 *>(op_lo + op_off(4 * blk + ch, c)) = *reinterpret_cast<const uint4 *>(&lo2[0]);
    }
    {
        // g * xs_b * A_b as a high and a low f16: block 2 st + blk of the super-block's min operand
        const float v = sg * asum;
        const float vh = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
        const __half2 hl = __floats2half2_rn(vh, v - vh);
        uint8_t *slot = img_min + ((size_t)blockIdx.x * n_sb + sb) * TC_MINOP_BYTES;
        *reinterpret_cast<uint32_t *>(slot + op_off(st >> 1, c) + ((st & 1) * 2 + blk) * 4) = *reinterpret_cast<const uint32_t *>(&hl);
        // the same pair as column xb of the wide variant's min GEMM: a high tile and a low tile per 32 blocks
        const uint32_t n_mit = (nb32 + TCW_MIN_J - 1) / TCW_MIN_J, mi = xb / TCW_MIN_J, jj = xb % TCW_MIN_J;
        uint8_t *xt = xm + ((size_t)blockIdx.x * n_mit + mi) * (2 * TCW_MINT_BYTES) + op_off(jj >> 3, c) + (jj & 7) * 2;
        *reinterpret_cast<__half *>(xt) = __low2half(hl);
        *reinterpret_cast<__half *>(xt + TCW_MINT_BYTES) = __high2half(hl);
    }
}

// ---- the weight operand of one stage: thread = (weight row r of the tile, half of the stage's bytes) -------------------
struct TcRawW {
    uint4 pc, h, hb;
};
// The stage's 32 quant bytes of a row are pieces 2 pair, 2 pair + 1 of the task (low nibbles = sub-block 2 pair, high =
// 2 pair + 1); the thread takes piece 2 pair + half: elements [16 half, +16) of both sub-blocks.
template <int T>
__device__ __forceinline__ TcRawW tc_fetch_w(const WeightView &w, uint32_t row, uint32_t half, uint32_t it) {
    TcRawW rw;
    const uint32_t st = it % TC_STAGES, sb = it / TC_STAGES, pair = st & 1, hf = st >> 1;
    rw.pc = ld_stream(q_piece_ptr(w, row, 4, (2 * sb + hf) * 4 + 2 * pair + half));
    const size_t sbi = sb_index(w, row, sb);
    rw.h = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sbi);
    rw.hb = make_uint4(0, 0, 0, 0);
    if (T == CERA_TYPE_Q5_K) rw.hb = __ldg(reinterpret_cast<const uint4 *>(w.qh + sbi * 32 + half * 16));
    return rw;
}
// sc * q as f16 into the operand tile `opb`; with half == 0 also the stage's two mins into the row side of the min
// operand `bmin` and, with the super-block's first stage, d and dmin into `dval`.  The destinations are shared memory in
// the GEMM kernel and global memory when the resident image is built.
template <int T>
__device__ __forceinline__ void tc_convert_w(const TcRawW &cur, uint32_t r, uint32_t half, uint32_t st, uint8_t *opb, uint8_t *bmin, float *dval) {
    const uint32_t pair = st & 1, hf = st >> 1;  // task 2 sb + hf, byte pair `pair`
    const uint4 v4 = cur.pc, h = cur.h, hbv = cur.hb;
    uint32_t scp, mnp;
    kq_quad(h, hf, scp, mnp);
    const uint32_t sc_lo = (scp >> (16 * pair)) & 0xFF, sc_hi = (scp >> (16 * pair + 8)) & 0xFF;
    const __half2 s_lo = __half2half2(__ushort2half_rn((unsigned short)sc_lo)), s_hi = __half2half2(__ushort2half_rn((unsigned short)sc_hi));
    const __half2 nb_lo = __hmul2(s_lo, __float2half2_rn(-1024.0f)), nb_hi = __hmul2(s_hi, __float2half2_rn(-1024.0f));
    {
        const uint32_t wv[4] = {v4.x, v4.y, v4.z, v4.w}, hw[4] = {hbv.x, hbv.y, hbv.z, hbv.w};
        __half2 lo8[8], hi8[8];  // 16 low-nibble and 16 high-nibble elements, two per half2
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t lo = wv[i] & 0x0F0F0F0Fu, hi = (wv[i] >> 4) & 0x0F0F0F0Fu;
            if (T == CERA_TYPE_Q5_K) {
                const int sh = 4 * hf + 2 * pair;
                lo |= ((hw[i] >> sh) & 0x01010101u) << 4;
                hi |= ((hw[i] >> (sh + 1)) & 0x01010101u) << 4;
            }
            __half2 a, b;
            bytes_to_h1024(lo, a, b);
            lo8[2 * i] = __hfma2(a, s_lo, nb_lo);  // (1024 + q) * sc - 1024 * sc = q * sc, one rounding of an exact value
            lo8[2 * i + 1] = __hfma2(b, s_lo, nb_lo);
            bytes_to_h1024(hi, a, b);
            hi8[2 * i] = __hfma2(a, s_hi, nb_hi);
            hi8[2 * i + 1] = __hfma2(b, s_hi, nb_hi);
        }
        // low nibbles: elements [16 half, +16) of the stage's first block; high nibbles: the same of its second block
        const uint32_t kc_lo = 2 * half, kc_hi = kc_lo + 4;
        *reinterpret_cast<uint4 *>(opb + op_off(kc_lo, r)) = *reinterpret_cast<const uint4 *>(&lo8[0]);
        *reinterpret_cast<uint4 *>(opb + op_off(kc_lo + 1, r)) = *reinterpret_cast<const uint4 *>(&lo8[4]);
        *reinterpret_cast<uint4 *>(opb + op_off(kc_hi, r)) = *reinterpret_cast<const uint4 *>(&hi8[0]);
        *reinterpret_cast<uint4 *>(opb + op_off(kc_hi + 1, r)) = *reinterpret_cast<const uint4 *>(&hi8[4]);
    }
    if (half == 0) {
        // the mins of the stage's two blocks, each twice (for the high and the low part of the token side): four
        // f16 = blocks 2 st, 2 st + 1 of the super-block's 16-column min operand
        const uint32_t mn0 = (mnp >> (16 * pair)) & 0xFF, mn1 = (mnp >> (16 * pair + 8)) & 0xFF;
        __half2 m2[2] = {__half2half2(__ushort2half_rn((unsigned short)mn0)), __half2half2(__ushort2half_rn((unsigned short)mn1))};
        *reinterpret_cast<uint2 *>(bmin + op_off(st >> 1, r) + (st & 1) * 8) = *reinterpret_cast<const uint2 *>(&m2[0]);
        if (st == 0) {
            dval[r] = h2f((uint16_t)(h.x & 0xFFFF));
            dval[TC_BN + r] = h2f((uint16_t)(h.x >> 16));
        }
    }
}

// The resident weight image: every stage's weight operand tile and every super-block's row-side tables, converted once
// (when the weight is prepared) into the shared-memory layout of the GEMM kernel.  grid (stages, row tiles), 256
// threads = (row, half) as the producer warps of the GEMM kernel.
template <int T>
__global__ void __launch_bounds__(TC_W_WARPS * 32) tc_weight_image_kernel(const WeightView w, uint8_t *__restrict__ img, uint8_t *__restrict__ side) {
    const uint32_t r = threadIdx.x >> 1, half = threadIdx.x & 1, it = blockIdx.x, tile = blockIdx.y;
    const uint32_t n_it = w.k / TC_KS, n_sb = w.k / 256, st = it % TC_STAGES, sb = it / TC_STAGES;
    const uint32_t row = min(tile * TC_BN + r, w.m - 1);  // rows past the edge repeat the last one; their results are not stored
    uint8_t *sd = side + ((size_t)tile * n_sb + sb) * TC_SIDE_BYTES;
    tc_convert_w<T>(tc_fetch_w<T>(w, row, half, it), r, half, st, img + ((size_t)tile * n_it + it) * TC_OP_BYTES, sd,
                    reinterpret_cast<float *>(sd + TC_MINOP_BYTES));
}

// The weight side of the wide variant's min GEMM: w[row][j] = dmin[row, j / 8] * min[row, j] * 2^s[row] for the k / 32
// blocks j of a row, as a high part (top 11 significant bits) and the remainder - both exact in f16, since the product
// of an f16 and a six-bit integer has 17 significant bits and 2^s[row] brings the row's largest entry to [2^14, 2^15).
// Tiles of 32 blocks in the operand layout, zero beyond k / 32; 2^-s[row] beside them.  grid = 128-row tiles, thread = row.
__global__ void __launch_bounds__(TC_BN) tc_weight_min_kernel(const WeightView w, uint8_t *__restrict__ wmin, float *__restrict__ rscale) {
    const uint32_t r = threadIdx.x, tile = blockIdx.x, n_sb = w.k / 256, n_mit = (w.k / 32 + TCW_MIN_J - 1) / TCW_MIN_J;
    const uint32_t row = min(tile * TC_BN + r, w.m - 1);
    float mx = 0.0f;
    for (uint32_t sb = 0; sb < n_sb; ++sb) {
        const uint4 h = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb_index(w, row, sb));
        const float dmin = fabsf(h2f((uint16_t)(h.x >> 16)));
        uint32_t sc, m0, m1;
        kq_quad(h, 0, sc, m0);
        kq_quad(h, 1, sc, m1);
        uint32_t mm = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) mm = max(mm, max((m0 >> (8 * i)) & 0xFF, (m1 >> (8 * i)) & 0xFF));
        const float v = dmin * (float)mm;
        mx = fmaxf(mx, v == v && v < 3.0e38f ? v : 0.0f);
    }
    int e = 0;
    if (mx > 0.0f) frexpf(mx, &e);  // mx < 2^e
    const float up = mx > 0.0f ? ldexpf(1.0f, 15 - e) : 1.0f;
    rscale[tile * TC_BN + r] = 1.0f / up;
    for (uint32_t mi = 0; mi < n_mit; ++mi) {
        uint8_t *hi_t = wmin + ((size_t)tile * n_mit + mi) * (2 * TCW_MINT_BYTES), *lo_t = hi_t + TCW_MINT_BYTES;
#pragma unroll 1
        for (uint32_t kc = 0; kc < TCW_MIN_J / 8; ++kc) {  // eight blocks = one super-block = one 16-byte k chunk
            const uint32_t sb = mi * (TCW_MIN_J / 8) + kc;
            __half2 hi2[4], lo2[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) hi2[q] = lo2[q] = __float2half2_rn(0.0f);
            if (sb < n_sb) {
                const uint4 h = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sb_index(w, row, sb));
                const float dm = h2f((uint16_t)(h.x >> 16)) * up;
                uint32_t sc, mp[2];
                kq_quad(h, 0, sc, mp[0]);
                kq_quad(h, 1, sc, mp[1]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float v[2], vh[2];
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const int b = 2 * q + t;
                        v[t] = dm * (float)((mp[b >> 2] >> (8 * (b & 3))) & 0xFF);
                        vh[t] = __uint_as_float(__float_as_uint(v[t]) & 0xFFFFE000u);
                    }
                    hi2[q] = __floats2half2_rn(vh[0], vh[1]);
                    lo2[q] = __floats2half2_rn(v[0] - vh[0], v[1] - vh[1]);
                }
            }
            *reinterpret_cast<uint4 *>(hi_t + op_off(kc, r)) = *reinterpret_cast<const uint4 *>(&hi2[0]);
            *reinterpret_cast<uint4 *>(lo_t + op_off(kc, r)) = *reinterpret_cast<const uint4 *>(&lo2[0]);
        }
    }
}

// The wide variant: one CTA = 128 tokens x 256 weight rows (two 128-row tiles of the weight image), for GEMMs with enough
// tiles to fill the device.  Against the 128 x 128 kernel the activation operands are fetched once for twice the MMAs
// (64 KB per 1024 tensor-pipe cycles instead of 48 KB per 512) and a stage hand-over pays for sixteen MMAs, which is what
// the 128-wide kernel is short of: its MMA thread waits a third of the time for operands.  TMEM then holds nothing but the
// two double-buffered accumulators (2 x 256 columns), so
//  * the running output lives in the epilogue threads' registers (thread = token lane x 128 rows), and
//  * the min term sum_b dmin * mn_b * (xs_b * A_b) is not accumulated per super-block but as ONE more GEMM over the k / 32
//    blocks of the whole row after the k loop - weights dmin * mn * 2^s[row] (tc_weight_min_kernel) and activations
//    g * xs_b * A_b, each as high and low f16 parts, three MMAs per step (the low x low product is below 2^-22) - into
//    the accumulator buffer of a virtual last super-block.
// Warps: 0 MMA issue (one thread), 1 operand loader (one thread), 2-9 epilogue.
__global__ void __launch_bounds__(TCW_THREADS, 1) gemm_tcw_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + TCW_TAIL_OFF);
    uint64_t *full_ab = bars, *empty_ab = bars + TCW_STAGES, *full_d = bars + 2 * TCW_STAGES, *empty_d = full_d + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TCW_STAGES + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const TcSub sub = tc_select(p);
    const uint32_t col0 = blockIdx.x * TC_BM, row0 = sub.by * 2 * TC_BN;
    const TcImage L = tc_image_layout(sub.m, p.k);
    const uint32_t n_sb = L.n_sb, n_it = L.n_it, n_mit = L.n_mit;
    if (tid == 0) {
        for (int s = 0; s < TCW_STAGES; ++s) {
            tma::mbar_init(full_ab + s, 1);   // the loader's expect_tx
            tma::mbar_init(empty_ab + s, 1);  // the commit of the stage's MMAs
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(full_d + b, 1);              // the commit after a super-block's last MMA
            tma::mbar_init(empty_d + b, TC_EPI_WARPS);  // every epilogue warp is done with the buffer and the slot
        }
        *abort_flag = 0;
        tma::mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TC_TMEM_COLS);
        tmem_relinquish();
    }
    pdl_trigger();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- MMA issue (one thread)
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(TC_BM, TC_BN);
            bool ok = true;
            uint32_t it = 0;
            for (uint32_t sb = 0; sb <= n_sb && ok; ++sb) {  // super-block n_sb is the min GEMM
                const uint32_t buf = sb & 1, d0 = tmem + buf * 2 * TC_BN;
                if (!tma::mbar_wait_blocking(empty_d + buf, ((sb >> 1) & 1) ^ 1, abort_flag, &g_tc_status, 2u)) break;
                tc_fence_after();
                const uint32_t n_st = sb < n_sb ? 4u : n_mit;
                for (uint32_t st = 0; st < n_st; ++st, ++it) {
                    const uint32_t s = it % TCW_STAGES;
                    if (!tma::mbar_wait_blocking(full_ab + s, (it / TCW_STAGES) & 1, abort_flag, &g_tc_status, 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t base = tma::smem_u32(tc_smem + s * TCW_STAGE_BYTES);
                    if (sb < n_sb) {
                        const uint32_t a_hi = base, a_lo = base + TC_OP_BYTES, b0 = a_lo + TC_OP_BYTES, b1 = b0 + TC_OP_BYTES;
#pragma unroll
                        for (uint32_t ks = 0; ks < TC_KS / 16; ++ks) {
                            const uint32_t o = 2 * ks * TC_KC_STRIDE;
                            const uint64_t ah = smem_desc(a_hi + o, TC_KC_STRIDE, 128), al = smem_desc(a_lo + o, TC_KC_STRIDE, 128);
                            const uint64_t bd0 = smem_desc(b0 + o, TC_KC_STRIDE, 128), bd1 = smem_desc(b1 + o, TC_KC_STRIDE, 128);
                            const uint32_t acc = (st | ks) != 0;
                            tc_mma_f16(d0, ah, bd0, idesc, acc);
                            tc_mma_f16(d0 + TC_BN, ah, bd1, idesc, acc);
                            tc_mma_f16(d0, al, bd0, idesc, 1);
                            tc_mma_f16(d0 + TC_BN, al, bd1, idesc, 1);
                        }
                    } else {
                        // min GEMM: [x high | x low | w high, w low of rows [0,128) | the same of rows [128,256)], 32 blocks = two steps
                        const uint32_t x_hi = base, x_lo = base + TCW_MINT_BYTES;
#pragma unroll
                        for (uint32_t ks = 0; ks < TCW_MIN_J / 16; ++ks) {
                            const uint32_t o = 2 * ks * TC_KC_STRIDE;
                            const uint64_t xh = smem_desc(x_hi + o, TC_KC_STRIDE, 128), xl = smem_desc(x_lo + o, TC_KC_STRIDE, 128);
#pragma unroll
                            for (uint32_t h = 0; h < 2; ++h) {
                                const uint32_t w_hi = base + (2 + 2 * h) * TCW_MINT_BYTES, w_lo = w_hi + TCW_MINT_BYTES;
                                const uint64_t wh = smem_desc(w_hi + o, TC_KC_STRIDE, 128), wl = smem_desc(w_lo + o, TC_KC_STRIDE, 128);
                                tc_mma_f16(d0 + h * TC_BN, xh, wh, idesc, (st | ks) != 0);
                                tc_mma_f16(d0 + h * TC_BN, xl, wh, idesc, 1);
                                tc_mma_f16(d0 + h * TC_BN, xh, wl, idesc, 1);
                            }
                        }
                    }
                    tc_commit(empty_ab + s);
                }
                if (ok) tc_commit(full_d + buf);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- operands: one thread asks for them (bulk asynchronous copies)
        if (lane == 0) {
            const uint32_t t0 = min(2 * sub.by, L.tiles - 1), t1 = min(2 * sub.by + 1, L.tiles - 1);  // (an odd last tile is read twice)
            const uint8_t *img = p.img + (size_t)blockIdx.x * n_it * (2 * TC_OP_BYTES);
            const uint8_t *w0 = sub.tc + (size_t)t0 * n_it * TC_OP_BYTES, *w1 = sub.tc + (size_t)t1 * n_it * TC_OP_BYTES;
            const uint8_t *sd0 = sub.tc + L.side + (size_t)t0 * n_sb * TC_SIDE_BYTES + TC_MINOP_BYTES;  // d[128] of a super-block
            const uint8_t *sd1 = sub.tc + L.side + (size_t)t1 * n_sb * TC_SIDE_BYTES + TC_MINOP_BYTES;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
                for (uint32_t st = 0; st < 4; ++st, ++it) {
                    const uint32_t s = it % TCW_STAGES;
                    if (!tma::mbar_wait_blocking(empty_ab + s, ((it / TCW_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 8u)) {
                        ok = false;
                        break;
                    }
                    // the d slot of this super-block was last read by the epilogue of super-block sb - 2
                    if (st == 0 && sb >= 2 && !tma::mbar_wait_blocking(empty_d + (sb & 1), ((sb - 2) >> 1) & 1, abort_flag, &g_tc_status, 8u)) {
                        ok = false;
                        break;
                    }
                    uint8_t *dst = tc_smem + s * TCW_STAGE_BYTES;
                    tma::mbar_expect_tx(full_ab + s, TCW_STAGE_BYTES + (st == 0 ? 2 * TC_BN * 4 : 0));
                    tma::bulk_g2s(dst, img + (size_t)it * (2 * TC_OP_BYTES), 2 * TC_OP_BYTES, full_ab + s);
                    tma::bulk_g2s(dst + 2 * TC_OP_BYTES, w0 + (size_t)it * TC_OP_BYTES, TC_OP_BYTES, full_ab + s);
                    tma::bulk_g2s(dst + 3 * TC_OP_BYTES, w1 + (size_t)it * TC_OP_BYTES, TC_OP_BYTES, full_ab + s);
                    if (st == 0) {
                        uint8_t *dv = tc_smem + TCW_DVAL_OFF + (sb & 1) * (2 * TC_BN * 4);
                        tma::bulk_g2s(dv, sd0 + (size_t)sb * TC_SIDE_BYTES, TC_BN * 4, full_ab + s);
                        tma::bulk_g2s(dv + TC_BN * 4, sd1 + (size_t)sb * TC_SIDE_BYTES, TC_BN * 4, full_ab + s);
                    }
                }
            }
            const uint8_t *xm = p.xm + (size_t)blockIdx.x * n_mit * (2 * TCW_MINT_BYTES);
            const uint8_t *m0 = sub.tc + L.wmin + (size_t)t0 * n_mit * (2 * TCW_MINT_BYTES), *m1 = sub.tc + L.wmin + (size_t)t1 * n_mit * (2 * TCW_MINT_BYTES);
            for (uint32_t mi = 0; mi < n_mit && ok; ++mi, ++it) {
                const uint32_t s = it % TCW_STAGES;
                if (!tma::mbar_wait_blocking(empty_ab + s, ((it / TCW_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 8u)) break;
                uint8_t *dst = tc_smem + s * TCW_STAGE_BYTES;
                tma::mbar_expect_tx(full_ab + s, 6 * TCW_MINT_BYTES + (mi == 0 ? 2 * TC_BN * 4 : 0));
                tma::bulk_g2s(dst, xm + (size_t)mi * (2 * TCW_MINT_BYTES), 2 * TCW_MINT_BYTES, full_ab + s);
                tma::bulk_g2s(dst + 2 * TCW_MINT_BYTES, m0 + (size_t)mi * (2 * TCW_MINT_BYTES), 2 * TCW_MINT_BYTES, full_ab + s);
                tma::bulk_g2s(dst + 4 * TCW_MINT_BYTES, m1 + (size_t)mi * (2 * TCW_MINT_BYTES), 2 * TCW_MINT_BYTES, full_ab + s);
                if (mi == 0) {  // 2^-s of the CTA's rows (read by the epilogue after the min GEMM)
                    tma::bulk_g2s(tc_smem + TCW_RS_OFF, sub.tc + L.rscale + (size_t)t0 * TC_BN * 4, TC_BN * 4, full_ab + s);
                    tma::bulk_g2s(tc_smem + TCW_RS_OFF + TC_BN * 4, sub.tc + L.rscale + (size_t)t1 * TC_BN * 4, TC_BN * 4, full_ab + s);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: thread = (token lane, 128 rows of one image tile)
        const uint32_t e = warp - 2, quad = warp & 3, hh = e >> 2;  // a warp reaches TMEM lanes [32 (warp % 4), +32)
        const uint32_t tl = quad * 32 + lane;
        const uint32_t lane_addr = tmem + ((quad * 32) << 16) + hh * TC_BN;
        float acc[TC_BN];
#pragma unroll
        for (int i = 0; i < TC_BN; ++i) acc[i] = 0.0f;
        float ginv = 1.0f;
        bool ok = true;
        for (uint32_t sb = 0; sb <= n_sb && ok; ++sb) {
            const uint32_t buf = sb & 1;
            if (!tma::mbar_wait_blocking(full_d + buf, (sb >> 1) & 1, abort_flag, &g_tc_status, 16u)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (sb == 0) ginv = __ldg(p.ginv + col0 + tl);
            // per super-block: out += d[row] * D / g; after the min GEMM: out -= 2^-s[row] * Dmin / g
            const float *fac = sb < n_sb ? reinterpret_cast<const float *>(tc_smem + TCW_DVAL_OFF + buf * (2 * TC_BN * 4)) + hh * TC_BN
                                         : reinterpret_cast<const float *>(tc_smem + TCW_RS_OFF) + hh * TC_BN;
            const float gs = sb < n_sb ? ginv : -ginv;
#pragma unroll
            for (uint32_t c = 0; c < TC_BN / 32; ++c) {
                uint32_t v0[16], v1[16];
                tmem_ld16(lane_addr + buf * 2 * TC_BN + c * 32, v0);
                tmem_ld16(lane_addr + buf * 2 * TC_BN + c * 32 + 16, v1);
                tmem_wait_ld();
                const float4 *fq = reinterpret_cast<const float4 *>(fac + c * 32);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    const float4 f = fq[q4];
                    const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = q4 * 4 + i;
                        const float dd = __uint_as_float(j < 16 ? v0[j & 15] : v1[j & 15]);
                        acc[c * 32 + j] = fmaf(fv[i] * dd, gs, acc[c * 32 + j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(empty_d + buf);  // the accumulator buffer and the d slot are free again
        }
        if (ok && col0 + tl < p.n) {
            // ---- the thread's 128 cells -> global memory: cell (row i, token j) at out[i * ldy + j * ldc]
            const uint32_t r0 = row0 + hh * TC_BN;
            float *o = sub.out + (size_t)r0 * p.ldy + (size_t)(col0 + tl) * sub.ldc;
            if (p.ldy == 1 && r0 + TC_BN <= sub.m && ((uintptr_t)o & 15) == 0) {  // token-major output: 512 contiguous bytes
#pragma unroll
                for (int i = 0; i < TC_BN / 4; ++i) {
                    float4 v = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                    float4 *o4 = reinterpret_cast<float4 *>(o) + i;
                    if (p.epilogue == EPI_ADD) {
                        const float4 c = *o4;
                        v = make_float4(__fadd_rn(c.x, v.x), __fadd_rn(c.y, v.y), __fadd_rn(c.z, v.z), __fadd_rn(c.w, v.w));
                    }
                    *o4 = v;
                }
            } else {
#pragma unroll
                for (int i = 0; i < TC_BN; ++i)
                    if (r0 + i < sub.m) {
                        float *oi = o + (size_t)i * p.ldy;
                        *oi = p.epilogue == EPI_ADD ? __fadd_rn(*oi, acc[i]) : acc[i];
                    }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TC_TMEM_COLS);
    }
}

template <int T, bool IMG>
__global__ void __launch_bounds__(IMG ? TC_THREADS_IMG : TC_THREADS, 1) gemm_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t *slots = tc_smem + TC_STAGES * TC_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + TC_TAIL_OFF);
    uint64_t *full_ab = bars, *empty_ab = bars + TC_STAGES, *full_d = bars + 2 * TC_STAGES, *empty_d = full_d + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TC_STAGES + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const TcSub sub = tc_select(p);
    const uint32_t col0 = blockIdx.x * TC_BM, row0 = sub.by * TC_BN;
    const uint32_t n_sb = p.k / 256, n_it = n_sb * TC_STAGES;
    constexpr int TC_LOADER_WARP = IMG ? 1 : TC_W_WARPS + 1;  // the epilogue warps follow it
    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            tma::mbar_init(full_ab + s, IMG ? 1 : TC_W_WARPS * 32 + 1);  // (every weight-producer thread +) the loader's expect_tx
            tma::mbar_init(empty_ab + s, 1);                              // the commit of the stage's MMAs
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(full_d + b, 1);              // the commit after a super-block's last MMA
            tma::mbar_init(empty_d + b, TC_EPI_WARPS);  // every epilogue warp is done with the buffer, Dm and the slot
        }
        *abort_flag = 0;
        tma::mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TC_TMEM_COLS);
        tmem_relinquish();
    }
    pdl_trigger();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- MMA issue (one thread)
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(TC_BM, TC_BN);
            bool ok = true;
            for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
                const uint32_t buf = sb & 1;
                // the epilogue has left this D buffer (super-block sb - 2)
                if (!tma::mbar_wait_blocking(empty_d + buf, ((sb >> 1) & 1) ^ 1, abort_flag, &g_tc_status, 2u)) break;
                tc_fence_after();
                for (uint32_t st = 0; st < (uint32_t)TC_STAGES; ++st) {
                    const uint32_t it = sb * TC_STAGES + st;
                    if (!tma::mbar_wait_blocking(full_ab + st, (it / TC_STAGES) & 1, abort_flag, &g_tc_status, 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_hi = tma::smem_u32(tc_smem + st * TC_STAGE_BYTES), a_lo = a_hi + TC_OP_BYTES, b_base = a_lo + TC_OP_BYTES;
#pragma unroll
                    for (uint32_t ks = 0; ks < TC_KS / 16; ++ks) {
                        const uint64_t bd = smem_desc(b_base + 2 * ks * TC_KC_STRIDE, TC_KC_STRIDE, 128);
                        tc_mma_f16(tmem + buf * TC_BN, smem_desc(a_hi + 2 * ks * TC_KC_STRIDE, TC_KC_STRIDE, 128), bd, idesc, (st | ks) != 0);
                        tc_mma_f16(tmem + buf * TC_BN, smem_desc(a_lo + 2 * ks * TC_KC_STRIDE, TC_KC_STRIDE, 128), bd, idesc, 1);
                    }
                    if (st + 1 == (uint32_t)TC_STAGES) {
                        // the super-block's min term.  Without the weight image Dm has one buffer (the fourth TMEM region holds
                        // the running output): the epilogue must have read super-block sb - 1's
                        if (!IMG && sb && !tma::mbar_wait_blocking(empty_d + (buf ^ 1), ((sb - 1) >> 1) & 1, abort_flag, &g_tc_status, 2u)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t slot = tma::smem_u32(slots + buf * TC_SLOT_BYTES);
                        tc_mma_f16(tmem + (IMG ? 2 + buf : 2) * TC_BN, smem_desc(slot, TC_KC_STRIDE, 128), smem_desc(slot + TC_MINOP_BYTES, TC_KC_STRIDE, 128),
                                   idesc, 0);
                    }
                    tc_commit(empty_ab + st);
                }
                if (ok) tc_commit(full_d + buf);
            }
        }
    } else if (!IMG && warp <= TC_W_WARPS) {
        // ---------------------------------------------------------------- weight operand: thread = (weight row, half of the stage's bytes)
        const uint32_t r = (tid - 32) >> 1, half = (tid - 32) & 1;
        const uint32_t row = min(row0 + r, sub.m - 1);  // rows past the edge repeat the last one; their results are not stored
        // the raw bytes of a stage are fetched one stage ahead of their conversion (a thread converts every stage itself:
        // a global round trip per stage would bound the pipeline)
        TcRawW nxt = tc_fetch_w<T>(p.w, row, half, 0);
        for (uint32_t it = 0; it < n_it; ++it) {
            const uint32_t st = it % TC_STAGES, sb = it / TC_STAGES;
            const TcRawW cur = nxt;
            if (it + 1 < n_it) nxt = tc_fetch_w<T>(p.w, row, half, it + 1);
            if (!tma::mbar_wait_blocking(empty_ab + st, ((it / TC_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 4u)) break;
            // the slot of this super-block (tables, min operand) was last used by super-block sb - 2
            if (st == 0 && sb >= 2 && !tma::mbar_wait_blocking(empty_d + (sb & 1), ((sb - 2) >> 1) & 1, abort_flag, &g_tc_status, 4u)) break;
            uint8_t *slot = slots + (sb & 1) * TC_SLOT_BYTES;
            tc_convert_w<T>(cur, r, half, st, tc_smem + st * TC_STAGE_BYTES + 2 * TC_OP_BYTES, slot + TC_MINOP_BYTES,
                            reinterpret_cast<float *>(slot + 2 * TC_MINOP_BYTES));
            fence_async_smem();
            tma::mbar_arrive(full_ab + st);
        }
    } else if (warp == TC_LOADER_WARP) {
        // ---------------------------------------------------------------- activation operands: one thread asks for them
        // (bulk asynchronous copies of the tiles tc_token_image_kernel wrote in this layout; 32 KB per stage, and the token
        // side of the min operand with a super-block's first stage)
        if (lane == 0) {
            const uint8_t *img = p.img + (size_t)blockIdx.x * n_it * (2 * TC_OP_BYTES);
            const uint8_t *img_min = p.img_min + (size_t)blockIdx.x * n_sb * TC_MINOP_BYTES;
            // the resident weight image of this row tile (null without one): operand tiles, then the per-super-block sides
            const uint32_t tiles_m = (sub.m + TC_BN - 1) / TC_BN;
            const uint8_t *wimg = IMG ? sub.tc + (size_t)sub.by * n_it * TC_OP_BYTES : nullptr;
            const uint8_t *wside = IMG ? sub.tc + (size_t)tiles_m * n_it * TC_OP_BYTES + (size_t)sub.by * n_sb * TC_SIDE_BYTES : nullptr;
            for (uint32_t it = 0; it < n_it; ++it) {
                const uint32_t st = it % TC_STAGES, sb = it / TC_STAGES;
                if (!tma::mbar_wait_blocking(empty_ab + st, ((it / TC_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 8u)) break;
                if (st == 0 && sb >= 2 && !tma::mbar_wait_blocking(empty_d + (sb & 1), ((sb - 2) >> 1) & 1, abort_flag, &g_tc_status, 8u)) break;
                tma::mbar_expect_tx(full_ab + st, (IMG ? 3 : 2) * TC_OP_BYTES + (st == 0 ? TC_MINOP_BYTES + (IMG ? TC_SIDE_BYTES : 0) : 0));
                tma::bulk_g2s(tc_smem + st * TC_STAGE_BYTES, img + (size_t)it * (2 * TC_OP_BYTES), 2 * TC_OP_BYTES, full_ab + st);
                if (IMG) tma::bulk_g2s(tc_smem + st * TC_STAGE_BYTES + 2 * TC_OP_BYTES, wimg + (size_t)it * TC_OP_BYTES, TC_OP_BYTES, full_ab + st);
                if (st == 0) {
                    uint8_t *slot = slots + (sb & 1) * TC_SLOT_BYTES;
                    tma::bulk_g2s(slot, img_min + (size_t)sb * TC_MINOP_BYTES, TC_MINOP_BYTES, full_ab + st);
                    if (IMG) tma::bulk_g2s(slot + TC_MINOP_BYTES, wside + (size_t)sb * TC_SIDE_BYTES, TC_SIDE_BYTES, full_ab + st);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: thread = (token lane, 64 rows)
        const uint32_t e = warp - (TC_LOADER_WARP + 1), quad = warp & 3, ch = e >> 2;  // a warp reaches TMEM lanes [32 (warp % 4), +32)
        const uint32_t tl = quad * 32 + lane;                                                    // token lane
        const uint32_t lane_addr = tmem + ((quad * 32) << 16);
        float ginv = 1.0f;
        bool ok = true;
        if constexpr (IMG) {
            // The running output of the thread's 64 rows stays in registers (this variant has no producer warps, so the
            // register file has the room), D and Dm are both double-buffered in TMEM: a super-block costs two TMEM reads
            // per cell and the MMAs of the next super-block never wait for this one's epilogue.
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
            for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
                const uint32_t buf = sb & 1;
                if (!tma::mbar_wait_blocking(full_d + buf, (sb >> 1) & 1, abort_flag, &g_tc_status, 16u)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (sb == 0) ginv = __ldg(p.ginv + col0 + tl);
                const float *dval = reinterpret_cast<const float *>(slots + buf * TC_SLOT_BYTES + 2 * TC_MINOP_BYTES);
#pragma unroll
                for (uint32_t c2 = 0; c2 < 2; ++c2) {  // 32 rows per round: four loads in flight
                    const uint32_t col = ch * 64 + c2 * 32;
                    uint32_t d0[16], m0[16], d1[16], m1[16];
                    tmem_ld16(lane_addr + buf * TC_BN + col, d0);
                    tmem_ld16(lane_addr + (2 + buf) * TC_BN + col, m0);
                    tmem_ld16(lane_addr + buf * TC_BN + col + 16, d1);
                    tmem_ld16(lane_addr + (2 + buf) * TC_BN + col + 16, m1);
                    tmem_wait_ld();
                    const float4 *dq = reinterpret_cast<const float4 *>(dval + col), *mq = dq + TC_BN / 4;
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        const float4 dv = dq[q4], mv = mq[q4];
                        const float dvv[4] = {dv.x, dv.y, dv.z, dv.w}, mvv[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int j = q4 * 4 + i;
                            const float dd = __uint_as_float(j < 16 ? d0[j & 15] : d1[j & 15]), mm = __uint_as_float(j < 16 ? m0[j & 15] : m1[j & 15]);
                            const float t = fmaf(dvv[i], dd, -(mvv[i] * mm));
                            acc[c2 * 32 + j] = fmaf(t, ginv, acc[c2 * 32 + j]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(empty_d + buf);  // D and Dm of this parity and the slot's tables are free again
            }
            if (ok && col0 + tl < p.n) {
                // ---- the thread's 64 cells -> global memory: cell (row i, token j) at out[i * ldy + j * ldc]
                float *o = sub.out + (size_t)(row0 + ch * 64) * p.ldy + (size_t)(col0 + tl) * sub.ldc;
                if (p.ldy == 1 && row0 + ch * 64 + 64 <= sub.m && ((uintptr_t)o & 15) == 0) {  // token-major output: 256 contiguous bytes
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float4 v = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                        float4 *o4 = reinterpret_cast<float4 *>(o) + i;
                        if (p.epilogue == EPI_ADD) {
                            const float4 c = *o4;
                            v = make_float4(__fadd_rn(c.x, v.x), __fadd_rn(c.y, v.y), __fadd_rn(c.z, v.z), __fadd_rn(c.w, v.w));
                        }
                        *o4 = v;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i)
                        if (row0 + ch * 64 + i < sub.m) {
                            float *oi = o + (size_t)i * p.ldy;
                            *oi = p.epilogue == EPI_ADD ? __fadd_rn(*oi, acc[i]) : acc[i];
                        }
                }
            }
            ok = false;  // (stored already: skip the TMEM-resident path below)
        }
        for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
            const uint32_t buf = sb & 1;
            if (!tma::mbar_wait_blocking(full_d + buf, (sb >> 1) & 1, abort_flag, &g_tc_status, 16u)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (sb == 0) ginv = __ldg(p.ginv + col0 + tl);
            const float *dval = reinterpret_cast<const float *>(slots + buf * TC_SLOT_BYTES + 2 * TC_MINOP_BYTES);
            // out[row] += (d[row] * D - dmin[row] * Dm) / g, the running sum in TMEM
#pragma unroll 1
            for (uint32_t c4 = 0; c4 < 4; ++c4) {
                const uint32_t col = ch * 64 + c4 * 16;
                uint32_t dreg[16], mreg[16], oreg[16];
                tmem_ld16(lane_addr + buf * TC_BN + col, dreg);
                tmem_ld16(lane_addr + 2 * TC_BN + col, mreg);
                if (sb) {
                    tmem_ld16(lane_addr + 3 * TC_BN + col, oreg);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) oreg[i] = 0u;
                }
                tmem_wait_ld();
                const float4 *dq = reinterpret_cast<const float4 *>(dval + col), *mq = dq + TC_BN / 4;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float4 dv = dq[q4], mv = mq[q4];
                    const float dvv[4] = {dv.x, dv.y, dv.z, dv.w}, mvv[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = q4 * 4 + i;
                        const float t = fmaf(dvv[i], __uint_as_float(dreg[j]), -(mvv[i] * __uint_as_float(mreg[j])));
                        oreg[j] = __float_as_uint(fmaf(t, ginv, __uint_as_float(oreg[j])));
                    }
                }
                tmem_st16(lane_addr + 3 * TC_BN + col, oreg);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(empty_d + buf);  // D buffer, Dm and the slot's tables are free again
        }
        if (ok) {
            // ---- the tile -> global memory: cell (row i, token j) at out[i * ldy + j * ldc]
            const bool tok_ok = col0 + tl < p.n;
#pragma unroll 1
            for (uint32_t c4 = 0; c4 < 4; ++c4) {
                uint32_t oreg[16];
                tmem_ld16(lane_addr + 3 * TC_BN + ch * 64 + c4 * 16, oreg);
                tmem_wait_ld();
                if (tok_ok) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t row = row0 + ch * 64 + c4 * 16 + i;
                        if (row < sub.m) {
                            float *o = sub.out + (size_t)row * p.ldy + (size_t)(col0 + tl) * sub.ldc;
                            const float v = __uint_as_float(oreg[i]);
                            *o = p.epilogue == EPI_ADD ? __fadd_rn(*o, v) : v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TC_TMEM_COLS);
    }
}

template <int T, bool IMG>
int32_t launch_tc_typed(const TcParams &p, uint32_t y_tiles, cudaStream_t st) {
    static thread_local int configured_dev = -1;  // (one per instantiation)
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<T, IMG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
        configured_dev = dev;
    }
    const dim3 grid((p.n + TC_BM - 1) / TC_BM, y_tiles);
    count_launch();
    return check_cuda(launch_k(gemm_tc_kernel<T, IMG>, grid, dim3(IMG ? TC_THREADS_IMG : TC_THREADS), (size_t)TC_SMEM_BYTES, st, p),
                      "gemm (tcgen05) launch");
}

// ---- Q6_K ---------------------------------------------------------------------------------------------------------
// w = d * sc * (q - 32) with an int8 scale per 16 elements: B = sc * (q - 32) reaches 4096 in magnitude, one bit more than
// f16 holds exactly.  The image therefore keeps B as TWO exact f16 operands, B with its lowest bit cleared (an even
// integer up to 4096) and that bit (0 or 1); per k-step the kernel issues three MMAs into one accumulator - even part x
// activations high, even part x activations low, low bit x activations high (low bit x activations low is below 2^-22
// of the sum) - and the epilogue is out += d * D / g per super-block (Q6_K has no min term).  128 tokens x 128 rows per
// CTA, stages of 32 k (activations 2 x 8 KB out of the 64-k tiles of tc_token_image_kernel, weights 16 KB), six stages.
constexpr int TC6_KS = 32, TC6_STAGES = 6;
constexpr uint32_t TC6_HALF = TC_OP_BYTES / 2;                 // one operand tile of a 32-k stage: 8 KB
constexpr uint32_t TC6_STAGE_BYTES = 4 * TC6_HALF;             // A high, A low, B even, B low bit
constexpr uint32_t TC6_DVAL_OFF = TC6_STAGES * TC6_STAGE_BYTES;
constexpr uint32_t TC6_TAIL_OFF = TC6_DVAL_OFF + 2 * TC_BN * 4;
constexpr uint32_t TC6_SMEM_BYTES = TC6_TAIL_OFF + 256;
constexpr uint32_t TC6_TMEM_COLS = 256;

// Image of a Q6_K weight: per (128-row tile, 32-k stage) [even part 8 KB | low bit 8 KB], then per (tile, super-block)
// d[128].  grid (k / 32, tiles), thread = row.
__global__ void __launch_bounds__(TC_BN) tc_weight_image6_kernel(const WeightView w, uint8_t *__restrict__ img, float *__restrict__ dvals) {
    const uint32_t r = threadIdx.x, xb = blockIdx.x, tile = blockIdx.y, n_it = w.k / TC6_KS, n_sb = w.k / 256;
    const uint32_t row = min(tile * TC_BN + r, w.m - 1);
    const uint32_t t = xb >> 2, g = xb & 3, sb = xb >> 3;  // 128-weight task, 32-element group of the task, super-block
    const size_t sbi = sb_index(w, row, sb);
    const uint4 sc16 = __ldg(reinterpret_cast<const uint4 *>(w.hdr) + sbi);
    const uint32_t scw[4] = {sc16.x, sc16.y, sc16.z, sc16.w};
    uint8_t *even_t = img + ((size_t)tile * n_it + xb) * (2 * TC6_HALF), *low_t = even_t + TC6_HALF;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        // elements [16 half, +16) of the group: low (groups 0, 1) or high (groups 2, 3) nibbles of piece 2 (g % 2) + half,
        // bits 2 g, 2 g + 1 of the task's high-bit piece `half`, scale 8 (t % 2) + 2 g + half of the super-block
        const uint4 pc = __ldg(reinterpret_cast<const uint4 *>(q_piece_ptr(w, row, 4, t * 4 + 2 * (g & 1) + half)));
        const uint4 hb = __ldg(reinterpret_cast<const uint4 *>(w.qh + sbi * 64 + (t & 1) * 32 + half * 16));
        const uint32_t si = (t & 1) * 8 + 2 * g + half;
        const int sc = (int)(int8_t)(scw[si >> 2] >> (8 * (si & 3)));
        const uint32_t pw[4] = {pc.x, pc.y, pc.z, pc.w}, hw[4] = {hb.x, hb.y, hb.z, hb.w};
        __align__(16) __half ev[16], lw[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t byte = (pw[j >> 2] >> (8 * (j & 3))) & 0xFF, hbyte = (hw[j >> 2] >> (8 * (j & 3))) & 0xFF;
            const int q = (int)((g < 2 ? byte & 0xF : byte >> 4) | (((hbyte >> (2 * g)) & 3) << 4)) - 32;
            const int b = sc * q, b0 = b & 1;
            ev[j] = __int2half_rn(b - b0);
            lw[j] = __int2half_rn(b0);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            *reinterpret_cast<uint4 *>(even_t + op_off(2 * half + c, r)) = *reinterpret_cast<const uint4 *>(&ev[8 * c]);
            *reinterpret_cast<uint4 *>(low_t + op_off(2 * half + c, r)) = *reinterpret_cast<const uint4 *>(&lw[8 * c]);
        }
    }
    if ((xb & 7) == 0) dvals[((size_t)tile * n_sb + sb) * TC_BN + r] = h2f(__ldg(reinterpret_cast<const uint16_t *>(w.d) + sbi));
}

__global__ void __launch_bounds__(TC_THREADS_IMG, 1) gemm_tc6_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + TC6_TAIL_OFF);
    uint64_t *full_ab = bars, *empty_ab = bars + TC6_STAGES, *full_d = bars + 2 * TC6_STAGES, *empty_d = full_d + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TC6_STAGES + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t col0 = blockIdx.x * TC_BM, row0 = blockIdx.y * TC_BN;
    const uint32_t n_sb = p.k / 256, n_it = p.k / TC6_KS, tiles_m = (p.m + TC_BN - 1) / TC_BN;
    if (tid == 0) {
        for (int s = 0; s < TC6_STAGES; ++s) {
            tma::mbar_init(full_ab + s, 1);
            tma::mbar_init(empty_ab + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(full_d + b, 1);
            tma::mbar_init(empty_d + b, TC_EPI_WARPS);
        }
        *abort_flag = 0;
        tma::mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TC6_TMEM_COLS);
        tmem_relinquish();
    }
    pdl_trigger();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {  // ---- MMA issue
            const uint32_t idesc = tc_idesc(TC_BM, TC_BN);
            bool ok = true;
            uint32_t it = 0;
            for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
                const uint32_t buf = sb & 1, d0 = tmem + buf * TC_BN;
                if (!tma::mbar_wait_blocking(empty_d + buf, ((sb >> 1) & 1) ^ 1, abort_flag, &g_tc_status, 2u)) break;
                tc_fence_after();
                for (uint32_t st = 0; st < 8; ++st, ++it) {
                    const uint32_t s = it % TC6_STAGES;
                    if (!tma::mbar_wait_blocking(full_ab + s, (it / TC6_STAGES) & 1, abort_flag, &g_tc_status, 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_hi = tma::smem_u32(tc_smem + s * TC6_STAGE_BYTES), a_lo = a_hi + TC6_HALF, b_ev = a_lo + TC6_HALF, b_lo = b_ev + TC6_HALF;
#pragma unroll
                    for (uint32_t ks = 0; ks < TC6_KS / 16; ++ks) {
                        const uint32_t o = 2 * ks * TC_KC_STRIDE;
                        const uint64_t ah = smem_desc(a_hi + o, TC_KC_STRIDE, 128), be = smem_desc(b_ev + o, TC_KC_STRIDE, 128);
                        tc_mma_f16(d0, ah, be, idesc, (st | ks) != 0);
                        tc_mma_f16(d0, smem_desc(a_lo + o, TC_KC_STRIDE, 128), be, idesc, 1);
                        tc_mma_f16(d0, ah, smem_desc(b_lo + o, TC_KC_STRIDE, 128), idesc, 1);
                    }
                    tc_commit(empty_ab + s);
                }
                if (ok) tc_commit(full_d + buf);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- operands (bulk asynchronous copies)
            const uint8_t *img = p.img + (size_t)blockIdx.x * (p.k / TC_KS) * (2 * TC_OP_BYTES);
            const uint8_t *wimg = p.w.tc + (size_t)blockIdx.y * n_it * (2 * TC6_HALF);
            const uint8_t *dv = p.w.tc + (size_t)tiles_m * n_it * (2 * TC6_HALF) + (size_t)blockIdx.y * n_sb * (TC_BN * 4);
            for (uint32_t it = 0; it < n_it; ++it) {
                const uint32_t s = it % TC6_STAGES, sb = it >> 3, st = it & 7;
                if (!tma::mbar_wait_blocking(empty_ab + s, ((it / TC6_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 8u)) break;
                if (st == 0 && sb >= 2 && !tma::mbar_wait_blocking(empty_d + (sb & 1), ((sb - 2) >> 1) & 1, abort_flag, &g_tc_status, 8u)) break;
                uint8_t *dst = tc_smem + s * TC6_STAGE_BYTES;
                // the 64-k activation stage it / 2 holds [high 16 KB | low 16 KB]; its k half it % 2 is 8 contiguous KB of each
                const uint8_t *a = img + (size_t)(it >> 1) * (2 * TC_OP_BYTES) + (it & 1) * TC6_HALF;
                tma::mbar_expect_tx(full_ab + s, TC6_STAGE_BYTES + (st == 0 ? TC_BN * 4 : 0));
                tma::bulk_g2s(dst, a, TC6_HALF, full_ab + s);
                tma::bulk_g2s(dst + TC6_HALF, a + TC_OP_BYTES, TC6_HALF, full_ab + s);
                tma::bulk_g2s(dst + 2 * TC6_HALF, wimg + (size_t)it * (2 * TC6_HALF), 2 * TC6_HALF, full_ab + s);
                if (st == 0) tma::bulk_g2s(tc_smem + TC6_DVAL_OFF + (sb & 1) * (TC_BN * 4), dv + (size_t)sb * (TC_BN * 4), TC_BN * 4, full_ab + s);
            }
        }
    } else {
        // ---- epilogue: thread = (token lane, 64 rows), the running output in registers
        const uint32_t e = warp - 2, quad = warp & 3, ch = e >> 2;
        const uint32_t tl = quad * 32 + lane;
        const uint32_t lane_addr = tmem + ((quad * 32) << 16);
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
        float ginv = 1.0f;
        bool ok = true;
        for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
            const uint32_t buf = sb & 1;
            if (!tma::mbar_wait_blocking(full_d + buf, (sb >> 1) & 1, abort_flag, &g_tc_status, 16u)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (sb == 0) ginv = __ldg(p.ginv + col0 + tl);
            const float *dval = reinterpret_cast<const float *>(tc_smem + TC6_DVAL_OFF + buf * (TC_BN * 4));
#pragma unroll
            for (uint32_t c2 = 0; c2 < 2; ++c2) {
                const uint32_t col = ch * 64 + c2 * 32;
                uint32_t v0[16], v1[16];
                tmem_ld16(lane_addr + buf * TC_BN + col, v0);
                tmem_ld16(lane_addr + buf * TC_BN + col + 16, v1);
                tmem_wait_ld();
                const float4 *dq = reinterpret_cast<const float4 *>(dval + col);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    const float4 dv = dq[q4];
                    const float dvv[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = q4 * 4 + i;
                        const float dd = __uint_as_float(j < 16 ? v0[j & 15] : v1[j & 15]);
                        acc[c2 * 32 + j] = fmaf(dvv[i] * dd, ginv, acc[c2 * 32 + j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(empty_d + buf);
        }
        if (ok && col0 + tl < p.n) {
            float *o = p.out + (size_t)(row0 + ch * 64) * p.ldy + (size_t)(col0 + tl) * p.ldc;
            if (p.ldy == 1 && row0 + ch * 64 + 64 <= p.m && ((uintptr_t)o & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float4 v = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                    float4 *o4 = reinterpret_cast<float4 *>(o) + i;
                    if (p.epilogue == EPI_ADD) {
                        const float4 c = *o4;
                        v = make_float4(__fadd_rn(c.x, v.x), __fadd_rn(c.y, v.y), __fadd_rn(c.z, v.z), __fadd_rn(c.w, v.w));
                    }
                    *o4 = v;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (row0 + ch * 64 + i < p.m) {
                        float *oi = o + (size_t)i * p.ldy;
                        *oi = p.epilogue == EPI_ADD ? __fadd_rn(*oi, acc[i]) : acc[i];
                    }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TC6_TMEM_COLS);
    }
}

int32_t launch_tc6(const TcParams &p, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc6_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC6_SMEM_BYTES));
        configured_dev = dev;
    }
    const dim3 grid((p.n + TC_BM - 1) / TC_BM, (p.m + TC_BN - 1) / TC_BN);
    count_launch();
    return check_cuda(launch_k(gemm_tc6_kernel, grid, dim3(TC_THREADS_IMG), (size_t)TC6_SMEM_BYTES, st, p), "gemm (tcgen05, Q6_K) launch");
}

int32_t launch_tc_wide(const TcParams &p, uint32_t y_tiles, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemm_tcw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TCW_SMEM_BYTES));
        configured_dev = dev;
    }
    const dim3 grid((p.n + TC_BM - 1) / TC_BM, y_tiles);
    count_launch();
    return check_cuda(launch_k(gemm_tcw_kernel, grid, dim3(TCW_THREADS), (size_t)TCW_SMEM_BYTES, st, p), "gemm (tcgen05, wide) launch");
}

}  // namespace

// The resident tensor-core image of a Q4_K / Q5_K weight: sc * q as f16 in the GEMM kernel's shared-memory tile layout
// (2 bytes per weight) plus 40 bytes per (row, super-block) of min operand and super-scales.  With it the prefill GEMM
// has no conversion work left: every stage is three bulk copies and eight MMAs.  Built once; a weight that is not this
// kernel's case, CERA_CUDA_TC_IMAGE=0, or a device without room leave the weight as it is (the GEMM then converts on
// the fly).  *built (optional) reports whether the weight now has an image.
int32_t weight_prepare_tc(cera_cuda_weight *w, bool *built) {
    if (built) *built = false;
    if (!w) return fail(CERA_CUDA_ERR_BAD_ARG, "weight_prepare_gemm: null weight");
    if (w->v.tc) {
        if (built) *built = true;
        return CERA_CUDA_OK;
    }
    static const bool off = [] {
        const char *e = getenv("CERA_CUDA_TC_IMAGE");
        return e && strcmp(e, "0") == 0;
    }();
    const WeightView &v = w->v;
    if (off || v.k % 256 || v.ilv != 8 || (v.type != CERA_TYPE_Q4_K && v.type != CERA_TYPE_Q5_K && v.type != CERA_TYPE_Q6_K)) return CERA_CUDA_OK;
    TcImage L = tc_image_layout(v.m, v.k);
    const bool q6 = v.type == CERA_TYPE_Q6_K;
    if (q6) L.total = (size_t)L.tiles * (v.k / TC6_KS) * (2 * TC6_HALF) + (size_t)L.tiles * L.n_sb * (TC_BN * 4);  // 4 bytes per weight + d
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != w->device) cudaSetDevice(w->device);
    size_t free_b = 0, total_b = 0;
    int32_t rc = CERA_CUDA_OK;
    void *img = nullptr;
    // keep a margin for KV caches and prefill scratch: the image is an accelerator, not a requirement
    if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && free_b > L.total + (4ull << 30) && cudaMalloc(&img, L.total) == cudaSuccess) {
        const dim3 grid(L.n_it, L.tiles);
        uint8_t *b = (uint8_t *)img;
        if (q6) {
            tc_weight_image6_kernel<<<dim3(v.k / TC6_KS, L.tiles), TC_BN>>>(
                v, b, reinterpret_cast<float *>(b + (size_t)L.tiles * (v.k / TC6_KS) * (2 * TC6_HALF)));
        } else if (v.type == CERA_TYPE_Q4_K)
            tc_weight_image_kernel<CERA_TYPE_Q4_K><<<grid, TC_W_WARPS * 32>>>(v, b, b + L.side);
        else
            tc_weight_image_kernel<CERA_TYPE_Q5_K><<<grid, TC_W_WARPS * 32>>>(v, b, b + L.side);
        if (!q6) tc_weight_min_kernel<<<L.tiles, TC_BN>>>(v, b + L.wmin, reinterpret_cast<float *>(b + L.rscale));  // (the header layout is the same for both types)
        count_launch();
        count_launch();
        rc = check_cuda(cudaGetLastError(), "weight image launch");
        if (rc == CERA_CUDA_OK) rc = check_cuda(cudaDeviceSynchronize(), "weight image");
        if (rc == CERA_CUDA_OK) {
            w->tc_image = img;
            w->tc_bytes = L.total;
            w->v.tc = (const uint8_t *)img;
            if (built) *built = true;
        } else {
            cudaFree(img);
        }
    } else {
        cudaGetLastError();  // no room: not an error
    }
    if (prev != w->device) cudaSetDevice(prev);
    return rc;
}

uint32_t gemm_tc_status() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v));
    return v;
}

// One activation matrix against up to three weights (q / k / v, gate / up): the activation operands are converted once
// and, when every weight has its image, ONE kernel launch covers all of them (the small matrices' CTAs run beside the
// large one's instead of after them).  *taken = false: not these kernels' case, nothing launched.
int32_t launch_gemm_tc_multi(const GemmTarget *t, int count, const ActView &x, size_t n, size_t ldy, int epilogue, cudaStream_t st,
                             bool *taken) {
    *taken = false;
    static const bool off = [] {
        const char *e = getenv("CERA_CUDA_GEMM");
        return e && (strcmp(e, "mma") == 0 || strcmp(e, "columns") == 0);
    }();
    if (off || count < 1 || count > 3 || n <= 32) return CERA_CUDA_OK;
    const WeightView &w = t[0].w;
    if (w.k % 256 || (w.type != CERA_TYPE_Q4_K && w.type != CERA_TYPE_Q5_K && w.type != CERA_TYPE_Q6_K)) return CERA_CUDA_OK;
    // Q6_K: only over its image, and only with at least two token tiles (a single tile of a long-k matrix leaves each of
    // the few CTAs a serial walk that the warp-level kernel's split-k clusters beat: 189 against 111 us at 4096 x 14336 x 64)
    if (w.type == CERA_TYPE_Q6_K && (!w.tc || n <= 128 || count > 1)) return CERA_CUDA_OK;
    for (int i = 1; i < count; ++i)  // several weights: the same k, Q4_K / Q5_K, every one with its image
        if (t[i].w.k != w.k || !t[i].w.tc || !w.tc || (t[i].w.type != CERA_TYPE_Q4_K && t[i].w.type != CERA_TYPE_Q5_K)) return CERA_CUDA_OK;
    if ((uintptr_t)x.quants % 16 || (uintptr_t)x.scales % 16 || (uintptr_t)x.sums % 16) return CERA_CUDA_OK;
    // the activation operands, converted once for all row tiles: a stream-ordered scratch allocation that lives for this
    // call (token tiles x stages x 32 KB, the min operand's token side, g and 1 / g)
    const uint32_t tiles = (uint32_t)((n + TC_BM - 1) / TC_BM), n_pad = tiles * TC_BM, n_it = w.k / TC_KS, n_sb = w.k / 256;
    const uint32_t nb32 = w.k / 32, n_mit = (nb32 + TCW_MIN_J - 1) / TCW_MIN_J;
    const size_t img_bytes = (size_t)tiles * n_it * (2 * TC_OP_BYTES), min_bytes = (size_t)tiles * n_sb * TC_MINOP_BYTES,
                 xm_bytes = (size_t)tiles * n_mit * (2 * TCW_MINT_BYTES);
    {
        // keep the stream-ordered pool's memory across synchronisations (by default a pool hands everything back to the
        // driver at every synchronise, and the next prompt's first allocations pay for mapping it again); once per device
        static thread_local int pooled_dev = -1;
        int dev = 0;
        cudaGetDevice(&dev);
        if (pooled_dev != dev) {
            cudaMemPool_t pool = nullptr;
            if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
                uint64_t keep = 1ull << 30;  // up to 1 GB of scratch stays cached
                cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            }
            cudaGetLastError();
            pooled_dev = dev;
        }
    }
    uint8_t *scratch = nullptr;
    if (cudaMallocAsync((void **)&scratch, img_bytes + min_bytes + xm_bytes + (size_t)n_pad * 8, st) != cudaSuccess) {
        cudaGetLastError();  // no room for the operand scratch: leave the GEMM to the kernels that need none
        return CERA_CUDA_OK;
    }
    uint8_t *xm = scratch + img_bytes + min_bytes;
    float *g_tab = reinterpret_cast<float *>(xm + xm_bytes), *ginv_tab = g_tab + n_pad;
    // the last min stage's columns beyond k / 32 are zero (never written by the image kernel)
    if (nb32 % TCW_MIN_J) CERA_CUDA_TRY(cudaMemsetAsync(xm, 0, xm_bytes, st));
    int32_t rc = check_cuda(launch_k(tc_token_range_kernel, dim3((n_pad + 7) / 8), dim3(256), 0, st, x, (uint32_t)n, (uint32_t)w.k, n_pad, g_tab, ginv_tab),
                            "gemm (tcgen05) token range launch");
    if (rc == CERA_CUDA_OK)
        rc = check_cuda(launch_k(tc_token_image_kernel, dim3(tiles, n_it), dim3(TC_IMG_THREADS), 0, st, x, (uint32_t)n, (uint32_t)w.k, (const float *)g_tab,
                                 scratch, scratch + img_bytes, xm),
                        "gemm (tcgen05) token image launch");
    count_launch();
    count_launch();
    TcParams p{};
    p.w = w;
    p.img = scratch;
    p.img_min = scratch + img_bytes;
    p.ginv = ginv_tab;
    p.xm = xm;
    p.out = t[0].out;
    p.m = w.m;
    p.n = (uint32_t)n;
    p.k = w.k;
    p.ldy = (uint32_t)ldy;
    p.ldc = (uint32_t)t[0].ldc;
    p.epilogue = epilogue;
    p.n_w = (uint32_t)count;
    *taken = true;
    // with weight images: the wide kernel when its 128 x 256 tiles alone fill the device, else the 128 x 128 one
    static const int tile_pref = [] {
        const char *e = getenv("CERA_CUDA_GEMM_TILE");
        return e ? atoi(e) : 0;
    }();
    uint32_t wide_y = 0;
    for (int i = 0; i < count; ++i) wide_y += (t[i].w.m + 2 * TC_BN - 1) / (2 * TC_BN);
    const bool wide = w.tc && (tile_pref == 256 || (tile_pref != 128 && tiles * wide_y >= 120));
    uint32_t y = 0;
    for (int i = 0; i < count; ++i) {
        y += wide ? (t[i].w.m + 2 * TC_BN - 1) / (2 * TC_BN) : (t[i].w.m + TC_BN - 1) / TC_BN;
        p.y_end[i] = y;
        if (i) {
            p.tc_x[i - 1] = t[i].w.tc;
            p.out_x[i - 1] = t[i].out;
            p.m_x[i - 1] = t[i].w.m;
            p.ldc_x[i - 1] = (uint32_t)t[i].ldc;
        }
    }
    if (rc == CERA_CUDA_OK && w.type == CERA_TYPE_Q6_K) {
        rc = launch_tc6(p, st);
    } else if (rc == CERA_CUDA_OK && wide) {
        rc = launch_tc_wide(p, y, st);
    } else if (rc == CERA_CUDA_OK) {
        if (w.tc)
            rc = w.type == CERA_TYPE_Q4_K ? launch_tc_typed<CERA_TYPE_Q4_K, true>(p, y, st) : launch_tc_typed<CERA_TYPE_Q5_K, true>(p, y, st);
        else
            rc = w.type == CERA_TYPE_Q4_K ? launch_tc_typed<CERA_TYPE_Q4_K, false>(p, y, st) : launch_tc_typed<CERA_TYPE_Q5_K, false>(p, y, st);
    }
    cudaFreeAsync(scratch, st);  // after the kernels above, in stream order
    return rc;
}

// tcgen05 GEMM for K-quant weights stored with interleaved row groups, k a multiple of 256, n > 32 columns.
// *taken = false: not this kernel's case, nothing launched.  CERA_CUDA_GEMM=mma keeps the warp-level kernel.
int32_t launch_gemm_tc(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                       cudaStream_t st, bool *taken) {
    const GemmTarget t{w, out, ldc};
    return launch_gemm_tc_multi(&t, 1, x, n, ldy, epilogue, st, taken);
}

}  // namespace cera
