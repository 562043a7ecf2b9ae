// Prefill GEMM on the fifth-generation tensor cores: out[m x n] = W (Q4_K / Q5_K) x X (Q8_0 columns) with
// tcgen05.mma, accumulators in tensor memory (TMEM), for n >= 33 columns and k a multiple of 256.
//
// The arithmetic contract (cera/src/backend/simd.rs:5248-5371, 5693-5878) scales every 32-element block's EXACT
// integer sum by (weight block scale) x (activation block scale), so a tensor-core instruction may accumulate over
// one block only and the rescale runs on the CUDA cores.  Four choices keep that rescale small:
//
//  * f16 operands with exact small integers.  A weight operand element is sc * q (six-bit sub-block scale times
//    the 4/5-bit quant, at most 63 * 31 = 1953 < 2048: exact in f16), an activation element is the int8 quant.
//    kind::f16 MMAs accumulate the products exactly in f32 (|sum| < 2^24), so the accumulator already holds the
//    float the rescale needs - no int-to-float conversion - and the sub-block scale is inside the product.
//  * Tokens on the TMEM lanes.  D[token][weight row]: an epilogue thread owns one token, so the activation block
//    scale is one value per thread; it keeps p[row] += D * xs for its 32 rows in registers - ONE FMA per cell
//    per block - and once per 256-element super-block folds out[row] += d[row] * p[row] into a TMEM region.
//  * The min term rides the tensor cores too.  sum_b dmin*mn_b * (xs_b * A_b) (A_b = the block's sum of quants)
//    has one factor per (row, block) and one per (token, block): a 16-column MMA per super-block multiplies the
//    eight six-bit mins (exact in f16, each twice) by the eight values g*xs_b*A_b split into an f16 high and low
//    part (g = a power of two per token that brings them below 2^15; 22 significant bits survive), into a third
//    accumulator; the fold subtracts dmin[row] * Dm / g.
//  * Operand tiles are built in shared memory by producer warps straight from the quantized bytes (weights:
//    nibble -> 0x6400|q -> one HFMA2 with the sub-block scale; activations: byte -> 0x6400|(b^0x80) -> HSUB2), in the
//    canonical K-major no-swizzle layout (8-row x 16-byte core matrices), three stages of 128 k-elements deep.
//
// Warp roles in a CTA of 25 warps (one 128-token x 128-row tile): warp 0 allocates TMEM and issues the MMAs from
// one thread; warps 1-4 build the weight operand (thread = weight row) and the row-side tables; warps 5-8 build
// the activation operand (thread = token); warps 9-24 are the epilogue (thread = token lane x 32 rows).  Stages
// and the two D buffers are handed over through mbarriers (tcgen05.commit arrives on them when the MMAs have
// finished).  Every wait is bounded: when a limit runs out the CTA raises an abort flag, its roles leave their
// loops, TMEM is freed and a status word reports it (cera_cuda_kernel_status).
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "gemv_task.cuh"
#include "tma.cuh"

namespace cera {

__device__ unsigned int g_tc_status = 0;  // nonzero: a bounded wait of gemm_tc_kernel ran out (bits name the role)

namespace {

constexpr int TC_BM = 128;      // tokens per tile (TMEM lanes)
constexpr int TC_BN = 128;      // weight rows per tile (TMEM columns)
constexpr int TC_KS = 128;      // k elements per stage
constexpr int TC_STAGES = 3;
constexpr int TC_EPI_WARPS = 16;                // four warpgroups: each covers the 128 token lanes for 32 weight rows
constexpr int TC_THREADS = (9 + TC_EPI_WARPS) * 32;
constexpr uint32_t TC_OP_BYTES = TC_BM * TC_KS * 2;                      // one operand tile of a stage: 32 KB
constexpr uint32_t TC_TAB_BYTES = 4 * TC_BM * 4;                         // xsv[4][128]: the stage's activation block scales per token
constexpr uint32_t TC_STAGE_BYTES = 2 * TC_OP_BYTES + TC_TAB_BYTES;      // 67 584
// per super-block (two stages), two slots: the min-term operands (16 k-columns each) and the row-side tables
constexpr uint32_t TC_MINOP_BYTES = TC_BM * 16 * 2;                      // 4 KB: [2 k chunks][128 rows][8 f16]
constexpr uint32_t TC_SLOT_BYTES = 2 * TC_MINOP_BYTES + 2 * TC_BN * 4;   // A, B, dval[128], dmin[128]
constexpr uint32_t TC_TAIL_OFF = TC_STAGES * TC_STAGE_BYTES + 2 * TC_SLOT_BYTES;  // ginv[128], then barriers, TMEM address, abort flag
constexpr uint32_t TC_SMEM_BYTES = TC_TAIL_OFF + TC_BM * 4 + 256;
constexpr uint32_t TC_TMEM_COLS = 512;                                   // D0 [0,128) D1 [128,256) Dm [256,384) OUT [384,512)
constexpr uint32_t TC_DBUFS = 2;
constexpr uint32_t TC_KC_STRIDE = TC_BM * 16;                            // bytes between 8-element k chunks: 2048

struct TcParams {
    WeightView w;
    ActView x;
    float *out;
    uint32_t m, n, k;
    uint32_t ldy, ldc;
    int epilogue;
};

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

template <int T>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t *slots = tc_smem + TC_STAGES * TC_STAGE_BYTES;
    float *ginv_tab = reinterpret_cast<float *>(tc_smem + TC_TAIL_OFF);  // [128]: 1 / g of every token lane
    uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + TC_TAIL_OFF + TC_BM * 4);
    uint64_t *full_ab = bars, *empty_ab = bars + TC_STAGES, *full_d = bars + 2 * TC_STAGES, *empty_d = full_d + TC_DBUFS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TC_STAGES + 2 * TC_DBUFS);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t col0 = blockIdx.x * TC_BM, row0 = blockIdx.y * TC_BN;
    const uint32_t n_it = p.k / TC_KS;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            tma::mbar_init(full_ab + s, 256);                 // every producer thread
            tma::mbar_init(empty_ab + s, 1 + TC_EPI_WARPS);   // the MMAs' commit + each epilogue warp (it reads the stage's tables)
        }
        for (int b = 0; b < (int)TC_DBUFS; ++b) {
            tma::mbar_init(full_d + b, 1);
            tma::mbar_init(empty_d + b, TC_EPI_WARPS);
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
            for (uint32_t it = 0; it < n_it && ok; ++it) {
                const uint32_t s = it % TC_STAGES;
                if (!tma::mbar_wait_blocking(full_ab + s, (it / TC_STAGES) & 1, abort_flag, &g_tc_status, 1u)) break;
                tc_fence_after();
                const uint32_t a_base = tma::smem_u32(tc_smem + s * TC_STAGE_BYTES), b_base = a_base + TC_OP_BYTES;
                for (uint32_t b = 0; b < 4; ++b) {
                    const uint32_t gb = it * 4 + b, buf = gb % TC_DBUFS;
                    if (!tma::mbar_wait_blocking(empty_d + buf, ((gb / TC_DBUFS) & 1) ^ 1, abort_flag, &g_tc_status, 2u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t j = 0; j < 2; ++j) {
                        const uint32_t kc = 4 * b + 2 * j;
                        tc_mma_f16(tmem + buf * TC_BN, smem_desc(a_base + kc * TC_KC_STRIDE, TC_KC_STRIDE, 128),
                                   smem_desc(b_base + kc * TC_KC_STRIDE, TC_KC_STRIDE, 128), idesc, j);
                    }
                    if ((it & 1) && b == 3) {
                        // the super-block's min term: Dm[token][row] = sum_b mn_b * (hi_b + lo_b).  The epilogue has read the
                        // previous Dm: it handed back a D buffer of THIS iteration, which it reaches only after that fold.
                        const uint32_t slot = tma::smem_u32(slots + ((it >> 1) & 1) * TC_SLOT_BYTES);
                        tc_mma_f16(tmem + 2 * TC_BN, smem_desc(slot, TC_KC_STRIDE, 128), smem_desc(slot + TC_MINOP_BYTES, TC_KC_STRIDE, 128),
                                   idesc, 0);
                    }
                    tc_commit(full_d + buf);
                }
                tc_commit(empty_ab + s);
            }
        }
    } else if (warp <= 4) {
        // ---------------------------------------------------------------- weight operand: thread = weight row
        const uint32_t r = tid - 32;
        const uint32_t row = min(row0 + r, p.m - 1);  // rows past the edge repeat the last one; their results are not stored
        struct RawW {
            uint4 piece[4], h, hb0, hb1;
        };
        auto fetch = [&](uint32_t it) {
            RawW rw;
#pragma unroll
            for (int c = 0; c < 4; ++c) rw.piece[c] = ld_stream(q_piece_ptr(p.w, row, 4, it * 4 + c));
            const size_t sbi = sb_index(p.w, row, it >> 1);
            rw.h = __ldg(reinterpret_cast<const uint4 *>(p.w.hdr) + sbi);
            rw.hb0 = make_uint4(0, 0, 0, 0);
            rw.hb1 = rw.hb0;
            if (T == CERA_TYPE_Q5_K) {
                rw.hb0 = __ldg(reinterpret_cast<const uint4 *>(p.w.qh + sbi * 32));
                rw.hb1 = __ldg(reinterpret_cast<const uint4 *>(p.w.qh + sbi * 32 + 16));
            }
            return rw;
        };
        // (fetching an iteration ahead of the conversion was measured: no gain, and its 28 live registers spill)
        for (uint32_t it = 0; it < n_it; ++it) {
            const uint32_t s = it % TC_STAGES;
            const RawW cur = fetch(it);
            const uint4 (&piece)[4] = cur.piece;
            const uint4 h = cur.h, hb0 = cur.hb0, hb1 = cur.hb1;
            if (!tma::mbar_wait_blocking(empty_ab + s, ((it / TC_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 4u)) break;
            uint8_t *stage = tc_smem + s * TC_STAGE_BYTES;
            uint8_t *opb = stage + TC_OP_BYTES;
            uint8_t *slot = slots + ((it >> 1) & 1) * TC_SLOT_BYTES;  // free: the stage it shares a phase with was released
            const uint32_t hf = it & 1;
            uint32_t scp, mnp;
            kq_quad(h, hf, scp, mnp);
            const float d = h2f((uint16_t)(h.x & 0xFFFF)), dmin = h2f((uint16_t)(h.x >> 16));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int pair = c >> 1, half = c & 1;
                const uint32_t sc_lo = (scp >> (8 * (2 * pair))) & 0xFF, sc_hi = (scp >> (8 * (2 * pair + 1))) & 0xFF;
                const __half2 s_lo = __half2half2(__ushort2half_rn((unsigned short)sc_lo)), s_hi = __half2half2(__ushort2half_rn((unsigned short)sc_hi));
                const __half2 nb_lo = __hmul2(s_lo, __float2half2_rn(-1024.0f)), nb_hi = __hmul2(s_hi, __float2half2_rn(-1024.0f));
                const uint4 v4 = piece[c];
                const uint4 hbv = half ? hb1 : hb0;
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
                // low nibbles: elements [16 half, +16) of sub-block 2 pair; high nibbles: the same of sub-block 2 pair + 1
                const uint32_t kc_lo = 8 * pair + 2 * half, kc_hi = kc_lo + 4;
                *reinterpret_cast<uint4 *>(opb + op_off(kc_lo, r)) = *reinterpret_cast<const uint4 *>(&lo8[0]);
                *reinterpret_cast<uint4 *>(opb + op_off(kc_lo + 1, r)) = *reinterpret_cast<const uint4 *>(&lo8[4]);
                *reinterpret_cast<uint4 *>(opb + op_off(kc_hi, r)) = *reinterpret_cast<const uint4 *>(&hi8[0]);
                *reinterpret_cast<uint4 *>(opb + op_off(kc_hi + 1, r)) = *reinterpret_cast<const uint4 *>(&hi8[4]);
            }
            {
                // the four mins of this half super-block, each twice (for the high and the low part of the token side):
                // k chunk `hf` of the min-term weight operand
                __half2 mn2[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) mn2[j] = __half2half2(__ushort2half_rn((unsigned short)((mnp >> (8 * j)) & 0xFF)));
                *reinterpret_cast<uint4 *>(slot + TC_MINOP_BYTES + op_off(hf, r)) = *reinterpret_cast<const uint4 *>(&mn2[0]);
                if (hf == 0) {
                    float *dval = reinterpret_cast<float *>(slot + 2 * TC_MINOP_BYTES);
                    dval[r] = d;
                    dval[TC_BN + r] = dmin;
                }
            }
            fence_async_smem();
            tma::mbar_arrive(full_ab + s);
        }
    } else if (warp <= 8) {
        // ---------------------------------------------------------------- activation operand: thread = token
        const uint32_t c = tid - 160;
        const uint32_t token = min(col0 + c, p.n - 1);
        const int8_t *src = p.x.quants + (size_t)token * p.k;
        const __half2 bias = __float2half2_rn(1152.0f);  // 1024 + 128
        const uint32_t nb32 = p.k >> 5, nb16 = p.k >> 4;
        struct RawX {
            uint4 v[8];
            float4 xs;  // the four block scales of the stage
            uint4 sm;   // the eight 16-element sums
        };
        auto fetch = [&](uint32_t it) {
            RawX rx;
#pragma unroll
            for (int j = 0; j < 8; ++j) rx.v[j] = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)it * TC_KS) + j);
            rx.xs = __ldg(reinterpret_cast<const float4 *>(p.x.scales + (size_t)token * nb32 + it * 4));
            rx.sm = __ldg(reinterpret_cast<const uint4 *>(p.x.sums + (size_t)token * nb16 + it * 8));
            return rx;
        };
        // g: a power of two that brings every xs_b * A_b of the token below 2^15, so that its f16 high / low parts keep
        // 22 significant bits whatever the magnitude of the activations
        float g = 1.0f;
        {
            float mx = 0.0f;
            for (uint32_t it = 0; it < n_it; ++it) {
                const float4 x4 = __ldg(reinterpret_cast<const float4 *>(p.x.scales + (size_t)token * nb32 + it * 4));
                const uint4 s4 = __ldg(reinterpret_cast<const uint4 *>(p.x.sums + (size_t)token * nb16 + it * 8));
                const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
                const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const float v = fabsf(xv[b] * (float)((int)(int16_t)(sw[b] & 0xFFFF) + (int)(int16_t)(sw[b] >> 16)));
                    mx = fmaxf(mx, v == v && v < 3.0e38f ? v : 0.0f);
                }
            }
            if (mx > 0.0f) {
                int e;
                frexpf(mx, &e);  // mx < 2^e
                g = ldexpf(1.0f, 15 - e);
            }
            ginv_tab[c] = 1.0f / g;  // published by the first full_ab arrival below
        }
        for (uint32_t it = 0; it < n_it; ++it) {
            const uint32_t s = it % TC_STAGES;
            const RawX cur = fetch(it);  // (a register prefetch of the next stage spills at 72 registers: measured no faster)
            const uint4 (&raw)[8] = cur.v;
            if (!tma::mbar_wait_blocking(empty_ab + s, ((it / TC_STAGES) & 1) ^ 1, abort_flag, &g_tc_status, 8u)) break;
            uint8_t *opa = tc_smem + s * TC_STAGE_BYTES;
            uint8_t *slot = slots + ((it >> 1) & 1) * TC_SLOT_BYTES;
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // 16 quants -> k chunks 2j, 2j+1
                const uint32_t wv[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
                __half2 o[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __half2 a, b;
                    bytes_to_h1024(wv[i] ^ 0x80808080u, a, b);  // signed byte + 128 -> unsigned
                    o[2 * i] = __hsub2(a, bias);
                    o[2 * i + 1] = __hsub2(b, bias);
                }
                *reinterpret_cast<uint4 *>(opa + op_off(2 * j, c)) = *reinterpret_cast<const uint4 *>(&o[0]);
                *reinterpret_cast<uint4 *>(opa + op_off(2 * j + 1, c)) = *reinterpret_cast<const uint4 *>(&o[4]);
            }
            {
                // per-token scalars of the stage's four blocks: the block scales for the epilogue, and g * xs_b * A_b as an f16
                // high and low part = k chunk (it & 1) of the min-term token operand
                float *xsv = reinterpret_cast<float *>(opa + 2 * TC_OP_BYTES);
                const float xv[4] = {cur.xs.x, cur.xs.y, cur.xs.z, cur.xs.w};
                const uint32_t sw[4] = {cur.sm.x, cur.sm.y, cur.sm.z, cur.sm.w};
                __half2 hl[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    xsv[b * TC_BM + c] = xv[b];
                    const float v = (xv[b] * (float)((int)(int16_t)(sw[b] & 0xFFFF) + (int)(int16_t)(sw[b] >> 16))) * g;
                    const __half hi = __float2half_rn(v);
                    const __half lo = __float2half_rn(v - __half2float(hi));
                    hl[b] = __halves2half2(hi, lo);
                }
                *reinterpret_cast<uint4 *>(slot + op_off(it & 1, c)) = *reinterpret_cast<const uint4 *>(&hl[0]);
            }
            fence_async_smem();
            tma::mbar_arrive(full_ab + s);
        }
    } else {
        // ---------------------------------------------------------------- epilogue: thread = (token lane, 32 rows)
        const uint32_t e = warp - 9, ch = e >> 2, quad = warp & 3;  // a warp reaches TMEM lanes [32 (warp % 4), +32)
        const uint32_t tl = quad * 32 + lane;                       // token lane
        const uint32_t lane_addr = tmem + ((quad * 32) << 16);
        float pacc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pacc[i] = 0.0f;
        float ginv = 1.0f;
        bool ok = true;
        for (uint32_t it = 0; it < n_it && ok; ++it) {
            const uint32_t s = it % TC_STAGES;
            const float *xsv = reinterpret_cast<const float *>(tc_smem + s * TC_STAGE_BYTES + 2 * TC_OP_BYTES);
            // the producers' release of this stage, observed directly: the tables are read with plain loads
            if (!tma::mbar_wait_blocking(full_ab + s, (it / TC_STAGES) & 1, abort_flag, &g_tc_status, 32u)) break;
            if (it == 0) ginv = ginv_tab[tl];
            for (uint32_t b = 0; b < 4; ++b) {
                const uint32_t gb = it * 4 + b, buf = gb % TC_DBUFS;
                const float xs = xsv[b * TC_BM + tl];
                if (!tma::mbar_wait_blocking(full_d + buf, (gb / TC_DBUFS) & 1, abort_flag, &g_tc_status, 16u)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                {
                    uint32_t dreg[16];
                    tmem_ld16(lane_addr + buf * TC_BN + ch * 32, dreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) pacc[i] = fmaf(__uint_as_float(dreg[i]), xs, pacc[i]);
                    tmem_ld16(lane_addr + buf * TC_BN + ch * 32 + 16, dreg);
                    tmem_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tma::mbar_arrive(empty_d + buf);  // the values are in registers: the buffer may be overwritten
#pragma unroll
                    for (int i = 0; i < 16; ++i) pacc[16 + i] = fmaf(__uint_as_float(dreg[i]), xs, pacc[16 + i]);
                }
            }
            if (!ok) break;
            if (it & 1) {
                // end of a 256-element super-block: out[row] += d[row] * p[row] - dmin[row] * Dm[row] / g; the running sum lives in TMEM
                const float *dval = reinterpret_cast<const float *>(slots + ((it >> 1) & 1) * TC_SLOT_BYTES + 2 * TC_MINOP_BYTES);
#pragma unroll
                for (int c4 = 0; c4 < 2; ++c4) {
                    uint32_t oreg[16], mreg[16];
                    const uint32_t addr = lane_addr + 3 * TC_BN + ch * 32 + c4 * 16;
                    tmem_ld16(lane_addr + 2 * TC_BN + ch * 32 + c4 * 16, mreg);
                    if (it > 1) {
                        tmem_ld16(addr, oreg);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) oreg[i] = 0u;
                    }
                    tmem_wait_ld();
                    const float4 *dq = reinterpret_cast<const float4 *>(dval + ch * 32 + c4 * 16), *mq = dq + TC_BN / 4;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 dv = dq[q4], mv = mq[q4];
                        const float dvv[4] = {dv.x, dv.y, dv.z, dv.w}, mvv[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int j = q4 * 4 + i;
                            float o = fmaf(pacc[c4 * 16 + j], dvv[i], __uint_as_float(oreg[j]));
                            o = fmaf(-mvv[i], __uint_as_float(mreg[j]) * ginv, o);
                            oreg[j] = __float_as_uint(o);
                            pacc[c4 * 16 + j] = 0.0f;
                        }
                    }
                    tmem_st16(addr, oreg);
                }
                tmem_wait_st();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(empty_ab + s);  // this warp is done with the stage's tables (and the slot's)
        }
        if (ok) {
            // ---- the tile -> global memory: cell (row i, token j) at out[i * ldy + j * ldc]
            const bool tok_ok = col0 + tl < p.n;
#pragma unroll
            for (int c4 = 0; c4 < 2; ++c4) {
                uint32_t oreg[16];
                tmem_ld16(lane_addr + 3 * TC_BN + ch * 32 + c4 * 16, oreg);
                tmem_wait_ld();
                if (tok_ok) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t row = row0 + ch * 32 + c4 * 16 + i;
                        if (row < p.m) {
                            float *o = p.out + (size_t)row * p.ldy + (size_t)(col0 + tl) * p.ldc;
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

template <int T>
int32_t launch_tc_typed(const TcParams &p, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
        configured_dev = dev;
    }
    const dim3 grid((p.n + TC_BM - 1) / TC_BM, (p.m + TC_BN - 1) / TC_BN);
    count_launch();
    return check_cuda(launch_k(gemm_tc_kernel<T>, grid, dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, st, p), "gemm (tcgen05) launch");
}

}  // namespace

uint32_t gemm_tc_status() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v));
    return v;
}

// tcgen05 GEMM for Q4_K / Q5_K weights stored with interleaved row groups, k a multiple of 256, n > 32 columns.
// *taken = false: not this kernel's case, nothing launched.  CERA_CUDA_GEMM=mma keeps the warp-level kernel.
int32_t launch_gemm_tc(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                       cudaStream_t st, bool *taken) {
    *taken = false;
    static const bool off = [] {
        const char *e = getenv("CERA_CUDA_GEMM");
        return e && (strcmp(e, "mma") == 0 || strcmp(e, "columns") == 0);
    }();
    if (off || n <= 32 || w.k % 256 || (w.type != CERA_TYPE_Q4_K && w.type != CERA_TYPE_Q5_K)) return CERA_CUDA_OK;
    if ((uintptr_t)x.quants % 16 || (uintptr_t)x.scales % 16 || (uintptr_t)x.sums % 16) return CERA_CUDA_OK;
    TcParams p{};
    p.w = w;
    p.x = x;
    p.out = out;
    p.m = w.m;
    p.n = (uint32_t)n;
    p.k = w.k;
    p.ldy = (uint32_t)ldy;
    p.ldc = (uint32_t)ldc;
    p.epilogue = epilogue;
    *taken = true;
    if (w.type == CERA_TYPE_Q4_K) return launch_tc_typed<CERA_TYPE_Q4_K>(p, st);
    return launch_tc_typed<CERA_TYPE_Q5_K>(p, st);
}

}  // namespace cera
