// Prefill GEMM on the integer tensor-core path: out[m x n] = W (Q4_0, Q4_K, Q5_K or Q6_K) x X (Q8_0 columns), n >= 5,
// and its expert-grouped form for the routed FFN.
//
// A CTA owns a 64-row x 128-column output tile and walks k one 256-element super-block at a time:
// weights of the 64 rows and the Q8_0 quants of the 128 columns are staged in shared memory with
// cp.async, the six-bit / int8 sub-block scales are expanded to f32 once per chunk, and every warp
// (16 rows x 64 columns) issues mma.sync int8 instructions whose int32 results are EXACT per-block sums:
//   Q4_0 : m16n8k32 (u8 x s8) per 32-element block,      out += d * xs * U - (8*d) * (xs*A32)
//   Q4_K : m16n8k32 (u8 x s8) per 32-element sub-block,  out += (d*sc) * xs * U - (dmin*mn) * (xs*A32)
//   Q5_K : the same with the fifth bit of every quant merged into the u8 operand
//   Q6_K : m16n8k16 (u8 x s8) per 16-element scale group, out += (d*sc) * (xs*U - 32*xs*A16)
// Each int32 tile is scaled and folded into f32 accumulators on the CUDA cores right after its mma:
// with one scale pair per (row, block, column) that per-block rescale, not the tensor pipe, bounds the
// throughput of an exact kernel (about 20 CUDA-core instructions per 4096 multiply-adds).
// This is the warp-level (mma.sync) form; the same tiling moved onto tcgen05 with TMEM accumulators
// would free the issue slots the mma instructions take here, but keeps the same rescale bound.
//
// Small batches (few column tiles) would leave most SMs idle and each CTA with a long serial chain of
// chunks, so the k range of one output tile is split over a thread-block CLUSTER of up to 8 CTAs: each
// CTA accumulates its share of the super-blocks, parks its 64 x BN partial tile in its own shared memory,
// and after a cluster barrier every CTA finishes 64/CL rows of the tile by adding the CL partials in rank
// order through distributed shared memory (a fixed order: results do not depend on timing).  The column
// width of the tile is a template parameter (16, 32, 64 or 128) picked from n.
//
// Arithmetic contract: cera/src/backend/simd.rs:5693-5878 (Q4_K) and 5988-6195 (Q6_K), per cell; the
// f32 order is this kernel's own (blocks in k order per thread).
#include <cooperative_groups.h>

#include <cstdlib>
#include <cstring>

#include "act.cuh"
#include "ops.h"

namespace cg = cooperative_groups;

namespace cera {

namespace {

constexpr int GM_BM = 64, GM_THREADS = 256;
constexpr int GM_WQ_STRIDE = 144;   // 128 quant bytes per row, padded so 8 rows x 4 words hit 32 banks
constexpr int GM_WH_STRIDE = 80;    // Q6_K high-bit plane: 64 bytes per row, padded likewise
constexpr int GM_AQ_STRIDE = 272;   // 256 activation quants per column, padded likewise

struct GemmParams {
    WeightView w;
    ActView x;
    float *out;
    uint32_t m, n, k;
    uint32_t ldy, ldc;
    int epilogue;
    // expert-grouped form (tiles != null): blockIdx.y walks the device-side work list; m is the row count per expert
    const MoeTile *tiles;
    const uint32_t *n_tiles;
};

__device__ __forceinline__ void cpa16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cpa_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
// D(16x8, s32) = A(16x16, u8, row) * B(16x8, s8, col)
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

// The per-block rescale on packed f32 pairs (sm_100 FFMA2 / FMUL2: one instruction per two cells, same rounding as the
// scalar forms).  A thread's two cells of an accumulator row share the weight row and differ in the activation column.
//   acc += (sc * xs) * sum - mn * xb       (Q4_0, Q4_K, Q5_K)
__device__ __forceinline__ void rescale_pair(float2 &acc, float2 sc, float2 neg_mn, float2 xs, float2 xb, int c0, int c1) {
    acc = __ffma2_rn(__fmul2_rn(sc, xs), make_float2((float)c0, (float)c1), __ffma2_rn(neg_mn, xb, acc));
}
//   acc += sc * (xs * sum + xb)            (Q6_K)
__device__ __forceinline__ void rescale_pair_q6(float2 &acc, float2 sc, float2 xs, float2 xb, int c0, int c1) {
    acc = __ffma2_rn(sc, __ffma2_rn(xs, make_float2((float)c0, (float)c1), xb), acc);
}

template <int BN>
constexpr size_t gm_smem_bytes() {
    return GM_BM * GM_WQ_STRIDE + GM_BM * GM_WH_STRIDE + GM_BM * 16 + GM_BM * 16 * 4 + GM_BM * 8 * 4 + BN * GM_AQ_STRIDE +
           8 * BN * 4 + 16 * BN * 4;
}

template <int T, int GM_BN>
__global__ void __launch_bounds__(GM_THREADS) gemm_mma_kernel(const GemmParams p) {
    constexpr int NT = GM_BN / 16;  // 8-column n-tiles per warp (the tile is 4 warps tall, 2 wide)
    static_assert((size_t)GM_BM * GM_BN * 4 <= gm_smem_bytes<GM_BN>(), "the partial tile reuses the staging buffers");
    extern __shared__ __align__(16) uint8_t smem[];
    // shared-memory carve-up
    uint8_t *wq = smem;                                            // [64][144]
    uint8_t *wqh = wq + GM_BM * GM_WQ_STRIDE;                      // [64][80]   (Q6_K)
    uint8_t *whd = wqh + GM_BM * GM_WH_STRIDE;                     // [64][16]   raw header / int8 scales
    float *wsc = reinterpret_cast<float *>(whd + GM_BM * 16);      // [64][16]   d*sc per sub-block (Q4_K uses 8)
    float *wmn = wsc + GM_BM * 16;                                 // [64][8]    dmin*mn (Q4_K)
    uint8_t *aq = reinterpret_cast<uint8_t *>(wmn + GM_BM * 8);    // [128][272]
    float *axs = reinterpret_cast<float *>(aq + GM_BN * GM_AQ_STRIDE);  // [8][128]  block scales
    float *axb = axs + 8 * GM_BN;                                  // [16][128] xs*A32 (Q4_K, 8 used) or -32*xs*A16 (Q6_K)

    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int wrow = (warp & 3) * 16, wcol = (warp >> 2) * (GM_BN / 2);  // this warp's 16 x BN/2 patch of the tile
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t CL = cluster.num_blocks(), crank = cluster.block_rank();
    uint32_t row0 = (blockIdx.x / CL) * GM_BM, col0 = blockIdx.y * GM_BN;
    uint32_t wrow0 = row0, n_cols = p.n;  // first weight row of the tile; one past the last valid activation column
    if (p.tiles) {
        if (blockIdx.y >= *p.n_tiles) return;  // uniform over the cluster (same blockIdx.y)
        const MoeTile tile = p.tiles[blockIdx.y];
        col0 = tile.first;
        n_cols = tile.first + tile.count;
        wrow0 = tile.expert * p.m + row0;
    }
    const uint32_t w_last = (p.tiles ? wrow0 - row0 : 0) + p.m - 1;  // last weight row this tile may touch
    const uint32_t nb = p.w.nb, nb32 = p.k >> 5, nb16 = p.k >> 4;
    const TypeInfo ti = type_info(T);

    float2 acc[NT][2];  // [n-tile][row gid / row gid + 8] x (column 2*tig, 2*tig + 1)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = make_float2(0.0f, 0.0f);

    // this CTA's share of the super-blocks
    const uint32_t n_chunks = p.k >> 8;  // 256 weights per chunk: a K-quant super-block, or eight Q4_0 blocks
    const uint32_t per = (n_chunks + CL - 1) / CL, bi_begin = min(n_chunks, crank * per), bi_end = min(n_chunks, bi_begin + per);
    for (uint32_t bi = bi_begin; bi < bi_end; ++bi) {
        // ---- stage the chunk: weights of 64 rows, activations of 128 columns (rows / columns past the
        // edge are clamped to the last valid one; their results are never stored)
        for (int i = tid; i < GM_BM * 8; i += GM_THREADS) {
            const int r = i >> 3, pc = i & 7;
            const uint32_t row = min(wrow0 + r, w_last);
            const uint8_t *src = q_piece_ptr(p.w, row, 4, bi * 8 + pc);
            cpa16(wq + r * GM_WQ_STRIDE + pc * 16, src);
        }
        if (T == CERA_TYPE_Q6_K) {
            for (int i = tid; i < GM_BM * 4; i += GM_THREADS) {
                const int r = i >> 2, pc = i & 3;
                const uint32_t row = min(wrow0 + r, w_last);
                cpa16(wqh + r * GM_WH_STRIDE + pc * 16, p.w.qh + sb_index(p.w, row, bi) * 64 + pc * 16);
            }
        }
        if (T == CERA_TYPE_Q5_K) {  // fifth bits: 32 bytes per row, bit s of byte l belongs to element l of sub-block s
            for (int i = tid; i < GM_BM * 2; i += GM_THREADS) {
                const int r = i >> 1, pc = i & 1;
                const uint32_t row = min(wrow0 + r, w_last);
                cpa16(wqh + r * GM_WH_STRIDE + pc * 16, p.w.qh + sb_index(p.w, row, bi) * 32 + pc * 16);
            }
        }
        for (int r = tid; r < GM_BM; r += GM_THREADS) {
            const uint32_t row = min(wrow0 + r, w_last);
            if (T == CERA_TYPE_Q4_0) cpa16(whd + r * 16, p.w.hdr + ((size_t)row * nb + bi * 8) * 2);  // eight f16 block scales
            else cpa16(whd + r * 16, p.w.hdr + sb_index(p.w, row, bi) * 16);
        }
        for (int i = tid; i < GM_BN * 16; i += GM_THREADS) {
            const int c = i >> 4, pc = i & 15;
            const uint32_t col = min(col0 + c, n_cols - 1);
            cpa16(aq + c * GM_AQ_STRIDE + pc * 16, p.x.quants + (size_t)col * p.k + (size_t)bi * 256 + pc * 16);
        }
        for (int i = tid; i < GM_BN * 8; i += GM_THREADS) {
            const int c = i % GM_BN, s = i / GM_BN;
            const uint32_t col = min(col0 + c, n_cols - 1);
            const float xs = p.x.scales[(size_t)col * nb32 + bi * 8 + s];
            const int16_t *sm = p.x.sums + (size_t)col * nb16 + (bi * 8 + s) * 2;
            axs[s * GM_BN + c] = xs;
            if (T != CERA_TYPE_Q6_K) {
                axb[s * GM_BN + c] = xs * (float)((int)sm[0] + (int)sm[1]);
            } else {
                axb[(2 * s) * GM_BN + c] = -32.0f * (xs * (float)sm[0]);
                axb[(2 * s + 1) * GM_BN + c] = -32.0f * (xs * (float)sm[1]);
            }
        }
        cpa_wait_all();
        __syncthreads();
        // ---- expand the sub-block scales of the 64 rows to f32
        if (T == CERA_TYPE_Q4_0) {
            // w = (q - 8) * d: the -8 is the "min" term with 8*d in the place of dmin*mn (cera/src/backend/simd.rs:5303-5314)
            for (int i = tid; i < GM_BM * 8; i += GM_THREADS) {
                const int r = i >> 3, s = i & 7;
                const float d = h2f(reinterpret_cast<const uint16_t *>(whd + r * 16)[s]);
                wsc[r * 16 + s] = d;
                wmn[r * 8 + s] = 8.0f * d;
            }
        } else if (T != CERA_TYPE_Q6_K) {
            for (int i = tid; i < GM_BM * 8; i += GM_THREADS) {
                const int r = i >> 3, s = i & 7;
                const uint8_t *h = whd + r * 16;
                int sc, mn;
                kscale(h + 4, s, sc, mn);
                const float d = h2f((uint16_t)(h[0] | (h[1] << 8))), dmin = h2f((uint16_t)(h[2] | (h[3] << 8)));
                wsc[r * 16 + s] = d * (float)sc;
                wmn[r * 8 + s] = dmin * (float)mn;
            }
        } else {
            for (int i = tid; i < GM_BM * 16; i += GM_THREADS) {
                const int r = i >> 4, e = i & 15;
                const uint32_t row = min(wrow0 + r, w_last);
                const float d = h2f(reinterpret_cast<const uint16_t *>(p.w.d)[sb_index(p.w, row, bi)]);
                wsc[r * 16 + e] = d * (float)(int8_t)whd[r * 16 + e];
            }
        }
        __syncthreads();

        // ---- tensor-core work of this chunk
        const uint8_t *qa = wq + (wrow + gid) * GM_WQ_STRIDE, *qb = qa + 8 * GM_WQ_STRIDE;
        if (T == CERA_TYPE_Q4_0) {
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                // block s = bytes [16s, 16s+16): low nibble of byte i = element i, high nibble = element i + 16
                const uint32_t wa = *reinterpret_cast<const uint32_t *>(qa + 16 * s + 4 * tig);
                const uint32_t wb = *reinterpret_cast<const uint32_t *>(qb + 16 * s + 4 * tig);
                const uint32_t a[4] = {wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, (wa >> 4) & 0x0F0F0F0Fu, (wb >> 4) & 0x0F0F0F0Fu};
                const float sca = wsc[(wrow + gid) * 16 + s], scb = wsc[(wrow + gid + 8) * 16 + s];
                const float mna = wmn[(wrow + gid) * 8 + s], mnb = wmn[(wrow + gid + 8) * 8 + s];
                const float2 sca2 = make_float2(sca, sca), scb2 = make_float2(scb, scb);
                const float2 mna2 = make_float2(-mna, -mna), mnb2 = make_float2(-mnb, -mnb);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int cb = wcol + 8 * j;
                    const uint8_t *bp = aq + (cb + gid) * GM_AQ_STRIDE + 32 * s + 4 * tig;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp + 16);
                    int c[4];
                    mma_u8s8_k32(c, a, b0, b1);
                    const float2 xs = *reinterpret_cast<const float2 *>(axs + s * GM_BN + cb + 2 * tig);
                    const float2 xb = *reinterpret_cast<const float2 *>(axb + s * GM_BN + cb + 2 * tig);
                    rescale_pair(acc[j][0], sca2, mna2, xs, xb, c[0], c[1]);
                    rescale_pair(acc[j][1], scb2, mnb2, xs, xb, c[2], c[3]);
                }
            }
        } else if (T != CERA_TYPE_Q6_K) {
            const uint8_t *h5a = wqh + (wrow + gid) * GM_WH_STRIDE, *h5b = h5a + 8 * GM_WH_STRIDE;
            uint32_t ha0 = 0, ha1 = 0, hb0 = 0, hb1 = 0;
            if (T == CERA_TYPE_Q5_K) {
                ha0 = *reinterpret_cast<const uint32_t *>(h5a + 4 * tig);
                ha1 = *reinterpret_cast<const uint32_t *>(h5a + 16 + 4 * tig);
                hb0 = *reinterpret_cast<const uint32_t *>(h5b + 4 * tig);
                hb1 = *reinterpret_cast<const uint32_t *>(h5b + 16 + 4 * tig);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                // 32-byte group g: low nibbles = sub-block 2g, high nibbles = sub-block 2g+1; byte l = element l
                const uint32_t wa0 = *reinterpret_cast<const uint32_t *>(qa + 32 * g + 4 * tig);
                const uint32_t wa1 = *reinterpret_cast<const uint32_t *>(qa + 32 * g + 16 + 4 * tig);
                const uint32_t wb0 = *reinterpret_cast<const uint32_t *>(qb + 32 * g + 4 * tig);
                const uint32_t wb1 = *reinterpret_cast<const uint32_t *>(qb + 32 * g + 16 + 4 * tig);
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int s = 2 * g + hi, sh = 4 * hi;
                    uint32_t a[4] = {(wa0 >> sh) & 0x0F0F0F0Fu, (wb0 >> sh) & 0x0F0F0F0Fu, (wa1 >> sh) & 0x0F0F0F0Fu,
                                     (wb1 >> sh) & 0x0F0F0F0Fu};
                    if (T == CERA_TYPE_Q5_K) {  // q = nibble + 16 * bit s of the high-bit byte (cera/src/quant.rs:846-866)
                        a[0] |= ((ha0 >> s) & 0x01010101u) << 4;
                        a[1] |= ((hb0 >> s) & 0x01010101u) << 4;
                        a[2] |= ((ha1 >> s) & 0x01010101u) << 4;
                        a[3] |= ((hb1 >> s) & 0x01010101u) << 4;
                    }
                    const float sca = wsc[(wrow + gid) * 16 + s], scb = wsc[(wrow + gid + 8) * 16 + s];
                    const float mna = wmn[(wrow + gid) * 8 + s], mnb = wmn[(wrow + gid + 8) * 8 + s];
                    const float2 sca2 = make_float2(sca, sca), scb2 = make_float2(scb, scb);
                    const float2 mna2 = make_float2(-mna, -mna), mnb2 = make_float2(-mnb, -mnb);
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const int cb = wcol + 8 * j;  // this n-tile's first column inside the CTA tile
                        const uint8_t *bp = aq + (cb + gid) * GM_AQ_STRIDE + 32 * s + 4 * tig;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp + 16);
                        int c[4];
                        mma_u8s8_k32(c, a, b0, b1);
                        const float2 xs = *reinterpret_cast<const float2 *>(axs + s * GM_BN + cb + 2 * tig);
                        const float2 xb = *reinterpret_cast<const float2 *>(axb + s * GM_BN + cb + 2 * tig);
                        rescale_pair(acc[j][0], sca2, mna2, xs, xb, c[0], c[1]);
                        rescale_pair(acc[j][1], scb2, mnb2, xs, xb, c[2], c[3]);
                    }
                }
            }
        } else {
            const uint8_t *ha = wqh + (wrow + gid) * GM_WH_STRIDE, *hb = ha + 8 * GM_WH_STRIDE;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                // scale group e = 8*nh + 2*g + half: elements [16e, 16e+16) of the super-block
                const int nh = e >> 3, g = (e >> 1) & 3, half = e & 1;
                const int qo = 64 * nh + 32 * (g & 1) + 16 * half + 4 * tig, ho = 32 * nh + 16 * half + 4 * tig;
                const int nsh = g >= 2 ? 4 : 0;
                const uint32_t la = *reinterpret_cast<const uint32_t *>(qa + qo), lb = *reinterpret_cast<const uint32_t *>(qb + qo);
                const uint32_t hha = *reinterpret_cast<const uint32_t *>(ha + ho), hhb = *reinterpret_cast<const uint32_t *>(hb + ho);
                const uint32_t a0 = ((la >> nsh) & 0x0F0F0F0Fu) | (((hha >> (2 * g)) & 0x03030303u) << 4);
                const uint32_t a1 = ((lb >> nsh) & 0x0F0F0F0Fu) | (((hhb >> (2 * g)) & 0x03030303u) << 4);
                const float sca = wsc[(wrow + gid) * 16 + e], scb = wsc[(wrow + gid + 8) * 16 + e];
                const float2 sca2 = make_float2(sca, sca), scb2 = make_float2(scb, scb);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int cb = wcol + 8 * j;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(aq + (cb + gid) * GM_AQ_STRIDE + 16 * e + 4 * tig);
                    int c[4];
                    mma_u8s8_k16(c, a0, a1, b0);
                    const float2 xs = *reinterpret_cast<const float2 *>(axs + (e >> 1) * GM_BN + cb + 2 * tig);
                    const float2 xb = *reinterpret_cast<const float2 *>(axb + e * GM_BN + cb + 2 * tig);
                    rescale_pair_q6(acc[j][0], sca2, xs, xb, c[0], c[1]);
                    rescale_pair_q6(acc[j][1], scb2, xs, xb, c[2], c[3]);
                }
            }
        }
        __syncthreads();  // the staging buffers are rewritten by the next chunk
    }

    // ---- combine the k shares of the cluster and store: cell (row, col) at out[row*ldy + col*ldc]
    if (CL == 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t row = row0 + wrow + gid + (i >= 2 ? 8 : 0);
                const uint32_t col = col0 + wcol + 8 * j + 2 * tig + (i & 1);
                if (row < p.m && col < n_cols) {
                    float *y = p.out + (size_t)row * p.ldy + (size_t)col * p.ldc;
                    const float v = (i & 1) ? acc[j][i >> 1].y : acc[j][i >> 1].x;
                    *y = p.epilogue == EPI_ADD ? __fadd_rn(*y, v) : v;
                }
            }
        return;
    }
    float *tile = reinterpret_cast<float *>(smem);  // [64][BN]; the last chunk's trailing barrier freed the staging buffers
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            tile[(wrow + gid + (i >= 2 ? 8 : 0)) * GM_BN + wcol + 8 * j + 2 * tig + (i & 1)] = (i & 1) ? acc[j][i >> 1].y : acc[j][i >> 1].x;
    cluster.sync();
    const uint32_t rows_each = GM_BM / CL;  // CL is 2, 4 or 8
    for (uint32_t idx = tid; idx < rows_each * GM_BN; idx += GM_THREADS) {
        const uint32_t r = crank * rows_each + idx / GM_BN, c = idx % GM_BN;
        float v = 0.0f;
        for (uint32_t q = 0; q < CL; ++q) v += cluster.map_shared_rank(tile, q)[r * GM_BN + c];
        const uint32_t row = row0 + r, col = col0 + c;
        if (row < p.m && col < n_cols) {
            float *y = p.out + (size_t)row * p.ldy + (size_t)col * p.ldc;
            *y = p.epilogue == EPI_ADD ? __fadd_rn(*y, v) : v;
        }
    }
    cluster.sync();  // peers may still be reading this CTA's partial tile
}

inline bool mma_type(int t) {
    return t == CERA_TYPE_Q4_0 || t == CERA_TYPE_Q4_K || t == CERA_TYPE_Q5_K || t == CERA_TYPE_Q6_K;
}

// grid_x / grid_y given: the expert-grouped form (row tiles of one expert x work items); else derived from m and n.
template <int T, int BN>
int32_t launch_mma_bn(const GemmParams &p, uint32_t cl, cudaStream_t st, uint32_t grid_x = 0, uint32_t grid_y = 0) {
    constexpr size_t smem = gm_smem_bytes<BN>();
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemm_mma_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid_x ? dim3(grid_x * cl, grid_y) : dim3(((p.m + GM_BM - 1) / GM_BM) * cl, (p.n + BN - 1) / BN);
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    count_launch();
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_mma_kernel<T, BN>, p), "gemm (mma) launch");
}

template <int T>
int32_t launch_mma_typed(const GemmParams &p, cudaStream_t st) {
    // CERA_CUDA_GEMM_BN=64 caps the column-tile width (A/B runs: narrower tiles trade operand reuse for occupancy)
    static const uint32_t bn_cap = [] {
        const char *e = getenv("CERA_CUDA_GEMM_BN");
        const long v = e ? atol(e) : 0;
        return (uint32_t)(v == 16 || v == 32 || v == 64 ? v : 128);
    }();
    uint32_t bn = p.n > 64 ? 128 : p.n > 32 ? 64 : p.n > 16 ? 32 : 16;
    if (bn > bn_cap) bn = bn_cap;
    // Split k over a cluster until the grid covers the machine once (wide tiles: a CTA's chunk is compute-heavy and a
    // split only adds the reduction), twice (64 columns) or four times (narrow tiles: a chunk is mostly load latency),
    // keeping at least two super-blocks per CTA.
    const uint32_t tiles = ((p.m + GM_BM - 1) / GM_BM) * ((p.n + bn - 1) / bn);
    const uint32_t want = (uint32_t)sm_count() * (bn >= 128 ? 1u : bn == 64 ? 2u : 4u);
    uint32_t cl = 1;
    while (cl < 8 && tiles * cl < want && (p.k >> 8) / (cl * 2) >= 2) cl *= 2;
    // Wave quantization: with two CTAs resident per SM, a grid of 1.5 (or 3.03) times that many wide tiles leaves the
    // machine nearly empty for its last round.  Splitting k over a cluster makes the rounds shorter, so the ragged last
    // one costs less than the reduction adds (14336 x 4096 x 256 columns: 295 -> 265 us with clusters of 4).
    if (cl == 1 && bn == 128) {
        const uint32_t slots = (uint32_t)sm_count() * 2, rounds = tiles / slots, rest = tiles % slots;
        if (rounds >= 1 && rounds <= 3 && rest != 0 && rest * 10 < slots * 6) {
            const uint32_t split = rounds == 1 ? 4u : 2u;
            if ((p.k >> 8) / (split * 2) >= 2) cl = split;
        }
    }
    switch (bn) {
        case 128: return launch_mma_bn<T, 128>(p, cl, st);
        case 64: return launch_mma_bn<T, 64>(p, cl, st);
        case 32: return launch_mma_bn<T, 32>(p, cl, st);
        default: return launch_mma_bn<T, 16>(p, cl, st);
    }
}

}  // namespace

// Tensor-core GEMM for Q4_K / Q5_K / Q6_K weights and n >= 5 columns.  *taken = false: not this kernel's case.
int32_t launch_gemm_mma(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                        cudaStream_t st, bool *taken) {
    *taken = false;
    static const bool off = [] {
        const char *e = getenv("CERA_CUDA_GEMM");
        return e && strcmp(e, "columns") == 0;
    }();
    if (off || n < 5 || !mma_type(w.type) || w.k % 256) return CERA_CUDA_OK;
    if ((uintptr_t)x.quants % 16 || w.k % 16) return CERA_CUDA_OK;
    GemmParams p{};
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
    if (w.type == CERA_TYPE_Q4_0) return launch_mma_typed<CERA_TYPE_Q4_0>(p, st);
    if (w.type == CERA_TYPE_Q4_K) return launch_mma_typed<CERA_TYPE_Q4_K>(p, st);
    if (w.type == CERA_TYPE_Q5_K) return launch_mma_typed<CERA_TYPE_Q5_K>(p, st);
    return launch_mma_typed<CERA_TYPE_Q6_K>(p, st);
}

bool gemm_mma_supports(int type, size_t k) { return mma_type(type) && k % 256 == 0; }

// Expert-grouped form: one 64-column tile per work item of a device-side list (see ops.h).
int32_t launch_gemm_mma_grouped(const WeightView &w, const ActView &x, const MoeTile *tiles, const uint32_t *n_tiles,
                                uint32_t max_tiles, uint32_t rows_per_expert, float *out, size_t ldc, uint32_t bn, cudaStream_t st,
                                bool *taken) {
    *taken = false;
    if (!mma_type(w.type) || w.k % 256 || (uintptr_t)x.quants % 16 || max_tiles == 0) return CERA_CUDA_OK;
    GemmParams p{};
    p.w = w;
    p.x = x;
    p.out = out;
    p.m = rows_per_expert;
    p.n = 0;
    p.k = w.k;
    p.ldy = 1;
    p.ldc = (uint32_t)ldc;
    p.epilogue = EPI_STORE;
    p.tiles = tiles;
    p.n_tiles = n_tiles;
    *taken = true;
    const uint32_t row_tiles = (rows_per_expert + GM_BM - 1) / GM_BM;
#define CERA_GROUPED(TT)                                                                     \
    return bn == 32 ? launch_mma_bn<TT, 32>(p, 1, st, row_tiles, max_tiles) : launch_mma_bn<TT, 64>(p, 1, st, row_tiles, max_tiles)
    if (w.type == CERA_TYPE_Q4_0) CERA_GROUPED(CERA_TYPE_Q4_0);
    if (w.type == CERA_TYPE_Q4_K) CERA_GROUPED(CERA_TYPE_Q4_K);
    if (w.type == CERA_TYPE_Q5_K) CERA_GROUPED(CERA_TYPE_Q5_K);
    CERA_GROUPED(CERA_TYPE_Q6_K);
#undef CERA_GROUPED
}

}  // namespace cera
