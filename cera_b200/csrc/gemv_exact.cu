// Decode GEMV for the K-quants (Q4_K, Q5_K, Q6_K) whose f32 results are BIT-IDENTICAL to the
// reference's x86 int8 kernels at one activation column (cera/src/backend/simd.rs:5693-5878 Q4_K,
// 5988-6195 Q6_K, the n == 1 path): not only the per-block integer sums but the whole f32
// combination is evaluated in the reference's order.
//
// The reference keeps, per output row, four round-robin accumulators of eight f32 lanes: 32-element
// activation block xb of the row goes to accumulator (xb mod 4); its lane L receives, by one fused
// multiply-add, (float)(sum of the four products of elements 4L..4L+3) x (block scale).  That is 32
// independent FMA chains per row, each walking the row's blocks in order, plus one scalar chain
// `macc` that adds one min / offset term per block, in block order.  At the end the four accumulators
// are tree-added, the eight lanes are added in the hsum256 order and macc is subtracted.
//
// Mapping.  A row's low-quant plane is four STRIPS: strip c collects piece c (sixteen bytes) of every
// 128-weight task t of the row, in task order.  Piece c = (pair, half) of task t holds, for
// Q4_K / Q5_K, sixteen bytes whose low nibbles are elements [16*half, 16*half+16) of block
// 4t + 2*pair and whose high nibbles are the same elements of block 4t + 2*pair + 1; for Q6_K the low
// nibbles belong to block 4t + pair and the high nibbles to block 4t + pair + 2.  Either way the four
// words of a piece feed eight chains - two accumulators x four lanes - that no other strip touches.
// So ONE LANE OWNS ONE STRIP of one row and carries its eight chains in registers; four lanes cover a
// row, a warp eight rows.  The planes interleave groups of eight rows (WeightView::ilv), task by
// task, so what a warp needs for eight consecutive tasks of its eight rows is ONE contiguous 4 KB
// range of the low-quant plane (plus 512 contiguous bytes of headers, and for Q5_K / Q6_K the
// matching high-bit ranges): a SEGMENT.
//
// Data movement.  Every warp owns a ring of segment buffers in shared memory, filled by bulk
// asynchronous copies (cp.async.bulk, the TMA unit) that one lane issues and an mbarrier counts.  The
// first segments are requested before the kernel waits for its predecessor (weights never change), and
// the ring keeps several segments per warp in flight whatever the register budget, across the warp's
// rounds.  Lanes read their pieces back with conflict-free 128-bit shared loads.
//
// Arithmetic.  Per task a lane forms the two f32 block scales  xs*(d*sc)  and one macc term exactly as
// the reference forms them, then, per 4 weights: one mask, one dp4a whose accumulator input is
// the bit pattern of 1.5 * 2^23 (so the integer sum arrives as a float: an exact conversion without a
// convert instruction), one subtraction of that constant and one FMA.  Operands come from shared memory
// one task ahead of their use.  The macc terms go to shared
// memory and are summed, one row per lane, by a fifth warp that trails the others segment by segment
// (named barriers) and finally subtracts, applies the epilogue and stores.
//
// Every wait on a copy is bounded; if a limit runs out the CTA's waits give up, the affected rows are
// left unwritten and a status word (cera_cuda_kernel_status) reports it.
#include <cstdlib>
#include <cstring>

#include "gemv_task.cuh"
#include "tma.cuh"

namespace cera {

__device__ unsigned int g_xg_status = 0;

namespace {

constexpr int XG_MAX_PRODUCERS = 8;                  // warps that stream and multiply (3..8 per CTA, picked per launch), + one chain warp
constexpr int XG_MAX_SEGS = 3;
constexpr int XG_SEG_TASKS = 4;                      // tasks (of 128 weights) per segment: two super-blocks
constexpr int XG_HAND_TASKS = 8;                     // tasks per hand-over of macc terms to the chain warp
constexpr int XG_MAX_HANDS = 14;                     // hand-overs per row: named barriers 1..14, 15 = row values ready
constexpr int XG_MAX_STAGES = 8;
constexpr int XG_HEAD_BYTES = 1024;                  // barriers [8][8] and the abort flag
constexpr int XG_MAGIC_I = 0x4B400000;               // bits of 12582912.0f = 1.5 * 2^23
constexpr float XG_MAGIC_F = 12582912.0f;

struct ExactParams {
    WeightView w[XG_MAX_SEGS];
    float *y[XG_MAX_SEGS];
    uint32_t row_end[XG_MAX_SEGS];
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k;
    int epilogue;
    int stages;
    GemvFusion f;
    TpHook tp;
};

template <int T>
struct SegLayout {  // bytes of one segment buffer
    static constexpr uint32_t SB = XG_SEG_TASKS / 2;                                         // super-blocks per segment
    static constexpr uint32_t Q = XG_SEG_TASKS * 512;                                        // tasks x 32 pieces
    static constexpr uint32_t HDR = SB * 8 * 16;                                             // super-blocks x 8 rows
    static constexpr uint32_t QH = T == CERA_TYPE_Q5_K ? SB * 8 * 32 : T == CERA_TYPE_Q6_K ? SB * 8 * 64 : 0;
    static constexpr uint32_t D = T == CERA_TYPE_Q6_K ? SB * 8 * 2 : 0;
    static constexpr uint32_t OFF_HDR = Q, OFF_QH = Q + HDR, OFF_D = Q + HDR + QH;
    static constexpr uint32_t BYTES = (Q + HDR + QH + D + 127) / 128 * 128;
    static constexpr uint32_t TX = Q + HDR + QH + D;
};

// Named barriers with literal ids.
#define XG_BAR(op, id) asm volatile(op " " #id ", %0;" ::"r"(nthreads) : "memory")
#define XG_BAR_SWITCH(op)                        \
    switch (id) {                                \
        case 1: XG_BAR(op, 1); break;            \
        case 2: XG_BAR(op, 2); break;            \
        case 3: XG_BAR(op, 3); break;            \
        case 4: XG_BAR(op, 4); break;            \
        case 5: XG_BAR(op, 5); break;            \
        case 6: XG_BAR(op, 6); break;            \
        case 7: XG_BAR(op, 7); break;            \
        case 8: XG_BAR(op, 8); break;            \
        case 9: XG_BAR(op, 9); break;            \
        case 10: XG_BAR(op, 10); break;          \
        case 11: XG_BAR(op, 11); break;          \
        case 12: XG_BAR(op, 12); break;          \
        case 13: XG_BAR(op, 13); break;          \
        case 14: XG_BAR(op, 14); break;          \
        default: XG_BAR(op, 15); break;          \
    }
__device__ __forceinline__ void bar_arrive(int id, int nthreads) { XG_BAR_SWITCH("bar.arrive") }
__device__ __forceinline__ void bar_sync(int id, int nthreads) { XG_BAR_SWITCH("bar.sync") }

// (float)(sum of four u8 x s8 products), exactly: the dp4a accumulates onto the bits of 1.5 * 2^23.
__device__ __forceinline__ float quad_dot(uint32_t w, int a) { return __fsub_rn(__int_as_float(dp_us(w, a, XG_MAGIC_I)), XG_MAGIC_F); }
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ int word_of(const int4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
// Small unsigned integer -> float without the convert pipe: 2^23 + v as bits, minus 2^23.
__device__ __forceinline__ float small_uint_f(uint32_t v) { return __fsub_rn(__uint_as_float(0x4B000000u | v), 8388608.0f); }

__host__ __device__ inline size_t xg_fixed_smem(uint32_t k, uint32_t P) {  // everything but the rings
    return XG_HEAD_BYTES + (size_t)k + (size_t)(k / 32) * 4 * 2 + (size_t)(k / 16) * 4 + (size_t)8 * P * (k / 32 + 4) * 4 + 8 * P * 4;
}

template <int T>
__global__ void __launch_bounds__((XG_MAX_PRODUCERS + 1) * 32) gemv_exact_kernel(const ExactParams p) {
    using L = SegLayout<T>;
    extern __shared__ __align__(128) uint8_t xg_smem[];
    const uint32_t k = p.k, nb32 = k >> 5, nb = k >> 8, n_seg = k / (128 * XG_SEG_TASKS);
    const uint32_t S = 1u << p.stages, s_mask = S - 1, s_shift = (uint32_t)p.stages;  // ring depth, a power of two
    const int nthreads = blockDim.x;
    const uint32_t P = blockDim.x / 32 - 1, XG_ROWS = 8 * P;  // producer warps, rows per round
    // carve-up: rings first (128-byte aligned buffers), then the barriers, the activation column and the per-round tables
    uint8_t *rings = xg_smem;
    uint8_t *fixed = rings + (size_t)P * S * L::BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(fixed);                     // [P][XG_MAX_STAGES]
    volatile uint32_t *abort_flag = reinterpret_cast<uint32_t *>(fixed + XG_HEAD_BYTES - 8);
    int8_t *aq = reinterpret_cast<int8_t *>(fixed + XG_HEAD_BYTES);           // [k]
    float *xs = reinterpret_cast<float *>(fixed + XG_HEAD_BYTES + k);         // [k/32]
    float *a32 = xs + nb32;                                                   // [k/32] sum of the block's quants
    float *a16 = a32 + nb32;                                                  // [k/16]
    const uint32_t tstride = nb32 + 4;  // row stride of the term table: a producer warp's 8 rows x 4 blocks fall in 32 distinct banks
    float *terms = a16 + 2 * nb32;                                            // [XG_ROWS][tstride]
    float *hs = terms + (size_t)XG_ROWS * tstride;                         // [XG_ROWS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = (uint32_t)warp < P;
    const uint32_t n_rounds = (p.total_rows + XG_ROWS - 1) / XG_ROWS;
    const uint32_t my_rounds = blockIdx.x < n_rounds ? (n_rounds - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t n_items = my_rounds * n_seg;  // segments this warp walks, over all its rounds

    if (tid == 0) *abort_flag = 0;
    if (producer && lane == 0)
        for (uint32_t s = 0; s < S; ++s) tma::mbar_init(bars + warp * XG_MAX_STAGES + s, 1);
    if (tid == 0) tma::mbar_init_fence();
    __syncthreads();

    // Issues the copies of this warp's next item (lane 0 only); items are walked in order, so the source addresses of
    // the round's row group are worked out once per round.
    uint8_t *ring = rings + (size_t)warp * S * L::BYTES;
    uint32_t is_j = 0, is_seg = 0, is_round = blockIdx.x;  // next item to request: index, segment, round
    const uint8_t *is_q = nullptr, *is_hdr = nullptr, *is_qh = nullptr, *is_d = nullptr;
    auto issue_next = [&]() {
        if (is_seg == 0) {
            uint32_t row = is_round * XG_ROWS + warp * 8;
            if (row >= p.total_rows) row = (p.total_rows - 1) & ~7u;  // a group past the end repeats the last one; nothing of it is stored
            int sg = 0;
            while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
            const uint32_t local = row - (sg ? p.row_end[sg - 1] : 0);
            const WeightView &w = p.w[sg];
            const size_t grp = local >> 3, sb0 = grp * nb * 8;  // first (super-block, row) slot of the group in the per-block planes
            is_q = w.q + grp * 8 * ((size_t)nb * 128);
            is_hdr = w.hdr + sb0 * 16;
            is_qh = L::QH ? w.qh + sb0 * (L::QH / (L::SB * 8)) : nullptr;
            is_d = L::D ? w.d + sb0 * 2 : nullptr;
        }
        uint8_t *dst = ring + (size_t)(is_j & s_mask) * L::BYTES;
        uint64_t *bar = bars + warp * XG_MAX_STAGES + (is_j & s_mask);
        tma::mbar_expect_tx(bar, L::TX);
        tma::bulk_g2s(dst, is_q + (size_t)is_seg * L::Q, L::Q, bar);
        tma::bulk_g2s(dst + L::OFF_HDR, is_hdr + (size_t)is_seg * L::HDR, L::HDR, bar);
        if (L::QH) tma::bulk_g2s(dst + L::OFF_QH, is_qh + (size_t)is_seg * L::QH, L::QH, bar);
        if (L::D) tma::bulk_g2s(dst + L::OFF_D, is_d + (size_t)is_seg * L::D, L::D, bar);
        ++is_j;
        if (++is_seg == n_seg) {
            is_seg = 0;
            is_round += gridDim.x;
        }
    };
    // weights do not depend on the previous kernel: fill the ring before waiting for it
    if (producer && lane == 0)
        for (uint32_t j = 0; j + 1 < S && j < n_items; ++j) issue_next();

    pdl_trigger();
    pdl_wait();
    tp_arrive_wait(p.tp.ctx, p.tp.wait_slot);
    // stage the activation column
    for (uint32_t i = tid; i < k / 16; i += nthreads) {
        reinterpret_cast<int4 *>(aq)[i] = reinterpret_cast<const int4 *>(p.x.quants)[i];
        a16[i] = (float)p.x.sums[i];
    }
    for (uint32_t i = tid; i < nb32; i += nthreads) {
        xs[i] = p.x.scales[i];
        a32[i] = (float)((int)p.x.sums[2 * i] + (int)p.x.sums[2 * i + 1]);
    }
    __syncthreads();

    uint32_t item = 0;
    for (uint32_t round = blockIdx.x; round < n_rounds; round += gridDim.x) {
        const uint32_t base = round * XG_ROWS;
        if (producer) {
            const int rr = lane >> 2, rslot = warp * 8 + rr, c = lane & 3, pair = c >> 1, half = c & 1;
            float *tr = terms + (size_t)rslot * tstride;
            float acc_lo[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc_hi[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            bool ok = true;
            for (uint32_t seg = 0; seg < n_seg; ++seg, ++item) {
                const uint8_t *buf = ring + (size_t)(item & s_mask) * L::BYTES;
                if (ok && !tma::mbar_wait_blocking(bars + warp * XG_MAX_STAGES + (item & s_mask), (item >> s_shift) & 1, abort_flag, &g_xg_status, 1u)) ok = false;
                if (ok) {
                    // Eight tasks, this lane's strip.  Everything a task needs from shared memory (piece, header, high
                    // bits, activation words, block scales and sums) is fetched one task ahead of its arithmetic, and
                    // a task's own work is independent of its neighbours' except for the eight chain FMAs.
                    struct Ops {
                        uint4 piece, hdr, hb;
                        int4 alo, ahi;
                        float xs_lo, xs_hi, am0, am1;  // block scales of the two blocks; sums for this lane's macc term
                        float d6;                      // Q6_K super-block scale
                    };
                    auto fetch = [&](int i) {
                        Ops o;
                        const uint32_t t = seg * XG_SEG_TASKS + i;
                        const int sbl = i >> 1;
                        o.piece = *reinterpret_cast<const uint4 *>(buf + (i * 32 + lane) * 16);
                        o.hdr = *reinterpret_cast<const uint4 *>(buf + L::OFF_HDR + (sbl * 8 + rr) * 16);
                        o.hb = make_uint4(0, 0, 0, 0);
                        o.d6 = 0.0f;
                        if (T == CERA_TYPE_Q6_K) {
                            // low nibbles block 4t + pair, high nibbles block 4t + pair + 2; task = (super-block i/2, half i&1)
                            const uint32_t xb_lo = 4 * t + pair, xb_hi = xb_lo + 2, xbm = half ? xb_hi : xb_lo;
                            o.alo = *reinterpret_cast<const int4 *>(aq + 32 * xb_lo + 16 * half);
                            o.ahi = *reinterpret_cast<const int4 *>(aq + 32 * xb_hi + 16 * half);
                            o.xs_lo = xs[xb_lo];
                            o.xs_hi = xs[xb_hi];
                            const float2 am = *reinterpret_cast<const float2 *>(a16 + 2 * xbm);
                            o.am0 = am.x;
                            o.am1 = am.y;
                            o.hb = *reinterpret_cast<const uint4 *>(buf + L::OFF_QH + (sbl * 8 + rr) * 64 + (i & 1) * 32 + half * 16);
                            o.d6 = h2f(*reinterpret_cast<const uint16_t *>(buf + L::OFF_D + (sbl * 8 + rr) * 2));
                        } else {
                            // low nibbles: block 4t + 2*pair, high nibbles: the next one
                            const uint32_t xb_lo = 4 * t + 2 * pair;
                            o.alo = *reinterpret_cast<const int4 *>(aq + 32 * xb_lo + 16 * half);
                            o.ahi = *reinterpret_cast<const int4 *>(aq + 32 * xb_lo + 32 + 16 * half);
                            const float2 x2 = *reinterpret_cast<const float2 *>(xs + xb_lo);
                            o.xs_lo = x2.x;
                            o.xs_hi = x2.y;
                            o.am0 = a32[xb_lo + half];
                            o.am1 = 0.0f;
                            if (T == CERA_TYPE_Q5_K) o.hb = *reinterpret_cast<const uint4 *>(buf + L::OFF_QH + (sbl * 8 + rr) * 32 + half * 16);
                        }
                        return o;
                    };
                    Ops cur = fetch(0);
#pragma unroll
                    for (int i = 0; i < XG_SEG_TASKS; ++i) {
                        Ops nxt = cur;
                        if (i + 1 < XG_SEG_TASKS) nxt = fetch(i + 1);
                        const uint32_t t = seg * XG_SEG_TASKS + i, hf = i & 1;
                        float sc_lo, sc_hi, term;
                        uint32_t xbm;
                        if (T == CERA_TYPE_Q6_K) {
                            // cur.hdr = the 16 int8 scales of the super-block; block (nh, g) uses scales 8nh + 2g (+1 for lanes 4-7)
                            const uint32_t sw_lo = hf ? cur.hdr.z : cur.hdr.x, sw_hi = hf ? cur.hdr.w : cur.hdr.y;  // [8nh, +4), [8nh+4, +4)
                            const float s_lo = (float)(int8_t)(sw_lo >> (8 * (2 * pair + half))), s_hi = (float)(int8_t)(sw_hi >> (8 * (2 * pair + half)));
                            sc_lo = __fmul_rn(__fmul_rn(s_lo, cur.d6), cur.xs_lo);
                            sc_hi = __fmul_rn(__fmul_rn(s_hi, cur.d6), cur.xs_hi);
                            // this lane's macc term: block xbm = the low-nibble block (half 0) or the high-nibble one (half 1)
                            const uint32_t swm = half ? sw_hi : sw_lo;
                            const float m0 = (float)(int8_t)(swm >> (8 * (2 * pair))), m1 = (float)(int8_t)(swm >> (8 * (2 * pair + 1)));
                            const float inner = __fadd_rn(__fmul_rn(m0, cur.am0), __fmul_rn(m1, cur.am1));
                            term = __fmul_rn(__fmul_rn(half ? cur.xs_hi : cur.xs_lo, __fmul_rn(cur.d6, 32.0f)), inner);
                            xbm = 4 * t + pair + 2 * half;
                        } else {
                            uint32_t scp, mnp;
                            kq_quad(cur.hdr, hf, scp, mnp);
                            const float d = h2f((uint16_t)(cur.hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(cur.hdr.x >> 16));
                            sc_lo = __fmul_rn(cur.xs_lo, __fmul_rn(d, small_uint_f((scp >> (16 * pair)) & 0xFF)));
                            sc_hi = __fmul_rn(cur.xs_hi, __fmul_rn(d, small_uint_f((scp >> (16 * pair + 8)) & 0xFF)));
                            const float mn = small_uint_f((mnp >> (16 * pair + 8 * half)) & 0xFF);
                            term = __fmul_rn(__fmul_rn(half ? cur.xs_hi : cur.xs_lo, __fmul_rn(dmin, mn)), cur.am0);
                            xbm = 4 * t + 2 * pair + half;
                        }
                        tr[xbm] = term;
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) {
                            const uint32_t v = word_of(cur.piece, wd), b = word_of(cur.hb, wd);
                            lo[wd] = v & 0x0F0F0F0Fu;
                            hi[wd] = (v >> 4) & 0x0F0F0F0Fu;
                            if (T == CERA_TYPE_Q5_K) {
                                const int sh_lo = 4 * hf + 2 * pair;  // fifth-bit position of the low-nibble sub-block
                                lo[wd] |= ((b >> sh_lo) & 0x01010101u) << 4;
                                hi[wd] |= ((b >> (sh_lo + 1)) & 0x01010101u) << 4;
                            }
                            if (T == CERA_TYPE_Q6_K) {
                                lo[wd] |= ((b >> (2 * pair)) & 0x03030303u) << 4;
                                hi[wd] |= ((b >> (2 * pair + 4)) & 0x03030303u) << 4;
                            }
                        }
                        float ql[4], qh[4];
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) {
                            ql[wd] = quad_dot(lo[wd], word_of(cur.alo, wd));
                            qh[wd] = quad_dot(hi[wd], word_of(cur.ahi, wd));
                        }
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) {
                            acc_lo[wd] = fmaf(ql[wd], sc_lo, acc_lo[wd]);
                            acc_hi[wd] = fmaf(qh[wd], sc_hi, acc_hi[wd]);
                        }
                        cur = nxt;
                    }
                }
                __syncwarp();  // every lane is done with this buffer
                if (lane == 0 && item + S - 1 < n_items) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue_next();
                }
                if ((seg + 1) % (XG_HAND_TASKS / XG_SEG_TASKS) == 0) {
                    __threadfence_block();
                    bar_arrive(1 + (int)(seg / (XG_HAND_TASKS / XG_SEG_TASKS)), nthreads);  // the chain warp may add these 32 blocks' terms
                }
            }
            // ---- the 32 chains of the row -> one value (tree over the accumulators, then the hsum256 order)
            float f[4];
            if (T == CERA_TYPE_Q6_K) {
                // lane (pair, half): acc_lo = accumulator `pair`, acc_hi = accumulator `pair + 2`
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    const float u = __fadd_rn(acc_lo[wd], __shfl_xor_sync(0xffffffffu, acc_lo[wd], 2));  // acc0 + acc1
                    const float z = __fadd_rn(acc_hi[wd], __shfl_xor_sync(0xffffffffu, acc_hi[wd], 2));  // acc2 + acc3
                    f[wd] = __fadd_rn(u, z);
                }
            } else {
                // lane (pair, half): acc_lo = accumulator 2*pair, acc_hi = accumulator 2*pair + 1
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    const float v = __fadd_rn(acc_lo[wd], acc_hi[wd]);
                    const float o = __shfl_xor_sync(0xffffffffu, v, 2);
                    f[wd] = pair ? __fadd_rn(o, v) : __fadd_rn(v, o);  // (acc0 + acc1) + (acc2 + acc3)
                }
            }
            // f[wd] is lane 4*half + wd of the summed accumulator: hsum256 adds lanes i and i+4, then (0,2), (1,3), then the two
            float sp[4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                const float o = __shfl_xor_sync(0xffffffffu, f[wd], 1);
                sp[wd] = half ? __fadd_rn(f[wd], o) : __fadd_rn(o, f[wd]);  // v[i+4] + v[i]
            }
            const float hsum = __fadd_rn(__fadd_rn(sp[0], sp[2]), __fadd_rn(sp[1], sp[3]));
            if (c == 0) hs[rslot] = ok ? hsum : __int_as_float(0x7FC00000);
            __threadfence_block();
            bar_arrive(15, nthreads);
        } else {
            // ---- chain warp: lane i owns rows base + i and, in rounds of more than 32 rows, base + 32 + i
            const uint32_t n_hand = k / (128 * XG_HAND_TASKS);
            const bool two = XG_ROWS > 32;
            const float4 *tr0 = reinterpret_cast<const float4 *>(terms + (size_t)(lane < XG_ROWS ? lane : 0) * tstride);
            const float4 *tr1 = reinterpret_cast<const float4 *>(terms + (size_t)(lane + 32 < XG_ROWS ? lane + 32 : 0) * tstride);
            float macc0 = 0.0f, macc1 = 0.0f;
            for (uint32_t hand = 0; hand < n_hand; ++hand) {
                bar_sync(1 + (int)hand, nthreads);
#pragma unroll
                for (uint32_t q = 0; q < 8; ++q) {
                    const float4 u = tr0[hand * 8 + q];
                    macc0 = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(macc0, u.x), u.y), u.z), u.w);
                    if (two) {
                        const float4 v = tr1[hand * 8 + q];
                        macc1 = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(macc1, v.x), v.y), v.z), v.w);
                    }
                }
            }
            bar_sync(15, nthreads);
            for (uint32_t rsel = 0; rsel < (two ? 2u : 1u); ++rsel) {
                const uint32_t rslot = lane + 32 * rsel;
                const uint32_t row = base + rslot;
                const float hv = rslot < XG_ROWS ? hs[rslot] : __int_as_float(0x7FC00000);
                const bool valid = rslot < XG_ROWS && row < p.total_rows && hv == hv;  // NaN marks a row whose copies never arrived
                const float r = __fsub_rn(hv, rsel ? macc1 : macc0);
                int sg = 0;
                while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
                const uint32_t local = row - (sg ? p.row_end[sg - 1] : 0);
                if (p.epilogue == EPI_ROPE_KV) {
                    // rows (2i, 2i+1) of a head are a NORM rotation pair (cera/src/backend/cpu.rs:5161-5180): adjacent lanes
                    const float other = __shfl_xor_sync(0xffffffffu, r, 1);
                    if (valid) {
                        const uint32_t pos = *p.f.pos_dev;
                        if (sg == 2) {
                            store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + local, r);
                        } else {
                            const uint32_t pi = (local % p.f.head_dim) >> 1;
                            const float *cs_sn = p.f.rope_cs + ((p.f.rope_by_pos ? (size_t)pos * (p.f.head_dim >> 1) : 0) + pi) * 2;
                            const float cs = cs_sn[0], sn = cs_sn[1];
                            const float x0 = (lane & 1) ? other : r, x1 = (lane & 1) ? r : other;
                            const float out = (lane & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs))
                                                         : __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
                            if (sg == 0) p.y[0][local] = out;
                            else store_kv(p.f.k_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + local, out);
                        }
                    }
                } else if (valid) {
                    float *y = p.y[sg] + local;
                    const float out = p.epilogue == EPI_ADD ? __fadd_rn(*y, r) : r;
                    *y = out;
                    if (p.tp.push) tp_push(p.tp.ctx, y, out);
                }
            }
        }
        __syncthreads();  // the terms of this round are consumed before the next round overwrites them
    }
}

template <int T>
int32_t launch_exact_typed(const ExactParams &p0, cudaStream_t st) {
    using L = SegLayout<T>;
    ExactParams p = p0;
    const uint32_t n_seg = p.k / (128 * XG_SEG_TASKS);
    (void)n_seg;
    // Producer warps per CTA (8 rows each) and ring depth (a power of two).  A CTA walks its rounds one after another, so
    // the launch takes `waves` rounds of whatever a round costs at that occupancy: about constant below a dozen producer
    // warps per SM (latency bound), proportional to their number above.  Among equal costs prefer enough copies in flight
    // to cover the memory latency (64 KB per SM), then the smaller CTA.
    const size_t sm_smem = 227 * 1024;
    const uint32_t sms = (uint32_t)sm_count();
    uint32_t best_P = 4, best_S = 1, best_slots = 1, best_rounds = 1;
    uint64_t best_cost = ~0ull, best_fly = 0;
    for (uint32_t P = 3; P <= XG_MAX_PRODUCERS; ++P) {
        for (uint32_t s_log = 1; s_log <= 3; ++s_log) {
            const size_t smem = xg_fixed_smem(p.k, P) + (size_t)P * (1u << s_log) * L::BYTES + 1024;
            if (smem > 200 * 1024) continue;
            uint32_t per_sm = (uint32_t)(sm_smem / smem);
            if (per_sm > 64 / (P + 1)) per_sm = 64 / (P + 1);
            if (per_sm == 0) continue;
            const uint32_t slots = sms * per_sm, rounds = (p.total_rows + 8 * P - 1) / (8 * P);
            const uint32_t waves = (rounds + slots - 1) / slots;
            const uint32_t resident = per_sm < (rounds + sms - 1) / sms ? per_sm : (rounds + sms - 1) / sms;
            const uint64_t warps = (uint64_t)resident * P, cost = waves * (warps > 12 ? warps : 12);
            uint64_t fly = (uint64_t)resident * P * ((1u << s_log) - 1) * L::BYTES;
            if (fly > 64 * 1024) fly = 64 * 1024;
            if (cost < best_cost || (cost == best_cost && fly > best_fly)) {
                best_cost = cost;
                best_fly = fly;
                best_P = P;
                best_S = s_log;
                best_slots = slots;
                best_rounds = rounds;
            }
        }
    }
    p.stages = (int)best_S;
    const size_t smem = xg_fixed_smem(p.k, best_P) + (size_t)best_P * (1u << best_S) * L::BYTES;
    static thread_local int raised_dev = -1;  // per instantiation: opt in to more than 48 KB once per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (raised_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemv_exact_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised_dev = dev;
    }
    // a balanced static schedule: every CTA walks the same number of rounds (the last of them may be missing)
    const uint32_t per_cta = (best_rounds + best_slots - 1) / best_slots;
    const uint32_t grid = (best_rounds + per_cta - 1) / per_cta;
    count_launch();
    return check_cuda(launch_k(gemv_exact_kernel<T>, dim3(grid), dim3((best_P + 1) * 32), smem, st, p), "gemv (reference order) launch");
}

}  // namespace

uint32_t gemv_exact_status() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_xg_status, sizeof(v));
    return v;
}

// CERA_CUDA_GEMV=rows keeps the decode GEMVs on the register-streaming kernel whose f32 order is its own (A/B runs); read once.
static bool exact_off() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_GEMV");
        return e && (strcmp(e, "rows") == 0 || strcmp(e, "tma") == 0 || strcmp(e, "direct") == 0);
    }();
    return v;
}

// Single-column GEMV in the reference's f32 order over up to three same-typed K-quant matrices.
// *taken = false: not a K-quant, k not a multiple of 1024, or a shape outside the kernel's rules;
// nothing was launched.
int32_t launch_gemv_exact(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp) {
    *taken = false;
    if (exact_off() || n_segs < 1 || n_segs > XG_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    if (type != CERA_TYPE_Q4_K && type != CERA_TYPE_Q5_K && type != CERA_TYPE_Q6_K) return CERA_CUDA_OK;
    const uint32_t k = segs[0].w.k;
    if (k % 1024 || (k >> 10) > XG_MAX_HANDS) return CERA_CUDA_OK;
    for (int i = 0; i < n_segs; ++i)
        if (segs[i].w.ilv != 8) return CERA_CUDA_OK;
    if (xg_fixed_smem(k, 3) + (size_t)3 * 2 * 4096 > 200 * 1024) return CERA_CUDA_OK;
    if ((uintptr_t)x.quants % 16) return CERA_CUDA_OK;
    ExactParams p{};
    if (fusion) p.f = *fusion;
    if (tp) p.tp = *tp;
    uint32_t rows = 0;
    for (int i = 0; i < n_segs; ++i) {
        if (segs[i].w.type != type || segs[i].w.k != k) return CERA_CUDA_OK;
        p.w[i] = segs[i].w;
        p.y[i] = segs[i].y;
        rows += segs[i].w.m;
        p.row_end[i] = rows;
    }
    for (int i = 0; i + 1 < n_segs; ++i)
        if (segs[i].w.m % 8) return CERA_CUDA_OK;  // a warp's eight rows must be one interleave group of one matrix
    if (epilogue == EPI_ROPE_KV) {
        if (n_segs != 3 || !p.f.rope_cs || !p.f.pos_dev || !p.f.k_cache || !p.f.v_cache || p.f.head_dim % 2 || segs[0].w.m % 32 ||
            segs[1].w.m % 32 || segs[2].w.m % 32)
            return CERA_CUDA_OK;
    }
    p.n_segs = n_segs;
    p.total_rows = rows;
    p.x = x;
    p.k = k;
    p.epilogue = epilogue;
    *taken = true;
    if (type == CERA_TYPE_Q4_K) return launch_exact_typed<CERA_TYPE_Q4_K>(p, st);
    if (type == CERA_TYPE_Q5_K) return launch_exact_typed<CERA_TYPE_Q5_K>(p, st);
    return launch_exact_typed<CERA_TYPE_Q6_K>(p, st);
}

}  // namespace cera
