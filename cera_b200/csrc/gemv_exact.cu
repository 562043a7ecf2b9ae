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
// row, a warp a GROUP of eight rows.  The planes interleave groups of eight rows (WeightView::ilv),
// task by task, so what a warp needs for four consecutive tasks of its group is ONE contiguous 2 KB
// range of the low-quant plane (plus 256 contiguous bytes of headers, and for Q5_K / Q6_K the
// matching high-bit ranges): a SEGMENT.
//
// Warps are independent.  Every warp owns a ring of segment buffers in shared memory, filled by bulk
// asynchronous copies (cp.async.bulk, the TMA unit) that its lane 0 issues and an mbarrier counts, a
// table of macc terms and a small table of block scales; it walks its share of the row groups on its
// own, with no CTA-wide barrier after the activation column has been staged.  The first segments are
// requested before the kernel waits for its predecessor (weights never change), and the ring keeps
// several segments per warp in flight across the warp's groups.  A launch puts one CTA on every SM
// with as many warps as the SM's share of the row groups (up to 32).
//
// Teams.  A matrix with few rows leaves an SM three or four groups, each a long serial walk over k
// for one warp.  There the launch forms TEAMS of W = 2 .. 16 warps per group: the team's warps take
// the group's segments round-robin, each forms the exact float sums of its segment on its own (that
// work does not depend on the chain state), then receives the group's chain state - eight
// accumulators and the macc sum per lane - from the warp that held the previous segment through a
// shared-memory mailbox, runs the segment's FMAs and macc adds (the same operations in the same
// order as a lone warp) and hands the state on; the warp with the last segment reduces and stores.
//
// Arithmetic.  Per segment, a SCALE PASS (one lane per (task, row)) forms the f32 block scales
// xs*(d*sc) and the macc terms exactly as the reference forms them.  Then, per 4 weights: one mask,
// one dp4a whose accumulator input is the bit pattern of 1.5 * 2^23 (so the integer sum arrives as a
// float: an exact conversion without a convert instruction), one subtraction of that constant and one
// FMA.  When a group is done the four lanes of a row combine their chains with shuffles, one lane per
// row adds the row's macc terms in block order, subtracts, applies the epilogue and stores.
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

constexpr int XG_MAX_WARPS = 16;                     // warps per CTA when they form teams (picked per launch)
constexpr int XG_LONE_MAX_WARPS = 32;                // ... when every warp walks its groups alone (64 registers per thread)
constexpr int XG_MAX_SEGS = 3;
constexpr int XG_SEG_TASKS = 4;                      // tasks (of 128 weights) per segment: two super-blocks
constexpr int XG_MAX_STAGES = 8;
constexpr int XG_HEAD_BYTES = 2112;                  // barriers [32][8], then the abort flag
constexpr int XG_MAGIC_I = 0x4B400000;               // bits of 12582912.0f = 1.5 * 2^23
constexpr float XG_MAGIC_F = 12582912.0f;
// The same trick for high nibbles left in place (16 x the quant in each byte, Q4_K): on the bits of 1.5 * 2^19, whose unit in
// the last place is 1/16, the accumulated 16 * sum moves the value by exactly sum - no shift of the nibbles needed.
constexpr int XG_MAGIC16_I = 0x49400000;
constexpr float XG_MAGIC16_F = 786432.0f;
constexpr size_t XG_SMEM_LIMIT = 224 * 1024;
constexpr uint32_t XG_SCT_BYTES = 1024;              // per warp: the segment's block scales, [task][row][...]

struct ExactParams {
    WeightView w[XG_MAX_SEGS];
    float *y[XG_MAX_SEGS];
    uint32_t row_end[XG_MAX_SEGS];
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k;
    int epilogue;
    int stages;  // log2 of the ring depth
    int team;    // log2 of the warps that share one row group's walk over k
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

// (float)(sum of four u8 x s8 products), exactly: a dp4a accumulates onto the bits of 1.5 * 2^23 and that constant is
// subtracted again (in the main loop, as packed pairs).
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ int word_of(const int4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
// Bulk copy / barrier forms on 32-bit shared addresses that are worked out once.
__device__ __forceinline__ void expect_tx_u32(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s_u32(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

__host__ __device__ inline size_t xg_cta_smem(uint32_t k) {  // what the CTA shares: barriers, activation column
    return XG_HEAD_BYTES + (size_t)k + (size_t)(k / 32) * 4 * 2 + (size_t)(k / 16) * 4;
}
// A team's mailbox: the chain state of a row group (eight chains and the macc sum of every lane) handed from the warp
// that finished one segment to the warp that holds the next.  Hand-overs are numbered along the team's walk (group by
// group, segment by segment) and use 2 W slots in turn, each with its own barrier: a warp that starts to wait for
// hand-over h has seen h - 2 W complete (at most 2 W - 2 are pending then), which is what a parity wait needs.
constexpr uint32_t XG_MAIL_SLOT = 9 * 32 * 4;
__host__ __device__ inline uint32_t xg_mail_bytes(uint32_t team_log) { return (2u << team_log) * (XG_MAIL_SLOT + 8); }
constexpr uint32_t XG_TERM_STRIDE = 20;              // floats per row of a term buffer (16 terms + padding: conflict-free stores)
constexpr uint32_t XG_TERM_BYTES = 8 * XG_TERM_STRIDE * 4;
__host__ __device__ inline size_t xg_warp_smem(uint32_t stages, uint32_t seg_bytes) {  // ring; two scale tables and two term buffers
    return (size_t)stages * seg_bytes + 2 * XG_SCT_BYTES + 2 * XG_TERM_BYTES;
}

template <int T, bool TEAM>
__global__ void __launch_bounds__((TEAM ? XG_MAX_WARPS : XG_LONE_MAX_WARPS) * 32) gemv_exact_kernel(const ExactParams p) {
    using L = SegLayout<T>;
    extern __shared__ __align__(128) uint8_t xg_smem[];
    const uint32_t k = p.k, nb32 = k >> 5, nb = k >> 8, n_seg = k / (128 * XG_SEG_TASKS);
    const uint32_t S = 1u << p.stages, s_mask = S - 1, s_shift = (uint32_t)p.stages;  // ring depth, a power of two
    const int nthreads = blockDim.x;
    const uint32_t P = blockDim.x >> 5;
    // carve-up: rings [P][S] (128-byte aligned buffers), barriers, activation column, per warp two scale tables and two term buffers
    uint8_t *rings = xg_smem;
    uint8_t *fixed = rings + (size_t)P * S * L::BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(fixed);                     // [P][XG_MAX_STAGES]
    volatile uint32_t *abort_flag = reinterpret_cast<uint32_t *>(fixed + XG_HEAD_BYTES - 8);
    int8_t *aq = reinterpret_cast<int8_t *>(fixed + XG_HEAD_BYTES);           // [k]
    float *xs = reinterpret_cast<float *>(fixed + XG_HEAD_BYTES + k);         // [k/32]
    float *a32 = xs + nb32;                                                   // [k/32] sum of the block's quants
    float *a16 = a32 + nb32;                                                  // [k/16]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *sct0 = a16 + 2 * nb32 + (size_t)warp * ((2 * XG_SCT_BYTES + 2 * XG_TERM_BYTES) / 4);  // [2][XG_SCT_BYTES / 4]
    float *terms0 = sct0 + 2 * (XG_SCT_BYTES / 4);                                                // [2][8][XG_TERM_STRIDE]
    uint8_t *ring = rings + (size_t)warp * S * L::BYTES;
    uint64_t *wbars = bars + warp * XG_MAX_STAGES;

    // this warp's row groups: CTAs take groups round-robin, the TEAMS of a CTA take the CTA's groups round-robin, and the
    // W warps of a team take a group's segments round-robin (W = 1: a warp walks its groups alone)
    const uint32_t n_groups = (p.total_rows + 7) >> 3;
    const uint32_t W = 1u << p.team, team = warp >> p.team, wj = warp & (W - 1);
    const uint32_t first = blockIdx.x + gridDim.x * team, step = gridDim.x * (P >> p.team);
    const uint32_t my_groups = first < n_groups ? (n_groups - first + step - 1) / step : 0;
    const uint32_t n_my_seg = wj < n_seg ? (n_seg - wj + W - 1) >> p.team : 0;  // this warp's segments of a group: wj, wj + W, ...
    const uint32_t n_items = my_groups * n_my_seg;  // segments this warp walks, over all its groups
    const uint32_t m_slots = 2 * W, m_log = p.team + 1;
    uint8_t *mail = reinterpret_cast<uint8_t *>(a16 + 2 * nb32) + (size_t)P * (2 * XG_SCT_BYTES + 2 * XG_TERM_BYTES) + (size_t)team * xg_mail_bytes(p.team);
    uint64_t *mbars = reinterpret_cast<uint64_t *>(mail + m_slots * XG_MAIL_SLOT);

    if (tid == 0) *abort_flag = 0;
    if (lane == 0) {
        for (uint32_t s = 0; s < S; ++s) tma::mbar_init(wbars + s, 1);
        if (W > 1 && wj == 0)
            for (uint32_t s = 0; s < m_slots; ++s) tma::mbar_init(mbars + s, 1);
        tma::mbar_init_fence();
    }

    // Lanes 0-3 request the warp's segments in order, one plane each (low quants, headers, high bits, super-block
    // scales); lane 0 also announces the byte count.  A lane's source address advances by its plane's bytes per segment
    // and is worked out afresh at every group.
    const uint32_t ring_u32 = tma::smem_u32(ring), bar_u32 = tma::smem_u32(wbars);
    const uint32_t my_bytes = lane == 0 ? L::Q : lane == 1 ? L::HDR : lane == 2 ? L::QH : lane == 3 ? L::D : 0;
    const uint32_t my_off = lane == 0 ? 0 : lane == 1 ? L::OFF_HDR : lane == 2 ? L::OFF_QH : L::OFF_D;
    uint32_t is_j = 0, is_seg = 0, is_group = first;
    const uint8_t *is_src = nullptr;
    auto issue_next = [&]() {  // called by the whole warp
        if (is_seg == 0 && my_bytes) {
            const uint32_t row = is_group * 8;
            int sg = 0;
            while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
            const uint32_t local = row - (sg ? p.row_end[sg - 1] : 0);
            const WeightView &w = p.w[sg];
            const size_t grp = local >> 3, sb0 = grp * nb * 8;  // first (super-block, row) slot of the group in the per-block planes
            is_src = lane == 0 ? w.q + grp * 8 * ((size_t)nb * 128)
                   : lane == 1 ? w.hdr + sb0 * 16
                   : lane == 2 ? w.qh + sb0 * (L::QH / (L::SB * 8))
                               : w.d + sb0 * 2;
            is_src += (size_t)wj * my_bytes;  // the warp's first segment of the group
        }
        const uint32_t st = is_j & s_mask, bar = bar_u32 + st * 8;
        if (lane == 0) expect_tx_u32(bar, L::TX);
        __syncwarp();
        if (my_bytes) {
            bulk_g2s_u32(ring_u32 + st * L::BYTES + my_off, is_src, my_bytes, bar);
            is_src += (size_t)my_bytes << p.team;
        }
        ++is_j;
        if (++is_seg == n_my_seg) {
            is_seg = 0;
            is_group += step;
        }
    };
    __syncwarp();  // the barriers are initialised before any lane's copy names them
    // weights do not depend on the previous kernel: fill the ring before waiting for it
    for (uint32_t j = 0; j < S && j < n_items; ++j) issue_next();

    pdl_trigger();
    pdl_wait();
    tp_arrive_wait(p.tp.ctx, p.tp.wait_slot);
    if (p.f.norm_x) {
        // ---- RMSNorm + Q8_0 of the f32 vector, in the arithmetic of the stand-alone kernel (1024 virtual threads of four
        // consecutive elements: f64 sum of squares per thread, butterfly per 32 threads, butterfly over the 32 partials;
        // then (x * inv) * w and the block quantizer of cera/src/backend/cpu.rs:942-958), whatever the CTA's size
        double *red = reinterpret_cast<double *>(a16 + 2 * nb32);  // 32 partials + the scale: the first warp's scale tables, unused so far
        float *inv_slot = reinterpret_cast<float *>(red + 32);
        const uint32_t nvec = k >> 2;
        const float4 *xc = reinterpret_cast<const float4 *>(p.f.norm_x), *wc = reinterpret_cast<const float4 *>(p.f.norm_w);
        for (uint32_t vw = warp; vw < 32; vw += P) {
            double ss = 0.0;
            for (uint32_t v = vw * 32 + lane; v < nvec; v += 1024) {
                const float4 xv = xc[v];
                ss += (double)xv.x * (double)xv.x;
                ss += (double)xv.y * (double)xv.y;
                ss += (double)xv.z * (double)xv.z;
                ss += (double)xv.w * (double)xv.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[vw] = ss;
        }
        __syncthreads();
        if (warp == 0) {
            double t = red[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) *inv_slot = (float)(1.0 / sqrt(t / (double)k + (double)p.f.norm_eps));
        }
        __syncthreads();
        const float inv = *inv_slot;
        for (uint32_t v = tid; v < nvec; v += nthreads) {  // whole warps: a block's eight lanes are all in or all out
            const float4 xv = xc[v], wv = wc[v];
            const float e[4] = {__fmul_rn(__fmul_rn(xv.x, inv), wv.x), __fmul_rn(__fmul_rn(xv.y, inv), wv.y),
                                __fmul_rn(__fmul_rn(xv.z, inv), wv.z), __fmul_rn(__fmul_rn(xv.w, inv), wv.w)};
            if (p.f.norm_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.f.norm_out)[v] = make_float4(e[0], e[1], e[2], e[3]);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = fabsf(e[i]);
                amax = fmaxf(amax, a == a ? a : 0.0f);  // f32::max ignores NaN
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float d = __fdiv_rn(amax, 127.0f);
            const float rcp = __fdiv_rn(1.0f, d);
            const float id = (d != 0.0f && isfinite(rcp)) ? rcp : 0.0f;
            int q[4], s4 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float pq = rintf(__fmul_rn(e[i], id));
                q[i] = pq != pq ? 0 : (int)fminf(fmaxf(pq, -128.0f), 127.0f);
                s4 += q[i];
            }
            s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
            s4 += __shfl_xor_sync(0xffffffffu, s4, 2);  // sum of the 16 elements of lanes 4j .. 4j+3
            const int s8 = s4 + __shfl_xor_sync(0xffffffffu, s4, 4);
            reinterpret_cast<uint32_t *>(aq)[v] = (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) | ((uint32_t)(uint8_t)q[2] << 16) |
                                                  ((uint32_t)(uint8_t)q[3] << 24);
            if ((lane & 7) == 0) {
                xs[v >> 3] = __half2float(__float2half_rn(d));
                a32[v >> 3] = (float)s8;
            }
            if ((lane & 3) == 0) a16[v >> 2] = (float)(int)(int16_t)s4;
        }
    } else {
        // stage the activation column
        for (uint32_t i = tid; i < k / 16; i += nthreads) {
            reinterpret_cast<int4 *>(aq)[i] = reinterpret_cast<const int4 *>(p.x.quants)[i];
            a16[i] = (float)p.x.sums[i];
        }
        for (uint32_t i = tid; i < nb32; i += nthreads) {
            xs[i] = p.x.scales[i];
            a32[i] = (float)((int)p.x.sums[2 * i] + (int)p.x.sums[2 * i + 1]);
        }
    }
    __syncthreads();

    const int rr = lane >> 2, c = lane & 3, pair = c >> 1, half = c & 1;
    const int pi = lane >> 3, pr = lane & 7;  // the scale pass works on (task pi of the segment, row pr)
    // ---- scale pass of one segment: one lane per (task, row) forms the task's f32 block scales and macc terms exactly
    // as the reference forms them, into scale table / term buffer `b`
    auto scale_pass = [&](const uint8_t *buf, uint32_t seg, uint32_t b) {
        float *sct = sct0 + b * (XG_SCT_BYTES / 4);
        const uint32_t t = seg * XG_SEG_TASKS + pi;
        const int slot = (pi >> 1) * 8 + pr;
        const uint4 h = *reinterpret_cast<const uint4 *>(buf + L::OFF_HDR + slot * 16);
        const float4 x4 = *reinterpret_cast<const float4 *>(xs + 4 * t);
        const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
        float tm[4];
        if (T == CERA_TYPE_Q6_K) {
            const float d6 = h2f(*reinterpret_cast<const uint16_t *>(buf + L::OFF_D + slot * 2));
            // the task's eight int8 scales: index 2g + e = 16-element half e of 32-element block g
            const uint32_t sw[2] = {(pi & 1) ? h.z : h.x, (pi & 1) ? h.w : h.y};
            const float4 am_a = *reinterpret_cast<const float4 *>(a16 + 8 * t), am_b = *reinterpret_cast<const float4 *>(a16 + 8 * t + 4);
            const float am[8] = {am_a.x, am_a.y, am_a.z, am_a.w, am_b.x, am_b.y, am_b.z, am_b.w};
            const float d32 = __fmul_rn(d6, 32.0f);
            float e[8];
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                const float s0 = (float)(int8_t)(sw[gq >> 1] >> (16 * (gq & 1))), s1 = (float)(int8_t)(sw[gq >> 1] >> (16 * (gq & 1) + 8));
                const float2 s2 = make_float2(s0, s1), x2 = make_float2(xv[gq], xv[gq]);
                const float2 ee = __fmul2_rn(__fmul2_rn(s2, make_float2(d6, d6)), x2);                  // (s * d) * xs, both halves
                const float2 pa = __fmul2_rn(s2, make_float2(am[2 * gq], am[2 * gq + 1]));              // s0 * A0, s1 * A1
                e[2 * gq] = ee.x;
                e[2 * gq + 1] = ee.y;
                tm[gq] = __fmul_rn(__fmul_rn(xv[gq], d32), __fadd_rn(pa.x, pa.y));
            }
            // strip c = (pair, half) multiplies block `pair` (low nibbles) and block `pair + 2` (high), half `half`
            float4 *dst = reinterpret_cast<float4 *>(sct + (pi * 8 + pr) * 8);
            dst[0] = make_float4(e[0], e[4], e[1], e[5]);
            dst[1] = make_float4(e[2], e[6], e[3], e[7]);
        } else {
            uint32_t scp, mnp;
            kq_quad(h, pi & 1, scp, mnp);
            const float d = h2f((uint16_t)(h.x & 0xFFFF)), dmin = h2f((uint16_t)(h.x >> 16));
            const float4 a4 = *reinterpret_cast<const float4 *>(a32 + 4 * t);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w};
            // the same products as packed pairs (mul.f32x2 / add.f32x2: each half is the scalar IEEE operation)
            float e[4];
            const float2 nb23 = make_float2(-8388608.0f, -8388608.0f), d2 = make_float2(d, d), dm2 = make_float2(dmin, dmin);
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                const float2 x2 = make_float2(xv[2 * jp], xv[2 * jp + 1]), a2 = make_float2(av[2 * jp], av[2 * jp + 1]);
                const float2 scf = __fadd2_rn(make_float2(__uint_as_float(0x4B000000u | ((scp >> (16 * jp)) & 0xFF)),
                                                          __uint_as_float(0x4B000000u | ((scp >> (16 * jp + 8)) & 0xFF))), nb23);
                const float2 mnf = __fadd2_rn(make_float2(__uint_as_float(0x4B000000u | ((mnp >> (16 * jp)) & 0xFF)),
                                                          __uint_as_float(0x4B000000u | ((mnp >> (16 * jp + 8)) & 0xFF))), nb23);
                const float2 ee = __fmul2_rn(x2, __fmul2_rn(d2, scf));
                const float2 tt = __fmul2_rn(__fmul2_rn(x2, __fmul2_rn(dm2, mnf)), a2);
                e[2 * jp] = ee.x, e[2 * jp + 1] = ee.y;
                tm[2 * jp] = tt.x, tm[2 * jp + 1] = tt.y;
            }
            *reinterpret_cast<float4 *>(sct + (pi * 8 + pr) * 4) = make_float4(e[0], e[1], e[2], e[3]);
        }
        *reinterpret_cast<float4 *>(terms0 + b * (8 * XG_TERM_STRIDE) + pr * XG_TERM_STRIDE + 4 * pi) = make_float4(tm[0], tm[1], tm[2], tm[3]);
    };

    bool ok = true;  // false once a wait on a copy gave up: nothing more is stored
    if (n_items) {
        if (!tma::mbar_wait_blocking(wbars, 0, abort_flag, &g_xg_status, 1u)) ok = false;
        if (ok) scale_pass(ring, wj, 0);
        __syncwarp();
    }
    uint32_t item = 0, gi = 0;  // gi counts the team's groups (the mailbox slots alternate with it)
    for (uint32_t g = first; g < n_groups; g += step, ++gi) {
        float2 acc_lo2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)}, acc_hi2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
        float macc = 0.0f;  // every lane of a row carries the row's macc chain (the same adds in the same order)
        bool last_mine = !TEAM;  // this warp holds the group's final chain state
        for (uint32_t sl = 0; sl < n_my_seg; ++sl, ++item) {
            const uint32_t seg = TEAM ? wj + (sl << p.team) : sl;
            const uint8_t *buf = ring + (size_t)(item & s_mask) * L::BYTES;
            const uint32_t b = item & 1;
            if (ok) {
                const float *sct = sct0 + b * (XG_SCT_BYTES / 4);
                // In a team the exact float sums of the segment are formed first (they do not depend on the chain state),
                // the state arrives from the warp that held the previous segment, and only the FMAs and the macc adds
                // run on the serial path; a lone warp feeds each sum straight into its FMA.
                float2 pl[XG_SEG_TASKS][2], ph[XG_SEG_TASKS][2], scs[XG_SEG_TASKS];
                // ---- the segment's tasks, this lane's strip: per 4 weights one mask, one dp4a, one subtraction, one FMA
#pragma unroll
                for (int i = 0; i < XG_SEG_TASKS; ++i) {
                    const uint32_t t = seg * XG_SEG_TASKS + i;
                    const int sbl = i >> 1, hf = i & 1;
                    const uint4 piece = *reinterpret_cast<const uint4 *>(buf + (i * 32 + lane) * 16);
                    uint4 hb = make_uint4(0, 0, 0, 0);
                    float2 sc2;
                    uint32_t xb_lo, xb_hi;
                    if (T == CERA_TYPE_Q6_K) {
                        xb_lo = 4 * t + pair;
                        xb_hi = xb_lo + 2;
                        sc2 = *reinterpret_cast<const float2 *>(sct + (i * 8 + rr) * 8 + c * 2);
                        hb = *reinterpret_cast<const uint4 *>(buf + L::OFF_QH + (sbl * 8 + rr) * 64 + hf * 32 + half * 16);
                    } else {
                        xb_lo = 4 * t + 2 * pair;
                        xb_hi = xb_lo + 1;
                        sc2 = *reinterpret_cast<const float2 *>(sct + (i * 8 + rr) * 4 + pair * 2);
                        if (T == CERA_TYPE_Q5_K) hb = *reinterpret_cast<const uint4 *>(buf + L::OFF_QH + (sbl * 8 + rr) * 32 + half * 16);
                    }
                    const int4 alo = *reinterpret_cast<const int4 *>(aq + 32 * xb_lo + 16 * half);
                    const int4 ahi = *reinterpret_cast<const int4 *>(aq + 32 * xb_hi + 16 * half);
                    if (!TEAM) {
                        const float4 tm = *reinterpret_cast<const float4 *>(terms0 + b * (8 * XG_TERM_STRIDE) + rr * XG_TERM_STRIDE + 4 * i);
                        macc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(macc, tm.x), tm.y), tm.z), tm.w);
                    }
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        const uint32_t v = word_of(piece, wd), hbw = word_of(hb, wd);
                        lo[wd] = v & 0x0F0F0F0Fu;
                        hi[wd] = T == CERA_TYPE_Q4_K ? v & 0xF0F0F0F0u : (v >> 4) & 0x0F0F0F0Fu;
                        if (T == CERA_TYPE_Q5_K) {
                            const int sh_lo = 4 * hf + 2 * pair;  // fifth-bit position of the low-nibble sub-block
                            lo[wd] |= ((hbw >> sh_lo) & 0x01010101u) << 4;
                            hi[wd] |= ((hbw >> (sh_lo + 1)) & 0x01010101u) << 4;
                        }
                        if (T == CERA_TYPE_Q6_K) {
                            // bits 2 pair, 2 pair + 1 of each high-bit byte belong to the low-nibble element, bits 2 pair + 4,
                            // 2 pair + 5 to the high-nibble one: one shift brings the first pair to bits 0-1 and the second to 4-5
                            const uint32_t hs = hbw >> (2 * pair);
                            lo[wd] |= (hs << 4) & 0x30303030u;
                            hi[wd] |= hs & 0x30303030u;
                        }
                    }
                    // the subtraction of the bias and the FMA run as packed pairs (add.f32x2 / fma.f32x2: each half is the
                    // IEEE operation of the scalar form, two chains per instruction)
                    const float2 nbias = make_float2(-XG_MAGIC_F, -XG_MAGIC_F), s_lo = make_float2(sc2.x, sc2.x), s_hi = make_float2(sc2.y, sc2.y);
                    constexpr int MAGIC_HI = T == CERA_TYPE_Q4_K ? XG_MAGIC16_I : XG_MAGIC_I;
                    const float2 nbias_hi = T == CERA_TYPE_Q4_K ? make_float2(-XG_MAGIC16_F, -XG_MAGIC16_F) : nbias;
                    scs[i] = sc2;
#pragma unroll
                    for (int wp = 0; wp < 2; ++wp) {
                        const float2 rl = make_float2(__int_as_float(dp_us(lo[2 * wp], word_of(alo, 2 * wp), XG_MAGIC_I)),
                                                      __int_as_float(dp_us(lo[2 * wp + 1], word_of(alo, 2 * wp + 1), XG_MAGIC_I)));
                        const float2 rh = make_float2(__int_as_float(dp_us(hi[2 * wp], word_of(ahi, 2 * wp), MAGIC_HI)),
                                                      __int_as_float(dp_us(hi[2 * wp + 1], word_of(ahi, 2 * wp + 1), MAGIC_HI)));
                        if (TEAM) {
                            pl[i][wp] = __fadd2_rn(rl, nbias);
                            ph[i][wp] = __fadd2_rn(rh, nbias_hi);
                        } else {
                            acc_lo2[wp] = __ffma2_rn(__fadd2_rn(rl, nbias), s_lo, acc_lo2[wp]);
                            acc_hi2[wp] = __ffma2_rn(__fadd2_rn(rh, nbias_hi), s_hi, acc_hi2[wp]);
                        }
                    }
                }
                // ---- the next segment's scale pass, one segment ahead of its use (it has its own table and term buffer)
                if (item + 1 < n_items) {
                    const uint32_t nx = item + 1;
                    if (!tma::mbar_wait_blocking(wbars + (nx & s_mask), (nx >> s_shift) & 1, abort_flag, &g_xg_status, 1u)) ok = false;
                    const uint32_t nseg = TEAM ? (sl + 1 == n_my_seg ? wj : seg + W) : (seg + 1 == n_seg ? 0 : seg + 1);
                    if (ok) scale_pass(ring + (size_t)(nx & s_mask) * L::BYTES, nseg, b ^ 1);
                }
                if (TEAM) {
                    // ---- the serial path: chain state in, the segment's FMAs and macc adds in task order, chain state out
                    if (seg > 0) {
                        const uint32_t h = gi * (n_seg - 1) + seg - 1, slot = h & (m_slots - 1);  // the hand-over after segment seg - 1
                        if (!tma::mbar_wait_blocking(mbars + slot, (h >> m_log) & 1, abort_flag, &g_xg_status, 2u)) ok = false;
                        const float *ms = reinterpret_cast<const float *>(mail + slot * XG_MAIL_SLOT) + lane;
                        acc_lo2[0] = make_float2(ms[0], ms[32]);
                        acc_lo2[1] = make_float2(ms[64], ms[96]);
                        acc_hi2[0] = make_float2(ms[128], ms[160]);
                        acc_hi2[1] = make_float2(ms[192], ms[224]);
                        macc = ms[256];
                    }
#pragma unroll
                    for (int i = 0; i < XG_SEG_TASKS; ++i) {
                        const float4 tm = *reinterpret_cast<const float4 *>(terms0 + b * (8 * XG_TERM_STRIDE) + rr * XG_TERM_STRIDE + 4 * i);
                        macc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(macc, tm.x), tm.y), tm.z), tm.w);
                        const float2 s_lo = make_float2(scs[i].x, scs[i].x), s_hi = make_float2(scs[i].y, scs[i].y);
#pragma unroll
                        for (int wp = 0; wp < 2; ++wp) {
                            acc_lo2[wp] = __ffma2_rn(pl[i][wp], s_lo, acc_lo2[wp]);
                            acc_hi2[wp] = __ffma2_rn(ph[i][wp], s_hi, acc_hi2[wp]);
                        }
                    }
                    if (seg + 1 < n_seg) {
                        const uint32_t slot = (gi * (n_seg - 1) + seg) & (m_slots - 1);
                        float *ms = reinterpret_cast<float *>(mail + slot * XG_MAIL_SLOT) + lane;
                        ms[0] = acc_lo2[0].x, ms[32] = acc_lo2[0].y, ms[64] = acc_lo2[1].x, ms[96] = acc_lo2[1].y;
                        ms[128] = acc_hi2[0].x, ms[160] = acc_hi2[0].y, ms[192] = acc_hi2[1].x, ms[224] = acc_hi2[1].y;
                        ms[256] = macc;
                        __syncwarp();
                        if (lane == 0 && ok) tma::mbar_arrive(mbars + slot);
                    } else {
                        last_mine = true;
                    }
                }
            }
            __syncwarp();  // every lane is done with this segment's buffer, table and terms; the next ones are written
            if (item + S < n_items) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_next();
            }
        }
        if (!last_mine) continue;  // another warp of the team finishes this group
        // ---- the 32 chains of the row -> one value (tree over the accumulators, then the hsum256 order)
        const float acc_lo[4] = {acc_lo2[0].x, acc_lo2[0].y, acc_lo2[1].x, acc_lo2[1].y}, acc_hi[4] = {acc_hi2[0].x, acc_hi2[0].y, acc_hi2[1].x, acc_hi2[1].y};
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
        const float r = __fsub_rn(hsum, macc);
        const uint32_t row = g * 8 + rr;
        const bool valid = ok && c == 0 && row < p.total_rows;
        int sg = 0;
        while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
        const uint32_t local = row - (sg ? p.row_end[sg - 1] : 0);
        if (p.epilogue == EPI_ROPE_KV) {
            // rows (2i, 2i+1) of a head are a NORM rotation pair (cera/src/backend/cpu.rs:5161-5180): the first lanes of adjacent rows
            const float other = __shfl_xor_sync(0xffffffffu, r, 4);
            if (valid) {
                const uint32_t pos = *p.f.pos_dev;
                if (sg == 2) {
                    store_kv(p.f.v_cache, p.f.kv_f16, (size_t)pos * p.f.kv_dim + local, r);
                } else {
                    const uint32_t pidx = (local % p.f.head_dim) >> 1;
                    const float *cs_sn = p.f.rope_cs + ((p.f.rope_by_pos ? (size_t)pos * (p.f.head_dim >> 1) : 0) + pidx) * 2;
                    const float cs = cs_sn[0], sn = cs_sn[1];
                    const float x0 = (rr & 1) ? other : r, x1 = (rr & 1) ? r : other;
                    const float out = (rr & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs))
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

template <int T>
int32_t launch_exact_typed(const ExactParams &p0, cudaStream_t st) {
    using L = SegLayout<T>;
    ExactParams p = p0;
    // One CTA per SM; its warps share the SM's row groups.  Warps per CTA = the SM's share of the groups (at most what
    // shared memory holds, at most 16); the ring is as deep as shared memory allows (8, 4 or 2 segments), so that a
    // CTA of few warps still keeps tens of KB in flight.
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t groups = (p.total_rows + 7) / 8;
    const uint32_t grid = groups < sms ? groups : sms;
    const uint32_t share = (groups + grid - 1) / grid;
    const size_t cta = xg_cta_smem(p.k);
    static const int env_cap = [] { const char *e = getenv("CERA_CUDA_XG_CAP"); return e ? atoi(e) : 0; }();
    // lone warps: up to 32 per CTA (28 672 gate / up rows give an SM 24 groups: one round of 25 warps instead of two of 16;
    // CERA_CUDA_XG_CAP lowers the cap for A/B runs)
    const uint32_t warp_cap = env_cap >= 1 && env_cap <= XG_LONE_MAX_WARPS ? (uint32_t)env_cap : (uint32_t)XG_LONE_MAX_WARPS;
    auto max_warps = [&](uint32_t stages) -> uint32_t {
        const size_t per_warp = xg_warp_smem(stages, L::BYTES);
        if (cta + per_warp > XG_SMEM_LIMIT) return 0;
        const size_t n = (XG_SMEM_LIMIT - cta) / per_warp;
        return n > (size_t)warp_cap ? warp_cap : (uint32_t)n;
    };
    uint32_t s_log = 3, P = share;
    if (P > max_warps(8)) s_log = 2;
    if (s_log == 2 && P > max_warps(4)) {
        // more groups than warps fit: keep the deeper ring unless that costs more than a quarter of the warps
        if (max_warps(4) * 4 >= (P < warp_cap ? P : warp_cap) * 3) P = max_warps(4);
        else s_log = 1;
    }
    if (s_log == 1 && P > max_warps(2)) P = max_warps(2);
    // CERA_CUDA_XG_WARPS / CERA_CUDA_XG_STAGES (log2) override the choice for tuning runs; read once
    static const int env_p = [] { const char *e = getenv("CERA_CUDA_XG_WARPS"); return e ? atoi(e) : 0; }();
    static const int env_s = [] { const char *e = getenv("CERA_CUDA_XG_STAGES"); return e ? atoi(e) : 0; }();
    if (env_s >= 1 && env_s <= 3) s_log = (uint32_t)env_s;
    if (env_p >= 1) P = (uint32_t)env_p < share ? (uint32_t)env_p : share;
    if (P > max_warps(1u << s_log)) P = max_warps(1u << s_log);
    if (P == 0) return fail(CERA_CUDA_ERR_BAD_ARG, "gemv (reference order): k too large for shared memory");
    // Few row groups per SM (o-proj, down-proj, a tensor-parallel rank's slices): the warps that would idle join TEAMS of
    // W = 2 .. 16 that share one
    // group's walk over k - each forms the exact sums of its segments on its own, only the FMA chains pass from warp to
    // warp in segment order.  CERA_CUDA_XG_TEAM (log2 W) overrides.
    static const int env_t = [] { const char *e = getenv("CERA_CUDA_XG_TEAM"); return e ? atoi(e) : -1; }();
    const uint32_t n_seg = p.k / (128 * XG_SEG_TASKS);
    uint32_t t_log = 0;
    if (env_p < 1) {
        while (t_log < 4 && (share << (t_log + 1)) <= (uint32_t)XG_MAX_WARPS && (2u << t_log) <= n_seg) ++t_log;
        if (env_t >= 0 && env_t <= 4) t_log = (uint32_t)env_t;
        while (t_log && ((1u << t_log) > n_seg)) --t_log;
        while (t_log) {
            // whole teams, at most sixteen warps, each warp with its ring, plus a mailbox per team; shrink the ring, then
            // the team, to fit
            uint32_t Pt = share << t_log;
            if (Pt > (uint32_t)XG_MAX_WARPS) Pt = (uint32_t)XG_MAX_WARPS;
            const size_t need = cta + (size_t)Pt * xg_warp_smem(1u << s_log, L::BYTES) + (size_t)(Pt >> t_log) * xg_mail_bytes(t_log);
            if (need <= XG_SMEM_LIMIT) {
                P = Pt;
                break;
            }
            if (s_log > 1) --s_log;
            else --t_log;
        }
    }
    p.stages = (int)s_log;
    p.team = (int)t_log;
    const size_t smem = cta + (size_t)P * xg_warp_smem(1u << s_log, L::BYTES) + (t_log ? (size_t)(P >> t_log) * xg_mail_bytes(t_log) : 0);
    static thread_local int raised_dev = -1;  // per instantiation: opt in to more than 48 KB once per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (raised_dev != dev) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemv_exact_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)XG_SMEM_LIMIT));
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemv_exact_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)XG_SMEM_LIMIT));
        raised_dev = dev;
    }
    count_launch();
    if (t_log) return check_cuda(launch_k(gemv_exact_kernel<T, true>, dim3(grid), dim3(P * 32), smem, st, p), "gemv (reference order, teams) launch");
    return check_cuda(launch_k(gemv_exact_kernel<T, false>, dim3(grid), dim3(P * 32), smem, st, p), "gemv (reference order) launch");
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
// *taken = false: not a K-quant, k not a multiple of 512, or a shape outside the kernel's rules;
// nothing was launched.
int32_t launch_gemv_exact(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp) {
    *taken = false;
    if (exact_off() || n_segs < 1 || n_segs > XG_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    if (type != CERA_TYPE_Q4_K && type != CERA_TYPE_Q5_K && type != CERA_TYPE_Q6_K) return CERA_CUDA_OK;
    const uint32_t k = segs[0].w.k;
    if (k % (128 * XG_SEG_TASKS)) return CERA_CUDA_OK;  // whole segments (512 weights)
    if (fusion && fusion->norm_x && k % 1024) return CERA_CUDA_OK;  // the norm prologue walks 1024 virtual threads of four elements
    for (int i = 0; i < n_segs; ++i)
        if (segs[i].w.ilv != 8) return CERA_CUDA_OK;
    if (xg_cta_smem(k) + xg_warp_smem(2, 4096) > XG_SMEM_LIMIT) return CERA_CUDA_OK;
    const bool norm = fusion && fusion->norm_x;
    if (norm ? ((uintptr_t)fusion->norm_x % 16 || (uintptr_t)fusion->norm_w % 16 || !fusion->norm_w) : ((uintptr_t)x.quants % 16 != 0)) return CERA_CUDA_OK;
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
