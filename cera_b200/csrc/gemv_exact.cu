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
// The planes interleave groups of eight rows (WeightView::ilv): the 8 x 4 strips of a group are stored
// task by task, 32 pieces = 512 contiguous bytes per task, which is exactly one warp-wide 128-bit load.
// So ONE LANE OWNS ONE STRIP of one row: it streams the strip with 128-bit loads in task order and
// carries its eight chains in registers; four lanes cover a row, a warp eight rows, a CTA of four
// such warps 32 rows per round.  Each product quad is one dp4a whose accumulator input is the bit
// pattern of 1.5 * 2^23, so the integer sum arrives already as a float (an exact conversion without
// a convert instruction).  The macc terms are written to shared memory and summed, one row per lane,
// by a fifth warp that trails the producers segment by segment (named barriers), so the serial chain
// overlaps the streaming; that warp also subtracts, applies the epilogue and stores.
//
// Activation quants, block scales and block sums are staged in shared memory once per CTA.
#include <cstdlib>
#include <cstring>

#include "gemv_task.cuh"

namespace cera {

namespace {

constexpr int XG_PRODUCERS = 4;                      // warps streaming weights
constexpr int XG_THREADS = (XG_PRODUCERS + 1) * 32;  // + the warp that runs the serial chains
constexpr int XG_ROWS = XG_PRODUCERS * 8;            // rows per round
constexpr int XG_MAX_SEGS = 3;
constexpr int XG_SEG_TASKS = 32;                     // tasks (of 128 weights) per hand-over to the chain warp
constexpr int XG_MAX_HANDOVERS = 6;                  // named barriers 1..6, 7 = row values ready
constexpr int XG_MAGIC_I = 0x4B400000;               // bits of 12582912.0f = 1.5 * 2^23
constexpr float XG_MAGIC_F = 12582912.0f;

struct ExactParams {
    WeightView w[XG_MAX_SEGS];
    float *y[XG_MAX_SEGS];
    uint32_t row_end[XG_MAX_SEGS];
    int n_segs;
    uint32_t total_rows;
    ActView x;
    uint32_t k, t128;
    int epilogue;
    GemvFusion f;
    TpHook tp;
};

// Named barriers with literal ids (a register id would make the compiler reserve all sixteen).
#define XG_BAR(op, id) asm volatile(op " " #id ", %0;" ::"r"(XG_THREADS) : "memory")
__device__ __forceinline__ void bar_arrive(int id) {
    switch (id) {
        case 1: XG_BAR("bar.arrive", 1); break;
        case 2: XG_BAR("bar.arrive", 2); break;
        case 3: XG_BAR("bar.arrive", 3); break;
        case 4: XG_BAR("bar.arrive", 4); break;
        case 5: XG_BAR("bar.arrive", 5); break;
        case 6: XG_BAR("bar.arrive", 6); break;
        default: XG_BAR("bar.arrive", 7); break;
    }
}
__device__ __forceinline__ void bar_sync(int id) {
    switch (id) {
        case 1: XG_BAR("bar.sync", 1); break;
        case 2: XG_BAR("bar.sync", 2); break;
        case 3: XG_BAR("bar.sync", 3); break;
        case 4: XG_BAR("bar.sync", 4); break;
        case 5: XG_BAR("bar.sync", 5); break;
        case 6: XG_BAR("bar.sync", 6); break;
        default: XG_BAR("bar.sync", 7); break;
    }
}

// (float)(sum of four u8 x s8 products), exactly: the dp4a accumulates onto the bits of 1.5 * 2^23.
__device__ __forceinline__ float quad_dot(uint32_t w, int a) { return __fsub_rn(__int_as_float(dp_us(w, a, XG_MAGIC_I)), XG_MAGIC_F); }

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ int word_of(const int4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Shared-memory carve-up for a row length k.
struct XgSmem {
    int8_t *aq;     // [k]
    float *xs;      // [k/32]
    float *a16;     // [k/16] sums of 16 quants, as floats
    float *terms;   // [XG_ROWS][k/32 + 1]
    float *hs;      // [XG_ROWS]
};
__host__ __device__ inline size_t xg_smem_bytes(uint32_t k) {
    return (size_t)k + (size_t)(k / 32) * 4 + (size_t)(k / 16) * 4 + (size_t)XG_ROWS * (k / 32 + 1) * 4 + XG_ROWS * 4;
}

template <int T>
__global__ void __launch_bounds__(XG_THREADS) gemv_exact_kernel(const ExactParams p) {
    extern __shared__ __align__(16) uint8_t xg_smem[];
    const uint32_t k = p.k, nb32 = k >> 5, t128 = p.t128, nb = k >> 8;
    XgSmem s;
    s.aq = reinterpret_cast<int8_t *>(xg_smem);
    s.xs = reinterpret_cast<float *>(xg_smem + k);
    s.a16 = s.xs + nb32;
    s.terms = s.a16 + 2 * nb32;
    s.hs = s.terms + (size_t)XG_ROWS * (nb32 + 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = warp < XG_PRODUCERS;
    const uint32_t n_rounds = (p.total_rows + XG_ROWS - 1) / XG_ROWS;
    const uint32_t n_hand = (t128 + XG_SEG_TASKS - 1) / XG_SEG_TASKS;
    const TypeInfo ti = type_info(T);

    pdl_trigger();
    pdl_wait();
    tp_arrive_wait(p.tp.ctx, p.tp.wait_slot);
    // stage the activation column
    for (uint32_t i = tid; i < k / 16; i += XG_THREADS) {
        reinterpret_cast<int4 *>(s.aq)[i] = reinterpret_cast<const int4 *>(p.x.quants)[i];
        s.a16[i] = (float)p.x.sums[i];
    }
    for (uint32_t i = tid; i < nb32; i += XG_THREADS) s.xs[i] = p.x.scales[i];
    __syncthreads();

    for (uint32_t round = blockIdx.x; round < n_rounds; round += gridDim.x) {
        const uint32_t base = round * XG_ROWS;
        if (producer) {
            const int rslot = warp * 8 + (lane >> 2), c = lane & 3, pair = c >> 1, half = c & 1;
            uint32_t row = base + rslot;
            if (row >= p.total_rows) row = p.total_rows - 1;  // clamped rows compute a value nobody stores
            int sg = 0;
            while (sg + 1 < p.n_segs && row >= p.row_end[sg]) ++sg;
            const uint32_t local = row - (sg ? p.row_end[sg - 1] : 0);
            const WeightView &w = p.w[sg];
            // interleaved planes: piece (t, c) of row `local` at group base + (t*32 + (local%8)*4 + c) * 16, so the 32 lanes
            // of a warp (eight consecutive rows x four strips) read 512 contiguous bytes per load
            const uint8_t *strip = w.q + (size_t)(local >> 3) * 8 * ((size_t)nb * ti.q_b) + ((size_t)(local & 7) * 4 + c) * 16;
            const size_t sb0 = sb_index(w, local, 0);  // + 8 per super-block
            float *terms = s.terms + (size_t)rslot * (nb32 + 1);
            float acc_lo[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc_hi[4] = {0.0f, 0.0f, 0.0f, 0.0f};

            for (uint32_t hand = 0; hand < n_hand; ++hand) {
                const uint32_t t_end = min(t128, (hand + 1) * XG_SEG_TASKS);
                for (uint32_t t0 = hand * XG_SEG_TASKS; t0 < t_end; t0 += 8) {
                    // eight tasks = four super-blocks: all loads first
                    uint4 piece[8], head[4], hb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) piece[i] = ld_stream(strip + (size_t)(t0 + i) * 512);
#pragma unroll
                    for (int i = 0; i < 4; ++i) head[i] = __ldg(reinterpret_cast<const uint4 *>(w.hdr + (sb0 + (size_t)((t0 >> 1) + i) * 8) * 16));
                    if (T == CERA_TYPE_Q5_K) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) hb[i] = __ldg(reinterpret_cast<const uint4 *>(w.qh + (sb0 + (size_t)((t0 >> 1) + i) * 8) * 32 + half * 16));
                    }
                    if (T == CERA_TYPE_Q6_K) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t t = t0 + i;
                            hb[i] = __ldg(reinterpret_cast<const uint4 *>(w.qh + (sb0 + (size_t)(t >> 1) * 8) * 64 + (t & 1) * 32 + half * 16));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t t = t0 + i, hf = t & 1;
                        const uint4 h = head[i >> 1];
                        if (T == CERA_TYPE_Q4_K || T == CERA_TYPE_Q5_K) {
                            // low nibbles: block 4t + 2*pair (sub-block 4hf + 2*pair), high nibbles: the next one
                            const uint32_t xb_lo = 4 * t + 2 * pair, xb_hi = xb_lo + 1;
                            const int4 alo = *reinterpret_cast<const int4 *>(s.aq + 32 * xb_lo + 16 * half);
                            const int4 ahi = *reinterpret_cast<const int4 *>(s.aq + 32 * xb_hi + 16 * half);
                            uint32_t scp, mnp;
                            kq_quad(h, hf, scp, mnp);
                            const float d = h2f((uint16_t)(h.x & 0xFFFF)), dmin = h2f((uint16_t)(h.x >> 16));
                            const float sc_lo = byte_f(scp, 2 * pair), sc_hi = byte_f(scp, 2 * pair + 1);
                            const float scale_lo = __fmul_rn(s.xs[xb_lo], __fmul_rn(d, sc_lo));
                            const float scale_hi = __fmul_rn(s.xs[xb_hi], __fmul_rn(d, sc_hi));
                            const int sh_lo = 4 * hf + 2 * pair;  // fifth-bit position of the low-nibble sub-block (Q5_K)
#pragma unroll
                            for (int wd = 0; wd < 4; ++wd) {
                                const uint32_t v = word_of(piece[i], wd);
                                uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
                                if (T == CERA_TYPE_Q5_K) {
                                    const uint32_t b = word_of(hb[i >> 1], wd);
                                    lo |= ((b >> sh_lo) & 0x01010101u) << 4;
                                    hi |= ((b >> (sh_lo + 1)) & 0x01010101u) << 4;
                                }
                                acc_lo[wd] = fmaf(quad_dot(lo, word_of(alo, wd)), scale_lo, acc_lo[wd]);
                                acc_hi[wd] = fmaf(quad_dot(hi, word_of(ahi, wd)), scale_hi, acc_hi[wd]);
                            }
                            // this lane's share of the macc terms: half 0 -> the low-nibble block, half 1 -> the high one
                            const uint32_t xbm = half ? xb_hi : xb_lo;
                            const float mn = byte_f(mnp, 2 * pair + half);
                            const float a32 = __fadd_rn(s.a16[2 * xbm], s.a16[2 * xbm + 1]);  // two exact integers
                            terms[xbm] = __fmul_rn(__fmul_rn(s.xs[xbm], __fmul_rn(dmin, mn)), a32);
                        } else {
                            // Q6_K: low nibbles block 4t + pair, high nibbles block 4t + pair + 2; task t = (super-block, half nh)
                            const uint32_t nh = hf, xb_lo = 4 * t + pair, xb_hi = xb_lo + 2;
                            const int4 alo = *reinterpret_cast<const int4 *>(s.aq + 32 * xb_lo + 16 * half);
                            const int4 ahi = *reinterpret_cast<const int4 *>(s.aq + 32 * xb_hi + 16 * half);
                            // h = the 16 int8 scales of the super-block; lanes 0-3 of a block use scales[8nh + 2g], lanes 4-7 the next
                            const uint32_t sw_lo = nh ? h.z : h.x, sw_hi = nh ? h.w : h.y;  // scales[8nh .. +3], [8nh+4 .. +7]
                            const float d = h2f(__ldg(reinterpret_cast<const uint16_t *>(w.d) + sb0 + (size_t)(t >> 1) * 8));
                            const float sc_lo = (float)(int8_t)(sw_lo >> (8 * (2 * pair + half)));
                            const float sc_hi = (float)(int8_t)(sw_hi >> (8 * (2 * pair + half)));
                            const float scale_lo = __fmul_rn(__fmul_rn(sc_lo, d), s.xs[xb_lo]);
                            const float scale_hi = __fmul_rn(__fmul_rn(sc_hi, d), s.xs[xb_hi]);
#pragma unroll
                            for (int wd = 0; wd < 4; ++wd) {
                                const uint32_t v = word_of(piece[i], wd), b = word_of(hb[i], wd);
                                const uint32_t lo = (v & 0x0F0F0F0Fu) | (((b >> (2 * pair)) & 0x03030303u) << 4);
                                const uint32_t hi = ((v >> 4) & 0x0F0F0F0Fu) | (((b >> (2 * pair + 4)) & 0x03030303u) << 4);
                                acc_lo[wd] = fmaf(quad_dot(lo, word_of(alo, wd)), scale_lo, acc_lo[wd]);
                                acc_hi[wd] = fmaf(quad_dot(hi, word_of(ahi, wd)), scale_hi, acc_hi[wd]);
                            }
                            // macc term of one block per lane: xs * (32 d) * (sc0 * A0 + sc1 * A1), both scale bytes of the block
                            const uint32_t xbm = half ? xb_hi : xb_lo;
                            const uint32_t swm = half ? sw_hi : sw_lo;
                            const float m0 = (float)(int8_t)(swm >> (8 * (2 * pair))), m1 = (float)(int8_t)(swm >> (8 * (2 * pair + 1)));
                            const float inner = __fadd_rn(__fmul_rn(m0, s.a16[2 * xbm]), __fmul_rn(m1, s.a16[2 * xbm + 1]));
                            terms[xbm] = __fmul_rn(__fmul_rn(s.xs[xbm], __fmul_rn(d, 32.0f)), inner);
                        }
                    }
                }
                __threadfence_block();
                bar_arrive(1 + (int)hand);  // the chain warp may add this segment's terms
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
            if (c == 0) s.hs[rslot] = hsum;
            __threadfence_block();
            bar_arrive(7);
        } else {
            // ---- chain warp: lane i owns row base + i
            const float *terms = s.terms + (size_t)lane * (nb32 + 1);
            float macc = 0.0f;
            for (uint32_t hand = 0; hand < n_hand; ++hand) {
                bar_sync(1 + (int)hand);
                const uint32_t b_end = min(nb32, (hand + 1) * XG_SEG_TASKS * 4);
#pragma unroll 8
                for (uint32_t xb = hand * XG_SEG_TASKS * 4; xb < b_end; ++xb) macc = __fadd_rn(macc, terms[xb]);
            }
            bar_sync(7);
            const uint32_t row = base + lane;
            const bool valid = row < p.total_rows;
            const float r = __fsub_rn(s.hs[lane], macc);
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
        __syncthreads();  // the terms of this round are consumed before the next round overwrites them
    }
}

template <int T>
int32_t launch_exact_typed(const ExactParams &p, cudaStream_t st) {
    const size_t smem = xg_smem_bytes(p.k);
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        CERA_CUDA_TRY(cudaFuncSetAttribute(gemv_exact_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = 200 * 1024;
    }
    const uint32_t rounds = (p.total_rows + XG_ROWS - 1) / XG_ROWS;
    const uint32_t cap = (uint32_t)sm_count() * 8;
    count_launch();
    return check_cuda(launch_k(gemv_exact_kernel<T>, dim3(rounds < cap ? rounds : cap), dim3(XG_THREADS), smem, st, p), "gemv (reference order) launch");
}

}  // namespace

// CERA_CUDA_GEMV=rows keeps the decode GEMVs on the register-streaming kernel whose f32 order is its own (A/B runs); read once.
static bool exact_off() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_GEMV");
        return e && (strcmp(e, "rows") == 0 || strcmp(e, "tma") == 0 || strcmp(e, "direct") == 0);
    }();
    return v;
}

// Single-column GEMV in the reference's f32 order over up to three same-typed K-quant matrices.
// *taken = false: not a K-quant, k not a multiple of 256, or a shape outside the kernel's rules;
// nothing was launched.
int32_t launch_gemv_exact(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp) {
    *taken = false;
    if (exact_off() || n_segs < 1 || n_segs > XG_MAX_SEGS) return CERA_CUDA_OK;
    const int type = segs[0].w.type;
    if (type != CERA_TYPE_Q4_K && type != CERA_TYPE_Q5_K && type != CERA_TYPE_Q6_K) return CERA_CUDA_OK;
    const uint32_t k = segs[0].w.k, t128 = segs[0].w.t128;
    if (k % 1024 || t128 != k / 128 || (t128 + XG_SEG_TASKS - 1) / XG_SEG_TASKS > XG_MAX_HANDOVERS) return CERA_CUDA_OK;
    for (int i = 0; i < n_segs; ++i)
        if (segs[i].w.ilv != 8) return CERA_CUDA_OK;
    if (xg_smem_bytes(k) > 200 * 1024) return CERA_CUDA_OK;
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
    p.t128 = t128;
    p.epilogue = epilogue;
    *taken = true;
    if (type == CERA_TYPE_Q4_K) return launch_exact_typed<CERA_TYPE_Q4_K>(p, st);
    if (type == CERA_TYPE_Q5_K) return launch_exact_typed<CERA_TYPE_Q5_K>(p, st);
    return launch_exact_typed<CERA_TYPE_Q6_K>(p, st);
}

}  // namespace cera
