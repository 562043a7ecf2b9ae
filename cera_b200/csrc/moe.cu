// Routed feed-forward of an lfm2moe layer for a batch of tokens, grouped by expert.
//
// Reference (per token, unbatched on every backend): cera/src/model/lfm2.rs:177-226
// (select_experts), 673-715 (route_experts), 735-901 (forward_moe_ffn), 914-937 (prefill_moe_ffn).
//   probs = sigmoid(router . x)                         F32 router, std exp
//   pick n_used experts by probs + exp_probs_b, ties to the lower index
//   weights = unbiased probs of the picked, divided by max(their sum, 2^-14)
//   out = sum over the picks in pick order of weight * down_e(silu(gate_e x) * up_e x)
// with every expert projection an int8 GEMV against Q8_0-quantized input, like the dense FFN.
//
// Here the (token, pick) pairs of the whole batch are bucketed by expert (counting sort on the
// device), the Q8_0 columns are gathered into bucket order, and one launch per projection walks a
// device-built list of (expert, column tile) work items: each expert's weights are streamed once per
// eight of its tokens instead of once per token -- or, for batches, once per 64 of its tokens through the
// tensor-core GEMM of gemm_mma.cu in its expert-grouped form.  The stacked expert tensors
// (blk.N.ffn_{gate,up,down}_exps.weight, [n_expert][m][k] with expert stride m rows,
// cera/src/model/gpu_weight_source.rs:179-257) are one weight matrix of n_expert*m rows here.
//
// Expert parallelism (cera_cuda_moe_create_ep, one process per GPU): rank r holds experts
// [r*E/G, (r+1)*E/G) and its own share of the tokens.  Per call, on the device and without a host
// round trip: route the local tokens; publish the per-expert counts to every rank; from the G x E
// count table every rank derives where its (token, pick) entries land in the owning rank's receive
// buffer (grouped by expert, then by source rank); DISPATCH = each entry's Q8_0 column is stored
// straight into the owner's buffer over NVLink together with (source rank, pair index); the owner
// runs the grouped GEMMs over what it received; COMBINE = each result row is stored straight into
// the source rank's return buffer at the pair index, and the source adds its picks in pick order.
// Both all-to-alls are peer stores issued by the kernels themselves, with the flag protocol of
// tp.cu between the phases.  Every (token, expert) product and the combine order are those of the
// single-GPU path, so results are bit-identical for any number of ranks.
#include <cstdlib>
#include <cstring>
#include <new>

#include "gemv_item.cuh"
#include "ops.h"
#include "weight.h"

using namespace cera;

namespace {

constexpr int MOE_MAX_EXPERTS = 256;  // the reference's stack buffer (lfm2.rs:180)
constexpr int MOE_MAX_USED = 16;
constexpr int MOE_NC = 8;             // token columns per work item
constexpr int MOE_WARPS = 8;

constexpr int MOE_NC_MMA = 64;        // ... when the projections run on the tensor-core GEMM

// ---- routing -------------------------------------------------------------------------------------
// One CTA per token.  Warps take experts round-robin; lane-strided f32 dot, shuffle tree.
__global__ void __launch_bounds__(256) moe_route_kernel(const float *__restrict__ x, const float *__restrict__ router,
                                                        const float *__restrict__ bias, uint32_t hidden, uint32_t n_expert,
                                                        uint32_t n_used, int softmax_gate, uint32_t *ids, float *weights,
                                                        uint32_t *counts) {
    __shared__ float probs[MOE_MAX_EXPERTS];
    const uint32_t j = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *xj = x + (size_t)j * hidden;
    for (uint32_t e = warp; e < n_expert; e += blockDim.x >> 5) {
        const float *r = router + (size_t)e * hidden;
        float acc = 0.0f;
        for (uint32_t i = lane; i < hidden; i += 32) acc = fmaf(r[i], xj[i], acc);
        acc = warp_sum(acc);
        if (lane == 0) probs[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (softmax_gate) {
        float mx = probs[0];
        for (uint32_t e = 1; e < n_expert; ++e) mx = fmaxf(mx, probs[e]);
        float sum = 0.0f;
        for (uint32_t e = 0; e < n_expert; ++e) {
            probs[e] = expf(probs[e] - mx);
            sum += probs[e];
        }
        for (uint32_t e = 0; e < n_expert; ++e) probs[e] = probs[e] / sum;
    } else {
        for (uint32_t e = 0; e < n_expert; ++e) probs[e] = 1.0f / (1.0f + expf(-probs[e]));
    }
    uint32_t picked[MOE_MAX_USED];
    float w[MOE_MAX_USED];
    float denom = 0.0f;
    for (uint32_t s = 0; s < n_used; ++s) {
        int best = -1;
        float best_v = 0.0f;
        for (uint32_t e = 0; e < n_expert; ++e) {
            bool taken = false;
            for (uint32_t t = 0; t < s; ++t) taken |= picked[t] == e;
            if (taken) continue;
            const float v = probs[e] + (bias ? bias[e] : 0.0f);
            // total order on finite values; strict > keeps the lower index on ties
            if (best < 0 || v > best_v) {
                best = (int)e;
                best_v = v;
            }
        }
        picked[s] = (uint32_t)best;
        w[s] = probs[best];
        denom += w[s];
    }
    denom = fmaxf(denom, 1.0f / 16384.0f);
    for (uint32_t s = 0; s < n_used; ++s) {
        ids[(size_t)j * n_used + s] = picked[s];
        weights[(size_t)j * n_used + s] = w[s] / denom;
        atomicAdd(counts + picked[s], 1u);
    }
}

// Appends the work items of one expert's `c` entries starting at bucket offset `off`: items of `nc` columns go to
// the main list; a last item of at most `small_nc` columns (0 = no such list) goes to the list of narrow items at
// tiles[cap...], which a narrower kernel serves.
__device__ __forceinline__ void moe_emit_items(MoeTile *tiles, uint32_t cap, uint32_t &t, uint32_t &ts, uint32_t e, uint32_t off,
                                               uint32_t c, uint32_t nc, uint32_t small_nc) {
    for (uint32_t f = 0; f < c; f += nc) {
        const uint32_t n = c - f < nc ? c - f : nc;
        if (small_nc && n <= small_nc) tiles[cap + ts++] = MoeTile{e, off + f, n};
        else tiles[t++] = MoeTile{e, off + f, n};
    }
}

// One CTA: bucket offsets, cursors, and the work lists (n_tiles[0] main, n_tiles[1] narrow).  counts is zeroed again
// for the next call.
__global__ void moe_plan_kernel(uint32_t *counts, uint32_t n_expert, uint32_t nc, uint32_t small_nc, uint32_t cap, uint32_t *cursor,
                                MoeTile *tiles, uint32_t *n_tiles) {
    if (threadIdx.x != 0) return;
    uint32_t off = 0, t = 0, ts = 0;
    for (uint32_t e = 0; e < n_expert; ++e) {
        const uint32_t c = counts[e];
        cursor[e] = off;
        moe_emit_items(tiles, cap, t, ts, e, off, c, nc, small_nc);
        off += c;
        counts[e] = 0;
    }
    n_tiles[0] = t;
    n_tiles[1] = ts;
}

// One CTA per (token, pick): take the next place in the expert's bucket and copy the token's Q8_0 column there.
__global__ void __launch_bounds__(128) moe_scatter_kernel(const uint32_t *__restrict__ ids, uint32_t n_used, uint32_t hidden,
                                                          ActView x, uint32_t *cursor, uint32_t *entry_of, float *g_scales,
                                                          int8_t *g_quants, int16_t *g_sums) {
    __shared__ uint32_t pos_s;
    const uint32_t pair = blockIdx.x, j = pair / n_used;
    if (threadIdx.x == 0) {
        pos_s = atomicAdd(cursor + ids[pair], 1u);
        entry_of[pair] = pos_s;
    }
    __syncthreads();
    const size_t pos = pos_s;
    const uint32_t *sq = (const uint32_t *)(x.quants + (size_t)j * hidden);
    uint32_t *dq = (uint32_t *)(g_quants + pos * hidden);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += blockDim.x) dq[i] = sq[i];
    for (uint32_t i = threadIdx.x; i < hidden / 32; i += blockDim.x)
        g_scales[pos * (hidden / 32) + i] = x.scales[(size_t)j * (hidden / 32) + i];
    for (uint32_t i = threadIdx.x; i < hidden / 16; i += blockDim.x)
        g_sums[pos * (hidden / 16) + i] = x.sums[(size_t)j * (hidden / 16) + i];
}

// ---- grouped GEMM ----------------------------------------------------------------------------------
// blockIdx.y walks the work list; inside an item the CTA's warps take rows of the expert's matrices
// (up to two segments sharing the activations: gate and up).  Cell (row i, entry c) -> y[c*ldc + i].
struct MoeGemmParams {
    WeightView w[2];
    float *y[2];
    int n_segs;
    uint32_t m;  // rows per expert and segment
    uint32_t k;
    ActView x;   // columns in bucket order
    uint32_t ldc;
    const MoeTile *tiles;
    const uint32_t *n_tiles;
};

template <int T, int NC>
__global__ void __launch_bounds__(MOE_WARPS * 32) moe_gemm_kernel(const MoeGemmParams p) {
    using F = Fmt<T>;
    if (blockIdx.y >= *p.n_tiles) return;
    const MoeTile tile = p.tiles[blockIdx.y];
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * MOE_WARPS + (threadIdx.x >> 5), n_warps = gridDim.x * MOE_WARPS;
    const int items = p.k >> 5;
    const ActView x{p.x.scales + (size_t)tile.first * (p.k / 32), p.x.quants + (size_t)tile.first * p.k,
                    p.x.sums + (size_t)tile.first * (p.k / 16)};
    const uint32_t total = p.m * p.n_segs;
    for (uint32_t row = warp; row < total; row += n_warps) {
        const int s = row >= p.m ? 1 : 0;
        const uint32_t local = row - s * p.m;
        const WeightView &w = p.w[s];
        const size_t wrow = (size_t)tile.expert * p.m + local;
        float acc[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] = 0.0f;
        for (int item = lane; item < items; item += 32) {
            const typename F::Raw raw = F::load(w, wrow, item);
            accumulate_item<T, NC>(raw, item, x, p.k, acc);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] = warp_sum(acc[c]);
        if (lane == 0) {
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if ((uint32_t)c < tile.count) p.y[s][(size_t)(tile.first + c) * p.ldc + local] = acc[c];
        }
    }
}

// out[j][i] = sum over picks in pick order of weight * expert_out[entry][i]; multiply and add rounded
// separately, as the reference's `*acc += weight * v` is (lfm2.rs:891-897).
__global__ void moe_combine_kernel(const float *__restrict__ expert_out, const uint32_t *__restrict__ entry_of,
                                   const float *__restrict__ weights, uint32_t n_used, uint32_t hidden, size_t n, float *out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * hidden) return;
    const size_t j = idx / hidden, i = idx - j * hidden;
    float acc = 0.0f;
    for (uint32_t s = 0; s < n_used; ++s) {
        const size_t e = entry_of ? entry_of[j * n_used + s] : j * n_used + s;
        acc = __fadd_rn(acc, __fmul_rn(weights[j * n_used + s], expert_out[e * hidden + i]));
    }
    out[idx] = acc;
}

// ---- expert-parallel pieces ------------------------------------------------------------------------
struct EpLayout {  // byte offsets inside every rank's exchange region
    uint32_t counts, r_scales, r_quants, r_sums, r_meta, ret_out;
};

// Status word values of the expert-parallel call beyond the timeout codes of tp.cuh.
constexpr uint32_t EP_STATUS_OVERFLOW = 0x40000000u;  // | destination rank << 24: more entries than a receive buffer holds

// One CTA.  counts_all[G][E] (every rank's per-expert entry counts) -> my_base[e] = first slot, in the
// receive buffer of e's owner, of this rank's entries for expert e; the work list over what THIS rank
// receives for its local experts; *n_recv.  Zeroes this rank's own count row for the next call.
// Every receive buffer holds `limit` entries.  If the counts of any destination add up to more (the
// ranks' token counts exceed what the layer was created for), or an earlier exchange of this layer ran
// out of time (the table may then mix rows of different calls), nothing may be stored into a peer:
// *skip is set, the work list and *n_recv are emptied, and the status word names the cause.
__global__ void moe_ep_plan_kernel(TpCtx c, EpLayout lay, uint32_t n_expert, uint32_t nc, uint32_t small_nc, uint32_t cap,
                                   uint32_t limit, uint32_t *my_base, uint32_t *cursor, MoeTile *tiles, uint32_t *n_tiles,
                                   uint32_t *n_recv, uint32_t *skip) {
    if (threadIdx.x != 0) return;
    uint32_t *counts = (uint32_t *)(c.peer[c.rank] + lay.counts);
    const uint32_t per = n_expert / c.size;
    uint32_t t = 0, ts = 0;
    bool bad = *(volatile uint32_t *)c.status != 0;
    for (uint32_t d = 0; d < c.size && !bad; ++d) {
        uint64_t tot_d = 0;
        for (uint32_t e = d * per; e < (d + 1) * per; ++e)
            for (uint32_t src = 0; src < c.size; ++src) tot_d += counts[src * n_expert + e];
        if (tot_d > limit) {
            atomicCAS(c.status, 0u, EP_STATUS_OVERFLOW | (d << 24));
            bad = true;
        }
    }
    for (uint32_t d = 0; d < c.size && !bad; ++d) {
        uint32_t off = 0;  // running slot in rank d's receive buffer
        for (uint32_t e = d * per; e < (d + 1) * per; ++e) {
            uint32_t tot = 0, before_me = 0;
            for (uint32_t src = 0; src < c.size; ++src) {
                const uint32_t n = counts[src * n_expert + e];
                if (src < c.rank) before_me += n;
                tot += n;
            }
            my_base[e] = off + before_me;
            cursor[e] = 0;
            if (d == c.rank) moe_emit_items(tiles, cap, t, ts, e - d * per, off, tot, nc, small_nc);
            off += tot;
        }
        if (d == c.rank) *n_recv = off;
    }
    if (bad) {
        t = ts = 0;
        *n_recv = 0;
    }
    *skip = bad ? 1u : 0u;
    n_tiles[0] = t;
    n_tiles[1] = ts;
    for (uint32_t e = 0; e < n_expert; ++e) counts[c.rank * n_expert + e] = 0;
}

// One CTA per local (token, pick): claim the next slot of this rank's range for the expert and store the
// token's Q8_0 column and its return address into the owner's receive buffer.
__global__ void __launch_bounds__(128) moe_ep_dispatch_kernel(TpCtx c, EpLayout lay, const uint32_t *__restrict__ ids,
                                                              uint32_t n_used, uint32_t hidden, uint32_t n_expert, ActView x,
                                                              const uint32_t *__restrict__ my_base, uint32_t *cursor,
                                                              const uint32_t *__restrict__ skip) {
    __shared__ uint32_t pos_s;
    if (*skip) return;  // the plan found the receive buffers too small, or an earlier exchange timed out
    const uint32_t pair = blockIdx.x, j = pair / n_used, e = ids[pair];
    if (threadIdx.x == 0) pos_s = my_base[e] + atomicAdd(cursor + e, 1u);
    __syncthreads();
    const size_t pos = pos_s;
    char *dst = c.peer[e / (n_expert / c.size)];
    const uint4 *sq = (const uint4 *)(x.quants + (size_t)j * hidden);
    uint4 *dq = (uint4 *)(dst + lay.r_quants + pos * hidden);
    for (uint32_t i = threadIdx.x; i < hidden / 16; i += blockDim.x) dq[i] = sq[i];
    float *ds = (float *)(dst + lay.r_scales) + pos * (hidden / 32);
    for (uint32_t i = threadIdx.x; i < hidden / 32; i += blockDim.x) ds[i] = x.scales[(size_t)j * (hidden / 32) + i];
    int16_t *dm = (int16_t *)(dst + lay.r_sums) + pos * (hidden / 16);
    for (uint32_t i = threadIdx.x; i < hidden / 16; i += blockDim.x) dm[i] = x.sums[(size_t)j * (hidden / 16) + i];
    if (threadIdx.x == 0) ((uint32_t *)(dst + lay.r_meta))[pos] = (c.rank << 24) | pair;
}

// SiLU*mul + Q8_0 over the first *n_rows rows (a device-side count) of g / u: one warp per 32-element block.
__global__ void moe_silu_q8_kernel(float *g, const float *__restrict__ u, uint32_t ff, const uint32_t *__restrict__ n_rows,
                                   float *scales, int8_t *quants, int16_t *sums) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)*n_rows * ff) return;  // ff % 32 == 0: whole warps leave together
    const float v = silu_mul(g[i], u[i]);
    float scale;
    int hs;
    const int q = quantize_lane(v, scale, hs);
    const int lane = threadIdx.x & 31;
    quants[i] = (int8_t)q;
    if (lane == 0) scales[i / 32] = scale;
    if ((lane & 15) == 0) sums[i / 16] = (int16_t)hs;
}

// One CTA per received entry: store its result row into the source rank's return buffer at the pair index.
__global__ void __launch_bounds__(128) moe_ep_return_kernel(TpCtx c, EpLayout lay, const float *__restrict__ expert_out,
                                                            uint32_t hidden, const uint32_t *__restrict__ n_recv) {
    const uint32_t i = blockIdx.x;
    if (i >= *n_recv) return;
    const uint32_t meta = ((const uint32_t *)(c.peer[c.rank] + lay.r_meta))[i];
    const uint32_t src = meta >> 24, pair = meta & 0xFFFFFFu;
    const float4 *s = (const float4 *)(expert_out + (size_t)i * hidden);
    float4 *d = (float4 *)(c.peer[src] + lay.ret_out) + (size_t)pair * (hidden / 4);
    for (uint32_t t = threadIdx.x; t < hidden / 4; t += blockDim.x) d[t] = s[t];
}

template <int T>
int32_t launch_moe_gemm(const MoeGemmParams &p, uint32_t max_tiles, bool single, cudaStream_t st) {
    const uint32_t rows = p.m * p.n_segs;
    uint32_t gx = (rows + MOE_WARPS - 1) / MOE_WARPS;
    const uint32_t want = (uint32_t)sm_count() * 8 / (max_tiles ? max_tiles : 1) + 1;  // a few waves over all items
    if (gx > want) gx = want;
    if (gx < 1) gx = 1;
    if (single)
        moe_gemm_kernel<T, 1><<<dim3(gx, max_tiles), MOE_WARPS * 32, 0, st>>>(p);
    else
        moe_gemm_kernel<T, MOE_NC><<<dim3(gx, max_tiles), MOE_WARPS * 32, 0, st>>>(p);
    count_launch();
    return check_cuda(cudaGetLastError(), "moe grouped gemm launch");
}

// CERA_CUDA_MOE=dp4a keeps the grouped projections on the dp4a kernel (A/B runs); read once.
bool moe_force_dp4a() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_MOE");
        return e && strcmp(e, "dp4a") == 0;
    }();
    return v;
}

// One grouped projection over the work list: the tensor-core GEMM when the plan was made for it, else the dp4a kernel.
// cap / max_small: where the list of narrow items starts inside p.tiles and how many it can hold (tensor-core plan only).
int32_t grouped_projection(bool mma, const MoeGemmParams &p, uint32_t max_tiles, uint32_t cap, uint32_t max_small, bool single,
                           cudaStream_t st) {
    if (mma) {
        for (int s = 0; s < p.n_segs; ++s) {
            bool taken = false;
            CERA_TRY(launch_gemm_mma_grouped(p.w[s], p.x, p.tiles, p.n_tiles, max_tiles, p.m, p.y[s], p.ldc, MOE_NC_MMA, st, &taken));
            if (!taken) return fail(CERA_CUDA_ERR_STATE, "moe: tensor-core plan without a tensor-core kernel");
            // an expert's last, at most half-filled item runs on the 32-column kernel
            CERA_TRY(launch_gemm_mma_grouped(p.w[s], p.x, p.tiles + cap, p.n_tiles + 1, max_small, p.m, p.y[s], p.ldc, MOE_NC_MMA / 2, st,
                                             &taken));
        }
        return CERA_CUDA_OK;
    }
    CERA_DISPATCH_BLOCK_TYPE(p.w[0].type, return (launch_moe_gemm<TT>(p, max_tiles, single, st)));
    return CERA_CUDA_OK;
}

}  // namespace

struct cera_cuda_moe {
    uint32_t n_expert = 0, n_used = 0, hidden = 0, ff = 0;
    size_t max_tokens = 0;
    int device = 0;
    cera_cuda_weight *gate = nullptr, *up = nullptr, *down = nullptr;
    char *base = nullptr;  // one allocation: router, bias and every scratch array
    size_t bytes = 0;
    float *router = nullptr, *bias = nullptr;
    // scratch
    float *xs = nullptr, *g_scales = nullptr, *f_scales = nullptr, *weights = nullptr, *g = nullptr, *u = nullptr,
          *expert_out = nullptr;
    int8_t *xq = nullptr, *g_quants = nullptr, *f_quants = nullptr;
    int16_t *xsum = nullptr, *g_sums = nullptr, *f_sums = nullptr;
    uint32_t *ids = nullptr, *counts = nullptr, *cursor = nullptr, *entry_of = nullptr, *n_tiles = nullptr;
    MoeTile *tiles = nullptr;
    // expert parallelism
    uint32_t ep_rank = 0, ep_size = 1;
    size_t max_total = 0;     // tokens of all ranks in one call
    char *region = nullptr;   // exchange region (its own allocation, mapped by the peers)
    size_t region_bytes = 0;
    TpCtx ep{};
    EpLayout lay{};
    void *opened[TP_MAX_RANKS] = {};
    bool connected = false;
    uint32_t *ep_words = nullptr;  // device: [0] sequence, [16] status, [32] n_recv
    uint32_t *my_base = nullptr;
};

namespace {

int32_t moe_create_impl(uint32_t n_expert, uint32_t n_used, uint32_t hidden, uint32_t ff, int32_t ggml_type,
                        const void *gate_exps, const void *up_exps, const void *down_exps, size_t gate_up_bytes,
                        size_t down_bytes, const float *router, const float *exp_probs_b, size_t max_tokens, uint32_t ep_rank,
                        uint32_t ep_size, size_t max_total_tokens, cera_cuda_moe **out) {
    if (!gate_exps || !up_exps || !down_exps || !router || !out) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: null argument");
    if (ep_size == 0 || ep_size > TP_MAX_RANKS || ep_rank >= ep_size || n_expert % ep_size)
        return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: rank %u of %u for %u experts", ep_rank, ep_size, n_expert);
    if (ep_size > 1 && max_total_tokens < max_tokens)
        return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: max_total_tokens %zu is below this rank's max_tokens %zu", max_total_tokens, max_tokens);
    if (ep_size > 1 && max_total_tokens * n_used >= (1u << 24))
        return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: %zu tokens x %u picks do not fit the 24-bit pair index", max_total_tokens, n_used);
    if (n_expert == 0 || n_expert > MOE_MAX_EXPERTS || n_used == 0 || n_used > MOE_MAX_USED || n_used > n_expert)
        return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: %u experts, %u used (limits %d, %d)", n_expert, n_used, MOE_MAX_EXPERTS, MOE_MAX_USED);
    if (hidden % 32 || ff % 32 || hidden == 0 || ff == 0 || max_tokens == 0)
        return fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: hidden %u and expert width %u must be positive multiples of 32", hidden, ff);
    auto *h = new (std::nothrow) cera_cuda_moe();
    if (!h) return fail(CERA_CUDA_ERR_OOM, "moe_create: host allocation failed");
    h->n_expert = n_expert;
    h->n_used = n_used;
    h->hidden = hidden;
    h->ff = ff;
    h->max_tokens = max_tokens;
    h->ep_rank = ep_rank;
    h->ep_size = ep_size;
    h->max_total = ep_size > 1 ? max_total_tokens : max_tokens;
    cudaGetDevice(&h->device);
    // this rank's experts: a contiguous row range of the stacked tensors (all of them on one GPU)
    const uint32_t n_local = n_expert / ep_size;
    int32_t st = CERA_CUDA_OK;
    if (gate_up_bytes % n_expert || down_bytes % n_expert)
        st = fail(CERA_CUDA_ERR_BAD_ARG, "moe_create: expert tensors of %zu / %zu bytes do not split into %u experts", gate_up_bytes, down_bytes, n_expert);
    const size_t gu_e = gate_up_bytes / n_expert, dn_e = down_bytes / n_expert;
    const char *gp = (const char *)gate_exps + (size_t)ep_rank * n_local * gu_e, *upp = (const char *)up_exps + (size_t)ep_rank * n_local * gu_e,
               *dp = (const char *)down_exps + (size_t)ep_rank * n_local * dn_e;
    if (st == CERA_CUDA_OK) st = weight_upload(ggml_type, (size_t)n_local * ff, hidden, gp, (size_t)n_local * gu_e, false, &h->gate);
    if (st == CERA_CUDA_OK) st = weight_upload(ggml_type, (size_t)n_local * ff, hidden, upp, (size_t)n_local * gu_e, false, &h->up);
    if (st == CERA_CUDA_OK) st = weight_upload(ggml_type, (size_t)n_local * hidden, ff, dp, (size_t)n_local * dn_e, false, &h->down);
    // entries this rank may have to process: its own tokens' picks, or with expert parallelism every rank's
    const size_t entries = h->max_total * n_used, pad = MOE_NC;  // a ragged tile still reads MOE_NC columns
    size_t off = 0;
    auto take = [&](size_t b) {
        const size_t at = off;
        off += (b + 255) & ~(size_t)255;
        return at;
    };
    const size_t o_router = take((size_t)n_expert * hidden * 4), o_bias = take((size_t)n_expert * 4),
                 o_xs = take(max_tokens * (hidden / 32) * 4), o_xq = take(max_tokens * hidden), o_xsum = take(max_tokens * (hidden / 16) * 2),
                 o_gs = take((entries + pad) * (hidden / 32) * 4), o_gq = take((entries + pad) * hidden),
                 o_gsum = take((entries + pad) * (hidden / 16) * 2), o_fs = take((entries + pad) * (ff / 32) * 4),
                 o_fq = take((entries + pad) * ff), o_fsum = take((entries + pad) * (ff / 16) * 2), o_w = take(entries * 4),
                 o_g = take(entries * ff * 4), o_u = take(entries * ff * 4), o_eo = take(entries * hidden * 4),
                 o_ids = take(entries * 4), o_counts = take((size_t)n_expert * 4), o_cursor = take((size_t)n_expert * 4),
                 o_entry = take(entries * 4), o_nt = take(8), o_tiles = take(2 * (entries + n_expert) * sizeof(MoeTile)),
                 o_words = take(64 * 4), o_base = take((size_t)n_expert * 4);
    h->bytes = off;
    if (st == CERA_CUDA_OK) st = check_cuda(cudaMalloc((void **)&h->base, off), "cudaMalloc(moe scratch)");
    if (st == CERA_CUDA_OK) st = check_cuda(cudaMemset(h->base, 0, off), "cudaMemset(moe scratch)");
    if (st == CERA_CUDA_OK) {
        char *b = h->base;
        h->router = (float *)(b + o_router);
        h->bias = exp_probs_b ? (float *)(b + o_bias) : nullptr;
        h->xs = (float *)(b + o_xs);
        h->xq = (int8_t *)(b + o_xq);
        h->xsum = (int16_t *)(b + o_xsum);
        h->g_scales = (float *)(b + o_gs);
        h->g_quants = (int8_t *)(b + o_gq);
        h->g_sums = (int16_t *)(b + o_gsum);
        h->f_scales = (float *)(b + o_fs);
        h->f_quants = (int8_t *)(b + o_fq);
        h->f_sums = (int16_t *)(b + o_fsum);
        h->weights = (float *)(b + o_w);
        h->g = (float *)(b + o_g);
        h->u = (float *)(b + o_u);
        h->expert_out = (float *)(b + o_eo);
        h->ids = (uint32_t *)(b + o_ids);
        h->counts = (uint32_t *)(b + o_counts);
        h->cursor = (uint32_t *)(b + o_cursor);
        h->entry_of = (uint32_t *)(b + o_entry);
        h->n_tiles = (uint32_t *)(b + o_nt);
        h->tiles = (MoeTile *)(b + o_tiles);
        h->ep_words = (uint32_t *)(b + o_words);
        h->my_base = (uint32_t *)(b + o_base);
        st = check_cuda(cudaMemcpy(h->router, router, (size_t)n_expert * hidden * 4, cudaMemcpyDefault), "cudaMemcpy(router)");
        if (st == CERA_CUDA_OK && exp_probs_b)
            st = check_cuda(cudaMemcpy(h->bias, exp_probs_b, (size_t)n_expert * 4, cudaMemcpyDefault), "cudaMemcpy(exp_probs_b)");
    }
    if (st == CERA_CUDA_OK && ep_size > 1) {
        // exchange region: count table, receive buffers for every entry of the job, return buffer for this rank's pairs
        size_t ro = 0;
        auto rtake = [&](size_t b) {
            const size_t at = ro;
            ro += (b + 255) & ~(size_t)255;
            return at;
        };
        const size_t rmax = h->max_total * n_used + MOE_NC;
        h->lay.counts = (uint32_t)rtake((size_t)ep_size * n_expert * 4);
        h->lay.r_scales = (uint32_t)rtake(rmax * (hidden / 32) * 4);
        h->lay.r_quants = (uint32_t)rtake(rmax * hidden);
        h->lay.r_sums = (uint32_t)rtake(rmax * (hidden / 16) * 2);
        h->lay.r_meta = (uint32_t)rtake(rmax * 4);
        h->lay.ret_out = (uint32_t)rtake(max_tokens * n_used * (size_t)hidden * 4);
        const size_t o_flags = rtake(4 * TP_MAX_RANKS * 4);
        h->region_bytes = (ro + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
        if (h->region_bytes > 0xFFFFFFFFull) st = fail(CERA_CUDA_ERR_UNSUPPORTED, "moe_create: exchange region of %zu bytes", h->region_bytes);
        if (st == CERA_CUDA_OK) st = check_cuda(cudaMalloc((void **)&h->region, h->region_bytes), "cudaMalloc(moe exchange region)");
        if (st == CERA_CUDA_OK) st = check_cuda(cudaMemset(h->region, 0, h->region_bytes), "cudaMemset(moe exchange region)");
        h->ep.rank = ep_rank;
        h->ep.size = ep_size;
        h->ep.peer[ep_rank] = h->region;
        h->ep.flags_off = (uint32_t)o_flags;
        h->ep.seq = h->ep_words;
        h->ep.status = h->ep_words + 16;
        const char *e = getenv("CERA_CUDA_TP_TIMEOUT_MS");
        const long ms = e ? atol(e) : 5000;
        h->ep.timeout_ns = (uint64_t)(ms > 0 ? ms : 5000) * 1000000ull;
    }
    if (st != CERA_CUDA_OK) {
        cera_cuda_moe_free(h);
        return st;
    }
    *out = h;
    return CERA_CUDA_OK;
}

// The expert-parallel call: see the file header.
int32_t moe_ffn_ep(cera_cuda_moe *h, const float *x_dev, size_t n, int32_t softmax_gate, float *out_dev, uint32_t *ids_out_dev,
                   float *weights_out_dev, cudaStream_t st) {
    if (!h->connected) return fail(CERA_CUDA_ERR_STATE, "moe_ffn: expert-parallel layer is not connected to its peers");
    const uint32_t hs = h->hidden, ff = h->ff, ku = h->n_used, E = h->n_expert;
    const size_t entries = n * ku, rmax = h->max_total * ku;
    const bool mma = gemm_mma_supports(h->gate->v.type, hs) && gemm_mma_supports(h->down->v.type, ff) && !moe_force_dp4a();
    const uint32_t nc = mma ? MOE_NC_MMA : MOE_NC;
    const uint32_t max_tiles = (uint32_t)(rmax / nc + E / h->ep_size);
    uint32_t *counts_mine = (uint32_t *)(h->region + h->lay.counts) + (size_t)h->ep_rank * E;
    uint32_t *n_recv = h->ep_words + 32;
    CERA_TRY(launch_tp_tick(h->ep_words, st));
    if (n) {
        CERA_TRY(launch_quantize(x_dev, hs, n, false, h->xs, h->xq, h->xsum, st));
        moe_route_kernel<<<(unsigned)n, 256, 0, st>>>(x_dev, h->router, h->bias, hs, E, ku, softmax_gate, h->ids, h->weights, counts_mine);
        count_launch();
    }
    // all ranks learn all counts
    const TpRange cr{(uint32_t)((char *)counts_mine - h->region), E * 4};
    CERA_TRY(launch_tp_exchange(h->ep, &cr, 1, 0, st));
    const uint32_t cap = (uint32_t)(rmax + E), max_small = E / h->ep_size;
    uint32_t *skip = h->ep_words + 33;
    moe_ep_plan_kernel<<<1, 32, 0, st>>>(h->ep, h->lay, E, nc, mma ? nc / 2 : 0, cap, (uint32_t)rmax, h->my_base, h->cursor, h->tiles,
                                         h->n_tiles, n_recv, skip);
    if (n)
        moe_ep_dispatch_kernel<<<(unsigned)entries, 128, 0, st>>>(h->ep, h->lay, h->ids, ku, hs, E, ActView{h->xs, h->xq, h->xsum},
                                                                   h->my_base, h->cursor, skip);
    count_launch(2);
    CERA_CUDA_TRY(cudaGetLastError());
    CERA_TRY(launch_tp_exchange(h->ep, nullptr, 0, 1, st));  // every rank's entries have landed
    char *rg = h->region;
    MoeGemmParams p{};
    p.w[0] = h->gate->v;
    p.w[1] = h->up->v;
    p.y[0] = h->g;
    p.y[1] = h->u;
    p.n_segs = 2;
    p.m = ff;
    p.k = hs;
    p.x = ActView{(const float *)(rg + h->lay.r_scales), (const int8_t *)(rg + h->lay.r_quants), (const int16_t *)(rg + h->lay.r_sums)};
    p.ldc = ff;
    p.tiles = h->tiles;
    p.n_tiles = h->n_tiles;
    CERA_TRY(grouped_projection(mma, p, max_tiles, cap, max_small, false, st));
    const size_t worst = rmax * ff;
    moe_silu_q8_kernel<<<(unsigned)((worst + 255) / 256), 256, 0, st>>>(h->g, h->u, ff, n_recv, h->f_scales, h->f_quants, h->f_sums);
    count_launch();
    MoeGemmParams d{};
    d.w[0] = h->down->v;
    d.y[0] = h->expert_out;
    d.n_segs = 1;
    d.m = hs;
    d.k = ff;
    d.x = ActView{h->f_scales, h->f_quants, h->f_sums};
    d.ldc = hs;
    d.tiles = h->tiles;
    d.n_tiles = h->n_tiles;
    CERA_TRY(grouped_projection(mma, d, max_tiles, cap, max_small, false, st));
    moe_ep_return_kernel<<<(unsigned)rmax, 128, 0, st>>>(h->ep, h->lay, h->expert_out, hs, n_recv);
    count_launch();
    CERA_CUDA_TRY(cudaGetLastError());
    CERA_TRY(launch_tp_exchange(h->ep, nullptr, 0, 2, st));  // every result row has come back
    if (n) {
        const size_t total = n * hs;
        moe_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const float *)(rg + h->lay.ret_out), nullptr, h->weights, ku, hs, n,
                                                                            out_dev);
        count_launch();
        CERA_CUDA_TRY(cudaGetLastError());
        if (ids_out_dev) CERA_CUDA_TRY(cudaMemcpyAsync(ids_out_dev, h->ids, entries * 4, cudaMemcpyDeviceToDevice, st));
        if (weights_out_dev) CERA_CUDA_TRY(cudaMemcpyAsync(weights_out_dev, h->weights, entries * 4, cudaMemcpyDeviceToDevice, st));
    }
    return CERA_CUDA_OK;
}

}  // namespace

extern "C" {

int32_t cera_cuda_moe_create(uint32_t n_expert, uint32_t n_used, uint32_t hidden, uint32_t ff, int32_t ggml_type,
                             const void *gate_exps, const void *up_exps, const void *down_exps, size_t gate_up_bytes,
                             size_t down_bytes, const float *router, const float *exp_probs_b, size_t max_tokens,
                             cera_cuda_moe **out) {
    return moe_create_impl(n_expert, n_used, hidden, ff, ggml_type, gate_exps, up_exps, down_exps, gate_up_bytes, down_bytes, router,
                           exp_probs_b, max_tokens, 0, 1, max_tokens, out);
}

int32_t cera_cuda_moe_create_ep(uint32_t n_expert, uint32_t n_used, uint32_t hidden, uint32_t ff, int32_t ggml_type,
                                const void *gate_exps, const void *up_exps, const void *down_exps, size_t gate_up_bytes,
                                size_t down_bytes, const float *router, const float *exp_probs_b, size_t max_tokens,
                                uint32_t ep_rank, uint32_t ep_size, size_t max_total_tokens, cera_cuda_moe **out) {
    return moe_create_impl(n_expert, n_used, hidden, ff, ggml_type, gate_exps, up_exps, down_exps, gate_up_bytes, down_bytes, router,
                           exp_probs_b, max_tokens, ep_rank, ep_size, max_total_tokens, out);
}

int32_t cera_cuda_moe_ep_handle(cera_cuda_moe *h, void *handle_out, size_t handle_bytes) {
    if (!h || !handle_out) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ep_handle: null argument");
    if (handle_bytes != sizeof(cudaIpcMemHandle_t)) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ep_handle: handle is %zu bytes", sizeof(cudaIpcMemHandle_t));
    if (h->ep_size < 2) return fail(CERA_CUDA_ERR_STATE, "moe_ep_handle: layer is not expert-parallel");
    cudaIpcMemHandle_t ih;
    CERA_CUDA_TRY(cudaIpcGetMemHandle(&ih, h->region));
    memcpy(handle_out, &ih, sizeof(ih));
    return CERA_CUDA_OK;
}

int32_t cera_cuda_moe_ep_connect(cera_cuda_moe *h, const void *handles, size_t n_handles) {
    if (!h || !handles) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ep_connect: null argument");
    if (n_handles != h->ep_size || h->ep_size < 2) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ep_connect: %zu handles for %u ranks", n_handles, h->ep_size);
    if (h->connected) return fail(CERA_CUDA_ERR_STATE, "moe_ep_connect: already connected");
    for (uint32_t p = 0; p < h->ep_size; ++p) {
        if (p == h->ep_rank) continue;
        cudaIpcMemHandle_t ih;
        memcpy(&ih, (const char *)handles + (size_t)p * sizeof(ih), sizeof(ih));
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, ih, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(CERA_CUDA_ERR_PEER, "moe_ep_connect: rank %u's receive region cannot be mapped: %s", p, cudaGetErrorString(e));
        }
        h->opened[p] = ptr;
        h->ep.peer[p] = (char *)ptr;
    }
    h->connected = true;
    return CERA_CUDA_OK;
}

int32_t cera_cuda_moe_ep_status(cera_cuda_moe *h, uint32_t *status_out) {
    if (!h || !status_out) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ep_status: null argument");
    *status_out = 0;
    if (h->ep_size < 2) return CERA_CUDA_OK;
    CERA_CUDA_TRY(cudaMemcpy(status_out, h->ep_words + 16, 4, cudaMemcpyDeviceToHost));
    if (*status_out & EP_STATUS_OVERFLOW && !(*status_out & 0x80000000u))
        return fail(CERA_CUDA_ERR_BAD_ARG,
                    "moe expert-parallel call: the ranks' tokens route more entries to rank %u than its receive buffer holds "
                    "(the layer was created for %zu tokens in total); nothing was exchanged and the output is undefined",
                    (*status_out >> 24) & 0x3Fu, h->max_total);
    if (*status_out)
        return fail(CERA_CUDA_ERR_TIMEOUT, "moe expert-parallel exchange %u: rank %u waited for rank %u too long", (*status_out & 0xFFFFFFu) - 1,
                    h->ep_rank, (*status_out >> 24) & 0x7Fu);
    return CERA_CUDA_OK;
}

int32_t cera_cuda_moe_ffn(cera_cuda_moe *h, const float *x_dev, size_t n, int32_t softmax_gate, float *out_dev,
                          uint32_t *ids_out_dev, float *weights_out_dev, void *stream) {
    if (!h || (n && (!x_dev || !out_dev))) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ffn: null argument");
    if (n > h->max_tokens) return fail(CERA_CUDA_ERR_BAD_ARG, "moe_ffn: %zu tokens, created for at most %zu", n, h->max_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    if (h->ep_size > 1) return moe_ffn_ep(h, x_dev, n, softmax_gate, out_dev, ids_out_dev, weights_out_dev, st);  // n == 0 still takes part
    if (n == 0) return CERA_CUDA_OK;
    const uint32_t hs = h->hidden, ff = h->ff, ku = h->n_used;
    const size_t entries = n * ku;
    const bool single = n == 1;
    // a handful of tokens: dp4a work items of 8 columns (1 for a single token); a batch: tensor-core items of 64
    const bool mma = n >= 16 && gemm_mma_supports(h->gate->v.type, hs) && gemm_mma_supports(h->down->v.type, ff) && !moe_force_dp4a();
    const uint32_t nc = single ? 1 : mma ? MOE_NC_MMA : MOE_NC;
    const uint32_t max_tiles = (uint32_t)(entries / nc + (single ? 0 : h->n_expert));
    CERA_TRY(launch_quantize(x_dev, hs, n, false, h->xs, h->xq, h->xsum, st));
    moe_route_kernel<<<(unsigned)n, 256, 0, st>>>(x_dev, h->router, h->bias, hs, h->n_expert, ku, softmax_gate, h->ids, h->weights,
                                                  h->counts);
    const uint32_t cap = (uint32_t)(h->max_total * ku + h->n_expert), max_small = h->n_expert;
    moe_plan_kernel<<<1, 32, 0, st>>>(h->counts, h->n_expert, nc, mma ? nc / 2 : 0, cap, h->cursor, h->tiles, h->n_tiles);
    moe_scatter_kernel<<<(unsigned)entries, 128, 0, st>>>(h->ids, ku, hs, ActView{h->xs, h->xq, h->xsum}, h->cursor, h->entry_of,
                                                          h->g_scales, h->g_quants, h->g_sums);
    count_launch(3);
    CERA_CUDA_TRY(cudaGetLastError());
    MoeGemmParams p{};
    p.w[0] = h->gate->v;
    p.w[1] = h->up->v;
    p.y[0] = h->g;
    p.y[1] = h->u;
    p.n_segs = 2;
    p.m = ff;
    p.k = hs;
    p.x = ActView{h->g_scales, h->g_quants, h->g_sums};
    p.ldc = ff;
    p.tiles = h->tiles;
    p.n_tiles = h->n_tiles;
    CERA_TRY(grouped_projection(mma, p, max_tiles, cap, max_small, single, st));
    CERA_TRY(launch_silu_mul(h->g, h->u, ff, entries, h->f_scales, h->f_quants, h->f_sums, st));
    MoeGemmParams d{};
    d.w[0] = h->down->v;
    d.y[0] = h->expert_out;
    d.n_segs = 1;
    d.m = hs;
    d.k = ff;
    d.x = ActView{h->f_scales, h->f_quants, h->f_sums};
    d.ldc = hs;
    d.tiles = h->tiles;
    d.n_tiles = h->n_tiles;
    CERA_TRY(grouped_projection(mma, d, max_tiles, cap, max_small, single, st));
    const size_t total = n * hs;
    moe_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(h->expert_out, h->entry_of, h->weights, ku, hs, n, out_dev);
    count_launch();
    CERA_CUDA_TRY(cudaGetLastError());
    if (ids_out_dev) CERA_CUDA_TRY(cudaMemcpyAsync(ids_out_dev, h->ids, entries * 4, cudaMemcpyDeviceToDevice, st));
    if (weights_out_dev) CERA_CUDA_TRY(cudaMemcpyAsync(weights_out_dev, h->weights, entries * 4, cudaMemcpyDeviceToDevice, st));
    return CERA_CUDA_OK;
}

size_t cera_cuda_moe_memory_bytes(const cera_cuda_moe *h) {
    if (!h) return 0;
    return h->bytes + (h->gate ? h->gate->bytes : 0) + (h->up ? h->up->bytes : 0) + (h->down ? h->down->bytes : 0);
}

void cera_cuda_moe_free(cera_cuda_moe *h) {
    if (!h) return;
    if (h->gate) cera_cuda_weight_free(h->gate);
    if (h->up) cera_cuda_weight_free(h->up);
    if (h->down) cera_cuda_weight_free(h->down);
    if (h->base) cudaFree(h->base);
    for (void *p : h->opened)
        if (p) cudaIpcCloseMemHandle(p);
    if (h->region) cudaFree(h->region);
    delete h;
}

}  // extern "C"
