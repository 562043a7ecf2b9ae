// Dense llama-architecture model on one B200: the object a `--device cuda`
// backend hands to cera's Session as its `Box<dyn Model>`.
//
// Weights, KV cache, scratch and the sequence-length counter live on the
// device side of the boundary (cera's wgpu / Metal models do the same:
// cera/src/model/mod.rs:184-199); every entry point takes one internal mutex.
// A decode token is one CUDA-graph launch: embedding row -> per layer
// [RMSNorm+Q8_0 -> q/k/v GEMV -> RoPE + KV append -> split-KV attention (+Q8_0)
// -> o-proj GEMV (+residual) -> RMSNorm+Q8_0 -> gate/up GEMV -> SiLU*mul+Q8_0 ->
// down GEMV (+residual)] -> final RMSNorm+Q8_0 -> LM-head GEMV [-> argmax].
// The token id and position are read from device memory so the graph is
// recorded once per attention split count and replayed.
// Layer wiring: cera/src/model/llama.rs:468-597, 1585-1605 and
// cera/src/model/transformer.rs:1313-1652.
//
// Tensor-parallel mode (cera_cuda_model_set_tp, one process per GPU): every matrix is split by
// output rows, rank r keeping rows [r*m/G, (r+1)*m/G) of the tensor it is handed in full; q/k/v
// rows are whole heads, so the KV cache and attention of a head live on one rank.  The vectors
// every rank needs in full (Q8_0 attention output, residual stream, Q8_0 SwiGLU activations,
// logits) sit in an exchange region whose slices the ranks push to each other (tp.cu) after the
// kernel that produced them: four exchanges per layer plus one for the logits or the greedy pick.
// RMSNorm, the embedding row and the RoPE table are recomputed on every rank.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <initializer_list>
#include <mutex>
#include <new>
#include <vector>

#include "ops.h"
#include "weight.h"

using namespace cera;

namespace {

struct ActBuf {
    float *scales = nullptr;
    int8_t *quants = nullptr;
    int16_t *sums = nullptr;
    ActView view() const { return ActView{scales, quants, sums}; }
};

// One LoRA pair of a projection (device copies of A [rank x k] and B [d x rank]).
struct Lora {
    float *a = nullptr, *b = nullptr;
    uint32_t rank = 0, k = 0, d = 0;
    float scale = 0.0f;
};

struct Layer {
    Lora lora[7];  // q, k, v, o, gate, up, down (the order of cera/src/lora.rs:63-70)
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    cera_cuda_weight *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *gate = nullptr, *up = nullptr,
                     *down = nullptr;
    void *kc = nullptr, *vc = nullptr;
};

constexpr size_t PREFILL_CHUNK = 512;

enum GraphKind { G_BODY = 0, G_LOGITS = 1, G_GREEDY = 2, G_CHAIN = 3 };

}  // namespace

struct cera_cuda_model {
    cera_cuda_config cfg{};
    std::mutex mu;
    bool finalized = false;
    bool tc_prepared = false;  // the prefill GEMM's weight images have been asked for
    cera_cuda_weight *embd = nullptr, *output = nullptr;
    cera_cuda_weight *embd_rows = nullptr;  // tensor parallel: this rank's rows of a tied embedding, as LM head
    cera_cuda_weight *embd_head = nullptr;  // LM head when output.weight is absent (embd or embd_rows)
    float *out_norm = nullptr, *rope_freqs = nullptr;
    std::vector<Layer> layers;
    std::vector<void *> owned;  // plain device allocations to free
    size_t mem_bytes = 0;
    // scratch
    float *hidden = nullptr, *final_hidden = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr,
          *g = nullptr, *u = nullptr, *logits = nullptr;
    ActBuf act_hs, act_q, act_ff;
    void *attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    uint32_t *argmax_scratch = nullptr;
    uint32_t *dyn = nullptr;      // device: [0]=token [1]=pos [2]=seq_len(pos+1)
    uint32_t *tok_out = nullptr;  // device
    uint32_t *h_dyn = nullptr;    // pinned host mirror of dyn + returned token
    float *h_logits = nullptr;    // pinned host staging for logits
    float theta_scale = 0.0f;
    float *rope_cs = nullptr;  // [head_dim/2][2] cos/sin at the current position
    float *rope_table = nullptr;  // [max_seq_len][head_dim/2][2] cos/sin of every position, computed on the host (null: too large)
    cudaStream_t stream = nullptr;
    std::map<uint32_t, cudaGraphExec_t> graphs;  // key = kind | n_splits << 8
    size_t seq_len = 0;
    uint64_t launches = 0;         // kernels launched by decode steps
    uint32_t nodes_per_step[4] = {0, 0, 0, 0};
    // batched prefill (chunks of PREFILL_CHUNK tokens, token-major buffers)
    uint32_t *pf_tokens = nullptr;
    float *pf_hidden = nullptr, *pf_q = nullptr, *pf_k = nullptr, *pf_v = nullptr, *pf_attn = nullptr, *pf_g = nullptr,
          *pf_u = nullptr;
    float *pf_attn_local = nullptr;  // = pf_attn (every rank computes all heads)
    ActBuf pf_act_hs, pf_act_q, pf_act_ff;
    float *pf_logits = nullptr;  // [PREFILL_CHUNK][vocab], allocated by the first logits-for-every-position call
    bool has_lora = false;
    float *normed = nullptr;       // f32 copy of the normed hidden state, written only while adapters are attached
    uint32_t *tok_hist = nullptr;  // device ring of generated tokens (chained greedy decode)
    uint32_t tok_hist_cap = 0;
    // tensor parallelism (tp_size == 1: a single device, no exchange)
    uint32_t tp_rank = 0, tp_size = 1;
    bool tp_connected = false;
    char *region = nullptr;  // exchange region: hidden, act_q, act_ff, logits, pairs, flags
    size_t region_bytes = 0;
    TpCtx tp{};
    void *tp_opened[TP_MAX_RANKS] = {};  // peer mappings to close
    uint32_t *tp_words = nullptr;        // device: [0] = step sequence, [16] = status, [32] = local greedy pick
    uint32_t tp_slots = 0;
    uint32_t *h_status = nullptr;  // pinned
    // per-rank extents
    uint32_t l_heads = 0, l_kv_heads = 0;
    size_t l_qd = 0, l_kvd = 0, l_ff = 0, l_hs = 0, l_vocab = 0;
};

namespace {

int32_t dev_alloc(cera_cuda_model *m, void **p, size_t bytes) {
    CERA_CUDA_TRY(cudaMalloc(p, bytes));
    m->owned.push_back(*p);
    m->mem_bytes += bytes;
    return CERA_CUDA_OK;
}

int32_t alloc_act(cera_cuda_model *m, ActBuf &a, size_t k) {
    CERA_TRY(dev_alloc(m, (void **)&a.scales, k / 32 * 4));
    CERA_TRY(dev_alloc(m, (void **)&a.quants, k));
    CERA_TRY(dev_alloc(m, (void **)&a.sums, k / 16 * 2));
    return CERA_CUDA_OK;
}

// After the argmax of a chained step: record the token, make it the next input, advance
// the position.  dyn = {token, pos, seq_len, step}.
__global__ void advance_kernel(uint32_t *dyn, const uint32_t *tok_out, uint32_t *hist, uint32_t cap) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = *tok_out, step = dyn[3];
    if (step < cap) hist[step] = t;
    dyn[0] = t;
    dyn[1] += 1;
    dyn[2] += 1;
    dyn[3] = step + 1;
}

// Enqueue one decode step on m->stream; token / position come from m->dyn.
int32_t enqueue_step(cera_cuda_model *m, int kind, uint32_t n_splits) {
    const auto &c = m->cfg;
    cudaStream_t st = m->stream;
    const size_t hs = c.hidden_size;
    const uint32_t r = m->tp_rank;
    const bool tp = m->tp_size > 1;
    const float scale = c.attention_scale != 0.0f ? c.attention_scale : 1.0f / sqrtf((float)c.head_dim);
    const float res_scale = c.residual_scale != 0.0f ? c.residual_scale : 1.0f;  // Granite: block outputs are scaled before the residual add
    // Exchange slots of layer l: 4l, 4l+1 = (unused), 4l+2 = Q8_0 SwiGLU
    // activations, 4l+3 = residual after down-proj; then 4L = logits, 4L+1 = greedy pairs.  The producing kernel
    // mirrors its stores into the peers' regions; the consuming kernel signals and waits in its prologue.
    const uint32_t n_layers = (uint32_t)m->layers.size();
    auto hook = [&](uint32_t wait_slot, bool push) {
        TpHook h;
        if (tp) {
            h.ctx = m->tp;
            h.wait_slot = wait_slot;
            h.push = push ? 1 : 0;
        }
        return h;
    };
    // this rank's part of a Q8_0 activation buffer that holds `l` of its elements per rank
    auto act_slice = [&](const ActBuf &a, size_t l) {
        return ActBuf{a.scales + r * (l / 32), a.quants + r * l, a.sums + r * (l / 16)};
    };
    float *hidden_slice = m->hidden + r * m->l_hs;

    if (tp) CERA_TRY(launch_tp_tick(m->tp_words, st));
    CERA_TRY(launch_embed(m->embd->v, 0, m->dyn, m->hidden, st));
    if (c.embedding_scale != 0.0f && c.embedding_scale != 1.0f) CERA_TRY(launch_scale(m->hidden, hs, c.embedding_scale, st));
    const bool norm_rope = c.rope_type == 0;
    // CERA_CUDA_FUSE_NORM=1: RMSNorm runs as the prologue of the GEMV that consumes it (reference-order kernels, one GPU,
    // no LoRA reading the normalised vector).  Off by default: it saves 65 launches per token but puts the norm on the
    // critical path of every CTA of the GEMV, and measured 4 % slower per token than the stand-alone kernel.
    static const bool fuse_norm_env = [] { const char *e = getenv("CERA_CUDA_FUSE_NORM"); return e && e[0] == '1'; }();
    const bool fuse_norm = fuse_norm_env && !tp && !m->has_lora && hs % 1024 == 0;
    if (norm_rope) CERA_TRY(launch_rope_table(m->dyn + 1, c.head_dim, m->theta_scale, m->rope_freqs, m->rope_cs, st, m->rope_table));
    for (uint32_t li = 0; li < n_layers; ++li) {
        Layer &L = m->layers[li];
        const uint32_t s0 = 4 * li;
        // (slots s0 and s0 + 1 are unused: every rank holds the whole attention block, so neither the attention output
        // nor the residual after the o-proj needs an exchange)
        const TpHook h_norm1 = hook(li ? s0 - 1 : TP_NO_SLOT, false), h_merge = hook(TP_NO_SLOT, false), h_wo = hook(TP_NO_SLOT, false),
                     h_norm2 = hook(TP_NO_SLOT, false), h_silu = hook(TP_NO_SLOT, true), h_down = hook(s0 + 2, true);
        // LoRA deltas read the f32 input of the projection they adapt (cera/src/model/transformer.rs:1383-1387,
        // 1519-1528, 1588-1605, 1642-1651): the normed hidden, the attention output, the SwiGLU product
        float *normed_f32 = m->has_lora ? m->normed : nullptr;
        auto lora = [&](int target, const float *x, float *y) -> int32_t {
            const Lora &t = L.lora[target];
            if (!t.rank || t.scale == 0.0f) return CERA_CUDA_OK;
            return launch_lora(x, t.a, t.b, t.rank, t.k, t.d, t.scale, y, st);
        };
        const bool lora_qkv = L.lora[0].rank || L.lora[1].rank || L.lora[2].rank;
        bool fused_qkv = false;
        bool normed = false;  // act_hs holds the normalised, quantized hidden state
        auto norm1 = [&]() -> int32_t {
            if (normed) return CERA_CUDA_OK;
            normed = true;
            return launch_rmsnorm(m->hidden, L.attn_norm, hs, 1, c.rms_norm_eps, normed_f32, m->act_hs.scales, m->act_hs.quants,
                                  m->act_hs.sums, st, &h_norm1);
        };
        if (!lora_qkv && norm_rope && L.wq->v.type == L.wk->v.type && L.wq->v.type == L.wv->v.type) {
            // q/k/v GEMV with RoPE and the KV-cache append as its epilogue
            GemvSeg segs[3] = {{L.wq->v, m->q}, {L.wk->v, m->k}, {L.wv->v, m->v}};
            GemvFusion f;
            f.rope_cs = m->rope_cs;
            f.pos_dev = m->dyn + 1;
            f.k_cache = L.kc;
            f.v_cache = L.vc;
            f.kv_f16 = c.kv_f16;
            f.head_dim = c.head_dim;
            f.kv_dim = (uint32_t)m->l_kvd;
            if (fuse_norm) {  // RMSNorm as the GEMV's prologue
                f.norm_x = m->hidden;
                f.norm_w = L.attn_norm;
                f.norm_eps = c.rms_norm_eps;
                CERA_TRY(launch_gemv_exact(segs, 3, m->act_hs.view(), EPI_ROPE_KV, &f, st, &fused_qkv));
                f.norm_x = nullptr;
            }
            if (!fused_qkv) {
                CERA_TRY(norm1());
                CERA_TRY(launch_gemv_exact(segs, 3, m->act_hs.view(), EPI_ROPE_KV, &f, st, &fused_qkv));
            }
            if (!fused_qkv) CERA_TRY(launch_gemv_fused(segs, 3, m->act_hs.view(), EPI_ROPE_KV, &f, st, &fused_qkv));
        }
        if (!fused_qkv) CERA_TRY(norm1());
        if (fused_qkv) {
        } else if (L.wq->v.type == L.wk->v.type && L.wq->v.type == L.wv->v.type) {
            GemvSeg segs[3] = {{L.wq->v, m->q}, {L.wk->v, m->k}, {L.wv->v, m->v}};
            CERA_TRY(launch_gemv(segs, 3, m->act_hs.view(), 1, 1, EPI_STORE, st));
        } else {
            GemvSeg sq{L.wq->v, m->q}, sk{L.wk->v, m->k}, sv{L.wv->v, m->v};
            CERA_TRY(launch_gemv(&sq, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
            CERA_TRY(launch_gemv(&sk, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
            CERA_TRY(launch_gemv(&sv, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
        }
        if (lora_qkv) {  // the deltas go in before RoPE, like the base projections
            CERA_TRY(lora(0, m->normed, m->q));
            CERA_TRY(lora(1, m->normed, m->k));
            CERA_TRY(lora(2, m->normed, m->v));
        }
        if (!fused_qkv)
            CERA_TRY(launch_rope(m->q, m->k, m->v, 0, m->dyn + 1, m->l_heads, m->l_kv_heads, c.head_dim, m->theta_scale,
                                 m->rope_freqs, c.rope_type, L.kc, L.vc, c.kv_f16, st, m->rope_table));
        const ActBuf aq = m->act_q;  // all heads on every rank
        CERA_TRY(launch_decode_attention_ex(m->q, L.kc, L.vc, c.kv_f16, m->l_heads, m->l_kv_heads, c.head_dim, 0,
                                            m->dyn + 2, n_splits, scale, m->attn, m->attn_ws, m->attn_ws_bytes,
                                            aq.scales, aq.quants, aq.sums, st, &h_merge));
        if (res_scale != 1.0f) {  // the block output on its own (g is free here), its LoRA delta, then hidden += out * s
            GemvSeg so{L.wo->v, m->g};
            CERA_TRY(launch_gemv(&so, 1, m->act_q.view(), 1, 1, EPI_STORE, st));
            CERA_TRY(lora(3, m->attn, m->g));
            CERA_TRY(launch_scaled_add(m->hidden, m->g, hs, res_scale, st));
        } else {
            GemvSeg so{L.wo->v, m->hidden};  // all rows on every rank
            CERA_TRY(launch_gemv(&so, 1, m->act_q.view(), 1, 1, EPI_ADD, st, 1, false, &h_wo));
            CERA_TRY(lora(3, m->attn, m->hidden));  // o-proj output lives in the residual stream already
        }
        bool fused_ffn = false;
        if (fuse_norm && L.gate->v.type == L.up->v.type) {
            GemvSeg segs[2] = {{L.gate->v, m->g}, {L.up->v, m->u}};
            GemvFusion f;
            f.norm_x = m->hidden;
            f.norm_w = L.ffn_norm;
            f.norm_eps = c.rms_norm_eps;
            CERA_TRY(launch_gemv_exact(segs, 2, m->act_hs.view(), EPI_STORE, &f, st, &fused_ffn));
        }
        if (!fused_ffn)
            CERA_TRY(launch_rmsnorm(m->hidden, L.ffn_norm, hs, 1, c.rms_norm_eps, normed_f32, m->act_hs.scales,
                                    m->act_hs.quants, m->act_hs.sums, st, &h_norm2));
        if (fused_ffn) {
        } else if (L.gate->v.type == L.up->v.type) {
            GemvSeg segs[2] = {{L.gate->v, m->g}, {L.up->v, m->u}};
            CERA_TRY(launch_gemv(segs, 2, m->act_hs.view(), 1, 1, EPI_STORE, st));
        } else {
            GemvSeg sg{L.gate->v, m->g}, su{L.up->v, m->u};
            CERA_TRY(launch_gemv(&sg, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
            CERA_TRY(launch_gemv(&su, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
        }
        CERA_TRY(lora(4, m->normed, m->g));
        CERA_TRY(lora(5, m->normed, m->u));
        const ActBuf af = act_slice(m->act_ff, m->l_ff);
        CERA_TRY(launch_silu_mul(m->g, m->u, m->l_ff, 1, af.scales, af.quants, af.sums, st, &h_silu));
        if (res_scale != 1.0f) {  // u is free once the SwiGLU product is in g
            GemvSeg sd{L.down->v, m->u};
            CERA_TRY(launch_gemv(&sd, 1, m->act_ff.view(), 1, 1, EPI_STORE, st));
            CERA_TRY(lora(6, m->g, m->u));
            CERA_TRY(launch_scaled_add(m->hidden, m->u, hs, res_scale, st));
        } else {
            GemvSeg sd{L.down->v, hidden_slice};
            CERA_TRY(launch_gemv(&sd, 1, m->act_ff.view(), 1, 1, EPI_ADD, st, 1, false, &h_down));
            CERA_TRY(lora(6, m->g, m->hidden));  // input: the SwiGLU product, left in g by the kernel above
        }
    }
    const uint32_t s_last = 4 * n_layers - 1, s_logits = 4 * n_layers, s_pick = 4 * n_layers + 1;
    if (kind == G_BODY) {
        // nothing in this graph consumes the last residual exchange; the next step's embedding row overwrites the
        // buffer the peers are still writing, so wait for their slices here
        if (tp) CERA_TRY(launch_tp_exchange(m->tp, nullptr, 0, s_last, st));
        return CERA_CUDA_OK;
    }
    const TpHook h_final = hook(s_last, false);
    const cera_cuda_weight *ow = m->output ? m->output : m->embd_head;
    float *logits_slice = m->logits + r * m->l_vocab;
    GemvSeg sl{ow->v, logits_slice};
    bool fused_head = false;
    if (fuse_norm) {
        GemvFusion f;
        f.norm_x = m->hidden;
        f.norm_w = m->out_norm;
        f.norm_eps = c.rms_norm_eps;
        f.norm_out = m->final_hidden;
        CERA_TRY(launch_gemv_exact(&sl, 1, m->act_hs.view(), EPI_STORE, &f, st, &fused_head));
    }
    if (!fused_head) {
        CERA_TRY(launch_rmsnorm(m->hidden, m->out_norm, hs, 1, c.rms_norm_eps, m->final_hidden, m->act_hs.scales,
                                m->act_hs.quants, m->act_hs.sums, st, &h_final));
        CERA_TRY(launch_gemv(&sl, 1, m->act_hs.view(), 1, 1, EPI_STORE, st));
    }
    if (c.logit_scale != 0.0f && c.logit_scale != 1.0f) CERA_TRY(launch_scale(logits_slice, m->l_vocab, 1.0f / c.logit_scale, st));
    if (kind == G_LOGITS && tp) {
        const TpRange rg{(uint32_t)((const char *)logits_slice - m->region), (uint32_t)(m->l_vocab * 4)};
        CERA_TRY(launch_tp_exchange(m->tp, &rg, 1, s_logits, st));
    }
    if (kind == G_GREEDY || kind == G_CHAIN) {
        if (!tp) {
            CERA_TRY(launch_argmax(m->logits, c.vocab_size, m->tok_out, m->argmax_scratch, st));
        } else {
            CERA_TRY(launch_argmax(logits_slice, m->l_vocab, m->tp_words + 32, m->argmax_scratch, st));
            CERA_TRY(launch_tp_argmax(m->tp, logits_slice, (uint32_t)m->l_vocab, m->tp_words + 32, m->tok_out, s_pick, st));
        }
    }
    if (kind == G_CHAIN) {
        count_launch();
        CERA_CUDA_TRY(launch_k(advance_kernel, dim3(1), dim3(1), 0, st, m->dyn, (const uint32_t *)m->tok_out, m->tok_hist,
                               m->tok_hist_cap));
    }
    return CERA_CUDA_OK;
}

int32_t get_graph(cera_cuda_model *m, int kind, uint32_t n_splits, cudaGraphExec_t *out) {
    const uint32_t key = (uint32_t)kind | (n_splits << 8);
    auto it = m->graphs.find(key);
    if (it != m->graphs.end()) {
        *out = it->second;
        return CERA_CUDA_OK;
    }
    const uint64_t before = launches_so_far();
    CERA_CUDA_TRY(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    int32_t st = enqueue_step(m, kind, n_splits);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->stream, &graph);
    if (st != CERA_CUDA_OK) {
        if (graph) cudaGraphDestroy(graph);
        return st;
    }
    CERA_CUDA_TRY(e);
    m->nodes_per_step[kind] = (uint32_t)(launches_so_far() - before);
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    CERA_CUDA_TRY(e);
    m->graphs[key] = exec;
    *out = exec;
    return CERA_CUDA_OK;
}

// Runs one token; leaves results in device buffers (logits / tok_out).
int32_t run_token(cera_cuda_model *m, uint32_t token, size_t pos, int kind) {
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "forward: model_finalize has not been called");
    if (token >= c.vocab_size) return fail(CERA_CUDA_ERR_BAD_ARG, "forward: token %u out of range (vocab %u)", token, c.vocab_size);
    if (pos != m->seq_len) return fail(CERA_CUDA_ERR_STATE, "forward: pos %zu != seq_len %zu", pos, m->seq_len);
    if (pos >= c.max_seq_len) return fail(CERA_CUDA_ERR_BAD_ARG, "forward: pos %zu exceeds max_seq_len %u", pos, c.max_seq_len);
    if (m->tp_size > 1 && !m->tp_connected) return fail(CERA_CUDA_ERR_STATE, "forward: tensor-parallel model is not connected to its peers");
    const uint32_t n_splits = attn_plan(m->l_heads, m->l_kv_heads, m->cfg.head_dim, pos + 1);
    cudaGraphExec_t g = nullptr;
    CERA_TRY(get_graph(m, kind, n_splits, &g));
    m->h_dyn[0] = token;
    m->h_dyn[1] = (uint32_t)pos;
    m->h_dyn[2] = (uint32_t)pos + 1;
    CERA_CUDA_TRY(cudaMemcpyAsync(m->dyn, m->h_dyn, 3 * sizeof(uint32_t), cudaMemcpyHostToDevice, m->stream));
    CERA_CUDA_TRY(cudaGraphLaunch(g, m->stream));
    m->launches += m->nodes_per_step[kind];
    m->seq_len = pos + 1;
    return CERA_CUDA_OK;
}

// One chunk (n <= PREFILL_CHUNK) of prompt tokens through every layer with batched kernels: column
// RMSNorm + Q8_0, multi-column GEMMs (token-major outputs), batched RoPE + KV append, causal attention,
// SiLU*mul + Q8_0 (cera/src/model/llama.rs:738-1523).  Leaves the hidden state of the chunk's last token
// in m->hidden so the ordinary LM-head path can finish.
int32_t prefill_chunk(cera_cuda_model *m, const uint32_t *tokens, size_t n, size_t start_pos) {
    const auto &c = m->cfg;
    cudaStream_t st = m->stream;
    const size_t hs = c.hidden_size, qd = (size_t)c.n_heads * c.head_dim, kvd = (size_t)c.n_kv_heads * c.head_dim,
                 ff = c.intermediate_size;
    const float scale = c.attention_scale != 0.0f ? c.attention_scale : 1.0f / sqrtf((float)c.head_dim);
    const float res_scale = c.residual_scale != 0.0f ? c.residual_scale : 1.0f;
    if (n > 32 && !m->tc_prepared) {
        // the first batched prompt builds the f16 operand images of the tensor-core GEMM's weights (a decode-only model
        // never pays their 2.3 bytes per weight; a weight that gets none is converted on the fly)
        m->tc_prepared = true;
        for (auto &L : m->layers)
            for (cera_cuda_weight *w : {L.wq, L.wk, L.wv, L.wo, L.gate, L.up, L.down}) {
                bool built = false;
                CERA_TRY(weight_prepare_tc(w, &built));
                if (built) m->mem_bytes += w->tc_bytes;
            }
    }
    // Tensor parallel: every rank runs the whole attention block and its rows of gate / up and down (its slice of the
    // SwiGLU product and of the residual), and after each row-split product copies its column
    // slice of the chunk-wide buffer into every peer's copy (strided device-to-device copies into the peers' exchange
    // regions), then signals and waits on the layer's exchange slot as the decode step does (bounded waits, tp.cu).
    const bool tp = m->tp_size > 1;
    const uint32_t r = m->tp_rank;
    const size_t l_qd = m->l_qd, l_kvd = m->l_kvd, l_ff = m->l_ff, l_hs = m->l_hs;
    auto gather = [&](float *full, size_t cols, size_t l_cols, const float *src, size_t src_pitch_elems, uint32_t slot) -> int32_t {
        // column slice [r * l_cols, +l_cols) of the [n x cols] buffer `full`: into this rank's copy (when it was formed
        // elsewhere) and into every peer's
        const size_t col_off = (size_t)r * l_cols;
        if (src != full + col_off)
            CERA_CUDA_TRY(cudaMemcpy2DAsync(full + col_off, cols * 4, src, src_pitch_elems * 4, l_cols * 4, n, cudaMemcpyDeviceToDevice, st));
        const size_t off = (size_t)((char *)(full + col_off) - m->region);
        for (uint32_t p = 0; p < m->tp_size; ++p)
            if (p != r)
                CERA_CUDA_TRY(cudaMemcpy2DAsync(m->tp.peer[p] + off, cols * 4, src, src_pitch_elems * 4, l_cols * 4, n, cudaMemcpyDeviceToDevice, st));
        return launch_tp_exchange(m->tp, nullptr, 0, slot, st);
    };
    // projections that share their activations (q / k / v, gate / up): one tensor-core launch when every weight has its
    // operand image, else one GEMM each
    auto gemm_group = [&](std::initializer_list<GemmTarget> ts, const ActView &x) -> int32_t {
        bool taken = false;
        CERA_TRY(launch_gemm_tc_multi(ts.begin(), (int)ts.size(), x, n, 1, EPI_STORE, st, &taken));
        if (taken) return CERA_CUDA_OK;
        for (const GemmTarget &t : ts) CERA_TRY(launch_gemm_ex(t.w, x, n, t.out, 1, t.ldc, EPI_STORE, st));
        return CERA_CUDA_OK;
    };
    if (tp) CERA_TRY(launch_tp_tick(m->tp_words, st));
    CERA_CUDA_TRY(cudaMemcpyAsync(m->pf_tokens, tokens, n * 4, cudaMemcpyHostToDevice, st));
    CERA_TRY(launch_embed_batch(m->embd->v, m->pf_tokens, n, m->pf_hidden, st));
    if (c.embedding_scale != 0.0f && c.embedding_scale != 1.0f) CERA_TRY(launch_scale(m->pf_hidden, n * hs, c.embedding_scale, st));
    const uint64_t before = launches_so_far();
    uint32_t li = 0;
    for (auto &L : m->layers) {
        const uint32_t s0 = 4 * li++;
        CERA_TRY(launch_rmsnorm(m->pf_hidden, L.attn_norm, hs, n, c.rms_norm_eps, nullptr, m->pf_act_hs.scales,
                                m->pf_act_hs.quants, m->pf_act_hs.sums, st));
        CERA_TRY(gemm_group({{L.wq->v, m->pf_q, l_qd}, {L.wk->v, m->pf_k, l_kvd}, {L.wv->v, m->pf_v, l_kvd}}, m->pf_act_hs.view()));
        CERA_TRY(launch_rope_batch(m->pf_q, m->pf_k, m->pf_v, start_pos, n, m->l_heads, m->l_kv_heads, c.head_dim,
                                   m->theta_scale, m->rope_freqs, c.rope_type, L.kc, L.vc, c.kv_f16, st, m->rope_table));
        CERA_TRY(launch_prefill_attention(m->pf_q, L.kc, L.vc, c.kv_f16, m->l_heads, m->l_kv_heads, c.head_dim, n, start_pos,
                                          scale, m->pf_attn_local, st));
        CERA_TRY(launch_quantize(m->pf_attn, qd, n, false, m->pf_act_q.scales, m->pf_act_q.quants, m->pf_act_q.sums, st));
        if (res_scale != 1.0f) {  // block output into pf_g (free until the gate projection), then hidden += out * s
            CERA_TRY(launch_gemm_ex(L.wo->v, m->pf_act_q.view(), n, m->pf_g, 1, hs, EPI_STORE, st));
            CERA_TRY(launch_scaled_add(m->pf_hidden, m->pf_g, n * hs, res_scale, st));
        } else {
            CERA_TRY(launch_gemm_ex(L.wo->v, m->pf_act_q.view(), n, m->pf_hidden, 1, hs, EPI_ADD, st));  // whole on every rank
        }
        CERA_TRY(launch_rmsnorm(m->pf_hidden, L.ffn_norm, hs, n, c.rms_norm_eps, nullptr, m->pf_act_hs.scales,
                                m->pf_act_hs.quants, m->pf_act_hs.sums, st));
        CERA_TRY(gemm_group({{L.gate->v, m->pf_g + (size_t)r * l_ff, ff}, {L.up->v, m->pf_u + (size_t)r * l_ff, ff}}, m->pf_act_hs.view()));
        if (tp) {
            // (two copies, one signal: the second gather carries the slot)
            const size_t col_off = (size_t)r * l_ff, off = (size_t)((char *)(m->pf_g + col_off) - m->region);
            for (uint32_t p = 0; p < m->tp_size; ++p)
                if (p != r)
                    CERA_CUDA_TRY(cudaMemcpy2DAsync(m->tp.peer[p] + off, ff * 4, m->pf_g + col_off, ff * 4, l_ff * 4, n, cudaMemcpyDeviceToDevice, st));
            CERA_TRY(gather(m->pf_u, ff, l_ff, m->pf_u + col_off, ff, s0 + 2));
        }
        CERA_TRY(launch_silu_mul(m->pf_g, m->pf_u, ff, n, m->pf_act_ff.scales, m->pf_act_ff.quants, m->pf_act_ff.sums, st));
        if (res_scale != 1.0f) {  // pf_u is free once the SwiGLU product is quantized
            CERA_TRY(launch_gemm_ex(L.down->v, m->pf_act_ff.view(), n, m->pf_u, 1, hs, EPI_STORE, st));
            CERA_TRY(launch_scaled_add(m->pf_hidden, m->pf_u, n * hs, res_scale, st));
        } else {
            CERA_TRY(launch_gemm_ex(L.down->v, m->pf_act_ff.view(), n, m->pf_hidden + (size_t)r * l_hs, 1, hs, EPI_ADD, st));
            if (tp) CERA_TRY(gather(m->pf_hidden, hs, l_hs, m->pf_hidden + (size_t)r * l_hs, hs, s0 + 3));
        }
    }
    CERA_CUDA_TRY(cudaMemcpyAsync(m->hidden, m->pf_hidden + (n - 1) * hs, hs * 4, cudaMemcpyDeviceToDevice, st));
    m->launches += launches_so_far() - before + 1;
    return CERA_CUDA_OK;
}

// Final RMSNorm + LM head on m->hidden (eager launches on the model's stream).
int32_t logits_from_hidden(cera_cuda_model *m) {
    const auto &c = m->cfg;
    CERA_TRY(launch_rmsnorm(m->hidden, m->out_norm, c.hidden_size, 1, c.rms_norm_eps, m->final_hidden, m->act_hs.scales,
                            m->act_hs.quants, m->act_hs.sums, m->stream));
    const cera_cuda_weight *ow = m->output ? m->output : m->embd;
    GemvSeg sl{ow->v, m->logits};
    m->launches += 2;
    CERA_TRY(launch_gemv(&sl, 1, m->act_hs.view(), 1, 1, EPI_STORE, m->stream));
    if (c.logit_scale != 0.0f && c.logit_scale != 1.0f) {
        m->launches += 1;
        CERA_TRY(launch_scale(m->logits, c.vocab_size, 1.0f / c.logit_scale, m->stream));
    }
    return CERA_CUDA_OK;
}

void set_extents(cera_cuda_model *m) {
    const auto &c = m->cfg;
    const uint32_t G = m->tp_size;
    // the attention block (q / k / v, the KV cache, attention, o-proj) is whole on every rank: its launches are
    // latency-bound whole or split, and a rank that holds all heads needs no exchange around the attention - only the
    // feed-forward matrices (four fifths of a layer's bytes) and the LM head are split by rows
    m->l_heads = c.n_heads;
    m->l_kv_heads = c.n_kv_heads;
    m->l_qd = (size_t)m->l_heads * c.head_dim;
    m->l_kvd = (size_t)m->l_kv_heads * c.head_dim;
    m->l_ff = c.intermediate_size / G;
    m->l_hs = c.hidden_size / G;
    m->l_vocab = c.vocab_size / G;
}

// Reads the exchange status word after a synchronisation; a set word is a wait that ran out.
int32_t tp_check(cera_cuda_model *m) {
    if (m->tp_size < 2) return CERA_CUDA_OK;
    CERA_CUDA_TRY(cudaMemcpyAsync(m->h_status, m->tp_words + 16, 4, cudaMemcpyDeviceToHost, m->stream));
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    const uint32_t w = *m->h_status;
    if (w == 0) return CERA_CUDA_OK;
    return fail(CERA_CUDA_ERR_TIMEOUT, "tensor-parallel exchange %u: rank %u waited for rank %u longer than %llu ms", (w & 0xFFFFFFu) - 1,
                m->tp_rank, (w >> 24) & 0x7Fu, (unsigned long long)(m->tp.timeout_ns / 1000000ull));
}

struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        cudaSetDevice(dev);
    }
    ~DeviceGuard() { cudaSetDevice(prev); }
};

}  // namespace

extern "C" {

int32_t cera_cuda_model_create(const cera_cuda_config *cfg, cera_cuda_model **out) {
    if (!cfg || !out) return fail(CERA_CUDA_ERR_BAD_ARG, "model_create: null argument");
    const auto &c = *cfg;
    if (!c.n_layers || !c.hidden_size || !c.intermediate_size || !c.n_heads || !c.n_kv_heads || !c.head_dim ||
        !c.vocab_size || !c.max_seq_len)
        return fail(CERA_CUDA_ERR_BAD_ARG, "model_create: zero dimension in config");
    if (c.n_heads % c.n_kv_heads) return fail(CERA_CUDA_ERR_BAD_ARG, "model_create: n_heads %% n_kv_heads != 0");
    if (c.hidden_size % 32 || c.intermediate_size % 32 || (c.n_heads * c.head_dim) % 32)
        return fail(CERA_CUDA_ERR_BAD_ARG, "model_create: hidden, intermediate and q dims must be multiples of 32");
    int n_dev = 0;
    CERA_CUDA_TRY(cudaGetDeviceCount(&n_dev));
    if (c.device < 0 || c.device >= n_dev) return fail(CERA_CUDA_ERR_BAD_ARG, "model_create: device %d of %d", c.device, n_dev);
    auto *m = new (std::nothrow) cera_cuda_model();
    if (!m) return fail(CERA_CUDA_ERR_OOM, "model_create: host allocation failed");
    m->cfg = c;
    m->layers.resize(c.n_layers);
    m->theta_scale = powf(c.rope_theta, -2.0f / (float)c.head_dim);
    set_extents(m);
    *out = m;
    return CERA_CUDA_OK;
}

int32_t cera_cuda_model_set_tp(cera_cuda_model *m, uint32_t rank, uint32_t size) {
    if (!m) return fail(CERA_CUDA_ERR_BAD_ARG, "set_tp: null model");
    std::lock_guard<std::mutex> lock(m->mu);
    const auto &c = m->cfg;
    if (m->finalized || m->embd || m->out_norm || m->output)
        return fail(CERA_CUDA_ERR_STATE, "set_tp: must precede the first add_tensor");
    for (const auto &L : m->layers)
        if (L.wq || L.wk || L.wv || L.wo || L.gate || L.up || L.down || L.attn_norm || L.ffn_norm)
            return fail(CERA_CUDA_ERR_STATE, "set_tp: must precede the first add_tensor");
    if (size == 0 || size > TP_MAX_RANKS || rank >= size)
        return fail(CERA_CUDA_ERR_BAD_ARG, "set_tp: rank %u of %u (at most %u ranks)", rank, size, TP_MAX_RANKS);
    if (size > 1 && c.residual_scale != 0.0f && c.residual_scale != 1.0f)
        return fail(CERA_CUDA_ERR_UNSUPPORTED, "set_tp: a residual scale (Granite) on a tensor-parallel model is not supported");
    if (c.n_kv_heads % size) return fail(CERA_CUDA_ERR_BAD_ARG, "set_tp: %u KV heads do not split over %u ranks", c.n_kv_heads, size);
    if (c.intermediate_size % (32 * size))
        return fail(CERA_CUDA_ERR_BAD_ARG, "set_tp: intermediate size %u must be a multiple of 32 x %u ranks", c.intermediate_size, size);
    if (c.hidden_size % size || c.vocab_size % size)
        return fail(CERA_CUDA_ERR_BAD_ARG, "set_tp: hidden size %u and vocabulary %u must be multiples of %u ranks", c.hidden_size,
                    c.vocab_size, size);
    m->tp_rank = rank;
    m->tp_size = size;
    set_extents(m);
    return CERA_CUDA_OK;
}

int32_t cera_cuda_model_add_tensor(cera_cuda_model *m, int32_t role, int32_t layer, int32_t type, size_t rows,
                                   size_t cols, const void *bytes, size_t nbytes) {
    if (!m || !bytes) return fail(CERA_CUDA_ERR_BAD_ARG, "add_tensor: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (m->finalized) return fail(CERA_CUDA_ERR_STATE, "add_tensor: model already finalized");
    const auto &c = m->cfg;
    const size_t qd = (size_t)c.n_heads * c.head_dim, kvd = (size_t)c.n_kv_heads * c.head_dim;
    const bool per_layer = role >= CERA_ROLE_ATTN_NORM && role <= CERA_ROLE_FFN_DOWN;
    if (per_layer && (layer < 0 || (uint32_t)layer >= c.n_layers))
        return fail(CERA_CUDA_ERR_BAD_ARG, "add_tensor: layer %d out of range", layer);

    auto f32_vector = [&](float **slot, size_t n) -> int32_t {
        if (type != CERA_TYPE_F32) return fail(CERA_CUDA_ERR_UNSUPPORTED, "add_tensor: role %d must be F32, got ggml type %d", role, type);
        if (rows * cols != n || nbytes != n * 4) return fail(CERA_CUDA_ERR_BAD_ARG, "add_tensor: role %d expects %zu floats", role, n);
        if (*slot) return fail(CERA_CUDA_ERR_STATE, "add_tensor: role %d layer %d given twice", role, layer);
        CERA_TRY(dev_alloc(m, (void **)slot, nbytes));
        return check_cuda(cudaMemcpy(*slot, bytes, nbytes, cudaMemcpyDefault), "cudaMemcpy(norm weights)");
    };
    // The caller always hands over the whole tensor; `split` keeps this rank's rows of it.
    auto matrix = [&](cera_cuda_weight **slot, size_t want_m, size_t want_k, bool split = true) -> int32_t {
        if (rows != want_m || cols != want_k)
            return fail(CERA_CUDA_ERR_BAD_ARG, "add_tensor: role %d expects [%zu x %zu], got [%zu x %zu]", role, want_m, want_k, rows, cols);
        if (*slot) return fail(CERA_CUDA_ERR_STATE, "add_tensor: role %d layer %d given twice", role, layer);
        const TypeInfo ti = type_info(type);
        if (!is_block_type(type) || cols % ti.elems || nbytes != rows * (cols / ti.elems) * ti.bytes || !split || m->tp_size == 1) {
            CERA_TRY(weight_upload(type, rows, cols, bytes, nbytes, false, slot));  // also reports the malformed cases
        } else {
            const size_t l_rows = rows / m->tp_size, row_bytes = (cols / ti.elems) * ti.bytes;
            CERA_TRY(weight_upload(type, l_rows, cols, (const char *)bytes + m->tp_rank * l_rows * row_bytes, l_rows * row_bytes, false, slot));
        }
        m->mem_bytes += (*slot)->bytes;
        return CERA_CUDA_OK;
    };
    Layer *L = per_layer ? &m->layers[layer] : nullptr;
    switch (role) {
        case CERA_ROLE_TOKEN_EMBD:
            CERA_TRY(matrix(&m->embd, c.vocab_size, c.hidden_size, false));
            if (m->tp_size > 1) CERA_TRY(matrix(&m->embd_rows, c.vocab_size, c.hidden_size));  // dropped if output.weight arrives
            return CERA_CUDA_OK;
        case CERA_ROLE_OUTPUT: return matrix(&m->output, c.vocab_size, c.hidden_size);
        case CERA_ROLE_OUTPUT_NORM: return f32_vector(&m->out_norm, c.hidden_size);
        case CERA_ROLE_ROPE_FREQS: return f32_vector(&m->rope_freqs, c.head_dim / 2);
        case CERA_ROLE_ATTN_NORM: return f32_vector(&L->attn_norm, c.hidden_size);
        case CERA_ROLE_FFN_NORM: return f32_vector(&L->ffn_norm, c.hidden_size);
        case CERA_ROLE_ATTN_Q: return matrix(&L->wq, qd, c.hidden_size, false);
        case CERA_ROLE_ATTN_K: return matrix(&L->wk, kvd, c.hidden_size, false);
        case CERA_ROLE_ATTN_V: return matrix(&L->wv, kvd, c.hidden_size, false);
        // q / k / v and the o-proj are kept whole on every rank of a tensor-parallel model (see set_extents)
        case CERA_ROLE_ATTN_OUTPUT: return matrix(&L->wo, c.hidden_size, qd, false);
        case CERA_ROLE_FFN_GATE: return matrix(&L->gate, c.intermediate_size, c.hidden_size);
        case CERA_ROLE_FFN_UP: return matrix(&L->up, c.intermediate_size, c.hidden_size);
        case CERA_ROLE_FFN_DOWN: return matrix(&L->down, c.hidden_size, c.intermediate_size);
        default: return fail(CERA_CUDA_ERR_BAD_ARG, "add_tensor: unknown role %d", role);
    }
}

int32_t cera_cuda_model_finalize(cera_cuda_model *m) {
    if (!m) return fail(CERA_CUDA_ERR_BAD_ARG, "finalize: null model");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (m->finalized) return CERA_CUDA_OK;
    const auto &c = m->cfg;
    if (!m->embd || !m->out_norm) return fail(CERA_CUDA_ERR_STATE, "finalize: token_embd / output_norm missing");
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        const Layer &L = m->layers[l];
        if (!L.attn_norm || !L.ffn_norm || !L.wq || !L.wk || !L.wv || !L.wo || !L.gate || !L.up || !L.down)
            return fail(CERA_CUDA_ERR_STATE, "finalize: layer %u is missing a tensor", l);
    }
    const size_t hs = c.hidden_size, qd = (size_t)c.n_heads * c.head_dim, kvd = (size_t)c.n_kv_heads * c.head_dim,
                 ff = c.intermediate_size;
    const size_t esz = c.kv_f16 ? 2 : 4;
    for (auto &L : m->layers) {
        CERA_TRY(dev_alloc(m, &L.kc, (size_t)c.max_seq_len * m->l_kvd * esz));
        CERA_TRY(dev_alloc(m, &L.vc, (size_t)c.max_seq_len * m->l_kvd * esz));
    }
    {
        // Exchange region: the vectors every rank holds in full, at the same offsets on every rank.
        size_t off = 0;
        auto take = [&](size_t bytes) {
            const size_t at = off;
            off += (bytes + 255) & ~(size_t)255;
            return at;
        };
        const size_t o_hidden = take(hs * 4), o_qs = take(qd / 32 * 4), o_qq = take(qd), o_qsum = take(qd / 16 * 2),
                     o_fs = take(ff / 32 * 4), o_fq = take(ff), o_fsum = take(ff / 16 * 2),
                     o_logits = take((size_t)c.vocab_size * 4), o_pairs = take(TP_MAX_RANKS * 8);
        m->tp_slots = 4 * c.n_layers + 2;
        const size_t o_flags = take((size_t)m->tp_slots * TP_MAX_RANKS * 4);
        // tensor-parallel batched prompt: the chunk-wide buffers whose column slices the peers fill
        const bool tp_pf = m->tp_size > 1;
        const size_t C = PREFILL_CHUNK;
        const size_t o_pf_hidden = tp_pf ? take(C * hs * 4) : 0, o_pf_attn = tp_pf ? take(C * qd * 4) : 0,
                     o_pf_g = tp_pf ? take(C * ff * 4) : 0, o_pf_u = tp_pf ? take(C * ff * 4) : 0;
        m->region_bytes = (off + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);  // an allocation of its own to export
        if (m->region_bytes > 0xFFFFFFFFull) return fail(CERA_CUDA_ERR_UNSUPPORTED, "finalize: exchange region of %zu bytes", m->region_bytes);
        CERA_TRY(dev_alloc(m, (void **)&m->region, m->region_bytes));
        CERA_CUDA_TRY(cudaMemset(m->region, 0, m->region_bytes));
        char *b = m->region;
        m->hidden = (float *)(b + o_hidden);
        m->act_q = ActBuf{(float *)(b + o_qs), (int8_t *)(b + o_qq), (int16_t *)(b + o_qsum)};
        m->act_ff = ActBuf{(float *)(b + o_fs), (int8_t *)(b + o_fq), (int16_t *)(b + o_fsum)};
        m->logits = (float *)(b + o_logits);
        if (tp_pf) {
            m->pf_hidden = (float *)(b + o_pf_hidden);
            m->pf_attn = (float *)(b + o_pf_attn);
            m->pf_g = (float *)(b + o_pf_g);
            m->pf_u = (float *)(b + o_pf_u);
        }
        CERA_TRY(dev_alloc(m, (void **)&m->tp_words, 64 * 4));
        CERA_CUDA_TRY(cudaMemset(m->tp_words, 0, 64 * 4));
        m->tp.rank = m->tp_rank;
        m->tp.size = m->tp_size;
        m->tp.peer[m->tp_rank] = m->region;
        m->tp.flags_off = (uint32_t)o_flags;
        m->tp.pairs_off = (uint32_t)o_pairs;
        m->tp.seq = m->tp_words;
        m->tp.status = m->tp_words + 16;
        const char *e = getenv("CERA_CUDA_TP_TIMEOUT_MS");
        const long ms = e ? atol(e) : 5000;
        m->tp.timeout_ns = (uint64_t)(ms > 0 ? ms : 5000) * 1000000ull;
    }
    if (m->output && m->embd_rows) {
        m->mem_bytes -= m->embd_rows->bytes;
        cera_cuda_weight_free(m->embd_rows);
        m->embd_rows = nullptr;
    }
    m->embd_head = m->embd_rows ? m->embd_rows : m->embd;
    // per-rank buffers
    CERA_TRY(dev_alloc(m, (void **)&m->final_hidden, hs * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->q, m->l_qd * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->k, m->l_kvd * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->v, m->l_kvd * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->attn, m->l_qd * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->g, m->l_ff * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->u, m->l_ff * 4));
    CERA_TRY(alloc_act(m, m->act_hs, hs));
    {
        const size_t C = PREFILL_CHUNK;
        CERA_TRY(dev_alloc(m, (void **)&m->pf_tokens, C * 4));
        CERA_TRY(dev_alloc(m, (void **)&m->pf_q, C * m->l_qd * 4));
        CERA_TRY(dev_alloc(m, (void **)&m->pf_k, C * m->l_kvd * 4));
        CERA_TRY(dev_alloc(m, (void **)&m->pf_v, C * m->l_kvd * 4));
        if (m->tp_size == 1) {
            CERA_TRY(dev_alloc(m, (void **)&m->pf_hidden, C * hs * 4));
            CERA_TRY(dev_alloc(m, (void **)&m->pf_attn, C * qd * 4));
            CERA_TRY(dev_alloc(m, (void **)&m->pf_g, C * ff * 4));
            CERA_TRY(dev_alloc(m, (void **)&m->pf_u, C * ff * 4));
            m->pf_attn_local = m->pf_attn;
        } else {
            m->pf_attn_local = m->pf_attn;  // (the chunk-wide buffers sit in the exchange region)
        }
        CERA_TRY(alloc_act(m, m->pf_act_hs, C * hs));
        CERA_TRY(alloc_act(m, m->pf_act_q, C * qd));
        CERA_TRY(alloc_act(m, m->pf_act_ff, C * ff));
    }
    m->attn_ws_bytes = attn_workspace_bytes(m->l_heads, c.head_dim, c.max_seq_len);
    CERA_TRY(dev_alloc(m, &m->attn_ws, m->attn_ws_bytes));
    CERA_TRY(dev_alloc(m, (void **)&m->argmax_scratch, argmax_scratch_words() * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->dyn, 4 * 4));
    CERA_TRY(dev_alloc(m, (void **)&m->tok_out, 4));
    CERA_TRY(dev_alloc(m, (void **)&m->rope_cs, (size_t)c.head_dim * 4));
    {
        // cos / sin of every position from the host's C library (see rope_table_host); skipped beyond 256 MB, where
        // the kernels evaluate sincosf themselves
        const size_t half = c.head_dim / 2, bytes = (size_t)c.max_seq_len * half * 2 * sizeof(float);
        if (bytes <= ((size_t)256 << 20)) {
            std::vector<float> ff;
            if (m->rope_freqs) {
                ff.resize(half);
                CERA_CUDA_TRY(cudaMemcpy(ff.data(), m->rope_freqs, half * sizeof(float), cudaMemcpyDeviceToHost));
            }
            std::vector<float> table((size_t)c.max_seq_len * half * 2);
            rope_table_host(c.max_seq_len, c.head_dim, c.rope_theta, ff.empty() ? nullptr : ff.data(), c.rope_type, table.data());
            CERA_TRY(dev_alloc(m, (void **)&m->rope_table, bytes));
            CERA_CUDA_TRY(cudaMemcpy(m->rope_table, table.data(), bytes, cudaMemcpyHostToDevice));
        }
    }
    m->tok_hist_cap = c.max_seq_len;
    CERA_TRY(dev_alloc(m, (void **)&m->tok_hist, (size_t)m->tok_hist_cap * 4));
    CERA_CUDA_TRY(cudaMallocHost((void **)&m->h_dyn, 8 * 4));
    CERA_CUDA_TRY(cudaMallocHost((void **)&m->h_status, 4));
    CERA_CUDA_TRY(cudaMallocHost((void **)&m->h_logits, (size_t)c.vocab_size * 4));
    CERA_CUDA_TRY(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    CERA_CUDA_TRY(cudaDeviceSynchronize());
    m->finalized = true;
    return CERA_CUDA_OK;
}

int32_t cera_cuda_forward(cera_cuda_model *m, uint32_t token, size_t pos, float *logits_out) {
    if (!m || !logits_out) return fail(CERA_CUDA_ERR_BAD_ARG, "forward: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    CERA_TRY(run_token(m, token, pos, G_LOGITS));
    const size_t bytes = (size_t)m->cfg.vocab_size * 4;
    CERA_CUDA_TRY(cudaMemcpyAsync(m->h_logits, m->logits, bytes, cudaMemcpyDeviceToHost, m->stream));
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    CERA_TRY(tp_check(m));
    memcpy(logits_out, m->h_logits, bytes);
    return CERA_CUDA_OK;
}

int32_t cera_cuda_forward_greedy(cera_cuda_model *m, uint32_t token, size_t pos, uint32_t *token_out) {
    if (!m || !token_out) return fail(CERA_CUDA_ERR_BAD_ARG, "forward_greedy: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    CERA_TRY(run_token(m, token, pos, G_GREEDY));
    CERA_CUDA_TRY(cudaMemcpyAsync(m->h_dyn + 4, m->tok_out, 4, cudaMemcpyDeviceToHost, m->stream));
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    CERA_TRY(tp_check(m));
    *token_out = m->h_dyn[4];
    return CERA_CUDA_OK;
}

int32_t cera_cuda_forward_prefill(cera_cuda_model *m, const uint32_t *tokens, size_t n, size_t start_pos,
                                  float *logits_out) {
    if (!m || (!tokens && n)) return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (start_pos != m->seq_len) return fail(CERA_CUDA_ERR_STATE, "forward_prefill: start_pos %zu != seq_len %zu", start_pos, m->seq_len);
    if (n == 0) return CERA_CUDA_OK;
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "forward_prefill: model_finalize has not been called");
    if (start_pos + n > c.max_seq_len)
        return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill: %zu tokens from %zu exceed max_seq_len %u", n, start_pos, c.max_seq_len);
    for (size_t i = 0; i < n; ++i)
        if (tokens[i] >= c.vocab_size) return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill: token %u out of range", tokens[i]);
    static const bool per_token = [] {
        const char *e = getenv("CERA_CUDA_PREFILL");
        return e && strcmp(e, "per_token") == 0;
    }();
    if (m->tp_size > 1 && !m->tp_connected) return fail(CERA_CUDA_ERR_STATE, "forward_prefill: tensor-parallel model is not connected to its peers");
    // a tensor-parallel model takes the batched kernels for prompts of at least 64 tokens: all but the last token in
    // chunks, the last one through the decode step (which carries the logits exchange)
    const bool tp_batched = m->tp_size > 1 && !per_token && !m->has_lora && n >= 65;
    if (tp_batched) {
        const size_t nb = n - 1;
        for (size_t done = 0; done < nb; done += PREFILL_CHUNK) {
            const size_t cn = nb - done < PREFILL_CHUNK ? nb - done : PREFILL_CHUNK;
            CERA_TRY(prefill_chunk(m, tokens + done, cn, start_pos + done));
            CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
            CERA_TRY(tp_check(m));
        }
        m->seq_len = start_pos + nb;
        CERA_TRY(run_token(m, tokens[nb], start_pos + nb, logits_out ? G_LOGITS : G_BODY));
        CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
        CERA_TRY(tp_check(m));
    } else if (per_token || n < 2 || m->tp_size > 1 || m->has_lora) {
        // Decode arithmetic for every prompt position (one graph launch per token).  h_dyn is rewritten per
        // token, so wait for the copy of the previous one before touching it again.
        for (size_t i = 0; i < n; ++i) {
            const bool last = i + 1 == n;
            CERA_TRY(run_token(m, tokens[i], start_pos + i, last && logits_out ? G_LOGITS : G_BODY));
            CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
        }
        CERA_TRY(tp_check(m));
    } else {
        // Batched kernels, PREFILL_CHUNK tokens at a time (the reference's ubatch loop, cera/src/model/mod.rs:303-332).
        for (size_t done = 0; done < n; done += PREFILL_CHUNK) {
            const size_t cn = n - done < PREFILL_CHUNK ? n - done : PREFILL_CHUNK;
            CERA_TRY(prefill_chunk(m, tokens + done, cn, start_pos + done));
            CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));  // the host token slice may go away after the call
        }
        m->seq_len = start_pos + n;
        if (logits_out) CERA_TRY(logits_from_hidden(m));
    }
    if (logits_out) {
        const size_t bytes = (size_t)m->cfg.vocab_size * 4;
        CERA_CUDA_TRY(cudaMemcpyAsync(m->h_logits, m->logits, bytes, cudaMemcpyDeviceToHost, m->stream));
        CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
        memcpy(logits_out, m->h_logits, bytes);
    }
    return CERA_CUDA_OK;
}

// Model::forward_prefill_logits_all (cera/src/model/mod.rs:507-533, used by speculative decoding): the logits of
// EVERY prompt position, logits_out[n][vocab] on the host, token-major.
int32_t cera_cuda_forward_prefill_logits_all(cera_cuda_model *m, const uint32_t *tokens, size_t n, size_t start_pos,
                                             float *logits_out) {
    if (!m || !tokens || !logits_out) return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill_logits_all: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "forward_prefill_logits_all: model_finalize has not been called");
    if (start_pos != m->seq_len) return fail(CERA_CUDA_ERR_STATE, "forward_prefill_logits_all: start_pos %zu != seq_len %zu", start_pos, m->seq_len);
    if (start_pos + n > c.max_seq_len)
        return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill_logits_all: %zu tokens from %zu exceed max_seq_len %u", n, start_pos, c.max_seq_len);
    for (size_t i = 0; i < n; ++i)
        if (tokens[i] >= c.vocab_size) return fail(CERA_CUDA_ERR_BAD_ARG, "forward_prefill_logits_all: token %u out of range", tokens[i]);
    const size_t vocab = c.vocab_size;
    if (m->tp_size > 1 || m->has_lora) {
        // tensor-parallel (each position with its logits exchange) or adapters attached: the decode step per position
        if (m->tp_size > 1 && !m->tp_connected) return fail(CERA_CUDA_ERR_STATE, "forward_prefill_logits_all: tensor-parallel model is not connected to its peers");
        for (size_t i = 0; i < n; ++i) {
            CERA_TRY(run_token(m, tokens[i], start_pos + i, G_LOGITS));
            CERA_CUDA_TRY(cudaMemcpyAsync(logits_out + i * vocab, m->logits, vocab * 4, cudaMemcpyDeviceToHost, m->stream));
            CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
        }
        return tp_check(m);
    }
    if (!m->pf_logits) CERA_TRY(dev_alloc(m, (void **)&m->pf_logits, PREFILL_CHUNK * vocab * 4));
    const cera_cuda_weight *ow = m->output ? m->output : m->embd;
    for (size_t done = 0; done < n; done += PREFILL_CHUNK) {
        const size_t cn = n - done < PREFILL_CHUNK ? n - done : PREFILL_CHUNK;
        CERA_TRY(prefill_chunk(m, tokens + done, cn, start_pos + done));
        CERA_TRY(launch_rmsnorm(m->pf_hidden, m->out_norm, c.hidden_size, cn, c.rms_norm_eps, nullptr, m->pf_act_hs.scales,
                                m->pf_act_hs.quants, m->pf_act_hs.sums, m->stream));
        CERA_TRY(launch_gemm_ex(ow->v, m->pf_act_hs.view(), cn, m->pf_logits, 1, vocab, EPI_STORE, m->stream));
        if (c.logit_scale != 0.0f && c.logit_scale != 1.0f) CERA_TRY(launch_scale(m->pf_logits, cn * vocab, 1.0f / c.logit_scale, m->stream));
        CERA_CUDA_TRY(cudaMemcpyAsync(logits_out + done * vocab, m->pf_logits, cn * vocab * 4, cudaMemcpyDeviceToHost, m->stream));
        CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
        m->seq_len = start_pos + done + cn;
    }
    return CERA_CUDA_OK;
}

int32_t cera_cuda_generate_greedy(cera_cuda_model *m, uint32_t first_token, size_t start_pos, size_t n,
                                  uint32_t *tokens_out, float *device_ms) {
    if (!m || !tokens_out) return fail(CERA_CUDA_ERR_BAD_ARG, "generate_greedy: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "generate_greedy: model_finalize has not been called");
    if (first_token >= c.vocab_size) return fail(CERA_CUDA_ERR_BAD_ARG, "generate_greedy: token out of range");
    if (start_pos != m->seq_len) return fail(CERA_CUDA_ERR_STATE, "generate_greedy: start_pos %zu != seq_len %zu", start_pos, m->seq_len);
    if (start_pos + n > c.max_seq_len) return fail(CERA_CUDA_ERR_BAD_ARG, "generate_greedy: %zu tokens from %zu exceed max_seq_len %u", n, start_pos, c.max_seq_len);
    if (m->tp_size > 1 && !m->tp_connected) return fail(CERA_CUDA_ERR_STATE, "generate_greedy: tensor-parallel model is not connected to its peers");
    if (n == 0) return CERA_CUDA_OK;
    m->h_dyn[0] = first_token;
    m->h_dyn[1] = (uint32_t)start_pos;
    m->h_dyn[2] = (uint32_t)start_pos + 1;
    m->h_dyn[3] = 0;
    CERA_CUDA_TRY(cudaMemcpyAsync(m->dyn, m->h_dyn, 4 * sizeof(uint32_t), cudaMemcpyHostToDevice, m->stream));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    CERA_CUDA_TRY(cudaEventCreate(&e0));
    CERA_CUDA_TRY(cudaEventCreate(&e1));
    // instantiate every graph the run needs before the timed region
    for (size_t i = 0; i < n; ++i) {
        cudaGraphExec_t g = nullptr;
        CERA_TRY(get_graph(m, G_CHAIN, attn_plan(m->l_heads, m->l_kv_heads, m->cfg.head_dim, start_pos + i + 1), &g));
    }
    CERA_CUDA_TRY(cudaEventRecord(e0, m->stream));
    for (size_t i = 0; i < n; ++i) {
        cudaGraphExec_t g = nullptr;
        CERA_TRY(get_graph(m, G_CHAIN, attn_plan(m->l_heads, m->l_kv_heads, m->cfg.head_dim, start_pos + i + 1), &g));
        CERA_CUDA_TRY(cudaGraphLaunch(g, m->stream));
    }
    CERA_CUDA_TRY(cudaEventRecord(e1, m->stream));
    m->launches += (uint64_t)m->nodes_per_step[G_CHAIN] * n;
    m->seq_len = start_pos + n;
    CERA_CUDA_TRY(cudaMemcpyAsync(tokens_out, m->tok_hist, n * 4, cudaMemcpyDeviceToHost, m->stream));
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    float ms = 0.0f;
    CERA_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    if (device_ms) *device_ms = ms;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return tp_check(m);
}

int32_t cera_cuda_model_tp_handle(cera_cuda_model *m, void *handle_out, size_t handle_bytes) {
    if (!m || !handle_out) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_handle: null argument");
    if (handle_bytes != sizeof(cudaIpcMemHandle_t)) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_handle: handle is %zu bytes", sizeof(cudaIpcMemHandle_t));
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "tp_handle: model_finalize has not been called");
    cudaIpcMemHandle_t h;
    CERA_CUDA_TRY(cudaIpcGetMemHandle(&h, m->region));
    memcpy(handle_out, &h, sizeof(h));
    return CERA_CUDA_OK;
}

int32_t cera_cuda_model_tp_connect(cera_cuda_model *m, const void *handles, size_t n_handles) {
    if (!m || !handles) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_connect: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "tp_connect: model_finalize has not been called");
    if (n_handles != m->tp_size) return fail(CERA_CUDA_ERR_BAD_ARG, "tp_connect: %zu handles for %u ranks", n_handles, m->tp_size);
    if (m->tp_connected) return fail(CERA_CUDA_ERR_STATE, "tp_connect: already connected");
    for (uint32_t p = 0; p < m->tp_size; ++p) {
        if (p == m->tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)p * sizeof(h), sizeof(h));
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(CERA_CUDA_ERR_PEER, "tp_connect: rank %u's exchange region cannot be mapped: %s", p, cudaGetErrorString(e));
        }
        m->tp_opened[p] = ptr;
        m->tp.peer[p] = (char *)ptr;
    }
    m->tp_connected = true;
    return CERA_CUDA_OK;
}

int32_t cera_cuda_truncate_kv(cera_cuda_model *m, size_t len) {
    if (!m) return fail(CERA_CUDA_ERR_BAD_ARG, "truncate_kv: null model");
    std::lock_guard<std::mutex> lock(m->mu);
    if (len < m->seq_len) m->seq_len = len;  // rows beyond seq_len are simply overwritten later
    return CERA_CUDA_OK;
}

// ---- LoRA (InferenceState::lora, cera/src/lora.rs) ---------------------------------------------------------

int32_t cera_cuda_model_attach_lora(cera_cuda_model *m, int32_t target, int32_t layer, size_t rank, size_t k, size_t d,
                                    const float *a, const float *b, float scale) {
    if (!m || !a || !b) return fail(CERA_CUDA_ERR_BAD_ARG, "attach_lora: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "attach_lora: model_finalize has not been called");
    if (m->tp_size > 1) return fail(CERA_CUDA_ERR_UNSUPPORTED, "attach_lora: adapters on a tensor-parallel model are not supported");
    if (target < 0 || target > 6 || layer < 0 || (uint32_t)layer >= c.n_layers)
        return fail(CERA_CUDA_ERR_BAD_ARG, "attach_lora: target %d layer %d", target, layer);
    const size_t hs = c.hidden_size, qd = (size_t)c.n_heads * c.head_dim, kvd = (size_t)c.n_kv_heads * c.head_dim, ff = c.intermediate_size;
    const size_t want_k[7] = {hs, hs, hs, qd, hs, hs, ff}, want_d[7] = {qd, kvd, kvd, hs, ff, ff, hs};
    if (k != want_k[target] || d != want_d[target] || rank == 0 || rank > 256)
        return fail(CERA_CUDA_ERR_BAD_ARG, "attach_lora: target %d expects A [rank<=256 x %zu], B [%zu x rank]; got rank %zu, k %zu, d %zu", target,
                    want_k[target], want_d[target], rank, k, d);
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    Lora &t = m->layers[layer].lora[target];
    float *da = nullptr, *db = nullptr;
    CERA_TRY(dev_alloc(m, (void **)&da, rank * k * 4));
    CERA_TRY(dev_alloc(m, (void **)&db, d * rank * 4));
    CERA_CUDA_TRY(cudaMemcpy(da, a, rank * k * 4, cudaMemcpyDefault));
    CERA_CUDA_TRY(cudaMemcpy(db, b, d * rank * 4, cudaMemcpyDefault));
    if (!m->normed) CERA_TRY(dev_alloc(m, (void **)&m->normed, hs * 4));
    t = Lora{da, db, (uint32_t)rank, (uint32_t)k, (uint32_t)d, scale};  // a replaced pair stays allocated until model_free
    m->has_lora = true;
    for (auto &kv : m->graphs) cudaGraphExecDestroy(kv.second);  // the recorded steps do not contain the new kernels
    m->graphs.clear();
    return CERA_CUDA_OK;
}

int32_t cera_cuda_model_detach_lora(cera_cuda_model *m) {
    if (!m) return fail(CERA_CUDA_ERR_BAD_ARG, "detach_lora: null model");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (m->stream) CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    for (auto &L : m->layers)
        for (auto &t : L.lora) t = Lora{};
    m->has_lora = false;
    for (auto &kv : m->graphs) cudaGraphExecDestroy(kv.second);
    m->graphs.clear();
    return CERA_CUDA_OK;
}

// ---- KV cache management (trait Model: shift_kv, snapshot / restore) -----------------------------------

int32_t cera_cuda_kv_shift(cera_cuda_model *m, size_t n_keep, size_t shift) {
    if (!m) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_shift: null model");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    const auto &c = m->cfg;
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "kv_shift: model_finalize has not been called");
    if (shift == 0) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_shift: shift must be > 0");
    if (n_keep + shift > m->seq_len)
        return fail(CERA_CUDA_ERR_BAD_ARG, "kv_shift: n_keep %zu + shift %zu exceed seq_len %zu", n_keep, shift, m->seq_len);
    const size_t n_rows = m->seq_len - n_keep - shift, esz = c.kv_f16 ? 2 : 4, row_bytes = m->l_kvd * esz;
    if (n_rows) {
        void *tmp = nullptr;  // the tail as it was, K then V (a rare operation: allocated per call)
        CERA_CUDA_TRY(cudaMalloc(&tmp, 2 * n_rows * row_bytes));
        int32_t st = CERA_CUDA_OK;
        for (auto &L : m->layers) {
            char *kt = (char *)tmp, *vt = kt + n_rows * row_bytes;
            st = check_cuda(cudaMemcpyAsync(kt, (char *)L.kc + (n_keep + shift) * row_bytes, n_rows * row_bytes, cudaMemcpyDeviceToDevice, m->stream), "kv_shift copy");
            if (st == CERA_CUDA_OK)
                st = check_cuda(cudaMemcpyAsync(vt, (char *)L.vc + (n_keep + shift) * row_bytes, n_rows * row_bytes, cudaMemcpyDeviceToDevice, m->stream), "kv_shift copy");
            if (st == CERA_CUDA_OK)
                st = launch_kv_shift(kt, vt, L.kc, L.vc, n_keep, shift, n_rows, m->l_kv_heads, c.head_dim, m->theta_scale, m->rope_freqs,
                                     c.rope_type, c.kv_f16, m->stream);
            if (st != CERA_CUDA_OK) break;
        }
        cudaError_t e = cudaStreamSynchronize(m->stream);
        cudaFree(tmp);
        CERA_TRY(st);
        CERA_CUDA_TRY(e);
    }
    m->seq_len -= shift;
    return CERA_CUDA_OK;
}

namespace {
struct SnapshotHeader {
    uint32_t magic, version, n_layers, kv_dim, elem_bytes, reserved;
    uint64_t seq_len;
};
constexpr uint32_t SNAPSHOT_MAGIC = 0x564B4243u;  // "CBKV"
}  // namespace

size_t cera_cuda_kv_snapshot_bytes(const cera_cuda_model *m) {
    if (!m || !m->finalized) return 0;
    const size_t esz = m->cfg.kv_f16 ? 2 : 4;
    return sizeof(SnapshotHeader) + 2 * (size_t)m->cfg.n_layers * m->seq_len * m->l_kvd * esz;
}

int32_t cera_cuda_kv_snapshot(cera_cuda_model *m, void *out, size_t out_bytes) {
    if (!m || !out) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_snapshot: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "kv_snapshot: model_finalize has not been called");
    const size_t esz = m->cfg.kv_f16 ? 2 : 4, rows = m->seq_len * m->l_kvd * esz;
    const size_t need = sizeof(SnapshotHeader) + 2 * (size_t)m->cfg.n_layers * rows;
    if (out_bytes < need) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_snapshot: %zu bytes given, %zu needed", out_bytes, need);
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    SnapshotHeader h{SNAPSHOT_MAGIC, 1, m->cfg.n_layers, (uint32_t)m->l_kvd, (uint32_t)esz, 0, (uint64_t)m->seq_len};
    memcpy(out, &h, sizeof(h));
    char *p = (char *)out + sizeof(h);
    for (auto &L : m->layers) {
        CERA_CUDA_TRY(cudaMemcpy(p, L.kc, rows, cudaMemcpyDeviceToHost));
        CERA_CUDA_TRY(cudaMemcpy(p + rows, L.vc, rows, cudaMemcpyDeviceToHost));
        p += 2 * rows;
    }
    return CERA_CUDA_OK;
}

int32_t cera_cuda_kv_restore(cera_cuda_model *m, const void *data, size_t bytes) {
    if (!m || !data) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "kv_restore: model_finalize has not been called");
    SnapshotHeader h;
    if (bytes < sizeof(h)) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: %zu bytes is shorter than the header", bytes);
    memcpy(&h, data, sizeof(h));
    const size_t esz = m->cfg.kv_f16 ? 2 : 4;
    if (h.magic != SNAPSHOT_MAGIC || h.version != 1) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: not a KV snapshot of this library");
    if (h.n_layers != m->cfg.n_layers || h.kv_dim != m->l_kvd || h.elem_bytes != esz)
        return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: snapshot of %u layers x %u x %u bytes does not fit this model (%u x %zu x %zu)",
                    h.n_layers, h.kv_dim, h.elem_bytes, m->cfg.n_layers, m->l_kvd, esz);
    if (h.seq_len > m->cfg.max_seq_len) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: %llu positions exceed max_seq_len %u",
                                                   (unsigned long long)h.seq_len, m->cfg.max_seq_len);
    const size_t rows = (size_t)h.seq_len * m->l_kvd * esz;
    if (bytes != sizeof(h) + 2 * (size_t)h.n_layers * rows) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore: truncated snapshot");
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    const char *p = (const char *)data + sizeof(h);
    for (auto &L : m->layers) {
        CERA_CUDA_TRY(cudaMemcpy(L.kc, p, rows, cudaMemcpyHostToDevice));
        CERA_CUDA_TRY(cudaMemcpy(L.vc, p + rows, rows, cudaMemcpyHostToDevice));
        p += 2 * rows;
    }
    m->seq_len = (size_t)h.seq_len;
    return CERA_CUDA_OK;
}

size_t cera_cuda_kv_layer_bytes(const cera_cuda_model *m) {
    return m ? m->seq_len * m->l_kvd * (m->cfg.kv_f16 ? 2 : 4) : 0;
}

int32_t cera_cuda_kv_snapshot_layer(cera_cuda_model *m, uint32_t layer, void *k_data, void *v_data, size_t bytes_each) {
    if (!m || !k_data || !v_data) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_snapshot_layer: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "kv_snapshot_layer: model not finalized");
    if (layer >= m->cfg.n_layers) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_snapshot_layer: layer %u of %u", layer, m->cfg.n_layers);
    const size_t rows = m->seq_len * m->l_kvd * (m->cfg.kv_f16 ? 2 : 4);
    if (bytes_each != rows) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_snapshot_layer: %zu bytes given, a layer holds %zu", bytes_each, rows);
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    CERA_CUDA_TRY(cudaMemcpy(k_data, m->layers[layer].kc, rows, cudaMemcpyDeviceToHost));
    return check_cuda(cudaMemcpy(v_data, m->layers[layer].vc, rows, cudaMemcpyDeviceToHost), "cudaMemcpy(kv_snapshot_layer)");
}

int32_t cera_cuda_kv_restore_layer(cera_cuda_model *m, uint32_t layer, const void *k_data, const void *v_data, size_t bytes_each,
                                   size_t seq_len) {
    if (!m || (bytes_each && (!k_data || !v_data))) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore_layer: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "kv_restore_layer: model not finalized");
    if (layer >= m->cfg.n_layers) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore_layer: layer %u of %u", layer, m->cfg.n_layers);
    if (seq_len > m->cfg.max_seq_len) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore_layer: %zu positions exceed max_seq_len %u", seq_len, m->cfg.max_seq_len);
    const size_t rows = seq_len * m->l_kvd * (m->cfg.kv_f16 ? 2 : 4);
    // a snapshot taken with the other element width has half / twice the bytes: the reference's cross-mode gate (kv_cache.rs:1411-1421)
    if (bytes_each != rows) return fail(CERA_CUDA_ERR_BAD_ARG, "kv_restore_layer: %zu bytes given, %zu positions of this cache are %zu", bytes_each, seq_len, rows);
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    if (rows) {
        CERA_CUDA_TRY(cudaMemcpy(m->layers[layer].kc, k_data, rows, cudaMemcpyHostToDevice));
        CERA_CUDA_TRY(cudaMemcpy(m->layers[layer].vc, v_data, rows, cudaMemcpyHostToDevice));
    }
    m->seq_len = seq_len;
    return CERA_CUDA_OK;
}

size_t cera_cuda_seq_len(const cera_cuda_model *m) { return m ? m->seq_len : 0; }
size_t cera_cuda_memory_bytes(const cera_cuda_model *m) { return m ? m->mem_bytes : 0; }
uint64_t cera_cuda_launch_count(const cera_cuda_model *m) { return m ? m->launches : 0; }

int32_t cera_cuda_last_hidden(cera_cuda_model *m, float *out) {
    if (!m || !out) return fail(CERA_CUDA_ERR_BAD_ARG, "last_hidden: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard dg(m->cfg.device);
    if (!m->finalized) return fail(CERA_CUDA_ERR_STATE, "last_hidden: model not finalized");
    CERA_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return check_cuda(cudaMemcpy(out, m->final_hidden, (size_t)m->cfg.hidden_size * 4, cudaMemcpyDeviceToHost),
                      "cudaMemcpy(last_hidden)");
}

void cera_cuda_model_free(cera_cuda_model *m) {
    if (!m) return;
    {
        DeviceGuard dg(m->cfg.device);
        if (m->stream) cudaStreamSynchronize(m->stream);
        for (auto &kv : m->graphs) cudaGraphExecDestroy(kv.second);
        for (void *p : m->owned) cudaFree(p);
        auto fw = [](cera_cuda_weight *w) {
            if (w) cera_cuda_weight_free(w);
        };
        fw(m->embd);
        fw(m->output);
        for (auto &L : m->layers) {
            fw(L.wq); fw(L.wk); fw(L.wv); fw(L.wo); fw(L.gate); fw(L.up); fw(L.down);
        }
        for (void *p : m->tp_opened)
            if (p) cudaIpcCloseMemHandle(p);
        fw(m->embd_rows);
        if (m->h_status) cudaFreeHost(m->h_status);
        if (m->h_dyn) cudaFreeHost(m->h_dyn);
        if (m->h_logits) cudaFreeHost(m->h_logits);
        if (m->stream) cudaStreamDestroy(m->stream);
    }
    delete m;
}

}  // extern "C"
