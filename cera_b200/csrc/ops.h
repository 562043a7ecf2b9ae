// Internal launch helpers shared between the C entry points and the model.
#pragma once

#include "act.cuh"
#include "common.cuh"
#include "tp.cuh"

namespace cera {

int32_t launch_quantize(const float *x, size_t k, size_t n, bool strided, float *scales, int8_t *quants,
                        int16_t *sums, cudaStream_t st);
// out_f32 and the quantized outputs are each optional (null = skip).
// tp (optional, tensor-parallel decode step): rmsnorm waits for the exchange that completes x; silu_mul mirrors its
// quantized output into the peers' regions.
int32_t launch_rmsnorm(const float *x, const float *weight, size_t n_elem, size_t n_cols, float eps, float *out_f32,
                       float *scales, int8_t *quants, int16_t *sums, cudaStream_t st, const TpHook *tp = nullptr);
int32_t launch_silu_mul(float *gate, const float *up, size_t n_elem, size_t n_cols, float *scales, int8_t *quants,
                        int16_t *sums, cudaStream_t st, const TpHook *tp = nullptr);

// Up to three weight matrices of one type sharing the same activations
// (q/k/v, gate/up), handled by one launch.
struct GemvSeg {
    WeightView w;
    float *y;  // [m x n] row-major
};
// EPI_STORE: y = Wx.  EPI_ADD: y += Wx (residual).  EPI_ROPE_KV: segments are q, k, v; q and k rows are
// rotated (NORM pairs) with the per-token cos/sin table, k and v go straight into the KV cache row.
enum { EPI_STORE = 0, EPI_ADD = 1, EPI_ROPE_KV = 2 };

// Work fused behind the single-column GEMV (EPI_ROPE_KV).
struct GemvFusion {
    const float *rope_cs = nullptr;       // [head_dim/2][2] cos, sin at the current position, or with rope_by_pos
                                          // the table of every position [max_seq][head_dim/2][2]
    int rope_by_pos = 0;
    const uint32_t *pos_dev = nullptr;
    void *k_cache = nullptr, *v_cache = nullptr;
    int kv_f16 = 0;
    uint32_t head_dim = 0, kv_dim = 0;
    // RMSNorm prologue (reference-order GEMV only): the activation column is formed in the kernel from the f32 vector
    // norm_x and the norm weights - normalise, scale, quantize to Q8_0 - instead of being read from `x`;
    // norm_out (optional) receives the normalised f32 vector
    const float *norm_x = nullptr, *norm_w = nullptr;
    float norm_eps = 0.0f;
    float *norm_out = nullptr;
};
// tp (optional): wait for the exchange that completes x before reading it and / or mirror the output stores
// (EPI_STORE / EPI_ADD, single column) into the peers' regions.
int32_t launch_gemv(const GemvSeg *segs, int n_segs, const ActView &x, size_t n_cols, size_t ldy, int epilogue,
                    cudaStream_t st, size_t ldc = 1, bool batch_tile = false, const TpHook *tp = nullptr);
int32_t launch_gemm_ex(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                       cudaStream_t st);
// Register-resident-activation single-column GEMV.  *taken = false: shape outside its rules,
// nothing was launched and the caller uses the item-wise kernel.
int32_t launch_gemv_rows(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                         cudaStream_t st, bool *taken, const TpHook *tp = nullptr);
// Same contract through the TMA-staged kernel (bulk asynchronous copies into a shared-memory ring).
int32_t launch_gemv_tma(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                        cudaStream_t st, bool *taken);
// Tries the TMA-staged kernel, then the register-streaming one.
int32_t launch_gemv_fused(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp = nullptr);
// The same GEMV in the reference's f32 summation order (K-quants, k a multiple of 1024): results are bit-identical to
// cera's x86 int8 kernels at one activation column.  *taken = false: not its case, nothing launched.
int32_t launch_gemv_exact(const GemvSeg *segs, int n_segs, const ActView &x, int epilogue, const GemvFusion *fusion,
                          cudaStream_t st, bool *taken, const TpHook *tp = nullptr);
// cos/sin of every rotation pair at position *pos_dev, same arithmetic as launch_rope.
int32_t launch_rope_table(const uint32_t *pos_dev, size_t head_dim, float theta_scale, const float *freq_factors,
                          float *table, cudaStream_t st, const float *full_table = nullptr);
int32_t launch_gemm(const WeightView &w, const ActView &x, size_t n, float *out, cudaStream_t st);
// Tensor-core (mma.sync int8) GEMM for Q4_0 / Q4_K / Q5_K / Q6_K (k a multiple of 256) and n >= 5.  *taken = false: not its case.
int32_t launch_gemm_mma(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                        cudaStream_t st, bool *taken);
// The same product on tcgen05 / TMEM (gemm_tc.cu): Q4_K / Q5_K, k a multiple of 256, more than 32 columns.
int32_t launch_gemm_tc(const WeightView &w, const ActView &x, size_t n, float *out, size_t ldy, size_t ldc, int epilogue,
                       cudaStream_t st, bool *taken);
// The same for up to three weights that take the same activations, in one launch when every weight has its image.
struct GemmTarget {
    WeightView w;
    float *out;
    size_t ldc;
};
int32_t launch_gemm_tc_multi(const GemmTarget *t, int count, const ActView &x, size_t n, size_t ldy, int epilogue, cudaStream_t st,
                             bool *taken);
uint32_t gemm_tc_status();  // nonzero after a bounded wait of that kernel ran out
uint32_t gemv_exact_status();
// One work item of an expert-grouped GEMM: `count` consecutive activation columns starting at `first` go through
// expert `expert`'s rows of a stacked weight matrix (built on the device by the routed-FFN kernels).
struct MoeTile {
    uint32_t expert, first, count;
};
// The tensor-core GEMM over a device-side list of such items (one column tile of up to `bn` = 64 or 32 columns per item):
// w stacks `rows_per_expert` rows per expert; cell (row i of the expert, column c) goes to out[c * ldc + i].
// *taken = false: no tensor-core path for this weight type / shape.
bool gemm_mma_supports(int type, size_t k);  // a tensor-core path exists for this weight type and row length
int32_t launch_gemm_mma_grouped(const WeightView &w, const ActView &x, const MoeTile *tiles, const uint32_t *n_tiles,
                                uint32_t max_tiles, uint32_t rows_per_expert, float *out, size_t ldc, uint32_t bn, cudaStream_t st,
                                bool *taken);
int32_t launch_gemv_q5k_f32(const WeightView &w, const float *x, float *y, cudaStream_t st);

// Rotates q and k in place at position pos (or *pos_dev when non-null).  When k_cache is
// non-null the rotated k and the untouched v are also appended as cache row `pos`
// (f32, or f16 through the round-to-nearest-even narrow of cera/src/quant.rs:117-164).
int32_t launch_rope(float *q, float *k, const float *v, size_t pos, const uint32_t *pos_dev, size_t n_heads,
                    size_t n_kv_heads, size_t head_dim, float theta_scale, const float *freq_factors, int rope_type,
                    void *k_cache, void *v_cache, int kv_f16, cudaStream_t st, const float *table = nullptr);
// table (optional, every rope launcher): cos / sin of every (position, rotation pair), [max_pos][head_dim/2][2], as
// rope_table_host() computes them; the kernels then read the table instead of evaluating sincosf.
void rope_table_host(size_t n_pos, size_t head_dim, float rope_theta, const float *freq_factors, int rope_type, float *out);

size_t attn_workspace_bytes(size_t n_heads, size_t head_dim, size_t seq_len);
// q8 outputs optional: the merge pass can emit the Q8_0 form of `out` for the next GEMV.
int32_t launch_decode_attention(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                size_t n_kv_heads, size_t head_dim, size_t seq_len, float scale, float *out,
                                void *workspace, size_t workspace_bytes, float *scales, int8_t *quants, int16_t *sums,
                                cudaStream_t st);

uint32_t attn_pick_splits(size_t n_kv_heads, size_t seq_len_hint);
// The plan word launch_decode_attention_ex takes: the reference-order kernels (attention_exact.cu) whenever they cover
// the head shape, else attn_pick_splits.
uint32_t attn_plan(size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t seq_len_hint);
bool attn_exact_supports(size_t n_heads, size_t n_kv_heads, size_t head_dim);
uint32_t attn_exact_plan(size_t seq_len_hint);
size_t attn_exact_workspace_bytes(size_t n_heads, size_t seq_len);
int32_t launch_decode_attention_exact(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads, size_t n_kv_heads,
                                      size_t head_dim, size_t seq_len, const uint32_t *seq_len_dev, uint32_t plan, float scale,
                                      float *out, void *workspace, size_t workspace_bytes, float *scales, int8_t *quants,
                                      int16_t *sums, cudaStream_t st, const TpHook *tp = nullptr);
// Split pass of a long-context decode attention through the shared-memory-staged kernel (attention_stream.cu); writes the
// same per-(head, split) records as the register-resident split kernel.  *taken = false: no instantiation.
int32_t launch_attention_stream(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_kv_heads, size_t group,
                                size_t head_dim, uint32_t seq_len, const uint32_t *seq_len_dev, uint32_t n_splits, float scale,
                                float *ws, cudaStream_t st, bool *taken);

// seq_len_dev != null: the kernel reads the length from device memory (graph replay).
int32_t launch_decode_attention_ex(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                   size_t n_kv_heads, size_t head_dim, size_t seq_len, const uint32_t *seq_len_dev,
                                   uint32_t n_splits, float scale, float *out, void *workspace, size_t workspace_bytes,
                                   float *scales, int8_t *quants, int16_t *sums, cudaStream_t st,
                                   const TpHook *tp = nullptr);  // tp: mirror the Q8_0 output into the peers' regions

int32_t launch_embed(const WeightView &w, uint32_t token, const uint32_t *token_dev, float *out, cudaStream_t st);
// n rows: out[j][k] = row tokens_dev[j] of the table.
// x[i] *= s, and y[i] += x[i] * s (product rounded, then the sum: cera/src/backend/cpu.rs scale_inplace + add_inplace)
int32_t launch_scale(float *x, size_t n, float s, cudaStream_t st);
int32_t launch_scaled_add(float *y, const float *x, size_t n, float s, cudaStream_t st);
int32_t launch_embed_batch(const WeightView &w, const uint32_t *tokens_dev, size_t n, float *out, cudaStream_t st);
// n tokens at positions start_pos + j: q is [n][n_heads*head_dim], k and v are [n][n_kv_heads*head_dim]
// (token-major); rotated k and v rows are appended to the caches.
int32_t launch_rope_batch(float *q, float *k, const float *v, size_t start_pos, size_t n, size_t n_heads, size_t n_kv_heads,
                          size_t head_dim, float theta_scale, const float *freq_factors, int rope_type, void *k_cache,
                          void *v_cache, int kv_f16, cudaStream_t st, const float *table = nullptr);
// Causal attention of n query tokens (positions start_pos + j) over cache rows [0, start_pos + j]
// (cera/src/backend/cpu.rs:4028-4241); q and out are token-major [n][n_heads*head_dim].
int32_t launch_prefill_attention(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                 size_t n_kv_heads, size_t head_dim, size_t n, size_t start_pos, float scale, float *out,
                                 cudaStream_t st);
// The same through the shared-memory-tiled kernel (attention_prefill.cu).  *taken = false: not its case, nothing launched.
int32_t launch_prefill_attention_tiled(const float *q, const void *kc, const void *vc, int kv_f16, size_t n_heads,
                                       size_t n_kv_heads, size_t head_dim, size_t n, size_t start_pos, float scale, float *out,
                                       cudaStream_t st, bool *taken);
// y[d] += B (scale * (A x)): one LoRA pair applied to one token (cera/src/lora.rs:794-821).
int32_t launch_lora(const float *x, const float *a, const float *b, size_t rank, size_t k, size_t d, float scale, float *y,
                    cudaStream_t st);
// Rows [n_keep + shift, n_keep + shift + n_rows) of a cache, given as a copy in k_src / v_src, re-enter it at
// [n_keep, n_keep + n_rows) with K rotated by R(-shift) (cera/src/kv_cache.rs:1091-1320).
int32_t launch_kv_shift(const void *k_src, const void *v_src, void *k_cache, void *v_cache, size_t n_keep, size_t shift,
                        size_t n_rows, size_t n_kv_heads, size_t head_dim, float theta_scale, const float *freq_factors,
                        int rope_type, int kv_f16, cudaStream_t st);
// First strict maximum (cera/src/sampler.rs:20-30).  scratch: 2*blocks words, see argmax_scratch_words().
size_t argmax_scratch_words();
int32_t launch_argmax(const float *x, size_t n, uint32_t *out, uint32_t *scratch, cudaStream_t st);

// ---- tensor-parallel exchange (tp.cu) -------------------------------------------
struct TpRange {
    uint32_t off, bytes;  // inside the exchange region
};
int32_t launch_tp_tick(uint32_t *seq, cudaStream_t st);
// Pushes the ranges (0 to 3) to the same offsets of every peer, then waits for every peer's push of this slot.
int32_t launch_tp_exchange(const TpCtx &ctx, const TpRange *ranges, int n_ranges, uint32_t slot, cudaStream_t st);
// logits_local[local_n] are this rank's rows, *local_idx its local first maximum; *tok_out = global pick.
int32_t launch_tp_argmax(const TpCtx &ctx, const float *logits_local, uint32_t local_n, const uint32_t *local_idx,
                         uint32_t *tok_out, uint32_t slot, cudaStream_t st);

}  // namespace cera
