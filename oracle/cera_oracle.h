/* CPU oracle for the quantized-matmul / decode-attention hot path of cera.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in scalar C++, the
 * arithmetic of cera's own CPU kernels so that the CUDA device can be checked
 * against it.  Nothing in the shipped CUDA path links, loads or calls it; only
 * the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity pin: the reference is Rust and cannot be compiled where this was
 * written, so the oracle is pinned by the reference's own known-answer tests
 * restated against it (tests/test_oracle_*.py): the half-precision converter
 * boundary list and LCG sweep of cera/src/quant.rs:982-1061 checked against an
 * independent IEEE implementation, the block dequantizer fixtures of
 * cera/src/quant.rs:1141-1879, the integer reference `ref_gemm` and extreme
 * fixtures of cera/src/backend/simd.rs:6437-6743, the dequantize-then-dot
 * references of cera/src/backend/simd.rs:7113-7213, and the routing cases of
 * cera/src/model/lfm2.rs:3619-3720.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the cera repository root).
 */
#ifndef CERA_ORACLE_H
#define CERA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML tensor type ids (cera/src/convert/writer.rs:23-37). */
enum {
    CERA_T_F32 = 0,
    CERA_T_F16 = 1,
    CERA_T_Q4_0 = 2,
    CERA_T_Q4_1 = 3,
    CERA_T_Q8_0 = 8,
    CERA_T_Q4_K = 12,
    CERA_T_Q5_K = 13,
    CERA_T_Q6_K = 14,
    CERA_T_BF16 = 30
};

/* cera/src/tensor.rs:3-62 (DType::block_size / block_bytes). */
int cera_oracle_block_elems(int type);
int cera_oracle_block_bytes(int type);
size_t cera_oracle_row_bytes(int type, size_t k);

/* cera/src/quant.rs:48-73, 117-164, 91-100. */
float cera_oracle_f16_to_f32(uint16_t bits);
uint16_t cera_oracle_f32_to_f16(float v);
float cera_oracle_bf16_to_f32(uint16_t bits);

/* cera/src/quant.rs:364-376, 422-435, 494-501, 610-670, 836-870, 735-767. */
int cera_oracle_dequantize_row(int type, const uint8_t *src, size_t k, float *dst);

/* Weight quantizers, cera/src/convert/quantize.rs:344-387 (Q8_0), 523-570
 * (Q4_0), 719-846 (Q4_K), 851-988 (Q5_K), 993-1094 (Q6_K).  Q4_1 has no
 * quantizer in the reference; it follows ggml's published quantize_row_q4_1_ref. */
int cera_oracle_quantize_weights(int type, const float *in, size_t n, uint8_t *out);

/* Q8_0 activation quantizer, cera/src/backend/cpu.rs:942-958.  SoA output:
 * scales[k/32] (f32 holding an f16-representable value) and quants[k]. */
void cera_oracle_quantize_q8_0(const float *x, size_t k, float *scales, int8_t *quants);
/* cera/src/model/transformer.rs:865-946: mat is [dim x n] with stride n
 * (column j = token j); output column-major scales[n][dim/32], quants[n][dim]. */
void cera_oracle_quantize_columns(const float *mat, size_t dim, size_t n, float *scales,
                                  int8_t *quants);

/* Canonical per-32-block integer sums of one weight row against one Q8_0
 * activation column.  For every 32-element activation block b of the row:
 *   u[2b], u[2b+1] : sum of q*a over elements 0..15 and 16..31 of the block
 *                    (q is the weight quant as the kernels see it: Q4_0 q-8,
 *                     Q8_0 signed, Q4_1/Q4_K/Q5_K unsigned, Q6_K unsigned 0..63)
 *   a[2b], a[2b+1] : sum of the activation quants over the same halves
 * (cera/src/backend/simd.rs:6611-6620, 5651-5684, 5818-5827, 6042-6061). */
int cera_oracle_block_sums(int type, const uint8_t *row, size_t k, const int8_t *aq, int32_t *u,
                           int32_t *a);

/* out[m x n] (row-major, row = out-feature) = W[m x k] * X, X given as Q8_0
 * columns.  Arithmetic follows the x86 int8 tier lane for lane
 * (cera/src/backend/simd.rs:4593-4637 Q4_0/Q8_0, 5693-5878 Q4_K, 5893-5976 Q4_1,
 * 5988-6195 Q6_K; the AVX2 and AVX-512-VNNI tiers are bit-identical by the
 * reference's own tests).  n==1 takes the decode fast path of the K-quant kernels.
 * Q5_K has no such kernel in the reference: type Q5_K here is the Q4_K formula
 * with 5-bit quants (an extension, not pinned by any reference test). */
int cera_oracle_gemm_preq(int type, const uint8_t *w, const float *b_scales, const int8_t *b_quants,
                          float *out, size_t m, size_t n, size_t k);

/* cera/src/backend/cpu.rs:2360-2474 (x86 arms): quantize x, then the int8
 * kernel; Q5_K takes the f32-activation scalar dot (cpu.rs:1830-1854,
 * quant.rs:892-937); F32/F16/BF16 rows are plain f32 dots. */
int cera_oracle_gemv(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k);

/* cera/src/backend/cpu.rs:2479-2496, 2504-2544, 2570-2575, 2617-2633. */
void cera_oracle_rmsnorm(float *x, const float *weight, size_t n, float eps);
float cera_oracle_expf(float x);
void cera_oracle_silu_mul(float *gate, const float *up, size_t n);
void cera_oracle_softmax(float *x, size_t n);

/* cera/src/backend/cpu.rs:5091-5180 (NORM, adjacent pairs, rope_type 0) and
 * 5009-5054 (NEOX, pairs (i, i+hd/2), rope_type 1); freq_factors may be NULL. */
void cera_oracle_rope(float *q, float *k, size_t pos, size_t n_heads, size_t n_kv_heads,
                      size_t head_dim, float freq_base, const float *freq_factors, int rope_type);

/* cera/src/model/transformer.rs:1166-1305 with the scalar loops of
 * cera/src/backend/cpu.rs:3222-3363 / 3627-3769.  kv_f16 != 0: caches hold raw
 * half bits.  scores_scratch needs seq_len floats. */
void cera_oracle_decode_attention(const float *q, const void *k_cache, const void *v_cache,
                                  int kv_f16, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                  size_t seq_len, float scale, float *out, float *scores_scratch);

/* cera/src/backend/cpu.rs:4028-4241 (scalar tiled online softmax, causal).
 * q is [q_dim x n] stride n, caches are time-major f32 rows of kv_dim, out is
 * [n_heads][n][head_dim]. */
void cera_oracle_flash_attention_gqa(const float *q, const float *k_cache, const float *v_cache,
                                     size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t n,
                                     size_t start_pos, float scale, float *out);

/* cera/src/sampler.rs:20-30. */
uint32_t cera_oracle_argmax(const float *logits, size_t n);

/* cera/src/model/lfm2.rs:177-226.  probs are the unbiased gate values; bias may
 * be NULL.  Writes n_used expert ids and weights in selection order. */
void cera_oracle_select_experts(const float *probs, const float *bias, size_t n_expert,
                                size_t n_used, uint32_t *ids, float *weights);

/* Deterministic synthetic inputs.  value(i) = sigma * IH12(seed, i), where IH12
 * sums twelve 16-bit uniforms drawn from three splitmix64 outputs and is
 * centred and scaled in exact integer arithmetic before one f32 multiply, so
 * the CPU and CUDA generators agree bit for bit. */
void cera_oracle_synth_normal(float *out, size_t n, uint64_t seed, uint64_t offset, float sigma);

/* ---- dense llama-architecture model (cera/src/model/llama.rs:468-597,
 * 1585-1605; cera/src/model/transformer.rs:1313-1652) ---- */
typedef struct cera_oracle_model cera_oracle_model;

typedef struct {
    uint32_t n_layers, hidden_size, intermediate_size, n_heads, n_kv_heads, head_dim, vocab_size,
        max_seq_len;
    float rope_theta, rms_norm_eps;
    int32_t rope_type; /* 0 NORM, 1 NEOX */
    int32_t kv_f16;
    int32_t n_threads; /* rows of each GEMV are split over this many threads */
    /* ScalarMultipliers (cera/src/model/mod.rs:49-112), 0 = absent = identity: hidden *= embedding after the lookup;
     * block outputs *= residual before the residual add; attention replaces 1/sqrt(head_dim); logits *= 1/logit. */
    float embedding_scale, residual_scale, attention_scale, logit_scale;
} cera_oracle_config;

enum {
    CERA_ROLE_TOKEN_EMBD = 0,
    CERA_ROLE_OUTPUT_NORM = 1,
    CERA_ROLE_OUTPUT = 2,
    CERA_ROLE_ATTN_NORM = 3,
    CERA_ROLE_ATTN_Q = 4,
    CERA_ROLE_ATTN_K = 5,
    CERA_ROLE_ATTN_V = 6,
    CERA_ROLE_ATTN_OUTPUT = 7,
    CERA_ROLE_FFN_NORM = 8,
    CERA_ROLE_FFN_GATE = 9,
    CERA_ROLE_FFN_UP = 10,
    CERA_ROLE_FFN_DOWN = 11,
    CERA_ROLE_ROPE_FREQS = 12
};

cera_oracle_model *cera_oracle_model_create(const cera_oracle_config *cfg);
/* Borrowed, not copied: bytes must outlive the model. */
int cera_oracle_model_set_tensor(cera_oracle_model *m, int role, int layer, int type, size_t rows,
                                 size_t cols, const void *bytes);
/* One decode token at position pos == current seq_len; logits may be NULL. */
int cera_oracle_model_forward(cera_oracle_model *m, uint32_t token, size_t pos, float *logits);
/* y += B (scale * (A x)), cera/src/lora.rs:799-821 apply_decode */
void cera_oracle_lora_apply(size_t rank, size_t k, size_t d, float scale, const float *a, const float *b, const float *x,
                            float *y);
/* One LoRA pair (cera/src/lora.rs:794-821): target 0..6 = q, k, v, o, gate, up, down; A [rank x k], B [d x rank]. */
int cera_oracle_model_set_lora(cera_oracle_model *m, int target, int layer, size_t rank, size_t k, size_t d, float scale,
                               const float *a, const float *b);
void cera_oracle_model_truncate_kv(cera_oracle_model *m, size_t len);
/* cera/src/kv_cache.rs:1091-1320 (shift_kv_with_rope); -1 on the reference's assertion cases */
int cera_oracle_model_shift_kv(cera_oracle_model *m, size_t n_keep, size_t shift);
void cera_oracle_model_set_threads(cera_oracle_model *m, int n_threads);
size_t cera_oracle_model_seq_len(const cera_oracle_model *m);
/* Bytes of one layer's key (which = 0) or value (1) cache, rows [0, seq_len): what InferenceState::snapshot copies
 * (cera/src/kv_cache.rs:780-800).  Returns the byte count; copies at most cap bytes when out is not NULL. */
size_t cera_oracle_model_kv(const cera_oracle_model *m, size_t layer, int which, void *out, size_t cap);
/* Copies the last hidden-state snapshots recorded by forward (for drift
 * diagnosis): which = 0 final normed hidden. */
int cera_oracle_model_last_hidden(const cera_oracle_model *m, float *out);
void cera_oracle_model_free(cera_oracle_model *m);

/* ---- AVX2 + threads build of the same int8 kernels (the timed CPU baseline;
 * cera/src/backend/simd.rs:6306-6359 instantiation).  Bit-identical to
 * cera_oracle_gemm_preq by test. ---- */
int cera_cpu_has_avx2(void);
/* The AVX-512 VNNI tier (cera_cpu_vnni.cpp): same entry points with the _vnni suffix, bit-identical results. */
int cera_cpu_has_avx2_vnni(void);
void cera_oracle_set_cpu_tier(int tier); /* model forward: 0 scalar, 1 AVX2 (default), 2 AVX-512 VNNI */
int cera_cpu_gemm_preq_vnni(int type, const uint8_t *w, const float *b_scales, const int8_t *b_quants, float *out,
                            size_t m, size_t n, size_t k, int n_threads);
int cera_cpu_gemv_vnni(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k, int n_threads);
int cera_cpu_gemm_preq(int type, const uint8_t *w, const float *b_scales, const int8_t *b_quants,
                       float *out, size_t m, size_t n, size_t k, int n_threads);
int cera_cpu_gemv(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k,
                  int n_threads);

#ifdef __cplusplus
}
#endif
#endif
