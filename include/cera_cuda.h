/* cera_cuda.h - C ABI of the B200 (sm_100a) CUDA device for cera's quantized
 * decode hot path: GGML-block quantized matmul against Q8_0 activations and
 * split-KV flash-decode GQA attention, plus the dense llama-architecture model
 * wired from them.
 *
 * This is the boundary a `--device cuda` backend of cera binds: plain pointers
 * and sizes, no C++ or torch types.  Every entry point returns an int32 status
 * (CERA_CUDA_OK == 0); cera_cuda_last_error() gives the text for the calling
 * thread.  Nothing here falls back to the CPU: with no usable CUDA device every
 * call fails with CERA_CUDA_ERR_CUDA.
 *
 * Conventions (cera's own, cera/src/backend/cpu.rs:1423): a weight matrix is
 * W[m x k], m = out-features (rows), k = in-features; a batch is n activation
 * columns (tokens); out is [m x n] row-major.  Pointers named *_dev are device
 * pointers on the current device; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  Operator-level calls are asynchronous
 * on `stream`; model-level calls take host buffers and return when the result
 * is on the host.
 */
#ifndef CERA_CUDA_H
#define CERA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define CERA_API __declspec(dllexport)
#else
#define CERA_API __attribute__((visibility("default")))
#endif

enum {
    CERA_CUDA_OK = 0,
    CERA_CUDA_ERR_BAD_ARG = 1,     /* extent / alignment / null contract violated   */
    CERA_CUDA_ERR_UNSUPPORTED = 2, /* (dtype, role) pair with no kernel: loud, never
                                      a silent fallback (cera/src/model/transformer.rs:607-633) */
    CERA_CUDA_ERR_OOM = 3,
    CERA_CUDA_ERR_CUDA = 4, /* driver / runtime error, text in last_error */
    CERA_CUDA_ERR_PEER = 5, /* peer-memory set-up between tensor- / expert-parallel ranks failed
                               (IPC handle, peer access); the library makes no NCCL call */
    CERA_CUDA_ERR_TIMEOUT = 6, /* a bounded device-side wait ran out */
    CERA_CUDA_ERR_STATE = 7    /* call order violated (e.g. pos != seq_len) */
};

/* GGML tensor type ids as stored in GGUF (cera/src/convert/writer.rs:23-37). */
enum {
    CERA_TYPE_F32 = 0,
    CERA_TYPE_F16 = 1,
    CERA_TYPE_Q4_0 = 2,
    CERA_TYPE_Q4_1 = 3,
    CERA_TYPE_Q8_0 = 8,
    CERA_TYPE_Q4_K = 12,
    CERA_TYPE_Q5_K = 13,
    CERA_TYPE_Q6_K = 14,
    CERA_TYPE_BF16 = 30
};

CERA_API const char *cera_cuda_last_error(void);
/* Device-side health word of the current device: 0 when no bounded wait inside a kernel has ever
 * run out (then the call returns CERA_CUDA_OK), else CERA_CUDA_ERR_TIMEOUT with the bits in
 * *status_out.  The counterpart of the reference's "a declined kernel must be loud" rule
 * (cera/src/model/transformer.rs:790-820) for kernels that wait on hardware barriers. */
CERA_API int32_t cera_cuda_kernel_status(uint32_t *status_out);
CERA_API int32_t cera_cuda_device_count(int32_t *count);

/* ------------------------------------------------------------------------ */
/* Weights.  Replaces the (WeightRef, mmap bytes) pair a CPU GEMV receives   */
/* (cera/src/model/transformer.rs:127-231, gpu_weight_source.rs:40-118).     */
/* `bytes` is the raw GGUF block data of an [m x k] tensor, host or device    */
/* memory; it is copied (and re-laid out into 16-byte aligned planes) before  */
/* the call returns.                                                          */
typedef struct cera_cuda_weight cera_cuda_weight;

CERA_API int32_t cera_cuda_weight_create(int32_t ggml_type, size_t m, size_t k, const void *bytes,
                                         size_t nbytes, cera_cuda_weight **out);
CERA_API void cera_cuda_weight_free(cera_cuda_weight *w);
/* Optional, for weights that will see many-column GEMMs (cera_cuda_gemm_preq with more than 32 columns; the reference
 * reaches that path through quantized_matmul_preq, cera/src/model/transformer.rs:790-820): builds a device-resident f16
 * operand image of a K-quant weight (k a multiple of 256) for the tensor-core kernels: about 2.3 extra bytes per weight
 * for Q4_K / Q5_K, 4 for Q6_K (whose products of scale and quant need two f16 operands).  *has_image (optional) = 1
 * when the weight now holds one; 0 when the type or shape is not those kernels', the device has no room, or
 * CERA_CUDA_TC_IMAGE=0 - Q4_K / Q5_K GEMMs then convert the quantized bytes on the fly and Q6_K runs the warp-level
 * kernel, same results within the path's tolerance.  A model (cera_cuda_model_*) prepares its own layer weights at its
 * first batched prompt.  Not thread-safe against concurrent calls on the same weight. */
CERA_API int32_t cera_cuda_weight_prepare_gemm(cera_cuda_weight *w, int32_t *has_image);
CERA_API int32_t cera_cuda_weight_info(const cera_cuda_weight *w, int32_t *ggml_type, size_t *m,
                                       size_t *k, size_t *device_bytes);

/* cera/src/quant.rs:321-356 dequantize_*_matrix, rows [row0, row0+nrows):
 * out_dev[nrows x k] f32, bit-identical to the reference's dequantizers. */
CERA_API int32_t cera_cuda_dequantize_rows(const cera_cuda_weight *w, size_t row0, size_t nrows,
                                           float *out_dev, void *stream);

/* ------------------------------------------------------------------------ */
/* Q8_0 activation quantizer (cera/src/backend/cpu.rs:942-1041).              */
/* x_dev: n columns, column j at x_dev + j*k (contiguous).  Outputs are the   */
/* reference's SoA layout (cera/src/model/transformer.rs:857-860):            */
/* scales_dev[n][k/32] f32, quants_dev[n][k] i8.  sums_dev (optional, may be  */
/* NULL) receives int16 sums of each 16 consecutive quants, [n][k/16]: the    */
/* kernels' form of cera/src/backend/simd.rs:5651-5684.                       */
CERA_API int32_t cera_cuda_quantize_q8_0(const float *x_dev, size_t k, size_t n, float *scales_dev,
                                         int8_t *quants_dev, int16_t *sums_dev, void *stream);
/* cera/src/model/transformer.rs:865-946: mat_dev is [dim x n] with row stride
 * n (token j = column j). */
CERA_API int32_t cera_cuda_quantize_columns(const float *mat_dev, size_t dim, size_t n,
                                            float *scales_dev, int8_t *quants_dev,
                                            int16_t *sums_dev, void *stream);

/* ------------------------------------------------------------------------ */
/* Matmul.                                                                    */
/* cera/src/model/transformer.rs:450-453 gemv -> cera/src/backend/cpu.rs:2360- */
/* 2474 gemv_dispatch: y[m] = W * x with x quantized to Q8_0 on the way in.    */
/* Uses the weight's own activation scratch: calls on one weight serialise on  */
/* the stream they are given.  Q5_K runs the Q8_0-activation extension unless  */
/* cera_cuda_gemv_q5k_f32 is used.                                             */
CERA_API int32_t cera_cuda_gemv(const cera_cuda_weight *w, const float *x_dev, float *y_dev,
                                void *stream);
/* cera/src/backend/cpu.rs:1830-1854: Q5_K against f32 activations, the only
 * Q5_K GEMV the reference has. */
CERA_API int32_t cera_cuda_gemv_q5k_f32(const cera_cuda_weight *w, const float *x_dev, float *y_dev,
                                        void *stream);
/* cera/src/model/transformer.rs:710-788 gemm_preq -> cpu.rs:1437-1557:
 * out_dev[m x n] = W * X for pre-quantized columns.  sums_dev as produced by
 * cera_cuda_quantize_q8_0 (required). */
CERA_API int32_t cera_cuda_gemm_preq(const cera_cuda_weight *w, const float *scales_dev,
                                     const int8_t *quants_dev, const int16_t *sums_dev,
                                     float *out_dev, size_t m, size_t n, size_t k, void *stream);
/* Parity probe: the integer sums the GEMV kernels form for one weight row and
 * one activation column, per 16-element half block: u_dev[k/16] = sum q*a (q as
 * the kernel sees it), a_dev[k/16] = sum a.  Exact, compared bit for bit. */
CERA_API int32_t cera_cuda_block_sums(const cera_cuda_weight *w, size_t row, const int8_t *quants_dev,
                                      int32_t *u_dev, int32_t *a_dev, void *stream);

/* ------------------------------------------------------------------------ */
/* Glue on the decode path.                                                   */
/* cera/src/backend/cpu.rs:2479-2496. out_dev may alias x_dev. */
CERA_API int32_t cera_cuda_rmsnorm(const float *x_dev, const float *weight_dev, size_t n, float eps,
                                   float *out_dev, void *stream);
/* cera/src/backend/cpu.rs:2570-2575: gate = silu(gate) * up. */
/* RMSNorm followed by the Q8_0 activation quantizer in one launch, as the decode step uses it before
 * every projection (cera/src/model/transformer.rs:1313-1345 runs cpu::rmsnorm then the quantizer of
 * cera/src/backend/cpu.rs:969-1041).  out_dev (f32, optional) receives the normed vector; scales /
 * quants / sums its Q8_0 form (n a multiple of 32). */
CERA_API int32_t cera_cuda_rmsnorm_q8_0(const float *x_dev, const float *weight_dev, size_t n, float eps,
                                        float *out_dev, float *scales_dev, int8_t *quants_dev,
                                        int16_t *sums_dev, void *stream);
CERA_API int32_t cera_cuda_silu_mul(float *gate_dev, const float *up_dev, size_t n, void *stream);
/* cera/src/backend/cpu.rs:5009-5180.  rope_type 0 = NORM (adjacent pairs,
 * optional freq_factors_dev[head_dim/2]), 1 = NEOX. */
CERA_API int32_t cera_cuda_rope(float *q_dev, float *k_dev, size_t pos, size_t n_heads,
                                size_t n_kv_heads, size_t head_dim, float freq_base,
                                const float *freq_factors_dev, int32_t rope_type, void *stream);

/* ------------------------------------------------------------------------ */
/* Flash-decode GQA attention (cera/src/model/transformer.rs:1249-1305).      */
/* Caches are time-major rows of n_kv_heads*head_dim, f32 (kv_f16 = 0) or raw  */
/* IEEE half bits (kv_f16 = 1), as cera/src/kv_cache.rs:201-221 keeps them.    */
/* One query token attends to rows [0, seq_len).  workspace_dev must hold      */
/* cera_cuda_decode_attention_workspace_bytes(...) bytes.                      */
/* Shapes: n_heads a multiple of n_kv_heads with at most 8 query heads per KV   */
/* head, head_dim a multiple of 32 up to 256: the result is then evaluated in   */
/* the reference's own f32 order (scores, plain softmax over all positions,     */
/* position-ordered value sums) and is bit-identical to it.  With the           */
/* environment variable CERA_CUDA_ATTN set the online-softmax kernels run       */
/* instead (groups of 4 or 8, head_dim 64 or 128; agreement within 1e-3         */
/* relative).  Any other shape: CERA_CUDA_ERR_UNSUPPORTED.                      */
CERA_API size_t cera_cuda_decode_attention_workspace_bytes(size_t n_heads, size_t head_dim,
                                                          size_t seq_len);
CERA_API int32_t cera_cuda_decode_attention(const float *q_dev, const void *k_cache_dev,
                                            const void *v_cache_dev, int32_t kv_f16, size_t n_heads,
                                            size_t n_kv_heads, size_t head_dim, size_t seq_len,
                                            float scale, float *out_dev, void *workspace_dev,
                                            size_t workspace_bytes, void *stream);

/* Causal attention of n prompt tokens (cera/src/backend/cpu.rs:4028-4241 flash_attention_gqa_cpu):
 * query j sits at position start_pos + j and attends to cache rows [0, start_pos + j].  q_dev and
 * out_dev are token-major [n][n_heads*head_dim]; the caches already hold rows up to start_pos + n. */
CERA_API int32_t cera_cuda_prefill_attention(const float *q_dev, const void *k_cache_dev,
                                             const void *v_cache_dev, int32_t kv_f16, size_t n_heads,
                                             size_t n_kv_heads, size_t head_dim, size_t n,
                                             size_t start_pos, float scale, float *out_dev, void *stream);

/* No counterpart in the reference.  The same attention for callers that cannot allocate device
 * memory (an embedding engine that owns the device heap, a thread on which allocation is forbidden,
 * a process with a frozen memory budget): the split-KV workspace is a fixed 2.1 MB array inside the
 * library, held by every GPU that loads it.  Limits: n_heads <= 64, head_dim <= 128; larger shapes
 * are rejected with CERA_CUDA_ERR_BAD_ARG.  The call allocates nothing.  The first call on each
 * device looks up the array's device address (cudaGetSymbolAddress, with that device current), so
 * make that first call before starting any stream capture.  All calls on a device share the array:
 * two calls that overlap on the GPU (different streams) race on it; calls on one stream do not.
 * The device that owns `stream` (and the buffers) must be the current device of the calling thread:
 * the array's address is looked up for the current device. */
CERA_API int32_t cera_cuda_decode_attention_noalloc(const float *q_dev, const void *k_cache_dev,
                                                    const void *v_cache_dev, int32_t kv_f16,
                                                    size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                                    size_t seq_len, float scale, float *out_dev,
                                                    void *stream);

/* ------------------------------------------------------------------------ */
/* Synthetic inputs for benchmarks and tests (the reference's counterpart is   */
/* its converter, cera/src/convert/quantize.rs:254-343 quantize_tensor_data).  */
/* out_dev[i] = sigma * IH12(seed, offset+i): twelve 16-bit uniforms from three */
/* splitmix64 draws, centred and scaled in integer arithmetic.                  */
CERA_API int32_t cera_cuda_synth_normal(float *out_dev, size_t n, uint64_t seed, uint64_t offset,
                                        float sigma, void *stream);
/* f32 -> GGML blocks with the reference's quantizer rules
 * (cera/src/convert/quantize.rs:344-387, 523-570, 719-1094). */
CERA_API int32_t cera_cuda_quantize_weights(int32_t ggml_type, const float *in_dev, size_t n,
                                            void *out_dev, void *stream);

/* ------------------------------------------------------------------------ */
/* Model: the object behind `Box<dyn Model>` for --device cuda                 */
/* (cera/src/model/mod.rs:200-606; config mirrors ModelConfig, mod.rs:117-145). */
typedef struct cera_cuda_model cera_cuda_model;

typedef struct {
    uint32_t n_layers;
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    uint32_t vocab_size;
    uint32_t max_seq_len;
    float rope_theta;
    float rms_norm_eps;
    int32_t rope_type; /* 0 NORM (llama), 1 NEOX */
    int32_t kv_f16;    /* 0: f32 KV (the CPU default), 1: f16 KV (KvCompression::F16) */
    int32_t device;    /* CUDA ordinal */
    int32_t reserved;
    /* ScalarMultipliers (Granite 3.x; cera/src/model/mod.rs:49-112).  0 = absent = identity, so a zeroed tail
     * is every other architecture.  embedding: hidden *= s after the token lookup (llama.rs:1544-1546);
     * residual: each attention / FFN block output *= s before its residual add (llama.rs:515-521, 543-549);
     * attention: softmax scale that REPLACES 1/sqrt(head_dim) (llama.rs:462); logit: logits *= 1/s
     * (llama.rs:591-594).  residual != 1 on a tensor-parallel model: CERA_CUDA_ERR_UNSUPPORTED. */
    float embedding_scale;
    float residual_scale;
    float attention_scale;
    float logit_scale;
} cera_cuda_config;

/* Tensor roles: the GGUF names a llama-architecture loader resolves
 * (cera/src/model/llama.rs:158-450). */
enum {
    CERA_ROLE_TOKEN_EMBD = 0,  /* token_embd.weight            */
    CERA_ROLE_OUTPUT_NORM = 1, /* output_norm.weight (F32)      */
    CERA_ROLE_OUTPUT = 2,      /* output.weight (optional: tied) */
    CERA_ROLE_ATTN_NORM = 3,   /* blk.N.attn_norm.weight (F32)   */
    CERA_ROLE_ATTN_Q = 4,
    CERA_ROLE_ATTN_K = 5,
    CERA_ROLE_ATTN_V = 6,
    CERA_ROLE_ATTN_OUTPUT = 7,
    CERA_ROLE_FFN_NORM = 8, /* blk.N.ffn_norm.weight (F32) */
    CERA_ROLE_FFN_GATE = 9,
    CERA_ROLE_FFN_UP = 10,
    CERA_ROLE_FFN_DOWN = 11,
    CERA_ROLE_ROPE_FREQS = 12 /* rope_freqs.weight (F32, optional) */
};

CERA_API int32_t cera_cuda_model_create(const cera_cuda_config *cfg, cera_cuda_model **out);
/* Tensor parallelism over output rows, the axis the reference itself parallelises
 * (cera/src/backend/cpu.rs:380-391, RowPool): this model becomes rank `rank` of `size` (<= 8)
 * cooperating models, one process and one GPU each.  Call before the first add_tensor; add_tensor
 * still receives every tensor in full (each rank's loader has the same mmap,
 * cera/src/model/gpu_weight_source.rs:40-118).  The feed-forward matrices (gate, up, down) and the
 * LM head keep rows [rank*m/size, (rank+1)*m/size); the attention block (q / k / v, KV cache,
 * o-proj) stays whole on every rank, since splitting its latency-bound launches costs more in
 * exchanges than it saves.  Needs n_kv_heads, hidden_size, vocab_size divisible by size and
 * intermediate_size by 32*size.  Per-row arithmetic is unchanged, so logits and greedy streams do
 * not depend on size. */
CERA_API int32_t cera_cuda_model_set_tp(cera_cuda_model *m, uint32_t rank, uint32_t size);
/* GpuWeightSource::weight_bytes (cera/src/model/gpu_weight_source.rs:40-118):
 * bytes are borrowed for the call only (host or device memory). */
CERA_API int32_t cera_cuda_model_add_tensor(cera_cuda_model *m, int32_t role, int32_t layer,
                                            int32_t ggml_type, size_t rows, size_t cols,
                                            const void *bytes, size_t nbytes);
/* Checks every required tensor is present, allocates KV and scratch, and
 * records the decode step.  Must precede the first forward. */
CERA_API int32_t cera_cuda_model_finalize(cera_cuda_model *m);
/* After finalize on a tensor-parallel model: a 64-byte handle (CUDA IPC) of this rank's
 * exchange region.  The host gathers the handles of all ranks in rank order (any transport:
 * the Python mirror uses torch.distributed) and gives every rank the whole list; the entry of
 * the rank itself is ignored.  Every forward call must then be made by all ranks with the same
 * arguments; a rank whose peers do not arrive within CERA_CUDA_TP_TIMEOUT_MS (default 5000)
 * returns CERA_CUDA_ERR_TIMEOUT from that call.  No counterpart in the reference, whose
 * backends are single-device. */
CERA_API int32_t cera_cuda_model_tp_handle(cera_cuda_model *m, void *handle_out, size_t handle_bytes);
CERA_API int32_t cera_cuda_model_tp_connect(cera_cuda_model *m, const void *handles, size_t n_handles);
/* One exchange on the current device against a peer buffer that nothing signals, with a wait
 * budget of timeout_ms (1..2000): *status_out receives the word the kernel leaves
 * (0x80000000 | peer << 24 | slot + 1; slot 3, peer 1 here), elapsed_ms the kernel time. */
CERA_API int32_t cera_cuda_tp_wait_selftest(uint32_t timeout_ms, uint32_t *status_out, float *elapsed_ms);
/* Model::forward (mod.rs:202): one token at pos == seq_len; logits_out[vocab]
 * on the host. */
CERA_API int32_t cera_cuda_forward(cera_cuda_model *m, uint32_t token, size_t pos,
                                   float *logits_out);
/* Model::forward_greedy (mod.rs:494-497): argmax on the device, first maximum
 * wins (cera/src/sampler.rs:20-30); 4 bytes come back. */
CERA_API int32_t cera_cuda_forward_greedy(cera_cuda_model *m, uint32_t token, size_t pos,
                                          uint32_t *token_out);
/* The greedy loop of Session::generate (cera/src/session.rs:1788-2310, which calls
 * forward_greedy once per token at 2233) kept on the device: n tokens are decoded
 * back to back, each argmax feeding the next step without a host round trip.
 * tokens_out[n] on the host; device_ms (optional) = CUDA-event time of the n steps. */
CERA_API int32_t cera_cuda_generate_greedy(cera_cuda_model *m, uint32_t first_token, size_t start_pos,
                                           size_t n, uint32_t *tokens_out, float *device_ms);
/* Model::forward_prefill (cera/src/model/llama.rs:1607-1649): start_pos must
 * equal seq_len; logits of the last token (may be NULL). */
CERA_API int32_t cera_cuda_forward_prefill(cera_cuda_model *m, const uint32_t *tokens, size_t n,
                                           size_t start_pos, float *logits_out);
/* Model::truncate_kv (mod.rs:251-283). */
CERA_API int32_t cera_cuda_truncate_kv(cera_cuda_model *m, size_t len);
/* LoRA adapters (cera/src/lora.rs; the reference carries them on InferenceState::lora and applies
 * them in forward_attn_block / forward_ffn_block, cera/src/model/transformer.rs:1383-1387, 1519-1528,
 * 1588-1605, 1642-1651): y = W x + scale * B (A x) on the f32 input of the projection, q/k/v before
 * RoPE, gate/up before the SwiGLU product.  target: 0 q, 1 k, 2 v, 3 attn_output, 4 ffn_gate,
 * 5 ffn_up, 6 ffn_down (the order of lora.rs:63-70); a is [rank x k], b is [d x rank], row-major F32,
 * host or device, copied; scale = alpha / rank.  While any pair is attached prompts are processed
 * with the decode step per token (the reference requires its batched form to equal the per-token form
 * bit for bit, lora.rs:830-844).  MoE targets and tensor-parallel models: CERA_CUDA_ERR_UNSUPPORTED /
 * not offered.  detach removes every pair. */
CERA_API int32_t cera_cuda_model_attach_lora(cera_cuda_model *m, int32_t target, int32_t layer, size_t rank,
                                             size_t k, size_t d, const float *a, const float *b, float scale);
CERA_API int32_t cera_cuda_model_detach_lora(cera_cuda_model *m);
/* Model::forward_prefill_logits_all (cera/src/model/mod.rs:507-533; the verifier side of speculative
 * decoding): like forward_prefill, but the logits of every position come back, logits_out[n][vocab]
 * on the host, token-major. */
CERA_API int32_t cera_cuda_forward_prefill_logits_all(cera_cuda_model *m, const uint32_t *tokens, size_t n,
                                                      size_t start_pos, float *logits_out);
/* Model::shift_kv (cera/src/model/llama.rs:1728-1738 -> InferenceState::shift_kv_with_rope,
 * cera/src/kv_cache.rs:1091-1320): drop cached positions [n_keep, n_keep + shift), move the rest down
 * and rotate every moved K head by R(-shift) with the model's RoPE layout and frequency factors; V
 * rows move unchanged; seq_len shrinks by shift.  shift == 0 or n_keep + shift > seq_len are errors
 * (the reference asserts). */
CERA_API int32_t cera_cuda_kv_shift(cera_cuda_model *m, size_t n_keep, size_t shift);
/* Model::snapshot / restore (cera/src/model/mod.rs:230-283): the cached positions [0, seq_len) of every
 * layer as host bytes, and back.  The layout is this library's own (a 32-byte header, then per layer the K
 * rows and the V rows in the cache's element type), not the reference's StateSnapshot: device backends
 * own their KV, and a snapshot is only ever restored into the model that made it or an identical one. */
CERA_API size_t cera_cuda_kv_snapshot_bytes(const cera_cuda_model *m);
CERA_API int32_t cera_cuda_kv_snapshot(cera_cuda_model *m, void *out, size_t out_bytes);
CERA_API int32_t cera_cuda_kv_restore(cera_cuda_model *m, const void *data, size_t bytes);
/* The same state in the shape of the reference's StateSnapshot (cera/src/kv_cache.rs:1379-1421: `seq_len` plus, per
 * attention layer, LayerSnapshot::Attention { k_data, v_data } - raw little-endian f32 rows - or ::AttentionF16 for an
 * f16 cache): one call per layer fills k_data and v_data with the layer's rows [0, seq_len), kv_dim elements each,
 * exactly the bytes InferenceState::snapshot takes from its key / value cache (kv_cache.rs:780-800).  bytes_each must
 * be cera_cuda_kv_layer_bytes(m).  restore_layer writes the rows back and sets seq_len (give every layer the same
 * value); the element width is the model's kv_f16 setting on both sides, as the reference's cross-mode gate demands. */
CERA_API size_t cera_cuda_kv_layer_bytes(const cera_cuda_model *m);
CERA_API int32_t cera_cuda_kv_snapshot_layer(cera_cuda_model *m, uint32_t layer, void *k_data, void *v_data, size_t bytes_each);
CERA_API int32_t cera_cuda_kv_restore_layer(cera_cuda_model *m, uint32_t layer, const void *k_data, const void *v_data,
                                            size_t bytes_each, size_t seq_len);
CERA_API size_t cera_cuda_seq_len(const cera_cuda_model *m);
/* Model::gpu_memory_bytes (mod.rs:500). */
CERA_API size_t cera_cuda_memory_bytes(const cera_cuda_model *m);
/* Final normed hidden state of the last forward, hidden_size floats on the
 * host (Model::hidden_states precedent; used for drift diagnosis). */
CERA_API int32_t cera_cuda_last_hidden(cera_cuda_model *m, float *out);
/* Kernels launched by this library on behalf of the model since creation. */
CERA_API uint64_t cera_cuda_launch_count(const cera_cuda_model *m);
CERA_API void cera_cuda_model_free(cera_cuda_model *m);

/* ------------------------------------------------------------------------ */
/* Routed feed-forward of an lfm2moe layer (cera/src/model/lfm2.rs:177-226 select_experts,
 * 673-715 route_experts, 735-901 forward_moe_ffn, 914-937 prefill_moe_ffn).
 *
 * gate_exps / up_exps are the stacked tensors blk.N.ffn_{gate,up}_exps.weight,
 * [n_expert][ff][hidden] raw GGUF blocks with expert stride ff rows; down_exps is
 * [n_expert][hidden][ff] (cera/src/model/gpu_weight_source.rs:179-257).  router is
 * blk.N.ffn_gate_inp.weight, F32 [n_expert][hidden]; exp_probs_b is blk.N.exp_probs_b.bias,
 * F32 [n_expert], or NULL for zero bias.  Pointers may be host or device; all are copied. */
typedef struct cera_cuda_moe cera_cuda_moe;
CERA_API int32_t cera_cuda_moe_create(uint32_t n_expert, uint32_t n_used, uint32_t hidden, uint32_t ff,
                                      int32_t ggml_type, const void *gate_exps, const void *up_exps,
                                      const void *down_exps, size_t gate_up_bytes, size_t down_bytes,
                                      const float *router, const float *exp_probs_b, size_t max_tokens,
                                      cera_cuda_moe **out);
/* x_dev and out_dev are token-major [n][hidden] f32 (the reference's prefill layout is the
 * transpose, hidden x n; its decode layout is n == 1).  softmax_gate == 0 is the reference's rule:
 * sigmoid probabilities, selection by probability + bias with ties to the lower index, weights =
 * unbiased probabilities of the selected experts over max(their sum, 2^-14).  softmax_gate != 0
 * replaces the sigmoid by a softmax over all experts and keeps the rest.  out = sum in selection
 * order of weight * expert FFN output; every expert projection is the int8 product against the
 * Q8_0 form of its input.  ids_out_dev / weights_out_dev (optional, [n][n_used]) receive the routing. */
CERA_API int32_t cera_cuda_moe_ffn(cera_cuda_moe *moe, const float *x_dev, size_t n, int32_t softmax_gate,
                                   float *out_dev, uint32_t *ids_out_dev, float *weights_out_dev,
                                   void *stream);
/* Expert parallelism, one process per GPU (no counterpart in the reference, which routes per token on
 * one device): this layer becomes rank ep_rank of ep_size.  It is still handed the whole stacked
 * tensors and keeps experts [ep_rank*n_expert/ep_size, (ep_rank+1)*n_expert/ep_size).  max_tokens
 * bounds the tokens THIS rank passes per call, max_total_tokens the tokens of all ranks together.
 * After creation exchange the 64-byte handles exactly as for a tensor-parallel model
 * (cera_cuda_moe_ep_handle -> gather in rank order -> cera_cuda_moe_ep_connect).  Every
 * cera_cuda_moe_ffn call is then collective: all ranks call it (n may differ per rank, 0 included);
 * tokens are dispatched to the ranks that own their experts and the results combined back, all by
 * peer stores from the kernels.  Outputs are bit-identical to the single-GPU layer.  A peer that does
 * not arrive within CERA_CUDA_TP_TIMEOUT_MS leaves a status word that cera_cuda_moe_ep_status
 * (call it after synchronising the stream) turns into CERA_CUDA_ERR_TIMEOUT.  If the ranks together
 * route more entries to one rank than max_total_tokens x n_used, the call stores nothing into any
 * peer, its output is undefined and cera_cuda_moe_ep_status returns CERA_CUDA_ERR_BAD_ARG. */
CERA_API int32_t cera_cuda_moe_create_ep(uint32_t n_expert, uint32_t n_used, uint32_t hidden, uint32_t ff,
                                         int32_t ggml_type, const void *gate_exps, const void *up_exps,
                                         const void *down_exps, size_t gate_up_bytes, size_t down_bytes,
                                         const float *router, const float *exp_probs_b, size_t max_tokens,
                                         uint32_t ep_rank, uint32_t ep_size, size_t max_total_tokens,
                                         cera_cuda_moe **out);
CERA_API int32_t cera_cuda_moe_ep_handle(cera_cuda_moe *moe, void *handle_out, size_t handle_bytes);
CERA_API int32_t cera_cuda_moe_ep_connect(cera_cuda_moe *moe, const void *handles, size_t n_handles);
CERA_API int32_t cera_cuda_moe_ep_status(cera_cuda_moe *moe, uint32_t *status_out);
CERA_API size_t cera_cuda_moe_memory_bytes(const cera_cuda_moe *moe);
CERA_API void cera_cuda_moe_free(cera_cuda_moe *moe);

#ifdef __cplusplus
}
#endif
#endif /* CERA_CUDA_H */
