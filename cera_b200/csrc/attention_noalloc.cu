// Flash-decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a plugin running inside an
// engine that owns the whole device heap and hands out no allocator, code on a latency-critical
// thread where an allocation (an implicit device synchronisation) is forbidden, or a process
// whose memory budget was fixed before the library was loaded.  cera_cuda_decode_attention needs
// a workspace for the per-split partial results; this variant keeps that workspace in a fixed
// array inside the library image instead, so the caller passes only inputs and outputs.
//
// The array is file-scope `static __device__`: every GPU that loads the library holds one copy
// (2.1 MB) until the process exits.  In host code its name is only a stand-in for the symbol, not
// a device address, so the address is looked up once per device with cudaGetSymbolAddress (with
// that device current) and it is that pointer the kernels receive.
#include <mutex>

#include "ops.h"

namespace cera {

namespace {

constexpr size_t NOALLOC_MAX_HEADS = 64;
constexpr size_t NOALLOC_MAX_HEAD_DIM = 128;
// One record of head_dim + 2 floats per (query head, split); the split count never exceeds 64.
constexpr size_t NOALLOC_WS_BYTES = NOALLOC_MAX_HEADS * 64 * (NOALLOC_MAX_HEAD_DIM + 2) * sizeof(float);

static __device__ __align__(256) unsigned char g_attention_scratch[NOALLOC_WS_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mu;
void *g_scratch_addr[MAX_DEVICES] = {};

// Device address of the scratch array on the current device; resolved on the first call per device.
int32_t scratch_for_current_device(void **out) {
    int dev = 0;
    CERA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention_noalloc: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        CERA_CUDA_TRY(cudaGetSymbolAddress(&p, g_attention_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return CERA_CUDA_OK;
}

}  // namespace
}  // namespace cera

using namespace cera;

extern "C" {

int32_t cera_cuda_decode_attention_noalloc(const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                           int32_t kv_f16, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                           size_t seq_len, float scale, float *out_dev, void *stream) {
    if (n_heads > NOALLOC_MAX_HEADS || head_dim > NOALLOC_MAX_HEAD_DIM)
        return fail(CERA_CUDA_ERR_BAD_ARG,
                    "decode_attention_noalloc: %zu heads x head_dim %zu exceeds the built-in scratch (at most %zu heads, "
                    "head_dim %zu); use cera_cuda_decode_attention with a caller workspace",
                    n_heads, head_dim, NOALLOC_MAX_HEADS, NOALLOC_MAX_HEAD_DIM);
    const size_t need = attn_workspace_bytes(n_heads, head_dim, seq_len);
    if (need > NOALLOC_WS_BYTES)
        return fail(CERA_CUDA_ERR_BAD_ARG, "decode_attention_noalloc: needs %zu scratch bytes, %zu are built in", need,
                    NOALLOC_WS_BYTES);
    void *ws = nullptr;
    CERA_TRY(scratch_for_current_device(&ws));
    // Every record the merge pass reads is written by the split pass of the same call, so nothing
    // has to be cleared even though the array keeps the previous call's contents.
    return launch_decode_attention(q_dev, k_cache_dev, v_cache_dev, kv_f16, n_heads, n_kv_heads, head_dim, seq_len, scale,
                                   out_dev, ws, NOALLOC_WS_BYTES, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

}  // extern "C"
