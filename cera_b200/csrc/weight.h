// Host-side handle of a device-resident quantized matrix.
#pragma once

#include "common.cuh"

struct cera_cuda_weight {
    cera::WeightView v{};
    void *base = nullptr;   // one allocation holding every plane
    size_t bytes = 0;       // size of that allocation
    // Q8_0 activation scratch for one column of length k, used by cera_cuda_gemv.
    float *xs = nullptr;
    int8_t *xq = nullptr;
    int16_t *xsum = nullptr;
    int device = 0;
    // optional f16 operand image for the tcgen05 prefill GEMM (weight_prepare_tc); v.tc points into it
    void *tc_image = nullptr;
    size_t tc_bytes = 0;
};

namespace cera {
// Allocates planes and re-lays `bytes` (host or device, raw GGUF blocks) into them.
int32_t weight_upload(int32_t type, size_t m, size_t k, const void *bytes, size_t nbytes, bool with_scratch,
                      cera_cuda_weight **out);
int32_t weight_prepare_tc(cera_cuda_weight *w, bool *built);
}  // namespace cera
