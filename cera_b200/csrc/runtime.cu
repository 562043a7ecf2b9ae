// Status plumbing shared by every entry point: thread-local error text, CUDA
// error translation, launch counter, cached device properties.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace cera {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int32_t fail(int32_t code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int32_t check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return CERA_CUDA_OK;
    const int32_t code = e == cudaErrorMemoryAllocation ? CERA_CUDA_ERR_OOM : CERA_CUDA_ERR_CUDA;
    return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

bool pdl_enabled() {
    static const bool v = [] {
        const char *e = getenv("CERA_CUDA_PDL");
        return !(e && e[0] == '0');
    }();
    return v;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace cera

extern "C" {

const char *cera_cuda_last_error(void) { return cera::g_err; }

int32_t cera_cuda_device_count(int32_t *count) {
    if (!count) return cera::fail(CERA_CUDA_ERR_BAD_ARG, "count is null");
    int n = 0;
    CERA_CUDA_TRY(cudaGetDeviceCount(&n));
    *count = n;
    return CERA_CUDA_OK;
}

}  // extern "C"
