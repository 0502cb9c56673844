// Host-side runtime shared by every translation unit of libashb200: the
// per-thread error text and cached device properties.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace ashb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cached;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
            cached = n;
            cached_dev = dev;
        }
    }
    return cached;
}

}  // namespace ashb

extern "C" {

const char* ashb_last_error_string(void) { return ashb::g_error; }

int ashb_version(void) { return 1; }

int ashb_set_l2_fetch_granularity(int bytes) {
    ASHB_REQUIRE(bytes == 32 || bytes == 64 || bytes == 128, "granularity must be 32, 64 or 128 bytes");
    ASHB_CUDA_TRY(cudaDeviceSetLimit(cudaLimitMaxL2FetchGranularity, (size_t)bytes));
    return ASHB_OK;
}

int ashb_get_l2_fetch_granularity(int* bytes_out) {
    ASHB_REQUIRE(bytes_out != nullptr, "null output");
    size_t v = 0;
    ASHB_CUDA_TRY(cudaDeviceGetLimit(&v, cudaLimitMaxL2FetchGranularity));
    *bytes_out = (int)v;
    return ASHB_OK;
}

}  // extern "C"
