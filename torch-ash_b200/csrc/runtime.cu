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

// Measurement aid: every thread reads one 16-byte word at a pseudo-random 64-byte-aligned place
// of a large buffer.  The rate it reaches (reads per second) is the ceiling for the library's
// probe and gather kernels, whose DRAM accesses are just as scattered: at that rate the memory
// is busy opening rows, whatever the number of bytes each access returns.
// READS independent reads per thread are issued back to back before any is consumed: if the rate
// rose with READS, the kernels that make one dependent access per thread would be latency-bound and
// could gain from more loads in flight; if it does not, the memory system itself is the limit.
template <bool FETCH64, int READS>
__global__ void __launch_bounds__(256) random_read_kernel(const uint4* __restrict__ buf, uint64_t granules, int64_t n,
                                                          uint32_t seed, unsigned long long* __restrict__ sink) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint4 v[READS];
#pragma unroll
    for (int r = 0; r < READS; ++r) {
        const int64_t i = t * READS + r;
        v[r] = make_uint4(0, 0, 0, 0);
        if (i >= n) continue;
        const uint64_t h = ((uint64_t)fmix32((uint32_t)i ^ seed) << 32) | fmix32((uint32_t)(i >> 32) + 0x9E3779B9u * (uint32_t)i + seed);
        const uint4* p = buf + (h % granules) * 4;
        if (FETCH64)
            asm volatile("ld.global.nc.L2::64B.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(p));
        else
            asm volatile("ld.global.nc.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(p));
    }
    unsigned acc = 0;
#pragma unroll
    for (int r = 0; r < READS; ++r) acc += (v[r].x ^ v[r].y ^ v[r].z ^ v[r].w) == 0x5A17C0DEu;
    if (acc) atomicAdd(sink, (unsigned long long)acc);  // keeps the loads alive
}

template <int READS>
static void launch_random_reads(const void* buffer, uint64_t granules, int64_t n_reads, int fetch_bytes, uint32_t seed,
                                void* sink_dev, cudaStream_t st) {
    const int64_t threads = (n_reads + READS - 1) / READS;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (fetch_bytes == 64)
        random_read_kernel<true, READS><<<grid, 256, 0, st>>>(static_cast<const uint4*>(buffer), granules, n_reads, seed,
                                                              static_cast<unsigned long long*>(sink_dev));
    else
        random_read_kernel<false, READS><<<grid, 256, 0, st>>>(static_cast<const uint4*>(buffer), granules, n_reads, seed,
                                                               static_cast<unsigned long long*>(sink_dev));
}

}  // namespace ashb

extern "C" {

int ashb_measure_random_reads_ilp(const void* buffer, int64_t bytes, int64_t n_reads, int fetch_bytes,
                                  int reads_per_thread, uint32_t seed, void* sink_dev, void* stream) {
    ASHB_REQUIRE(buffer != nullptr && sink_dev != nullptr, "null buffer");
    ASHB_REQUIRE(bytes >= 64 && n_reads >= 0, "bad sizes");
    ASHB_REQUIRE(fetch_bytes == 64 || fetch_bytes == 128, "fetch size must be 64 or 128");
    ASHB_REQUIRE(reads_per_thread == 1 || reads_per_thread == 2 || reads_per_thread == 4 || reads_per_thread == 8,
                 "reads per thread must be 1, 2, 4 or 8");
    ASHB_REQUIRE(((uintptr_t)buffer & 63) == 0, "buffer must be 64-byte aligned");
    if (n_reads == 0) return ASHB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint64_t granules = (uint64_t)bytes / 64;
    switch (reads_per_thread) {
        case 1: ashb::launch_random_reads<1>(buffer, granules, n_reads, fetch_bytes, seed, sink_dev, st); break;
        case 2: ashb::launch_random_reads<2>(buffer, granules, n_reads, fetch_bytes, seed, sink_dev, st); break;
        case 4: ashb::launch_random_reads<4>(buffer, granules, n_reads, fetch_bytes, seed, sink_dev, st); break;
        default: ashb::launch_random_reads<8>(buffer, granules, n_reads, fetch_bytes, seed, sink_dev, st); break;
    }
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_measure_random_reads(const void* buffer, int64_t bytes, int64_t n_reads, int fetch_bytes, uint32_t seed,
                              void* sink_dev, void* stream) {
    return ashb_measure_random_reads_ilp(buffer, bytes, n_reads, fetch_bytes, 1, seed, sink_dev, stream);
}

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
