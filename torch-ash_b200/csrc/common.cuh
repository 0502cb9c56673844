// Shared host/device helpers of libashb200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "ashb200.h"

namespace ashb {

// ---- host-side error plumbing -------------------------------------------------
void set_error(const char* fmt, ...);

#define ASHB_CUDA_TRY(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess) {                                                         \
            ::ashb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                              __FILE__, __LINE__);                                       \
            return ASHB_ERR_CUDA;                                                        \
        }                                                                                \
    } while (0)

#define ASHB_REQUIRE(cond, ...)               \
    do {                                      \
        if (!(cond)) {                        \
            ::ashb::set_error(__VA_ARGS__);   \
            return ASHB_ERR_INVALID;          \
        }                                     \
    } while (0)

// Launch check: catches configuration errors without synchronising.
#define ASHB_LAUNCH_CHECK() ASHB_CUDA_TRY(cudaGetLastError())

// Number of SMs of the current device (148 on B200); cached per process.
int sm_count();

// Grid size for a grid-stride kernel: a whole number of waves of resident CTAs.
inline unsigned wave_grid(int64_t work_items, int threads, int ctas_per_sm) {
    int64_t need = (work_items + threads - 1) / threads;
    int64_t wave = (int64_t)sm_count() * ctas_per_sm;
    if (need < 1) need = 1;
    if (need <= wave) return (unsigned)need;
    int64_t waves = (need + wave - 1) / wave;
    if (waves > 8) waves = 8;
    return (unsigned)(waves * wave);
}

// ---- device helpers -----------------------------------------------------------
__device__ __forceinline__ uint32_t fmix32(uint32_t h) {
    h ^= h >> 16;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    h *= 0xC2B2AE35u;
    h ^= h >> 16;
    return h;
}

// Slot hash of a packed int32 key (unused columns are zero).
__device__ __forceinline__ uint32_t hash_key(int k0, int k1, int k2, int k3) {
    uint32_t h = fmix32((uint32_t)k0 * 0x9E3779B1u + 0x7F4A7C15u);
    h = fmix32(h ^ ((uint32_t)k1 * 0x85EBCA77u));
    h = fmix32(h ^ ((uint32_t)k2 * 0xC2B2AE3Du));
    if (k3 != 0) h = fmix32(h ^ ((uint32_t)k3 * 0x27D4EB2Fu));
    return h;
}

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

}  // namespace ashb
