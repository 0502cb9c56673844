// Key routing for the key-hash-partitioned hash map (one process per GPU): groups a batch of
// packed int32 keys by owner rank so that one all-to-all(v) can ship every group to its owner.
// The reference is single-GPU and has no counterpart.
//
//   count    per-CTA histogram of owners in shared memory, one atomic per (CTA, rank)
//   scatter  each warp groups its lanes by owner (__match_any_sync), the groups of a CTA meet in
//            shared memory and one atomic per (CTA, rank) reserves their output range; rows land
//            grouped by owner, and `perm` remembers where each came from so that answers can be
//            put back in caller order.
#include "common.cuh"

namespace ashb {

constexpr int kMaxWorld = 64;

// Owner rank of a key: multiplicative mix of the columns, independent of the slot hash of the
// local tables.  Must stay bit-identical to ash.distributed.owner_of (int64 arithmetic with
// wrap-around, arithmetic right shifts, non-negative remainder).
__device__ __forceinline__ int owner_of_key(const int32_t* k, int dim, int world) {
    const unsigned long long primes[4] = {73856093ull, 19349663ull, 83492791ull, 2654435761ull};
    long long h = 0;
    for (int d = 0; d < dim; ++d) h ^= (long long)((unsigned long long)(long long)k[d] * primes[d & 3]);
    h = (long long)((unsigned long long)(h ^ (h >> 15)) * 0x2C1B3C6Dull);
    h ^= h >> 12;
    long long r = h % world;
    return (int)(r < 0 ? r + world : r);
}

__global__ void __launch_bounds__(256) route_count_kernel(const int32_t* __restrict__ keys, int64_t n, int dim,
                                                          int world, unsigned long long* __restrict__ counts) {
    __shared__ unsigned int hist[kMaxWorld];
    for (int r = threadIdx.x; r < world; r += blockDim.x) hist[r] = 0;
    __syncthreads();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        atomicAdd(&hist[owner_of_key(keys + i * dim, dim, world)], 1u);
    __syncthreads();
    for (int r = threadIdx.x; r < world; r += blockDim.x)
        if (hist[r]) atomicAdd(&counts[r], (unsigned long long)hist[r]);
}

struct RouteOffsets {
    long long start[kMaxWorld];
};

__global__ void __launch_bounds__(256) route_scatter_kernel(const int32_t* __restrict__ keys, int64_t n, int dim,
                                                            int world, RouteOffsets offsets,
                                                            unsigned long long* __restrict__ cursors,
                                                            int32_t* __restrict__ keys_out,
                                                            int64_t* __restrict__ perm_out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const bool live = i < n;
    // lanes without a key take a negative owner of their own, so that they match nobody
    const int owner = live ? owner_of_key(keys + i * dim, dim, world) : -1 - lane;
    // output ranges are reserved per CTA: the warps' per-owner groups meet in shared memory and one
    // global atomic per (CTA, owner) follows
    __shared__ unsigned int cta_count[kMaxWorld];
    __shared__ unsigned long long cta_base[kMaxWorld];
    for (int o = threadIdx.x; o < world; o += blockDim.x) cta_count[o] = 0;
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, owner);
    const int leader = __ffs(peers) - 1;
    unsigned int within = 0;
    if (live && lane == leader) within = atomicAdd(&cta_count[owner], (unsigned)__popc(peers));
    within = __shfl_sync(0xffffffffu, within, leader);
    __syncthreads();
    for (int o = threadIdx.x; o < world; o += blockDim.x)
        cta_base[o] = cta_count[o] ? atomicAdd(&cursors[o], (unsigned long long)cta_count[o]) : 0ull;
    __syncthreads();
    if (!live) return;
    const int64_t pos = offsets.start[owner] + (int64_t)cta_base[owner] + within + __popc(peers & lanemask_lt());
    for (int d = 0; d < dim; ++d) keys_out[pos * dim + d] = keys[i * dim + d];
    perm_out[pos] = i;
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_route_by_owner(const int32_t* keys, int64_t n, int key_dim, int world, int32_t* keys_out,
                        int64_t* perm_out, int64_t* counts_host, void* scratch_dev, void* stream) {
    ASHB_REQUIRE(key_dim >= 1 && key_dim <= 4 && world >= 1 && world <= kMaxWorld, "key_dim 1..4 and world 1..%d",
                 kMaxWorld);
    ASHB_REQUIRE(n >= 0 && counts_host != nullptr && scratch_dev != nullptr, "bad count or null scratch");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long* counts = static_cast<unsigned long long*>(scratch_dev);
    unsigned long long* cursors = counts + kMaxWorld;
    ASHB_CUDA_TRY(cudaMemsetAsync(scratch_dev, 0, 2 * kMaxWorld * sizeof(unsigned long long), st));
    for (int r = 0; r < world; ++r) counts_host[r] = 0;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(keys && keys_out && perm_out, "null buffer");
    route_count_kernel<<<wave_grid(n, 256, 8), 256, 0, st>>>(keys, n, key_dim, world, counts);
    ASHB_LAUNCH_CHECK();
    unsigned long long host_counts[kMaxWorld];
    ASHB_CUDA_TRY(cudaMemcpyAsync(host_counts, counts, world * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    RouteOffsets off{};
    long long run = 0;
    for (int r = 0; r < world; ++r) {
        off.start[r] = run;
        run += (long long)host_counts[r];
        counts_host[r] = (int64_t)host_counts[r];
    }
    route_scatter_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(keys, n, key_dim, world, off, cursors, keys_out,
                                                                       perm_out);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
