// Ray sampler over the hashed block structure (sm_100a): near/far estimation and
// two-pass interval sampling with one hash probe per step.  Semantics follow
// ash/src/sampler.cu:7-294; every length is in cell units.
//
// Arithmetic contract (so that the block a sample falls in is decided the same
// way everywhere): position = fma(t, d, o) per component in float32, block =
// floor(position * (float)(1.0 / grid2cell)).
//
// One thread marches one ray; the loops are data dependent and bounded by
// (t_max - t_min) / step.  The table of a scene (<= a few hundred thousand
// blocks x 16 bytes) stays L2 resident.
#include "sampler.cuh"

namespace ashb {

// ash/src/sampler.cu:7-71
__global__ void __launch_bounds__(128) ray_near_far_kernel(Table16 t, const float* __restrict__ ray_o,
                                                           const float* __restrict__ ray_d,
                                                           const float* __restrict__ bbox_min,
                                                           const float* __restrict__ bbox_max,
                                                           float* __restrict__ nears, float* __restrict__ fars,
                                                           float t_min, float t_max, float grid2cell, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float lo[3] = {bbox_min[0], bbox_min[1], bbox_min[2]};
    const float hi[3] = {bbox_max[0], bbox_max[1], bbox_max[2]};
    const float o[3] = {ray_o[3 * i], ray_o[3 * i + 1], ray_o[3 * i + 2]};
    const float d[3] = {ray_d[3 * i], ray_d[3 * i + 1], ray_d[3 * i + 2]};
    float near, far;
    march_near_far(t, o, d, lo, hi, t_min, t_max, grid2cell, near, far);
    nears[i] = near;
    fars[i] = far;
}

// ash/src/sampler.cu:123-215.  FILL = false: count samples per ray; FILL = true:
// write (ray index, t_near, t_far) at the ray's segment of the inclusive prefix sum.
template <bool FILL>
__global__ void __launch_bounds__(128) ray_sample_kernel(Table16 t, const float* __restrict__ ray_o,
                                                         const float* __restrict__ ray_d,
                                                         const float* __restrict__ ray_nears,
                                                         const float* __restrict__ ray_fars,
                                                         int64_t* __restrict__ counts,
                                                         const int64_t* __restrict__ prefix,
                                                         int64_t* __restrict__ ray_indices,
                                                         float* __restrict__ t_nears, float* __restrict__ t_fars,
                                                         int64_t max_samples, float grid2cell, int64_t n,
                                                         uint32_t* status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float o[3] = {ray_o[3 * i], ray_o[3 * i + 1], ray_o[3 * i + 2]};
    const float d[3] = {ray_d[3 * i], ray_d[3 * i + 1], ray_d[3 * i + 2]};
    const float ray_near = ray_nears[i], ray_far = ray_fars[i];
    const float cell2grid = (float)(1.0 / (double)grid2cell);
    const float cell_step = sample_cell_step(ray_near, ray_far, max_samples);
    const float grid_step = cell_step * grid2cell;
    int64_t local = 0;
    int64_t start = 0, end = 0;
    if (FILL) {
        start = i == 0 ? 0 : prefix[i - 1];
        end = prefix[i];
    }
    march_intervals(t, o, d, ray_near, ray_far, cell_step, grid_step, cell2grid, [&](float seg_near, float seg_far) {
        if (FILL && start + local < end) {
            ray_indices[start + local] = i;
            t_nears[start + local] = seg_near;
            t_fars[start + local] = seg_far;
        }
        ++local;
    });
    if (!FILL) counts[i] = local;
    // The two passes must agree; a mismatch means the table changed in between.
    if (FILL && start + local != end) atomicOr(status, ASHB_STATUS_PROBE);
}

}  // namespace ashb

using namespace ashb;

static int check_sampler_map(ashb_map* m) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    // ash/src/sampler.cu:89-99: ray sampling is for 3-D int maps only
    ASHB_REQUIRE(m->key_dim == 3, "hashmap is not a GPU hashmap of type <int, 3>, ray sample not supported");
    return ASHB_OK;
}

extern "C" {

int ashb_ray_find_near_far(ashb_map* m, const float* ray_o, const float* ray_d, const float* bbox_min,
                           const float* bbox_max, float* nears, float* fars, float t_min, float t_max,
                           float t_step, float grid2cell, int64_t n, void* stream) {
    (void)t_step;  // accepted and unused, as in ash/src/sampler.cu:7-71
    if (int rc = check_sampler_map(m)) return rc;
    ASHB_REQUIRE(n >= 0 && grid2cell > 0.f, "bad ray count or grid_dim");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o && ray_d && bbox_min && bbox_max && nears && fars, "null buffer");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ray_near_far_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(table16_of(m), ray_o, ray_d, bbox_min,
                                                                      bbox_max, nears, fars, t_min, t_max,
                                                                      grid2cell, n);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_ray_sample_count(ashb_map* m, const float* ray_o, const float* ray_d, const float* ray_nears,
                          const float* ray_fars, int64_t* counts, int64_t max_samples_per_ray,
                          float grid2cell, int64_t n, void* stream) {
    if (int rc = check_sampler_map(m)) return rc;
    ASHB_REQUIRE(n >= 0 && grid2cell > 0.f && max_samples_per_ray > 0, "bad ray count, grid_dim or sample limit");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o && ray_d && ray_nears && ray_fars && counts, "null buffer");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ray_sample_kernel<false><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(
            table16_of(m), ray_o, ray_d, ray_nears, ray_fars, counts, nullptr, nullptr, nullptr, nullptr,
            max_samples_per_ray, grid2cell, n, m->status);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_ray_sample_fill(ashb_map* m, const float* ray_o, const float* ray_d, const float* ray_nears,
                         const float* ray_fars, const int64_t* prefix_sum, int64_t* ray_indices,
                         float* t_nears, float* t_fars, int64_t max_samples_per_ray, float grid2cell,
                         int64_t n, void* stream) {
    if (int rc = check_sampler_map(m)) return rc;
    ASHB_REQUIRE(n >= 0 && grid2cell > 0.f && max_samples_per_ray > 0, "bad ray count, grid_dim or sample limit");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o && ray_d && ray_nears && ray_fars && prefix_sum, "null buffer");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ray_sample_kernel<true><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(
            table16_of(m), ray_o, ray_d, ray_nears, ray_fars, nullptr, prefix_sum, ray_indices, t_nears, t_fars,
            max_samples_per_ray, grid2cell, n, m->status);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
