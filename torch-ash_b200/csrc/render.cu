// Volume-rendering accumulation over the packed ray samples the ray sampler produces (sm_100a).
// It stands in for the two third-party calls the reference's training step makes right after the
// grid query (demo/train_scene_recon.py:111-150, nerfacc.render_weight_from_density and
// nerfacc.accumulate_along_rays; nerfacc is not part of the reference tree): the standard
// emission-absorption quadrature
//     alpha_j = 1 - exp(-sigma_j * (t_end_j - t_start_j)),   T_j = prod_{k<j} (1 - alpha_k),
//     w_j = T_j * alpha_j,          out[ray] = sum_j w_j * value_j
// with samples of a ray contiguous and in marching order (ray_indices non-decreasing).
//
// One warp per ray: the optical depth is prefix-summed with warp shuffles in chunks of 32 samples,
// so a ray of 128 samples takes 4 rounds instead of 128 sequential steps.
#include "common.cuh"

namespace ashb {

__device__ __forceinline__ float warp_inclusive_sum(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// First and one-past-last sample of every ray; rays without samples keep 0, 0 (pre-zeroed).
__global__ void __launch_bounds__(256) segment_bounds_kernel(const int64_t* __restrict__ ray_indices, int64_t m,
                                                             int64_t n_rays, int64_t* __restrict__ seg_start,
                                                             int64_t* __restrict__ seg_end) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= m) return;
    const int64_t r = ray_indices[j];
    if (r < 0 || r >= n_rays) return;
    if (j == 0 || ray_indices[j - 1] != r) seg_start[r] = j;
    if (j == m - 1 || ray_indices[j + 1] != r) seg_end[r] = j + 1;
}

__global__ void __launch_bounds__(256) render_weights_forward_kernel(
        const float* __restrict__ t_starts, const float* __restrict__ t_ends, const float* __restrict__ sigmas,
        const int64_t* __restrict__ seg_start, const int64_t* __restrict__ seg_end, int64_t n_rays,
        float* __restrict__ weights) {
    const int64_t ray = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (ray >= n_rays) return;
    const int64_t s = seg_start[ray], e = seg_end[ray];
    float carry = 0.f;  // optical depth of the samples before this chunk
    for (int64_t base = s; base < e; base += 32) {
        const int64_t j = base + lane;
        const float tau = j < e ? sigmas[j] * (t_ends[j] - t_starts[j]) : 0.f;
        const float incl = warp_inclusive_sum(tau, lane);
        if (j < e) weights[j] = expf(-(carry + incl - tau)) * -expm1f(-tau);
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// d w_j / d sigma_j = dt_j * T_j * (1 - alpha_j) = dt_j * (T_j - w_j);  d w_k / d sigma_j = -dt_j * w_k (k > j)
// => grad_sigma_j = dt_j * (g_j * (T_j - w_j) - sum_{k>j} g_k w_k)
__global__ void __launch_bounds__(256) render_weights_backward_kernel(
        const float* __restrict__ t_starts, const float* __restrict__ t_ends, const float* __restrict__ sigmas,
        const float* __restrict__ weights, const float* __restrict__ grad_weights,
        const int64_t* __restrict__ seg_start, const int64_t* __restrict__ seg_end, int64_t n_rays,
        float* __restrict__ grad_sigmas) {
    const int64_t ray = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (ray >= n_rays) return;
    const int64_t s = seg_start[ray], e = seg_end[ray];
    float total = 0.f;  // sum_k g_k w_k over the ray
    for (int64_t base = s; base < e; base += 32) {
        const int64_t j = base + lane;
        total += j < e ? grad_weights[j] * weights[j] : 0.f;
    }
    total = warp_sum(total);
    float carry_tau = 0.f, carry_gw = 0.f;
    for (int64_t base = s; base < e; base += 32) {
        const int64_t j = base + lane;
        const bool live = j < e;
        const float dt = live ? t_ends[j] - t_starts[j] : 0.f;
        const float tau = live ? sigmas[j] * dt : 0.f;
        const float w = live ? weights[j] : 0.f;
        const float g = live ? grad_weights[j] : 0.f;
        const float incl_tau = warp_inclusive_sum(tau, lane);
        const float incl_gw = warp_inclusive_sum(g * w, lane);
        if (live) {
            const float T = expf(-(carry_tau + incl_tau - tau));
            const float suffix = total - (carry_gw + incl_gw);
            grad_sigmas[j] = dt * (g * (T - w) - suffix);
        }
        carry_tau += __shfl_sync(0xffffffffu, incl_tau, 31);
        carry_gw += __shfl_sync(0xffffffffu, incl_gw, 31);
    }
}

// out[ray][c] = sum_j w_j * values[j][c]  (values == nullptr: C = 1, value 1)
__global__ void __launch_bounds__(256) accumulate_forward_kernel(const float* __restrict__ weights,
                                                                 const float* __restrict__ values, int C,
                                                                 const int64_t* __restrict__ seg_start,
                                                                 const int64_t* __restrict__ seg_end, int64_t n_rays,
                                                                 float* __restrict__ out) {
    const int64_t ray = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (ray >= n_rays) return;
    const int64_t s = seg_start[ray], e = seg_end[ray];
    for (int c = 0; c < C; ++c) {
        float acc = 0.f;
        for (int64_t j = s + lane; j < e; j += 32) acc += weights[j] * (values ? values[j * C + c] : 1.f);
        acc = warp_sum(acc);
        if (lane == 0) out[ray * C + c] = acc;
    }
}

__global__ void __launch_bounds__(256) accumulate_backward_kernel(const float* __restrict__ weights,
                                                                  const float* __restrict__ values,
                                                                  const float* __restrict__ grad_out,
                                                                  const int64_t* __restrict__ ray_indices, int64_t m,
                                                                  int64_t n_rays, int C, float* __restrict__ grad_weights,
                                                                  float* __restrict__ grad_values) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= m) return;
    const int64_t r = ray_indices[j];
    const bool ok = r >= 0 && r < n_rays;
    const float w = weights[j];
    float gw = 0.f;
    for (int c = 0; c < C; ++c) {
        const float go = ok ? grad_out[r * C + c] : 0.f;
        gw += go * (values ? values[j * C + c] : 1.f);
        if (grad_values) grad_values[j * C + c] = w * go;
    }
    if (grad_weights) grad_weights[j] = gw;
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_render_segments(const int64_t* ray_indices, int64_t m, int64_t n_rays, int64_t* seg_start,
                         int64_t* seg_end, void* stream) {
    ASHB_REQUIRE(m >= 0 && n_rays >= 0, "negative count");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(seg_start && seg_end, "null buffer");
    ASHB_CUDA_TRY(cudaMemsetAsync(seg_start, 0, (size_t)n_rays * sizeof(int64_t), st));
    ASHB_CUDA_TRY(cudaMemsetAsync(seg_end, 0, (size_t)n_rays * sizeof(int64_t), st));
    if (m == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_indices != nullptr, "null ray_indices");
    segment_bounds_kernel<<<(unsigned)((m + 255) / 256), 256, 0, st>>>(ray_indices, m, n_rays, seg_start, seg_end);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_weights_forward(const float* t_starts, const float* t_ends, const float* sigmas,
                                const int64_t* seg_start, const int64_t* seg_end, int64_t n_rays, float* weights,
                                void* stream) {
    ASHB_REQUIRE(n_rays >= 0, "negative count");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(seg_start && seg_end, "null segment bounds");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    render_weights_forward_kernel<<<(unsigned)((n_rays * 32 + 255) / 256), 256, 0, st>>>(
            t_starts, t_ends, sigmas, seg_start, seg_end, n_rays, weights);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_weights_backward(const float* t_starts, const float* t_ends, const float* sigmas,
                                 const float* weights, const float* grad_weights, const int64_t* seg_start,
                                 const int64_t* seg_end, int64_t n_rays, float* grad_sigmas, void* stream) {
    ASHB_REQUIRE(n_rays >= 0, "negative count");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(seg_start && seg_end, "null segment bounds");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    render_weights_backward_kernel<<<(unsigned)((n_rays * 32 + 255) / 256), 256, 0, st>>>(
            t_starts, t_ends, sigmas, weights, grad_weights, seg_start, seg_end, n_rays, grad_sigmas);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_accumulate_forward(const float* weights, const float* values, int C, const int64_t* seg_start,
                                   const int64_t* seg_end, int64_t n_rays, float* out, void* stream) {
    ASHB_REQUIRE(n_rays >= 0 && C >= 1, "bad sizes");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(seg_start && seg_end && out, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    accumulate_forward_kernel<<<(unsigned)((n_rays * 32 + 255) / 256), 256, 0, st>>>(weights, values, C, seg_start,
                                                                                     seg_end, n_rays, out);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_accumulate_backward(const float* weights, const float* values, const float* grad_out,
                                    const int64_t* ray_indices, int64_t m, int64_t n_rays, int C,
                                    float* grad_weights, float* grad_values, void* stream) {
    ASHB_REQUIRE(m >= 0 && C >= 1, "bad sizes");
    if (m == 0) return ASHB_OK;
    ASHB_REQUIRE(weights && grad_out && ray_indices, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    accumulate_backward_kernel<<<(unsigned)((m + 255) / 256), 256, 0, st>>>(weights, values, grad_out, ray_indices, m,
                                                                            n_rays, C, grad_weights, grad_values);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
