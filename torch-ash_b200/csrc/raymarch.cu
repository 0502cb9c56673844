// Fused ray renderer over a sparse-dense grid (sm_100a): near/far estimation, interval sampling,
// trilinear query with its spatial gradient, signed distance -> density, and emission-absorption
// accumulation in ONE launch per direction, with no per-sample tensor in memory.
//
// It computes what the reference's training step composes from separate pieces
// (demo/train_scene_recon.py:64-161): grid.ray_find_near_far (ash/src/sampler.cu:7-71) ->
// grid.ray_sample (:123-215) -> x = o + t_mid * d -> grid(x) (ash/src/grid.cu:69-132) ->
// autograd.grad(sdf, x) (:178-255) -> normalize -> SDFToDensity (demo/train_scene_recon.py:20-31)
// -> render_weight_from_density / accumulate_along_rays (third-party, standard quadrature).
// The marching code is the sampler's own (sampler.cuh) and the split / corner addressing the query
// kernels' own (query.cuh), and every intermediate length is rounded where the composition rounds
// it, so a sample lands in the same cell in both.
//
// Channel convention of that step: channel 0 of an embedding row is the signed distance, channels
// 1..3 the colour.  One thread marches one ray; the 8 corner rows of a sample are 8 independent
// loads (one float4 each when the row stride allows).  The backward pass re-marches the ray and
// needs no saved per-sample state: the suffix sum of the transmittance gradient is closed with the
// forward outputs (sum_k g_k w_k = <grad_out, out> over the accumulated channels).
#include <climits>

#include "query.cuh"
#include "sampler.cuh"

namespace ashb {

constexpr int kRayOut = 16;  // floats per ray in the output row (see ashb200.h)

struct RayGrid {
    Table16 table;
    const float* __restrict__ emb;
    const int32_t* __restrict__ nb_lut;
    int64_t n_emb, cells_per_grid;
    int G, D, interp;
    float G_f, inv_G;
    float org[3];
    float inv_cell;        // (float)(1 / cell_size): world -> cell
    float cell;            // (float)cell_size: cell -> world for ray lengths
    float grid2cell;       // (float)G, the sampler's block edge in cells
    const float* __restrict__ bbox_min;  // cell units
    const float* __restrict__ bbox_max;
    float t_min, t_max;    // cell units
    int64_t max_samples;
    int skip_missed;
};

struct Sample {
    float t_mid, dt;       // world units
    float sdf, rgb[3];
    float g[3], gnorm;     // d sdf / d world position
    float nrm[3];
    float sigma, hit;      // hit: the sample's own block is active (the mask of the query)
    bool ok;               // all 8 corner rows exist
    int64_t base[8];
    AxisWeights<float> aw;
};

template <bool ALIGNED>
__device__ __forceinline__ void load_row4(const float* p, float* v) {
    if (ALIGNED) {
        // 64-byte L2 fetch size: one 16-byte row slice of a random line is wanted
        asm volatile("ld.global.nc.L2::64B.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3])
                     : "l"(p));
    } else {
        v[0] = __ldg(p); v[1] = __ldg(p + 1); v[2] = __ldg(p + 2); v[3] = __ldg(p + 3);
    }
}

template <bool ALIGNED>
__device__ __forceinline__ void add_row4(float* p, const float* v) {
    if (ALIGNED) {
        atomicAdd(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) atomicAdd(p + k, v[k]);
    }
}

// Laplace-CDF density of demo/train_scene_recon.py:20-31, operation by operation.
__device__ __forceinline__ float density(float sdf, float beta, float alpha) {
    const float sgn = sdf > 0.f ? 1.f : (sdf < 0.f ? -1.f : 0.f);
    const float em = expm1f(__fdiv_rn(-fabsf(sdf), beta));
    return __fmul_rn(alpha, __fadd_rn(0.5f, __fmul_rn(__fmul_rn(0.5f, sgn), em)));
}

// Everything the renderer needs of the interval [t0c, t1c] (cell units) of a ray.
template <bool ALIGNED>
__device__ __forceinline__ void eval_sample(const RayGrid& G, const float* o_w, const float* d, float t0c, float t1c,
                                            const int* hint_blk, int hint_gi, float beta, float alpha, Sample& s) {
    const float t0w = __fmul_rn(t0c, G.cell), t1w = __fmul_rn(t1c, G.cell);
    s.t_mid = __fmul_rn(0.5f, __fadd_rn(t0w, t1w));
    s.dt = __fsub_rn(t1w, t0w);
    float xw[3], off[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) xw[k] = __fadd_rn(o_w[k], __fmul_rn(s.t_mid, d[k]));
    int blk[3], cell[3];
    split_world_position(xw, G.org, G.inv_cell, G.inv_G, G.G_f, G.G, blk, cell, off);
    // the march has just probed the block at the interval's start: the midpoint is usually in it
    const int gi = (blk[0] == hint_blk[0] && blk[1] == hint_blk[1] && blk[2] == hint_blk[2])
                           ? hint_gi : lookup(G.table, blk[0], blk[1], blk[2], 0);
    s.hit = gi >= 0 && gi < G.n_emb ? 1.f : 0.f;
    s.ok = s.hit != 0.f && corner_rows(G.nb_lut, gi, cell, G.G, G.n_emb, G.cells_per_grid, G.D, s.base);
    s.sdf = 0.f;
    s.rgb[0] = s.rgb[1] = s.rgb[2] = 0.f;
    s.g[0] = s.g[1] = s.g[2] = 0.f;
    if (s.ok) {
        s.aw.init(G.interp, off);
        float e[8][4];
#pragma unroll
        for (int c = 0; c < 8; ++c) load_row4<ALIGNED>(G.emb + s.base[c], e[c]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float w = s.aw.weight(c);
            float wg[3];
            s.aw.grad(c, wg);
            s.sdf += w * e[c][0];
            s.rgb[0] += w * e[c][1];
            s.rgb[1] += w * e[c][2];
            s.rgb[2] += w * e[c][3];
            s.g[0] += e[c][0] * wg[0];
            s.g[1] += e[c][0] * wg[1];
            s.g[2] += e[c][0] * wg[2];
        }
#pragma unroll
        for (int k = 0; k < 3; ++k) s.g[k] *= G.inv_cell;
    }
    s.gnorm = sqrtf(s.g[0] * s.g[0] + s.g[1] * s.g[1] + s.g[2] * s.g[2]);
    const float den = fmaxf(s.gnorm, 1e-12f);  // torch.nn.functional.normalize
#pragma unroll
    for (int k = 0; k < 3; ++k) s.nrm[k] = s.g[k] / den;
    s.sigma = density(s.sdf, beta, alpha) * s.hit;
}

// Gradient of one sample given d loss / d (its weight) = gw, its weight w, the transmittance T in
// front of it and the sum of gw * w over the samples behind it: adds the embedding gradient of its
// 8 corner rows and returns its contribution to d loss / d beta.
template <bool ALIGNED>
__device__ __forceinline__ float sample_gradient(const RayGrid& G, const Sample& s, const float* go, float w, float T,
                                                 float gw, float behind, float beta, float alpha,
                                                 float* __restrict__ grad_emb) {
    // d loss / d sigma_j = dt_j * (g_j * (T_j - w_j) - sum_{k>j} g_k w_k)
    const float dsigma = s.dt * (gw * (T - w) - behind) * s.hit;
    // density(sdf, beta) = alpha * h, h = 0.5 + 0.5 * sign * expm1(-|sdf| / beta)
    const float a = fabsf(s.sdf);
    const float sgn = s.sdf > 0.f ? 1.f : (s.sdf < 0.f ? -1.f : 0.f);
    const float ex = expf(-a / beta);
    const float h = 0.5f + 0.5f * sgn * expm1f(-a / beta);
    const float gbeta = dsigma * (-h * alpha * alpha + alpha * 0.5f * sgn * ex * a * alpha * alpha);
    if (!s.ok) return gbeta;
    const float dsdf = dsigma * (-0.5f * alpha * alpha * ex * sgn * sgn);
    // d loss / d (world gradient of the signed distance): through the rendered normal and
    // through the two eikonal sums
    float dn[3] = {w * go[4], w * go[5], w * go[6]}, dg[3];
    if (s.gnorm > 1e-12f) {
        const float nd = s.nrm[0] * dn[0] + s.nrm[1] * dn[1] + s.nrm[2] * dn[2];
        const float r = s.gnorm - 1.f;
        const float eik = go[8] * (r > 0.f ? 1.f : (r < 0.f ? -1.f : 0.f)) + go[9] * 2.f * r;
#pragma unroll
        for (int k = 0; k < 3; ++k) dg[k] = (dn[k] - s.nrm[k] * nd) / s.gnorm + eik * s.nrm[k];
    } else {
#pragma unroll
        for (int k = 0; k < 3; ++k) dg[k] = dn[k] / 1e-12f;
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float wc = s.aw.weight(c);
        float wg[3];
        s.aw.grad(c, wg);
        float v[4];
        v[0] = wc * dsdf + (wg[0] * dg[0] + wg[1] * dg[1] + wg[2] * dg[2]) * G.inv_cell;
        v[1] = wc * w * go[0];
        v[2] = wc * w * go[1];
        v[3] = wc * w * go[2];
        add_row4<ALIGNED>(grad_emb + s.base[c], v);
    }
    return gbeta;
}

// Near/far + the sampler's march as a resumable state: next() advances the ray to its next
// interval inside an occupied block.  The kernels call it in warp-converged rounds (every lane
// marches to its next interval, then all lanes evaluate their intervals together), so a warp pays
// for one evaluation per round instead of one per march step in which any lane has a sample.
struct RayMarcher {
    float tt, seg_near, ray_far, cell_step, grid_step, cell2grid;
    bool active;

    // KNOWN_RANGE: near_w / far_w come in (the backward pass reads them from the forward's output
    // row) and the first stage is not repeated.
    template <bool KNOWN_RANGE>
    __device__ __forceinline__ void start(const RayGrid& G, const float* o_c, const float* d, bool live, float& near_w,
                                          float& far_w) {
        active = live;
        tt = seg_near = ray_far = cell_step = grid_step = cell2grid = 0.f;
        if (!live) return;
        if (!KNOWN_RANGE) {
            const float lo[3] = {G.bbox_min[0], G.bbox_min[1], G.bbox_min[2]};
            const float hi[3] = {G.bbox_max[0], G.bbox_max[1], G.bbox_max[2]};
            float near_c, far_c;
            march_near_far(G.table, o_c, d, lo, hi, G.t_min, G.t_max, G.grid2cell, near_c, far_c);
            // lengths leave the first stage in world units and re-enter the second in cell units
            near_w = __fmul_rn(near_c, G.cell);
            far_w = __fmul_rn(far_c, G.cell);
        }
        if (near_w < 0.f && G.skip_missed) {  // no occupied block met: the ray is not sampled
            active = false;
            return;
        }
        const float ray_near = __fmul_rn(near_w, G.inv_cell);
        ray_far = __fmul_rn(far_w, G.inv_cell);
        cell2grid = (float)(1.0 / (double)G.grid2cell);
        cell_step = sample_cell_step(ray_near, ray_far, G.max_samples);
        grid_step = cell_step * G.grid2cell;
        tt = seg_near = ray_near;
    }

    // The interval [t0c, t1c] (cell units), the active block found at its start and that block's
    // index; false when the ray is finished.
    __device__ __forceinline__ bool next(const RayGrid& G, const float* o_c, const float* d, float& t0c, float& t1c,
                                         int* blk, int& gi) {
        while (active && tt < ray_far) {
            float p[3];
            ray_at(o_c, d, tt, p);
            blk[0] = (int)floorf(p[0] * cell2grid);  // as block_active places it
            blk[1] = (int)floorf(p[1] * cell2grid);
            blk[2] = (int)floorf(p[2] * cell2grid);
            gi = lookup(G.table, blk[0], blk[1], blk[2], 0);
            if (gi < 0) {
                tt += grid_step;
            } else {
                t0c = seg_near;
                tt += cell_step;
                t1c = seg_near = tt;
                return true;
            }
        }
        active = false;
        return false;
    }
};

template <bool ALIGNED>
__global__ void __launch_bounds__(128) render_rays_forward_kernel(RayGrid G, const float* __restrict__ ray_o_world,
                                                                  const float* __restrict__ ray_o_cell,
                                                                  const float* __restrict__ ray_d,
                                                                  const float* __restrict__ beta_ptr,
                                                                  float* __restrict__ out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < n;  // whole warps stay together for the round votes below
    const int64_t r3 = live ? 3 * i : 0;
    const float o_w[3] = {ray_o_world[r3], ray_o_world[r3 + 1], ray_o_world[r3 + 2]};
    const float o_c[3] = {ray_o_cell[r3], ray_o_cell[r3 + 1], ray_o_cell[r3 + 2]};
    const float d[3] = {ray_d[r3], ray_d[r3 + 1], ray_d[r3 + 2]};
    const float beta = beta_ptr[0];
    const float alpha = __frcp_rn(beta);
    float acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};  // rgb, depth, normal, weight, eikonal L1, L2
    float depth_tau = 0.f, count = 0.f, near_w = 0.f, far_w = 0.f;
    RayMarcher m;
    m.start<false>(G, o_c, d, live, near_w, far_w);
    for (;;) {
        float t0c, t1c;
        int blk[3], gi;
        const bool have = m.next(G, o_c, d, t0c, t1c, blk, gi);
        if (!__any_sync(0xffffffffu, have)) break;
        if (have) {
            Sample s;
            eval_sample<ALIGNED>(G, o_w, d, t0c, t1c, blk, gi, beta, alpha, s);
            const float tau = s.sigma * s.dt;
            const float w = expf(-depth_tau) * -expm1f(-tau);
            depth_tau += tau;
            acc[0] += w * s.rgb[0];
            acc[1] += w * s.rgb[1];
            acc[2] += w * s.rgb[2];
            acc[3] += w * s.t_mid;
            acc[4] += w * s.nrm[0];
            acc[5] += w * s.nrm[1];
            acc[6] += w * s.nrm[2];
            acc[7] += w;
            const float r = s.gnorm - 1.f;
            acc[8] += fabsf(r);
            acc[9] += r * r;
            count += 1.f;
        }
    }
    if (!live) return;
    float* row = out + i * kRayOut;
#pragma unroll
    for (int k = 0; k < 10; ++k) row[k] = acc[k];
    row[10] = count;
    row[11] = near_w;
    row[12] = far_w;
    row[13] = row[14] = row[15] = 0.f;
}

template <bool ALIGNED>
__global__ void __launch_bounds__(128) render_rays_backward_kernel(RayGrid G, const float* __restrict__ ray_o_world,
                                                                   const float* __restrict__ ray_o_cell,
                                                                   const float* __restrict__ ray_d,
                                                                   const float* __restrict__ beta_ptr,
                                                                   const float* __restrict__ out,
                                                                   const float* __restrict__ grad_out,
                                                                   float* __restrict__ grad_emb,
                                                                   float* __restrict__ grad_beta, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < n;
    const int64_t r3 = live ? 3 * i : 0, r16 = live ? i * kRayOut : 0;
    const float o_w[3] = {ray_o_world[r3], ray_o_world[r3 + 1], ray_o_world[r3 + 2]};
    const float o_c[3] = {ray_o_cell[r3], ray_o_cell[r3 + 1], ray_o_cell[r3 + 2]};
    const float d[3] = {ray_d[r3], ray_d[r3 + 1], ray_d[r3 + 2]};
    const float beta = beta_ptr[0];
    const float alpha = __frcp_rn(beta);
    float go[10];
#pragma unroll
    for (int k = 0; k < 10; ++k) go[k] = grad_out[r16 + k];
    // sum over the ray of (d loss / d w_k) * w_k, from the forward outputs
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += go[k] * out[r16 + k];
    float depth_tau = 0.f, prefix = 0.f, gbeta = 0.f;
    float near_w = out[r16 + 11], far_w = out[r16 + 12];
    RayMarcher m;
    m.start<true>(G, o_c, d, live, near_w, far_w);
    for (;;) {
        float t0c, t1c;
        int blk[3], gi;
        const bool have = m.next(G, o_c, d, t0c, t1c, blk, gi);
        if (!__any_sync(0xffffffffu, have)) break;
        if (!have) continue;
        Sample s;
        eval_sample<ALIGNED>(G, o_w, d, t0c, t1c, blk, gi, beta, alpha, s);
        const float tau = s.sigma * s.dt;
        const float T = expf(-depth_tau);
        const float w = T * -expm1f(-tau);
        depth_tau += tau;
        const float gw = go[0] * s.rgb[0] + go[1] * s.rgb[1] + go[2] * s.rgb[2] + go[3] * s.t_mid +
                         go[4] * s.nrm[0] + go[5] * s.nrm[1] + go[6] * s.nrm[2] + go[7];
        prefix += gw * w;
        gbeta += sample_gradient<ALIGNED>(G, s, go, w, T, gw, total - prefix, beta, alpha, grad_emb);
    }
    // one atomic per warp for the density parameter
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gbeta += __shfl_xor_sync(0xffffffffu, gbeta, o);
    if ((threadIdx.x & 31) == 0 && gbeta != 0.f) atomicAdd(grad_beta, gbeta);
}

// ---- the same renderer with the samples of a ray evaluated in parallel -------------------------
// One thread per ray only marches (near/far + interval sampler) and writes the ray's intervals into
// a fixed-stride list; then one WARP per ray evaluates 32 intervals at a time (queries, gradient of
// the signed distance, density) and closes the transmittance with a warp scan.  The dependent chain
// of a ray is then its probes plus ceil(samples / 32) evaluation rounds instead of one evaluation
// per sample; the backward reuses the list and does not march at all.
__global__ void __launch_bounds__(128) ray_intervals_kernel(RayGrid G, const float* __restrict__ ray_o_cell,
                                                            const float* __restrict__ ray_d,
                                                            float2* __restrict__ intervals, int* __restrict__ counts,
                                                            float* __restrict__ near_far, int stride, int64_t n,
                                                            uint32_t* __restrict__ status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float o_c[3] = {ray_o_cell[3 * i], ray_o_cell[3 * i + 1], ray_o_cell[3 * i + 2]};
    const float d[3] = {ray_d[3 * i], ray_d[3 * i + 1], ray_d[3 * i + 2]};
    float near_w = 0.f, far_w = 0.f;
    RayMarcher m;
    m.start<false>(G, o_c, d, true, near_w, far_w);
    int k = 0;
    if (m.active)
        march_intervals(G.table, o_c, d, m.tt, m.ray_far, m.cell_step, m.grid_step, m.cell2grid,
                        [&](float seg_near, float seg_far) {
                            if (k < stride)
                                intervals[i * stride + k] = make_float2(seg_near, seg_far);
                            else
                                atomicOr(status, ASHB_STATUS_CAPACITY);  // more intervals than the list holds
                            ++k;
                        });
    counts[i] = k < stride ? k : stride;
    near_far[2 * i] = near_w;
    near_far[2 * i + 1] = far_w;
}

__device__ __forceinline__ float warp_scan_inclusive(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}

template <bool ALIGNED>
__global__ void __launch_bounds__(256) render_intervals_forward_kernel(
        RayGrid G, const float* __restrict__ ray_o_world, const float* __restrict__ ray_d,
        const float* __restrict__ beta_ptr, const float2* __restrict__ intervals, const int* __restrict__ counts,
        const float* __restrict__ near_far, int stride, float* __restrict__ out, int64_t n) {
    const int64_t ray = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (ray >= n) return;  // whole warps
    const float o_w[3] = {ray_o_world[3 * ray], ray_o_world[3 * ray + 1], ray_o_world[3 * ray + 2]};
    const float d[3] = {ray_d[3 * ray], ray_d[3 * ray + 1], ray_d[3 * ray + 2]};
    const float beta = beta_ptr[0];
    const float alpha = __frcp_rn(beta);
    const int count = counts[ray];
    const int no_hint[3] = {INT_MIN, INT_MIN, INT_MIN};
    float acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    float carry = 0.f;
    for (int base = 0; base < count; base += 32) {
        const int j = base + lane;
        const bool live = j < count;
        Sample s;
        float tau = 0.f;
        if (live) {
            const float2 iv = intervals[ray * stride + j];
            eval_sample<ALIGNED>(G, o_w, d, iv.x, iv.y, no_hint, -1, beta, alpha, s);
            tau = s.sigma * s.dt;
        }
        const float incl = warp_scan_inclusive(tau, lane);
        if (live) {
            const float w = expf(-(carry + incl - tau)) * -expm1f(-tau);
            acc[0] += w * s.rgb[0];
            acc[1] += w * s.rgb[1];
            acc[2] += w * s.rgb[2];
            acc[3] += w * s.t_mid;
            acc[4] += w * s.nrm[0];
            acc[5] += w * s.nrm[1];
            acc[6] += w * s.nrm[2];
            acc[7] += w;
            const float r = s.gnorm - 1.f;
            acc[8] += fabsf(r);
            acc[9] += r * r;
        }
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
#pragma unroll
    for (int k = 0; k < 10; ++k) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    }
    if (lane == 0) {
        float* row = out + ray * kRayOut;
#pragma unroll
        for (int k = 0; k < 10; ++k) row[k] = acc[k];
        row[10] = (float)count;
        row[11] = near_far[2 * ray];
        row[12] = near_far[2 * ray + 1];
        row[13] = row[14] = row[15] = 0.f;
    }
}

template <bool ALIGNED>
__global__ void __launch_bounds__(256) render_intervals_backward_kernel(
        RayGrid G, const float* __restrict__ ray_o_world, const float* __restrict__ ray_d,
        const float* __restrict__ beta_ptr, const float2* __restrict__ intervals, const int* __restrict__ counts,
        int stride, const float* __restrict__ out, const float* __restrict__ grad_out, float* __restrict__ grad_emb,
        float* __restrict__ grad_beta, int64_t n) {
    const int64_t ray = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (ray >= n) return;  // whole warps
    const float o_w[3] = {ray_o_world[3 * ray], ray_o_world[3 * ray + 1], ray_o_world[3 * ray + 2]};
    const float d[3] = {ray_d[3 * ray], ray_d[3 * ray + 1], ray_d[3 * ray + 2]};
    const float beta = beta_ptr[0];
    const float alpha = __frcp_rn(beta);
    const int count = counts[ray];
    const int no_hint[3] = {INT_MIN, INT_MIN, INT_MIN};
    float go[10];
#pragma unroll
    for (int k = 0; k < 10; ++k) go[k] = grad_out[ray * kRayOut + k];
    float total = 0.f;  // sum over the ray of (d loss / d w_k) * w_k, from the forward outputs
#pragma unroll
    for (int k = 0; k < 8; ++k) total += go[k] * out[ray * kRayOut + k];
    float carry_tau = 0.f, carry_gw = 0.f, gbeta = 0.f;
    for (int base = 0; base < count; base += 32) {
        const int j = base + lane;
        const bool live = j < count;
        Sample s;
        float tau = 0.f, gw = 0.f;
        if (live) {
            const float2 iv = intervals[ray * stride + j];
            eval_sample<ALIGNED>(G, o_w, d, iv.x, iv.y, no_hint, -1, beta, alpha, s);
            tau = s.sigma * s.dt;
            gw = go[0] * s.rgb[0] + go[1] * s.rgb[1] + go[2] * s.rgb[2] + go[3] * s.t_mid + go[4] * s.nrm[0] +
                 go[5] * s.nrm[1] + go[6] * s.nrm[2] + go[7];
        }
        const float incl_tau = warp_scan_inclusive(tau, lane);
        const float T = expf(-(carry_tau + incl_tau - tau));
        const float w = live ? T * -expm1f(-tau) : 0.f;
        const float incl_gw = warp_scan_inclusive(gw * w, lane);
        if (live)
            gbeta += sample_gradient<ALIGNED>(G, s, go, w, T, gw, total - (carry_gw + incl_gw), beta, alpha, grad_emb);
        carry_tau += __shfl_sync(0xffffffffu, incl_tau, 31);
        carry_gw += __shfl_sync(0xffffffffu, incl_gw, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gbeta += __shfl_xor_sync(0xffffffffu, gbeta, o);
    if (lane == 0 && gbeta != 0.f) atomicAdd(grad_beta, gbeta);
}

}  // namespace ashb

using namespace ashb;

static int make_ray_grid(RayGrid& g, ashb_map* m, int interp, const float* emb, int64_t n_emb, int grid_dim, int D,
                         const int32_t* nb_lut, double cell_size, const float* origin, const float* bbox_min,
                         const float* bbox_max, float t_min, float t_max, int64_t max_samples, int skip_missed,
                         bool marches = true) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim == 3, "ray rendering needs a 3-D map");
    ASHB_REQUIRE(interp == ASHB_LINEAR || interp == ASHB_SMOOTH_STEP, "unknown interpolation");
    ASHB_REQUIRE(emb && nb_lut && (!marches || (bbox_min && bbox_max)), "null buffer");
    ASHB_REQUIRE(n_emb > 0 && grid_dim >= 1 && D >= 4, "needs embedding_dim >= 4 (signed distance + colour)");
    ASHB_REQUIRE(cell_size > 0.0 && max_samples > 0, "bad cell size or sample limit");
    ASHB_REQUIRE(t_min == t_min && t_max == t_max && t_max - t_min < 3.0e38f, "ray range must be finite");
    g.table = table16_of(m);
    g.emb = emb;
    g.nb_lut = nb_lut;
    g.n_emb = n_emb;
    g.G = grid_dim;
    g.cells_per_grid = (int64_t)grid_dim * grid_dim * grid_dim;
    g.D = D;
    g.interp = interp;
    g.G_f = (float)grid_dim;
    g.inv_G = (float)(1.0 / (double)grid_dim);
    for (int k = 0; k < 3; ++k) g.org[k] = origin ? origin[k] : 0.f;
    g.inv_cell = (float)(1.0 / cell_size);
    g.cell = (float)cell_size;
    g.grid2cell = (float)grid_dim;
    g.bbox_min = bbox_min;
    g.bbox_max = bbox_max;
    g.t_min = t_min;
    g.t_max = t_max;
    g.max_samples = max_samples;
    g.skip_missed = skip_missed;
    return ASHB_OK;
}

extern "C" {

int ashb_render_rays_forward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                             const int32_t* nb_lut, double cell_size, const float* origin, const float* ray_o_world,
                             const float* ray_o_cell, const float* ray_d, const float* bbox_min_cell,
                             const float* bbox_max_cell, float t_min_cell, float t_max_cell,
                             int64_t max_samples_per_ray, int skip_missed, const float* beta, float* out,
                             int64_t n_rays, void* stream) {
    RayGrid g;
    if (int rc = make_ray_grid(g, map, interp, embeddings, n_emb, grid_dim, D, nb_lut, cell_size, origin, bbox_min_cell,
                               bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed))
        return rc;
    ASHB_REQUIRE(n_rays >= 0, "negative ray count");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o_world && ray_o_cell && ray_d && beta && out, "null buffer");
    DeviceGuard guard(map->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((n_rays + 127) / 128);
    if (D % 4 == 0)
        render_rays_forward_kernel<true><<<grid, 128, 0, st>>>(g, ray_o_world, ray_o_cell, ray_d, beta, out, n_rays);
    else
        render_rays_forward_kernel<false><<<grid, 128, 0, st>>>(g, ray_o_world, ray_o_cell, ray_d, beta, out, n_rays);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_rays_backward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                              const int32_t* nb_lut, double cell_size, const float* origin, const float* ray_o_world,
                              const float* ray_o_cell, const float* ray_d, const float* bbox_min_cell,
                              const float* bbox_max_cell, float t_min_cell, float t_max_cell,
                              int64_t max_samples_per_ray, int skip_missed, const float* beta, const float* out,
                              const float* grad_out, float* grad_embeddings, float* grad_beta, int64_t n_rays,
                              void* stream) {
    RayGrid g;
    if (int rc = make_ray_grid(g, map, interp, embeddings, n_emb, grid_dim, D, nb_lut, cell_size, origin, bbox_min_cell,
                               bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed))
        return rc;
    ASHB_REQUIRE(n_rays >= 0, "negative ray count");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o_world && ray_o_cell && ray_d && beta && out && grad_out && grad_embeddings && grad_beta,
                 "null buffer");
    DeviceGuard guard(map->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((n_rays + 127) / 128);
    if (D % 4 == 0)
        render_rays_backward_kernel<true><<<grid, 128, 0, st>>>(g, ray_o_world, ray_o_cell, ray_d, beta, out, grad_out,
                                                                grad_embeddings, grad_beta, n_rays);
    else
        render_rays_backward_kernel<false><<<grid, 128, 0, st>>>(g, ray_o_world, ray_o_cell, ray_d, beta, out, grad_out,
                                                                 grad_embeddings, grad_beta, n_rays);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_rays_intervals(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                               const int32_t* nb_lut, double cell_size, const float* origin,
                               const float* ray_o_cell, const float* ray_d, const float* bbox_min_cell,
                               const float* bbox_max_cell, float t_min_cell, float t_max_cell,
                               int64_t max_samples_per_ray, int skip_missed, float* intervals, int32_t* counts,
                               float* near_far, int64_t stride, int64_t n_rays, void* stream) {
    RayGrid g;
    if (int rc = make_ray_grid(g, map, interp, embeddings, n_emb, grid_dim, D, nb_lut, cell_size, origin, bbox_min_cell,
                               bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed))
        return rc;
    ASHB_REQUIRE(n_rays >= 0 && stride >= 1 && stride <= 0x7fffffffll, "bad ray count or stride");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o_cell && ray_d && intervals && counts && near_far, "null buffer");
    ASHB_REQUIRE(((uintptr_t)intervals & 7) == 0, "interval list must be 8-byte aligned");
    DeviceGuard guard(map->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ray_intervals_kernel<<<(unsigned)((n_rays + 127) / 128), 128, 0, st>>>(
            g, ray_o_cell, ray_d, reinterpret_cast<float2*>(intervals), counts, near_far, (int)stride, n_rays,
            map->status);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_intervals_forward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim,
                                  int D, const int32_t* nb_lut, double cell_size, const float* origin,
                                  const float* ray_o_world, const float* ray_d, const float* beta,
                                  const float* intervals, const int32_t* counts, const float* near_far, int64_t stride,
                                  float* out, int64_t n_rays, void* stream) {
    RayGrid g;  // no marching here: the box and the ray range are not used
    if (int rc = make_ray_grid(g, map, interp, embeddings, n_emb, grid_dim, D, nb_lut, cell_size, origin, nullptr,
                               nullptr, 0.f, 1.f, 1, 0, false))
        return rc;
    ASHB_REQUIRE(n_rays >= 0 && stride >= 1, "bad ray count or stride");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o_world && ray_d && beta && intervals && counts && near_far && out, "null buffer");
    DeviceGuard guard(map->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((n_rays * 32 + 255) / 256);
    const float2* iv = reinterpret_cast<const float2*>(intervals);
    if (D % 4 == 0)
        render_intervals_forward_kernel<true><<<grid, 256, 0, st>>>(g, ray_o_world, ray_d, beta, iv, counts, near_far,
                                                                    (int)stride, out, n_rays);
    else
        render_intervals_forward_kernel<false><<<grid, 256, 0, st>>>(g, ray_o_world, ray_d, beta, iv, counts, near_far,
                                                                     (int)stride, out, n_rays);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_render_intervals_backward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim,
                                   int D, const int32_t* nb_lut, double cell_size, const float* origin,
                                   const float* ray_o_world, const float* ray_d, const float* beta,
                                   const float* intervals, const int32_t* counts, int64_t stride, const float* out,
                                   const float* grad_out, float* grad_embeddings, float* grad_beta, int64_t n_rays,
                                   void* stream) {
    RayGrid g;  // no marching here: the box and the ray range are not used
    if (int rc = make_ray_grid(g, map, interp, embeddings, n_emb, grid_dim, D, nb_lut, cell_size, origin, nullptr,
                               nullptr, 0.f, 1.f, 1, 0, false))
        return rc;
    ASHB_REQUIRE(n_rays >= 0 && stride >= 1, "bad ray count or stride");
    if (n_rays == 0) return ASHB_OK;
    ASHB_REQUIRE(ray_o_world && ray_d && beta && intervals && counts && out && grad_out && grad_embeddings && grad_beta,
                 "null buffer");
    DeviceGuard guard(map->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((n_rays * 32 + 255) / 256);
    const float2* iv = reinterpret_cast<const float2*>(intervals);
    if (D % 4 == 0)
        render_intervals_backward_kernel<true><<<grid, 256, 0, st>>>(g, ray_o_world, ray_d, beta, iv, counts,
                                                                     (int)stride, out, grad_out, grad_embeddings,
                                                                     grad_beta, n_rays);
    else
        render_intervals_backward_kernel<false><<<grid, 256, 0, st>>>(g, ray_o_world, ray_d, beta, iv, counts,
                                                                      (int)stride, out, grad_out, grad_embeddings,
                                                                      grad_beta, n_rays);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
