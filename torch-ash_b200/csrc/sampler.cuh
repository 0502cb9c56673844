// Ray marching over the hashed block structure, shared by the sampler kernels and the fused ray
// renderer, so that both place every step identically.  Semantics of ash/src/sampler.cu:7-215;
// lengths in cell units; position = fma(t, d, o) per component in float32, block =
// floor(position * (float)(1.0 / grid2cell)).
#pragma once
#include "hashmap.cuh"

namespace ashb {

__device__ __forceinline__ bool block_active(const Table16& t, const float* p, float cell2grid) {
    const int bx = (int)floorf(p[0] * cell2grid);
    const int by = (int)floorf(p[1] * cell2grid);
    const int bz = (int)floorf(p[2] * cell2grid);
    return lookup(t, bx, by, bz, 0) >= 0;
}

__device__ __forceinline__ void ray_at(const float* o, const float* d, float t, float* p) {
    p[0] = __fmaf_rn(t, d[0], o[0]);
    p[1] = __fmaf_rn(t, d[1], o[1]);
    p[2] = __fmaf_rn(t, d[2], o[2]);
}

// A table lookup split in two so that several can be in flight: probe_begin reads the key's home
// slot (when `wanted`), probe_finish walks on from there and says whether the block is active.
struct ProbeStart {
    int k[3];
    uint32_t slot;
    Entry e;
};

__device__ __forceinline__ ProbeStart probe_begin(const Table16& t, const float* p, float cell2grid, bool wanted) {
    ProbeStart ps;
    ps.k[0] = (int)floorf(p[0] * cell2grid);
    ps.k[1] = (int)floorf(p[1] * cell2grid);
    ps.k[2] = (int)floorf(p[2] * cell2grid);
    ps.slot = hash_key(ps.k[0], ps.k[1], ps.k[2], 0) & t.mask;
    ps.e = wanted ? t.read_const(ps.slot) : Entry{0, 0, 0, 0, kEmpty};
    return ps;
}

__device__ __forceinline__ bool probe_finish(const Table16& t, const ProbeStart& ps) {
    Entry e = ps.e;
    uint32_t s = ps.slot;
    for (uint32_t probe = 0; probe <= t.mask; ++probe) {
        if (e.val == kEmpty) return false;
        if (e.val >= 0 && key_match(e, ps.k[0], ps.k[1], ps.k[2], 0)) return true;
        s = (s + 1) & t.mask;
        e = t.read_const(s);
    }
    return false;
}

// First / last occupied stretch of a ray inside the box (ash/src/sampler.cu:7-71): marches in
// half-block steps from t_min; near = -1 when no occupied block is met.
__device__ __forceinline__ void march_near_far(const Table16& t, const float* o, const float* d, const float* lo,
                                               const float* hi, float t_min, float t_max, float grid2cell,
                                               float& near, float& far) {
    const float cell2grid = (float)(1.0 / (double)grid2cell);
    const float step = (float)((double)grid2cell * 0.5);
    near = -1.f;
    far = t_max;
    float tt = t_min;
    // step > 0 is checked by the host, so the march ends after (t_max - t_min) / step rounds.
    // The positions of consecutive steps do not depend on what the probes find, so four steps are
    // taken per round: their first table reads are issued together, then the steps are replayed
    // in order (same sequence of `tt`, same results as one step at a time).
#ifndef ASHB_NEAR_FAR_AHEAD
#define ASHB_NEAR_FAR_AHEAD 4
#endif
    constexpr int kAhead = ASHB_NEAR_FAR_AHEAD;
    bool ended = false;
    while (!ended && tt < t_max) {
        float ts[kAhead];
        bool inside[kAhead];
        ProbeStart ps[kAhead];
        float t_k = tt;
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            ts[k] = t_k;
            float p[3];
            ray_at(o, d, t_k, p);
            inside[k] = t_k < t_max && p[0] >= lo[0] && p[0] <= hi[0] && p[1] >= lo[1] && p[1] <= hi[1] &&
                        p[2] >= lo[2] && p[2] <= hi[2];
            ps[k] = probe_begin(t, p, cell2grid, inside[k]);
            t_k += step;
        }
#pragma unroll
        for (int k = 0; k < kAhead; ++k) {
            if (ended) break;
            if (!(ts[k] < t_max) || !inside[k]) {
                ended = true;
                break;
            }
            if (probe_finish(t, ps[k])) {
                near = near < 0.f ? ts[k] : fmaxf(near - step, t_min);
                far = fminf(ts[k] + step, t_max);
            }
        }
        tt = t_k;
    }
}

// Step of the interval sampler inside occupied blocks (ash/src/sampler.cu:151): max(0.7, float) is
// a double max whose result is stored as float.
__device__ __forceinline__ float sample_cell_step(float ray_near, float ray_far, int64_t max_samples) {
    return (float)fmax(0.7, (double)((ray_far - ray_near) / (float)max_samples));
}

// The interval sampler's march (ash/src/sampler.cu:123-215) with four probes in flight: from
// `near` to `far`, a cell step inside occupied blocks -- each such step is an interval, reported to
// emit(t_start, t_end) -- and a block step outside.  The next positions are guessed from the kind of
// step taken last, their probes are issued together, and the steps are replayed in order; the
// first step whose outcome differs from the guess ends the round, because the positions after it
// were guessed with the wrong stride.  `tt` goes through exactly the values of the
// one-probe-at-a-time march.
template <class Emit>
__device__ __forceinline__ void march_intervals(const Table16& t, const float* o, const float* d, float ray_near,
                                                float ray_far, float cell_step, float grid_step, float cell2grid,
                                                Emit&& emit) {
    constexpr int kAhead = 4;
    float tt = ray_near, seg_near = ray_near;
    bool guess_active = true;
    while (tt < ray_far) {
        const float stride_guess = guess_active ? cell_step : grid_step;
        float ts[kAhead];
        ProbeStart ps[kAhead];
        float t_k = tt;
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            ts[a] = t_k;
            float p[3];
            ray_at(o, d, t_k, p);
            ps[a] = probe_begin(t, p, cell2grid, t_k < ray_far);
            t_k += stride_guess;
        }
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
            if (!(ts[a] < ray_far)) {
                tt = ts[a];
                break;
            }
            const bool active = probe_finish(t, ps[a]);
            if (active) {
                tt = ts[a] + cell_step;
                emit(seg_near, tt);
                seg_near = tt;
            } else {
                tt = ts[a] + grid_step;
            }
            if (active != guess_active) {
                guess_active = active;
                break;
            }
        }
    }
}

}  // namespace ashb
