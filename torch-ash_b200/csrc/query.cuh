// Pieces of the sparse-dense grid query shared by the query kernels and the fused ray renderer:
// interpolation weights, the world-position split and the corner-row addressing.
#pragma once
#include "hashmap.cuh"

namespace ashb {

// ash/src/grid.cu:7-41
template <typename T>
__device__ __forceinline__ T interp_fn(int interp, T x) {
    return interp == ASHB_SMOOTH_STEP ? x * x * (3 - 2 * x) : x;
}
template <typename T>
__device__ __forceinline__ T dinterp_fn(int interp, T x) {
    return interp == ASHB_SMOOTH_STEP ? 6 * x * (1 - x) : T(1);
}

// Per-axis weights of the two corners along each axis and their derivatives.
// w[d][b]: b = 0 -> corner at the cell origin (argument 1 - offset, evaluated
// in float as the reference does, grid.cu:117), b = 1 -> far corner.
template <typename T>
struct AxisWeights {
    T w[3][2];
    T dw[3][2];
    __device__ __forceinline__ void init(int interp, const float* off) {
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            const T x1 = (T)off[d];
            const T x0 = (T)(1.0f - off[d]);
            w[d][0] = interp_fn<T>(interp, x0);
            w[d][1] = interp_fn<T>(interp, x1);
            dw[d][0] = -dinterp_fn<T>(interp, x0);
            dw[d][1] = dinterp_fn<T>(interp, x1);
        }
    }
    __device__ __forceinline__ T weight(int c) const {
        return w[0][c & 1] * w[1][(c >> 1) & 1] * w[2][(c >> 2) & 1];
    }
    __device__ __forceinline__ void grad(int c, T* g) const {
        const int bx = c & 1, by = (c >> 1) & 1, bz = (c >> 2) & 1;
        g[0] = dw[0][bx] * w[1][by] * w[2][bz];
        g[1] = w[0][bx] * dw[1][by] * w[2][bz];
        g[2] = w[0][bx] * w[1][by] * dw[2][bz];
    }
};

// ---- per-lane slices of an embedding row --------------------------------------------------
// A query is served by a group of 2^k lanes; lane j owns VEC consecutive channels of the row.
template <typename T, int VEC>
struct Vec;
template <>
struct Vec<float, 1> { using type = float; };
template <>
struct Vec<float, 2> { using type = float2; };
template <>
struct Vec<float, 4> { using type = float4; };
template <>
struct Vec<double, 1> { using type = double; };
template <>
struct Vec<double, 2> { using type = double2; };

template <typename T, int VEC>
struct Pack {
    T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> load_pack(const T* p) {
    using V = typename Vec<T, VEC>::type;
    Pack<T, VEC> r;
    *reinterpret_cast<V*>(r.v) = __ldg(reinterpret_cast<const V*>(p));
    return r;
}

// Rows of 4 floats per lane are gathered from random lines: naming a 64-byte L2 fetch size keeps
// the DRAM fill to the half line that holds the 64-byte row.
template <>
__device__ __forceinline__ Pack<float, 1> load_pack<float, 1>(const float* p) {
    Pack<float, 1> r;
    asm volatile("ld.global.nc.L2::64B.f32 %0, [%1];" : "=f"(r.v[0]) : "l"(p));
    return r;
}
template <>
__device__ __forceinline__ Pack<float, 2> load_pack<float, 2>(const float* p) {
    Pack<float, 2> r;
    asm volatile("ld.global.nc.L2::64B.v2.f32 {%0,%1}, [%2];" : "=f"(r.v[0]), "=f"(r.v[1]) : "l"(p));
    return r;
}
template <>
__device__ __forceinline__ Pack<double, 1> load_pack<double, 1>(const double* p) {
    Pack<double, 1> r;
    asm volatile("ld.global.nc.L2::64B.f64 %0, [%1];" : "=d"(r.v[0]) : "l"(p));
    return r;
}
template <>
__device__ __forceinline__ Pack<double, 2> load_pack<double, 2>(const double* p) {
    Pack<double, 2> r;
    asm volatile("ld.global.nc.L2::64B.v2.f64 {%0,%1}, [%2];" : "=d"(r.v[0]), "=d"(r.v[1]) : "l"(p));
    return r;
}
template <>
__device__ __forceinline__ Pack<float, 4> load_pack<float, 4>(const float* p) {
    Pack<float, 4> r;
    asm volatile("ld.global.nc.L2::64B.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                 : "l"(p));
    return r;
}

template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, VEC>& r) {
    using V = typename Vec<T, VEC>::type;
    *reinterpret_cast<V*>(p) = *reinterpret_cast<const V*>(r.v);
}

// Gradient scatter: one vector reduction per lane where the hardware has one
// (fp32 x2 / x4 on sm_90+), scalar atomics otherwise.
template <typename T, int VEC>
__device__ __forceinline__ void atomic_add_pack(T* p, const Pack<T, VEC>& r) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) atomicAdd(p + k, r.v[k]);
}
template <>
__device__ __forceinline__ void atomic_add_pack<float, 4>(float* p, const Pack<float, 4>& r) {
    atomicAdd(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
}
template <>
__device__ __forceinline__ void atomic_add_pack<float, 2>(float* p, const Pack<float, 2>& r) {
    atomicAdd(reinterpret_cast<float2*>(p), make_float2(r.v[0], r.v[1]));
}

template <typename T>
__device__ __forceinline__ T group_sum(T v, int lanes) {
    for (int o = lanes >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// World position -> (block coordinate, cell inside the block, fractional offset).  The split
// follows the Python layer operation by operation as it evaluates on a CUDA tensor
// (ash/grid.py:192-197, :756, :846): divisions by the cell size and by G are multiplications by
// float reciprocals, each rounded.
__device__ __forceinline__ void split_world_position(const float* xw, const float* org, float inv_cell, float inv_G,
                                                     float G_f, int G, int* blk, int* cell, float* off) {
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        const float xc = __fmul_rn(__fsub_rn(xw[d], org[d]), inv_cell);
        const float bf = floorf(__fmul_rn(xc, inv_G));
        const float local = __fsub_rn(xc, __fmul_rn(bf, G_f));
        const float cf = floorf(local);
        off[d] = __fsub_rn(local, cf);
        blk[d] = (int)bf;
        // `local` can round up to exactly G for tiny negative positions
        cell[d] = min(max((int)cf, 0), G - 1);
    }
}

// Element offsets of the 8 corner rows of a query in block `gi`, cell `cell`: corner cells by
// add-with-carry, the int32 block-neighbour row read only for corners across a +x/+y/+z face.
// False when a needed neighbour block is absent (the reference leaves such queries zero).
__device__ __forceinline__ bool corner_rows(const int32_t* __restrict__ nb_lut, int gi, const int* cell, int G,
                                            int64_t n_emb, int64_t cells_per_grid, int64_t D, int64_t* base) {
    const int32_t* row = nb_lut + (int64_t)gi * 8;
    bool ok = true;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        int cc[3], nb = 0;
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            cc[d] = cell[d] + ((c >> d) & 1);
            if (cc[d] == G) {
                cc[d] = 0;
                nb |= 1 << d;
            }
        }
        const int g = nb ? __ldg(row + nb) : gi;
        ok = ok && g >= 0 && g < n_emb;
        base[c] = ((int64_t)g * cells_per_grid + (cc[0] + (cc[1] + cc[2] * G) * G)) * D;
    }
    return ok;
}

// The same corners as (block index, linear cell index) pairs, for the row-list gradient.
__device__ __forceinline__ bool corner_blocks_cells(const int32_t* __restrict__ nb_lut, int gi, const int* cell, int G,
                                                    int64_t n_emb, int* blocks, int* cells) {
    const int32_t* row = nb_lut + (int64_t)gi * 8;
    bool ok = true;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        int cc[3], nb = 0;
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            cc[d] = cell[d] + ((c >> d) & 1);
            if (cc[d] == G) {
                cc[d] = 0;
                nb |= 1 << d;
            }
        }
        const int g = nb ? __ldg(row + nb) : gi;
        ok = ok && g >= 0 && g < n_emb;
        blocks[c] = g;
        cells[c] = cc[0] + (cc[1] + cc[2] * G) * G;
    }
    return ok;
}

}  // namespace ashb
