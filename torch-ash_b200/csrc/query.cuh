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

}  // namespace ashb
