// Depth-wise window convolution over the sparse-dense structure (sm_100a),
// driven by the radius-R neighbour lookup tables of ash/grid.py:494-502.
// Semantics follow ash/src/grid.cu:951-1043: out[g, c, :] = sum over the K window
// taps k of in[neighbour_k(g, c), :] * w[k, :], skipping taps whose block is absent.
//
// One CTA works on one active block: its row of the block-neighbour table is
// staged in shared memory once, and a group of lanes shares each output cell
// (lane j owns VEC channels) so that every tap is one coalesced vector load.
#include "common.cuh"

namespace ashb {

constexpr int kMaxGridNbs = 125;  // block window of radius <= 2

template <typename T, int VEC>
__global__ void __launch_bounds__(256) conv_forward_kernel(
        const T* __restrict__ in, const T* __restrict__ w, const uint8_t* __restrict__ masks,
        const int64_t* __restrict__ grid_indices, const int64_t* __restrict__ cell_indices,
        const int64_t* __restrict__ g2g, const int64_t* __restrict__ c2c, const int64_t* __restrict__ c2g,
        T* __restrict__ out, int num_cell_nbs, int num_grid_nbs, int64_t cells_per_grid, int D, int lane_shift,
        int64_t n_emb) {
    __shared__ int64_t nb_block[kMaxGridNbs];
    const int64_t grid_i = blockIdx.x;
    const int64_t grid_idx = grid_indices[grid_i];
    const bool block_ok = grid_idx >= 0 && grid_idx < n_emb;
    for (int k = threadIdx.x; k < num_grid_nbs; k += blockDim.x)
        nb_block[k] = block_ok ? g2g[grid_idx * num_grid_nbs + k] : -1;
    __syncthreads();
    if (!block_ok) return;

    const int lanes = 1 << lane_shift;
    const int lane = threadIdx.x & (lanes - 1);
    const int ch = lane * VEC;
    if (ch >= D) return;
    const int cells_per_pass = blockDim.x >> lane_shift;
    for (int64_t cell_i = threadIdx.x >> lane_shift; cell_i < cells_per_grid; cell_i += cells_per_pass) {
        if (!masks[grid_i * cells_per_grid + cell_i]) continue;  // grid.cu:968-969
        const int64_t cell_idx = cell_indices[cell_i];
        const int64_t* nb_cell = c2c + (int64_t)num_cell_nbs * cell_idx;
        const int64_t* nb_cg = c2g + (int64_t)num_cell_nbs * cell_idx;
        T acc[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = 0;
        for (int k = 0; k < num_cell_nbs; ++k) {
            const int64_t gnb = __ldg(nb_cg + k);
            const int64_t g = (gnb >= 0 && gnb < num_grid_nbs) ? nb_block[gnb] : -1;
            if (g < 0 || g >= n_emb) continue;
            const T* src = in + (g * cells_per_grid + __ldg(nb_cell + k)) * D + ch;
            const T* wk = w + (int64_t)k * D + ch;
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] += __ldg(src + v) * __ldg(wk + v);
        }
        T* dst = out + (grid_idx * cells_per_grid + cell_idx) * D + ch;
#pragma unroll
        for (int v = 0; v < VEC; ++v) dst[v] = acc[v];
    }
}

// ---- shared-memory tiled variant ---------------------------------------------------------
// For the window the Python layer actually builds (radius R <= G, two-sided, block window 3^3)
// the two per-cell tables are pure arithmetic, so the kernel needs only the 27-entry block
// row.  One CTA per active block stages the block plus its R-cell halo ((G+2R)^3 cells, CH
// channels at a time) in shared memory -- neighbour blocks are read with coalesced 16-byte
// loads, absent ones count as zero -- and the K^3 weights beside it.  Each thread then
// produces XT outputs that are adjacent in x from one sliding row segment held in registers, so
// a tile value is read from shared memory once per XT outputs and a weight once per XT outputs.
// Taps are accumulated in the reference's order (x fastest, then y, then z).
// RT > 0 fixes the radius at compile time (fully unrolled taps, row segment in registers);
// RT == 0 takes it at run time.
template <int CH, int XT, int RT>
__global__ void __launch_bounds__(256) conv_tiled_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                         const int64_t* __restrict__ grid_indices,
                                                         const int64_t* __restrict__ g2g27, float* __restrict__ out,
                                                         int G, int R_arg, int D, int64_t n_emb) {
    extern __shared__ float smem[];
    const int R = RT > 0 ? RT : R_arg;
    const int S = 2 * R + 1, T = G + 2 * R;
    const int cells = G * G * G, taps = S * S * S, tile_cells = T * T * T;
    float* tile = smem;                       // [tile_cells][CH]
    float* wsm = smem + (size_t)tile_cells * CH;  // [taps][CH]
    __shared__ int64_t nb[27];
    const int64_t gidx = grid_indices[blockIdx.x];
    const bool ok = gidx >= 0 && gidx < n_emb;
    if (threadIdx.x < 27) nb[threadIdx.x] = ok ? g2g27[gidx * 27 + threadIdx.x] : -1;
    __syncthreads();
    if (!ok) return;
    const int xt_per_row = G / XT;
    const int n_items = G * G * xt_per_row;  // (z, y, x-chunk) work items
    for (int ch0 = 0; ch0 < D; ch0 += CH) {
        for (int k = threadIdx.x; k < taps * CH; k += blockDim.x) wsm[k] = w[(int64_t)(k / CH) * D + ch0 + (k % CH)];
        for (int h = threadIdx.x; h < tile_cells; h += blockDim.x) {
            const int hx = h % T, hy = (h / T) % T, hz = h / (T * T);
            const int cx = hx - R, cy = hy - R, cz = hz - R;            // cell coordinate relative to this block
            const int bx = cx < 0 ? -1 : (cx >= G ? 1 : 0), by = cy < 0 ? -1 : (cy >= G ? 1 : 0),
                      bz = cz < 0 ? -1 : (cz >= G ? 1 : 0);
            const int64_t g = nb[(bx + 1) + (by + 1) * 3 + (bz + 1) * 9];
            float v[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) v[c] = 0.f;
            if (g >= 0 && g < n_emb) {
                const int lin = (cx - bx * G) + ((cy - by * G) + (cz - bz * G) * G) * G;
                const float* src = in + (g * cells + lin) * D + ch0;
                if (CH == 4) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4*>(src));
                    v[0] = t4.x, v[1] = t4.y, v[2] = t4.z, v[3] = t4.w;
                } else {
#pragma unroll
                    for (int c = 0; c < CH; ++c) v[c] = __ldg(src + c);
                }
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) tile[(size_t)h * CH + c] = v[c];
        }
        __syncthreads();
        for (int item = threadIdx.x; item < n_items; item += blockDim.x) {
            const int xc = item % xt_per_row, y = (item / xt_per_row) % G, z = item / (xt_per_row * G);
            const int x0 = xc * XT;
            float acc[XT][CH];
#pragma unroll
            for (int o = 0; o < XT; ++o)
#pragma unroll
                for (int c = 0; c < CH; ++c) acc[o][c] = 0.f;
            for (int kz = 0; kz < S; ++kz)
                for (int ky = 0; ky < S; ++ky) {
                    const float* row = tile + ((size_t)((z + kz) * T + (y + ky)) * T + x0) * CH;
                    const float* wrow = wsm + (size_t)((kz * S + ky) * S) * CH;
                    // sliding window along x: XT outputs share the S + XT - 1 inputs of this row
                    if constexpr (RT > 0) {
                        constexpr int SS = 2 * RT + 1;
                        float seg[SS + XT - 1][CH];
#pragma unroll
                        for (int i = 0; i < SS + XT - 1; ++i)
#pragma unroll
                            for (int c = 0; c < CH; ++c) seg[i][c] = row[i * CH + c];
#pragma unroll
                        for (int kx = 0; kx < SS; ++kx) {
                            float wv[CH];
#pragma unroll
                            for (int c = 0; c < CH; ++c) wv[c] = wrow[kx * CH + c];
#pragma unroll
                            for (int o = 0; o < XT; ++o)
#pragma unroll
                                for (int c = 0; c < CH; ++c) acc[o][c] += seg[o + kx][c] * wv[c];
                        }
                    } else {
                        for (int kx = 0; kx < S; ++kx) {
                            float wv[CH];
#pragma unroll
                            for (int c = 0; c < CH; ++c) wv[c] = wrow[kx * CH + c];
#pragma unroll
                            for (int o = 0; o < XT; ++o)
#pragma unroll
                                for (int c = 0; c < CH; ++c) acc[o][c] += row[(o + kx) * CH + c] * wv[c];
                        }
                    }
                }
#pragma unroll
            for (int o = 0; o < XT; ++o) {
                float* dst = out + (gidx * cells + (x0 + o) + (y + z * G) * G) * D + ch0;
#pragma unroll
                for (int c = 0; c < CH; ++c) dst[c] = acc[o][c];
            }
        }
        __syncthreads();
    }
}

// Separable window: weights[z][y][x][c] = wz[z][c] * wy[y][c] * wx[x][c] (a Gaussian is one).  The
// same halo tile is staged, then three 1-D passes run inside shared memory -- along x over the
// whole (G+2R)^2 cross-section, along y over the (G+2R) slabs that remain, along z -- so a
// (2R+1)^3 window costs 3 (2R+1) multiply-adds per cell and channel instead of (2R+1)^3, and the
// intermediate sums never exist for cells outside the tile (absent neighbour blocks count as zero
// exactly as in the full window).  w1: [3][S][D], axis 0 = x.
template <int CH>
__global__ void __launch_bounds__(256) conv_separable_kernel(const float* __restrict__ in, const float* __restrict__ w1,
                                                             const int64_t* __restrict__ grid_indices,
                                                             const int64_t* __restrict__ g2g27, float* __restrict__ out,
                                                             int G, int R, int D, int64_t n_emb) {
    extern __shared__ float smem[];
    const int S = 2 * R + 1, T = G + 2 * R;
    const int cells = G * G * G, tile_cells = T * T * T;
    float* tile = smem;                                   // [T][T][T][CH]; reused for the y-pass sums [T][G][G][CH]
    float* t1 = smem + (size_t)tile_cells * CH;           // x-pass sums [T][T][G][CH]
    float* wsm = t1 + (size_t)T * T * G * CH;             // [3][S][CH]
    __shared__ int64_t nb[27];
    const int64_t gidx = grid_indices[blockIdx.x];
    const bool ok = gidx >= 0 && gidx < n_emb;
    if (threadIdx.x < 27) nb[threadIdx.x] = ok ? g2g27[gidx * 27 + threadIdx.x] : -1;
    __syncthreads();
    if (!ok) return;
    for (int ch0 = 0; ch0 < D; ch0 += CH) {
        for (int k = threadIdx.x; k < 3 * S * CH; k += blockDim.x) wsm[k] = w1[(int64_t)(k / CH) * D + ch0 + (k % CH)];
        for (int h = threadIdx.x; h < tile_cells; h += blockDim.x) {
            const int hx = h % T, hy = (h / T) % T, hz = h / (T * T);
            const int cx = hx - R, cy = hy - R, cz = hz - R;
            const int bx = cx < 0 ? -1 : (cx >= G ? 1 : 0), by = cy < 0 ? -1 : (cy >= G ? 1 : 0),
                      bz = cz < 0 ? -1 : (cz >= G ? 1 : 0);
            const int64_t g = nb[(bx + 1) + (by + 1) * 3 + (bz + 1) * 9];
            float v[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) v[c] = 0.f;
            if (g >= 0 && g < n_emb) {
                const int lin = (cx - bx * G) + ((cy - by * G) + (cz - bz * G) * G) * G;
                const float* src = in + (g * cells + lin) * D + ch0;
                if (CH == 4) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4*>(src));
                    v[0] = t4.x, v[1] = t4.y, v[2] = t4.z, v[3] = t4.w;
                } else {
#pragma unroll
                    for (int c = 0; c < CH; ++c) v[c] = __ldg(src + c);
                }
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) tile[(size_t)h * CH + c] = v[c];
        }
        __syncthreads();
        // along x: t1[z'][y'][x] = sum_k wx[k] * tile[z'][y'][x + k]
        for (int i = threadIdx.x; i < T * T * G; i += blockDim.x) {
            const int x = i % G, zy = i / G;
            const float* row = tile + ((size_t)zy * T + x) * CH;
            float acc[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) acc[c] = 0.f;
            for (int k = 0; k < S; ++k)
#pragma unroll
                for (int c = 0; c < CH; ++c) acc[c] += row[k * CH + c] * wsm[k * CH + c];
#pragma unroll
            for (int c = 0; c < CH; ++c) t1[(size_t)i * CH + c] = acc[c];
        }
        __syncthreads();
        // along y: t2[z'][y][x] = sum_k wy[k] * t1[z'][y + k][x]   (t2 takes the tile's place)
        float* t2 = tile;
        for (int i = threadIdx.x; i < T * G * G; i += blockDim.x) {
            const int x = i % G, y = (i / G) % G, zp = i / (G * G);
            const float* col = t1 + ((size_t)(zp * T + y) * G + x) * CH;
            float acc[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) acc[c] = 0.f;
            for (int k = 0; k < S; ++k)
#pragma unroll
                for (int c = 0; c < CH; ++c) acc[c] += col[(size_t)k * G * CH + c] * wsm[(S + k) * CH + c];
#pragma unroll
            for (int c = 0; c < CH; ++c) t2[(size_t)i * CH + c] = acc[c];
        }
        __syncthreads();
        // along z: out[z][y][x] = sum_k wz[k] * t2[z + k][y][x]
        for (int i = threadIdx.x; i < cells; i += blockDim.x) {
            const float* col = t2 + (size_t)i * CH;
            float acc[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) acc[c] = 0.f;
            for (int k = 0; k < S; ++k)
#pragma unroll
                for (int c = 0; c < CH; ++c) acc[c] += col[(size_t)k * G * G * CH + c] * wsm[(2 * S + k) * CH + c];
            float* dst = out + (gidx * cells + i) * D + ch0;
            if (CH == 4) {
                *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            } else {
#pragma unroll
                for (int c = 0; c < CH; ++c) dst[c] = acc[c];
            }
        }
        __syncthreads();
    }
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_conv_forward(int dtype, const void* inputs, const void* weights, const uint8_t* masks,
                      const int64_t* grid_indices, const int64_t* cell_indices, const int64_t* g2g,
                      const int64_t* c2c, const int64_t* c2g, void* outputs, int zero_output,
                      int64_t num_grids, int64_t n_emb, int64_t cells_per_grid, int64_t D,
                      int64_t num_cell_nbs, int64_t num_grid_nbs, void* stream) {
    ASHB_REQUIRE(dtype == ASHB_F32 || dtype == ASHB_F64, "unknown dtype code %d", dtype);
    ASHB_REQUIRE(D >= 1 && D <= 16, "embedding_dim %lld not in 1..16", (long long)D);
    ASHB_REQUIRE(num_grid_nbs >= 1 && num_grid_nbs <= kMaxGridNbs, "block window of %lld neighbours unsupported",
                 (long long)num_grid_nbs);
    ASHB_REQUIRE(num_grids >= 0 && n_emb >= 1 && cells_per_grid >= 1 && num_cell_nbs >= 1, "bad sizes");
    ASHB_REQUIRE(outputs != nullptr, "null outputs");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elem = dtype == ASHB_F32 ? 4 : 8;
    if (zero_output)  // grid.cu:1016: rows of inactive blocks stay zero
        ASHB_CUDA_TRY(cudaMemsetAsync(outputs, 0, (size_t)n_emb * cells_per_grid * D * elem, st));
    if (num_grids == 0) return ASHB_OK;
    ASHB_REQUIRE(inputs && weights && masks && grid_indices && cell_indices && g2g && c2c && c2g, "null buffer");
    int shift = 0;
    while ((1 << shift) < D) ++shift;
    const unsigned grid = (unsigned)num_grids;
    if (dtype == ASHB_F32)
        conv_forward_kernel<float, 1><<<grid, 256, 0, st>>>(
                static_cast<const float*>(inputs), static_cast<const float*>(weights), masks, grid_indices,
                cell_indices, g2g, c2c, c2g, static_cast<float*>(outputs), (int)num_cell_nbs, (int)num_grid_nbs,
                cells_per_grid, (int)D, shift, n_emb);
    else
        conv_forward_kernel<double, 1><<<grid, 256, 0, st>>>(
                static_cast<const double*>(inputs), static_cast<const double*>(weights), masks, grid_indices,
                cell_indices, g2g, c2c, c2g, static_cast<double*>(outputs), (int)num_cell_nbs,
                (int)num_grid_nbs, cells_per_grid, (int)D, shift, n_emb);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_conv_forward_tiled(const float* inputs, const float* weights, const int64_t* grid_indices,
                            const int64_t* lut_grid_nb27, float* outputs, int zero_output, int64_t num_grids,
                            int64_t n_emb, int G, int radius, int64_t D, void* stream) {
    ASHB_REQUIRE(D >= 1 && D <= 16, "embedding_dim %lld not in 1..16", (long long)D);
    ASHB_REQUIRE(G >= 1 && G <= 16 && radius >= 1 && radius <= G, "window radius %d must be within one block (G=%d)",
                 radius, G);
    ASHB_REQUIRE(num_grids >= 0 && n_emb >= 1 && outputs != nullptr, "bad sizes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t cells = (int64_t)G * G * G;
    if (zero_output) ASHB_CUDA_TRY(cudaMemsetAsync(outputs, 0, (size_t)n_emb * cells * D * sizeof(float), st));
    if (num_grids == 0) return ASHB_OK;
    ASHB_REQUIRE(inputs && weights && grid_indices && lut_grid_nb27, "null buffer");
    const int ch = (D % 4 == 0 && (((uintptr_t)inputs) & 15) == 0) ? 4 : (D % 2 == 0 ? 2 : 1);
    const int T = G + 2 * radius, S = 2 * radius + 1;
    const size_t smem = ((size_t)T * T * T + (size_t)S * S * S) * ch * sizeof(float);
    ASHB_REQUIRE(smem <= 200 * 1024, "halo tile of %zu bytes does not fit in shared memory", smem);
    const int xt = G % 4 == 0 ? 4 : (G % 2 == 0 ? 2 : 1);
    const int items = G * G * (G / xt);
    const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
#define ASHB_CONV_LAUNCH(CH, XT, RT)                                                                        \
    {                                                                                                       \
        if (smem > 48 * 1024)                                                                               \
            ASHB_CUDA_TRY(cudaFuncSetAttribute(conv_tiled_kernel<CH, XT, RT>,                               \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
        conv_tiled_kernel<CH, XT, RT><<<(unsigned)num_grids, threads, smem, st>>>(                          \
                inputs, weights, grid_indices, lut_grid_nb27, outputs, G, radius, (int)D, n_emb);           \
    }
#define ASHB_CONV_RADIUS(CH, XT)                                   \
    switch (radius) {                                              \
        case 1: ASHB_CONV_LAUNCH(CH, XT, 1) break;                 \
        case 2: ASHB_CONV_LAUNCH(CH, XT, 2) break;                 \
        case 3: ASHB_CONV_LAUNCH(CH, XT, 3) break;                 \
        default: ASHB_CONV_LAUNCH(CH, XT, 0)                       \
    }
    if (ch == 4 && xt == 4) ASHB_CONV_RADIUS(4, 4)
    else if (ch == 4 && xt == 2) ASHB_CONV_RADIUS(4, 2)
    else if (ch == 4) ASHB_CONV_RADIUS(4, 1)
    else if (ch == 2 && xt == 4) ASHB_CONV_RADIUS(2, 4)
    else if (ch == 2 && xt == 2) ASHB_CONV_RADIUS(2, 2)
    else if (ch == 2) ASHB_CONV_RADIUS(2, 1)
    else if (xt == 4) ASHB_CONV_RADIUS(1, 4)
    else if (xt == 2) ASHB_CONV_RADIUS(1, 2)
    else ASHB_CONV_RADIUS(1, 1)
#undef ASHB_CONV_RADIUS
#undef ASHB_CONV_LAUNCH
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_conv_forward_separable(const float* inputs, const float* weights_1d, const int64_t* grid_indices,
                                const int64_t* lut_grid_nb27, float* outputs, int zero_output, int64_t num_grids,
                                int64_t n_emb, int G, int radius, int64_t D, void* stream) {
    ASHB_REQUIRE(D >= 1 && D <= 16, "embedding_dim %lld not in 1..16", (long long)D);
    ASHB_REQUIRE(G >= 1 && G <= 16 && radius >= 1 && radius <= G, "window radius %d must be within one block (G=%d)",
                 radius, G);
    ASHB_REQUIRE(num_grids >= 0 && n_emb >= 1 && outputs != nullptr, "bad sizes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t cells = (int64_t)G * G * G;
    if (zero_output) ASHB_CUDA_TRY(cudaMemsetAsync(outputs, 0, (size_t)n_emb * cells * D * sizeof(float), st));
    if (num_grids == 0) return ASHB_OK;
    ASHB_REQUIRE(inputs && weights_1d && grid_indices && lut_grid_nb27, "null buffer");
    const int ch = (D % 4 == 0 && ((((uintptr_t)inputs) | ((uintptr_t)outputs)) & 15) == 0) ? 4 : (D % 2 == 0 ? 2 : 1);
    const int T = G + 2 * radius, S = 2 * radius + 1;
    const size_t smem = ((size_t)T * T * T + (size_t)T * T * G + (size_t)3 * S) * ch * sizeof(float);
    ASHB_REQUIRE(smem <= 200 * 1024, "halo tile of %zu bytes does not fit in shared memory", smem);
#define ASHB_SEP_LAUNCH(CH)                                                                                   \
    {                                                                                                         \
        if (smem > 48 * 1024)                                                                                 \
            ASHB_CUDA_TRY(cudaFuncSetAttribute(conv_separable_kernel<CH>,                                     \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
        conv_separable_kernel<CH><<<(unsigned)num_grids, 256, smem, st>>>(inputs, weights_1d, grid_indices,   \
                                                                           lut_grid_nb27, outputs, G, radius, \
                                                                           (int)D, n_emb);                    \
    }
    if (ch == 4) ASHB_SEP_LAUNCH(4)
    else if (ch == 2) ASHB_SEP_LAUNCH(2)
    else ASHB_SEP_LAUNCH(1)
#undef ASHB_SEP_LAUNCH
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
