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

}  // extern "C"
