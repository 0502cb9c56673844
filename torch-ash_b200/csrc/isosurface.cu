// Vertex-only iso-surface extraction over the sparse-dense structure (sm_100a).
// Semantics follow ash/src/grid.cu:453-604: every cell of the listed blocks whose weight
// reaches the threshold looks at its +x, +y, +z neighbour in turn; a sign change of
// (sdf - iso_value) towards a neighbour that also has enough weight emits the linearly
// interpolated crossing, in cell units.  A missing neighbour BLOCK ends the cell's loop, later
// axes included (grid.cu:508-510).  The output order is unspecified, as in the reference.
//
// One thread per (block, cell); the output cursor is bumped once per warp per axis (ballot +
// one atomic) instead of once per vertex.  FILL = false only counts.
#include "common.cuh"

namespace ashb {

template <bool FILL>
__global__ void __launch_bounds__(256) isosurface_kernel(
        const float* __restrict__ sdfs, const float* __restrict__ weights, const int64_t* __restrict__ grid_indices,
        const int32_t* __restrict__ grid_coords, const int64_t* __restrict__ g2g,
        const int32_t* __restrict__ cell_coords, const int64_t* __restrict__ c2c, const int64_t* __restrict__ c2g,
        unsigned long long* cursor, float* __restrict__ positions, int64_t max_out, float iso_value, float weight_thr,
        int grid_dim, int64_t cells, int64_t n_emb, int64_t len) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool alive = i < len;
    int64_t grid_idx = 0, cell_idx = 0;
    float self_iso = 0.f;
    if (alive) {
        grid_idx = grid_indices[i / cells];
        cell_idx = i % cells;
        alive = grid_idx >= 0 && grid_idx < n_emb;
    }
    if (alive) {
        self_iso = sdfs[grid_idx * cells + cell_idx] - iso_value;
        alive = weights[grid_idx * cells + cell_idx] >= weight_thr;
    }
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        bool emit = false;
        float ratio = 0.f;
        if (alive) {
            const int cell_nb = 1 << d;
            const int64_t gnb = c2g[cell_idx * 8 + cell_nb] & 7;
            const int64_t nb_grid = g2g[grid_idx * 8 + gnb];
            if (nb_grid < 0 || nb_grid >= n_emb) {
                alive = false;  // the reference returns here: no later axis either
            } else {
                const int64_t nb_cell = c2c[cell_idx * 8 + cell_nb];
                const float nb_iso = sdfs[nb_grid * cells + nb_cell] - iso_value;
                if (self_iso * nb_iso < 0.f && weights[nb_grid * cells + nb_cell] >= weight_thr) {
                    emit = true;
                    ratio = self_iso / (self_iso - nb_iso);
                }
            }
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, emit);
        if (ballot == 0) continue;
        const int leader = __ffs(ballot) - 1;
        unsigned long long base = 0;
        if ((int)(threadIdx.x & 31) == leader) base = atomicAdd(cursor, (unsigned long long)__popc(ballot));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (FILL && emit) {
            const int64_t o = (int64_t)base + __popc(ballot & lanemask_lt());
            if (o < max_out) {
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    const int self_pos = grid_coords[grid_idx * 3 + k] * grid_dim + cell_coords[cell_idx * 3 + k];
                    positions[o * 3 + k] = (float)self_pos + (k == d ? ratio : 0.f);
                }
            }
        }
    }
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_isosurface_extraction(const float* sdfs, const float* weights, const int64_t* grid_indices,
                               const int32_t* grid_coords_table, const int64_t* lut_grid_nb2grid_idx,
                               const int32_t* cell_coords_table, const int64_t* lut_cell_nb2cell_idx,
                               const int64_t* lut_cell_nb2grid_nb, float* positions, int64_t max_out,
                               int64_t* n_out, void* cursor_dev, float iso_value, float weight_thr, int grid_dim,
                               int64_t cells_per_grid, int64_t n_emb, int64_t num_grids, void* stream) {
    ASHB_REQUIRE(n_out != nullptr && cursor_dev != nullptr, "null counter");
    ASHB_REQUIRE(num_grids >= 0 && cells_per_grid >= 1 && n_emb >= 1 && max_out >= 0, "bad sizes");
    *n_out = 0;
    if (num_grids == 0) return ASHB_OK;
    ASHB_REQUIRE(sdfs && weights && grid_indices && grid_coords_table && lut_grid_nb2grid_idx && cell_coords_table &&
                         lut_cell_nb2cell_idx && lut_cell_nb2grid_nb,
                 "null buffer");
    ASHB_REQUIRE(max_out == 0 || positions != nullptr, "null output");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long* cursor = static_cast<unsigned long long*>(cursor_dev);
    ASHB_CUDA_TRY(cudaMemsetAsync(cursor, 0, sizeof(unsigned long long), st));
    const int64_t len = num_grids * cells_per_grid;
    const unsigned grid = (unsigned)((len + 255) / 256);
    if (positions != nullptr && max_out > 0)
        isosurface_kernel<true><<<grid, 256, 0, st>>>(sdfs, weights, grid_indices, grid_coords_table,
                                                      lut_grid_nb2grid_idx, cell_coords_table, lut_cell_nb2cell_idx,
                                                      lut_cell_nb2grid_nb, cursor, positions, max_out, iso_value,
                                                      weight_thr, grid_dim, cells_per_grid, n_emb, len);
    else
        isosurface_kernel<false><<<grid, 256, 0, st>>>(sdfs, weights, grid_indices, grid_coords_table,
                                                       lut_grid_nb2grid_idx, cell_coords_table, lut_cell_nb2cell_idx,
                                                       lut_cell_nb2grid_nb, cursor, nullptr, 0, iso_value, weight_thr,
                                                       grid_dim, cells_per_grid, n_emb, len);
    ASHB_LAUNCH_CHECK();
    unsigned long long total = 0;
    ASHB_CUDA_TRY(cudaMemcpyAsync(&total, cursor, sizeof(total), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    *n_out = (int64_t)total;
    return ASHB_OK;
}

}  // extern "C"
