// Triangle mesh of the iso-surface over the sparse-dense structure (sm_100a): marching cubes
// in three launches and ONE host read.  Stages and validity rules follow ash/src/grid.cu:607-946:
// a cube sits at every cell of a listed block whose own weight and the weights of its 8 corners
// (the cell and its +x/+y/+z neighbours through the lookup tables) reach the threshold and whose
// neighbour blocks all exist; corner c is inside when sdf - iso < 0; every cut edge of a valid
// cube gets one vertex, owned by the cell at the edge's lower corner, placed by linear
// interpolation; triangles index those vertices.
//
//   classify   per cell: corner pattern -> codes[]; each cut edge is requested at its owner with an
//              atomic exchange, so the number of distinct vertices is counted in the same pass, as
//              is the number of triangles (one atomic per warp each)
//   (host reads the two counts and allocates)
//   vertices   per cell and direction: requested edges get a slot (one atomic per warp) and a position
//   triangles  per cell: slots for its triangles (warp scan + one atomic per warp), vertex ids
//              looked up at the owners
//
// The triangulation table is this repository's own (mc_tables.h, derived by gen_mc_tables.py):
// the reference's table is not reproduced, so which diagonal splits an ambiguous pattern, the
// order of a triangle's corners and the output order are not comparable with the reference;
// vertex positions are.
#include "common.cuh"

#define ASHB_MC_TABLE static __device__ const
#include "mc_tables.h"

namespace ashb {

constexpr int kEdgeUnwanted = (int)0xFEFEFEFE;  // what a byte-wise fill with 0xFE leaves
constexpr int kEdgeWanted = -1;

struct McLuts {
    const int64_t* __restrict__ grid_indices;
    const int64_t* __restrict__ g2g;
    const int64_t* __restrict__ c2c;
    const int64_t* __restrict__ c2g;
    int64_t cells, n_emb, len;
};

// Flat (embedding row * cells + cell) address of corner c of the cube at (grid_idx, cell_idx), or -1.
__device__ __forceinline__ int64_t corner_address(const McLuts& L, int64_t grid_idx, int64_t cell_idx, int c) {
    const int64_t g = L.g2g[grid_idx * 8 + (L.c2g[cell_idx * 8 + c] & 7)];
    if (g < 0 || g >= L.n_emb) return -1;
    const int64_t cc = L.c2c[cell_idx * 8 + c];
    if (cc < 0 || cc >= L.cells) return -1;
    return g * L.cells + cc;
}

__device__ __forceinline__ int edge_lower_corner(int e) {
    const int d = e >> 2, j = e & 3;
    return ((j & 1) << ((d + 1) % 3)) | ((j >> 1) << ((d + 2) % 3));
}

__global__ void __launch_bounds__(256) mc_classify_kernel(const float* __restrict__ sdfs,
                                                          const float* __restrict__ weights, McLuts L,
                                                          uint8_t* __restrict__ codes, int* __restrict__ edge_vertex,
                                                          unsigned long long* __restrict__ counters, float iso_value,
                                                          float weight_thr) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int code = 0;
    int64_t corner[8];
    if (i < L.len) {
        const int64_t grid_idx = L.grid_indices[i / L.cells];
        const int64_t cell_idx = i % L.cells;
        bool valid = grid_idx >= 0 && grid_idx < L.n_emb;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            corner[c] = valid ? corner_address(L, grid_idx, cell_idx, c) : -1;
            valid = valid && corner[c] >= 0;
        }
        if (valid) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                valid = valid && weights[corner[c]] >= weight_thr;
                code |= (int)((sdfs[corner[c]] - iso_value) < 0.f) << c;
            }
        }
        if (!valid || code == 255) code = 0;
        codes[i] = (uint8_t)code;
    }
    int new_vertices = 0;
    if (code) {
        const int mask = kMcEdgeMask[code];
#pragma unroll
        for (int e = 0; e < 12; ++e) {
            if (!(mask & (1 << e))) continue;
            const int old = atomicExch(edge_vertex + corner[edge_lower_corner(e)] * 3 + (e >> 2), kEdgeWanted);
            new_vertices += old == kEdgeUnwanted;
        }
    }
    const int v = __reduce_add_sync(0xffffffffu, new_vertices);
    const int t = __reduce_add_sync(0xffffffffu, code ? (int)kMcTriCount[code] : 0);
    if ((threadIdx.x & 31) == 0) {
        if (v) atomicAdd(counters, (unsigned long long)v);
        if (t) atomicAdd(counters + 1, (unsigned long long)t);
    }
}

__global__ void __launch_bounds__(256) mc_vertex_kernel(const float* __restrict__ sdfs, McLuts L,
                                                        const int32_t* __restrict__ grid_coords,
                                                        const int32_t* __restrict__ cell_coords,
                                                        int* __restrict__ edge_vertex,
                                                        unsigned long long* __restrict__ cursor,
                                                        float* __restrict__ vertices, int64_t max_vertices,
                                                        float iso_value, int grid_dim) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < L.len;
    int64_t grid_idx = 0, cell_idx = 0, self = 0;
    if (live) {
        grid_idx = L.grid_indices[i / L.cells];
        cell_idx = i % L.cells;
        self = grid_idx * L.cells + cell_idx;
    }
    const bool in_range = live && grid_idx >= 0 && grid_idx < L.n_emb;
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        const bool emit = in_range && edge_vertex[self * 3 + d] == kEdgeWanted;
        const unsigned ballot = __ballot_sync(0xffffffffu, emit);
        if (ballot == 0) continue;
        const int leader = __ffs(ballot) - 1;
        unsigned long long base = 0;
        if ((int)(threadIdx.x & 31) == leader) base = atomicAdd(cursor, (unsigned long long)__popc(ballot));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (!emit) continue;
        const int64_t o = (int64_t)base + __popc(ballot & lanemask_lt());
        edge_vertex[self * 3 + d] = (int)o;
        const int64_t nb = corner_address(L, grid_idx, cell_idx, 1 << d);
        if (o >= max_vertices || nb < 0) continue;  // cannot happen for edges a valid cube requested
        const float self_iso = sdfs[self] - iso_value;
        const float nb_iso = sdfs[nb] - iso_value;
        const float ratio = self_iso / (self_iso - nb_iso);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const int self_pos = grid_coords[grid_idx * 3 + k] * grid_dim + cell_coords[cell_idx * 3 + k];
            vertices[o * 3 + k] = (float)self_pos + (k == d ? ratio : 0.f);
        }
    }
}

__global__ void __launch_bounds__(256) mc_triangle_kernel(McLuts L, const uint8_t* __restrict__ codes,
                                                          const int* __restrict__ edge_vertex,
                                                          unsigned long long* __restrict__ cursor,
                                                          int32_t* __restrict__ triangles, int64_t max_triangles) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int code = i < L.len ? codes[i] : 0;
    const int n = code ? (int)kMcTriCount[code] : 0;
    // exclusive scan of the triangle counts over the warp, one atomic for the warp's total
    int incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) return;
    unsigned long long base = 0;
    if (lane == 31) base = atomicAdd(cursor, (unsigned long long)total);
    base = __shfl_sync(0xffffffffu, base, 31);
    if (n == 0) return;
    const int64_t grid_idx = L.grid_indices[i / L.cells];
    const int64_t cell_idx = i % L.cells;
    int64_t out = (int64_t)base + (incl - n);
    for (int t = 0; t < n; ++t, ++out) {
        if (out >= max_triangles) return;
#pragma unroll
        for (int v = 0; v < 3; ++v) {
            const int e = kMcTris[code][3 * t + v];
            const int64_t owner = corner_address(L, grid_idx, cell_idx, edge_lower_corner(e));
            triangles[out * 3 + v] = owner >= 0 ? edge_vertex[owner * 3 + (e >> 2)] : -1;
        }
    }
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_marching_cubes_count(const float* sdfs, const float* weights, const int64_t* grid_indices,
                              const int64_t* lut_grid_nb2grid_idx, const int64_t* lut_cell_nb2cell_idx,
                              const int64_t* lut_cell_nb2grid_nb, uint8_t* codes, int32_t* edge_vertex,
                              void* counters_dev, float iso_value, float weight_thr, int64_t cells_per_grid,
                              int64_t n_emb, int64_t num_grids, int64_t* n_vertices, int64_t* n_triangles,
                              void* stream) {
    ASHB_REQUIRE(n_vertices && n_triangles && counters_dev, "null counter");
    ASHB_REQUIRE(num_grids >= 0 && cells_per_grid >= 1 && n_emb >= 1, "bad sizes");
    *n_vertices = *n_triangles = 0;
    if (num_grids == 0) return ASHB_OK;
    ASHB_REQUIRE(sdfs && weights && grid_indices && lut_grid_nb2grid_idx && lut_cell_nb2cell_idx &&
                         lut_cell_nb2grid_nb && codes && edge_vertex,
                 "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long* counters = static_cast<unsigned long long*>(counters_dev);
    ASHB_CUDA_TRY(cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned long long), st));
    ASHB_CUDA_TRY(cudaMemsetAsync(edge_vertex, 0xFE, (size_t)n_emb * cells_per_grid * 3 * sizeof(int32_t), st));
    const McLuts L{grid_indices, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx, lut_cell_nb2grid_nb,
                   cells_per_grid, n_emb, num_grids * cells_per_grid};
    mc_classify_kernel<<<(unsigned)((L.len + 255) / 256), 256, 0, st>>>(sdfs, weights, L, codes, edge_vertex, counters,
                                                                       iso_value, weight_thr);
    ASHB_LAUNCH_CHECK();
    unsigned long long host[2] = {0, 0};
    ASHB_CUDA_TRY(cudaMemcpyAsync(host, counters, sizeof(host), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    *n_vertices = (int64_t)host[0];
    *n_triangles = (int64_t)host[1];
    return ASHB_OK;
}

int ashb_marching_cubes_fill(const float* sdfs, const int64_t* grid_indices, const int32_t* grid_coords_table,
                             const int64_t* lut_grid_nb2grid_idx, const int32_t* cell_coords_table,
                             const int64_t* lut_cell_nb2cell_idx, const int64_t* lut_cell_nb2grid_nb,
                             const uint8_t* codes, int32_t* edge_vertex, void* counters_dev, float* vertices,
                             int64_t n_vertices, int32_t* triangles, int64_t n_triangles, float iso_value,
                             int grid_dim, int64_t cells_per_grid, int64_t n_emb, int64_t num_grids, void* stream) {
    ASHB_REQUIRE(num_grids >= 0 && cells_per_grid >= 1 && n_emb >= 1 && n_vertices >= 0 && n_triangles >= 0,
                 "bad sizes");
    if (num_grids == 0 || (n_vertices == 0 && n_triangles == 0)) return ASHB_OK;
    ASHB_REQUIRE(sdfs && grid_indices && grid_coords_table && lut_grid_nb2grid_idx && cell_coords_table &&
                         lut_cell_nb2cell_idx && lut_cell_nb2grid_nb && codes && edge_vertex && counters_dev,
                 "null buffer");
    ASHB_REQUIRE((n_vertices == 0 || vertices) && (n_triangles == 0 || triangles), "null output");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long* counters = static_cast<unsigned long long*>(counters_dev);
    ASHB_CUDA_TRY(cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned long long), st));
    const McLuts L{grid_indices, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx, lut_cell_nb2grid_nb,
                   cells_per_grid, n_emb, num_grids * cells_per_grid};
    const unsigned grid = (unsigned)((L.len + 255) / 256);
    mc_vertex_kernel<<<grid, 256, 0, st>>>(sdfs, L, grid_coords_table, cell_coords_table, edge_vertex, counters,
                                           vertices, n_vertices, iso_value, grid_dim);
    ASHB_LAUNCH_CHECK();
    mc_triangle_kernel<<<grid, 256, 0, st>>>(L, codes, edge_vertex, counters + 1, triangles, n_triangles);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
