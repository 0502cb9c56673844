/*
 * libashb200 -- C ABI of the B200 (sm_100a) implementation of torch-ash's
 * native hot path: the collision-free spatial hash engine and the sparse-dense
 * grid kernels.  It replaces the reference's pybind module `__ash`
 * (ash/src/pybind.cpp:8-38) and its stdgpu dependency.
 *
 * Conventions
 *   - every pointer named *_dev or documented "device" is a CUDA device
 *     pointer owned by the caller and only borrowed for the call;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream); all work is enqueued on it and, unless stated otherwise, the
 *     call returns without synchronising;
 *   - every function returns 0 on success or an ASHB_ERR_* code; a text for
 *     the calling thread's last failure is available from
 *     ashb_last_error_string();
 *   - sizes and counts are int64_t; keys are int32 rows of `key_dim` columns;
 *   - entry points that take an ashb_map select the map's device for the call; those that take only
 *     buffers (ashb_query_*, ashb_conv_*, ashb_tsdf_integrate, ashb_route_by_owner, ashb_peer_route_keys,
 *     ashb_peer_unpack_answers, ashb_routed_unpack_*, ashb_routed_send_z, ashb_rows_scatter_add, ...) launch on
 *     the CURRENT device: the caller makes the buffers' device current first.
 *
 * There is no CPU implementation behind this interface: without a CUDA device
 * every compute entry point fails with ASHB_ERR_CUDA.
 */
#ifndef ASHB200_H_
#define ASHB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASHB_OK 0
#define ASHB_ERR_INVALID 1   /* bad argument (dimension, size, null pointer, dtype code) */
#define ASHB_ERR_CUDA 2      /* a CUDA runtime call failed */
#define ASHB_ERR_UNSUPPORTED 3

/* Bits of the device-side status word returned by ashb_map_status(). */
#define ASHB_STATUS_CAPACITY 1u   /* an insert needed more than `capacity` indices; the key was dropped */
#define ASHB_STATUS_PROBE 2u      /* a probe sequence visited every slot without finishing */
#define ASHB_STATUS_SPIN 4u       /* a bounded wait on a slot being written ran out */
#define ASHB_STATUS_DUPLICATE 8u  /* load_states met a key twice */

/* dtype / interpolation codes of the grid entry points */
#define ASHB_F32 0
#define ASHB_F64 1
#define ASHB_LINEAR 0
#define ASHB_SMOOTH_STEP 1

typedef struct ashb_map ashb_map;

const char* ashb_last_error_string(void);
int ashb_version(void);

/* ---------------------------------------------------------------- hash engine */

/* Replaces HashMap::HashMap / HashMapGPUImpl ctor (ash/src/hashmap.cpp:8-18,
 * ash/src/hashmap_gpu.cuh:119-137, ash/src/hashmap_impl.h:11-24).
 * key_dim in 1..4.  heap_dev: caller-owned int32[capacity] free-index stack,
 * aliased for the life of the map, mutated in place and NOT rewritten here.
 * device: CUDA ordinal the map lives on. */
int ashb_map_create(int key_dim, int64_t capacity, int32_t* heap_dev, int device, ashb_map** out);

/* Replaces ~HashMapGPUImpl (ash/src/hashmap_gpu.cuh:127, :134-137). */
int ashb_map_destroy(ashb_map* map);

/* Replaces HashMapGPUImpl::clear + HashMapImpl::reset_heap
 * (ash/src/hashmap_gpu.cuh:355-358, ash/src/hashmap_impl.h:26-33). */
int ashb_map_clear(ashb_map* map, void* stream);

/* Replaces HashMapGPUImpl::size (ash/src/hashmap_gpu.cuh:157).  Synchronises `stream`. */
int ashb_map_size(ashb_map* map, void* stream, int64_t* size_out);

/* Reads and clears the device status word (ASHB_STATUS_* bits).  Synchronises
 * `stream`.  The reference has no counterpart: it prints from the device or
 * has undefined behaviour (ash/src/hashmap_gpu.cuh:226-227, :420). */
int ashb_map_status(ashb_map* map, void* stream, uint32_t* status_out);

/* The same without waiting: the status word is copied to status_out_host (host memory, pinned for
 * the copy to be asynchronous) and cleared, both enqueued on `stream`; the caller reads the host
 * word once work it enqueued later on that stream (an event) has completed.  No counterpart in the
 * reference. */
int ashb_map_status_async(ashb_map* map, uint32_t* status_out_host, void* stream);

/* Replaces find_kernel + HashMapGPUImpl::find (ash/src/hashmap_gpu.cuh:164-208).
 * keys_dev int32[n][key_dim]; indices_dev int64[n] (0 on a miss); masks_dev
 * uint8[n] (1 hit / 0 miss).  Every output element is written. */
int ashb_map_find(ashb_map* map, const int32_t* keys_dev, int64_t n, int64_t* indices_dev,
                  uint8_t* masks_dev, void* stream);

/* Replaces insert_kernel (keys) + insert_keys (ash/src/hashmap_gpu.cuh:212-247).
 * Insert-if-absent; each new key takes heap[counter++]. */
int ashb_map_insert_keys(ashb_map* map, const int32_t* keys_dev, int64_t n, void* stream);

/* Replaces insert_kernel (values) + insert + ValueContext
 * (ash/src/hashmap_gpu.cuh:23-114, :250-313).  For each NEW key i with index
 * idx, row i of src_dev[j] (row_bytes[j] bytes) is copied to row idx of
 * dst_dev[j], j < n_values <= 16.  src_dev/dst_dev/row_bytes are HOST arrays of
 * device pointers / sizes. */
int ashb_map_insert_values(ashb_map* map, const int32_t* keys_dev, int64_t n, int n_values,
                           const void* const* src_dev, void* const* dst_dev,
                           const int64_t* row_bytes, void* stream);

/* Replaces erase_kernel + erase (ash/src/hashmap_gpu.cuh:317-351): each erased
 * key pushes its index back, heap[--counter] = idx. */
int ashb_map_erase(ashb_map* map, const int32_t* keys_dev, int64_t n, void* stream);

/* Replaces HashMapGPUImpl::items (ash/src/hashmap_gpu.cuh:377-405).  Writes up
 * to max_n active (key, index) pairs, order unspecified; *n_out (host) gets the
 * number of active pairs found.  Synchronises `stream`. */
int ashb_map_items(ashb_map* map, int32_t* keys_out_dev, int64_t* indices_out_dev, int64_t max_n,
                   int64_t* n_out, void* stream);

/* Replaces load_states_kernel + load_states (ash/src/hashmap_gpu.cuh:408-450):
 * the table is emptied, counter = n, heap contents copied from heap_src_dev
 * (may alias the map's heap), every (key, index) pair stored verbatim. */
int ashb_map_load_states(ashb_map* map, const int32_t* keys_dev, const int64_t* indices_dev,
                         int64_t n, const int32_t* heap_src_dev, void* stream);

/* Rebuilds the table from its live entries, dropping the tombstones that erase leaves behind
 * (open addressing keeps erased slots occupied so that probe chains stay intact; after heavy
 * insert / erase traffic they lengthen every probe).  Indices, heap and size are unchanged.  The
 * reference has no counterpart: its chained third-party map frees nodes on erase.  Allocates a
 * second table for the duration of the call (cudaMalloc / cudaFree: the table is transiently
 * doubled, and the call is illegal inside stream capture), synchronises `stream` and frees the old
 * table: no other stream may still have work queued that probes this map. */
int ashb_map_rehash(ashb_map* map, void* stream);

/* ---------------------------------------------------------------- grid query
 * Layouts (ash/grid_query.py:40-55): embeddings [n_emb][cells_per_grid][D]
 * (D <= 16), offsets float32 [n][3] (always float32, ash/src/grid.cu:71),
 * grid_indices / cell_indices int64 [n], masks uint8 [n], lut_grid_nb2grid_idx
 * int64 [n_emb][8] (-1 = absent block), lut_cell_nb2cell_idx and
 * lut_cell_nb2grid_nb int64 [cells_per_grid][8].  dtype = ASHB_F32 | ASHB_F64
 * is the type of embeddings and of every floating output/input except offsets.
 */

/* Replaces query_forward_kernel + query_forward (ash/src/grid.cu:69-175).
 * out [n][D]; rows of masked-out queries and of queries with an absent
 * neighbour block are written as zeros (the reference zero-fills first). */
int ashb_query_forward(int dtype, int interp, const void* embeddings, const float* offsets,
                       const int64_t* grid_indices, const int64_t* cell_indices,
                       const uint8_t* masks, const int64_t* lut_grid_nb2grid_idx,
                       const int64_t* lut_cell_nb2cell_idx, const int64_t* lut_cell_nb2grid_nb,
                       void* out, int64_t n, int64_t n_emb, int64_t cells_per_grid, int64_t D,
                       void* stream);

/* Replaces query_backward_forward_kernel + host (ash/src/grid.cu:178-307).
 * z [n][D].  grad_offsets [n][3] is fully written.  grad_embeddings
 * [n_emb][cells][D] is ACCUMULATED into (atomic adds); pass zero_grad != 0 to
 * have it zero-filled on `stream` first, which reproduces the reference's fresh
 * dense gradient. */
int ashb_query_backward_forward(int dtype, int interp, const void* z, const void* embeddings,
                                const float* offsets, const int64_t* grid_indices,
                                const int64_t* cell_indices, const uint8_t* masks,
                                const int64_t* lut_grid_nb2grid_idx,
                                const int64_t* lut_cell_nb2cell_idx,
                                const int64_t* lut_cell_nb2grid_nb, void* grad_embeddings,
                                void* grad_offsets, int zero_grad, int64_t n, int64_t n_emb,
                                int64_t cells_per_grid, int64_t D, void* stream);

/* Replaces query_backward_backward_kernel + host (ash/src/grid.cu:310-451).
 * grad_grad_offsets [n][3], z [n][D]; grad_z [n][D] is fully written;
 * grad_embeddings accumulated as above.  The reference's third output
 * (grad_offsets) is identically zero (grid.cu:417-418) and its first input
 * (grad_grad_embeddings) is unused (grid.cu:426); neither crosses this ABI. */
int ashb_query_backward_backward(int dtype, int interp, const void* grad_grad_offsets,
                                 const void* z, const void* embeddings, const float* offsets,
                                 const int64_t* grid_indices, const int64_t* cell_indices,
                                 const uint8_t* masks, const int64_t* lut_grid_nb2grid_idx,
                                 const int64_t* lut_cell_nb2cell_idx,
                                 const int64_t* lut_cell_nb2grid_nb, void* grad_z,
                                 void* grad_embeddings, int zero_grad, int64_t n, int64_t n_emb,
                                 int64_t cells_per_grid, int64_t D, void* stream);

/* ---------------------------------------------------------------- fused grid query
 * Positions in, features out: the work of SparseDenseGrid.forward (ash/grid.py:201-238) --
 * world -> cell transform, block / cell / offset split (ash/grid.py:183-199), hash find of the
 * block, neighbour resolution, gather and interpolation -- in one launch instead of ~15 torch
 * launches + find + query_forward.  x float32 [n][3] world positions; cell = (x - origin) *
 * (float)(1.0 / cell_size) (the reciprocal is formed in double and rounded once, which is what
 * `tensor / python_float` evaluates to on a CUDA tensor) with origin a HOST float[3] (NULL = zero); nb_lut int32 [n_emb][8]: index of
 * the block at offset (bit0, bit1, bit2) of the column, -1 absent (column 0 is the block
 * itself); the map must have key_dim 3.  Results are identical to the split + pre-split entry
 * points above. */

/* Builds nb_lut (and optionally grid_coords int32 [n_emb][3], -1 rows for inactive indices)
 * from the map; replaces SparseDenseGrid.construct_grid_neighbor_lut(radius=1,
 * bidirectional=False) (ash/grid.py:566-617). */
int ashb_grid_build_neighbor_lut(ashb_map* map, int32_t* nb_lut, int32_t* grid_coords, int64_t n_emb,
                                 void* stream);

/* out [n][D]; masks uint8 [n] = hash hit (a query whose neighbour block is absent keeps mask 1
 * and gets a zero row, as ash/src/grid.cu:109-111); block_idx_out int32 [n] (optional) = block
 * index per query, -1 on a miss, to be handed to the two backward entry points. */
int ashb_grid_query_forward(ashb_map* map, int dtype, int interp, const void* embeddings, const float* x,
                            double cell_size, const float* origin, int G, const int32_t* nb_lut, void* out,
                            uint8_t* masks, int32_t* block_idx_out, int64_t n, int64_t n_emb, int64_t D,
                            void* stream);

/* grad_x [n][3] (type of embeddings) = d/d offsets * (1 / cell_size), fully written; pass NULL
 * when the positions need no gradient and the eight embedding rows per query are not read at
 * all.  grad_embeddings accumulated (zero_grad as above); pass NULL when only grad_x is wanted (the
 * first-order pass of a gradient-of-gradient loss) and nothing is scattered.  block_idx NULL =
 * probe the map again. */
int ashb_grid_query_backward(ashb_map* map, int dtype, int interp, const void* z, const void* embeddings,
                             const float* x, double cell_size, const float* origin, int G,
                             const int32_t* nb_lut, const int32_t* block_idx, void* grad_embeddings,
                             void* grad_x, int zero_grad, int64_t n, int64_t n_emb, int64_t D, void* stream);

/* grad_grad_x [n][3] (type of embeddings): gradient arriving at grad_x. */
int ashb_grid_query_backward_backward(ashb_map* map, int dtype, int interp, const void* grad_grad_x,
                                      const void* z, const void* embeddings, const float* x,
                                      double cell_size, const float* origin, int G, const int32_t* nb_lut,
                                      const int32_t* block_idx, void* grad_z, void* grad_embeddings,
                                      int zero_grad, int64_t n, int64_t n_emb, int64_t D, void* stream);

/* The two backward passes above with the embedding gradient WRITTEN as a row list instead of added
 * into a table-sized buffer (the dense `at::zeros_like(embeddings)` of ash/src/grid.cu:276 and :415):
 * idx_out int64 [2][8 n] and rows_out [8 n][D] (type of embeddings), record 8 q + c = corner c of
 * query q: idx_out[0] = block index, idx_out[1] = cell index, rows_out = that corner's gradient row.
 * Together they are an uncoalesced sparse tensor of the table's shape (repeated cells add up).
 * Queries without a gradient write zero rows pointing at valid cells.  second_order == 0: the
 * first-order pass, side_out = grad_x [n][3] or NULL (then the embedding rows are not read);
 * second_order != 0: the double backward, grad_grad_x required, side_out = grad_z [n][D].
 * Nothing is read-modify-written and every store is coalesced. */
int ashb_grid_query_backward_rows(ashb_map* map, int dtype, int interp, int second_order, const void* grad_grad_x,
                                  const void* z, const void* embeddings, const float* x, double cell_size,
                                  const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx,
                                  int64_t* idx_out, void* rows_out, void* side_out, int64_t n, int64_t n_emb,
                                  int64_t D, void* stream);

/* Applies a row list to a dense buffer shaped like the table: dst[idx[0][r]][idx[1][r]][:] +=
 * alpha * rows[r][:] for r < m (idx int64 [2][m]); records with an index out of range and all-zero
 * rows are skipped.  dst may be a gradient buffer (alpha = 1) or the parameters themselves
 * (alpha = -learning rate).  No counterpart in the reference. */
int ashb_rows_scatter_add(int dtype, void* dst, const int64_t* idx, const void* rows, int64_t m, int64_t n_emb,
                          int64_t cells_per_grid, int64_t D, double alpha, void* stream);

/* Block allocation from points: replaces SparseDenseGrid.spatial_init_ (ash/grid.py:121-159) --
 * floor(points / cell / G), neighbourhood enumeration, the temporary HashSet used to
 * deduplicate, insert_keys and find -- with one launch.  points float32 [n][3] world positions.
 * Every block within `dilation` blocks (two-sided if bidirectional, else offsets 0..dilation)
 * of a point's block is inserted if absent; points whose own block lies outside
 * [bound_lo, bound_hi) (HOST int32[3], NULL = unbounded) are ignored, as are neighbours
 * outside it.  For each such block idx: grid_coords[idx] (int32 [n_emb][3]) gets its
 * coordinate, touched[idx] (uint32 [n_emb]) gets `stamp` (non-zero, different per call) and,
 * if given, touched_list int32 [n_emb] / touched_count int32 [1] get the compact list. */
int ashb_grid_spatial_init(ashb_map* map, const float* points, int64_t n, double cell_size,
                           const float* origin, int G, int dilation, int bidirectional,
                           const int32_t* bound_lo, const int32_t* bound_hi, int32_t* grid_coords,
                           uint32_t* touched, uint32_t stamp, int32_t* touched_list,
                           int32_t* touched_count, void* stream);

/* Writes zeros to the 8 corner rows of every query of the batch in grad_embeddings: clears
 * exactly what ashb_grid_query_backward / _backward_backward added for that batch, at the cost of
 * one pass over the batch instead of a table-sized memset.  No counterpart in the reference. */
int ashb_grid_zero_rows(ashb_map* map, int dtype, void* grad_embeddings, const float* x, double cell_size,
                        const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx,
                        int64_t n, int64_t n_emb, int64_t D, void* stream);

/* ---------------------------------------------------------------- neighbourhood convolution */

/* Replaces convolution_forward_kernel + convolution_forward (ash/src/grid.cu:951-1043).
 * inputs/outputs [n_emb][cells_per_grid][D]; weights [num_cell_nbs][D]; masks uint8
 * [num_grids * cells_per_grid]; grid_indices int64 [num_grids]; cell_indices int64
 * [cells_per_grid]; lut_grid_nb2grid_idx int64 [n_emb][num_grid_nbs] (<= 125, -1 = absent);
 * the two per-cell tables int64 [cells_per_grid][num_cell_nbs].  Rows of the listed
 * blocks are written; zero_output != 0 zero-fills the whole output first, as the
 * reference does. */
int ashb_conv_forward(int dtype, const void* inputs, const void* weights, const uint8_t* masks,
                      const int64_t* grid_indices, const int64_t* cell_indices,
                      const int64_t* lut_grid_nb2grid_idx, const int64_t* lut_cell_nb2cell_idx,
                      const int64_t* lut_cell_nb2grid_nb, void* outputs, int zero_output,
                      int64_t num_grids, int64_t n_emb, int64_t cells_per_grid, int64_t D,
                      int64_t num_cell_nbs, int64_t num_grid_nbs, void* stream);

/* The same convolution for the window SparseDenseGrid.convolution builds (ash/grid.py:476-520):
 * two-sided, radius <= G, float32.  The two per-cell tables are implied by (G, radius) and are
 * not passed; lut_grid_nb27 int64 [n_emb][27] is the radius-1 two-sided block table
 * (column = (ox+1) + 3 (oy+1) + 9 (oz+1)); weights [(2R+1)^3][D] with x fastest.  One CTA per
 * listed block works from a shared-memory halo tile.  Same results as ashb_conv_forward. */
int ashb_conv_forward_tiled(const float* inputs, const float* weights, const int64_t* grid_indices,
                            const int64_t* lut_grid_nb27, float* outputs, int zero_output,
                            int64_t num_grids, int64_t n_emb, int G, int radius, int64_t D, void* stream);

/* The tiled form for a SEPARABLE window, weights[z][y][x][c] = wz[z][c] * wy[y][c] * wx[x][c] (the
 * Gaussian of SparseDenseGrid.gaussian_filter_, ash/grid.py:449-462, is one): weights_1d float32
 * [3][2 radius + 1][D], axis 0 = x.  Three 1-D passes inside the shared-memory halo tile: 3 (2R+1)
 * multiply-adds per cell and channel instead of (2R+1)^3; same result up to the order of the sums. */
int ashb_conv_forward_separable(const float* inputs, const float* weights_1d, const int64_t* grid_indices,
                                const int64_t* lut_grid_nb27, float* outputs, int zero_output, int64_t num_grids,
                                int64_t n_emb, int G, int radius, int64_t D, void* stream);

/* ---------------------------------------------------------------- iso-surface vertices */

/* Replaces isosurface_extraction_kernel + isosurface_extraction (ash/src/grid.cu:453-604),
 * float32.  sdfs / weights [n_emb][cells_per_grid]; grid_indices int64 [num_grids];
 * grid_coords_table int32 [n_emb][3]; cell_coords_table int32 [cells_per_grid][3]; the three
 * radius-1 one-sided tables as for the query.  One call with positions == NULL counts (the
 * reference's first launch); a second call with positions float32 [max_out][3] fills (its second
 * launch).  *n_out (HOST) = number of crossings found; cursor_dev: 8 bytes of device scratch.
 * Positions are in cell units, order unspecified.  Synchronises `stream`. */
int ashb_isosurface_extraction(const float* sdfs, const float* weights, const int64_t* grid_indices,
                               const int32_t* grid_coords_table, const int64_t* lut_grid_nb2grid_idx,
                               const int32_t* cell_coords_table, const int64_t* lut_cell_nb2cell_idx,
                               const int64_t* lut_cell_nb2grid_nb, float* positions, int64_t max_out,
                               int64_t* n_out, void* cursor_dev, float iso_value, float weight_thr,
                               int grid_dim, int64_t cells_per_grid, int64_t n_emb, int64_t num_grids,
                               void* stream);

/* ---------------------------------------------------------------- iso-surface triangles
 * Replaces marching_cubes_table_idx_kernel / _vertex_kernel / _triangle_kernel + marching_cubes
 * (ash/src/grid.cu:607-946), float32, tables as for ashb_isosurface_extraction.  A cube sits at
 * every cell of a listed block whose 8 corners (cell and +x/+y/+z neighbours) exist and reach
 * weight_thr; corner c is inside when sdf - iso_value < 0.
 *   _count classifies every cube into codes uint8 [num_grids * cells_per_grid], requests the
 *          vertices of cut edges in edge_vertex int32 [n_emb * cells_per_grid * 3] (both are
 *          caller-allocated scratch, passed on to _fill) and returns the number of distinct
 *          vertices and of triangles (HOST).  Synchronises `stream`.
 *   _fill  writes vertices float32 [n_vertices][3] (cell units, the reference's interpolation)
 *          and triangles int32 [n_triangles][3] (vertex ids).  No host synchronisation.
 * counters_dev: 16 bytes of device scratch.  The triangulation table is this library's own, not
 * the reference's (ash/src/mc_macros.h): how ambiguous patterns are split, the order of a
 * triangle's corners (normals point towards increasing sdf) and the output order differ. */
int ashb_marching_cubes_count(const float* sdfs, const float* weights, const int64_t* grid_indices,
                              const int64_t* lut_grid_nb2grid_idx, const int64_t* lut_cell_nb2cell_idx,
                              const int64_t* lut_cell_nb2grid_nb, uint8_t* codes, int32_t* edge_vertex,
                              void* counters_dev, float iso_value, float weight_thr, int64_t cells_per_grid,
                              int64_t n_emb, int64_t num_grids, int64_t* n_vertices, int64_t* n_triangles,
                              void* stream);
int ashb_marching_cubes_fill(const float* sdfs, const int64_t* grid_indices, const int32_t* grid_coords_table,
                             const int64_t* lut_grid_nb2grid_idx, const int32_t* cell_coords_table,
                             const int64_t* lut_cell_nb2cell_idx, const int64_t* lut_cell_nb2grid_nb,
                             const uint8_t* codes, int32_t* edge_vertex, void* counters_dev, float* vertices,
                             int64_t n_vertices, int32_t* triangles, int64_t n_triangles, float iso_value,
                             int grid_dim, int64_t cells_per_grid, int64_t n_emb, int64_t num_grids,
                             void* stream);

/* ---------------------------------------------------------------- ray sampler
 * All lengths in cell units; rays float32 [n][3]; bbox float32 [3] each; the map
 * must have key_dim 3 (ash/src/sampler.cu:89-99).  Positions are fma(t, d, o) in
 * float32 and the block of a position is floor(position * (float)(1.0 / grid2cell)). */

/* Replaces ray_find_near_far_kernel + ray_find_near_far (ash/src/sampler.cu:7-121).
 * nears[i] = -1 when the ray meets no active block.  t_step is accepted and unused,
 * as in the reference. */
int ashb_ray_find_near_far(ashb_map* map, const float* ray_origins, const float* ray_directions,
                           const float* bbox_min, const float* bbox_max, float* nears, float* fars,
                           float t_min, float t_max, float t_step, float grid2cell, int64_t n,
                           void* stream);

/* Replace the two launches of ray_sample_count_kernel inside ray_sample
 * (ash/src/sampler.cu:123-294): pass 1 writes counts int64 [n]; the caller forms their
 * inclusive prefix sum; pass 2 writes ray_indices int64, t_nears and t_fars float32
 * at [prefix[i-1], prefix[i]). */
int ashb_ray_sample_count(ashb_map* map, const float* ray_origins, const float* ray_directions,
                          const float* ray_nears, const float* ray_fars, int64_t* counts,
                          int64_t max_samples_per_ray, float grid2cell, int64_t n, void* stream);
int ashb_ray_sample_fill(ashb_map* map, const float* ray_origins, const float* ray_directions,
                         const float* ray_nears, const float* ray_fars, const int64_t* prefix_sum,
                         int64_t* ray_indices, float* t_nears, float* t_fars,
                         int64_t max_samples_per_ray, float grid2cell, int64_t n, void* stream);

/* ---------------------------------------------------------------- RGB-D TSDF integration
 * Two launches replace one TSDFFusion.fuse_frame call (demo/rgbd_fusion.py:199-254),
 * which in the reference is ~40 torch operations, a temporary hash set
 * (ash/grid.py:145-147) and a third-party depth unprojection (demo/rgbd_fusion.py:57-74).
 * intrinsic: HOST float[9] row-major pinhole matrix without skew; cam_to_world /
 * world_to_cam: HOST float[12], rows of [R | t]; origin: HOST float[3], the world
 * position of cell (0,0,0) (zero for unbounded grids, bbox_min for bounded ones);
 * depth float32 [H][W] in metres and color float32 [H][W][3] are device buffers. */

/* Step 1, allocation (unprojection + SparseDenseGrid.spatial_init_ with
 * bidirectional dilation): every block within `dilation` blocks of a valid depth point
 * (0 < depth < depth_max) is inserted if absent; for each such block idx,
 * grid_coords[idx] (int32 [n_emb][3]) receives its coordinate and touched[idx]
 * (uint32 [n_emb]) receives `stamp` (non-zero, different per frame).  bound_lo/bound_hi:
 * HOST int32[3] half-open range of admissible block coordinates, or NULL for none.
 * touched_list int32 [n_emb] + touched_count int32 [1] (both device, both optional): the
 * compact list of the blocks stamped by this call, for ashb_tsdf_integrate. */
int ashb_tsdf_touch(ashb_map* map, const float* depth, int H, int W, const float* intrinsic,
                    const float* cam_to_world, float depth_max, double cell_size, const float* origin,
                    int G, int dilation, const int32_t* bound_lo, const int32_t* bound_hi,
                    int32_t* grid_coords, uint32_t* touched, uint32_t stamp, int32_t* touched_list,
                    int32_t* touched_count, void* stream);

/* Step 2, fusion (project_points_to_rgbd + the running average,
 * demo/rgbd_fusion.py:76-110, :236-254) over every cell of every block whose
 * touched[idx] == stamp.  embeddings float32 [n_emb][G^3][D], 5 <= D <= 16, with sdf at
 * sdf_channel, colour at rgb_channel..+2 and the weight at weight_channel (the demo uses
 * 0, 1, 4).  n_integrated_dev: optional device counter incremented once per fused block.
 * With the list of step 1 a few persistent CTAs walk exactly the stamped blocks -- and when a
 * block's rows are a 16-byte aligned multiple of 16 bytes they travel by bulk copies (global ->
 * shared on an mbarrier, shared -> global), two tiles per CTA, so that loading, arithmetic and
 * storing overlap; without it (NULL, NULL) one CTA per embedding row checks its stamp. */
int ashb_tsdf_integrate(void* embeddings, int64_t n_emb, int G, int64_t D, const int32_t* grid_coords,
                        const uint32_t* touched, uint32_t stamp, const float* depth, const float* color,
                        int H, int W, const float* intrinsic, const float* world_to_cam, float depth_max,
                        double cell_size, const float* origin, float trunc, int sdf_channel,
                        int rgb_channel, int weight_channel, unsigned long long* n_integrated_dev,
                        const int32_t* touched_list, const int32_t* touched_count, void* stream);

/* Steps 1 and 2 in one call (TSDFFusion.fuse_frame, demo/rgbd_fusion.py:199-254, as one entry point:
 * half the host work per frame); arguments as above, scratch provided by the caller. */
int ashb_tsdf_fuse_frame(ashb_map* map, void* embeddings, int64_t n_emb, int G, int64_t D, const float* depth,
                         const float* color, int H, int W, const float* intrinsic, const float* world_to_cam,
                         const float* cam_to_world, float depth_max, double cell_size, const float* origin,
                         int dilation, const int32_t* bound_lo, const int32_t* bound_hi, float trunc, int sdf_channel,
                         int rgb_channel, int weight_channel, int32_t* grid_coords, uint32_t* touched, uint32_t stamp,
                         int32_t* touched_list, int32_t* touched_count, unsigned long long* n_integrated_dev,
                         void* stream);

/* A sequence of frames of one size in one call (TSDFFusion.fuse_dataset, demo/rgbd_fusion.py:256-262): the two
 * launches of every frame are enqueued back to back from native code, so the sequence is not limited by the
 * caller's per-frame host work.  depths / colors: HOST arrays of n_frames device pointers; intrinsics
 * [n_frames][9], world_to_cams and cam_to_worlds [n_frames][12]: host floats; frame f uses stamp first_stamp + f.
 * With double_buffered != 0 (touched_list int32 [2][n_emb], touched_count int32 [2]) the allocation pass of frame
 * f + 1 runs on an internal side stream while frame f is fused on `stream` (events order the two; `stream` ends
 * ordered after all of it); the first such call on a device creates that stream and should come outside stream
 * capture. */
int ashb_tsdf_fuse_frames(ashb_map* map, void* embeddings, int64_t n_emb, int G, int64_t D, int n_frames,
                          const float* const* depths, const float* const* colors, int H, int W,
                          const float* intrinsics, const float* world_to_cams, const float* cam_to_worlds,
                          float depth_max, double cell_size, const float* origin, int dilation, const int32_t* bound_lo,
                          const int32_t* bound_hi, float trunc, int sdf_channel, int rgb_channel, int weight_channel,
                          int32_t* grid_coords, uint32_t* touched, uint32_t first_stamp, int32_t* touched_list,
                          int32_t* touched_count, int double_buffered, unsigned long long* n_integrated_dev,
                          void* stream);

/* One whole fusion step (allocation + fusion, as the two calls above) that allocates nothing.
 * It has no counterpart in the reference.  It exists for callers that must not allocate device
 * memory while they run: a capture or playback loop that reserved all of its memory up front, a
 * host application whose allocator the library may not touch, or code running where a
 * cudaMalloc would stall every stream of the device.  The per-block scratch (a stamp word and a
 * block coordinate) sits in a fixed array inside the library image instead of being passed in,
 * which limits the grid to ashb_tsdf_static_max_blocks() = 262144 blocks (n_emb beyond that is
 * rejected with ASHB_ERR_INVALID) and costs 4 MiB on every GPU that loads the library, until
 * the process exits.  The caller still owns and passes the map, the embeddings and the frame.
 * The first call on a device looks up the array's device address; make that first call before
 * any stream capture.  All calls share the one array (it is cleared at the start of each call),
 * so two calls whose work overlaps on the GPU race with each other: issue them on one stream
 * or order them yourself.  No cudaMalloc, cudaFree or other allocating routine is called. */
int ashb_tsdf_static_max_blocks(void);

/* The bulk-copy path of ashb_tsdf_integrate bounds every wait on a copy; a wait that runs out is
 * counted (on the current device) and the CTA stops.  *out = that count since the library was
 * loaded: 0 in any healthy run.  Synchronises with the device. */
int ashb_tsdf_copy_timeouts(unsigned int* out);
int ashb_tsdf_fuse_frame_static(ashb_map* map, void* embeddings, int64_t n_emb, int G, int64_t D,
                                const float* depth, const float* color, int H, int W,
                                const float* intrinsic, const float* world_to_cam,
                                const float* cam_to_world, float depth_max, double cell_size,
                                const float* origin, int dilation, const int32_t* bound_lo,
                                const int32_t* bound_hi, float trunc, int sdf_channel, int rgb_channel,
                                int weight_channel, void* stream);

/* ---------------------------------------------------------------- volume-rendering accumulation
 * The step right after the grid query in the reference's training loop, which the reference
 * delegates to a third-party package outside its tree (demo/train_scene_recon.py:111-150:
 * nerfacc.render_weight_from_density, nerfacc.accumulate_along_rays).  Samples are packed as the
 * ray sampler emits them: ray_indices int64 [m] non-decreasing, per-sample t_starts / t_ends /
 * sigmas float32 [m].  alpha = 1 - exp(-sigma (t_end - t_start)), T = running product of
 * (1 - alpha) over the earlier samples of the ray, weight = T alpha. */

/* seg_start / seg_end int64 [n_rays]: first and one-past-last sample of every ray (0, 0 for rays
 * without samples). */
int ashb_render_segments(const int64_t* ray_indices, int64_t m, int64_t n_rays, int64_t* seg_start,
                         int64_t* seg_end, void* stream);
int ashb_render_weights_forward(const float* t_starts, const float* t_ends, const float* sigmas,
                                const int64_t* seg_start, const int64_t* seg_end, int64_t n_rays,
                                float* weights, void* stream);
/* grad_sigmas [m] from grad_weights [m] (and the forward's weights). */
int ashb_render_weights_backward(const float* t_starts, const float* t_ends, const float* sigmas,
                                 const float* weights, const float* grad_weights,
                                 const int64_t* seg_start, const int64_t* seg_end, int64_t n_rays,
                                 float* grad_sigmas, void* stream);
/* out [n_rays][C] = sum over the ray's samples of weight * values [m][C] (values NULL: C = 1, value 1). */
int ashb_render_accumulate_forward(const float* weights, const float* values, int C,
                                   const int64_t* seg_start, const int64_t* seg_end, int64_t n_rays,
                                   float* out, void* stream);
/* grad_weights [m] and/or grad_values [m][C] (either may be NULL) from grad_out [n_rays][C]. */
int ashb_render_accumulate_backward(const float* weights, const float* values, const float* grad_out,
                                    const int64_t* ray_indices, int64_t m, int64_t n_rays, int C,
                                    float* grad_weights, float* grad_values, void* stream);

/* ---------------------------------------------------------------- fused ray renderer
 * One launch per direction for what the reference's training step composes from
 * ray_find_near_far -> ray_sample -> grid query -> autograd.grad(sdf, x) -> normalize ->
 * SDFToDensity -> render_weight_from_density / accumulate_along_rays
 * (demo/train_scene_recon.py:64-161, ash/src/sampler.cu:7-215, ash/src/grid.cu:69-255): no
 * per-sample tensor is written.  Channel 0 of an embedding row is the signed distance, channels
 * 1..3 the colour (D >= 4).  The map must be the grid's 3-D block map; nb_lut int32 [n_emb][8]
 * from ashb_grid_build_neighbor_lut; cell_size / origin (host float[3] or NULL) as in
 * ashb_grid_query_forward; ray_o_world and ray_o_cell float [n_rays][3] are the ray origins in
 * world and in cell units, ray_d the (unscaled) directions; bbox and t range in cell units as for
 * ashb_ray_find_near_far; beta: DEVICE float[1], the density scale (min_beta + |parameter|).
 * skip_missed != 0: rays that meet no occupied block are not sampled (all outputs 0).
 * out float [n_rays][16]: rgb[0..2], depth[3] (sum w * t_mid, world units), normal[4..6],
 * accumulated weight[7], sum | |grad sdf| - 1 | [8], sum (|grad sdf| - 1)^2 [9], sample count[10],
 * near[11], far[12] (world units, as ray_find_near_far returns them), [13..15] = 0. */
int ashb_render_rays_forward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                             const int32_t* nb_lut, double cell_size, const float* origin,
                             const float* ray_o_world, const float* ray_o_cell, const float* ray_d,
                             const float* bbox_min_cell, const float* bbox_max_cell, float t_min_cell,
                             float t_max_cell, int64_t max_samples_per_ray, int skip_missed, const float* beta,
                             float* out, int64_t n_rays, void* stream);
/* Gradients of a scalar loss given grad_out float [n_rays][16] (columns 0..9 are read) and the
 * forward's `out`: ADDS into grad_embeddings (same shape as embeddings) and grad_beta (DEVICE
 * float[1]); the caller zero-fills both (or keeps accumulating).  Re-marches every ray. */
int ashb_render_rays_backward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                              const int32_t* nb_lut, double cell_size, const float* origin,
                              const float* ray_o_world, const float* ray_o_cell, const float* ray_d,
                              const float* bbox_min_cell, const float* bbox_max_cell, float t_min_cell,
                              float t_max_cell, int64_t max_samples_per_ray, int skip_missed, const float* beta,
                              const float* out, const float* grad_out, float* grad_embeddings, float* grad_beta,
                              int64_t n_rays, void* stream);

/* ---------------------------------------------------------------- multi-GPU key routing
 * For a hash map partitioned over `world` ranks by key hash (no counterpart in the reference,
 * which is single-GPU): groups keys int32 [n][key_dim] by owner rank into keys_out (same shape),
 * writes perm_out int64 [n] (source row of every output row) and counts_host int64 [world]
 * (HOST: rows per owner, i.e. the send counts of the all-to-all).  scratch_dev: device buffer
 * of at least 1024 bytes.  Synchronises `stream`. */
int ashb_route_by_owner(const int32_t* keys, int64_t n, int key_dim, int world, int32_t* keys_out,
                        int64_t* perm_out, int64_t* counts_host, void* scratch_dev, void* stream);

/* The same renderer with the samples of a ray evaluated in parallel: _intervals marches every ray
 * once (one thread per ray) and lists its intervals, float32 [n_rays][stride][2] (t0, t1 in cell
 * units), with counts int32 [n_rays] and near_far float32 [n_rays][2] (world units); intervals
 * beyond `stride` are dropped and ASHB_STATUS_CAPACITY is set in the map's status word (stride =
 * max_samples_per_ray + 2 always suffices).  _forward / _backward then spend one WARP per ray on
 * the listed intervals (32 at a time, transmittance by a warp scan); `out` and the gradients are
 * as for ashb_render_rays_forward / _backward, up to floating-point summation order. */
int ashb_render_rays_intervals(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim, int D,
                               const int32_t* nb_lut, double cell_size, const float* origin,
                               const float* ray_o_cell, const float* ray_d, const float* bbox_min_cell,
                               const float* bbox_max_cell, float t_min_cell, float t_max_cell,
                               int64_t max_samples_per_ray, int skip_missed, float* intervals, int32_t* counts,
                               float* near_far, int64_t stride, int64_t n_rays, void* stream);
int ashb_render_intervals_forward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim,
                                  int D, const int32_t* nb_lut, double cell_size, const float* origin,
                                  const float* ray_o_world, const float* ray_d, const float* beta,
                                  const float* intervals, const int32_t* counts, const float* near_far, int64_t stride,
                                  float* out, int64_t n_rays, void* stream);
int ashb_render_intervals_backward(ashb_map* map, int interp, const float* embeddings, int64_t n_emb, int grid_dim,
                                   int D, const int32_t* nb_lut, double cell_size, const float* origin,
                                   const float* ray_o_world, const float* ray_d, const float* beta,
                                   const float* intervals, const int32_t* counts, int64_t stride, const float* out,
                                   const float* grad_out, float* grad_embeddings, float* grad_beta, int64_t n_rays,
                                   void* stream);

/* ---------------------------------------------------------------- table sharded over the GPUs of a box
 * ashb_grid_query_forward / _backward for an embedding table split by block over `world` GPUs
 * (no counterpart in the reference): block g lives on GPU g % world as row g / world of that
 * GPU's shard float32 [ceil(n_emb / world)][G^3][D]; emb_bases_dev / grad_bases_dev are DEVICE
 * arrays [world] of the shards' addresses as mapped into this GPU (peer memory).  The map and
 * nb_lut are this rank's replicas of the block structure (n_emb = global number of rows).  The
 * forward reads corner rows from their owners with plain loads; the backward ADDS gradient rows
 * straight into the owners' gradient shards with vector reductions unless need_grad_embeddings is 0
 * (a pass that only wants d/dx), and writes grad_x, or skips it when NULL.  The caller orders the launches across the ranks: parameters must be final on every
 * rank before any forward, and every backward must be complete before a gradient shard is read. */
int ashb_grid_query_forward_sharded(ashb_map* map, int interp, const void* const* emb_bases_dev, int world,
                                    const float* x, double cell_size, const float* origin, int G,
                                    const int32_t* nb_lut, float* out, uint8_t* masks, int32_t* block_idx_out,
                                    float* rows_out, int64_t n, int64_t n_emb, int64_t D, void* stream);
int ashb_grid_query_backward_sharded(ashb_map* map, int interp, const float* z, const void* const* emb_bases_dev,
                                     void* const* grad_bases_dev, int world, const float* x, double cell_size,
                                     const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx,
                                     float* grad_x, int need_grad_embeddings, const float* rows_in, int64_t n,
                                     int64_t n_emb, int64_t D, void* stream);

/* Double backward over the sharded table (as ashb_grid_query_backward_backward): grad_z [n][D] is
 * written, the embedding gradient is ADDED into the owners' gradient shards. */
int ashb_grid_query_backward_backward_sharded(ashb_map* map, int interp, const float* grad_grad_x, const float* z,
                                              const void* const* emb_bases_dev, void* const* grad_bases_dev,
                                              int world, const float* x, double cell_size, const float* origin,
                                              int G, const int32_t* nb_lut, const int32_t* block_idx, float* grad_z,
                                              const float* rows_in, int64_t n, int64_t n_emb, int64_t D,
                                              void* stream);

/* ---------------------------------------------------------------- peer-memory transport
 * find over the key-hash-partitioned map without a data collective (no counterpart in the
 * reference).  Every rank has a mailbox of mailbox_bytes, mapped into every other rank;
 * peer_bases_dev is a DEVICE array [world] with the address of every rank's mailbox as seen from
 * this rank.  Sections of a mailbox: inbox (12-byte records {k0, k1, k2}, unused columns zero; world regions of
 * region_capacity <= 2^26 records, region r written by rank r), counts int32 [world], answers int32
 * [world][region_capacity] (region o written by owner o, in the order of its inbox region).  A
 * batch has at most answer_capacity keys.  Keys of 1 to 3 columns.
 *   ashb_peer_route_keys   writes every key of the batch into its owner's inbox and publishes the
 *                          per-region counts; cursor_dev int32 [world] scratch; where_dev int32 [n]
 *                          (or NULL) receives owner << 26 | slot of every key (-1: dropped);
 *                          records beyond region_capacity are dropped and ASHB_STATUS_CAPACITY is
 *                          or-ed into status_dev.
 *   ashb_peer_find_answer  probes the records of this rank's inbox and stores the answers (the
 *                          owner's local index, or -1) into its region of the asker's answers
 *                          section, contiguously in inbox order.
 *   ashb_peer_unpack_answers  the asker's side, after the second barrier: indices int64 [n] (0 for
 *                          a miss; global index = owner's local index * world + owner) and masks uint8
 *                          [n] gathered from its own answers section.
 * The caller orders the two across the ranks (all route calls complete before any answer call
 * starts, all answer calls complete before the answers are read or the next route call starts),
 * e.g. with a small collective on the same stream between them.  No host synchronisation. */
int ashb_peer_route_keys(const int32_t* keys, int64_t n, int key_dim, int world, int rank,
                         void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_offset,
                         int64_t counts_offset, int64_t answers_offset, int64_t region_capacity,
                         int64_t answer_capacity, int32_t* cursor_dev, int32_t* where_dev, uint32_t* status_dev,
                         void* stream);
int ashb_peer_find_answer(ashb_map* map, int world, int rank, void* const* peer_bases_dev, int64_t mailbox_bytes,
                          int64_t inbox_offset, int64_t counts_offset, int64_t answers_offset,
                          int64_t region_capacity, int64_t answer_capacity, void* stream);
int ashb_peer_unpack_answers(const int32_t* where_dev, int64_t n, int world, int rank, void* const* peer_bases_dev,
                             int64_t mailbox_bytes, int64_t inbox_offset, int64_t counts_offset,
                             int64_t answers_offset, int64_t region_capacity, int64_t answer_capacity,
                             int64_t* indices, uint8_t* masks, void* stream);
/* Insert-if-absent (erase == 0) or erase (erase != 0) of the records in this rank's inbox, after an
 * ashb_peer_route_keys on every rank and the barrier; nothing goes back to the askers. */
int ashb_peer_update(ashb_map* map, int erase, int world, int rank, void* const* peer_bases_dev,
                     int64_t mailbox_bytes, int64_t inbox_offset, int64_t counts_offset, int64_t answers_offset,
                     int64_t region_capacity, int64_t answer_capacity, void* stream);

/* ---------------------------------------------------------------- table sharded over the GPUs, queries routed to the owners
 * (no counterpart in the reference, which is single-GPU).  The table is split by BLOCK over `world`
 * ranks: row_of uint32 [n_emb] (replicated) = owner << 26 | row of the block in the owner's shard;
 * emb_bases_dev / grad_bases_dev: device arrays [world] of the shards' (and gradient shards') base
 * addresses as mapped into this rank; the hash map and nb_lut are replicated.  Instead of reading
 * rows from their owners, every query is SENT to the owner of its block, which interpolates in its
 * own memory and returns the result row; the backward sends dL/dy the same way and the owner adds
 * the gradient rows into its own gradient shard and returns dL/dx.  Corner rows in a neighbour
 * block of another owner are read / reduced over peer memory directly.
 *
 * Mailbox (symmetric memory, one per rank, peer_bases_dev [world]): inbox_x float4 [world][cap]
 * {x, y, z, block index}, counts int32 [world], inbox_z float [world][cap][D], out_y float
 * [world][cap][D], out_gx float4 [world][cap], inbox_g float4 [world][cap]; all offsets in bytes,
 * multiples of 16 (counts: 4).
 * Rank r writes only region r of another rank's sections.  world <= 32, region_capacity < 2^26.
 * A step on every rank: route | barrier | forward | barrier | unpack_y | ... | send_z | barrier |
 * backward | barrier | unpack_grad_x, the barriers being collectives the caller enqueues on the
 * same stream; no kernel waits on another GPU.  where_dev int32 [n]: owner << 26 | slot per query
 * (-1: no block there, or dropped because its region was full -> ASHB_STATUS_CAPACITY in
 * status_dev). */
int ashb_routed_route(ashb_map* map, const float* x, int64_t n, double cell_size, const float* origin, int G,
                      const int32_t* nb_lut, const uint32_t* row_of, int64_t n_emb, int64_t D,
                      void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                      int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset,
                      int64_t inbox_g_offset, int64_t region_capacity, int world, int rank, int32_t* cursor_dev, int32_t* where_dev,
                      uint32_t* status_dev, void* stream);
/* Owner side: interpolate every record of this rank's inbox (semantics of ashb_grid_query_forward)
 * and store row j of region r into rank r's out_y[rank][j]. */
int ashb_routed_forward(ashb_map* map, int interp, const void* const* emb_bases_dev, double cell_size,
                        const float* origin, int G, const int32_t* nb_lut, const uint32_t* row_of, int64_t n_emb,
                        int64_t D, void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                        int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset, int64_t inbox_g_offset,
                        int64_t region_capacity, int world, int rank, void* stream);
/* Asker side: y [n][D] and masks uint8 [n] (optional) from this rank's out_y, in query order. */
int ashb_routed_unpack_y(const int32_t* where_dev, int64_t n, float* y, uint8_t* masks, int64_t D,
                         void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                         int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset, int64_t inbox_g_offset,
                         int64_t region_capacity, int world, int rank, void* stream);
/* Asker side: z [n][D] = dL/dy of every query into its owner's inbox_z, at the slot routing gave it. */
int ashb_routed_send_z(const int32_t* where_dev, int64_t n, const float* z, int64_t D,
                       void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                       int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset, int64_t inbox_g_offset,
                       int64_t region_capacity, int world, int rank, void* stream);
/* Owner side: semantics of ashb_grid_query_backward for every record: gradient rows ADDED into the
 * owners' gradient shards unless need_grad_embeddings == 0 (the first-order pass of a
 * gradient-of-gradient loss), dL/dx (times 1 / cell_size) stored into the asker's out_gx unless
 * need_grad_x == 0 (then the embedding rows are not read). */
int ashb_routed_backward(ashb_map* map, int interp, const void* const* emb_bases_dev, void* const* grad_bases_dev,
                         int need_grad_x, int need_grad_embeddings, double cell_size, const float* origin, int G, const int32_t* nb_lut,
                         const uint32_t* row_of, int64_t n_emb, int64_t D, void* const* peer_bases_dev,
                         int64_t mailbox_bytes, int64_t inbox_x_offset, int64_t counts_offset,
                         int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset, int64_t inbox_g_offset,
                         int64_t region_capacity, int world, int rank, void* stream);
/* Asker side: grad_x [n][3] from this rank's out_gx, zero rows for queries without a block. */
int ashb_routed_unpack_grad_x(const int32_t* where_dev, int64_t n, float* grad_x, int64_t D,
                              void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                              int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset,
                              int64_t out_gx_offset, int64_t inbox_g_offset, int64_t region_capacity, int world, int rank, void* stream);

/* Double backward over the routed table.  Asker side: grad_grad_x [n][3], the gradient arriving at dL/dx,
 * into every query's owner's inbox_g (send dL/dy again with ashb_routed_send_z first: another pass may have
 * replaced it).  Owner side: semantics of ashb_grid_query_backward_backward for every record -- second-order
 * gradient rows ADDED into the owners' gradient shards, the gradient with respect to dL/dy stored into the
 * asker's out_y (gather it with ashb_routed_unpack_y, masks NULL). */
int ashb_routed_send_g(const int32_t* where_dev, int64_t n, const float* grad_grad_x, int64_t D,
                       void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                       int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset,
                       int64_t inbox_g_offset, int64_t region_capacity, int world, int rank, void* stream);
int ashb_routed_backward_backward(ashb_map* map, int interp, const void* const* emb_bases_dev,
                                  void* const* grad_bases_dev, double cell_size, const float* origin, int G,
                                  const int32_t* nb_lut, const uint32_t* row_of, int64_t n_emb, int64_t D,
                                  void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset,
                                  int64_t counts_offset, int64_t inbox_z_offset, int64_t out_y_offset,
                                  int64_t out_gx_offset, int64_t inbox_g_offset, int64_t region_capacity, int world,
                                  int rank, void* stream);

/* ---------------------------------------------------------------- runtime knobs */

/* Selects how ashb_query_backward_forward and ashb_grid_query_backward scatter the embedding
 * gradient: 0 = one vector reduction per lane and corner (default), 1 = lanes of a warp that add to
 * the same row slice are combined first and one of them issues the reduction.  Same sums up to
 * floating-point order. */
int ashb_set_scatter_aggregation(int enable);

/* Selects the kernel behind ashb_map_find for key_dim <= 3: 0 = one thread per key (default),
 * 1 = eight lanes per key reading a whole 128-byte line of slots per step.  Same results. */
int ashb_set_find_cooperative(int enable);

/* The same choice for ashb_map_erase (replaces the probe of ash/src/hashmap_gpu.cuh:317-336):
 * 0 = one thread per key (default), 1 = eight lanes per key.  Same results. */
int ashb_set_erase_cooperative(int enable);

/* Occupancy filter of ashb_map_find for key_dim <= 3 (no counterpart in the reference).  Every map
 * keeps one bit per slot, set when a key is first stored there; a find whose home slot never held a
 * key is a miss and is answered from that bit map, which stays in L2 for tables far larger than L2,
 * without touching the table.  mode -1 (default): used for tables of 64 MB and more; 0: never;
 * 1: always.  Same results in every mode. */
int ashb_set_find_filter(int mode);

/* Measurement aid (no counterpart in the reference): launches n_reads threads that each read one
 * 16-byte word at a pseudo-random 64-byte-aligned place of `buffer` (device, 64-byte aligned,
 * `bytes` long, any content), naming an L2 fetch size of fetch_bytes (64 or 128).  Timed by the
 * caller, the reads per second it reaches are the ceiling for the probe and gather kernels, whose
 * accesses are as scattered.  sink_dev: 8 bytes of device scratch. */
int ashb_measure_random_reads(const void* buffer, int64_t bytes, int64_t n_reads, int fetch_bytes, uint32_t seed,
                              void* sink_dev, void* stream);
/* The same with reads_per_thread (1, 2, 4 or 8) independent reads issued by every thread before any
 * is consumed (n_reads in total): tells a latency limit (the rate rises with it) from a limit of the
 * memory system (it does not). */
int ashb_measure_random_reads_ilp(const void* buffer, int64_t bytes, int64_t n_reads, int fetch_bytes,
                                  int reads_per_thread, uint32_t seed, void* sink_dev, void* stream);

/* cudaLimitMaxL2FetchGranularity of the current context (32, 64 or 128 bytes); a
 * performance hint that lasts as long as the process.  No counterpart in the reference. */
int ashb_set_l2_fetch_granularity(int bytes);
int ashb_get_l2_fetch_granularity(int* bytes_out);

#ifdef __cplusplus
}
#endif
#endif /* ASHB200_H_ */
