/*
 * CPU restatement of torch-ash's native hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the parity oracle and the timed CPU baseline.  It is never
 * linked into, imported by or called from the product library; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Each function cites the reference source it follows (paths relative to the
 * torch-ash project root).  The hash table underneath the reference is the
 * third-party stdgpu::unordered_map (git submodule ext/stdgpu, no pinned
 * version is recorded in the tree and the sources are not vendored), so slot
 * placement and enumeration order are NOT restated: only the key -> index
 * association, hit/miss masks, the heap discipline and sizes are, which is
 * exactly what the reference's own tests pin (unittests/test_engine.py:21-83).
 *
 * Plain C99 + OpenMP.  Build: see oracle/Makefile.
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_MAX_KEY_DIM 4 /* ash/src/dispatch.h:48 kMaxKeyDim */

/* ------------------------------------------------------------------------- */
/* Hash engine                                                               */
/* ------------------------------------------------------------------------- */

typedef struct {
    int key_dim;
    int64_t capacity;
    int64_t n_slots;    /* power of two, >= 2 * capacity */
    int32_t* slot_keys; /* n_slots * key_dim */
    int32_t* slot_vals; /* >= 0 index, -1 empty, -2 tombstone */
    int32_t* heap;      /* borrowed: the caller's int32[capacity] free-index stack */
    int32_t heap_counter; /* ash/src/hashmap_impl.h:21 heap_counter_ */
} oracle_map;

#define SLOT_EMPTY (-1)
#define SLOT_TOMB (-2)

/* ash/src/dispatch.h:109-124 MiniVecHash: FNV-1a style over the int elements
 * cast to uint64 (sign extending). */
static uint64_t key_hash(const int32_t* key, int dim) {
    uint64_t h = UINT64_C(14695981039346656037);
    for (int i = 0; i < dim; ++i) {
        h ^= (uint64_t)(int64_t)key[i];
        h *= UINT64_C(1099511628211);
    }
    return h;
}

/* ash/src/dispatch.h:126-140 MiniVecEq */
static int key_eq(const int32_t* a, const int32_t* b, int dim) {
    for (int i = 0; i < dim; ++i)
        if (a[i] != b[i]) return 0;
    return 1;
}

/* ash/src/hashmap_impl.h:26-33 reset_heap: counter 0, heap = arange */
static void map_reset_heap(oracle_map* m) {
    m->heap_counter = 0;
    for (int64_t i = 0; i < m->capacity; ++i) m->heap[i] = (int32_t)i;
}

/* ash/src/hashmap_impl.h:11-24 + hashmap_gpu.cuh:119-133: the constructor
 * aliases the caller's heap and zeroes the counter; it does NOT rewrite the
 * heap contents. */
oracle_map* oracle_map_create(int key_dim, int64_t capacity, int32_t* heap) {
    if (key_dim < 1 || key_dim > ORACLE_MAX_KEY_DIM || capacity < 1) return NULL;
    oracle_map* m = (oracle_map*)calloc(1, sizeof(oracle_map));
    m->key_dim = key_dim;
    m->capacity = capacity;
    int64_t n = 16;
    while (n < 2 * capacity) n <<= 1;
    m->n_slots = n;
    m->slot_keys = (int32_t*)malloc(sizeof(int32_t) * n * key_dim);
    m->slot_vals = (int32_t*)malloc(sizeof(int32_t) * n);
    for (int64_t i = 0; i < n; ++i) m->slot_vals[i] = SLOT_EMPTY;
    m->heap = heap;
    m->heap_counter = 0;
    return m;
}

void oracle_map_destroy(oracle_map* m) {
    if (!m) return;
    free(m->slot_keys);
    free(m->slot_vals);
    free(m);
}

/* ash/src/hashmap_gpu.cuh:355-358 clear(): empty the table, reset the heap */
void oracle_map_clear(oracle_map* m) {
    for (int64_t i = 0; i < m->n_slots; ++i) m->slot_vals[i] = SLOT_EMPTY;
    map_reset_heap(m);
}

/* ash/src/hashmap_gpu.cuh:157 size() */
int64_t oracle_map_size(const oracle_map* m) { return m->heap_counter; }

static int64_t map_lookup(const oracle_map* m, const int32_t* key) {
    const int64_t mask = m->n_slots - 1;
    int64_t s = (int64_t)(key_hash(key, m->key_dim) & (uint64_t)mask);
    for (int64_t probe = 0; probe < m->n_slots; ++probe) {
        int32_t v = m->slot_vals[s];
        if (v == SLOT_EMPTY) return -1;
        if (v != SLOT_TOMB && key_eq(m->slot_keys + s * m->key_dim, key, m->key_dim))
            return s;
        s = (s + 1) & mask;
    }
    return -1;
}

/* ash/src/hashmap_gpu.cuh:164-178 find_kernel: indices[i] = hit ? value : 0,
 * masks[i] = hit.  Read only, so the query loop runs on all cores. */
void oracle_map_find(const oracle_map* m, const int32_t* keys, int64_t n,
                     int64_t* indices, uint8_t* masks) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int64_t s = map_lookup(m, keys + i * m->key_dim);
        masks[i] = (uint8_t)(s >= 0);
        indices[i] = s >= 0 ? (int64_t)m->slot_vals[s] : 0;
    }
}

/* Insert-if-absent returning the slot, or -1 if the key was present, or -2 if
 * the index heap is exhausted (the reference reads heap[top] out of bounds in
 * that case, hashmap_gpu.cuh:226-227; the oracle refuses instead). */
static int64_t map_emplace(oracle_map* m, const int32_t* key, int32_t* idx_out) {
    const int64_t mask = m->n_slots - 1;
    int64_t s = (int64_t)(key_hash(key, m->key_dim) & (uint64_t)mask);
    int64_t first_free = -1;
    for (int64_t probe = 0; probe < m->n_slots; ++probe) {
        int32_t v = m->slot_vals[s];
        if (v == SLOT_EMPTY) {
            if (first_free < 0) first_free = s;
            break;
        }
        if (v == SLOT_TOMB) {
            if (first_free < 0) first_free = s;
        } else if (key_eq(m->slot_keys + s * m->key_dim, key, m->key_dim)) {
            return -1;
        }
        s = (s + 1) & mask;
    }
    if (first_free < 0) return -2;
    if (m->heap_counter >= m->capacity) return -2;
    /* hashmap_gpu.cuh:224-230: top = counter++, idx = heap[top] */
    int32_t top = m->heap_counter++;
    int32_t idx = m->heap[top];
    memcpy(m->slot_keys + first_free * m->key_dim, key, sizeof(int32_t) * m->key_dim);
    m->slot_vals[first_free] = idx;
    *idx_out = idx;
    return first_free;
}

/* ash/src/hashmap_gpu.cuh:212-232 insert_kernel (keys only).  Sequential: the
 * first occurrence of an in-batch duplicate wins (the reference's winner is
 * nondeterministic).  Returns the number of keys refused for lack of heap. */
int64_t oracle_map_insert_keys(oracle_map* m, const int32_t* keys, int64_t n) {
    int64_t refused = 0;
    for (int64_t i = 0; i < n; ++i) {
        int32_t idx;
        if (map_emplace(m, keys + i * m->key_dim, &idx) == -2) ++refused;
    }
    return refused;
}

/* ash/src/hashmap_gpu.cuh:250-283 insert_kernel (with values): the inserting
 * winner copies row i of every source array into row idx of its destination.
 * row_bytes[j] is the byte size of one row of value j (blob size * blob count
 * of hashmap_gpu.cuh:79-114; the blob factorisation only chooses a copy width
 * and has no arithmetic effect). */
int64_t oracle_map_insert_values(oracle_map* m, const int32_t* keys, int64_t n,
                                 int n_values, const void* const* src,
                                 void* const* dst, const int64_t* row_bytes) {
    int64_t refused = 0;
    for (int64_t i = 0; i < n; ++i) {
        int32_t idx;
        int64_t s = map_emplace(m, keys + i * m->key_dim, &idx);
        if (s == -2) ++refused;
        if (s < 0) continue;
        for (int j = 0; j < n_values; ++j)
            memcpy((char*)dst[j] + (int64_t)idx * row_bytes[j],
                   (const char*)src[j] + i * row_bytes[j], (size_t)row_bytes[j]);
    }
    return refused;
}

/* ash/src/hashmap_gpu.cuh:317-336 erase_kernel: on success top = counter--,
 * heap[top - 1] = erased index. */
void oracle_map_erase(oracle_map* m, const int32_t* keys, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        int64_t s = map_lookup(m, keys + i * m->key_dim);
        if (s < 0) continue;
        int32_t idx = m->slot_vals[s];
        m->slot_vals[s] = SLOT_TOMB;
        int32_t top = m->heap_counter--;
        m->heap[top - 1] = idx;
    }
}

/* ash/src/hashmap_gpu.cuh:377-405 items(): active keys (n, dim) and their
 * indices (n,), in table order (unspecified in the reference).  Returns n. */
int64_t oracle_map_items(const oracle_map* m, int32_t* keys_out, int64_t* idx_out) {
    int64_t n = 0;
    for (int64_t s = 0; s < m->n_slots; ++s) {
        if (m->slot_vals[s] < 0) continue;
        memcpy(keys_out + n * m->key_dim, m->slot_keys + s * m->key_dim,
               sizeof(int32_t) * m->key_dim);
        idx_out[n] = m->slot_vals[s];
        ++n;
    }
    return n;
}

/* ash/src/hashmap_gpu.cuh:408-450 load_states: counter = count, heap copied,
 * every (key, saved index) pair emplaced verbatim.  Returns the number of
 * pairs that could not be emplaced (duplicates; "should never reach here"). */
int64_t oracle_map_load_states(oracle_map* m, const int32_t* keys,
                               const int64_t* indices, int64_t n,
                               const int32_t* heap) {
    m->heap_counter = (int32_t)n;
    if (heap != m->heap) memmove(m->heap, heap, sizeof(int32_t) * m->capacity);
    int64_t bad = 0;
    const int64_t mask = m->n_slots - 1;
    for (int64_t i = 0; i < n; ++i) {
        const int32_t* key = keys + i * m->key_dim;
        if (map_lookup(m, key) >= 0) { ++bad; continue; }
        int64_t s = (int64_t)(key_hash(key, m->key_dim) & (uint64_t)mask);
        while (m->slot_vals[s] >= 0) s = (s + 1) & mask;
        memcpy(m->slot_keys + s * m->key_dim, key, sizeof(int32_t) * m->key_dim);
        m->slot_vals[s] = (int32_t)indices[i];
    }
    return bad;
}

/* ------------------------------------------------------------------------- */
/* Grid query: forward, backward, double backward                            */
/* ------------------------------------------------------------------------- */

/* ash/src/grid.cu:7-41 interpolation functors. interp: 0 linear, 1 smooth_step */
#define DEFINE_QUERY(T, SUF)                                                              \
    static inline T interp_##SUF(int interp, T x) {                                       \
        return interp ? x * x * (3 - 2 * x) : x;                                          \
    }                                                                                     \
    static inline T dinterp_##SUF(int interp, T x) {                                      \
        return interp ? 6 * x * (1 - x) : (T)1;                                           \
    }                                                                                     \
    /* grid.cu:85-111 / :197-216: resolve the 8 corner rows; 0 if any neighbour   */     \
    /* block is absent (-1), in which case the kernels leave the outputs zero.    */     \
    static inline int corners_##SUF(const int64_t* g2g, const int64_t* c2c,               \
                                    const int64_t* c2g, int64_t grid_idx,                 \
                                    int64_t cell_idx, int64_t cells_per_grid,             \
                                    int64_t D, int64_t* base) {                           \
        for (int c = 0; c < 8; ++c) {                                                     \
            int64_t grid_nb = c2g[cell_idx * 8 + c];                                      \
            int64_t grid_nb_idx = g2g[grid_idx * 8 + grid_nb];                            \
            if (grid_nb_idx == -1) return 0;                                              \
            base[c] = (grid_nb_idx * cells_per_grid + c2c[cell_idx * 8 + c]) * D;         \
        }                                                                                 \
        return 1;                                                                         \
    }                                                                                     \
    /* grid.cu:113-119, :221-236: corner weight and its gradient w.r.t. offsets. */      \
    /* `1 - offset[d]` is evaluated in float even for double embeddings because  */      \
    /* offsets are MiniVec<float,3> (grid.cu:71,117).                            */      \
    static inline T weights_##SUF(int interp, const float* off, int c, T* wg) {           \
        T weight = 1;                                                                     \
        wg[0] = wg[1] = wg[2] = 1;                                                        \
        for (int d = 0; d < 3; ++d) {                                                     \
            int code = (c >> d) & 1;                                                      \
            T x = code ? (T)off[d] : (T)(1 - off[d]);                                     \
            T w = interp_##SUF(interp, x);                                                \
            T dw = dinterp_##SUF(interp, x) * (code ? 1 : -1);                            \
            weight *= w;                                                                  \
            wg[0] *= (d == 0) ? dw : w;                                                   \
            wg[1] *= (d == 1) ? dw : w;                                                   \
            wg[2] *= (d == 2) ? dw : w;                                                   \
        }                                                                                 \
        return weight;                                                                    \
    }                                                                                     \
    /* grid.cu:69-132 query_forward_kernel; output must be zero-filled (:146) */         \
    void oracle_query_forward_##SUF(                                                      \
            const T* emb, const float* offsets, const int64_t* grid_indices,              \
            const int64_t* cell_indices, const uint8_t* masks, const int64_t* g2g,        \
            const int64_t* c2c, const int64_t* c2g, T* out, int64_t cells_per_grid,       \
            int64_t D, int64_t n, int interp) {                                           \
        _Pragma("omp parallel for schedule(static)")                                      \
        for (int64_t i = 0; i < n; ++i) {                                                 \
            if (!masks[i]) continue;                                                      \
            int64_t base[8];                                                              \
            if (!corners_##SUF(g2g, c2c, c2g, grid_indices[i], cell_indices[i],           \
                               cells_per_grid, D, base))                                  \
                continue;                                                                 \
            T acc[16] = {0};                                                              \
            for (int c = 0; c < 8; ++c) {                                                 \
                T wg[3];                                                                  \
                T w = weights_##SUF(interp, offsets + 3 * i, c, wg);                      \
                for (int64_t k = 0; k < D; ++k) acc[k] += w * emb[base[c] + k];           \
            }                                                                             \
            for (int64_t k = 0; k < D; ++k) out[i * D + k] = acc[k];                      \
        }                                                                                 \
    }                                                                                     \
    /* grid.cu:178-255 query_backward_forward_kernel; grad_emb and grad_off must */      \
    /* be zero-filled (:276-277).  Scatter order differs per run as on the GPU.  */      \
    void oracle_query_backward_forward_##SUF(                                             \
            const T* z, const T* emb, const float* offsets,                               \
            const int64_t* grid_indices, const int64_t* cell_indices,                     \
            const uint8_t* masks, const int64_t* g2g, const int64_t* c2c,                 \
            const int64_t* c2g, T* grad_emb, T* grad_off, int64_t cells_per_grid,         \
            int64_t D, int64_t n, int interp) {                                           \
        _Pragma("omp parallel for schedule(static)")                                      \
        for (int64_t i = 0; i < n; ++i) {                                                 \
            if (!masks[i]) continue;                                                      \
            int64_t base[8];                                                              \
            if (!corners_##SUF(g2g, c2c, c2g, grid_indices[i], cell_indices[i],           \
                               cells_per_grid, D, base))                                  \
                continue;                                                                 \
            T go[3] = {0, 0, 0};                                                          \
            for (int c = 0; c < 8; ++c) {                                                 \
                T wg[3];                                                                  \
                T w = weights_##SUF(interp, offsets + 3 * i, c, wg);                      \
                T dot = 0;                                                                \
                for (int64_t k = 0; k < D; ++k) {                                         \
                    T zk = z[i * D + k];                                                  \
                    T add = w * zk;                                                       \
                    _Pragma("omp atomic")                                                 \
                    grad_emb[base[c] + k] += add;                                         \
                    dot += emb[base[c] + k] * zk;                                         \
                }                                                                         \
                for (int d = 0; d < 3; ++d) go[d] += dot * wg[d];                         \
            }                                                                             \
            for (int d = 0; d < 3; ++d) grad_off[i * 3 + d] = go[d];                      \
        }                                                                                 \
    }                                                                                     \
    /* grid.cu:310-387 query_backward_backward_kernel; grad_z and grad_emb must  */      \
    /* be zero-filled (:414-415); the third output (grad_offsets) stays zero     */      \
    /* (:417-418) and grad_grad_embeddings is unused (:426).                     */      \
    void oracle_query_backward_backward_##SUF(                                            \
            const T* ggo, const T* z, const T* emb, const float* offsets,                 \
            const int64_t* grid_indices, const int64_t* cell_indices,                     \
            const uint8_t* masks, const int64_t* g2g, const int64_t* c2c,                 \
            const int64_t* c2g, T* grad_z, T* grad_emb, int64_t cells_per_grid,           \
            int64_t D, int64_t n, int interp) {                                           \
        _Pragma("omp parallel for schedule(static)")                                      \
        for (int64_t i = 0; i < n; ++i) {                                                 \
            if (!masks[i]) continue;                                                      \
            int64_t base[8];                                                              \
            if (!corners_##SUF(g2g, c2c, c2g, grid_indices[i], cell_indices[i],           \
                               cells_per_grid, D, base))                                  \
                continue;                                                                 \
            for (int c = 0; c < 8; ++c) {                                                 \
                T wg[3];                                                                  \
                (void)weights_##SUF(interp, offsets + 3 * i, c, wg);                      \
                T dot = wg[0] * ggo[i * 3] + wg[1] * ggo[i * 3 + 1] +                     \
                        wg[2] * ggo[i * 3 + 2];                                           \
                for (int64_t k = 0; k < D; ++k) {                                         \
                    T add = dot * z[i * D + k];                                           \
                    _Pragma("omp atomic")                                                 \
                    grad_emb[base[c] + k] += add;                                         \
                    grad_z[i * D + k] += dot * emb[base[c] + k];                          \
                }                                                                         \
            }                                                                             \
        }                                                                                 \
    }                                                                                     \
    /* grid.cu:951-1004 convolution_forward_kernel (depth-wise window sum through */     \
    /* the radius-R lookup tables); outputs must be zero-filled (:1016).          */     \
    void oracle_convolution_forward_##SUF(                                                \
            const T* inputs, const T* weights, const uint8_t* masks,                      \
            const int64_t* grid_indices, const int64_t* cell_indices,                     \
            const int64_t* g2g, const int64_t* c2c, const int64_t* c2g, T* outputs,       \
            int64_t num_cell_nbs, int64_t num_grid_nbs, int64_t cells_per_grid,           \
            int64_t D, int64_t num_grids) {                                               \
        const int64_t len = num_grids * cells_per_grid;                                   \
        _Pragma("omp parallel for schedule(static)")                                      \
        for (int64_t i = 0; i < len; ++i) {                                               \
            if (!masks[i]) continue;                                                      \
            int64_t grid_idx = grid_indices[i / cells_per_grid];                          \
            int64_t cell_idx = cell_indices[i % cells_per_grid];                          \
            const int64_t* nb_g = g2g + num_grid_nbs * grid_idx;                          \
            const int64_t* nb_c = c2c + num_cell_nbs * cell_idx;                          \
            const int64_t* nb_cg = c2g + num_cell_nbs * cell_idx;                         \
            T acc[16] = {0};                                                              \
            for (int64_t k = 0; k < num_cell_nbs; ++k) {                                  \
                int64_t gi = nb_g[nb_cg[k]];                                              \
                if (gi < 0) continue;                                                     \
                const T* in = inputs + (gi * cells_per_grid + nb_c[k]) * D;               \
                const T* w = weights + k * D;                                             \
                for (int64_t c = 0; c < D; ++c) acc[c] += in[c] * w[c];                   \
            }                                                                             \
            T* out = outputs + (grid_idx * cells_per_grid + cell_idx) * D;                \
            for (int64_t c = 0; c < D; ++c) out[c] = acc[c];                              \
        }                                                                                 \
    }

DEFINE_QUERY(float, f32)
DEFINE_QUERY(double, f64)

/* ------------------------------------------------------------------------- */
/* Ray sampler                                                               */
/* ------------------------------------------------------------------------- */

/* Position along a ray, o + t * d, as one fused multiply-add per component:
 * the arithmetic both the oracle and the CUDA kernels commit to so that the
 * block a sample falls into is decided identically. */
static inline void ray_at(const float* o, const float* d, float t, float* p) {
    for (int k = 0; k < 3; ++k) p[k] = fmaf(t, d[k], o[k]);
}

static inline int ray_block_found(const oracle_map* m, const float* p, float cell2grid) {
    int32_t key[3];
    for (int k = 0; k < 3; ++k) key[k] = (int32_t)floorf(p[k] * cell2grid);
    return map_lookup(m, key) >= 0;
}

/* ash/src/sampler.cu:7-71 ray_find_near_far_kernel.  All lengths in cell
 * units; t_step is accepted and unused as in the reference. */
void oracle_ray_find_near_far(const oracle_map* m, const float* ray_o,
                              const float* ray_d, const float* bbox_min,
                              const float* bbox_max, float* nears, float* fars,
                              float t_min, float t_max, float t_step,
                              float grid2cell, int64_t n) {
    (void)t_step;
    const float cell2grid = (float)(1.0 / grid2cell);
    const float t_grid_step = (float)(grid2cell * 0.5);
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
        float near = -1, far = t_max, t = t_min;
        while (t < t_max) {
            float p[3];
            ray_at(ray_o + 3 * i, ray_d + 3 * i, t, p);
            int in_bound = 1;
            for (int k = 0; k < 3; ++k)
                in_bound = in_bound && (p[k] >= bbox_min[k] && p[k] <= bbox_max[k]);
            if (!in_bound) break;
            if (!ray_block_found(m, p, cell2grid)) {
                t += t_grid_step;
                continue;
            }
            near = (near < 0) ? t : fmaxf(near - t_grid_step, t_min);
            far = fminf(t + t_grid_step, t_max);
            t += t_grid_step;
        }
        nears[i] = near;
        fars[i] = far;
    }
}

/* ash/src/sampler.cu:123-215 ray_sample_count_kernel, run as the counting
 * pass (counts != NULL) or the assignment pass (ray_indices/t_nears/t_fars and
 * the inclusive prefix sum != NULL), :217-294. */
void oracle_ray_sample_pass(const oracle_map* m, const float* ray_o,
                            const float* ray_d, const float* ray_nears,
                            const float* ray_fars, int64_t* counts,
                            int64_t* ray_indices, float* t_nears, float* t_fars,
                            const int64_t* prefix_sum, int64_t max_samples_per_ray,
                            float grid2cell, int64_t n) {
    const float cell2grid = (float)(1.0 / grid2cell);
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
        const float ray_near = ray_nears[i], ray_far = ray_fars[i];
        /* sampler.cu:151: max(0.7, float) is evaluated in double, stored as float */
        const float t_step =
                (float)fmax(0.7, (double)((ray_far - ray_near) / (float)max_samples_per_ray));
        const float t_cell_step = t_step;
        const float t_grid_step = t_step * grid2cell;
        float t = ray_near, t_near = ray_near;
        int64_t local = 0;
        int64_t start = 0;
        if (!counts) start = (i == 0) ? 0 : prefix_sum[i - 1];
        while (t < ray_far) {
            float p[3];
            ray_at(ray_o + 3 * i, ray_d + 3 * i, t, p);
            if (!ray_block_found(m, p, cell2grid)) {
                t += t_grid_step;
            } else {
                t += t_cell_step;
                if (!counts) {
                    ray_indices[start + local] = i;
                    t_nears[start + local] = t_near;
                    t_fars[start + local] = t;
                }
                t_near = t;
                ++local;
            }
        }
        if (counts) counts[i] = local;
    }
}

/* ------------------------------------------------------------------------- */
/* Iso-surface vertices                                                      */
/* ------------------------------------------------------------------------- */

/* ash/src/grid.cu:453-532 isosurface_extraction_kernel: for every cell of the listed
 * blocks with weight >= weight_thr, look at its +x, +y, +z neighbour in turn; a sign
 * change of (sdf - iso_value) towards a neighbour with enough weight emits the linearly
 * interpolated crossing, in cell units.  A missing neighbour BLOCK ends the cell's loop
 * (`return`, :508-510), later axes included.  positions == NULL counts only (:556-572).
 * Sequential, so the output order is the scan order (the reference's is the order of its
 * atomic counter, i.e. unspecified).  Returns the number of vertices. */
int64_t oracle_isosurface_extraction_f32(
        const float* sdfs, const float* weights, const int64_t* grid_indices,
        const int32_t* grid_coords_table, const int64_t* g2g, const int32_t* cell_coords_table,
        const int64_t* c2c, const int64_t* c2g, float* positions, float iso_value,
        float weight_thr, int grid_dim, int64_t cells_per_grid, int64_t num_grids) {
    int64_t count = 0;
    for (int64_t i = 0; i < num_grids * cells_per_grid; ++i) {
        const int64_t grid_idx = grid_indices[i / cells_per_grid];
        const int64_t cell_idx = i % cells_per_grid;
        const float self_sdf = sdfs[grid_idx * cells_per_grid + cell_idx];
        const float self_weight = weights[grid_idx * cells_per_grid + cell_idx];
        const float self_isodiff = self_sdf - iso_value;
        if (self_weight < weight_thr) continue;
        for (int d = 0; d < 3; ++d) {
            const int cell_nb = 1 << d;
            const int64_t grid_nb_idx = g2g[grid_idx * 8 + c2g[cell_idx * 8 + cell_nb]];
            if (grid_nb_idx == -1) break;
            const int64_t cell_nb_idx = c2c[cell_idx * 8 + cell_nb];
            const float nb_sdf = sdfs[grid_nb_idx * cells_per_grid + cell_nb_idx];
            const float nb_weight = weights[grid_nb_idx * cells_per_grid + cell_nb_idx];
            const float nb_isodiff = nb_sdf - iso_value;
            if (self_isodiff * nb_isodiff < 0 && nb_weight >= weight_thr) {
                if (positions) {
                    const float ratio = self_isodiff / (self_isodiff - nb_isodiff);
                    for (int k = 0; k < 3; ++k) {
                        const int self_pos = grid_coords_table[grid_idx * 3 + k] * grid_dim +
                                             cell_coords_table[cell_idx * 3 + k];
                        positions[count * 3 + k] = (float)self_pos + ratio * (k == d ? 1.0f : 0.0f);
                    }
                }
                ++count;
            }
        }
    }
    return count;
}

/* ash/src/grid.cu:607-946 (marching_cubes: table-index, vertex and triangle kernels), in the
 * same three stages.  A cube sits at every cell of an active block whose own weight and the
 * weights of its 8 corners (the cell and its +x/+y/+z neighbours through the lookup tables)
 * reach weight_thr and whose neighbour blocks all exist (:640-668); corner c is inside when
 * sdf - iso_value < 0.  Every cut edge of a valid cube gets ONE vertex, owned by the cell at
 * the edge's lower corner and placed by linear interpolation (:744-770); triangles index
 * those vertices (:800-836).
 *
 * The reference's triangulation table (ash/src/mc_macros.h) is not reproduced: corner / edge
 * numbering and the table come from the generated mc_tables.h, so WHICH vertices a cube
 * connects in ambiguous patterns, the order of a triangle's corners, and the output order are
 * parity-unpinned against the reference; vertex positions follow the reference's formula.
 *
 * scratch: int32[num_embeddings * cells_per_grid * 3], vertex index per (cell, direction).
 * vertices / triangles == NULL counts only.  Returns 0, fills *n_vertices, *n_triangles. */
#include "mc_tables.h"

int64_t oracle_marching_cubes_f32(
        const float* sdfs, const float* weights, const int64_t* grid_indices,
        const int32_t* grid_coords_table, const int64_t* g2g, const int32_t* cell_coords_table,
        const int64_t* c2c, const int64_t* c2g, int32_t* scratch, int64_t num_embeddings,
        float* vertices, int32_t* triangles, float iso_value, float weight_thr, int grid_dim,
        int64_t cells_per_grid, int64_t num_grids, int64_t* n_vertices, int64_t* n_triangles) {
    const int64_t n_cells = num_grids * cells_per_grid;
    uint8_t* codes = (uint8_t*)calloc((size_t)(n_cells > 0 ? n_cells : 1), 1);
    for (int64_t i = 0; i < num_embeddings * cells_per_grid * 3; ++i) scratch[i] = -2;  /* no vertex wanted */
    /* stage 1: corner pattern of every valid cube; request the vertices of its cut edges */
    for (int64_t i = 0; i < n_cells; ++i) {
        const int64_t grid_idx = grid_indices[i / cells_per_grid];
        const int64_t cell_idx = i % cells_per_grid;
        int code = 0, valid = 1;
        int64_t corner_cell[8];
        for (int c = 0; c < 8 && valid; ++c) {
            const int64_t g = g2g[grid_idx * 8 + c2g[cell_idx * 8 + c]];
            if (g == -1) { valid = 0; break; }
            corner_cell[c] = g * cells_per_grid + c2c[cell_idx * 8 + c];
            if (weights[corner_cell[c]] < weight_thr) { valid = 0; break; }
            code |= ((sdfs[corner_cell[c]] - iso_value) < 0) << c;
        }
        if (!valid || code == 0 || code == 255) continue;
        codes[i] = (uint8_t)code;
        for (int e = 0; e < 12; ++e) {
            if (!(kMcEdgeMask[code] & (1 << e))) continue;
            const int d = e / 4, j = e % 4;
            const int lower = ((j & 1) << ((d + 1) % 3)) | ((j >> 1) << ((d + 2) % 3));
            scratch[corner_cell[lower] * 3 + d] = -1;  /* wanted */
        }
    }
    /* stage 2: one vertex per wanted edge, in the scan order of the owning cells */
    int64_t nv = 0;
    for (int64_t i = 0; i < n_cells; ++i) {
        const int64_t grid_idx = grid_indices[i / cells_per_grid];
        const int64_t cell_idx = i % cells_per_grid;
        const int64_t self = grid_idx * cells_per_grid + cell_idx;
        for (int d = 0; d < 3; ++d) {
            if (scratch[self * 3 + d] != -1) continue;
            const int64_t g = g2g[grid_idx * 8 + c2g[cell_idx * 8 + (1 << d)]];
            const int64_t nb = g * cells_per_grid + c2c[cell_idx * 8 + (1 << d)];
            const float self_isodiff = sdfs[self] - iso_value;
            const float nb_isodiff = sdfs[nb] - iso_value;
            if (vertices) {
                const float ratio = self_isodiff / (self_isodiff - nb_isodiff);
                for (int k = 0; k < 3; ++k) {
                    const int self_pos = grid_coords_table[grid_idx * 3 + k] * grid_dim +
                                         cell_coords_table[cell_idx * 3 + k];
                    vertices[nv * 3 + k] = (float)self_pos + ratio * (k == d ? 1.0f : 0.0f);
                }
            }
            scratch[self * 3 + d] = (int32_t)nv++;
        }
    }
    /* stage 3: triangles of every valid cube */
    int64_t nt = 0;
    for (int64_t i = 0; i < n_cells; ++i) {
        const int code = codes[i];
        if (!code) continue;
        const int64_t grid_idx = grid_indices[i / cells_per_grid];
        const int64_t cell_idx = i % cells_per_grid;
        for (int t = 0; t < kMcTriCount[code]; ++t) {
            if (triangles) {
                for (int v = 0; v < 3; ++v) {
                    const int e = kMcTris[code][3 * t + v];
                    const int d = e / 4, j = e % 4;
                    const int lower = ((j & 1) << ((d + 1) % 3)) | ((j >> 1) << ((d + 2) % 3));
                    const int64_t g = g2g[grid_idx * 8 + c2g[cell_idx * 8 + lower]];
                    const int64_t owner = g * cells_per_grid + c2c[cell_idx * 8 + lower];
                    triangles[nt * 3 + v] = scratch[owner * 3 + d];
                }
            }
            ++nt;
        }
    }
    free(codes);
    *n_vertices = nv;
    *n_triangles = nt;
    return 0;
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp master
        n = omp_get_num_threads();
    }
#endif
    return n;
}
