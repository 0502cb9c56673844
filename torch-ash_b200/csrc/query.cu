// Sparse-dense grid query for sm_100a: 8-corner gather + trilinear / smooth-step
// interpolation, its backward (gradient scatter + d/d offset) and double
// backward, over the lookup tables the reference's Python layer builds
// (ash/grid.py:526-617).  Semantics follow ash/src/grid.cu:69-451.
//
// Work decomposition: a query is served by a group of LANES = 2^k threads; lane
// j owns VEC consecutive channels of the D-wide embedding row, so one corner row
// is fetched with one coalesced 16-byte load per lane (D = 16 fp32: 4 lanes x
// float4 = the whole 64-byte row) and scattered with one vector atomic per
// lane.  All 8 corner loads of a lane are independent and issued back to back.
// Row offsets are 64-bit (the reference's 32-bit `base_idx` overflows beyond
// 2^31 table elements).
#include "common.cuh"

namespace ashb {

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

struct QueryLuts {
    const int64_t* __restrict__ grid_indices;
    const int64_t* __restrict__ cell_indices;
    const uint8_t* __restrict__ masks;
    const int64_t* __restrict__ g2g;
    const int64_t* __restrict__ c2c;
    const int64_t* __restrict__ c2g;
    int64_t n_emb;
    int64_t cells_per_grid;
};

// Resolve the 8 corner rows of query q (element offsets into the table).
// False when the query is masked out, its indices are out of range, or any
// neighbour block is absent: the reference leaves such rows zero
// (grid.cu:81-83, :109-111, :209-216).
__device__ __forceinline__ bool resolve_corners(const QueryLuts& L, int64_t q, int64_t D, int64_t* base) {
    if (!L.masks[q]) return false;
    const int64_t gi = L.grid_indices[q];
    const int64_t ci = L.cell_indices[q];
    if (gi < 0 || gi >= L.n_emb || ci < 0 || ci >= L.cells_per_grid) return false;
    const longlong2* nb_cg = reinterpret_cast<const longlong2*>(L.c2g + ci * 8);
    const longlong2* nb_cc = reinterpret_cast<const longlong2*>(L.c2c + ci * 8);
    const int64_t* nb_g = L.g2g + gi * 8;
    bool ok = true;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const longlong2 cg = __ldg(nb_cg + h);
        const longlong2 cc = __ldg(nb_cc + h);
        const int64_t g0 = __ldg(nb_g + (cg.x & 7));
        const int64_t g1 = __ldg(nb_g + (cg.y & 7));
        ok = ok && g0 >= 0 && g0 < L.n_emb && g1 >= 0 && g1 < L.n_emb && cc.x >= 0 &&
             cc.x < L.cells_per_grid && cc.y >= 0 && cc.y < L.cells_per_grid;
        base[2 * h] = (g0 * L.cells_per_grid + cc.x) * D;
        base[2 * h + 1] = (g1 * L.cells_per_grid + cc.y) * D;
    }
    return ok;
}

template <typename T>
__device__ __forceinline__ T group_sum(T v, int lanes) {
    for (int o = lanes >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- forward -------------------------------------------------------------------
template <typename T, int VEC>
__global__ void __launch_bounds__(256) query_forward_kernel(const T* __restrict__ emb,
                                                            const float* __restrict__ offsets, QueryLuts L,
                                                            T* __restrict__ out, int64_t n, int D,
                                                            int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    if (q >= n || ch >= D) return;
    Pack<T, VEC> acc;
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc.v[k] = 0;
    int64_t base[8];
    if (resolve_corners(L, q, D, base)) {
        const float off[3] = {offsets[3 * q], offsets[3 * q + 1], offsets[3 * q + 2]};
        AxisWeights<T> aw;
        aw.init(interp, off);
        Pack<T, VEC> e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) e[c] = load_pack<T, VEC>(emb + base[c] + ch);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const T w = aw.weight(c);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc.v[k] += w * e[c].v[k];
        }
    }
    store_pack<T, VEC>(out + q * D + ch, acc);
}

// ---- backward: d/d embeddings (scatter) and d/d offsets -----------------------------
template <typename T, int VEC>
__global__ void __launch_bounds__(256) query_backward_forward_kernel(
        const T* __restrict__ z, const T* __restrict__ emb, const float* __restrict__ offsets, QueryLuts L,
        T* __restrict__ grad_emb, T* __restrict__ grad_off, int64_t n, int D, int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lanes = 1 << lane_shift;
    const int lane = (int)(tid & (lanes - 1));
    const int ch = lane * VEC;
    // Whole groups stay together for the shuffles below; n is padded by the
    // launch to a multiple of the groups per block.
    const bool live = q < n;
    const bool has_ch = ch < D;
    T go[3] = {0, 0, 0};
    int64_t base[8];
    if (live && resolve_corners(L, q, D, base)) {
        const float off[3] = {offsets[3 * q], offsets[3 * q + 1], offsets[3 * q + 2]};
        AxisWeights<T> aw;
        aw.init(interp, off);
        if (has_ch) {
            const Pack<T, VEC> zv = load_pack<T, VEC>(z + q * D + ch);
            Pack<T, VEC> e[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) e[c] = load_pack<T, VEC>(emb + base[c] + ch);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const T w = aw.weight(c);
                Pack<T, VEC> g;
                T dot = 0;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    g.v[k] = w * zv.v[k];
                    dot += e[c].v[k] * zv.v[k];
                }
                atomic_add_pack<T, VEC>(grad_emb + base[c] + ch, g);
                T wg[3];
                aw.grad(c, wg);
                go[0] += dot * wg[0];
                go[1] += dot * wg[1];
                go[2] += dot * wg[2];
            }
        }
    }
#pragma unroll
    for (int d = 0; d < 3; ++d) go[d] = group_sum(go[d], lanes);
    if (live && lane == 0) {
        grad_off[3 * q] = go[0];
        grad_off[3 * q + 1] = go[1];
        grad_off[3 * q + 2] = go[2];
    }
}

// ---- double backward ----------------------------------------------------------------
template <typename T, int VEC>
__global__ void __launch_bounds__(256) query_backward_backward_kernel(
        const T* __restrict__ ggo, const T* __restrict__ z, const T* __restrict__ emb,
        const float* __restrict__ offsets, QueryLuts L, T* __restrict__ grad_z, T* __restrict__ grad_emb,
        int64_t n, int D, int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    if (q >= n || ch >= D) return;
    Pack<T, VEC> gz;
#pragma unroll
    for (int k = 0; k < VEC; ++k) gz.v[k] = 0;
    int64_t base[8];
    if (resolve_corners(L, q, D, base)) {
        const float off[3] = {offsets[3 * q], offsets[3 * q + 1], offsets[3 * q + 2]};
        const T g3[3] = {ggo[3 * q], ggo[3 * q + 1], ggo[3 * q + 2]};
        AxisWeights<T> aw;
        aw.init(interp, off);
        const Pack<T, VEC> zv = load_pack<T, VEC>(z + q * D + ch);
        Pack<T, VEC> e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) e[c] = load_pack<T, VEC>(emb + base[c] + ch);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            T wg[3];
            aw.grad(c, wg);
            const T dot = wg[0] * g3[0] + wg[1] * g3[1] + wg[2] * g3[2];
            Pack<T, VEC> g;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                g.v[k] = dot * zv.v[k];
                gz.v[k] += dot * e[c].v[k];
            }
            atomic_add_pack<T, VEC>(grad_emb + base[c] + ch, g);
        }
    }
    store_pack<T, VEC>(grad_z + q * D + ch, gz);
}

// ---- host-side dispatch ---------------------------------------------------------------
struct Shape {
    int vec;         // channels per lane
    int lane_shift;  // log2(lanes per query)
};

// Widest vector (<= 16 bytes) that divides D and that every row pointer is
// aligned for; lanes = next power of two >= D / vec.
static Shape pick_shape(int64_t D, size_t elem, const void* const* ptrs, int n_ptrs) {
    int vec = (int)(16 / elem);
    uintptr_t bits = 0;
    for (int i = 0; i < n_ptrs; ++i) bits |= (uintptr_t)ptrs[i];
    while (vec > 1 && (D % vec != 0 || (bits & (uintptr_t)(vec * elem - 1)))) vec >>= 1;
    int chunks = (int)(D / vec);
    int shift = 0;
    while ((1 << shift) < chunks) ++shift;
    return Shape{vec, shift};
}

static int check_query_args(int dtype, int interp, int64_t n, int64_t n_emb, int64_t cells, int64_t D) {
    ASHB_REQUIRE(dtype == ASHB_F32 || dtype == ASHB_F64, "unknown dtype code %d", dtype);
    ASHB_REQUIRE(interp == ASHB_LINEAR || interp == ASHB_SMOOTH_STEP, "unknown interpolation code %d", interp);
    ASHB_REQUIRE(n >= 0 && n_emb >= 1 && cells >= 1, "bad sizes n=%lld n_emb=%lld cells=%lld", (long long)n,
                 (long long)n_emb, (long long)cells);
    ASHB_REQUIRE(D >= 1 && D <= 16, "embedding_dim %lld not in 1..16", (long long)D);
    return ASHB_OK;
}

// The two per-cell tables are read as 16-byte pairs.
static int check_lut_alignment(const void* c2c, const void* c2g) {
    ASHB_REQUIRE((((uintptr_t)c2c | (uintptr_t)c2g) & 15) == 0, "cell lookup tables must be 16-byte aligned");
    return ASHB_OK;
}

#define ASHB_VEC_SWITCH(T, shape, ...)                      \
    switch ((shape).vec) {                                  \
        case 4:                                             \
            if constexpr (sizeof(T) == 4) {                 \
                constexpr int VEC = 4;                      \
                __VA_ARGS__;                                \
            }                                               \
            break;                                          \
        case 2: {                                           \
            constexpr int VEC = 2;                          \
            __VA_ARGS__;                                    \
        } break;                                            \
        default: {                                          \
            constexpr int VEC = 1;                          \
            __VA_ARGS__;                                    \
        }                                                   \
    }

template <typename T>
static int forward_impl(int interp, const void* emb, const float* offsets, const QueryLuts& L, void* out,
                        int64_t n, int64_t D, cudaStream_t st) {
    const void* ptrs[] = {emb, out};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 2);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_forward_kernel<T, VEC><<<grid, 256, 0, st>>>(static_cast<const T*>(emb), offsets, L,
                                                                         static_cast<T*>(out), n, (int)D,
                                                                         sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T>
static int backward_forward_impl(int interp, const void* z, const void* emb, const float* offsets,
                                 const QueryLuts& L, void* grad_emb, void* grad_off, int64_t n, int64_t D,
                                 cudaStream_t st) {
    const void* ptrs[] = {emb, z, grad_emb};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 3);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_backward_forward_kernel<T, VEC><<<grid, 256, 0, st>>>(
                            static_cast<const T*>(z), static_cast<const T*>(emb), offsets, L,
                            static_cast<T*>(grad_emb), static_cast<T*>(grad_off), n, (int)D, sh.lane_shift,
                            interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T>
static int backward_backward_impl(int interp, const void* ggo, const void* z, const void* emb,
                                  const float* offsets, const QueryLuts& L, void* grad_z, void* grad_emb,
                                  int64_t n, int64_t D, cudaStream_t st) {
    const void* ptrs[] = {emb, z, grad_emb, grad_z};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 4);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_backward_backward_kernel<T, VEC><<<grid, 256, 0, st>>>(
                            static_cast<const T*>(ggo), static_cast<const T*>(z), static_cast<const T*>(emb),
                            offsets, L, static_cast<T*>(grad_z), static_cast<T*>(grad_emb), n, (int)D,
                            sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // namespace ashb

using namespace ashb;

extern "C" {

int ashb_query_forward(int dtype, int interp, const void* embeddings, const float* offsets,
                       const int64_t* grid_indices, const int64_t* cell_indices, const uint8_t* masks,
                       const int64_t* g2g, const int64_t* c2c, const int64_t* c2g, void* out, int64_t n,
                       int64_t n_emb, int64_t cells_per_grid, int64_t D, void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, cells_per_grid, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(embeddings && offsets && grid_indices && cell_indices && masks && g2g && c2c && c2g && out,
                 "null buffer");
    if (int rc = check_lut_alignment(c2c, c2g)) return rc;
    const QueryLuts L{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == ASHB_F32 ? forward_impl<float>(interp, embeddings, offsets, L, out, n, D, st)
                             : forward_impl<double>(interp, embeddings, offsets, L, out, n, D, st);
}

int ashb_query_backward_forward(int dtype, int interp, const void* z, const void* embeddings,
                                const float* offsets, const int64_t* grid_indices,
                                const int64_t* cell_indices, const uint8_t* masks, const int64_t* g2g,
                                const int64_t* c2c, const int64_t* c2g, void* grad_embeddings,
                                void* grad_offsets, int zero_grad, int64_t n, int64_t n_emb,
                                int64_t cells_per_grid, int64_t D, void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, cells_per_grid, D)) return rc;
    ASHB_REQUIRE(grad_embeddings != nullptr, "null grad_embeddings");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elem = dtype == ASHB_F32 ? 4 : 8;
    if (zero_grad)
        ASHB_CUDA_TRY(cudaMemsetAsync(grad_embeddings, 0, (size_t)n_emb * cells_per_grid * D * elem, st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(z && embeddings && offsets && grid_indices && cell_indices && masks && g2g && c2c && c2g &&
                         grad_offsets,
                 "null buffer");
    if (int rc = check_lut_alignment(c2c, c2g)) return rc;
    const QueryLuts L{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid};
    return dtype == ASHB_F32 ? backward_forward_impl<float>(interp, z, embeddings, offsets, L, grad_embeddings,
                                                            grad_offsets, n, D, st)
                             : backward_forward_impl<double>(interp, z, embeddings, offsets, L,
                                                             grad_embeddings, grad_offsets, n, D, st);
}

int ashb_query_backward_backward(int dtype, int interp, const void* grad_grad_offsets, const void* z,
                                 const void* embeddings, const float* offsets, const int64_t* grid_indices,
                                 const int64_t* cell_indices, const uint8_t* masks, const int64_t* g2g,
                                 const int64_t* c2c, const int64_t* c2g, void* grad_z, void* grad_embeddings,
                                 int zero_grad, int64_t n, int64_t n_emb, int64_t cells_per_grid, int64_t D,
                                 void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, cells_per_grid, D)) return rc;
    ASHB_REQUIRE(grad_embeddings != nullptr, "null grad_embeddings");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elem = dtype == ASHB_F32 ? 4 : 8;
    if (zero_grad)
        ASHB_CUDA_TRY(cudaMemsetAsync(grad_embeddings, 0, (size_t)n_emb * cells_per_grid * D * elem, st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(grad_grad_offsets && z && embeddings && offsets && grid_indices && cell_indices && masks &&
                         g2g && c2c && c2g && grad_z,
                 "null buffer");
    if (int rc = check_lut_alignment(c2c, c2g)) return rc;
    const QueryLuts L{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid};
    return dtype == ASHB_F32
                   ? backward_backward_impl<float>(interp, grad_grad_offsets, z, embeddings, offsets, L, grad_z,
                                                   grad_embeddings, n, D, st)
                   : backward_backward_impl<double>(interp, grad_grad_offsets, z, embeddings, offsets, L,
                                                    grad_z, grad_embeddings, n, D, st);
}

}  // extern "C"
