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
//
// Two front ends feed the same gather / scatter bodies:
//   LutSource    the reference's native interface: pre-split (grid index, cell index,
//                offset, mask) per query and three int64 neighbour tables;
//   FusedSource  positions in, everything else in-kernel: world -> cell transform,
//                block / cell / offset split (ash/grid.py:183-199), hash probe of the
//                block, corner cells by add-with-carry, and an int32 block-neighbour
//                row read only by queries whose cell touches a +x/+y/+z block face.
#include "query.cuh"

namespace ashb {

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

// Pre-split queries + lookup tables.  resolve() yields the 8 corner rows of query q
// (element offsets into the table) and its offsets; false when the query is masked
// out, its indices are out of range, or any neighbour block is absent: the
// reference leaves such rows zero (grid.cu:81-83, :109-111, :209-216).
struct LutSource {
    static constexpr int kForwardMinBlocks = 1;
    const float* __restrict__ offsets;
    QueryLuts L;

    // Row addressing: one table in this GPU's memory.
    template <typename T>
    __device__ __forceinline__ const T* in_row(const T* emb, int64_t b) const { return emb + b; }
    template <typename T>
    __device__ __forceinline__ T* out_row(T* grad, int64_t b) const { return grad + b; }
    template <typename T, int VEC>
    __device__ __forceinline__ Pack<T, VEC> corner(const T* emb, int64_t b, int64_t, int, int ch, int) const {
        return load_pack<T, VEC>(emb + b + ch);
    }


    __device__ __forceinline__ bool resolve(int64_t q, int lane, int64_t D, int64_t* base, float* off) const {
        (void)lane;
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
        off[0] = offsets[3 * q];
        off[1] = offsets[3 * q + 1];
        off[2] = offsets[3 * q + 2];
        return ok;
    }
};

// Positions in.  The split follows the Python layer operation by operation as it
// evaluates on a CUDA tensor (ash/grid.py:192-197, :756, :846): divisions by the
// cell size and by G are multiplications by float reciprocals, each rounded.
// The forward kernel with this source is built for 6 resident CTAs (<= 40 registers): faster than
// unconstrained (48 registers) and than 8 CTAs (spills).
#ifndef ASHB_FWD_MIN_BLOCKS
#define ASHB_FWD_MIN_BLOCKS 6
#endif
struct FusedSource {
    static constexpr int kForwardMinBlocks = ASHB_FWD_MIN_BLOCKS;
    // Row addressing: one table in this GPU's memory.
    template <typename T>
    __device__ __forceinline__ const T* in_row(const T* emb, int64_t b) const { return emb + b; }
    template <typename T>
    __device__ __forceinline__ T* out_row(T* grad, int64_t b) const { return grad + b; }
    template <typename T, int VEC>
    __device__ __forceinline__ Pack<T, VEC> corner(const T* emb, int64_t b, int64_t, int, int ch, int) const {
        return load_pack<T, VEC>(emb + b + ch);
    }

    Table16 table;
    const float* __restrict__ x;          // (n, 3) world positions
    float org[3];                         // world position of cell (0,0,0)
    float inv_cell;                       // 1 / cell_size (1 for plain grids)
    float G_f, inv_G;
    int G;
    const int32_t* __restrict__ nb_lut;   // (n_emb, 8) block -> neighbour block, -1 absent
    const int32_t* __restrict__ gi_in;    // saved block index per query (-1 = miss) or null: probe
    int32_t* __restrict__ gi_out;         // forward only: block index per query for the backward passes
    uint8_t* __restrict__ mask_out;       // forward only: hash hit mask
    int64_t n_emb;
    int64_t cells_per_grid;

    // Block index of query q (probe or saved), its cell and offsets; side outputs written by lane 0.
    __device__ __forceinline__ int locate(int64_t q, int lane, int* cell, float* off) const {
        int blk[3];
        const float xw[3] = {x[3 * q], x[3 * q + 1], x[3 * q + 2]};
        split_world_position(xw, org, inv_cell, inv_G, G_f, G, blk, cell, off);
        const int gi = gi_in ? gi_in[q] : lookup(table, blk[0], blk[1], blk[2], 0);
        if (lane == 0) {
            if (gi_out) gi_out[q] = gi;
            if (mask_out) mask_out[q] = (uint8_t)(gi >= 0);
        }
        return gi;
    }

    __device__ __forceinline__ bool resolve(int64_t q, int lane, int64_t D, int64_t* base, float* off) const {
        int cell[3];
        const int gi = locate(q, lane, cell, off);
        if (gi < 0 || gi >= n_emb) return false;
        return corner_rows(nb_lut, gi, cell, G, n_emb, cells_per_grid, D, base);
    }
};

// The table split over `world` GPUs by block: block g lives on GPU g % world as row g / world of
// that GPU's shard, and every shard is mapped into this GPU (peer memory over NVLink).  A corner
// row is then a peer address: rows are read with plain loads from, and gradients reduced straight
// into, the owner's memory -- the exchange a replicated table would need afterwards (a table-sized
// all-reduce) does not exist.  `base` carries the owner in its top byte.
struct ShardedSource : FusedSource {
    static constexpr int kForwardMinBlocks = 1;
    const void* const* __restrict__ emb_bases;   // device array [world]
    void* const* __restrict__ grad_bases;        // device array [world] (backward only)
    int world;

    static constexpr int kOwnerShift = 56;
    template <typename T>
    __device__ __forceinline__ const T* in_row(const T*, int64_t b) const {
        return static_cast<const T*>(emb_bases[b >> kOwnerShift]) + (b & ((1ll << kOwnerShift) - 1));
    }
    template <typename T>
    __device__ __forceinline__ T* out_row(T*, int64_t b) const {
        return static_cast<T*>(grad_bases[b >> kOwnerShift]) + (b & ((1ll << kOwnerShift) - 1));
    }
    // Corner c of query q.  The forward can keep a LOCAL copy of the rows it fetched (rows_out,
    // [n][8][D]) and the backward passes read that copy (rows_in) instead of crossing NVLink again.
    float* __restrict__ rows_out;
    const float* __restrict__ rows_in;
    template <typename T, int VEC>
    __device__ __forceinline__ Pack<T, VEC> corner(const T* emb, int64_t b, int64_t q, int c, int ch, int D) const {
        using V = typename Vec<T, VEC>::type;
        Pack<T, VEC> r;
        const int64_t kept = (q * 8 + c) * D + ch;
        if (rows_in) {
            *reinterpret_cast<V*>(r.v) = *reinterpret_cast<const V*>(reinterpret_cast<const T*>(rows_in) + kept);
            return r;
        }
        *reinterpret_cast<V*>(r.v) = *reinterpret_cast<const V*>(in_row(emb, b) + ch);  // plain load: may be a peer's
        if (rows_out) *reinterpret_cast<V*>(reinterpret_cast<T*>(rows_out) + kept) = *reinterpret_cast<const V*>(r.v);
        return r;
    }

    __device__ __forceinline__ bool resolve(int64_t q, int lane, int64_t D, int64_t* base, float* off) const {
        int cell[3];
        const int gi = locate(q, lane, cell, off);
        if (gi < 0 || gi >= n_emb) return false;
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
            const bool here = g >= 0 && g < n_emb;
            ok = ok && here;
            const int64_t local = here ? g / world : 0, owner = here ? g % world : 0;
            base[c] = ((local * cells_per_grid + (cc[0] + (cc[1] + cc[2] * G) * G)) * D) | (owner << kOwnerShift);
        }
        return ok;
    }
};

// ---- forward -------------------------------------------------------------------
template <typename T, int VEC, class Src>
__global__ void __launch_bounds__(256, Src::kForwardMinBlocks) query_forward_kernel(const T* __restrict__ emb, Src src,
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
    float off[3];
    if (src.resolve(q, lane, D, base, off)) {
        AxisWeights<T> aw;
        aw.init(interp, off);
        Pack<T, VEC> e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) e[c] = src.template corner<T, VEC>(emb, base[c], q, c, ch, D);
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
// grad_off receives d/d offset times `go_scale` (1 for the pre-split interface, 1 / cell_size
// when the caller differentiates w.r.t. world positions).  With grad_off == nullptr only the
// scatter runs: the eight embedding rows are not read at all.
#ifndef ASHB_BWD_MIN_BLOCKS
#define ASHB_BWD_MIN_BLOCKS 1
#endif
template <typename T, int VEC, class Src, bool NEED_GO, bool NEED_GE = true>
__global__ void __launch_bounds__(256, ASHB_BWD_MIN_BLOCKS) query_backward_forward_kernel(
        const T* __restrict__ z, const T* __restrict__ emb, Src src, T* __restrict__ grad_emb,
        T* __restrict__ grad_off, T go_scale, int64_t n, int D, int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lanes = 1 << lane_shift;
    const int lane = (int)(tid & (lanes - 1));
    const int ch = lane * VEC;
    // Whole groups stay together for the shuffles below (no early return).
    const bool live = q < n;
    const bool has_ch = ch < D;
    T go[3] = {0, 0, 0};
    int64_t base[8];
    float off[3];
    if (live && src.resolve(q, lane, D, base, off)) {
        AxisWeights<T> aw;
        aw.init(interp, off);
        if (has_ch) {
            const Pack<T, VEC> zv = load_pack<T, VEC>(z + q * D + ch);
            Pack<T, VEC> e[8];
            if (NEED_GO) {
#pragma unroll
                for (int c = 0; c < 8; ++c) e[c] = src.template corner<T, VEC>(emb, base[c], q, c, ch, D);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const T w = aw.weight(c);
                Pack<T, VEC> g;
                T dot = 0;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    g.v[k] = w * zv.v[k];
                    if (NEED_GO) dot += e[c].v[k] * zv.v[k];
                }
                if (NEED_GE) atomic_add_pack<T, VEC>(src.out_row(grad_emb, base[c]) + ch, g);
                if (NEED_GO) {
                    T wg[3];
                    aw.grad(c, wg);
                    go[0] += dot * wg[0];
                    go[1] += dot * wg[1];
                    go[2] += dot * wg[2];
                }
            }
        }
    }
    if (!NEED_GO) return;
#pragma unroll
    for (int d = 0; d < 3; ++d) go[d] = group_sum(go[d], lanes);
    if (live && lane == 0) {
        grad_off[3 * q] = go[0] * go_scale;
        grad_off[3 * q + 1] = go[1] * go_scale;
        grad_off[3 * q + 2] = go[2] * go_scale;
    }
}

// ---- backward with warp-aggregated scatter ----------------------------------------------
// Lanes of a warp that are about to add to the SAME gradient row slice (queries that share a corner,
// as consecutive samples along a ray do) are found with a match on the element offset; their
// contributions are summed with shuffles and the lowest lane issues one vector reduction for all.
// Every lane of the warp takes part in the match (lanes without a contribution use a key of their
// own), and the shuffle rounds are bounded by the largest peer group in the warp: none when no
// two lanes collide.
template <typename T, int VEC>
__device__ __forceinline__ void scatter_aggregated(T* grad, int64_t elem_off, const Pack<T, VEC>& g, bool valid) {
    const int wl = threadIdx.x & 31;
    const unsigned long long key = valid ? (unsigned long long)elem_off : (0xFFFFFFFF00000000ull | (unsigned)wl);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const int rounds = __reduce_max_sync(0xffffffffu, __popc(peers));
    Pack<T, VEC> sum = g;
    unsigned rest = peers & ~(1u << wl);
    for (int it = 1; it < rounds; ++it) {
        const bool take = rest != 0;
        const int from = take ? __ffs(rest) - 1 : wl;
        rest &= rest - 1;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const T v = __shfl_sync(0xffffffffu, g.v[k], from);
            if (take) sum.v[k] += v;
        }
    }
    if (valid && wl == __ffs(peers) - 1) atomic_add_pack<T, VEC>(grad + elem_off, sum);
}

template <typename T, int VEC, class Src, bool NEED_GO>
__global__ void __launch_bounds__(256) query_backward_forward_agg_kernel(
        const T* __restrict__ z, const T* __restrict__ emb, Src src, T* __restrict__ grad_emb,
        T* __restrict__ grad_off, T go_scale, int64_t n, int D, int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lanes = 1 << lane_shift;
    const int lane = (int)(tid & (lanes - 1));
    const int ch = lane * VEC;
    const bool live = q < n;
    int64_t base[8];
    float off[3] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 8; ++c) base[c] = 0;
    const bool ok = live && src.resolve(q, lane, D, base, off);
    const bool valid = ok && ch < D;
    AxisWeights<T> aw;
    aw.init(interp, off);
    Pack<T, VEC> zv;
#pragma unroll
    for (int k = 0; k < VEC; ++k) zv.v[k] = 0;
    if (valid) zv = load_pack<T, VEC>(z + q * D + ch);
    Pack<T, VEC> e[8];
    if (NEED_GO && valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) e[c] = src.template corner<T, VEC>(emb, base[c], q, c, ch, D);
    }
    T go[3] = {0, 0, 0};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const T w = aw.weight(c);
        Pack<T, VEC> g;
        T dot = 0;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            g.v[k] = w * zv.v[k];
            if (NEED_GO && valid) dot += e[c].v[k] * zv.v[k];
        }
        scatter_aggregated<T, VEC>(src.out_row(grad_emb, 0), base[c] + ch, g, valid);
        if (NEED_GO) {
            T wg[3];
            aw.grad(c, wg);
            go[0] += dot * wg[0];
            go[1] += dot * wg[1];
            go[2] += dot * wg[2];
        }
    }
    if (!NEED_GO) return;
#pragma unroll
    for (int d = 0; d < 3; ++d) go[d] = group_sum(go[d], lanes);
    if (live && lane == 0) {
        grad_off[3 * q] = go[0] * go_scale;
        grad_off[3 * q + 1] = go[1] * go_scale;
        grad_off[3 * q + 2] = go[2] * go_scale;
    }
}

// ---- clear the rows a batch touches ---------------------------------------------------
// Writes zeros to the 8 corner rows of every query: the sparse counterpart of zero-filling a
// table-sized gradient buffer between steps when gradients are accumulated in place.
template <typename T, int VEC, class Src>
__global__ void __launch_bounds__(256) query_zero_rows_kernel(Src src, T* __restrict__ grad_emb, int64_t n, int D,
                                                              int lane_shift) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    if (q >= n || ch >= D) return;
    int64_t base[8];
    float off[3];
    if (!src.resolve(q, lane, D, base, off)) return;
    Pack<T, VEC> zero;
#pragma unroll
    for (int k = 0; k < VEC; ++k) zero.v[k] = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) store_pack<T, VEC>(src.out_row(grad_emb, base[c]) + ch, zero);
}

// ---- double backward ----------------------------------------------------------------
template <typename T, int VEC, class Src>
__global__ void __launch_bounds__(256, ASHB_BWD_MIN_BLOCKS) query_backward_backward_kernel(
        const T* __restrict__ ggo, const T* __restrict__ z, const T* __restrict__ emb, Src src,
        T* __restrict__ grad_z, T* __restrict__ grad_emb, T go_scale, int64_t n, int D, int lane_shift,
        int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    if (q >= n || ch >= D) return;
    Pack<T, VEC> gz;
#pragma unroll
    for (int k = 0; k < VEC; ++k) gz.v[k] = 0;
    int64_t base[8];
    float off[3];
    if (src.resolve(q, lane, D, base, off)) {
        const T g3[3] = {ggo[3 * q] * go_scale, ggo[3 * q + 1] * go_scale, ggo[3 * q + 2] * go_scale};
        AxisWeights<T> aw;
        aw.init(interp, off);
        const Pack<T, VEC> zv = load_pack<T, VEC>(z + q * D + ch);
        Pack<T, VEC> e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) e[c] = src.template corner<T, VEC>(emb, base[c], q, c, ch, D);
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
            atomic_add_pack<T, VEC>(src.out_row(grad_emb, base[c]) + ch, g);
        }
    }
    store_pack<T, VEC>(grad_z + q * D + ch, gz);
}

// ---- backward passes that WRITE the embedding gradient as a row list ---------------------------
// Instead of adding eight rows per query into a table-sized buffer (a read-modify-write of eight
// random lines, on top of a table-sized zero-fill when the buffer is fresh), the gradient leaves as
// 8 n records in query-major order: record 8 q + c = (block index, cell index, row of D values) of
// corner c of query q, so a CTA writes three contiguous streams.
// Every store is coalesced and nothing is read back, so the pass moves its algorithmic bytes and
// no more.  The list is an uncoalesced sparse tensor of the table's shape (duplicates mean
// "add"); ashb_rows_scatter_add applies it to any dense buffer (a gradient, or the parameters
// themselves with a step size).  Queries that produce no gradient (miss, absent neighbour block)
// write zero rows that point at valid cells spread over the table, so the list is well-formed as it is.
// SECOND = false: first-order pass (rows = w_c * z, d/d offset as in query_backward_forward_kernel);
// SECOND = true: double backward (rows = (grad w_c . ggo) * z, grad_z as in
// query_backward_backward_kernel; `side` is grad_z [n][D], `ggo` the incoming gradient).
// Resident CTAs per SM each variant is built for (register budget): the double backward holds 8 rows
// and 8 products at once and runs best with room (2), the first-order pass with d/dx at 3, the
// write-only pass without the row reads at 4.
template <typename T, int VEC, bool SECOND, bool NEED_GO>
__global__ void __launch_bounds__(256, SECOND ? 3 : (NEED_GO ? 3 : 4)) query_backward_rows_kernel(
        const T* __restrict__ z, const T* __restrict__ emb, FusedSource src, const T* __restrict__ ggo,
        int64_t* __restrict__ idx_out, T* __restrict__ rows_out, T* __restrict__ side, T go_scale, int64_t n, int D,
        int lane_shift, int interp) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> lane_shift;
    const int lanes = 1 << lane_shift;
    const int lane = (int)(tid & (lanes - 1));
    const int ch = lane * VEC;
    const bool live = q < n;
    const bool has_ch = ch < D;
    // The records of a warp's queries are one contiguous stretch of the list (4 KB of rows when a lane
    // holds 16 bytes of a row and the lanes cover it exactly), but a lane produces them corner by
    // corner: 64 bytes here, 64 bytes half a kilobyte on.  So the warp first lays its records out in
    // shared memory and then copies them out with every store instruction covering 512 contiguous
    // bytes.  16-byte chunk j of the warp's stretch sits at j ^ ((its query * lanes) & 7): the lanes of
    // a quarter warp then write different banks, and a row of 8 chunks stays a row for the copy.
    __shared__ uint4 stage_rows[8][256];
    __shared__ int64_t stage_idx[8][2][64];
    const bool staged = sizeof(T) * VEC == 16 && D == lanes * VEC && lanes >= 4;
    const int warp = threadIdx.x >> 5, warp_lane = threadIdx.x & 31;
    const int ql = warp_lane >> lane_shift;   // query within the warp
    const int swizzle = (ql * lanes) & 7;
    T go[3] = {0, 0, 0};
    Pack<T, VEC> gz;
#pragma unroll
    for (int k = 0; k < VEC; ++k) gz.v[k] = 0;
    if (live) {
        int cell[3], blocks[8], cells[8];
        float off[3];
        const int gi = src.locate(q, lane, cell, off);
        const bool ok = gi >= 0 && gi < src.n_emb && corner_blocks_cells(src.nb_lut, gi, cell, src.G, src.n_emb, blocks, cells);
        // the 8 index pairs of the query are shared out over its lanes
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if ((c & (lanes - 1)) != lane) continue;
            const int64_t block = ok ? blocks[c] : (int64_t)(q % src.n_emb);
            const int64_t cell_of = ok ? cells[c] : (int64_t)(c % src.cells_per_grid);
            if (staged) {
                stage_idx[warp][0][ql * 8 + c] = block;
                stage_idx[warp][1][ql * 8 + c] = cell_of;
            } else {
                idx_out[q * 8 + c] = block;
                idx_out[(n + q) * 8 + c] = cell_of;
            }
        }
        if (has_ch && !ok) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (staged) stage_rows[warp][(((ql * 8 + c) << lane_shift) + lane) ^ swizzle] = make_uint4(0, 0, 0, 0);
                else store_pack<T, VEC>(rows_out + (q * 8 + c) * D + ch, gz);
            }
            if (SECOND) store_pack<T, VEC>(side + q * D + ch, gz);
        } else if (has_ch) {
            AxisWeights<T> aw;
            aw.init(interp, off);
            const Pack<T, VEC> zv = load_pack<T, VEC>(z + q * D + ch);
            Pack<T, VEC> e[8];
            if (SECOND || NEED_GO) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    e[c] = load_pack<T, VEC>(emb + ((int64_t)blocks[c] * src.cells_per_grid + cells[c]) * D + ch);
            }
            T g3[3] = {0, 0, 0};
            if (SECOND) {
                g3[0] = ggo[3 * q] * go_scale;
                g3[1] = ggo[3 * q + 1] * go_scale;
                g3[2] = ggo[3 * q + 2] * go_scale;
            }
            T* out = rows_out + q * 8 * D + ch;
            const int64_t corner_stride = D;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                T wg[3] = {0, 0, 0};
                if (SECOND || NEED_GO) aw.grad(c, wg);
                const T w = SECOND ? wg[0] * g3[0] + wg[1] * g3[1] + wg[2] * g3[2] : aw.weight(c);
                Pack<T, VEC> g;
                T dot = 0;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    g.v[k] = w * zv.v[k];
                    if (SECOND) gz.v[k] += w * e[c].v[k];
                    if (!SECOND && NEED_GO) dot += e[c].v[k] * zv.v[k];
                }
                if (staged) stage_rows[warp][(((ql * 8 + c) << lane_shift) + lane) ^ swizzle] = *reinterpret_cast<const uint4*>(g.v);
                else store_pack<T, VEC>(out, g);
                out += corner_stride;
                if (!SECOND && NEED_GO) {
                    go[0] += dot * wg[0];
                    go[1] += dot * wg[1];
                    go[2] += dot * wg[2];
                }
            }
            if (SECOND) store_pack<T, VEC>(side + q * D + ch, gz);
        }
    }
    if (staged) {
        __syncwarp();
        const int64_t q0 = (tid - warp_lane) >> lane_shift;   // the warp's first query
        if (q0 < n) {
            uint4* dst = reinterpret_cast<uint4*>(rows_out + q0 * 8 * D);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int j = k * 32 + warp_lane;
                const int jq = j >> (3 + lane_shift);
                if (q0 + jq < n) dst[j] = stage_rows[warp][j ^ ((jq * lanes) & 7)];
            }
            for (int j = warp_lane; j < (256 >> lane_shift); j += 32) {
                if (q0 + (j >> 3) >= n) continue;
                idx_out[q0 * 8 + j] = stage_idx[warp][0][j];
                idx_out[(n + q0) * 8 + j] = stage_idx[warp][1][j];
            }
        }
    }
    if (SECOND || !NEED_GO) return;
#pragma unroll
    for (int d = 0; d < 3; ++d) go[d] = group_sum(go[d], lanes);
    if (live && lane == 0) {
        side[3 * q] = go[0] * go_scale;
        side[3 * q + 1] = go[1] * go_scale;
        side[3 * q + 2] = go[2] * go_scale;
    }
}

// dst[idx[0][r]][idx[1][r]][:] += alpha * rows[r][:] for the m records of a row list.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) rows_scatter_add_kernel(T* __restrict__ dst, const int64_t* __restrict__ idx,
                                                               const T* __restrict__ rows, int64_t m, int64_t n_emb,
                                                               int64_t cells, int D, int lane_shift, T alpha) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t r = tid >> lane_shift;
    const int ch = (int)(tid & ((1 << lane_shift) - 1)) * VEC;
    if (r >= m || ch >= D) return;
    const int64_t g = idx[r], c = idx[m + r];
    if (g < 0 || g >= n_emb || c < 0 || c >= cells) return;
    using V = typename Vec<T, VEC>::type;
    Pack<T, VEC> v;
    *reinterpret_cast<V*>(v.v) = *reinterpret_cast<const V*>(rows + r * D + ch);
    bool any = false;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        any = any || v.v[k] != 0;
        v.v[k] *= alpha;
    }
    if (any) atomic_add_pack<T, VEC>(dst + (g * cells + c) * D + ch, v);
}

// ---- host-side dispatch ---------------------------------------------------------------
// Process-wide: scatter the first-order embedding gradient with warp aggregation of duplicate rows.
static bool g_scatter_aggregation = false;

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

template <typename T, class Src>
static int forward_impl(int interp, const void* emb, const Src& src, void* out, int64_t n, int64_t D,
                        cudaStream_t st) {
    const void* ptrs[] = {emb, out};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 2);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_forward_kernel<T, VEC, Src><<<grid, 256, 0, st>>>(static_cast<const T*>(emb), src,
                                                                              static_cast<T*>(out), n, (int)D,
                                                                              sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T, class Src>
static int backward_forward_impl(int interp, const void* z, const void* emb, const Src& src, void* grad_emb,
                                 void* grad_off, double go_scale, int64_t n, int64_t D, cudaStream_t st) {
    const void* ptrs[] = {emb, z, grad_emb};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 3);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (g_scatter_aggregation && grad_emb != nullptr) {
        ASHB_VEC_SWITCH(T, sh,
                        if (grad_off != nullptr) {
                            query_backward_forward_agg_kernel<T, VEC, Src, true><<<grid, 256, 0, st>>>(
                                    static_cast<const T*>(z), static_cast<const T*>(emb), src,
                                    static_cast<T*>(grad_emb), static_cast<T*>(grad_off), (T)go_scale, n, (int)D,
                                    sh.lane_shift, interp);
                        } else {
                            query_backward_forward_agg_kernel<T, VEC, Src, false><<<grid, 256, 0, st>>>(
                                    static_cast<const T*>(z), static_cast<const T*>(emb), src,
                                    static_cast<T*>(grad_emb), nullptr, (T)go_scale, n, (int)D, sh.lane_shift,
                                    interp);
                        });
        ASHB_LAUNCH_CHECK();
        return ASHB_OK;
    }
    ASHB_VEC_SWITCH(T, sh,
                    if (grad_emb == nullptr) {
                        query_backward_forward_kernel<T, VEC, Src, true, false><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src, nullptr,
                                static_cast<T*>(grad_off), (T)go_scale, n, (int)D, sh.lane_shift, interp);
                    } else if (grad_off != nullptr) {
                        query_backward_forward_kernel<T, VEC, Src, true><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src,
                                static_cast<T*>(grad_emb), static_cast<T*>(grad_off), (T)go_scale, n, (int)D,
                                sh.lane_shift, interp);
                    } else {
                        query_backward_forward_kernel<T, VEC, Src, false><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src,
                                static_cast<T*>(grad_emb), nullptr, (T)go_scale, n, (int)D, sh.lane_shift, interp);
                    });
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T, class Src>
static int backward_backward_impl(int interp, const void* ggo, const void* z, const void* emb, const Src& src,
                                  void* grad_z, void* grad_emb, double go_scale, int64_t n, int64_t D,
                                  cudaStream_t st) {
    const void* ptrs[] = {emb, z, grad_emb, grad_z};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 4);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_backward_backward_kernel<T, VEC, Src><<<grid, 256, 0, st>>>(
                            static_cast<const T*>(ggo), static_cast<const T*>(z), static_cast<const T*>(emb), src,
                            static_cast<T*>(grad_z), static_cast<T*>(grad_emb), (T)go_scale, n, (int)D,
                            sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

// ---- block-neighbour table ---------------------------------------------------------------
// For every live (block coordinate -> index) pair: the indices of the 8 blocks at offsets
// {0,1}^3 (bit d of the column = offset along axis d), -1 where absent, and optionally the
// coordinate itself.  One table scan + 8 probes per block replaces items() + find(8n) + two
// scatters of ash/grid.py:566-617.  Rows of inactive indices must be pre-filled with -1.
__global__ void __launch_bounds__(256) build_nb_lut_kernel(Table16 t, int32_t* __restrict__ lut,
                                                           int32_t* __restrict__ coords, int64_t n_emb) {
    const uint64_t n_slots = (uint64_t)t.mask + 1;
    for (uint64_t s = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; s < n_slots;
         s += (uint64_t)gridDim.x * blockDim.x) {
        const Entry e = t.read_const((uint32_t)s);
        if (e.val < 0 || e.val >= n_emb) continue;
        int32_t row[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
            row[c] = c == 0 ? e.val : lookup(t, e.k0 + (c & 1), e.k1 + ((c >> 1) & 1), e.k2 + ((c >> 2) & 1), 0);
        int4* dst = reinterpret_cast<int4*>(lut + (int64_t)e.val * 8);
        dst[0] = make_int4(row[0], row[1], row[2], row[3]);
        dst[1] = make_int4(row[4], row[5], row[6], row[7]);
        if (coords) {
            coords[3 * (int64_t)e.val] = e.k0;
            coords[3 * (int64_t)e.val + 1] = e.k1;
            coords[3 * (int64_t)e.val + 2] = e.k2;
        }
    }
}

static int make_fused_source(ashb_map* m, const float* x, double cell_size, const float* origin, int G,
                             const int32_t* nb_lut, const int32_t* gi_in, int32_t* gi_out, uint8_t* mask_out,
                             int64_t n_emb, FusedSource* out) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim == 3, "the grid query needs a 3-D map");
    ASHB_REQUIRE(G >= 1 && G <= 64 && cell_size > 0.0, "bad grid_dim or cell_size");
    ASHB_REQUIRE(x && nb_lut, "null buffer");
    ASHB_REQUIRE(((uintptr_t)nb_lut & 15) == 0, "neighbour table must be 16-byte aligned");
    FusedSource f{};
    f.table = table16_of(m);
    f.x = x;
    for (int d = 0; d < 3; ++d) f.org[d] = origin ? origin[d] : 0.f;
    // the reciprocal is formed in double and rounded once, as torch does for `tensor / python_float`
    f.inv_cell = (float)(1.0 / cell_size);
    f.G = G;
    f.G_f = (float)G;
    f.inv_G = 1.0f / (float)G;
    f.nb_lut = nb_lut;
    f.gi_in = gi_in;
    f.gi_out = gi_out;
    f.mask_out = mask_out;
    f.n_emb = n_emb;
    f.cells_per_grid = (int64_t)G * G * G;
    *out = f;
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
    const LutSource src{offsets, QueryLuts{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid}};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == ASHB_F32 ? forward_impl<float>(interp, embeddings, src, out, n, D, st)
                             : forward_impl<double>(interp, embeddings, src, out, n, D, st);
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
    const LutSource src{offsets, QueryLuts{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid}};
    return dtype == ASHB_F32 ? backward_forward_impl<float>(interp, z, embeddings, src, grad_embeddings,
                                                            grad_offsets, 1.0, n, D, st)
                             : backward_forward_impl<double>(interp, z, embeddings, src, grad_embeddings,
                                                             grad_offsets, 1.0, n, D, st);
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
    const LutSource src{offsets, QueryLuts{grid_indices, cell_indices, masks, g2g, c2c, c2g, n_emb, cells_per_grid}};
    return dtype == ASHB_F32
                   ? backward_backward_impl<float>(interp, grad_grad_offsets, z, embeddings, src, grad_z,
                                                   grad_embeddings, 1.0, n, D, st)
                   : backward_backward_impl<double>(interp, grad_grad_offsets, z, embeddings, src, grad_z,
                                                    grad_embeddings, 1.0, n, D, st);
}

int ashb_grid_build_neighbor_lut(ashb_map* m, int32_t* lut, int32_t* grid_coords, int64_t n_emb, void* stream) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim == 3 && lut != nullptr && n_emb >= 1, "needs a 3-D map and an output table");
    ASHB_REQUIRE(((uintptr_t)lut & 15) == 0, "neighbour table must be 16-byte aligned");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemsetAsync(lut, 0xFF, (size_t)n_emb * 8 * sizeof(int32_t), st));
    if (grid_coords) ASHB_CUDA_TRY(cudaMemsetAsync(grid_coords, 0xFF, (size_t)n_emb * 3 * sizeof(int32_t), st));
    build_nb_lut_kernel<<<wave_grid((int64_t)m->n_slots, 256, 8), 256, 0, st>>>(table16_of(m), lut, grid_coords,
                                                                                 n_emb);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_grid_query_forward(ashb_map* m, int dtype, int interp, const void* embeddings, const float* x,
                            double cell_size, const float* origin, int G, const int32_t* nb_lut, void* out,
                            uint8_t* masks, int32_t* block_idx_out, int64_t n, int64_t n_emb, int64_t D,
                            void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(embeddings && out && masks, "null buffer");
    FusedSource src;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, nullptr, block_idx_out, masks, n_emb, &src))
        return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == ASHB_F32 ? forward_impl<float>(interp, embeddings, src, out, n, D, st)
                             : forward_impl<double>(interp, embeddings, src, out, n, D, st);
}

int ashb_grid_query_backward(ashb_map* m, int dtype, int interp, const void* z, const void* embeddings,
                             const float* x, double cell_size, const float* origin, int G, const int32_t* nb_lut,
                             const int32_t* block_idx, void* grad_embeddings, void* grad_x, int zero_grad,
                             int64_t n, int64_t n_emb, int64_t D, void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    ASHB_REQUIRE(grad_embeddings != nullptr || grad_x != nullptr, "nothing to compute: both outputs are null");
    ASHB_REQUIRE(m != nullptr, "null map");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elem = dtype == ASHB_F32 ? 4 : 8;
    if (zero_grad && grad_embeddings)
        ASHB_CUDA_TRY(cudaMemsetAsync(grad_embeddings, 0, (size_t)n_emb * G * G * G * D * elem, st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(z && embeddings, "null buffer");
    FusedSource src;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, block_idx, nullptr, nullptr, n_emb, &src))
        return rc;
    const double scale = (double)(float)(1.0 / cell_size);  // the float reciprocal the forward split multiplies by
    return dtype == ASHB_F32 ? backward_forward_impl<float>(interp, z, embeddings, src, grad_embeddings, grad_x,
                                                            scale, n, D, st)
                             : backward_forward_impl<double>(interp, z, embeddings, src, grad_embeddings, grad_x,
                                                             scale, n, D, st);
}

// ---- the table split over the GPUs of one box (peer memory) ---------------------------------
static int make_sharded_source(ashb_map* m, const void* const* emb_bases, void* const* grad_bases, int world,
                               const float* x, double cell_size, const float* origin, int G, const int32_t* nb_lut,
                               const int32_t* gi_in, int32_t* gi_out, uint8_t* mask_out, int64_t n_emb,
                               float* rows_out, const float* rows_in, ShardedSource* out) {
    ASHB_REQUIRE(world >= 1 && world <= 64 && emb_bases != nullptr, "bad world size or null shard table");
    FusedSource f;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, gi_in, gi_out, mask_out, n_emb, &f)) return rc;
    ShardedSource s{};
    static_cast<FusedSource&>(s) = f;
    s.emb_bases = emb_bases;
    s.grad_bases = grad_bases;
    s.world = world;
    s.rows_out = rows_out;
    s.rows_in = rows_in;
    *out = s;
    return ASHB_OK;
}

int ashb_grid_query_forward_sharded(ashb_map* m, int interp, const void* const* emb_bases_dev, int world,
                                    const float* x, double cell_size, const float* origin, int G,
                                    const int32_t* nb_lut, float* out, uint8_t* masks, int32_t* block_idx_out,
                                    float* rows_out, int64_t n, int64_t n_emb, int64_t D, void* stream) {
    if (int rc = check_query_args(ASHB_F32, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(out && masks, "null buffer");
    ShardedSource src;
    if (int rc = make_sharded_source(m, emb_bases_dev, nullptr, world, x, cell_size, origin, G, nb_lut, nullptr,
                                     block_idx_out, masks, n_emb, rows_out, nullptr, &src))
        return rc;
    DeviceGuard guard(m->device);
    return forward_impl<float>(interp, nullptr, src, out, n, D, static_cast<cudaStream_t>(stream));
}

int ashb_grid_query_backward_sharded(ashb_map* m, int interp, const float* z, const void* const* emb_bases_dev,
                                     void* const* grad_bases_dev, int world, const float* x, double cell_size,
                                     const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx,
                                     float* grad_x, int need_grad_embeddings, const float* rows_in, int64_t n,
                                     int64_t n_emb, int64_t D, void* stream) {
    if (int rc = check_query_args(ASHB_F32, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(z && (grad_bases_dev || !need_grad_embeddings), "null buffer");
    ASHB_REQUIRE(need_grad_embeddings || grad_x, "nothing to compute");
    ShardedSource src;
    if (int rc = make_sharded_source(m, emb_bases_dev, grad_bases_dev, world, x, cell_size, origin, G, nb_lut,
                                     block_idx, nullptr, nullptr, n_emb, nullptr, rows_in, &src))
        return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const void* ptrs[] = {z, rows_in};
    const Shape sh = pick_shape(D, sizeof(float), ptrs, 1);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    const float scale = (float)(1.0 / cell_size);
    float* none = nullptr;
    ASHB_VEC_SWITCH(float, sh,
                    if (!need_grad_embeddings) {
                        query_backward_forward_kernel<float, VEC, ShardedSource, true, false><<<grid, 256, 0, st>>>(
                                z, none, src, none, grad_x, scale, n, (int)D, sh.lane_shift, interp);
                    } else if (grad_x != nullptr) {
                        query_backward_forward_kernel<float, VEC, ShardedSource, true><<<grid, 256, 0, st>>>(
                                z, none, src, none, grad_x, scale, n, (int)D, sh.lane_shift, interp);
                    } else {
                        query_backward_forward_kernel<float, VEC, ShardedSource, false><<<grid, 256, 0, st>>>(
                                z, none, src, none, none, scale, n, (int)D, sh.lane_shift, interp);
                    });
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_grid_query_backward_backward_sharded(ashb_map* m, int interp, const float* grad_grad_x, const float* z,
                                              const void* const* emb_bases_dev, void* const* grad_bases_dev,
                                              int world, const float* x, double cell_size, const float* origin,
                                              int G, const int32_t* nb_lut, const int32_t* block_idx, float* grad_z,
                                              const float* rows_in, int64_t n, int64_t n_emb, int64_t D,
                                              void* stream) {
    if (int rc = check_query_args(ASHB_F32, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(grad_grad_x && z && grad_z && grad_bases_dev, "null buffer");
    ShardedSource src;
    if (int rc = make_sharded_source(m, emb_bases_dev, grad_bases_dev, world, x, cell_size, origin, G, nb_lut,
                                     block_idx, nullptr, nullptr, n_emb, nullptr, rows_in, &src))
        return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const void* ptrs[] = {z, grad_z, rows_in};
    const Shape sh = pick_shape(D, sizeof(float), ptrs, 2);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    const float scale = (float)(1.0 / cell_size);
    float* none = nullptr;
    ASHB_VEC_SWITCH(float, sh,
                    (query_backward_backward_kernel<float, VEC, ShardedSource><<<grid, 256, 0, st>>>(
                            grad_grad_x, z, none, src, grad_z, none, scale, n, (int)D, sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_grid_query_backward_backward(ashb_map* m, int dtype, int interp, const void* grad_grad_x, const void* z,
                                      const void* embeddings, const float* x, double cell_size,
                                      const float* origin, int G, const int32_t* nb_lut,
                                      const int32_t* block_idx, void* grad_z, void* grad_embeddings,
                                      int zero_grad, int64_t n, int64_t n_emb, int64_t D, void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    ASHB_REQUIRE(grad_embeddings != nullptr, "null grad_embeddings");
    ASHB_REQUIRE(m != nullptr, "null map");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t elem = dtype == ASHB_F32 ? 4 : 8;
    if (zero_grad)
        ASHB_CUDA_TRY(cudaMemsetAsync(grad_embeddings, 0, (size_t)n_emb * G * G * G * D * elem, st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(grad_grad_x && z && embeddings && grad_z, "null buffer");
    FusedSource src;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, block_idx, nullptr, nullptr, n_emb, &src))
        return rc;
    const double scale = (double)(float)(1.0 / cell_size);  // the float reciprocal the forward split multiplies by
    return dtype == ASHB_F32 ? backward_backward_impl<float>(interp, grad_grad_x, z, embeddings, src, grad_z,
                                                             grad_embeddings, scale, n, D, st)
                             : backward_backward_impl<double>(interp, grad_grad_x, z, embeddings, src, grad_z,
                                                              grad_embeddings, scale, n, D, st);
}

}  // extern "C"

template <typename T>
static int backward_rows_impl(int interp, bool second, const void* ggo, const void* z, const void* emb,
                              const FusedSource& src, int64_t* idx_out, void* rows_out, void* side, double go_scale,
                              int64_t n, int64_t D, cudaStream_t st) {
    const void* ptrs[] = {emb, z, rows_out, second ? side : nullptr};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 4);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    if (second) {
                        query_backward_rows_kernel<T, VEC, true, false><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src, static_cast<const T*>(ggo),
                                idx_out, static_cast<T*>(rows_out), static_cast<T*>(side), (T)go_scale, n, (int)D,
                                sh.lane_shift, interp);
                    } else if (side != nullptr) {
                        query_backward_rows_kernel<T, VEC, false, true><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src, nullptr, idx_out,
                                static_cast<T*>(rows_out), static_cast<T*>(side), (T)go_scale, n, (int)D, sh.lane_shift,
                                interp);
                    } else {
                        query_backward_rows_kernel<T, VEC, false, false><<<grid, 256, 0, st>>>(
                                static_cast<const T*>(z), static_cast<const T*>(emb), src, nullptr, idx_out,
                                static_cast<T*>(rows_out), nullptr, (T)go_scale, n, (int)D, sh.lane_shift, interp);
                    });
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T>
static int rows_scatter_add_impl(void* dst, const int64_t* idx, const void* rows, int64_t m, int64_t n_emb,
                                 int64_t cells, int64_t D, double alpha, cudaStream_t st) {
    const void* ptrs[] = {dst, rows};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 2);
    const int64_t threads = m << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (rows_scatter_add_kernel<T, VEC><<<grid, 256, 0, st>>>(static_cast<T*>(dst), idx,
                                                                            static_cast<const T*>(rows), m, n_emb, cells,
                                                                            (int)D, sh.lane_shift, (T)alpha)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

template <typename T>
static int zero_rows_impl(const FusedSource& src, void* grad_emb, int64_t n, int64_t D, cudaStream_t st) {
    const void* ptrs[] = {grad_emb};
    const Shape sh = pick_shape(D, sizeof(T), ptrs, 1);
    const int64_t threads = n << sh.lane_shift;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    ASHB_VEC_SWITCH(T, sh,
                    (query_zero_rows_kernel<T, VEC, FusedSource><<<grid, 256, 0, st>>>(src, static_cast<T*>(grad_emb), n,
                                                                                        (int)D, sh.lane_shift)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

extern "C" {

int ashb_grid_zero_rows(ashb_map* m, int dtype, void* grad_embeddings, const float* x, double cell_size,
                        const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx, int64_t n,
                        int64_t n_emb, int64_t D, void* stream) {
    if (int rc = check_query_args(dtype, ASHB_LINEAR, n, n_emb, (int64_t)G * G * G, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(grad_embeddings != nullptr && m != nullptr, "null buffer");
    FusedSource src;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, block_idx, nullptr, nullptr, n_emb, &src))
        return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == ASHB_F32 ? zero_rows_impl<float>(src, grad_embeddings, n, D, st)
                             : zero_rows_impl<double>(src, grad_embeddings, n, D, st);
}

int ashb_grid_query_backward_rows(ashb_map* m, int dtype, int interp, int second_order, const void* grad_grad_x,
                                  const void* z, const void* embeddings, const float* x, double cell_size,
                                  const float* origin, int G, const int32_t* nb_lut, const int32_t* block_idx,
                                  int64_t* idx_out, void* rows_out, void* side_out, int64_t n, int64_t n_emb, int64_t D,
                                  void* stream) {
    if (int rc = check_query_args(dtype, interp, n, n_emb, (int64_t)G * G * G, D)) return rc;
    ASHB_REQUIRE(m != nullptr, "null map");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(z && embeddings && idx_out && rows_out, "null buffer");
    ASHB_REQUIRE(!second_order || (grad_grad_x && side_out), "the double backward needs grad_grad_x and grad_z");
    FusedSource src;
    if (int rc = make_fused_source(m, x, cell_size, origin, G, nb_lut, block_idx, nullptr, nullptr, n_emb, &src))
        return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const double scale = (double)(float)(1.0 / cell_size);
    return dtype == ASHB_F32 ? backward_rows_impl<float>(interp, second_order != 0, grad_grad_x, z, embeddings, src,
                                                         idx_out, rows_out, side_out, scale, n, D, st)
                             : backward_rows_impl<double>(interp, second_order != 0, grad_grad_x, z, embeddings, src,
                                                          idx_out, rows_out, side_out, scale, n, D, st);
}

int ashb_rows_scatter_add(int dtype, void* dst, const int64_t* idx, const void* rows, int64_t m, int64_t n_emb,
                          int64_t cells_per_grid, int64_t D, double alpha, void* stream) {
    ASHB_REQUIRE(dtype == ASHB_F32 || dtype == ASHB_F64, "unknown dtype code %d", dtype);
    ASHB_REQUIRE(m >= 0 && n_emb >= 1 && cells_per_grid >= 1 && D >= 1 && D <= 16, "bad sizes");
    if (m == 0) return ASHB_OK;
    ASHB_REQUIRE(dst && idx && rows, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == ASHB_F32 ? rows_scatter_add_impl<float>(dst, idx, rows, m, n_emb, cells_per_grid, D, alpha, st)
                             : rows_scatter_add_impl<double>(dst, idx, rows, m, n_emb, cells_per_grid, D, alpha, st);
}

int ashb_set_scatter_aggregation(int enable) {
    g_scatter_aggregation = enable != 0;
    return ASHB_OK;
}

}  // extern "C"
