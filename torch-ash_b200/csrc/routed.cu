// Sparse-dense grid query over a table SPLIT across the GPUs of one box, with the QUERIES routed
// to the owners of their blocks (one process per GPU, every rank's shard, gradient shard and
// mailbox mapped into every other rank over NVLink).  The reference is single-GPU and has no
// counterpart.
//
// Why route queries instead of rows: a query needs 8 rows of D values from the table and adds 8
// rows to its gradient (D = 16: 512 bytes each way), but is itself 12 bytes in and D values out.
// Sending the position to the rank that holds the block and letting that rank gather, interpolate
// and scatter in its OWN memory moves 16 + 4 D (+ 4 D + 16 in the backward pass) bytes per query
// over NVLink instead of ~64 D.  Blocks are assigned to ranks by a hash of their coarse
// coordinate (block >> 3 per axis, fewer bits when that balances badly), so a block and its
// +x/+y/+z neighbours mostly share an owner;
// the few corner rows that do not are read from, and reduced into, the neighbour's owner directly
// (plain peer loads and `red.global.add` over NVLink).
//
// One training step is, on every rank,
//   route     every position -> 16-byte record {x, y, z, block index} in its owner's inbox (slot
//             from a local cursor: rank r owns region r of every inbox, no remote atomic)
//   (barrier: a one-element collective enqueued on the same stream)
//   forward   the owner interpolates the records of its inbox and stores each result row straight
//             into the asker's result buffer, region by region in inbox order (contiguous stores)
//   (barrier) the asker gathers its rows locally (it noted owner and slot per query while routing)
//   send_z    the asker stores dL/dy of every query into the owner's second inbox at the same slot
//   (barrier)
//   backward  the owner adds the 8 gradient rows per record into its gradient shard and stores
//             dL/dx into the asker's buffer
//   (barrier) the asker gathers dL/dx.
// The double backward (a loss on dL/dx, e.g. an eikonal term) is one more round of the same kind: the
// asker sends dL/dy again together with the gradient arriving at dL/dx, the owner adds the second-order
// gradient rows into its shard and returns the gradient with respect to dL/dy through the result buffer.
// No kernel waits on another GPU; ordering comes from the collectives between the launches.  Every
// remote address is base[peer] + offset with offsets checked against the mailbox size on the host
// and slots re-checked on the device; records that do not fit are dropped and reported.
#include "query.cuh"

namespace ashb {

constexpr int kRoutedMaxWorld = 32;                       // owner << 26 | slot must stay a non-negative int32
constexpr int kRowOwnerShift = 26;                       // row_of[g] = owner << 26 | row in the owner's shard
constexpr uint32_t kRowLocalMask = (1u << kRowOwnerShift) - 1;

struct RoutedLayout {
    void* const* bases;       // device array [world]: every rank's mailbox as mapped here
    int64_t inbox_x;          // float4 [world][cap]: {x, y, z, block index bits}
    int64_t counts;           // int32 [world]
    int64_t inbox_z;          // float [world][cap][D]
    int64_t out_y;            // float [world][cap][D]: region o = rows computed by owner o, in its inbox order
    int64_t out_gx;           // float4 [world][cap]
    int64_t inbox_g;          // float4 [world][cap]: gradient arriving at dL/dx (double backward)
    int64_t cap;              // records per region
    int world, rank;
};

struct RoutedGrid {
    Table16 table;
    const int32_t* __restrict__ nb_lut;    // (n_emb, 8) replicated
    const uint32_t* __restrict__ row_of;   // (n_emb) replicated
    const void* const* emb_bases;          // [world] embedding shards
    void* const* grad_bases;               // [world] gradient shards
    float org[3];
    float inv_cell, G_f, inv_G;
    int G;
    int64_t n_emb, cells;
};

// ---- asker: route positions ------------------------------------------------------------------
__global__ void __launch_bounds__(256) routed_route_kernel(const float* __restrict__ x, int64_t n, RoutedGrid g,
                                                           RoutedLayout L, int* __restrict__ cursor,
                                                           int32_t* __restrict__ where, uint32_t* __restrict__ status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int gi = -1;
    float xw[3] = {0.f, 0.f, 0.f};
    if (i < n) {
        xw[0] = x[3 * i];
        xw[1] = x[3 * i + 1];
        xw[2] = x[3 * i + 2];
        int blk[3], cell[3];
        float off[3];
        split_world_position(xw, g.org, g.inv_cell, g.inv_G, g.G_f, g.G, blk, cell, off);
        gi = lookup(g.table, blk[0], blk[1], blk[2], 0);
        if (gi >= g.n_emb) gi = -1;
    }
    const bool live = gi >= 0;
    // lanes without a record take a negative owner of their own, so that they match nobody
    const int owner = live ? (int)(g.row_of[gi] >> kRowOwnerShift) : -1 - lane;
    __shared__ int cta_count[kRoutedMaxWorld];
    __shared__ int cta_base[kRoutedMaxWorld];
    for (int o = threadIdx.x; o < L.world; o += blockDim.x) cta_count[o] = 0;
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, owner);
    const int leader = __ffs(peers) - 1;
    int within = 0;
    if (live && lane == leader) within = atomicAdd(&cta_count[owner], __popc(peers));
    within = __shfl_sync(0xffffffffu, within, leader);
    __syncthreads();
    for (int o = threadIdx.x; o < L.world; o += blockDim.x)
        cta_base[o] = cta_count[o] ? atomicAdd(&cursor[o], cta_count[o]) : 0;
    __syncthreads();
    if (i >= n) return;
    if (!live || owner >= L.world) {
        where[i] = -1;
        return;
    }
    const int64_t slot = (int64_t)cta_base[owner] + within + __popc(peers & lanemask_lt());
    if (slot >= L.cap) {
        atomicOr(status, ASHB_STATUS_CAPACITY);
        where[i] = -1;
        return;
    }
    float4* inbox = reinterpret_cast<float4*>(static_cast<char*>(L.bases[owner]) + L.inbox_x);
    inbox[(int64_t)L.rank * L.cap + slot] = make_float4(xw[0], xw[1], xw[2], __int_as_float(gi));
    where[i] = (int)((unsigned)owner << kRowOwnerShift | (unsigned)slot);
}

__global__ void routed_publish_counts_kernel(RoutedLayout L, const int* __restrict__ cursor) {
    const int o = threadIdx.x;
    if (o >= L.world) return;
    int* counts = reinterpret_cast<int*>(static_cast<char*>(L.bases[o]) + L.counts);
    const int64_t c = cursor[o];
    counts[L.rank] = (int)(c < L.cap ? c : L.cap);
}

// ---- owner side: corner rows of a record --------------------------------------------------------
// Element offsets of the 8 corner rows inside their owners' shards, with the owner in the top byte.
constexpr int kOwnerByteShift = 56;

__device__ __forceinline__ bool routed_corner_rows(const RoutedGrid& g, int gi, const int* cell, int D, int64_t* base,
                                                   bool* all_mine, int rank) {
    const int32_t* row = g.nb_lut + (int64_t)gi * 8;
    bool ok = true, mine = true;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        int cc[3], nb = 0;
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            cc[d] = cell[d] + ((c >> d) & 1);
            if (cc[d] == g.G) {
                cc[d] = 0;
                nb |= 1 << d;
            }
        }
        const int b = nb ? __ldg(row + nb) : gi;
        const bool here = b >= 0 && b < g.n_emb;
        ok = ok && here;
        const uint32_t r = here ? __ldg(g.row_of + b) : 0u;
        const int64_t owner = r >> kRowOwnerShift, local = r & kRowLocalMask;
        mine = mine && owner == rank;
        base[c] = ((local * g.cells + (cc[0] + (cc[1] + cc[2] * g.G) * g.G)) * D) | (owner << kOwnerByteShift);
    }
    *all_mine = mine;
    return ok;
}

__device__ __forceinline__ const float* routed_in_row(const RoutedGrid& g, int64_t b) {
    return static_cast<const float*>(g.emb_bases[b >> kOwnerByteShift]) + (b & ((1ll << kOwnerByteShift) - 1));
}
__device__ __forceinline__ float* routed_out_row(const RoutedGrid& g, int64_t b) {
    return static_cast<float*>(g.grad_bases[b >> kOwnerByteShift]) + (b & ((1ll << kOwnerByteShift) - 1));
}

template <int VEC>
__device__ __forceinline__ Pack<float, VEC> routed_corner(const RoutedGrid& g, int64_t b, int ch, bool mine) {
    const float* p = routed_in_row(g, b) + ch;
    if (mine) return load_pack<float, VEC>(p);   // this GPU's own rows: read-only path, 64-byte fills
    using V = typename Vec<float, VEC>::type;     // a neighbour's owner: plain peer load
    Pack<float, VEC> r;
    *reinterpret_cast<V*>(r.v) = *reinterpret_cast<const V*>(p);
    return r;
}

// Record j of region `region` of this rank's inbox; false when there is none.
__device__ __forceinline__ bool routed_record(const RoutedLayout& L, int region, int64_t j, float4* rec) {
    const char* mine = static_cast<const char*>(L.bases[L.rank]);
    const int count = __ldcg(reinterpret_cast<const int*>(mine + L.counts) + region);
    if (j >= count || j >= L.cap) return false;
    *rec = __ldcg(reinterpret_cast<const float4*>(mine + L.inbox_x) + (int64_t)region * L.cap + j);
    return true;
}

// ---- owner: forward -----------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256, 5) routed_forward_kernel(RoutedGrid g, RoutedLayout L, int D, int lane_shift,
                                                             int interp) {
    const int region = blockIdx.y;   // the rank that asked
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t j = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    float4 rec;
    if (ch >= D || !routed_record(L, region, j, &rec)) return;
    Pack<float, VEC> acc;
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc.v[k] = 0;
    const int gi = __float_as_int(rec.w);
    if (gi >= 0 && gi < g.n_emb) {
        const float xw[3] = {rec.x, rec.y, rec.z};
        int blk[3], cell[3];
        float off[3];
        split_world_position(xw, g.org, g.inv_cell, g.inv_G, g.G_f, g.G, blk, cell, off);
        int64_t base[8];
        bool mine;
        if (routed_corner_rows(g, gi, cell, D, base, &mine, L.rank)) {
            AxisWeights<float> aw;
            aw.init(interp, off);
            Pack<float, VEC> e[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) e[c] = routed_corner<VEC>(g, base[c], ch, mine);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float w = aw.weight(c);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc.v[k] += w * e[c].v[k];
            }
        }
    }
    float* out = reinterpret_cast<float*>(static_cast<char*>(L.bases[region]) + L.out_y);
    store_pack<float, VEC>(out + ((int64_t)L.rank * L.cap + j) * D + ch, acc);   // my region of the asker's rows
}

// ---- asker: gather result rows / send dL/dy / gather dL/dx -----------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256) routed_unpack_y_kernel(RoutedLayout L, const int32_t* __restrict__ where,
                                                              int64_t n, float* __restrict__ y,
                                                              uint8_t* __restrict__ masks, int D, int lane_shift) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t i = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    if (i >= n || ch >= D) return;
    const int w = where[i];
    Pack<float, VEC> r;
#pragma unroll
    for (int k = 0; k < VEC; ++k) r.v[k] = 0;
    if (w >= 0) {
        const int owner = (int)((unsigned)w >> kRowOwnerShift);
        const int64_t slot = (unsigned)w & kRowLocalMask;
        const float* rows = reinterpret_cast<const float*>(static_cast<const char*>(L.bases[L.rank]) + L.out_y);
        using V = typename Vec<float, VEC>::type;
        *reinterpret_cast<V*>(r.v) = __ldcg(reinterpret_cast<const V*>(rows + ((int64_t)owner * L.cap + slot) * D + ch));
    }
    store_pack<float, VEC>(y + i * D + ch, r);
    if (lane == 0 && masks) masks[i] = (uint8_t)(w >= 0);
}

// The asker's dL/dy rows go to the slots its positions took in the owners' inboxes.  A CTA handles the
// 256 queries one route CTA handled, so those that went to one owner hold consecutive slots there: the
// CTA orders its queries by (owner, slot) in shared memory and stores the rows in that order, a warp
// instruction covering up to 512 contiguous bytes of one owner's inbox instead of eight 64-byte pieces
// in eight places (what a link carries well is long segments).  Nothing depends on the slots really
// being consecutive: a query whose slot falls outside its owner's run stores its row on its own.
template <int VEC>
__global__ void __launch_bounds__(256) routed_send_z_kernel(RoutedLayout L, const int32_t* __restrict__ where, int64_t n,
                                                            const float* __restrict__ z, int D, int lane_shift) {
    __shared__ int lowest[kRoutedMaxWorld], count[kRoutedMaxWorld], start[kRoutedMaxWorld + 1];
    __shared__ short order[256];   // order[p] = the tile's query at position p of the (owner, slot) order
    const int t = threadIdx.x;
    const int64_t first = (int64_t)blockIdx.x * 256;
    for (int o = t; o < L.world; o += blockDim.x) {
        lowest[o] = 0x7fffffff;
        count[o] = 0;
    }
    order[t] = -1;
    __syncthreads();
    const int64_t i = first + t;
    const int w = i < n ? where[i] : -1;
    const int owner = w >= 0 ? (int)((unsigned)w >> kRowOwnerShift) : 0;
    const int slot = w >= 0 ? (int)((unsigned)w & kRowLocalMask) : 0;
    const bool sends = w >= 0 && owner < L.world && slot < L.cap;
    if (sends) {
        atomicMin(&lowest[owner], slot);
        atomicAdd(&count[owner], 1);
    }
    __syncthreads();
    if (t == 0) {
        int sum = 0;
        for (int o = 0; o < L.world; ++o) {
            start[o] = sum;
            sum += count[o];
        }
        start[L.world] = sum;
    }
    __syncthreads();
    const bool placed = sends && slot - lowest[owner] < count[owner];
    if (placed) order[start[owner] + slot - lowest[owner]] = (short)t;
    __syncthreads();
    const int lanes = 1 << lane_shift;
    const int ch = (t & (lanes - 1)) * VEC;
    if (ch < D) {
        for (int p = t >> lane_shift; p < start[L.world]; p += 256 >> lane_shift) {
            const int query = order[p];
            if (query < 0) continue;
            const int wq = where[first + query];
            float* inbox = reinterpret_cast<float*>(static_cast<char*>(L.bases[(unsigned)wq >> kRowOwnerShift]) + L.inbox_z);
            store_pack<float, VEC>(inbox + ((int64_t)L.rank * L.cap + ((unsigned)wq & kRowLocalMask)) * D + ch,
                                   load_pack<float, VEC>(z + (first + query) * D + ch));
        }
    }
    if (sends && !placed) {
        float* inbox = reinterpret_cast<float*>(static_cast<char*>(L.bases[owner]) + L.inbox_z) + ((int64_t)L.rank * L.cap + slot) * D;
        for (int c = 0; c < D; ++c) inbox[c] = z[i * D + c];
    }
}

__global__ void __launch_bounds__(256) routed_unpack_gx_kernel(RoutedLayout L, const int32_t* __restrict__ where,
                                                               int64_t n, float* __restrict__ grad_x) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int w = where[i];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (w >= 0) {
        const int owner = (int)((unsigned)w >> kRowOwnerShift);
        const int64_t slot = (unsigned)w & kRowLocalMask;
        const float4* rows = reinterpret_cast<const float4*>(static_cast<const char*>(L.bases[L.rank]) + L.out_gx);
        v = __ldcg(rows + (int64_t)owner * L.cap + slot);
    }
    grad_x[3 * i] = v.x;
    grad_x[3 * i + 1] = v.y;
    grad_x[3 * i + 2] = v.z;
}

// ---- owner: backward ----------------------------------------------------------------------------
template <int VEC, bool NEED_GO, bool NEED_GE>
__global__ void __launch_bounds__(256, 3) routed_backward_kernel(RoutedGrid g, RoutedLayout L, float go_scale, int D,
                                                              int lane_shift, int interp) {
    const int region = blockIdx.y;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t j = tid >> lane_shift;
    const int lanes = 1 << lane_shift;
    const int lane = (int)(tid & (lanes - 1));
    const int ch = lane * VEC;
    // whole lane groups stay together for the shuffles below (no early return)
    float4 rec;
    const bool live = routed_record(L, region, j, &rec);
    float go[3] = {0.f, 0.f, 0.f};
    const int gi = live ? __float_as_int(rec.w) : -1;
    if (gi >= 0 && gi < g.n_emb) {
        const float xw[3] = {rec.x, rec.y, rec.z};
        int blk[3], cell[3];
        float off[3];
        split_world_position(xw, g.org, g.inv_cell, g.inv_G, g.G_f, g.G, blk, cell, off);
        int64_t base[8];
        bool mine;
        if (routed_corner_rows(g, gi, cell, D, base, &mine, L.rank) && ch < D) {
            AxisWeights<float> aw;
            aw.init(interp, off);
            const float* zin = reinterpret_cast<const float*>(static_cast<const char*>(L.bases[L.rank]) + L.inbox_z);
            using V = typename Vec<float, VEC>::type;
            Pack<float, VEC> zv;
            *reinterpret_cast<V*>(zv.v) = __ldcg(reinterpret_cast<const V*>(zin + ((int64_t)region * L.cap + j) * D + ch));
            Pack<float, VEC> e[8];
            if (NEED_GO) {
#pragma unroll
                for (int c = 0; c < 8; ++c) e[c] = routed_corner<VEC>(g, base[c], ch, mine);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float w = aw.weight(c);
                Pack<float, VEC> gr;
                float dot = 0.f;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    gr.v[k] = w * zv.v[k];
                    if (NEED_GO) dot += e[c].v[k] * zv.v[k];
                }
                if (NEED_GE) atomic_add_pack<float, VEC>(routed_out_row(g, base[c]) + ch, gr);
                if (NEED_GO) {
                    float wg[3];
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
        float4* out = reinterpret_cast<float4*>(static_cast<char*>(L.bases[region]) + L.out_gx);
        out[(int64_t)L.rank * L.cap + j] = make_float4(go[0] * go_scale, go[1] * go_scale, go[2] * go_scale, 0.f);
    }
}

// ---- double backward ------------------------------------------------------------------------------
// asker: the gradient arriving at dL/dx of every query, into the owner's inbox_g at the query's slot
__global__ void __launch_bounds__(256) routed_send_g_kernel(RoutedLayout L, const int32_t* __restrict__ where, int64_t n,
                                                            const float* __restrict__ ggx) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int w = where[i];
    if (w < 0) return;
    const int owner = (int)((unsigned)w >> kRowOwnerShift);
    const int64_t slot = (unsigned)w & kRowLocalMask;
    float4* inbox = reinterpret_cast<float4*>(static_cast<char*>(L.bases[owner]) + L.inbox_g);
    inbox[(int64_t)L.rank * L.cap + slot] = make_float4(ggx[3 * i], ggx[3 * i + 1], ggx[3 * i + 2], 0.f);
}

// owner: semantics of query_backward_backward_kernel for every record; the gradient with respect to
// dL/dy goes back through the asker's result buffer (out_y), the second-order gradient rows into the shards
template <int VEC>
__global__ void __launch_bounds__(256, 3) routed_backward_backward_kernel(RoutedGrid g, RoutedLayout L, float go_scale,
                                                                       int D, int lane_shift, int interp) {
    const int region = blockIdx.y;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t j = tid >> lane_shift;
    const int lane = (int)(tid & ((1 << lane_shift) - 1));
    const int ch = lane * VEC;
    float4 rec;
    if (ch >= D || !routed_record(L, region, j, &rec)) return;
    Pack<float, VEC> gz;
#pragma unroll
    for (int k = 0; k < VEC; ++k) gz.v[k] = 0;
    const int gi = __float_as_int(rec.w);
    if (gi >= 0 && gi < g.n_emb) {
        const float xw[3] = {rec.x, rec.y, rec.z};
        int blk[3], cell[3];
        float off[3];
        split_world_position(xw, g.org, g.inv_cell, g.inv_G, g.G_f, g.G, blk, cell, off);
        int64_t base[8];
        bool mine;
        if (routed_corner_rows(g, gi, cell, D, base, &mine, L.rank)) {
            AxisWeights<float> aw;
            aw.init(interp, off);
            const char* box = static_cast<const char*>(L.bases[L.rank]);
            const int64_t r = (int64_t)region * L.cap + j;
            const float4 gg = __ldcg(reinterpret_cast<const float4*>(box + L.inbox_g) + r);
            const float g3[3] = {gg.x * go_scale, gg.y * go_scale, gg.z * go_scale};
            using V = typename Vec<float, VEC>::type;
            Pack<float, VEC> zv;
            *reinterpret_cast<V*>(zv.v) = __ldcg(reinterpret_cast<const V*>(reinterpret_cast<const float*>(box + L.inbox_z) + r * D + ch));
            Pack<float, VEC> e[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) e[c] = routed_corner<VEC>(g, base[c], ch, mine);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float wg[3];
                aw.grad(c, wg);
                const float dot = wg[0] * g3[0] + wg[1] * g3[1] + wg[2] * g3[2];
                Pack<float, VEC> gr;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    gr.v[k] = dot * zv.v[k];
                    gz.v[k] += dot * e[c].v[k];
                }
                atomic_add_pack<float, VEC>(routed_out_row(g, base[c]) + ch, gr);
            }
        }
    }
    float* out = reinterpret_cast<float*>(static_cast<char*>(L.bases[region]) + L.out_y);
    store_pack<float, VEC>(out + ((int64_t)L.rank * L.cap + j) * D + ch, gz);
}

}  // namespace ashb

using namespace ashb;

namespace {

int check_routed_layout(const RoutedLayout& L, int64_t mailbox_bytes, int64_t D) {
    ASHB_REQUIRE(L.bases != nullptr, "null peer table");
    ASHB_REQUIRE(L.world >= 1 && L.world <= kRoutedMaxWorld && L.rank >= 0 && L.rank < L.world, "bad world / rank");
    ASHB_REQUIRE(L.cap >= 1 && L.cap <= (int64_t)kRowLocalMask, "a region holds 1 to 2^26 - 1 records");
    ASHB_REQUIRE(D >= 1 && D <= 16, "embedding_dim %lld not in 1..16", (long long)D);
    ASHB_REQUIRE((L.inbox_x | L.inbox_z | L.out_y | L.out_gx | L.inbox_g) % 16 == 0 && L.counts % 4 == 0 && L.inbox_x >= 0,
                 "misaligned mailbox sections");
    const int64_t recs = (int64_t)L.world * L.cap;
    const int64_t ends[6][2] = {{L.inbox_x, L.inbox_x + recs * 16}, {L.counts, L.counts + (int64_t)L.world * 4},
                                {L.inbox_z, L.inbox_z + recs * D * 4}, {L.out_y, L.out_y + recs * D * 4},
                                {L.out_gx, L.out_gx + recs * 16}, {L.inbox_g, L.inbox_g + recs * 16}};
    for (int a = 0; a < 6; ++a) {
        ASHB_REQUIRE(ends[a][0] >= 0 && ends[a][1] <= mailbox_bytes, "a mailbox section exceeds the mailbox");
        for (int b = a + 1; b < 6; ++b)
            ASHB_REQUIRE(ends[a][1] <= ends[b][0] || ends[b][1] <= ends[a][0], "mailbox sections overlap");
    }
    return ASHB_OK;
}

int make_routed_grid(ashb_map* m, const int32_t* nb_lut, const uint32_t* row_of, const void* const* emb_bases,
                     void* const* grad_bases, double cell_size, const float* origin, int G, int64_t n_emb,
                     RoutedGrid* out) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim == 3, "the grid query needs a 3-D map");
    ASHB_REQUIRE(G >= 1 && G <= 64 && cell_size > 0.0 && n_emb >= 1, "bad grid_dim, cell_size or table size");
    ASHB_REQUIRE(nb_lut && row_of, "null table");
    RoutedGrid g{};
    g.table = table16_of(m);
    g.nb_lut = nb_lut;
    g.row_of = row_of;
    g.emb_bases = emb_bases;
    g.grad_bases = grad_bases;
    for (int d = 0; d < 3; ++d) g.org[d] = origin ? origin[d] : 0.f;
    g.inv_cell = (float)(1.0 / cell_size);
    g.G = G;
    g.G_f = (float)G;
    g.inv_G = 1.0f / (float)G;
    g.n_emb = n_emb;
    g.cells = (int64_t)G * G * G;
    *out = g;
    return ASHB_OK;
}

struct LaneShape {
    int vec, lane_shift;
};

// Rows of the mailbox start on 16-byte boundaries when D is a multiple of 4 floats.
LaneShape lane_shape(int64_t D, const void* a = nullptr, const void* b = nullptr) {
    int vec = 4;
    const uintptr_t bits = (uintptr_t)a | (uintptr_t)b;
    while (vec > 1 && (D % vec != 0 || (bits & (uintptr_t)(vec * 4 - 1)))) vec >>= 1;
    int shift = 0;
    while ((1 << shift) < D / vec) ++shift;
    return LaneShape{vec, shift};
}

#define ASHB_ROUTED_VEC(shape, ...)     \
    switch ((shape).vec) {              \
        case 4: {                       \
            constexpr int VEC = 4;      \
            __VA_ARGS__;                \
        } break;                        \
        case 2: {                       \
            constexpr int VEC = 2;      \
            __VA_ARGS__;                \
        } break;                        \
        default: {                      \
            constexpr int VEC = 1;      \
            __VA_ARGS__;                \
        }                               \
    }

}  // namespace

extern "C" {

#define ASHB_ROUTED_LAYOUT_ARGS                                                                                  \
    void *const *peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_x_offset, int64_t counts_offset,           \
            int64_t inbox_z_offset, int64_t out_y_offset, int64_t out_gx_offset, int64_t inbox_g_offset,             \
            int64_t region_capacity, int world, int rank
#define ASHB_ROUTED_LAYOUT                                                                                         \
    RoutedLayout {                                                                                                 \
        peer_bases_dev, inbox_x_offset, counts_offset, inbox_z_offset, out_y_offset, out_gx_offset, inbox_g_offset,  \
                region_capacity, world, rank                                                                       \
    }

int ashb_routed_route(ashb_map* m, const float* x, int64_t n, double cell_size, const float* origin, int G,
                      const int32_t* nb_lut, const uint32_t* row_of, int64_t n_emb, int64_t D, ASHB_ROUTED_LAYOUT_ARGS,
                      int32_t* cursor_dev, int32_t* where_dev, uint32_t* status_dev, void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    ASHB_REQUIRE(n >= 0 && cursor_dev && status_dev && (n == 0 || (x && where_dev)), "null buffer or negative count");
    RoutedGrid g;
    if (int rc = make_routed_grid(m, nb_lut, row_of, nullptr, nullptr, cell_size, origin, G, n_emb, &g)) return rc;
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemsetAsync(cursor_dev, 0, (size_t)world * sizeof(int32_t), st));
    if (n > 0) {
        routed_route_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, n, g, L, cursor_dev, where_dev, status_dev);
        ASHB_LAUNCH_CHECK();
    }
    routed_publish_counts_kernel<<<1, kRoutedMaxWorld, 0, st>>>(L, cursor_dev);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_forward(ashb_map* m, int interp, const void* const* emb_bases_dev, double cell_size,
                        const float* origin, int G, const int32_t* nb_lut, const uint32_t* row_of, int64_t n_emb,
                        int64_t D, ASHB_ROUTED_LAYOUT_ARGS, void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    ASHB_REQUIRE(interp == ASHB_LINEAR || interp == ASHB_SMOOTH_STEP, "unknown interpolation code %d", interp);
    ASHB_REQUIRE(emb_bases_dev != nullptr, "null shard table");
    RoutedGrid g;
    if (int rc = make_routed_grid(m, nb_lut, row_of, emb_bases_dev, nullptr, cell_size, origin, G, n_emb, &g)) return rc;
    DeviceGuard guard(m->device);
    const LaneShape sh = lane_shape(D);
    const dim3 grid((unsigned)(((region_capacity << sh.lane_shift) + 255) / 256), (unsigned)world);
    ASHB_ROUTED_VEC(sh, (routed_forward_kernel<VEC><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                                g, L, (int)D, sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_unpack_y(const int32_t* where_dev, int64_t n, float* y, uint8_t* masks, int64_t D,
                         ASHB_ROUTED_LAYOUT_ARGS, void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(n > 0 && where_dev && y, "null buffer or negative count");
    const LaneShape sh = lane_shape(D, y);
    const unsigned grid = (unsigned)(((n << sh.lane_shift) + 255) / 256);
    ASHB_ROUTED_VEC(sh, (routed_unpack_y_kernel<VEC><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                                L, where_dev, n, y, masks, (int)D, sh.lane_shift)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_send_z(const int32_t* where_dev, int64_t n, const float* z, int64_t D, ASHB_ROUTED_LAYOUT_ARGS,
                       void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(n > 0 && where_dev && z, "null buffer or negative count");
    const LaneShape sh = lane_shape(D, z);
    const unsigned grid = (unsigned)((n + 255) / 256);   // one CTA per 256 queries, whatever the lanes per query
    ASHB_ROUTED_VEC(sh, (routed_send_z_kernel<VEC><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                                L, where_dev, n, z, (int)D, sh.lane_shift)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_backward(ashb_map* m, int interp, const void* const* emb_bases_dev, void* const* grad_bases_dev,
                         int need_grad_x, int need_grad_embeddings, double cell_size, const float* origin, int G, const int32_t* nb_lut,
                         const uint32_t* row_of, int64_t n_emb, int64_t D, ASHB_ROUTED_LAYOUT_ARGS, void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    ASHB_REQUIRE(interp == ASHB_LINEAR || interp == ASHB_SMOOTH_STEP, "unknown interpolation code %d", interp);
    ASHB_REQUIRE(emb_bases_dev != nullptr && grad_bases_dev != nullptr, "null shard table");
    RoutedGrid g;
    if (int rc = make_routed_grid(m, nb_lut, row_of, emb_bases_dev, grad_bases_dev, cell_size, origin, G, n_emb, &g))
        return rc;
    DeviceGuard guard(m->device);
    const LaneShape sh = lane_shape(D);
    const dim3 grid((unsigned)(((region_capacity << sh.lane_shift) + 255) / 256), (unsigned)world);
    const float scale = (float)(1.0 / cell_size);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_REQUIRE(need_grad_x || need_grad_embeddings, "nothing to compute");
    ASHB_ROUTED_VEC(sh, if (need_grad_x && need_grad_embeddings) {
        routed_backward_kernel<VEC, true, true><<<grid, 256, 0, st>>>(g, L, scale, (int)D, sh.lane_shift, interp);
    } else if (need_grad_x) {
        routed_backward_kernel<VEC, true, false><<<grid, 256, 0, st>>>(g, L, scale, (int)D, sh.lane_shift, interp);
    } else { routed_backward_kernel<VEC, false, true><<<grid, 256, 0, st>>>(g, L, scale, (int)D, sh.lane_shift, interp); });
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_unpack_grad_x(const int32_t* where_dev, int64_t n, float* grad_x, int64_t D, ASHB_ROUTED_LAYOUT_ARGS,
                              void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(n > 0 && where_dev && grad_x, "null buffer or negative count");
    routed_unpack_gx_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(L, where_dev, n,
                                                                                                        grad_x);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_send_g(const int32_t* where_dev, int64_t n, const float* grad_grad_x, int64_t D, ASHB_ROUTED_LAYOUT_ARGS,
                       void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(n > 0 && where_dev && grad_grad_x, "null buffer or negative count");
    routed_send_g_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(L, where_dev, n,
                                                                                                     grad_grad_x);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_routed_backward_backward(ashb_map* m, int interp, const void* const* emb_bases_dev, void* const* grad_bases_dev,
                                  double cell_size, const float* origin, int G, const int32_t* nb_lut,
                                  const uint32_t* row_of, int64_t n_emb, int64_t D, ASHB_ROUTED_LAYOUT_ARGS,
                                  void* stream) {
    const RoutedLayout L = ASHB_ROUTED_LAYOUT;
    if (int rc = check_routed_layout(L, mailbox_bytes, D)) return rc;
    ASHB_REQUIRE(interp == ASHB_LINEAR || interp == ASHB_SMOOTH_STEP, "unknown interpolation code %d", interp);
    ASHB_REQUIRE(emb_bases_dev != nullptr && grad_bases_dev != nullptr, "null shard table");
    RoutedGrid g;
    if (int rc = make_routed_grid(m, nb_lut, row_of, emb_bases_dev, grad_bases_dev, cell_size, origin, G, n_emb, &g))
        return rc;
    DeviceGuard guard(m->device);
    const LaneShape sh = lane_shape(D);
    const dim3 grid((unsigned)(((region_capacity << sh.lane_shift) + 255) / 256), (unsigned)world);
    const float scale = (float)(1.0 / cell_size);
    ASHB_ROUTED_VEC(sh, (routed_backward_backward_kernel<VEC><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                                g, L, scale, (int)D, sh.lane_shift, interp)));
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
