// Fused RGB-D TSDF integration for sm_100a: block allocation from a depth frame
// and the running weighted average of sdf / colour / weight per cell.
//
// It replaces the ~40 torch launches per frame of TSDFFusion.fuse_frame
// (demo/rgbd_fusion.py:199-254) and project_points_to_rgbd (:76-110), the temporary
// hash set of SparseDenseGrid.spatial_init_ (ash/grid.py:121-159) and the
// third-party depth unprojection (demo/rgbd_fusion.py:57-74) with two launches and
// no host synchronisation:
//
//   touch     one thread per depth pixel: unproject with the pinhole model, take the
//             block of the point, and for every block of the (2*dilation+1)^3
//             neighbourhood insert-if-absent into the grid's hash table, record the
//             block coordinate and stamp the block as touched by this frame.  A warp
//             first elects one lane per distinct block among its 32 pixels, so the
//             27 probes are issued once per block, not once per pixel.
//   integrate one CTA per embedding row; CTAs of untouched rows exit at once.  The
//             10 KB of a block (512 cells x 5 floats) is staged in shared memory with
//             coalesced 16-byte accesses, every cell is projected into the frame and
//             fused, and the block is written back the same way.
#include <mutex>

#include "hashmap.cuh"

// Scratch of ashb_tsdf_fuse_frame_static: per block one stamp word and one int32x3
// coordinate.  It lives in the library image, so no allocation is ever made for it; every
// GPU that loads the library holds these bytes until the process exits.
#define ASHB_TSDF_STATIC_MAX_BLOCKS 262144
static __device__ __align__(256) unsigned char g_tsdf_static_scratch[ASHB_TSDF_STATIC_MAX_BLOCKS * 16];

namespace ashb {

struct Camera {
    float K[9];    // intrinsic, row major
    float E[12];   // world -> camera, rows of [R | t]
    float Ei[12];  // camera -> world, rows of [R' | c]
};

// Every product and sum below is individually rounded (no fused multiply-add), so the
// block a point falls in and the pixel a cell projects to are bit-reproducible.
__device__ __forceinline__ float affine3(const float* r, float x, float y, float z) {
    return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(r[0], x), __fmul_rn(r[1], y)), __fmul_rn(r[2], z)), r[3]);
}
__device__ __forceinline__ float dot3(const float* r, float x, float y, float z) {
    return __fadd_rn(__fadd_rn(__fmul_rn(r[0], x), __fmul_rn(r[1], y)), __fmul_rn(r[2], z));
}

// ---- touch -------------------------------------------------------------------------
struct TouchTarget {
    int32_t* heap;
    int32_t* counter;
    int32_t capacity;
    int lo_off, hi_off;  // neighbourhood offsets per axis: [-dilation, dilation] or [0, dilation]
    int3 lo, hi;         // admissible block coordinates (half open) when bounded
    int bounded;
    int32_t* grid_coords;
    uint32_t* touched;
    uint32_t stamp;
    int32_t* touched_list;
    int32_t* touched_count;
};

// Insert-if-absent of block (kx, ky, kz), its coordinate recorded and its stamp set; appended to the
// compact list by the first toucher of the call.
__device__ __forceinline__ void touch_block(const Table16& t, const TouchTarget& tt, int kx, int ky, int kz) {
    if (tt.bounded && (kx < tt.lo.x || ky < tt.lo.y || kz < tt.lo.z || kx >= tt.hi.x || ky >= tt.hi.y || kz >= tt.hi.z))
        return;
    // fast path: the block exists already (probe at L2: this launch mutates the table)
    int idx = -1;
    {
        uint32_t s = hash_key(kx, ky, kz, 0) & t.mask;
        for (uint32_t probe = 0; probe <= t.mask; ++probe) {
            const Entry e = t.read_fresh(s);
            if (e.val == kEmpty) break;
            if (e.val >= 0 && key_match(e, kx, ky, kz, 0)) {
                idx = e.val;
                break;
            }
            s = (s + 1) & t.mask;
        }
    }
    if (idx < 0) {
        bool present = false;
        const int64_t slot = emplace(t, kx, ky, kz, 0, kPending, &present);
        if (slot < 0) return;  // another thread of this launch owns it and stamps it
        const int top = atomicAdd(tt.counter, 1);
        if (top >= tt.capacity) {
            atomicSub(tt.counter, 1);
            *reinterpret_cast<volatile int*>(t.val_ptr((uint32_t)slot)) = kTomb;
            atomicOr(t.status, ASHB_STATUS_CAPACITY);
            return;
        }
        idx = tt.heap[top];
        *reinterpret_cast<volatile int*>(t.val_ptr((uint32_t)slot)) = idx;
    }
    // many pixels of a frame fall in the same few thousand blocks: whoever finds the block already
    // stamped by this call has nothing left to do (the first toucher recorded it)
    if (__ldcg(&tt.touched[idx]) == tt.stamp) return;
    // the coordinate is recorded for blocks allocated by other means too
    tt.grid_coords[3 * idx] = kx;
    tt.grid_coords[3 * idx + 1] = ky;
    tt.grid_coords[3 * idx + 2] = kz;
    if (tt.touched_list) {
        // first toucher of the call appends the block to the compact work list
        if (atomicExch(&tt.touched[idx], tt.stamp) != tt.stamp) tt.touched_list[atomicAdd(tt.touched_count, 1)] = idx;
    } else {
        tt.touched[idx] = tt.stamp;
    }
}

// Called by EVERY lane of a warp (`valid` lanes carry a block).  The distinct blocks of the warp are
// found with a match; then, one distinct block after the other, the lanes of the whole warp share
// out its neighbourhood -- lane k takes neighbour k -- so the (2 dilation + 1)^3 probes / inserts
// of a block run side by side instead of one after the other on a single lane.
__device__ __forceinline__ void touch_neighbourhood(const Table16& t, const TouchTarget& tt, bool valid, int bx,
                                                    int by, int bz) {
    const int lane = threadIdx.x & 31;
    // a point whose own block is out of bounds contributes nothing (ash/grid.py:134-135)
    if (valid && tt.bounded &&
        (bx < tt.lo.x || by < tt.lo.y || bz < tt.lo.z || bx >= tt.hi.x || by >= tt.hi.y || bz >= tt.hi.z))
        valid = false;
    const unsigned active = __ballot_sync(0xffffffffu, valid);
    bool lead = false;
    if (valid) {
        const unsigned long long packed = ((unsigned long long)(unsigned)bx * 0x9E3779B97F4A7C15ull) ^
                                          ((unsigned long long)(unsigned)by << 21) ^
                                          ((unsigned long long)(unsigned)bz << 42) ^ (unsigned)bz;
        const unsigned peers = __match_any_sync(active, packed);
        const int leader = __ffs(peers) - 1;
        const int lbx = __shfl_sync(peers, bx, leader), lby = __shfl_sync(peers, by, leader),
                  lbz = __shfl_sync(peers, bz, leader);
        // `packed` is not injective; lanes that collide without being equal lead their own block
        lead = lane == leader || lbx != bx || lby != by || lbz != bz;
    }
    unsigned leaders = __ballot_sync(0xffffffffu, lead);
    const int w = tt.hi_off - tt.lo_off + 1, n_nb = w * w * w;
    while (leaders) {
        const int from = __ffs(leaders) - 1;
        leaders &= leaders - 1;
        const int cx = __shfl_sync(0xffffffffu, bx, from), cy = __shfl_sync(0xffffffffu, by, from),
                  cz = __shfl_sync(0xffffffffu, bz, from);
        for (int k = lane; k < n_nb; k += 32)
            touch_block(t, tt, cx + tt.lo_off + k % w, cy + tt.lo_off + (k / w) % w, cz + tt.lo_off + k / (w * w));
        __syncwarp();
    }
}

// world -> cell -> block as the Python layer does on a CUDA tensor: multiply by the float
// reciprocals (ash/grid.py:132-134, :756, :846)
__device__ __forceinline__ int block_of(float w, float org, float inv_cell, float inv_G) {
    return (int)floorf(__fmul_rn(__fmul_rn(__fsub_rn(w, org), inv_cell), inv_G));
}

__global__ void __launch_bounds__(256, 8) tsdf_touch_kernel(Table16 t, TouchTarget tt, const float* __restrict__ depth,
                                                         int H, int W, Camera cam, float depth_max, float inv_cell,
                                                         float3 origin, float inv_G) {
    const int64_t pix = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool valid = pix < (int64_t)H * W;
    int bx = 0, by = 0, bz = 0;
    if (valid) {
        const float d = depth[pix];
        valid = d > 0.f && d < depth_max;
        if (valid) {
            const int v = (int)(pix / W), u = (int)(pix - (int64_t)v * W);
            // camera point of pixel (u, v) at depth d for K = [fx 0 cx; 0 fy cy; 0 0 1]
            const float xc = __fdiv_rn(__fmul_rn(__fsub_rn((float)u, cam.K[2]), d), cam.K[0]);
            const float yc = __fdiv_rn(__fmul_rn(__fsub_rn((float)v, cam.K[5]), d), cam.K[4]);
            bx = block_of(affine3(cam.Ei, xc, yc, d), origin.x, inv_cell, inv_G);
            by = block_of(affine3(cam.Ei + 4, xc, yc, d), origin.y, inv_cell, inv_G);
            bz = block_of(affine3(cam.Ei + 8, xc, yc, d), origin.z, inv_cell, inv_G);
        }
    }
    touch_neighbourhood(t, tt, valid, bx, by, bz);
}

// SparseDenseGrid.spatial_init_ (ash/grid.py:121-159) without its temporary hash set: one
// thread per point.
__global__ void __launch_bounds__(256) points_touch_kernel(Table16 t, TouchTarget tt, const float* __restrict__ pts,
                                                           int64_t n, float inv_cell, float3 origin, float inv_G) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = i < n;
    int bx = 0, by = 0, bz = 0;
    if (valid) {
        bx = block_of(pts[3 * i], origin.x, inv_cell, inv_G);
        by = block_of(pts[3 * i + 1], origin.y, inv_cell, inv_G);
        bz = block_of(pts[3 * i + 2], origin.z, inv_cell, inv_G);
    }
    touch_neighbourhood(t, tt, valid, bx, by, bz);
}

// ---- integrate ---------------------------------------------------------------------
struct IntegrateFrame {
    const float* __restrict__ depth;
    const float* __restrict__ color;
    int H, W;
    Camera cam;
    float depth_max, cell_size;
    float3 origin;
    int G, cells;
    float trunc;
    int sdf_ch, rgb_ch, w_ch;
};

// One observation fused into every cell of block (gx, gy, gz), whose rows sit in `tile` (cells * D floats).
template <int D>
__device__ __forceinline__ void integrate_cells(float* tile, int gx, int gy, int gz, const IntegrateFrame& f) {
    const int G = f.G;
    for (int c = threadIdx.x; c < f.cells; c += blockDim.x) {
        const int cx = c % G, cy = (c / G) % G, cz = c / (G * G);
        // cell_to_world: (block * G + cell) * cell_size (+ origin for bounded grids)
        const float px = __fadd_rn(__fmul_rn((float)(gx * G + cx), f.cell_size), f.origin.x);
        const float py = __fadd_rn(__fmul_rn((float)(gy * G + cy), f.cell_size), f.origin.y);
        const float pz = __fadd_rn(__fmul_rn((float)(gz * G + cz), f.cell_size), f.origin.z);
        const float x = affine3(f.cam.E, px, py, pz);
        const float y = affine3(f.cam.E + 4, px, py, pz);
        const float z = affine3(f.cam.E + 8, px, py, pz);
        const float un = dot3(f.cam.K, x, y, z);
        const float vn = dot3(f.cam.K + 3, x, y, z);
        const float d = dot3(f.cam.K + 6, x, y, z);
        float w = 0.f, sdf = 0.f, r = 0.f, g = 0.f, b = 0.f;
        if (d > 0.f) {
            const float uf = rintf(__fdiv_rn(un, d)), vf = rintf(__fdiv_rn(vn, d));  // torch.round: half to even
            if (uf >= 0.f && vf >= 0.f && uf < (float)f.W && vf < (float)f.H) {
                const int u = (int)uf, v = (int)vf;
                const float dr = __ldg(f.depth + (int64_t)v * f.W + u);
                const float* col = f.color + ((int64_t)v * f.W + u) * 3;
                r = __ldg(col), g = __ldg(col + 1), b = __ldg(col + 2);
                sdf = __fsub_rn(dr, d);
                if (dr > 0.f && dr < f.depth_max && sdf >= -f.trunc) w = 1.f;
                if (sdf >= f.trunc) sdf = f.trunc;
            }
        }
        // outside the image or behind the camera the observation has weight 0 and its
        // value does not matter (demo/rgbd_fusion.py:93-108)
        float* cell = tile + c * D;
        const float w_sum = cell[f.w_ch];
        // demo/rgbd_fusion.py:247-249: mean' = (mean * w_sum + obs * w) / (w_sum + w + 1e-6)
        const float w_new = __fadd_rn(w_sum, w);
        const float den = __fadd_rn(w_new, 1e-6f);
        auto fuse = [&](float mean, float obs) {
            return __fdiv_rn(__fadd_rn(__fmul_rn(mean, w_sum), __fmul_rn(obs, w)), den);
        };
        cell[f.sdf_ch] = fuse(cell[f.sdf_ch], sdf);
        cell[f.rgb_ch] = fuse(cell[f.rgb_ch], r);
        cell[f.rgb_ch + 1] = fuse(cell[f.rgb_ch + 1], g);
        cell[f.rgb_ch + 2] = fuse(cell[f.rgb_ch + 2], b);
        cell[f.w_ch] = w_new;
    }
}

template <int D>
__global__ void __launch_bounds__(256, 8) tsdf_integrate_kernel(
        float* __restrict__ emb, const int32_t* __restrict__ grid_coords, const uint32_t* __restrict__ touched,
        uint32_t stamp, IntegrateFrame f, unsigned long long* n_integrated, int64_t n_emb,
        const int32_t* __restrict__ touched_list, const int32_t* __restrict__ touched_count) {
    extern __shared__ float tile[];  // cells * D floats
    // Work items: the compact list written by the touch kernel (a few persistent CTAs walk it),
    // or, without a list, every embedding row whose stamp matches (one CTA per row).
    const int64_t n_items = touched_list ? (int64_t)*touched_count : n_emb;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int64_t idx = touched_list ? (int64_t)touched_list[item] : item;
        if (!touched_list && touched[idx] != stamp) continue;
        float* block = emb + idx * (int64_t)f.cells * D;
        const int n_float = f.cells * D;
        // rows are 16-byte aligned when cells * D * 4 is a multiple of 16
        const bool vec_ok = (n_float & 3) == 0 && (((uintptr_t)block) & 15) == 0;
        if (vec_ok) {
            for (int i = threadIdx.x; i < n_float / 4; i += blockDim.x)
                reinterpret_cast<float4*>(tile)[i] = reinterpret_cast<const float4*>(block)[i];
        } else {
            for (int i = threadIdx.x; i < n_float; i += blockDim.x) tile[i] = block[i];
        }
        __syncthreads();
        integrate_cells<D>(tile, grid_coords[3 * idx], grid_coords[3 * idx + 1], grid_coords[3 * idx + 2], f);
        __syncthreads();
        if (vec_ok) {
            for (int i = threadIdx.x; i < n_float / 4; i += blockDim.x)
                reinterpret_cast<float4*>(block)[i] = reinterpret_cast<const float4*>(tile)[i];
        } else {
            for (int i = threadIdx.x; i < n_float; i += blockDim.x) block[i] = tile[i];
        }
        if (threadIdx.x == 0 && n_integrated) atomicAdd(n_integrated, 1ull);
        __syncthreads();  // the tile is reused by the next item
    }
}

// Number of waits of the bulk-copy variant below that ran out (0 in any healthy run): read with
// ashb_tsdf_copy_timeouts.
__device__ unsigned int g_tsdf_copy_timeouts = 0;

__device__ __forceinline__ uint32_t smem_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Waits, with a limit, for phase `parity` of the mbarrier at `bar`; false when the limit ran out.
__device__ __forceinline__ bool wait_phase(uint32_t bar, uint32_t parity) {
    for (int spin = 0; spin < (1 << 18); ++spin) {
        uint32_t done;
        asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(bar), "r"(parity)
                : "memory");
        if (done) return true;
    }
    return false;
}

// The same pass over a work list with the block rows moved by the copy engine: a persistent CTA keeps
// two tiles in shared memory; while it fuses the observation into one, the next block's rows arrive in
// the other (cp.async.bulk global -> shared, completion on an mbarrier) and the finished tile leaves
// as one bulk store (shared -> global), so loading, arithmetic and storing overlap instead of taking
// turns.  A block's rows are one contiguous, 16-byte aligned stretch of cells * D * 4 bytes (a multiple
// of 16: checked by the host).  Every wait has an iteration limit; a CTA whose wait runs out counts it
// in g_tsdf_copy_timeouts, waits for its own stores and stops.
template <int D>
__global__ void __launch_bounds__(256, 8) tsdf_integrate_bulk_kernel(
        float* __restrict__ emb, const int32_t* __restrict__ grid_coords, IntegrateFrame f,
        unsigned long long* n_integrated, const int32_t* __restrict__ touched_list,
        const int32_t* __restrict__ touched_count) {
    extern __shared__ __align__(128) float tiles[];  // 2 tiles of cells * D floats
    __shared__ __align__(8) unsigned long long full[2];
    const int n_float = f.cells * D;
    const uint32_t bytes = (uint32_t)n_float * 4u;
    const int64_t n_items = (int64_t)*touched_count;
    const bool boss = threadIdx.x == 0;
    if (boss) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&full[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&full[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto fetch = [&](int64_t item, int buf) {   // thread 0 only
        const float* src = emb + (int64_t)touched_list[item] * n_float;
        const uint32_t bar = smem_address(&full[buf]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_address(tiles + (int64_t)buf * n_float)),
                     "l"(src), "r"(bytes), "r"(bar)
                     : "memory");
    };
    if (boss && (int64_t)blockIdx.x < n_items) fetch(blockIdx.x, 0);
    int round = 0;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x, ++round) {
        const int buf = round & 1;
        const int64_t next = item + gridDim.x;
        if (boss && next < n_items) {
            // the other tile was handed to a bulk store one round ago: it may be refilled once that store has read it
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            fetch(next, buf ^ 1);
        }
        const bool arrived = wait_phase(smem_address(&full[buf]), (uint32_t)(round >> 1) & 1u);
        if (!__syncthreads_and(arrived)) {
            if (boss) {
                atomicAdd(&g_tsdf_copy_timeouts, 1u);
                // the copy already requested for the next round must not land in a dead CTA's memory
                if (next < n_items) wait_phase(smem_address(&full[buf ^ 1]), (uint32_t)((round + 1) >> 1) & 1u);
            }
            break;
        }
        float* tile = tiles + (int64_t)buf * n_float;
        const int64_t idx = touched_list[item];
        integrate_cells<D>(tile, grid_coords[3 * idx], grid_coords[3 * idx + 1], grid_coords[3 * idx + 2], f);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tile as written, visible to the copy engine
        __syncthreads();
        if (boss) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(emb + idx * (int64_t)n_float),
                         "r"(smem_address(tile)), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            if (n_integrated) atomicAdd(n_integrated, 1ull);
        }
    }
    if (boss) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores complete before the CTA's memory goes
}

}  // namespace ashb

using namespace ashb;

extern "C" {

static int make_touch_target(ashb_map* m, int dilation, int bidirectional, const int32_t* bound_lo,
                             const int32_t* bound_hi, int32_t* grid_coords, uint32_t* touched, uint32_t stamp,
                             int32_t* touched_list, int32_t* touched_count, TouchTarget* out) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim == 3, "block allocation needs a 3-D map");
    ASHB_REQUIRE(grid_coords && touched, "null buffer");
    ASHB_REQUIRE(dilation >= 0 && dilation <= 4, "dilation %d not in 0..4", dilation);
    ASHB_REQUIRE(stamp != 0, "stamp 0 is reserved for 'never touched'");
    ASHB_REQUIRE((touched_list == nullptr) == (touched_count == nullptr),
                 "pass both the list and its counter, or neither");
    TouchTarget tt{};
    tt.heap = m->heap;
    tt.counter = m->counter;
    tt.capacity = (int32_t)m->capacity;
    tt.lo_off = bidirectional ? -dilation : 0;
    tt.hi_off = dilation;
    tt.bounded = bound_lo != nullptr && bound_hi != nullptr;
    if (tt.bounded) {
        tt.lo = make_int3(bound_lo[0], bound_lo[1], bound_lo[2]);
        tt.hi = make_int3(bound_hi[0], bound_hi[1], bound_hi[2]);
    }
    tt.grid_coords = grid_coords;
    tt.touched = touched;
    tt.stamp = stamp;
    tt.touched_list = touched_list;
    tt.touched_count = touched_count;
    *out = tt;
    return ASHB_OK;
}

int ashb_tsdf_touch(ashb_map* m, const float* depth, int H, int W, const float* intrinsic,
                    const float* cam_to_world, float depth_max, double cell_size, const float* origin, int G,
                    int dilation, const int32_t* bound_lo, const int32_t* bound_hi, int32_t* grid_coords,
                    uint32_t* touched, uint32_t stamp, int32_t* touched_list, int32_t* touched_count,
                    void* stream) {
    TouchTarget tt;
    if (int rc = make_touch_target(m, dilation, 1, bound_lo, bound_hi, grid_coords, touched, stamp, touched_list,
                                   touched_count, &tt))
        return rc;
    ASHB_REQUIRE(depth && intrinsic && cam_to_world && origin, "null buffer");
    ASHB_REQUIRE(H > 0 && W > 0 && G > 0 && cell_size > 0.0, "bad frame or grid geometry");
    DeviceGuard guard(m->device);
    Camera cam{};
    for (int i = 0; i < 9; ++i) cam.K[i] = intrinsic[i];
    for (int i = 0; i < 12; ++i) cam.Ei[i] = cam_to_world[i];
    ASHB_REQUIRE(cam.K[0] != 0.f && cam.K[4] != 0.f && cam.K[1] == 0.f && cam.K[3] == 0.f,
                 "intrinsic must be a skew-free pinhole matrix");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n = (int64_t)H * W;
    if (touched_count) ASHB_CUDA_TRY(cudaMemsetAsync(touched_count, 0, sizeof(int32_t), st));
    tsdf_touch_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
            table16_of(m), tt, depth, H, W, cam, depth_max, (float)(1.0 / cell_size),
            make_float3(origin[0], origin[1], origin[2]), 1.0f / (float)G);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_grid_spatial_init(ashb_map* m, const float* points, int64_t n, double cell_size, const float* origin, int G,
                           int dilation, int bidirectional, const int32_t* bound_lo, const int32_t* bound_hi,
                           int32_t* grid_coords, uint32_t* touched, uint32_t stamp, int32_t* touched_list,
                           int32_t* touched_count, void* stream) {
    TouchTarget tt;
    if (int rc = make_touch_target(m, dilation, bidirectional, bound_lo, bound_hi, grid_coords, touched, stamp,
                                   touched_list, touched_count, &tt))
        return rc;
    ASHB_REQUIRE(n >= 0 && G > 0 && cell_size > 0.0, "bad point count or grid geometry");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (touched_count) ASHB_CUDA_TRY(cudaMemsetAsync(touched_count, 0, sizeof(int32_t), st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(points != nullptr, "null points");
    const float3 org = origin ? make_float3(origin[0], origin[1], origin[2]) : make_float3(0.f, 0.f, 0.f);
    points_touch_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(table16_of(m), tt, points, n, (float)(1.0 / cell_size),
                                                                      org, 1.0f / (float)G);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_tsdf_integrate(void* embeddings, int64_t n_emb, int G, int64_t D, const int32_t* grid_coords,
                        const uint32_t* touched, uint32_t stamp, const float* depth, const float* color, int H,
                        int W, const float* intrinsic, const float* world_to_cam, float depth_max,
                        double cell_size, const float* origin, float trunc, int sdf_channel, int rgb_channel,
                        int weight_channel, unsigned long long* n_integrated_dev, const int32_t* touched_list,
                        const int32_t* touched_count, void* stream) {
    ASHB_REQUIRE((touched_list == nullptr) == (touched_count == nullptr), "pass both the list and its counter, or neither");
    ASHB_REQUIRE(embeddings && grid_coords && touched && depth && color && intrinsic && world_to_cam && origin,
                 "null buffer");
    ASHB_REQUIRE(n_emb >= 1 && G >= 1 && G <= 16 && H > 0 && W > 0, "bad sizes");
    ASHB_REQUIRE(D >= 5 && D <= 16, "embedding_dim %lld cannot hold sdf + rgb + weight", (long long)D);
    ASHB_REQUIRE(sdf_channel >= 0 && sdf_channel < D && weight_channel >= 0 && weight_channel < D &&
                         rgb_channel >= 0 && rgb_channel + 2 < D,
                 "channel layout out of range");
    Camera cam{};
    for (int i = 0; i < 9; ++i) cam.K[i] = intrinsic[i];
    for (int i = 0; i < 12; ++i) cam.E[i] = world_to_cam[i];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int cells = G * G * G;
    const size_t smem = (size_t)cells * D * sizeof(float);
    ASHB_REQUIRE(smem <= 200 * 1024, "block of %zu bytes does not fit in shared memory", smem);
    const IntegrateFrame frame{depth, color, H, W, cam, depth_max, (float)cell_size,
                               make_float3(origin[0], origin[1], origin[2]), G, cells, trunc, sdf_channel, rgb_channel,
                               weight_channel};
    // The copy-engine variant needs a work list, 16-byte aligned rows of a multiple of 16 bytes, and room
    // for two tiles per CTA; everything else takes the plain kernel.
    const bool bulk = touched_list != nullptr && smem % 16 == 0 && ((uintptr_t)embeddings & 15) == 0 && 2 * smem <= 96 * 1024;
    // with a work list: exactly the CTAs that are resident at once walk it (more would queue behind them
    // as a partly filled second wave); without: one CTA per row
    // The pass is bound by arithmetic (seven IEEE divisions per cell), which half of an SM's thread slots
    // already saturate; the other half is left to the allocation pass of the NEXT frame, which runs
    // beside it on a second stream when a sequence is fused (ashb_tsdf_fuse_frames).
    constexpr int kIntegrateCtasPerSm = 4;
#define ASHB_TSDF_LAUNCH(DD)                                                                               \
    case DD: {                                                                                             \
        const size_t dyn = bulk ? 2 * smem : smem;                                                         \
        const void* fn = bulk ? (const void*)tsdf_integrate_bulk_kernel<DD> : (const void*)tsdf_integrate_kernel<DD>; \
        if (dyn > 48 * 1024)                                                                               \
            ASHB_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn)); \
        int per_sm = 0;                                                                                    \
        ASHB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, 256, dyn));               \
        if (per_sm > kIntegrateCtasPerSm) per_sm = kIntegrateCtasPerSm;                                    \
        const int64_t resident = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                          \
        const unsigned launch_ctas = touched_list ? (unsigned)(n_emb < resident ? n_emb : resident) : (unsigned)n_emb; \
        if (bulk)                                                                                          \
            tsdf_integrate_bulk_kernel<DD><<<launch_ctas, 256, dyn, st>>>(                                 \
                    static_cast<float*>(embeddings), grid_coords, frame, n_integrated_dev, touched_list, touched_count); \
        else                                                                                               \
            tsdf_integrate_kernel<DD><<<launch_ctas, 256, dyn, st>>>(                                      \
                    static_cast<float*>(embeddings), grid_coords, touched, stamp, frame, n_integrated_dev, n_emb, \
                    touched_list, touched_count);                                                          \
    } break;
    switch ((int)D) {
        ASHB_TSDF_LAUNCH(5)
        ASHB_TSDF_LAUNCH(6)
        ASHB_TSDF_LAUNCH(7)
        ASHB_TSDF_LAUNCH(8)
        ASHB_TSDF_LAUNCH(9)
        ASHB_TSDF_LAUNCH(10)
        ASHB_TSDF_LAUNCH(11)
        ASHB_TSDF_LAUNCH(12)
        ASHB_TSDF_LAUNCH(13)
        ASHB_TSDF_LAUNCH(14)
        ASHB_TSDF_LAUNCH(15)
        ASHB_TSDF_LAUNCH(16)
    }
#undef ASHB_TSDF_LAUNCH
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

// Device address of g_tsdf_static_scratch on the current device.  In host code the array's
// name is only a handle; the address the kernels need comes from cudaGetSymbolAddress, looked
// up once per device with that device current.
static int static_scratch_for_current_device(unsigned char** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static unsigned char* cached[kMaxDevices] = {};
    int dev = -1;
    ASHB_CUDA_TRY(cudaGetDevice(&dev));
    ASHB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        ASHB_CUDA_TRY(cudaGetSymbolAddress(&p, g_tsdf_static_scratch));
        ASHB_REQUIRE(p != nullptr, "static scratch has no device address");
        cached[dev] = static_cast<unsigned char*>(p);
    }
    *out = cached[dev];
    return ASHB_OK;
}

int ashb_tsdf_fuse_frame(ashb_map* m, void* embeddings, int64_t n_emb, int G, int64_t D, const float* depth,
                         const float* color, int H, int W, const float* intrinsic, const float* world_to_cam,
                         const float* cam_to_world, float depth_max, double cell_size, const float* origin,
                         int dilation, const int32_t* bound_lo, const int32_t* bound_hi, float trunc, int sdf_channel,
                         int rgb_channel, int weight_channel, int32_t* grid_coords, uint32_t* touched, uint32_t stamp,
                         int32_t* touched_list, int32_t* touched_count, unsigned long long* n_integrated_dev,
                         void* stream) {
    if (int rc = ashb_tsdf_touch(m, depth, H, W, intrinsic, cam_to_world, depth_max, cell_size, origin, G, dilation,
                                 bound_lo, bound_hi, grid_coords, touched, stamp, touched_list, touched_count, stream))
        return rc;
    DeviceGuard guard(m->device);
    return ashb_tsdf_integrate(embeddings, n_emb, G, D, grid_coords, touched, stamp, depth, color, H, W, intrinsic,
                               world_to_cam, depth_max, cell_size, origin, trunc, sdf_channel, rgb_channel,
                               weight_channel, n_integrated_dev, touched_list, touched_count, stream);
}

// Side stream and events of the two-stage frame pipeline below, one set per device, created on first
// use and kept for the life of the process.
struct FramePipeline {
    cudaStream_t side = nullptr;
    cudaEvent_t start = nullptr, touched[2] = {nullptr, nullptr}, integrated[2] = {nullptr, nullptr};
};

static int frame_pipeline_for_current_device(FramePipeline** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static FramePipeline cached[kMaxDevices];
    int dev = -1;
    ASHB_CUDA_TRY(cudaGetDevice(&dev));
    ASHB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    FramePipeline& p = cached[dev];
    if (p.side == nullptr) {
        ASHB_CUDA_TRY(cudaStreamCreateWithFlags(&p.side, cudaStreamNonBlocking));
        ASHB_CUDA_TRY(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        for (int i = 0; i < 2; ++i) {
            ASHB_CUDA_TRY(cudaEventCreateWithFlags(&p.touched[i], cudaEventDisableTiming));
            ASHB_CUDA_TRY(cudaEventCreateWithFlags(&p.integrated[i], cudaEventDisableTiming));
        }
    }
    *out = &p;
    return ASHB_OK;
}

int ashb_tsdf_fuse_frames(ashb_map* m, void* embeddings, int64_t n_emb, int G, int64_t D, int n_frames,
                          const float* const* depths, const float* const* colors, int H, int W,
                          const float* intrinsics, const float* world_to_cams, const float* cam_to_worlds,
                          float depth_max, double cell_size, const float* origin, int dilation, const int32_t* bound_lo,
                          const int32_t* bound_hi, float trunc, int sdf_channel, int rgb_channel, int weight_channel,
                          int32_t* grid_coords, uint32_t* touched, uint32_t first_stamp, int32_t* touched_list,
                          int32_t* touched_count, int double_buffered, unsigned long long* n_integrated_dev,
                          void* stream) {
    ASHB_REQUIRE(n_frames >= 0 && (n_frames == 0 || (depths && colors && intrinsics && world_to_cams && cam_to_worlds)),
                 "null frame tables");
    ASHB_REQUIRE((uint64_t)first_stamp + (uint64_t)n_frames <= 0x7FFFFFFFull && first_stamp != 0, "stamps would wrap");
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    if (!double_buffered || touched_list == nullptr || touched_count == nullptr || n_frames < 2) {
        for (int f = 0; f < n_frames; ++f) {
            if (int rc = ashb_tsdf_fuse_frame(m, embeddings, n_emb, G, D, depths[f], colors[f], H, W, intrinsics + 9 * f,
                                              world_to_cams + 12 * f, cam_to_worlds + 12 * f, depth_max, cell_size,
                                              origin, dilation, bound_lo, bound_hi, trunc, sdf_channel, rgb_channel,
                                              weight_channel, grid_coords, touched, first_stamp + (uint32_t)f,
                                              touched_list, touched_count, n_integrated_dev, stream))
                return rc;
        }
        return ASHB_OK;
    }
    // Two-stage pipeline: the allocation pass of frame f + 1 (side stream) runs while frame f is fused
    // (caller's stream).  The allocation pass writes the hash table, the free-index stack, the stamps and
    // ITS work list (lists and counts alternate between two buffers); the fusion pass of the frame before
    // reads its own list, the coordinates of blocks that already exist (re-written with the same values at
    // most) and embedding rows no allocation touches -- so the two only meet through the events below.
    DeviceGuard guard(m->device);
    FramePipeline* p = nullptr;
    if (int rc = frame_pipeline_for_current_device(&p)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaEventRecord(p->start, st));
    ASHB_CUDA_TRY(cudaStreamWaitEvent(p->side, p->start, 0));   // after whatever the caller enqueued before
    for (int f = 0; f < n_frames; ++f) {
        const int b = f & 1;
        if (f >= 2) ASHB_CUDA_TRY(cudaStreamWaitEvent(p->side, p->integrated[b], 0));   // list b is free again
        if (int rc = ashb_tsdf_touch(m, depths[f], H, W, intrinsics + 9 * f, cam_to_worlds + 12 * f, depth_max, cell_size,
                                     origin, G, dilation, bound_lo, bound_hi, grid_coords, touched,
                                     first_stamp + (uint32_t)f, touched_list + (int64_t)b * n_emb, touched_count + b,
                                     p->side))
            return rc;
        ASHB_CUDA_TRY(cudaEventRecord(p->touched[b], p->side));
        ASHB_CUDA_TRY(cudaStreamWaitEvent(st, p->touched[b], 0));
        if (int rc = ashb_tsdf_integrate(embeddings, n_emb, G, D, grid_coords, touched, first_stamp + (uint32_t)f,
                                         depths[f], colors[f], H, W, intrinsics + 9 * f, world_to_cams + 12 * f,
                                         depth_max, cell_size, origin, trunc, sdf_channel, rgb_channel, weight_channel,
                                         n_integrated_dev, touched_list + (int64_t)b * n_emb, touched_count + b, st))
            return rc;
        ASHB_CUDA_TRY(cudaEventRecord(p->integrated[b], st));
    }
    return ASHB_OK;   // the caller's stream has waited for every allocation pass: it is ordered after all the work
}

int ashb_tsdf_static_max_blocks(void) { return ASHB_TSDF_STATIC_MAX_BLOCKS; }

int ashb_tsdf_copy_timeouts(unsigned int* out) {
    ASHB_REQUIRE(out != nullptr, "out is null");
    ASHB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_tsdf_copy_timeouts, sizeof(unsigned int)));
    return ASHB_OK;
}

int ashb_tsdf_fuse_frame_static(ashb_map* m, void* embeddings, int64_t n_emb, int G, int64_t D,
                                const float* depth, const float* color, int H, int W, const float* intrinsic,
                                const float* world_to_cam, const float* cam_to_world, float depth_max,
                                double cell_size, const float* origin, int dilation, const int32_t* bound_lo,
                                const int32_t* bound_hi, float trunc, int sdf_channel, int rgb_channel,
                                int weight_channel, void* stream) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(n_emb >= 1 && n_emb <= ASHB_TSDF_STATIC_MAX_BLOCKS,
                 "ashb_tsdf_fuse_frame_static handles at most %d blocks (got %lld); use ashb_tsdf_touch + "
                 "ashb_tsdf_integrate with caller-provided scratch for larger grids",
                 ASHB_TSDF_STATIC_MAX_BLOCKS, (long long)n_emb);
    ASHB_REQUIRE(n_emb == m->capacity, "n_emb must equal the map's capacity");
    DeviceGuard guard(m->device);
    unsigned char* scratch = nullptr;
    if (int rc = static_scratch_for_current_device(&scratch)) return rc;
    uint32_t* touched = reinterpret_cast<uint32_t*>(scratch);
    int32_t* coords = reinterpret_cast<int32_t*>(scratch + (size_t)ASHB_TSDF_STATIC_MAX_BLOCKS * 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array is shared by every call and keeps the previous call's stamps: start from zero.
    ASHB_CUDA_TRY(cudaMemsetAsync(touched, 0, (size_t)n_emb * sizeof(uint32_t), st));
    const uint32_t stamp = 1;
    if (int rc = ashb_tsdf_touch(m, depth, H, W, intrinsic, cam_to_world, depth_max, cell_size, origin, G, dilation,
                                 bound_lo, bound_hi, coords, touched, stamp, nullptr, nullptr, stream))
        return rc;
    return ashb_tsdf_integrate(embeddings, n_emb, G, D, coords, touched, stamp, depth, color, H, W, intrinsic,
                               world_to_cam, depth_max, cell_size, origin, trunc, sdf_channel, rgb_channel,
                               weight_channel, nullptr, nullptr, nullptr, stream);
}

}  // extern "C"
