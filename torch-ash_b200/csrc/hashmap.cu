// Collision-free spatial hash engine for sm_100a: a lock-free open-addressing
// table over packed int32 keys.
//
// Layout in HBM
//   key_dim 1..3 : one 16-byte slot {k0, k1, k2, value}; a probe is one 128-bit
//                  load and an insert claims a slot with one 128-bit CAS, so no
//                  reader ever waits for a half-written key.
//   key_dim 4    : one 32-byte slot {k0..k3, value, pad}; the value word is
//                  claimed with a 32-bit CAS (LOCKED), the key written, then the
//                  value released; readers that meet LOCKED wait with a bound.
//   value        : >= 0 index into the caller's value/embedding rows,
//                  EMPTY (-1), TOMB (-2, erased), PENDING (-3, index not yet
//                  assigned; only inside an insert launch), LOCKED (-4).
//   n_slots      : power of two >= 2 * capacity (load factor <= 0.5), linear
//                  probing: consecutive probes stay inside one 128-byte line.
//   heap         : the caller's int32[capacity] free-index stack; counter is a
//                  device int32 (= number of live keys).  Pops and pushes are
//                  warp-aggregated: one atomic per warp, not per key.
//
// Semantics follow ash/src/hashmap_gpu.cuh (find :164-178, insert-if-absent +
// heap pop :212-232, value copy by the winner :250-283, erase + heap push
// :317-336, clear :355-358, items :377-405, load_states :408-450).
#include <cstring>
#include <new>

#include "hashmap.cuh"

namespace ashb {

// ---- find ----------------------------------------------------------------------
// FILTER (16-byte slots only): the one-bit-per-slot occupancy map is consulted first.  A key whose
// home slot never held anything is absent, and the map (1/128 of the table) sits in L2 when the
// table itself is far beyond it, so such a miss costs no DRAM access at all.
template <class Table, int DIM, bool FILTER = false>
__global__ void __launch_bounds__(256) find_kernel(Table t, const int32_t* __restrict__ keys, int64_t n,
                                                   int64_t* __restrict__ indices,
                                                   uint8_t* __restrict__ masks) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int k0, k1, k2, k3;
    if constexpr (FILTER) {   // the batch and the slots pass through L2 once (first out); the bit map stays
        const int32_t* p = keys + i * DIM;
        k0 = __ldcs(p);
        k1 = DIM > 1 ? __ldcs(p + 1) : 0;
        k2 = DIM > 2 ? __ldcs(p + 2) : 0;
        k3 = 0;
    } else {
        load_key<DIM>(keys, i, k0, k1, k2, k3);
    }
    uint32_t s = hash_key(k0, k1, k2, k3) & t.mask;
    int found = -1;
    bool absent = false;
    if constexpr (FILTER) absent = t.never_used(s);
    if (!absent) {
        for (uint32_t probe = 0; probe <= t.mask; ++probe) {
            Entry e;
            if constexpr (FILTER) e = t.read_const_passing(s);
            else e = t.read_const(s);
            if (e.val == kEmpty) break;
            if (e.val >= 0 && key_match(e, k0, k1, k2, k3)) {
                found = e.val;
                break;
            }
            s = (s + 1) & t.mask;
        }
    }
    if constexpr (FILTER) {
        __stcs(indices + i, found >= 0 ? (int64_t)found : 0);
        __stcs(masks + i, (uint8_t)(found >= 0));
    } else {
        indices[i] = found >= 0 ? (int64_t)found : 0;
        masks[i] = (uint8_t)(found >= 0);
    }
}

// Sub-warp cooperative variant for 16-byte slots: 8 lanes serve one query and read the whole
// 128-byte line (8 slots) that holds the key's home slot with one coalesced request, then the
// next line, and so on; a ballot finds the first slot in probe order that is empty or holds the
// key, so the answer is identical to the one-thread probe.  It moves the same DRAM lines as the
// one-thread kernel but needs one round trip per LINE of the probe chain instead of one per slot.
template <int DIM>
__global__ void __launch_bounds__(256) find_coop_kernel(Table16 t, const int32_t* __restrict__ keys, int64_t n,
                                                        int64_t* __restrict__ indices, uint8_t* __restrict__ masks) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> 3;
    const int sub = (int)(tid & 7);
    const int group_shift = (int)(threadIdx.x & 31) & ~7;  // first lane of this 8-lane group in the warp
    const bool live = q < n;
    int k0 = 0, k1 = 0, k2 = 0, k3 = 0;
    if (live) load_key<DIM>(keys, q, k0, k1, k2, k3);
    const uint32_t home = hash_key(k0, k1, k2, k3) & t.mask;
    uint32_t line = home & ~7u;
    bool done = !live, first = true;
    int found = -1;
    const uint32_t n_lines = (t.mask >> 3) + 1;
    for (uint32_t it = 0; it <= n_lines && __any_sync(0xffffffffu, !done); ++it) {
        Entry e{0, 0, 0, 0, kTomb};
        const uint32_t slot = line + sub;
        if (!done) e = t.read_const(slot);
        const bool in_chain = !first || slot >= home;  // the chain starts at the home slot
        const unsigned hit = __ballot_sync(0xffffffffu, !done && in_chain && e.val >= 0 && key_match(e, k0, k1, k2, k3));
        const unsigned empty = __ballot_sync(0xffffffffu, !done && in_chain && e.val == kEmpty);
        const unsigned g_hit = (hit >> group_shift) & 0xFFu, g_empty = (empty >> group_shift) & 0xFFu;
        const int first_hit = g_hit ? __ffs(g_hit) - 1 : 99, first_empty = g_empty ? __ffs(g_empty) - 1 : 99;
        const int src = group_shift + (first_hit < 99 ? first_hit : 0);
        const int val = __shfl_sync(0xffffffffu, e.val, src);
        if (!done) {
            if (first_hit < first_empty) {
                found = val;
                done = true;
            } else if (first_empty < 99) {
                done = true;
            } else {
                line = (line + 8) & t.mask;
                first = false;
            }
        }
    }
    if (live && sub == 0) {
        indices[q] = found >= 0 ? (int64_t)found : 0;
        masks[q] = (uint8_t)(found >= 0);
    }
}

// ---- insert ----------------------------------------------------------------------
struct ValueCtx {
    int n;
    const char* src[kMaxValues];
    char* dst[kMaxValues];
    long long row_bytes[kMaxValues];
    int word[kMaxValues];  // widest power-of-two copy word (<= 16) both sides allow
};

__device__ __forceinline__ void copy_row(const char* __restrict__ src, char* __restrict__ dst,
                                         long long bytes, int word) {
    switch (word) {
        case 16:
            for (long long b = 0; b < bytes; b += 16)
                *reinterpret_cast<int4*>(dst + b) = *reinterpret_cast<const int4*>(src + b);
            break;
        case 8:
            for (long long b = 0; b < bytes; b += 8)
                *reinterpret_cast<int2*>(dst + b) = *reinterpret_cast<const int2*>(src + b);
            break;
        case 4:
            for (long long b = 0; b < bytes; b += 4)
                *reinterpret_cast<int*>(dst + b) = *reinterpret_cast<const int*>(src + b);
            break;
        case 2:
            for (long long b = 0; b < bytes; b += 2)
                *reinterpret_cast<short*>(dst + b) = *reinterpret_cast<const short*>(src + b);
            break;
        default:
            for (long long b = 0; b < bytes; ++b) dst[b] = src[b];
    }
}

template <class Table, int DIM>
__global__ void __launch_bounds__(256) insert_kernel(Table t, const int32_t* __restrict__ keys, int64_t n,
                                                     int32_t* __restrict__ heap, int32_t* counter,
                                                     int32_t capacity, ValueCtx vctx) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t slot = -1;
    if (i < n) {
        int k0, k1, k2, k3;
        load_key<DIM>(keys, i, k0, k1, k2, k3);
        bool present = false;
        slot = emplace(t, k0, k1, k2, k3, kPending, &present);
    }
    // one atomic on the stack counter per CTA (launched with 256 threads) instead of one per warp
    const int idx = pop_index_for_slot_cta(t, slot, heap, counter, capacity);
    if (idx < 0) return;
    for (int j = 0; j < vctx.n; ++j)
        copy_row(vctx.src[j] + i * vctx.row_bytes[j], vctx.dst[j] + (long long)idx * vctx.row_bytes[j],
                 vctx.row_bytes[j], vctx.word[j]);
    publish_index(t, slot, idx);
}

// ---- erase -----------------------------------------------------------------------
template <class Table, int DIM>
__global__ void __launch_bounds__(256) erase_kernel(Table t, const int32_t* __restrict__ keys, int64_t n,
                                                    int32_t* __restrict__ heap, int32_t* counter) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int idx = -1;
    if (i < n) {
        int k0, k1, k2, k3;
        load_key<DIM>(keys, i, k0, k1, k2, k3);
        idx = tombstone_key(t, k0, k1, k2, k3);
    }
    push_freed_index_cta(idx, heap, counter);  // launched with 256 threads
}

// Sub-warp cooperative erase for 16-byte slots, the counterpart of find_coop_kernel: 8 lanes serve
// one key and read the whole 128-byte line (8 slots) that holds its home slot per step; a ballot
// finds the first slot in probe order that is empty or holds the key, one lane turns it into a
// tombstone and the freed indices go back on the stack with one atomic per CTA.  Same result as
// erase_kernel.
template <int DIM>
__global__ void __launch_bounds__(256) erase_coop_kernel(Table16 t, const int32_t* __restrict__ keys, int64_t n,
                                                         int32_t* __restrict__ heap, int32_t* counter) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t q = tid >> 3;
    const int sub = (int)(tid & 7);
    const int group_shift = (int)(threadIdx.x & 31) & ~7;
    const bool live = q < n;
    int k0 = 0, k1 = 0, k2 = 0, k3 = 0;
    if (live) load_key<DIM>(keys, q, k0, k1, k2, k3);
    const uint32_t home = hash_key(k0, k1, k2, k3) & t.mask;
    uint32_t line = home & ~7u;
    bool done = !live, first = true;
    int idx = -1;
    const uint32_t n_lines = (t.mask >> 3) + 1;
    for (uint32_t it = 0; it <= n_lines && __any_sync(0xffffffffu, !done); ++it) {
        Entry e{0, 0, 0, 0, kTomb};
        const uint32_t slot = line + sub;
        if (!done) e = t.read_fresh(slot);
        const bool in_chain = !first || slot >= home;
        const unsigned hit = __ballot_sync(0xffffffffu, !done && in_chain && e.val >= 0 && key_match(e, k0, k1, k2, k3));
        const unsigned empty = __ballot_sync(0xffffffffu, !done && in_chain && e.val == kEmpty);
        const unsigned g_hit = (hit >> group_shift) & 0xFFu, g_empty = (empty >> group_shift) & 0xFFu;
        const int first_hit = g_hit ? __ffs(g_hit) - 1 : 99, first_empty = g_empty ? __ffs(g_empty) - 1 : 99;
        if (!done) {
            if (first_hit < first_empty) {
                // the lane that read the key's slot erases it; in-batch duplicates race, one CAS wins
                if (sub == first_hit && atomicCAS(t.val_ptr(slot), e.val, kTomb) == e.val) idx = e.val;
                done = true;
            } else if (first_empty < 99) {
                done = true;
            } else {
                line = (line + 8) & t.mask;
                first = false;
            }
        }
    }
    push_freed_index_cta(idx, heap, counter);  // launched with 256 threads
}

// ---- load_states -----------------------------------------------------------------
template <class Table, int DIM>
__global__ void __launch_bounds__(256) load_states_kernel(Table t, const int32_t* __restrict__ keys,
                                                          const int64_t* __restrict__ indices, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int k0, k1, k2, k3;
    load_key<DIM>(keys, i, k0, k1, k2, k3);
    bool present = false;
    emplace(t, k0, k1, k2, k3, (int)indices[i], &present);
    if (present) atomicOr(t.status, ASHB_STATUS_DUPLICATE);
}

// ---- rehash ------------------------------------------------------------------------
// Copies every live (key, index) pair of `src` into the empty table `dst`; erased slots
// (tombstones) are left behind, so probe sequences are short again.
template <class Table, int DIM>
__global__ void __launch_bounds__(256) rehash_kernel(Table dst, Table src) {
    const uint64_t n_slots = (uint64_t)src.mask + 1;
    for (uint64_t s = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; s < n_slots;
         s += (uint64_t)gridDim.x * blockDim.x) {
        const Entry e = src.read_const((uint32_t)s);
        if (e.val < 0) continue;
        bool present = false;
        emplace(dst, e.k0, e.k1, e.k2, e.k3, e.val, &present);
        if (present) atomicOr(dst.status, ASHB_STATUS_DUPLICATE);
    }
}

__global__ void set_counter_kernel(int32_t* counter, int32_t v) { *counter = v; }

__global__ void reset_heap_kernel(int32_t* __restrict__ heap, int64_t capacity) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < capacity;
         i += (int64_t)gridDim.x * blockDim.x)
        heap[i] = (int32_t)i;
}

// ---- items -----------------------------------------------------------------------
// Compacted enumeration.  A CTA scans a tile of 256 x 4 slots per round, ranks its
// live slots with a block-wide prefix sum and reserves its output range with ONE
// atomic, so the shared cursor sees n_slots / 1024 atomics instead of one per warp.
template <class Table, int DIM>
__global__ void __launch_bounds__(256) items_kernel(Table t, int32_t* __restrict__ keys_out,
                                                    int64_t* __restrict__ indices_out, int64_t max_n,
                                                    unsigned long long* cursor) {
    constexpr int kPerThread = 4;
    __shared__ unsigned warp_totals[8];
    __shared__ unsigned long long tile_base;
    const uint64_t n_slots = (uint64_t)t.mask + 1;
    const uint64_t tile = 256ull * kPerThread;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint64_t start = (uint64_t)blockIdx.x * tile; start < n_slots; start += (uint64_t)gridDim.x * tile) {
        Entry e[kPerThread];
        unsigned mine = 0;
#pragma unroll
        for (int j = 0; j < kPerThread; ++j) {
            const uint64_t s = start + (uint64_t)j * 256 + threadIdx.x;
            e[j] = Entry{0, 0, 0, 0, kEmpty};
            if (s < n_slots) e[j] = t.read_const((uint32_t)s);
            mine += e[j].val >= 0;
        }
        // exclusive prefix of `mine` over the CTA
        unsigned incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_totals[warp] = incl;
        __syncthreads();
        unsigned before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const unsigned v = warp_totals[w];
            if (w < warp) before += v;
            total += v;
        }
        if (threadIdx.x == 0) tile_base = total ? atomicAdd(cursor, (unsigned long long)total) : 0ull;
        __syncthreads();
        int64_t o = (int64_t)tile_base + before + (incl - mine);
#pragma unroll
        for (int j = 0; j < kPerThread; ++j) {
            if (e[j].val < 0) continue;
            if (o < max_n) {
                int32_t* k = keys_out + o * DIM;
                k[0] = e[j].k0;
                if (DIM > 1) k[1] = e[j].k1;
                if (DIM > 2) k[2] = e[j].k2;
                if (DIM > 3) k[3] = e[j].k3;
                indices_out[o] = e[j].val;
            }
            ++o;
        }
        __syncthreads();  // warp_totals / tile_base are reused next round
    }
}

}  // namespace ashb

using namespace ashb;

namespace {

template <class F16, class F32>
int dispatch(ashb_map* m, F16&& f16, F32&& f32) {
    if (m->key_dim == 4) {
        Table32 t{static_cast<Slot32*>(m->slots), (uint32_t)(m->n_slots - 1), m->status};
        return f32(t);
    }
    return f16(table16_of(m));
}

inline unsigned blocks_for(int64_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

int check_map(ashb_map* m) {
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    return ASHB_OK;
}

#define ASHB_MAP_PROLOGUE(m)                      \
    if (int _rc = check_map(m)) return _rc;       \
    DeviceGuard _guard((m)->device);              \
    if (!_guard.ok) {                             \
        set_error("cannot select device %d", (m)->device); \
        return ASHB_ERR_CUDA;                     \
    }

#define ASHB_DIM_LAUNCH(KERNEL, m, grid, block, st, ...)                                   \
    dispatch(                                                                              \
            m,                                                                             \
            [&](Table16 t) {                                                               \
                switch ((m)->key_dim) {                                                    \
                    case 1: KERNEL<Table16, 1><<<grid, block, 0, st>>>(t, __VA_ARGS__); break; \
                    case 2: KERNEL<Table16, 2><<<grid, block, 0, st>>>(t, __VA_ARGS__); break; \
                    default: KERNEL<Table16, 3><<<grid, block, 0, st>>>(t, __VA_ARGS__); break; \
                }                                                                          \
                return 0;                                                                  \
            },                                                                             \
            [&](Table32 t) {                                                               \
                KERNEL<Table32, 4><<<grid, block, 0, st>>>(t, __VA_ARGS__);                \
                return 0;                                                                  \
            })

}  // namespace

// Which find kernel ashb_map_find launches for 16-byte slots (process-wide switches).
static bool g_find_cooperative = false;
// Occupancy filter in find: -1 = automatic (tables of kFilterMinBytes and more, i.e. those that do
// not stay in L2 anyway), 0 = never, 1 = always.
static int g_find_filter = -1;
static bool g_erase_cooperative = false;
constexpr size_t kFilterMinBytes = (size_t)64 << 20;

static size_t occupied_bytes(uint64_t n_slots) { return (size_t)(n_slots / 8 < 4 ? 4 : n_slots / 8); }

extern "C" {

int ashb_map_create(int key_dim, int64_t capacity, int32_t* heap_dev, int device, ashb_map** out) {
    ASHB_REQUIRE(out != nullptr, "out is null");
    *out = nullptr;
    ASHB_REQUIRE(key_dim >= 1 && key_dim <= 4, "key_dim %d not in 1..4", key_dim);
    ASHB_REQUIRE(capacity >= 1 && capacity <= (int64_t)1 << 30, "capacity %lld not in 1..2^30",
                 (long long)capacity);
    ASHB_REQUIRE(heap_dev != nullptr, "heap is null");
    DeviceGuard guard(device);
    if (!guard.ok) {
        set_error("cannot select device %d", device);
        return ASHB_ERR_CUDA;
    }
    ashb_map* m = new (std::nothrow) ashb_map();
    ASHB_REQUIRE(m != nullptr, "out of host memory");
    m->key_dim = key_dim;
    m->capacity = capacity;
    m->device = device;
    m->heap = heap_dev;
    uint64_t n = 32;
    while (n < 2ull * (uint64_t)capacity) n <<= 1;
    m->n_slots = n;
    m->slot_bytes = key_dim == 4 ? sizeof(Slot32) : sizeof(uint4);
    cudaError_t e = cudaMalloc(&m->slots, n * m->slot_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&m->small, 256);
    if (e == cudaSuccess && key_dim <= 3) e = cudaMalloc(reinterpret_cast<void**>(&m->occupied), occupied_bytes(n));
    if (e != cudaSuccess) {
        set_error("cudaMalloc of %llu-slot table failed: %s", (unsigned long long)n, cudaGetErrorString(e));
        if (m->slots) cudaFree(m->slots);
        if (m->small) cudaFree(m->small);
        delete m;
        return ASHB_ERR_CUDA;
    }
    m->counter = reinterpret_cast<int32_t*>(m->small);
    m->status = reinterpret_cast<uint32_t*>(static_cast<char*>(m->small) + 64);
    m->cursor = reinterpret_cast<unsigned long long*>(static_cast<char*>(m->small) + 128);
    // 0xFF bytes: every key word -1 and every value word EMPTY (-1); for 32-byte
    // slots the pad words too.  Ordered before any later work on any stream by
    // the synchronising memset on the legacy stream.
    e = cudaMemset(m->slots, 0xFF, n * m->slot_bytes);
    if (e == cudaSuccess) e = cudaMemset(m->small, 0, 256);
    if (e == cudaSuccess && m->occupied) e = cudaMemset(m->occupied, 0, occupied_bytes(n));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("table initialisation failed: %s", cudaGetErrorString(e));
        cudaFree(m->slots);
        cudaFree(m->small);
        if (m->occupied) cudaFree(m->occupied);
        delete m;
        return ASHB_ERR_CUDA;
    }
    *out = m;
    return ASHB_OK;
}

int ashb_map_destroy(ashb_map* m) {
    if (m == nullptr) return ASHB_OK;
    DeviceGuard guard(m->device);
    if (m->slots) cudaFree(m->slots);
    if (m->small) cudaFree(m->small);
    if (m->occupied) cudaFree(m->occupied);
    m->slots = nullptr;
    delete m;
    return ASHB_OK;
}

int ashb_map_clear(ashb_map* m, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemsetAsync(m->slots, 0xFF, m->n_slots * m->slot_bytes, st));
    if (m->occupied) ASHB_CUDA_TRY(cudaMemsetAsync(m->occupied, 0, occupied_bytes(m->n_slots), st));
    ASHB_CUDA_TRY(cudaMemsetAsync(m->counter, 0, sizeof(int32_t), st));
    reset_heap_kernel<<<wave_grid(m->capacity, 256, 8), 256, 0, st>>>(m->heap, m->capacity);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_map_size(ashb_map* m, void* stream, int64_t* size_out) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(size_out != nullptr, "size_out is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t v = 0;
    ASHB_CUDA_TRY(cudaMemcpyAsync(&v, m->counter, sizeof(v), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    *size_out = v;
    return ASHB_OK;
}

int ashb_map_status(ashb_map* m, void* stream, uint32_t* status_out) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(status_out != nullptr, "status_out is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t v = 0;
    ASHB_CUDA_TRY(cudaMemcpyAsync(&v, m->status, sizeof(v), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaMemsetAsync(m->status, 0, sizeof(v), st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    *status_out = v;
    return ASHB_OK;
}

int ashb_map_status_async(ashb_map* m, uint32_t* status_out_host, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(status_out_host != nullptr, "status_out_host is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemcpyAsync(status_out_host, m->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaMemsetAsync(m->status, 0, sizeof(uint32_t), st));
    return ASHB_OK;
}

int ashb_map_find(ashb_map* m, const int32_t* keys, int64_t n, int64_t* indices, uint8_t* masks,
                  void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(n >= 0, "negative count");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(keys && indices && masks, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g_find_cooperative && m->key_dim <= 3) {
        const Table16 t = table16_of(m);
        const unsigned grid = blocks_for(n * 8, 256);
        switch (m->key_dim) {
            case 1: find_coop_kernel<1><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
            case 2: find_coop_kernel<2><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
            default: find_coop_kernel<3><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
        }
    } else if (m->occupied != nullptr &&
               (g_find_filter > 0 || (g_find_filter < 0 && m->n_slots * m->slot_bytes >= kFilterMinBytes))) {
        const Table16 t = table16_of(m);
        const unsigned grid = blocks_for(n, 256);
        switch (m->key_dim) {
            case 1: find_kernel<Table16, 1, true><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
            case 2: find_kernel<Table16, 2, true><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
            default: find_kernel<Table16, 3, true><<<grid, 256, 0, st>>>(t, keys, n, indices, masks); break;
        }
    } else {
        ASHB_DIM_LAUNCH(find_kernel, m, blocks_for(n, 256), 256, st, keys, n, indices, masks);
    }
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_set_find_cooperative(int enable) {
    g_find_cooperative = enable != 0;
    return ASHB_OK;
}

int ashb_set_find_filter(int mode) {
    ASHB_REQUIRE(mode >= -1 && mode <= 1, "mode must be -1 (automatic), 0 (off) or 1 (on)");
    g_find_filter = mode;
    return ASHB_OK;
}

static int insert_impl(ashb_map* m, const int32_t* keys, int64_t n, const ValueCtx& vctx, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(n >= 0, "negative count");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(keys != nullptr, "null keys");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_DIM_LAUNCH(insert_kernel, m, blocks_for(n, 256), 256, st, keys, n, m->heap, m->counter,
                    (int32_t)m->capacity, vctx);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_map_insert_keys(ashb_map* m, const int32_t* keys, int64_t n, void* stream) {
    ValueCtx v;
    std::memset(&v, 0, sizeof(v));
    return insert_impl(m, keys, n, v, stream);
}

int ashb_map_insert_values(ashb_map* m, const int32_t* keys, int64_t n, int n_values,
                           const void* const* src, void* const* dst, const int64_t* row_bytes,
                           void* stream) {
    ASHB_REQUIRE(n_values >= 0 && n_values <= kMaxValues, "n_values %d not in 0..%d", n_values, kMaxValues);
    ASHB_REQUIRE(n_values == 0 || (src && dst && row_bytes), "null value tables");
    ValueCtx v;
    std::memset(&v, 0, sizeof(v));
    v.n = n_values;
    for (int j = 0; j < n_values; ++j) {
        ASHB_REQUIRE(src[j] && dst[j] && row_bytes[j] > 0, "value %d: null pointer or empty row", j);
        v.src[j] = static_cast<const char*>(src[j]);
        v.dst[j] = static_cast<char*>(dst[j]);
        v.row_bytes[j] = row_bytes[j];
        int w = 16;
        const uintptr_t bits = (uintptr_t)src[j] | (uintptr_t)dst[j] | (uintptr_t)row_bytes[j];
        while (w > 1 && (bits & (uintptr_t)(w - 1))) w >>= 1;
        v.word[j] = w;
    }
    return insert_impl(m, keys, n, v, stream);
}

int ashb_map_erase(ashb_map* m, const int32_t* keys, int64_t n, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(n >= 0, "negative count");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(keys != nullptr, "null keys");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g_erase_cooperative && m->key_dim <= 3) {
        const Table16 t = table16_of(m);
        const unsigned grid = blocks_for(n * 8, 256);
        switch (m->key_dim) {
            case 1: erase_coop_kernel<1><<<grid, 256, 0, st>>>(t, keys, n, m->heap, m->counter); break;
            case 2: erase_coop_kernel<2><<<grid, 256, 0, st>>>(t, keys, n, m->heap, m->counter); break;
            default: erase_coop_kernel<3><<<grid, 256, 0, st>>>(t, keys, n, m->heap, m->counter); break;
        }
    } else {
        ASHB_DIM_LAUNCH(erase_kernel, m, blocks_for(n, 256), 256, st, keys, n, m->heap, m->counter);
    }
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_set_erase_cooperative(int enable) {
    g_erase_cooperative = enable != 0;
    return ASHB_OK;
}

int ashb_map_items(ashb_map* m, int32_t* keys_out, int64_t* indices_out, int64_t max_n, int64_t* n_out,
                   void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(max_n >= 0 && n_out != nullptr, "bad output arguments");
    ASHB_REQUIRE(max_n == 0 || (keys_out && indices_out), "null output buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemsetAsync(m->cursor, 0, sizeof(unsigned long long), st));
    const unsigned grid = wave_grid((int64_t)(m->n_slots / 4 + 1), 256, 8);
    ASHB_DIM_LAUNCH(items_kernel, m, grid, 256, st, keys_out, indices_out, max_n, m->cursor);
    ASHB_LAUNCH_CHECK();
    unsigned long long total = 0;
    ASHB_CUDA_TRY(cudaMemcpyAsync(&total, m->cursor, sizeof(total), cudaMemcpyDeviceToHost, st));
    ASHB_CUDA_TRY(cudaStreamSynchronize(st));
    *n_out = (int64_t)total;
    return ASHB_OK;
}

int ashb_map_load_states(ashb_map* m, const int32_t* keys, const int64_t* indices, int64_t n,
                         const int32_t* heap_src, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    ASHB_REQUIRE(n >= 0 && n <= m->capacity, "count %lld not in 0..capacity", (long long)n);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Start from an empty table: loading on top of live entries would mix two states.
    ASHB_CUDA_TRY(cudaMemsetAsync(m->slots, 0xFF, m->n_slots * m->slot_bytes, st));
    if (m->occupied) ASHB_CUDA_TRY(cudaMemsetAsync(m->occupied, 0, occupied_bytes(m->n_slots), st));
    set_counter_kernel<<<1, 1, 0, st>>>(m->counter, (int32_t)n);
    ASHB_LAUNCH_CHECK();
    if (heap_src != nullptr && heap_src != m->heap)
        ASHB_CUDA_TRY(cudaMemcpyAsync(m->heap, heap_src, sizeof(int32_t) * m->capacity,
                                      cudaMemcpyDeviceToDevice, st));
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(keys && indices, "null buffer");
    ASHB_DIM_LAUNCH(load_states_kernel, m, blocks_for(n, 256), 256, st, keys, indices, n);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_map_rehash(ashb_map* m, void* stream) {
    ASHB_MAP_PROLOGUE(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* fresh = nullptr;
    uint32_t* fresh_occ = nullptr;
    ASHB_CUDA_TRY(cudaMalloc(&fresh, m->n_slots * m->slot_bytes));
    cudaError_t e = cudaSuccess;
    if (m->occupied) e = cudaMalloc(reinterpret_cast<void**>(&fresh_occ), occupied_bytes(m->n_slots));
    if (e == cudaSuccess) e = cudaMemsetAsync(fresh, 0xFF, m->n_slots * m->slot_bytes, st);
    if (e == cudaSuccess && fresh_occ) e = cudaMemsetAsync(fresh_occ, 0, occupied_bytes(m->n_slots), st);
    if (e == cudaSuccess) {
        const unsigned grid = wave_grid((int64_t)m->n_slots, 256, 8);
        const uint32_t mask = (uint32_t)(m->n_slots - 1);
        if (m->key_dim == 4) {
            rehash_kernel<Table32, 4><<<grid, 256, 0, st>>>(Table32{static_cast<Slot32*>(fresh), mask, m->status},
                                                            Table32{static_cast<Slot32*>(m->slots), mask, m->status});
        } else {
            rehash_kernel<Table16, 3><<<grid, 256, 0, st>>>(
                    Table16{static_cast<uint4*>(fresh), mask, m->status, fresh_occ}, table16_of(m));
        }
        e = cudaGetLastError();
    }
    // the old table must outlive the copy; rehashing is rare, so simply wait for it
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        set_error("rehash failed: %s", cudaGetErrorString(e));
        cudaFree(fresh);
        if (fresh_occ) cudaFree(fresh_occ);
        return ASHB_ERR_CUDA;
    }
    cudaFree(m->slots);
    if (m->occupied) cudaFree(m->occupied);
    m->slots = fresh;
    m->occupied = fresh_occ;
    return ASHB_OK;
}

}  // extern "C"
