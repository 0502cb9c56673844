// Peer-memory transport for the key-hash-partitioned hash map (one process per GPU, every rank's
// mailbox mapped into every other rank over NVLink).  The reference is single-GPU and has no
// counterpart.  A find over the partitioned map is two launches per rank and no data collective:
//
//   route   every key is written straight into its OWNER's inbox as a 12-byte record
//           {k0, k1, k2} (unused columns zero).  Rank r owns region r of every inbox, so
//           the write position comes from a LOCAL cursor (one atomic per CTA and owner) and no
//           remote atomic is needed; a CTA gathers the records of its 1024 keys per owner in shared
//           memory and stores each owner's run as one contiguous segment; the per-region counts
//           are published to the owners at the end.
//   (stream-ordered barrier across the ranks: a collective on a one-element tensor)
//   answer  every owner probes the records of its inbox and stores the answers (its local index
//           or -1, 4 bytes) straight into the ASKER's answer buffer, region by region in inbox order, so that
//           the peer stores of a warp are contiguous (scattered 8-byte peer stores ran at a
//           fraction of the link rate); the asker remembers, per key, which owner and slot it
//           used and gathers its answers locally afterwards.
//   (barrier)
//
// Neither kernel waits on another GPU: ordering comes from the barriers the host enqueues between
// them.  Every remote address is base[peer] + offset with the offset checked against the layout
// the caller describes; records that would not fit are dropped and reported in a status word.
#include "hashmap.cuh"

namespace ashb {

constexpr int kPeerMaxWorld = 32;   // where[i] = owner << 26 | slot must stay a non-negative int32

// Same owner function as route.cu / ash.distributed.owner_of (int64 wrap-around arithmetic).
__device__ __forceinline__ int peer_owner_of(int k0, int k1, int k2, int dim, int world) {
    const unsigned long long primes[3] = {73856093ull, 19349663ull, 83492791ull};
    const int k[3] = {k0, k1, k2};
    long long h = 0;
    for (int d = 0; d < dim; ++d) h ^= (long long)((unsigned long long)(long long)k[d] * primes[d]);
    h = (long long)((unsigned long long)(h ^ (h >> 15)) * 0x2C1B3C6Dull);
    h ^= h >> 12;
    long long r = h % world;
    return (int)(r < 0 ? r + world : r);
}

struct PeerLayout {
    void* const* bases;      // device array [world]: base address of every rank's mailbox as mapped here
    int64_t inbox_offset;    // int32 [world][region_capacity][3]: 12-byte records, region r written by rank r
    int64_t counts_offset;   // int32 [world]: records in each region
    int64_t answers_offset;  // int32 [world][region_capacity]: region o = answers of owner o, in inbox order
    int64_t region_capacity;
    int64_t answer_capacity;
    int world, rank;
};

constexpr int kWhereOwnerShift = 26;  // where[i] = owner << 26 | slot

struct PeerKey {
    int x, y, z;
};
// Record j of region `region` of this rank's inbox.
__device__ __forceinline__ PeerKey peer_read_key(const PeerLayout& L, int region, int64_t j) {
    const int* rec = reinterpret_cast<const int*>(static_cast<const char*>(L.bases[L.rank]) + L.inbox_offset) +
                     ((int64_t)region * L.region_capacity + j) * 3;
    return PeerKey{__ldcg(rec), __ldcg(rec + 1), __ldcg(rec + 2)};
}

// One CTA routes a tile of kRouteTile keys.  Its records are first gathered per owner in shared
// memory and then written out run by run, consecutive threads storing consecutive 4-byte words of
// the run's 12-byte records: a link carries few long segments far better than many short ones (one
// store per lane to whichever owner its key hashes to was 128 bytes per warp and owner at best).
constexpr int kRouteKeysPerThread = 4;
constexpr int kRouteTile = 256 * kRouteKeysPerThread;

template <int DIM>
__global__ void __launch_bounds__(256) peer_route_kernel(const int32_t* __restrict__ keys, int64_t n, PeerLayout L,
                                                         int* __restrict__ cursor, int32_t* __restrict__ where,
                                                         uint32_t* __restrict__ status) {
    __shared__ int staged[kRouteTile * 3];
    __shared__ unsigned char staged_owner[kRouteTile];
    __shared__ int cta_count[kPeerMaxWorld];   // records of this tile per owner
    __shared__ int cta_base[kPeerMaxWorld];    // first slot of the tile's run in the owner's region
    __shared__ int run_start[kPeerMaxWorld + 1];
    const int lane = threadIdx.x & 31;
    const int64_t tile_first = (int64_t)blockIdx.x * kRouteTile;
    for (int o = threadIdx.x; o < L.world; o += blockDim.x) cta_count[o] = 0;
    __syncthreads();
    int rec[kRouteKeysPerThread][3];
    int owner[kRouteKeysPerThread], within[kRouteKeysPerThread];
#pragma unroll
    for (int j = 0; j < kRouteKeysPerThread; ++j) {
        const int64_t i = tile_first + j * 256 + threadIdx.x;
        const bool live = i < n;
        int k0 = 0, k1 = 0, k2 = 0, k3 = 0;
        if (live) load_key<DIM>(keys, i, k0, k1, k2, k3);
        rec[j][0] = k0;
        rec[j][1] = k1;
        rec[j][2] = k2;
        // lanes without a key take a negative owner of their own, so that they match nobody
        owner[j] = live ? peer_owner_of(k0, k1, k2, DIM, L.world) : -1 - lane;
        const unsigned peers = __match_any_sync(0xffffffffu, owner[j]);
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if (live && lane == leader) base = atomicAdd(&cta_count[owner[j]], __popc(peers));
        within[j] = __shfl_sync(0xffffffffu, base, leader) + __popc(peers & lanemask_lt());
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int sum = 0;
        for (int o = 0; o < L.world; ++o) {
            run_start[o] = sum;
            sum += cta_count[o];
        }
        run_start[L.world] = sum;
    }
    for (int o = threadIdx.x; o < L.world; o += blockDim.x)
        cta_base[o] = cta_count[o] ? atomicAdd(&cursor[o], cta_count[o]) : 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kRouteKeysPerThread; ++j) {
        const int64_t i = tile_first + j * 256 + threadIdx.x;
        if (i >= n) continue;
        const int at = run_start[owner[j]] + within[j];
        staged[3 * at] = rec[j][0];
        staged[3 * at + 1] = rec[j][1];
        staged[3 * at + 2] = rec[j][2];
        staged_owner[at] = (unsigned char)owner[j];
        const int64_t slot = (int64_t)cta_base[owner[j]] + within[j];
        if (slot >= L.region_capacity) atomicOr(status, ASHB_STATUS_CAPACITY);
        if (where) where[i] = slot < L.region_capacity ? (int)((unsigned)owner[j] << kWhereOwnerShift | (unsigned)slot) : -1;
    }
    __syncthreads();
    const int total_words = 3 * run_start[L.world];
    for (int word = threadIdx.x; word < total_words; word += blockDim.x) {
        const int at = word / 3;
        const int o = staged_owner[at];
        const int64_t slot = (int64_t)cta_base[o] + (at - run_start[o]);
        if (slot >= L.region_capacity) continue;   // dropped and reported above
        int* inbox = reinterpret_cast<int*>(static_cast<char*>(L.bases[o]) + L.inbox_offset);
        inbox[((int64_t)L.rank * L.region_capacity + slot) * 3 + (word - 3 * at)] = staged[word];
    }
}

__global__ void peer_publish_counts_kernel(PeerLayout L, const int* __restrict__ cursor) {
    const int o = threadIdx.x;
    if (o >= L.world) return;
    int* counts = reinterpret_cast<int*>(static_cast<char*>(L.bases[o]) + L.counts_offset);
    const int64_t c = cursor[o];
    counts[L.rank] = (int)(c < L.region_capacity ? c : L.region_capacity);
}

// A region holds region_capacity records in the worst case (every key of a batch to one owner) and
// about 1 / world of that usually, so the kernels below do not launch one CTA per 256 possible
// records: a fixed grid walks the tiles of 256 records that the regions actually hold.  Every CTA
// reads the region counts once and numbers the occupied tiles of all regions in one sequence.
struct PeerTiles {
    int count[kPeerMaxWorld];          // records per region (clamped to the capacity)
    int64_t first[kPeerMaxWorld + 1];  // number of the first tile of every region in that sequence
};

__device__ __forceinline__ void peer_number_tiles(const PeerLayout& L, PeerTiles* tiles) {
    if (threadIdx.x == 0) {
        const int* counts = reinterpret_cast<const int*>(static_cast<const char*>(L.bases[L.rank]) + L.counts_offset);
        int64_t sum = 0;
        for (int r = 0; r < L.world; ++r) {
            int64_t c = __ldcg(counts + r);
            c = c < 0 ? 0 : (c > L.region_capacity ? L.region_capacity : c);
            tiles->count[r] = (int)c;
            tiles->first[r] = sum;
            sum += (c + 255) / 256;
        }
        tiles->first[L.world] = sum;
    }
    __syncthreads();
}

__device__ __forceinline__ int peer_region_of_tile(const PeerTiles& tiles, int64_t tile) {
    int region = 0;
    while (tile >= tiles.first[region + 1]) ++region;   // at most world <= 32 steps
    return region;
}

__global__ void __launch_bounds__(256) peer_answer_kernel(Table16 t, PeerLayout L, bool filter) {
    __shared__ PeerTiles tiles;
    peer_number_tiles(L, &tiles);
    const char* mine = static_cast<const char*>(L.bases[L.rank]);
    for (int64_t tile = blockIdx.x; tile < tiles.first[L.world]; tile += gridDim.x) {
        const int region = peer_region_of_tile(tiles, tile);  // the rank that asked
        const int64_t j = (tile - tiles.first[region]) * 256 + threadIdx.x;
        if (j >= tiles.count[region]) continue;
        const PeerKey rec = peer_read_key(L, region, j);
        const int idx = filter ? lookup_filtered(t, rec.x, rec.y, rec.z) : lookup(t, rec.x, rec.y, rec.z, 0);
        int32_t* answers = reinterpret_cast<int32_t*>(static_cast<char*>(L.bases[region]) + L.answers_offset);
        answers[(int64_t)L.rank * L.region_capacity + j] = idx >= 0 ? idx : -1;   // my region of the asker's answers
    }
}

// The asker's side: answer of key i = answers[owner(i)][slot(i)] of its own mailbox; the global index
// of a key is its owner's local index * world + owner.
__global__ void __launch_bounds__(256) peer_unpack_kernel(PeerLayout L, const int32_t* __restrict__ where, int64_t n,
                                                          int64_t* __restrict__ indices, uint8_t* __restrict__ masks) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int w = where[i];
    long long answer = -1;
    if (w >= 0) {
        const int owner = (int)((unsigned)w >> kWhereOwnerShift);
        const int64_t slot = (unsigned)w & ((1u << kWhereOwnerShift) - 1);
        const char* mine = static_cast<const char*>(L.bases[L.rank]);
        if (owner < L.world && slot < L.region_capacity) {
            const int local = __ldcg(reinterpret_cast<const int32_t*>(mine + L.answers_offset) + (int64_t)owner * L.region_capacity + slot);
            if (local >= 0) answer = (long long)local * L.world + owner;
        }
    }
    indices[i] = answer >= 0 ? answer : 0;
    masks[i] = (uint8_t)(answer >= 0);
}

// insert-if-absent / erase of the records in this rank's inbox (no answers go back)
template <bool ERASE>
__global__ void __launch_bounds__(256) peer_update_kernel(Table16 t, PeerLayout L, int32_t* __restrict__ heap,
                                                          int32_t* counter, int32_t capacity) {
    __shared__ PeerTiles tiles;
    peer_number_tiles(L, &tiles);
    const char* mine = static_cast<const char*>(L.bases[L.rank]);
    for (int64_t tile = blockIdx.x; tile < tiles.first[L.world]; tile += gridDim.x) {
        const int region = peer_region_of_tile(tiles, tile);
        const int64_t j = (tile - tiles.first[region]) * 256 + threadIdx.x;
        const bool live = j < tiles.count[region];
        PeerKey rec{0, 0, 0};
        if (live) rec = peer_read_key(L, region, j);
        // the whole CTA (256 threads) goes through the stack operations below: one atomic per CTA
        if (ERASE) {
            push_freed_index_cta(live ? tombstone_key(t, rec.x, rec.y, rec.z, 0) : -1, heap, counter);
        } else {
            bool present = false;
            const int64_t slot = live ? emplace(t, rec.x, rec.y, rec.z, 0, kPending, &present) : -1;
            const int idx = pop_index_for_slot_cta(t, slot, heap, counter, capacity);
            if (idx >= 0) publish_index(t, slot, idx);
        }
        __syncthreads();   // the shared words of the CTA-wide stack operations are reused by the next tile
    }
}

}  // namespace ashb

using namespace ashb;

static int check_layout(const PeerLayout& L, int64_t mailbox_bytes) {
    ASHB_REQUIRE(L.bases != nullptr, "null peer table");
    ASHB_REQUIRE(L.world >= 1 && L.world <= kPeerMaxWorld && L.rank >= 0 && L.rank < L.world, "bad world / rank");
    ASHB_REQUIRE(L.region_capacity >= 1 && L.region_capacity <= (1ll << kWhereOwnerShift) && L.answer_capacity >= 1 &&
                         L.answer_capacity <= 0x7fffffffll,
                 "bad capacities (a region holds at most 2^26 records)");
    ASHB_REQUIRE(L.inbox_offset >= 0 && L.inbox_offset % 16 == 0 && L.counts_offset % 4 == 0 && L.answers_offset % 8 == 0,
                 "misaligned mailbox sections");
    const int64_t inbox_end = L.inbox_offset + (int64_t)L.world * L.region_capacity * 12;
    const int64_t counts_end = L.counts_offset + (int64_t)L.world * 4;
    const int64_t answers_end = L.answers_offset + (int64_t)L.world * L.region_capacity * 4;
    ASHB_REQUIRE(inbox_end <= L.counts_offset && counts_end <= L.answers_offset && answers_end <= mailbox_bytes,
                 "mailbox sections overlap or exceed the mailbox");
    return ASHB_OK;
}

extern "C" {

int ashb_peer_route_keys(const int32_t* keys, int64_t n, int key_dim, int world, int rank,
                         void* const* peer_bases_dev, int64_t mailbox_bytes, int64_t inbox_offset,
                         int64_t counts_offset, int64_t answers_offset, int64_t region_capacity,
                         int64_t answer_capacity, int32_t* cursor_dev, int32_t* where_dev, uint32_t* status_dev,
                         void* stream) {
    const PeerLayout L{peer_bases_dev, inbox_offset, counts_offset, answers_offset, region_capacity, answer_capacity,
                       world, rank};
    if (int rc = check_layout(L, mailbox_bytes)) return rc;
    ASHB_REQUIRE(key_dim >= 1 && key_dim <= 3, "the peer transport carries keys of 1 to 3 columns");
    ASHB_REQUIRE(n >= 0 && n <= answer_capacity, "batch of %lld keys exceeds the mailbox's %lld", (long long)n,
                 (long long)answer_capacity);
    ASHB_REQUIRE(cursor_dev && status_dev && (n == 0 || keys), "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ASHB_CUDA_TRY(cudaMemsetAsync(cursor_dev, 0, (size_t)world * sizeof(int32_t), st));
    if (n > 0) {
        const unsigned grid = (unsigned)((n + kRouteTile - 1) / kRouteTile);
        switch (key_dim) {
            case 1: peer_route_kernel<1><<<grid, 256, 0, st>>>(keys, n, L, cursor_dev, where_dev, status_dev); break;
            case 2: peer_route_kernel<2><<<grid, 256, 0, st>>>(keys, n, L, cursor_dev, where_dev, status_dev); break;
            default: peer_route_kernel<3><<<grid, 256, 0, st>>>(keys, n, L, cursor_dev, where_dev, status_dev); break;
        }
        ASHB_LAUNCH_CHECK();
    }
    peer_publish_counts_kernel<<<1, kPeerMaxWorld, 0, st>>>(L, cursor_dev);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_peer_find_answer(ashb_map* m, int world, int rank, void* const* peer_bases_dev, int64_t mailbox_bytes,
                          int64_t inbox_offset, int64_t counts_offset, int64_t answers_offset,
                          int64_t region_capacity, int64_t answer_capacity, void* stream) {
    const PeerLayout L{peer_bases_dev, inbox_offset, counts_offset, answers_offset, region_capacity, answer_capacity,
                       world, rank};
    if (int rc = check_layout(L, mailbox_bytes)) return rc;
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim <= 3, "the peer transport carries keys of 1 to 3 columns");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = wave_grid(((region_capacity + 255) / 256) * 256 * (int64_t)world, 256, 8);
    // as in ashb_map_find: the occupancy filter pays off for tables that do not stay in L2
    const bool filter = m->occupied != nullptr && m->n_slots * m->slot_bytes >= ((size_t)64 << 20);
    peer_answer_kernel<<<grid, 256, 0, st>>>(table16_of(m), L, filter);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_peer_unpack_answers(const int32_t* where_dev, int64_t n, int world, int rank, void* const* peer_bases_dev,
                             int64_t mailbox_bytes, int64_t inbox_offset, int64_t counts_offset,
                             int64_t answers_offset, int64_t region_capacity, int64_t answer_capacity,
                             int64_t* indices, uint8_t* masks, void* stream) {
    const PeerLayout L{peer_bases_dev, inbox_offset, counts_offset, answers_offset, region_capacity, answer_capacity,
                       world, rank};
    if (int rc = check_layout(L, mailbox_bytes)) return rc;
    ASHB_REQUIRE(n >= 0 && n <= answer_capacity, "bad count");
    if (n == 0) return ASHB_OK;
    ASHB_REQUIRE(where_dev && indices && masks, "null buffer");
    peer_unpack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(L, where_dev, n,
                                                                                                   indices, masks);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

int ashb_peer_update(ashb_map* m, int erase, int world, int rank, void* const* peer_bases_dev,
                     int64_t mailbox_bytes, int64_t inbox_offset, int64_t counts_offset, int64_t answers_offset,
                     int64_t region_capacity, int64_t answer_capacity, void* stream) {
    const PeerLayout L{peer_bases_dev, inbox_offset, counts_offset, answers_offset, region_capacity, answer_capacity,
                       world, rank};
    if (int rc = check_layout(L, mailbox_bytes)) return rc;
    ASHB_REQUIRE(m != nullptr && m->slots != nullptr, "null or destroyed map");
    ASHB_REQUIRE(m->key_dim <= 3, "the peer transport carries keys of 1 to 3 columns");
    DeviceGuard guard(m->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = wave_grid(((region_capacity + 255) / 256) * 256 * (int64_t)world, 256, 8);
    if (erase)
        peer_update_kernel<true><<<grid, 256, 0, st>>>(table16_of(m), L, m->heap, m->counter, (int32_t)m->capacity);
    else
        peer_update_kernel<false><<<grid, 256, 0, st>>>(table16_of(m), L, m->heap, m->counter, (int32_t)m->capacity);
    ASHB_LAUNCH_CHECK();
    return ASHB_OK;
}

}  // extern "C"
