// Device-side view of the hash table of libashb200, shared by every kernel that
// probes it (hash engine, ray sampler, fused grid query, TSDF integration).
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
#pragma once

#include "common.cuh"

namespace ashb {

constexpr int kEmpty = -1;
constexpr int kTomb = -2;
constexpr int kPending = -3;
constexpr int kLocked = -4;
constexpr int kSpinLimit = 1 << 20;
constexpr int kMaxValues = 16;

struct Entry {
    int k0, k1, k2, k3;
    int val;
};

__device__ __forceinline__ bool key_match(const Entry& e, int k0, int k1, int k2, int k3) {
    return e.k0 == k0 && e.k1 == k1 && e.k2 == k2 && e.k3 == k3;
}

union U128 {
    unsigned __int128 q;
    uint4 v;
};

// ---- 16-byte slots, key_dim <= 3 ---------------------------------------------
struct Table16 {
    uint4* slots;
    uint32_t mask;
    uint32_t* status;
    // One bit per slot, set when a key is first stored there and cleared only with the whole table
    // (erased slots keep it: probe chains run through them).  At 1/128 of the table's size it stays
    // in L2 where the table does not, so a find whose home slot never held a key is answered without
    // a DRAM access.  Null for tables built without one.
    uint32_t* occupied;

    __device__ __forceinline__ Entry unpack(uint4 r) const {
        return Entry{(int)r.x, (int)r.y, (int)r.z, 0, (int)r.w};
    }
    // Read-only probe (find / items): table is constant for the launch.
    // The loads name a 64-byte L2 fetch size: a probe needs one 16-byte slot of a random line, and
    // the default fill of the whole 128-byte line from DRAM is wasted traffic.
    __device__ __forceinline__ Entry read_const(uint32_t s) const {
        uint4 u;
        asm volatile("ld.global.nc.L2::64B.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                     : "l"(slots + s));
        return unpack(u);
    }
    // The same with the line marked first to leave L2: beside the bit map, which a filtered find
    // wants to keep there, a slot read once is only passing through.
    __device__ __forceinline__ Entry read_const_passing(uint32_t s) const {
        uint4 u;
        uint64_t policy;
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        asm volatile("ld.global.nc.L2::cache_hint.L2::64B.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                     : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                     : "l"(slots + s), "l"(policy));
        return unpack(u);
    }
    // Probe inside a mutating launch: read at L2, where the atomics resolve.
    __device__ __forceinline__ Entry read_fresh(uint32_t s) const {
        uint4 u;
        asm volatile("ld.global.cg.L2::64B.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                     : "l"(slots + s)
                     : "memory");
        return unpack(u);
    }
    // Try to turn the free slot `s` (last seen as `expected`) into {key, PENDING}.
    // On failure `observed` holds what is there now.
    __device__ __forceinline__ bool claim(uint32_t s, const Entry& expected, int k0, int k1, int k2,
                                          int k3, int new_val, Entry& observed) const {
        (void)k3;
        U128 cmp, val, old;
        cmp.v = make_uint4((unsigned)expected.k0, (unsigned)expected.k1, (unsigned)expected.k2,
                           (unsigned)expected.val);
        val.v = make_uint4((unsigned)k0, (unsigned)k1, (unsigned)k2, (unsigned)new_val);
        old.q = atomicCAS(reinterpret_cast<unsigned __int128*>(slots + s), cmp.q, val.q);
        observed = unpack(old.v);
        if (old.q != cmp.q) return false;
        // an erased slot was marked when its first key arrived
        if (occupied != nullptr && expected.val == kEmpty) atomicOr(occupied + (s >> 5), 1u << (s & 31));
        return true;
    }
    __device__ __forceinline__ bool never_used(uint32_t s) const {
        uint32_t word;   // marked last to leave L2
        uint64_t policy;
        asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
        asm volatile("ld.global.nc.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(word) : "l"(occupied + (s >> 5)), "l"(policy));
        return ((word >> (s & 31)) & 1u) == 0;
    }
    __device__ __forceinline__ int* val_ptr(uint32_t s) const {
        return reinterpret_cast<int*>(slots + s) + 3;
    }
};

// ---- 32-byte slots, key_dim == 4 -----------------------------------------------
struct __align__(32) Slot32 {
    int k[4];
    int val;
    int pad[3];
};

struct Table32 {
    Slot32* slots;
    uint32_t mask;
    uint32_t* status;

    __device__ __forceinline__ Entry read_const(uint32_t s) const {
        const int4 k = __ldg(reinterpret_cast<const int4*>(slots[s].k));
        const int v = __ldg(&slots[s].val);
        return Entry{k.x, k.y, k.z, k.w, v};
    }
    // Waits (bounded) while another thread is between claiming the slot and
    // publishing its key; on a timeout the slot is reported as an unrelated
    // occupied one and the status word records it.
    __device__ __forceinline__ Entry read_fresh(uint32_t s) const {
        volatile int* vp = &slots[s].val;
        int v = *vp;
        for (int spin = 0; v == kLocked; ++spin) {
            if (spin >= kSpinLimit) {
                atomicOr(status, ASHB_STATUS_SPIN);
                return Entry{0, 0, 0, 0, kLocked};
            }
            __nanosleep(32);
            v = *vp;
        }
        __threadfence();
        const int4 k = __ldcg(reinterpret_cast<const int4*>(slots[s].k));
        return Entry{k.x, k.y, k.z, k.w, v};
    }
    __device__ __forceinline__ bool claim(uint32_t s, const Entry& expected, int k0, int k1, int k2,
                                          int k3, int new_val, Entry& observed) const {
        const int old = atomicCAS(&slots[s].val, expected.val, kLocked);
        if (old != expected.val) {
            observed = read_fresh(s);
            return false;
        }
        __stcg(reinterpret_cast<int4*>(slots[s].k), make_int4(k0, k1, k2, k3));
        __threadfence();
        *reinterpret_cast<volatile int*>(&slots[s].val) = new_val;
        observed = Entry{k0, k1, k2, k3, new_val};
        return true;
    }
    __device__ __forceinline__ int* val_ptr(uint32_t s) const { return &slots[s].val; }
};

template <int DIM>
__device__ __forceinline__ void load_key(const int32_t* __restrict__ keys, int64_t i, int& k0, int& k1,
                                         int& k2, int& k3) {
    const int32_t* p = keys + i * DIM;
    k0 = p[0];
    k1 = DIM > 1 ? p[1] : 0;
    k2 = DIM > 2 ? p[2] : 0;
    k3 = DIM > 3 ? p[3] : 0;
}

// Insert-if-absent of one key; returns the claimed slot or -1 (present, lost a
// duplicate race, or table exhausted).  `new_val` is what the slot holds when
// claimed: PENDING for inserts (index assigned afterwards) or a saved index.
template <class Table>
__device__ __forceinline__ int64_t emplace(const Table& t, int k0, int k1, int k2, int k3,
                                           int new_val, bool* already_present) {
    uint32_t s = hash_key(k0, k1, k2, k3) & t.mask;
    int64_t free_slot = -1;
    Entry free_entry{};
    // A failed claim restarts the scan at the contested slot, so the bound is on
    // total steps rather than on one pass.
    for (uint64_t steps = 0; steps <= 4ull * t.mask + 8; ++steps) {
        const Entry e = t.read_fresh(s);
        if (e.val == kEmpty) {
            const uint32_t target = free_slot >= 0 ? (uint32_t)free_slot : s;
            const Entry expected = free_slot >= 0 ? free_entry : e;
            Entry seen;
            if (t.claim(target, expected, k0, k1, k2, k3, new_val, seen)) return (int64_t)target;
            if (seen.val != kEmpty && seen.val != kTomb && seen.val != kLocked &&
                key_match(seen, k0, k1, k2, k3)) {
                *already_present = true;
                return -1;
            }
            s = target;  // somebody else's key landed there: rescan from it
            free_slot = -1;
            continue;
        }
        if (e.val == kTomb) {
            if (free_slot < 0) {
                free_slot = s;
                free_entry = e;
            }
        } else if (e.val != kLocked && key_match(e, k0, k1, k2, k3)) {
            *already_present = true;
            return -1;
        }
        s = (s + 1) & t.mask;
    }
    atomicOr(t.status, ASHB_STATUS_PROBE);
    return -1;
}

// Second half of an insert, called by ALL lanes of a warp: the lanes that claimed a slot (slot >= 0)
// pop their row indices from the free-index stack with one atomic for the warp.  Returns the
// index, or -1 for lanes without a slot or when the stack is empty (the slot is then given back and
// ASHB_STATUS_CAPACITY recorded).  The caller copies its value rows and then publishes the index
// with publish_index.
template <class Table>
__device__ __forceinline__ int pop_index_for_slot(const Table& t, int64_t slot, int32_t* __restrict__ heap,
                                                  int32_t* counter, int32_t capacity) {
    const bool won = slot >= 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, won);
    if (ballot == 0) return -1;
    const int leader = __ffs(ballot) - 1;
    int base = 0;
    if ((int)(threadIdx.x & 31) == leader) base = atomicAdd(counter, __popc(ballot));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (!won) return -1;
    const int top = base + __popc(ballot & lanemask_lt());
    if (top >= capacity) {
        // No free index left: undo the pop, give the slot back, record it.
        atomicSub(counter, 1);
        *reinterpret_cast<volatile int*>(t.val_ptr((uint32_t)slot)) = kTomb;
        atomicOr(t.status, ASHB_STATUS_CAPACITY);
        return -1;
    }
    return heap[top];
}

// The same for a whole CTA of 256 threads (all of them call it): the warps' counts meet in shared
// memory and ONE atomic per CTA reserves the indices, an eighth of the same-address atomics of the
// warp-level form.
template <class Table>
__device__ __forceinline__ int pop_index_for_slot_cta(const Table& t, int64_t slot, int32_t* __restrict__ heap,
                                                      int32_t* counter, int32_t capacity) {
    __shared__ int warp_count[8];
    __shared__ int cta_base;
    const bool won = slot >= 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, won);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_count[warp] = __popc(ballot);
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += warp_count[w];
        cta_base = total ? atomicAdd(counter, total) : 0;
    }
    __syncthreads();
    if (!won) return -1;
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_count[w];
    const int top = cta_base + before + __popc(ballot & lanemask_lt());
    if (top >= capacity) {
        atomicSub(counter, 1);
        *reinterpret_cast<volatile int*>(t.val_ptr((uint32_t)slot)) = kTomb;
        atomicOr(t.status, ASHB_STATUS_CAPACITY);
        return -1;
    }
    return heap[top];
}

template <class Table>
__device__ __forceinline__ void publish_index(const Table& t, int64_t slot, int idx) {
    *reinterpret_cast<volatile int*>(t.val_ptr((uint32_t)slot)) = idx;
}

// First half of an erase: turns the key's slot into a tombstone; returns the freed row index or -1.
template <class Table>
__device__ __forceinline__ int tombstone_key(const Table& t, int k0, int k1, int k2, int k3) {
    uint32_t s = hash_key(k0, k1, k2, k3) & t.mask;
    for (uint32_t probe = 0; probe <= t.mask; ++probe) {
        const Entry e = t.read_fresh(s);
        if (e.val == kEmpty) break;
        if (e.val >= 0 && key_match(e, k0, k1, k2, k3)) {
            // In-batch duplicates race here; exactly one CAS succeeds.
            if (atomicCAS(t.val_ptr(s), e.val, kTomb) == e.val) return e.val;
            break;
        }
        s = (s + 1) & t.mask;
    }
    return -1;
}

// Second half of an erase, called by ALL lanes of a warp: freed indices (idx >= 0) go back on the
// stack with one atomic for the warp.
__device__ __forceinline__ void push_freed_index(int idx, int32_t* __restrict__ heap, int32_t* counter) {
    const bool won = idx >= 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, won);
    if (ballot == 0) return;
    const int leader = __ffs(ballot) - 1;
    int base = 0;
    if ((int)(threadIdx.x & 31) == leader) base = atomicSub(counter, __popc(ballot));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (!won) return;
    const int top = base - __popc(ballot & lanemask_lt());
    if (top >= 1) heap[top - 1] = idx;
}

// The same for a whole CTA of 256 threads: one atomic per CTA.
__device__ __forceinline__ void push_freed_index_cta(int idx, int32_t* __restrict__ heap, int32_t* counter) {
    __shared__ int warp_count[8];
    __shared__ int cta_base;
    const bool won = idx >= 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, won);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_count[warp] = __popc(ballot);
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += warp_count[w];
        cta_base = total ? atomicSub(counter, total) : 0;
    }
    __syncthreads();
    if (!won) return;
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_count[w];
    const int top = cta_base - before - __popc(ballot & lanemask_lt());
    if (top >= 1) heap[top - 1] = idx;
}

// Read-only lookup: index of the key or -1.
template <class Table>
__device__ __forceinline__ int lookup(const Table& t, int k0, int k1, int k2, int k3) {
    uint32_t s = hash_key(k0, k1, k2, k3) & t.mask;
    for (uint32_t probe = 0; probe <= t.mask; ++probe) {
        const Entry e = t.read_const(s);
        if (e.val == kEmpty) return -1;
        if (e.val >= 0 && key_match(e, k0, k1, k2, k3)) return e.val;
        s = (s + 1) & t.mask;
    }
    return -1;
}

// The same for 16-byte-slot tables that are far larger than L2: the occupancy bit of the home slot
// is read first, and a key whose home slot never held anything is reported absent without a probe.
__device__ __forceinline__ int lookup_filtered(const Table16& t, int k0, int k1, int k2) {
    uint32_t s = hash_key(k0, k1, k2, 0) & t.mask;
    if (t.occupied != nullptr && t.never_used(s)) return -1;
    for (uint32_t probe = 0; probe <= t.mask; ++probe) {
        const Entry e = t.read_const_passing(s);   // the slots pass through L2, the bit map stays
        if (e.val == kEmpty) return -1;
        if (e.val >= 0 && key_match(e, k0, k1, k2, 0)) return e.val;
        s = (s + 1) & t.mask;
    }
    return -1;
}

}  // namespace ashb

// The host-side map object behind the opaque `ashb_map*` of the C ABI.
struct ashb_map {
    int key_dim;
    int64_t capacity;
    int device;
    uint64_t n_slots;
    void* slots;
    size_t slot_bytes;
    uint32_t* occupied;          // device: one bit per 16-byte slot (null for key_dim 4)
    int32_t* heap;               // borrowed: the caller's free-index stack
    int32_t* counter;            // device: live keys == popped indices
    uint32_t* status;            // device: ASHB_STATUS_* bits
    unsigned long long* cursor;  // device scratch for items()
    void* small;                 // one allocation backing the three words above
};

namespace ashb {

inline Table16 table16_of(const ashb_map* m) {
    return Table16{static_cast<uint4*>(m->slots), (uint32_t)(m->n_slots - 1), m->status, m->occupied};
}

// Selects the map's device for the scope of a call.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
        if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace ashb
