// Shared device/host helpers of the lattice_b200 library (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "lattice_b200.h"

namespace lat {

// ---- host-side error plumbing ------------------------------------------------

void set_error(const std::string& message);
int fail(int code, const std::string& message);

#define LAT_CUDA_CHECK(expr)                                                        \
    do {                                                                            \
        cudaError_t lat_err__ = (expr);                                             \
        if (lat_err__ != cudaSuccess) {                                             \
            return ::lat::fail(                                                     \
                LAT_CUDA_ERROR,                                                     \
                std::string(#expr) + ": " + cudaGetErrorString(lat_err__));         \
        }                                                                           \
    } while (0)

// Clock budget of the bounded in-kernel waits (lat_set_wait_budget_cycles).
long long wait_budget_cycles();

// Every kernel launch site is followed by this macro, so it also counts launches.
void count_launch();
#define LAT_LAUNCH_CHECK()                                                          \
    do {                                                                            \
        ::lat::count_launch();                                                      \
        LAT_CUDA_CHECK(cudaGetLastError());                                         \
    } while (0)

#define LAT_REQUIRE(cond, message)                                                  \
    do {                                                                            \
        if (!(cond)) {                                                              \
            return ::lat::fail(LAT_INVALID_ARGUMENT, (message));                    \
        }                                                                           \
    } while (0)

inline cudaStream_t as_stream(void* stream) { return static_cast<cudaStream_t>(stream); }

inline size_t align_up(size_t value, size_t alignment = 256) {
    return (value + alignment - 1) / alignment * alignment;
}

// smallest power of two >= value, never below 4 (one hash bucket)
inline int next_pow2(long long value) {
    long long out = 4;
    while (out < value) {
        out <<= 1;
    }
    return static_cast<int>(out);
}

// Slots of the hash table that holds `rows` keys: a power of two with a load factor in
// (1/8, 1/4], so that a bucket of four slots is almost never full and a probe is one
// sector read. Beyond 2^28 rows the factor halves to keep the slot count in an int.
inline int table_slots(long long rows) {
    rows = rows < 1 ? 1 : rows;
    return next_pow2((rows > (1LL << 28) ? 2 : 4) * rows);
}

// Bump allocator over the caller's workspace.
struct Workspace {
    char* base;
    size_t size;
    size_t used = 0;
    bool ok = true;

    Workspace(void* ptr, size_t bytes) : base(static_cast<char*>(ptr)), size(bytes) {}

    template <typename T> T* take(size_t count) {
        size_t bytes = align_up(count * sizeof(T));
        if (base == nullptr || used + bytes > size) {
            ok = false;
            used += bytes;
            return nullptr;
        }
        T* out = reinterpret_cast<T*>(base + used);
        used += bytes;
        return out;
    }
};

// ---- device helpers -----------------------------------------------------------

struct Coord {
    int b, x, y, z;
};

__device__ __forceinline__ bool operator==(const Coord& l, const Coord& r) {
    return l.b == r.b && l.x == r.x && l.y == r.y && l.z == r.z;
}

__device__ __forceinline__ Coord load_coord(const int32_t* coords, int row) {
    int4 v = __ldg(reinterpret_cast<const int4*>(coords) + row);
    return {v.x, v.y, v.z, v.w};
}

__device__ __forceinline__ void store_coord(int32_t* coords, int row, Coord c) {
    reinterpret_cast<int4*>(coords)[row] = make_int4(c.b, c.x, c.y, c.z);
}

// FNV-1a over (b,x,y,z) as in the reference (coordinates/cpu/common_detail.h:66-77)
// followed by a finaliser so that the low bits used for the slot index are mixed.
__device__ __forceinline__ uint32_t hash_coord(Coord c) {
    uint32_t h = 2166136261u;
    h = (h ^ static_cast<uint32_t>(c.b)) * 16777619u;
    h = (h ^ static_cast<uint32_t>(c.x)) * 16777619u;
    h = (h ^ static_cast<uint32_t>(c.y)) * 16777619u;
    h = (h ^ static_cast<uint32_t>(c.z)) * 16777619u;
    h ^= h >> 16;
    h *= 0x85ebca6bu;
    h ^= h >> 13;
    h *= 0xc2b2ae35u;
    h ^= h >> 16;
    return h;
}

// floor division toward -inf (coordinates/cpu/quantization_detail.h:3-10).
__device__ __forceinline__ int floor_div(int value, int divisor) {
    int q = value / divisor;
    int r = value % divisor;
    if (r != 0 && ((r < 0) != (divisor < 0))) {
        --q;
    }
    return q;
}

__device__ __forceinline__ void raise_status(int32_t* status, int bit) {
    if (status != nullptr) {
        atomicOr(status, bit);
    }
}

__device__ __forceinline__ int clamp_count(const int32_t* ptr, int capacity) {
    int v = __ldg(ptr);
    return v < 0 ? 0 : (v > capacity ? capacity : v);
}

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned mask;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
    return mask;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

// exclusive prefix inside a warp; total returned through `total`
__device__ __forceinline__ int warp_exclusive_scan(int v, int& total) {
    int lane = threadIdx.x & 31;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) {
            inc += n;
        }
    }
    total = __shfl_sync(0xffffffffu, inc, 31);
    return inc - v;
}

// ---- open-addressing table: 8-byte slots (tag << 32 | row) ---------------------------
//
// slots[capacity] (capacity a power of two, load factor <= 1/4) hold (tag << 32) | row
// or kEmptySlot, in buckets of four consecutive slots. Bucket index and tag are two
// 32-bit hashes of the key; a probe reads one bucket, compares tags, and loads the
// stored row's coordinate only on a tag match, so a miss costs one sector read. Equal
// keys keep the smallest row id (first row wins, like the reference's first_row_map,
// coordinates/cpu/quantization_detail.h:
// 394-402): equal keys have equal tags, so a 64-bit atomicMin on the slot is a min
// over the row ids. Linear probing: consecutive slots share 32-byte sectors.
using Slot = unsigned long long;
constexpr Slot kEmptySlot = ~0ull;

// Two 32-bit hashes of a coordinate. Both start from a linear form of the four ints, so
// the form of `base + offset` is the sum of the forms: a kernel map computes the form of
// each output row once and adds a per-offset constant. `index` pushes its form through an
// integer finaliser and picks the bucket; `tag` is the second form as it is and only has to
// differ between keys that share a bucket.
//
// The index form takes z in groups of four (z >> 2, flooring): the four voxels of an aligned
// z-run share their home bucket, which has exactly their four slots. A kernel map probes
// z - 1, z, z + 1 of every (x, y) column of its footprint, and those lie in one group (two
// when z sits at a group's edge): one bucket read answers them (see the probe loop of
// map_single_pass_kernel). The tag keeps the full z, so the keys of a group differ in it.
constexpr uint32_t kHashX = 0x9E3779B1u, kHashY = 0x85EBCA77u, kHashZ = 0xC2B2AE3Du, kHashB = 0x27D4EB2Fu;
constexpr int kHashZShift = 2;

// index form without its z term, and the tag form
__device__ __forceinline__ void hash_linear(Coord c, uint32_t& u_xyb, uint32_t& t) {
    const uint32_t b = static_cast<uint32_t>(c.b), x = static_cast<uint32_t>(c.x);
    const uint32_t y = static_cast<uint32_t>(c.y), z = static_cast<uint32_t>(c.z);
    u_xyb = x * kHashX + y * kHashY + b * kHashB;
    t = x * 0x165667B1u + y * 0xD3A2646Du + z * 0xFD7046C5u + b * 0xB55A4F09u;
}

// z term of the index form
__device__ __forceinline__ uint32_t hash_z_term(int z) {
    return static_cast<uint32_t>(z >> kHashZShift) * kHashZ;
}

__device__ __forceinline__ uint32_t hash_finalize(uint32_t u) {
    u ^= u >> 16;
    u *= 0x7FEB352Du;
    u ^= u >> 15;
    u *= 0x846CA68Bu;
    u ^= u >> 16;
    return u;
}

__device__ __forceinline__ void hash_coord(Coord c, uint32_t& index, uint32_t& tag) {
    uint32_t u;
    hash_linear(c, u, tag);
    index = hash_finalize(u + hash_z_term(c.z));
}

// Buckets of four consecutive slots (one 32-byte sector). Inserts take the first empty
// slot of a bucket in slot order, so a bucket fills from the front and a lookup that
// meets an empty slot knows the key is absent; one sector read decides most probes.
constexpr uint32_t kBucketSlots = 4;

template <typename KeyOf>
__device__ __forceinline__ bool
table_insert(Slot* slots, uint32_t mask, int row, Coord key, KeyOf key_of, bool* met_duplicate) {
    uint32_t index, tag;
    hash_coord(key, index, tag);
    const Slot want = (static_cast<Slot>(tag) << 32) | static_cast<uint32_t>(row);
    uint32_t base = index & mask & ~(kBucketSlots - 1);
    for (uint32_t probe = 0; probe <= mask; probe += kBucketSlots) {
#pragma unroll
        for (uint32_t i = 0; i < kBucketSlots; ++i) {
            Slot* ptr = slots + base + i;
            // at this load factor the slot is usually empty: try to take it outright
            // (one round trip) instead of reading it first
            const Slot cur = atomicCAS(ptr, kEmptySlot, want);
            if (cur == kEmptySlot) {
                return true;
            }
            if (static_cast<uint32_t>(cur >> 32) == tag &&
                key_of(static_cast<int>(cur & 0xFFFFFFFFu)) == key) {
                atomicMin(ptr, want);
                if (met_duplicate != nullptr) {
                    *met_duplicate = true;
                }
                return true;
            }
        }
        base = (base + kBucketSlots) & mask;
    }
    return false;
}

// The four slots of a bucket as 32-bit words: rows in lo.x lo.z hi.x hi.z, tags in
// lo.y lo.w hi.y hi.w (a slot's low word is its row).
struct Bucket {
    uint4 lo, hi;
};

// one 256-bit read-only load (sm_100): the bucket is 32-byte aligned
__device__ __forceinline__ Bucket load_bucket(const Slot* slots, uint32_t base) {
    Bucket b;
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(b.lo.x), "=r"(b.lo.y), "=r"(b.lo.z), "=r"(b.lo.w), "=r"(b.hi.x), "=r"(b.hi.y),
                   "=r"(b.hi.z), "=r"(b.hi.w)
                 : "l"(slots + base));
    return b;
}

// The same load under a predicate, without a branch (the result is undefined when `wanted`
// is false): independent probes of a loop body stay independent loads.
__device__ __forceinline__ Bucket load_bucket_if(const Slot* slots, uint32_t base, bool wanted) {
    Bucket b;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %9, 0;\n"
        "@p ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
        "}"
        : "=r"(b.lo.x), "=r"(b.lo.y), "=r"(b.lo.z), "=r"(b.lo.w), "=r"(b.hi.x), "=r"(b.hi.y),
          "=r"(b.hi.z), "=r"(b.hi.w)
        : "l"(slots + base), "r"(wanted ? 1 : 0));
    return b;
}

// Scan one loaded bucket without data-dependent branches except the rare verification
// of a tag match: returns the row (>= 0), -1 when the key is absent for sure, -2 when
// the bucket is full without a match (continue with the next bucket). A row word of all
// ones marks an empty slot (row ids are non-negative).
template <typename KeyOf>
__device__ __forceinline__ int
scan_bucket(const Bucket& b, uint32_t tag, Coord key, KeyOf key_of) {
    const unsigned empty = (b.lo.x == 0xFFFFFFFFu ? 1u : 0u) | (b.lo.z == 0xFFFFFFFFu ? 2u : 0u) |
                           (b.hi.x == 0xFFFFFFFFu ? 4u : 0u) | (b.hi.z == 0xFFFFFFFFu ? 8u : 0u);
    unsigned match = (b.lo.y == tag ? 1u : 0u) | (b.lo.w == tag ? 2u : 0u) |
                     (b.hi.y == tag ? 4u : 0u) | (b.hi.w == tag ? 8u : 0u);
    match &= ((empty & (0u - empty)) - 1u) & 0xFu;  // only slots before the first empty one
    while (match != 0) {
        const int i = __ffs(match) - 1;
        match &= match - 1;
        const uint32_t row = i == 0 ? b.lo.x : i == 1 ? b.lo.z : i == 2 ? b.hi.x : b.hi.z;
        if (key_of(static_cast<int>(row)) == key) {
            return static_cast<int>(row);
        }
    }
    return empty != 0 ? -1 : -2;
}

// Tag-only scan without branches: the row of the first slot, in slot order, whose tag
// matches (the caller still has to compare coordinates), -1 when the key is absent for
// sure, -2 when the bucket is full without a tag match. A bucket fills from the front and
// an empty slot is all ones, tag word included: a key that is present sits before the
// first empty slot and is met first; a tag of all ones that meets an empty slot reads its
// row word, -1, which says "absent", as it should. The bucket is full exactly when its
// last slot is taken.
__device__ __forceinline__ int scan_bucket_tags(const Bucket& b, uint32_t tag) {
    const int none = b.hi.z != 0xFFFFFFFFu ? -2 : -1;
    return b.lo.y == tag   ? static_cast<int>(b.lo.x)
           : b.lo.w == tag ? static_cast<int>(b.lo.z)
           : b.hi.y == tag ? static_cast<int>(b.hi.x)
           : b.hi.w == tag ? static_cast<int>(b.hi.z)
                           : none;
}

template <typename KeyOf>
__device__ __forceinline__ int
table_find(const Slot* slots, uint32_t mask, Coord key, KeyOf key_of) {
    uint32_t index, tag;
    hash_coord(key, index, tag);
    uint32_t base = index & mask & ~(kBucketSlots - 1);
    for (uint32_t probe = 0; probe <= mask; probe += kBucketSlots) {
        const Bucket b = load_bucket(slots, base);
        int found = scan_bucket(b, tag, key, key_of);
        if (found != -2) {
            return found;
        }
        base = (base + kBucketSlots) & mask;
    }
    return -1;
}

// ---- 4-byte-slot variant (row ids only) -------------------------------------------
//
// slots[capacity] (capacity a power of two) hold a row id or -1. The key of a slot
// is whatever `key_of(row)` says for the stored row, so the table itself stays
// 4 bytes per slot; equal keys keep the smallest row id (first row wins, like the
// reference's first_row_map, coordinates/cpu/quantization_detail.h:394-402).

template <typename KeyOf>
__device__ __forceinline__ bool
table32_insert(int32_t* slots, uint32_t mask, int row, Coord key, KeyOf key_of, bool* met_duplicate) {
    uint32_t slot = hash_coord(key) & mask;
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        int cur = *reinterpret_cast<volatile int32_t*>(slots + slot);
        if (cur == -1) {
            int old = atomicCAS(&slots[slot], -1, row);
            if (old == -1) {
                return true;
            }
            cur = old;
        }
        if (key_of(cur) == key) {
            atomicMin(&slots[slot], row);
            if (met_duplicate != nullptr) {
                *met_duplicate = true;
            }
            return true;
        }
        slot = (slot + 1) & mask;
    }
    return false;
}

template <typename KeyOf>
__device__ __forceinline__ int
table32_find(const int32_t* slots, uint32_t mask, Coord key, KeyOf key_of) {
    uint32_t slot = hash_coord(key) & mask;
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        int cur = __ldg(slots + slot);
        if (cur == -1) {
            return -1;
        }
        if (key_of(cur) == key) {
            return cur;
        }
        slot = (slot + 1) & mask;
    }
    return -1;
}

struct PlainKey {
    const int32_t* coords;
    __device__ __forceinline__ Coord operator()(int row) const { return load_coord(coords, row); }
};

struct DownsampledKey {
    const int32_t* coords;
    int sx, sy, sz;
    __device__ __forceinline__ Coord operator()(int row) const {
        Coord c = load_coord(coords, row);
        return {c.b, floor_div(c.x, sx), floor_div(c.y, sy), floor_div(c.z, sz)};
    }
};

// kernel offset k of a (Kx,Ky,Kz) footprint, x-major / z-fastest, odd sizes centred,
// even sizes starting at 0, times dilation (coordinates/offsets.cpp:11-45).
struct KernelGeometry {
    int kx, ky, kz;
    int dx, dy, dz;
    int volume;

    __host__ __device__ void offset(int k, int& ox, int& oy, int& oz) const {
        int ix = k / (ky * kz);
        int rem = k - ix * ky * kz;
        int iy = rem / kz;
        int iz = rem - iy * kz;
        ox = (ix - ((kx & 1) ? kx / 2 : 0)) * dx;
        oy = (iy - ((ky & 1) ? ky / 2 : 0)) * dy;
        oz = (iz - ((kz & 1) ? kz / 2 : 0)) * dz;
    }
};

inline KernelGeometry make_geometry(lat_triple size, lat_triple dilation) {
    return {size.x, size.y, size.z, dilation.x, dilation.y, dilation.z,
            size.x * size.y * size.z};
}

} // namespace lat
