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

inline int next_pow2(long long value) {
    long long out = 1;
    while (out < value) {
        out <<= 1;
    }
    return static_cast<int>(out);
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
// slots[capacity] (capacity a power of two) hold (tag << 32) | row or kEmptySlot. The
// tag is the upper half of a 64-bit hash of the key, the slot index its lower bits; a
// probe compares tags first and loads the stored row's coordinate only on a tag match,
// so a miss costs slot reads only. Equal keys keep the smallest row id (first row
// wins, like the reference's first_row_map, coordinates/cpu/quantization_detail.h:
// 394-402): equal keys have equal tags, so a 64-bit atomicMin on the slot is a min
// over the row ids. Linear probing: consecutive slots share 32-byte sectors.
using Slot = unsigned long long;
constexpr Slot kEmptySlot = ~0ull;

__device__ __forceinline__ unsigned long long hash_coord64(Coord c) {
    unsigned long long k0 =
        (static_cast<unsigned long long>(static_cast<uint32_t>(c.b)) << 32) | static_cast<uint32_t>(c.x);
    unsigned long long k1 =
        (static_cast<unsigned long long>(static_cast<uint32_t>(c.y)) << 32) | static_cast<uint32_t>(c.z);
    unsigned long long h = k0 * 0x9E3779B97F4A7C15ull;
    h ^= h >> 32;
    h = (h ^ k1) * 0xC2B2AE3D27D4EB4Full;
    h ^= h >> 29;
    h *= 0x165667B19E3779F9ull;
    h ^= h >> 32;
    return h;
}

template <typename KeyOf>
__device__ __forceinline__ bool
table_insert(Slot* slots, uint32_t mask, int row, Coord key, KeyOf key_of, bool* met_duplicate) {
    const unsigned long long h = hash_coord64(key);
    const Slot tag = h & 0xFFFFFFFF00000000ull;
    const Slot want = tag | static_cast<uint32_t>(row);
    uint32_t slot = static_cast<uint32_t>(h) & mask;
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        Slot cur = *reinterpret_cast<volatile Slot*>(slots + slot);
        if (cur == kEmptySlot) {
            Slot old = atomicCAS(slots + slot, kEmptySlot, want);
            if (old == kEmptySlot) {
                return true;
            }
            cur = old;
        }
        if ((cur & 0xFFFFFFFF00000000ull) == tag && key_of(static_cast<int>(cur & 0xFFFFFFFFu)) == key) {
            atomicMin(slots + slot, want);
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
table_find(const Slot* slots, uint32_t mask, Coord key, KeyOf key_of) {
    const unsigned long long h = hash_coord64(key);
    const Slot tag = h & 0xFFFFFFFF00000000ull;
    uint32_t slot = static_cast<uint32_t>(h) & mask;
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        Slot cur = __ldg(slots + slot);
        if (cur == kEmptySlot) {
            return -1;
        }
        if ((cur & 0xFFFFFFFF00000000ull) == tag) {
            int row = static_cast<int>(cur & 0xFFFFFFFFu);
            if (key_of(row) == key) {
                return row;
            }
        }
        slot = (slot + 1) & mask;
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
