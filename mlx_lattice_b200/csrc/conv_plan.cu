// Gather plan of the tensor-core convolution for one kernel relation.
//
// The output rows, taken through an optional permutation, are cut into 256-row tiles.
// For every tile the plan holds
//   tile_info[tile] = (mask, base): the kernel offsets any row of the tile uses, and the
//                     index of the tile's first row vector;
//   tile_order:       the tiles by falling number of used offsets (equal counts in tile
//                     order, tiles that use none last). A tile's cost in the convolution is
//                     its number of used offsets, and with mask-sorted rows that number
//                     varies from 1 to K along the tiles: handing the tiles out round-robin
//                     in their natural order left the busiest CTA 19-39 % above the mean on
//                     LiDAR-like supports; the serpentine over the sorted order (plan_position)
//                     leaves it 2-5 % above;
//   one row vector per used offset, in ascending offset order: the input row of each of
//   the 256 tile rows at that offset, -1 where the row has no neighbour there.
// The convolution kernel then streams these vectors instead of walking the CSR rows of
// the relation tile by tile (three dependent loads per row before the first gather),
// and a relation is usually consumed by several convolutions.
//
// A row vector is stored in the order the gather threads read it: tile row r sits at
// (r % 32) * 8 + r / 32, so the eight rows q, q + 32, ... q + 224 of gather thread group
// q are 32 contiguous bytes.
#include <algorithm>

#include "common.cuh"
#include "conv_plan.cuh"

namespace lat {

namespace {

// Up to this many tiles (1 M output rows) every block of the fill kernel sums the masks of
// the tiles before it itself; above it a one-block scan runs first.
constexpr int kSelfScanTiles = 4096;

struct PlanBuildParams {
    const int32_t* in_rows;
    const int32_t* kernel_ids;
    const int32_t* row_offsets;
    const int32_t* counts;
    const int32_t* row_order;
    const int32_t* row_masks;   // optional: bit k of row_masks[row] = the row has an edge at offset k
    int edge_capacity;
    int in_capacity;
    int out_capacity;
    int kernel_count;
    int num_tiles;
    int prescanned;         // 1: plan_scan_kernel has filled tile_info[].y and the closing entry
    int2* tile_info;
    int32_t* tile_order;
    int32_t* vectors;
    int32_t* status;
};

// the output row a tile position stands for, -1 beyond the capacity or when invalid
__device__ __forceinline__ int plan_row(const PlanBuildParams& p, int position) {
    if (position >= p.out_capacity) {
        return -1;
    }
    int row = p.row_order != nullptr ? __ldg(p.row_order + position) : position;
    if (row < 0 || row >= p.out_capacity) {
        raise_status(p.status, LAT_STATUS_BAD_INDEX);
        return -1;
    }
    return row;
}

// pass 1: offset mask of every tile
__global__ void __launch_bounds__(kPlanTileRows) plan_mask_kernel(PlanBuildParams p) {
    __shared__ uint32_t tile_mask;
    if (threadIdx.x == 0) {
        tile_mask = 0;
    }
    __syncthreads();
    const int n_out = clamp_count(p.counts + 1, p.out_capacity);
    const int edge_total = clamp_count(p.counts, p.edge_capacity);
    const int row = plan_row(p, blockIdx.x * kPlanTileRows + threadIdx.x);
    uint32_t mask = 0;
    if (p.row_masks != nullptr) {
        // the kernel map already knows which offsets each row uses
        if (row >= 0 && row < n_out) {
            mask = static_cast<uint32_t>(__ldg(p.row_masks + row));
            if (p.kernel_count < 32) {
                mask &= (1u << p.kernel_count) - 1u;
            }
        }
    } else if (row >= 0 && row < n_out) {
        const int begin = max(__ldg(p.row_offsets + row), 0);
        const int end = min(__ldg(p.row_offsets + row + 1), edge_total);
        for (int e0 = begin; e0 < end; e0 += 4) {
            int k[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                k[u] = e0 + u < end ? __ldg(p.kernel_ids + e0 + u) : -1;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (k[u] >= 0 && k[u] < p.kernel_count) {
                    mask |= 1u << k[u];
                }
            }
        }
    }
    mask = __reduce_or_sync(0xffffffffu, mask);
    if ((threadIdx.x & 31) == 0 && mask != 0) {
        atomicOr(&tile_mask, mask);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        p.tile_info[blockIdx.x] = make_int2(static_cast<int>(tile_mask), 0);
    }
}

// pass 1b, relations of more than kSelfScanTiles tiles only: exclusive scan of the vectors
// per tile (one block); the entry after the last tile receives the vector total
__global__ void __launch_bounds__(1024) plan_scan_kernel(int2* tile_info, int num_tiles) {
    __shared__ int warp_totals[32];
    __shared__ int carry;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry = 0;
    }
    __syncthreads();
    for (int first = 0; first < num_tiles; first += 1024) {
        const int tile = first + threadIdx.x;
        int2 info = make_int2(0, 0);
        if (tile < num_tiles) {
            info = tile_info[tile];
        }
        int wtotal;
        const int prefix = warp_exclusive_scan(__popc(static_cast<uint32_t>(info.x)), wtotal);
        if (lane == 0) {
            warp_totals[warp] = wtotal;
        }
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; ++w) {
            before += warp_totals[w];
        }
        if (tile < num_tiles) {
            tile_info[tile] = make_int2(info.x, before + prefix);
        }
        __syncthreads();
        if (threadIdx.x == 1023) {
            carry = before + prefix + __popc(static_cast<uint32_t>(info.x));
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        tile_info[num_tiles].y = carry;   // .x (tiles in use) comes from plan_order_kernel
    }
}

// pass 1c: tile_order, a stable counting sort of the tiles by 32 - popcount(mask) (one block:
// its 32 warps take contiguous runs of tiles, count per warp, scan over (key, warp), place),
// and the number of tiles whose mask is not empty into the closing entry.
constexpr int kOrderKeys = 33;

__global__ void __launch_bounds__(1024) plan_order_kernel(
    const int2* tile_info, int num_tiles, int32_t* tile_order, int2* closing
) {
    __shared__ int start[kOrderKeys][32];   // counts, then where (key, warp) starts
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kOrderKeys * 32; i += 1024) {
        (&start[0][0])[i] = 0;
    }
    __syncthreads();
    const int run = (num_tiles + 31) / 32;
    const int first = warp * run;
    const int last = min(first + run, num_tiles);
    for (int t0 = first; t0 < last; t0 += 32) {
        const int t = t0 + lane;
        const int key = t < last ? 32 - __popc(static_cast<uint32_t>(__ldg(&tile_info[t].x))) : -1 - lane;
        const unsigned peers = __match_any_sync(0xffffffffu, key);
        if (key >= 0 && (peers & lanemask_lt()) == 0) {
            start[key][warp] += __popc(peers);
        }
        __syncwarp();
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int key = 0; key < kOrderKeys; ++key) {
            int total;
            const int count = start[key][lane];
            const int before = warp_exclusive_scan(count, total);
            start[key][lane] = carry + before;
            if (key == kOrderKeys - 1 && lane == 0) {
                closing->x = carry;   // tiles with at least one offset: everything before key 32
            }
            carry += total;
        }
    }
    __syncthreads();
    for (int t0 = first; t0 < last; t0 += 32) {
        const int t = t0 + lane;
        const int key = t < last ? 32 - __popc(static_cast<uint32_t>(__ldg(&tile_info[t].x))) : -1 - lane;
        const unsigned peers = __match_any_sync(0xffffffffu, key);
        const int rank = __popc(peers & lanemask_lt());
        if (key >= 0) {
            tile_order[start[key][warp] + rank] = t;
        }
        __syncwarp();
        if (key >= 0 && rank == 0) {
            start[key][warp] += __popc(peers);
        }
        __syncwarp();
    }
}

// pass 2: the row vectors. A block first finds where its tile's vectors start: the number
// of offsets the tiles before it use. Up to kSelfScanTiles tiles it adds up their masks'
// population counts itself (a few KB from L2, rather than wait for a one-block scan kernel),
// records the sum in tile_info[tile].y for the convolution, and the last tile also writes
// the vector total into the closing entry; beyond that size, where every block reading
// every mask before it would cost more than the scan, plan_scan_kernel has left both in
// place. Thread t owns vector slot t, that is tile row (t % 8) * 32 + t / 8: the lanes of a
// warp then write 32 consecutive entries of a vector (one 128-byte line) instead of 32
// entries that lie 32 bytes apart.
__global__ void __launch_bounds__(kPlanTileRows) plan_fill_kernel(PlanBuildParams p) {
    __shared__ int warp_before[kPlanTileRows / 32];
    const int n_out = clamp_count(p.counts + 1, p.out_capacity);
    const int edge_total = clamp_count(p.counts, p.edge_capacity);
    const int tile = blockIdx.x;
    const uint32_t mask = static_cast<uint32_t>(p.tile_info[tile].x);
    const int present = __popc(mask);
    // masks live in the .x words; the .y words are being written by the other blocks
    const bool closing = tile == p.num_tiles - 1;
    int before = 0;
    for (int t = threadIdx.x; t < tile && !p.prescanned; t += kPlanTileRows) {
        before += __popc(static_cast<uint32_t>(__ldg(&p.tile_info[t].x)));
    }
    before = warp_sum(before);
    if ((threadIdx.x & 31) == 0) {
        warp_before[threadIdx.x >> 5] = before;
    }
    __syncthreads();
    before = 0;
#pragma unroll
    for (int w = 0; w < kPlanTileRows / 32; ++w) {
        before += warp_before[w];
    }
    if (p.prescanned) {
        before = p.tile_info[tile].y;
    } else if (threadIdx.x == 0) {
        p.tile_info[tile].y = before;
        if (closing) {
            p.tile_info[p.num_tiles].y = before + present;   // .x comes from plan_order_kernel
        }
    }
    const int2 info = make_int2(static_cast<int>(mask), before);
    const int slot = threadIdx.x;
    const int r = (slot & 7) * 32 + (slot >> 3);   // plan_slot(r) == slot
    int32_t* mine = p.vectors + static_cast<size_t>(info.y) * kPlanTileRows + slot;
    for (int o = 0; o < present; ++o) {
        mine[static_cast<size_t>(o) * kPlanTileRows] = -1;
    }
    const int row = plan_row(p, blockIdx.x * kPlanTileRows + r);
    if (row >= 0 && row < n_out) {
        const int begin = max(__ldg(p.row_offsets + row), 0);
        const int end = min(__ldg(p.row_offsets + row + 1), edge_total);
        // four edges per step: their loads are independent and overlap
        for (int e0 = begin; e0 < end; e0 += 4) {
            int k[4], in_row[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const bool live = e0 + u < end;
                k[u] = live ? __ldg(p.kernel_ids + e0 + u) : -1;
                in_row[u] = live ? __ldg(p.in_rows + e0 + u) : -1;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (in_row[u] < 0 || k[u] < 0) {
                    continue;
                }
                if (in_row[u] >= p.in_capacity || k[u] >= p.kernel_count) {
                    raise_status(p.status, LAT_STATUS_BAD_INDEX);
                    continue;
                }
                const int o = __popc(mask & ((1u << k[u]) - 1u));
                mine[static_cast<size_t>(o) * kPlanTileRows] = in_row[u];
            }
        }
    }
}

// the plan of the identity relation (output row i reads input row i at the only offset):
// every tile uses offset 0 and its row vector is the tile's own rows
__global__ void __launch_bounds__(kPlanTileRows) identity_plan_kernel(int rows, int num_tiles, int2* tile_info,
                                                                    int32_t* tile_order, int32_t* vectors) {
    const int tile = blockIdx.x;
    const int row = tile * kPlanTileRows + threadIdx.x;
    vectors[static_cast<size_t>(tile) * kPlanTileRows + plan_slot(threadIdx.x)] = row < rows ? row : -1;
    if (threadIdx.x == 0) {
        tile_info[tile] = make_int2(1, tile);
        tile_order[tile] = tile;
        if (tile == 0) {
            tile_info[num_tiles] = make_int2(num_tiles, num_tiles);
        }
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_conv_plan_bytes(int32_t out_capacity, int32_t kernel_count) {
    const size_t tiles = static_cast<size_t>(plan_tiles(out_capacity));
    return plan_vectors_offset(static_cast<int>(tiles)) +
           tiles * static_cast<size_t>(std::max(kernel_count, 1)) * kPlanTileRows * sizeof(int32_t);
}

int lat_build_identity_conv_plan(int32_t rows, void* plan, size_t plan_bytes, void* stream_ptr) {
    LAT_REQUIRE(rows >= 0, "rows must be non-negative.");
    LAT_REQUIRE(plan != nullptr && reinterpret_cast<uintptr_t>(plan) % 16 == 0,
                "plan must be a 16-byte aligned device buffer.");
    LAT_REQUIRE(plan_bytes >= lat_conv_plan_bytes(rows, 1), "plan buffer is smaller than lat_conv_plan_bytes.");
    if (rows == 0) {
        return LAT_OK;
    }
    const int tiles = plan_tiles(rows);
    identity_plan_kernel<<<tiles, kPlanTileRows, 0, as_stream(stream_ptr)>>>(
        rows, tiles, static_cast<int2*>(plan),
        reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_info_bytes(tiles)),
        reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_vectors_offset(tiles)));
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_build_conv_plan(
    const int32_t* in_rows, const int32_t* kernel_ids, int32_t edge_capacity,
    const int32_t* counts, const int32_t* row_offsets, int32_t in_capacity,
    int32_t out_capacity, int32_t kernel_count, const int32_t* row_order, const int32_t* row_masks,
    void* plan, size_t plan_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(out_capacity >= 0 && edge_capacity >= 0 && in_capacity >= 0,
                "capacities must be non-negative.");
    LAT_REQUIRE(kernel_count >= 1 && kernel_count <= 32,
                "the gather plan serves kernels of at most 32 offsets.");
    LAT_REQUIRE(counts != nullptr && row_offsets != nullptr, "counts and row_offsets are required.");
    LAT_REQUIRE((in_rows != nullptr && kernel_ids != nullptr) || edge_capacity == 0,
                "in_rows and kernel_ids are required.");
    LAT_REQUIRE(plan != nullptr && reinterpret_cast<uintptr_t>(plan) % 16 == 0,
                "plan must be a 16-byte aligned device buffer.");
    LAT_REQUIRE(plan_bytes >= lat_conv_plan_bytes(out_capacity, kernel_count),
                "plan buffer is smaller than lat_conv_plan_bytes.");
    if (out_capacity == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    PlanBuildParams p{};
    p.in_rows = in_rows;
    p.kernel_ids = kernel_ids;
    p.row_offsets = row_offsets;
    p.counts = counts;
    p.row_order = row_order;
    p.row_masks = row_masks;
    p.edge_capacity = edge_capacity;
    p.in_capacity = in_capacity;
    p.out_capacity = out_capacity;
    p.kernel_count = kernel_count;
    p.num_tiles = plan_tiles(out_capacity);
    p.prescanned = p.num_tiles > kSelfScanTiles ? 1 : 0;
    p.tile_info = static_cast<int2*>(plan);
    p.tile_order = reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_info_bytes(p.num_tiles));
    p.vectors = reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_vectors_offset(p.num_tiles));
    p.status = status;
    plan_mask_kernel<<<p.num_tiles, kPlanTileRows, 0, stream>>>(p);
    LAT_LAUNCH_CHECK();
    plan_order_kernel<<<1, 1024, 0, stream>>>(p.tile_info, p.num_tiles, p.tile_order,
                                              p.tile_info + p.num_tiles);
    LAT_LAUNCH_CHECK();
    if (p.prescanned) {
        plan_scan_kernel<<<1, 1024, 0, stream>>>(p.tile_info, p.num_tiles);
        LAT_LAUNCH_CHECK();
    }
    plan_fill_kernel<<<p.num_tiles, kPlanTileRows, 0, stream>>>(p);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"
