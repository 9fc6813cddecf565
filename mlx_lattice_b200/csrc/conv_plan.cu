// Gather plan of the tensor-core convolution for one kernel relation.
//
// The output rows, taken through an optional permutation, are cut into 256-row tiles.
// For every tile the plan holds
//   tile_info[tile] = (mask, base): the kernel offsets any row of the tile uses, and the
//                     index of the tile's first row vector;
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

struct PlanBuildParams {
    const int32_t* in_rows;
    const int32_t* kernel_ids;
    const int32_t* row_offsets;
    const int32_t* counts;
    const int32_t* row_order;
    int edge_capacity;
    int in_capacity;
    int out_capacity;
    int kernel_count;
    int num_tiles;
    int2* tile_info;
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

// One block per tile, tiles taken in ticket order. The block reads its rows' edges once
// for the tile's offset mask, learns the index of its first row vector from a decoupled
// look-back over the tiles before it (it publishes its own vector count, then one warp
// sums its predecessors' counts 32 at a time until it meets one that knows its prefix;
// every wait is clock-bounded), and writes its row vectors from a second read of the
// same edges (cache-hot).
constexpr unsigned long long kPlanAggregate = 1ull << 62;
constexpr unsigned long long kPlanPrefix = 2ull << 62;
constexpr unsigned long long kPlanValueMask = (1ull << 62) - 1;
constexpr long long kPlanLookbackBudgetCycles = 4000000000LL;  // about two seconds

__global__ void __launch_bounds__(kPlanTileRows) plan_single_pass_kernel(
    PlanBuildParams p, unsigned long long* tile_status, int* ticket
) {
    __shared__ uint32_t tile_mask;
    __shared__ int s_tile;
    __shared__ int s_base;
    __shared__ int s_failed;
    if (threadIdx.x == 0) {
        s_tile = atomicAdd(ticket, 1);
        tile_mask = 0;
        s_failed = 0;
    }
    __syncthreads();
    const int tile = s_tile;
    if (tile >= p.num_tiles) {
        return;
    }
    const int lane = threadIdx.x & 31;
    const int n_out = clamp_count(p.counts + 1, p.out_capacity);
    const int edge_total = clamp_count(p.counts, p.edge_capacity);
    const int r = threadIdx.x;
    const int row = plan_row(p, tile * kPlanTileRows + r);
    int begin = 0, end = 0;
    uint32_t mask = 0;
    if (row >= 0 && row < n_out) {
        begin = max(__ldg(p.row_offsets + row), 0);
        end = min(__ldg(p.row_offsets + row + 1), edge_total);
        for (int e = begin; e < end; ++e) {
            const int k = __ldg(p.kernel_ids + e);
            const int in_row = __ldg(p.in_rows + e);
            if (in_row >= 0 && in_row < p.in_capacity && k >= 0 && k < p.kernel_count) {
                mask |= 1u << k;
            }
        }
    }
    mask = __reduce_or_sync(0xffffffffu, mask);
    if (lane == 0 && mask != 0) {
        atomicOr(&tile_mask, mask);
    }
    __syncthreads();
    const uint32_t used = tile_mask;
    const int present = __popc(used);
    if (threadIdx.x < 32) {
        volatile unsigned long long* status = tile_status;
        long long exclusive = 0;
        bool failed = false;
        if (tile > 0) {
            if (lane == 0) {
                status[tile] = kPlanAggregate | static_cast<unsigned long long>(present);
            }
            const long long start = clock64();
            int top = tile - 1;
            while (true) {
                const int t = top - lane;
                unsigned long long v = 2ull << 62;  // before tile 0: a prefix of zero
                if (t >= 0) {
                    v = status[t];
                }
                const unsigned ready = __ballot_sync(0xffffffffu, v != 0);
                const unsigned prefix = __ballot_sync(0xffffffffu, (v >> 63) != 0);
                const int nearest = prefix != 0 ? __ffs(prefix) - 1 : 31;
                const unsigned need = nearest >= 31 ? 0xffffffffu : ((2u << nearest) - 1u);
                if ((ready & need) != need) {
                    if (clock64() - start > kPlanLookbackBudgetCycles) {
                        failed = true;
                        break;
                    }
                    continue;
                }
                long long part = lane <= nearest ? static_cast<long long>(v & kPlanValueMask) : 0;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    part += __shfl_xor_sync(0xffffffffu, part, d);
                }
                exclusive += part;
                if (prefix != 0) {
                    break;
                }
                top -= 32;
            }
        }
        if (lane == 0) {
            if (failed) {
                s_failed = 1;
                raise_status(p.status, LAT_STATUS_WAIT_TIMEOUT);
            } else {
                status[tile] = kPlanPrefix | static_cast<unsigned long long>(exclusive + present);
                p.tile_info[tile] = make_int2(static_cast<int>(used), static_cast<int>(exclusive));
                if (used != 0) {
                    atomicMax(&p.tile_info[p.num_tiles].x, tile + 1);
                }
                if (tile == p.num_tiles - 1) {
                    p.tile_info[p.num_tiles].y = static_cast<int>(exclusive + present);
                }
            }
            s_base = static_cast<int>(exclusive);
        }
    }
    __syncthreads();
    if (s_failed) {
        return;
    }
    int32_t* mine = p.vectors + static_cast<size_t>(s_base) * kPlanTileRows + plan_slot(r);
    for (int o = 0; o < present; ++o) {
        mine[static_cast<size_t>(o) * kPlanTileRows] = -1;
    }
    for (int e = begin; e < end; ++e) {
        const int k = __ldg(p.kernel_ids + e);
        const int in_row = __ldg(p.in_rows + e);
        if (in_row < 0 || k < 0) {
            continue;
        }
        if (in_row >= p.in_capacity || k >= p.kernel_count) {
            raise_status(p.status, LAT_STATUS_BAD_INDEX);
            continue;
        }
        const int o = __popc(used & ((1u << k) - 1u));
        mine[static_cast<size_t>(o) * kPlanTileRows] = in_row;
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_conv_plan_bytes(int32_t out_capacity, int32_t kernel_count) {
    const size_t tiles = static_cast<size_t>(plan_tiles(out_capacity));
    return plan_info_bytes(static_cast<int>(tiles)) +
           tiles * static_cast<size_t>(std::max(kernel_count, 1)) * kPlanTileRows * sizeof(int32_t);
}

int lat_build_conv_plan(
    const int32_t* in_rows, const int32_t* kernel_ids, int32_t edge_capacity,
    const int32_t* counts, const int32_t* row_offsets, int32_t in_capacity,
    int32_t out_capacity, int32_t kernel_count, const int32_t* row_order,
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
    p.edge_capacity = edge_capacity;
    p.in_capacity = in_capacity;
    p.out_capacity = out_capacity;
    p.kernel_count = kernel_count;
    p.num_tiles = plan_tiles(out_capacity);
    p.tile_info = static_cast<int2*>(plan);
    p.vectors = reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_info_bytes(p.num_tiles));
    p.status = status;
    // the look-back words, the ticket and the trailing tile_info entry start at zero
    char* scratch = static_cast<char*>(plan) + plan_tile_info_bytes(p.num_tiles);
    unsigned long long* tile_status = reinterpret_cast<unsigned long long*>(scratch);
    int* ticket = reinterpret_cast<int*>(tile_status + p.num_tiles);
    LAT_CUDA_CHECK(cudaMemsetAsync(scratch, 0, sizeof(unsigned long long) * (p.num_tiles + 1), stream));
    LAT_CUDA_CHECK(cudaMemsetAsync(p.tile_info + p.num_tiles, 0, sizeof(int2), stream));
    plan_single_pass_kernel<<<p.num_tiles, kPlanTileRows, 0, stream>>>(p, tile_status, ticket);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"
