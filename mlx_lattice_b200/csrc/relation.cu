// Coordinate hash, output-support generation and kernel-map construction.
//
// Pipeline of one map build (all on the caller's stream, no host read-back):
//   1. table_clear + insert_rows       first-row-wins table of the active inputs
//   2. (strided only) insert by floor(coord/stride), mark winners, stable compact
//      -> output support in first-seen order
//   3. map_count   one warp per output row, lane = kernel offset: probe, ballot the
//                  hits into a row mask, reduce per-block edge totals and per-block
//                  per-offset totals
//   4. scan_blocks exclusive scan of the block totals (and, per offset, of the
//                  per-block offset totals) -> E and the per-offset list starts
//   5. map_fill    same warp/lane layout: local scan of the mask popcounts gives each
//                  row's first edge, hit lanes re-probe and write (in, out, k) in
//                  (out asc, k asc) order plus the per-offset pair lists
// The order of the emitted edges is the reference's (out row ascending, kernel id
// ascending; coordinates/cpu/relation_build_detail.h:19-34).
#include <algorithm>
#include <cstdlib>

#include <type_traits>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kBlockThreads = 256;
constexpr int kWarpsPerBlock = kBlockThreads / 32;
constexpr int kRowsPerBlock = kBlockThreads;  // 32 rows per warp
constexpr int kMaxMaskWords = 11;             // kernel volume <= 352 (7x7x7 = 343)

enum class MapRule : int {
    Forward = 0,            // cand = out*stride + off - pad
    TransposedGather = 1,   // cand = (out + pad - off) / stride when divisible
};

struct MapParams {
    const int32_t* coords;        // source coords
    const Slot* table;            // source table
    uint32_t table_mask;
    const int32_t* out_coords;    // coordinates of the output rows
    const int32_t* out_count_ptr; // device count of output rows (already clamped source)
    int out_capacity;             // rows the grid covers
    int out_count_cap;            // clamp for *out_count_ptr
    KernelGeometry geo;
    int sx, sy, sz, px, py, pz;
    int rule;
    int words;
    int32_t* masks;               // [out_capacity, words]
    int32_t* block_sums;          // [nblocks]
    int32_t* block_hist;          // [nblocks, K] or nullptr
    // fill outputs
    int32_t* in_rows;
    int32_t* out_rows;
    int32_t* kernel_ids;
    int32_t* row_offsets;
    int32_t* counts;
    int32_t* kernel_row_offsets;  // optional
    int32_t* kernel_edge_ids;     // optional
    const int32_t* hist_totals;   // [K] totals per offset (after scan)
    int tail_is_total;            // rows >= n_out get E (target maps) instead of 0
    int edge_capacity;
    int32_t* status;
    long long wait_budget;        // clock budget of the look-back wait
};

__global__ void fill_i32_kernel(int32_t* data, size_t count, int value) {
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (; i < count; i += stride) {
        data[i] = value;
    }
}

// insert rows [0, active) keyed by their own coordinate
__global__ void insert_rows_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, Slot* table,
    uint32_t mask, int32_t* status, int flag_duplicates
) {
    int active = clamp_count(active_ptr, rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= active) {
        return;
    }
    PlainKey key_of{coords};
    bool dup = false;
    if (!table_insert(table, mask, row, key_of(row), key_of, &dup)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
    if (dup && flag_duplicates) {
        raise_status(status, LAT_STATUS_DUPLICATE_INPUT);
    }
}

// insert all rows [0, rows) regardless of an active count
__global__ void insert_all_rows_kernel(
    const int32_t* coords, int rows, Slot* table, uint32_t mask, int32_t* status
) {
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) {
        return;
    }
    PlainKey key_of{coords};
    if (!table_insert(table, mask, row, key_of(row), key_of, nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

__global__ void insert_downsampled_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, int sx, int sy, int sz,
    Slot* table, uint32_t mask, int32_t* status
) {
    int active = active_ptr ? clamp_count(active_ptr, rows) : rows;
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= active) {
        return;
    }
    DownsampledKey key_of{coords, sx, sy, sz};
    if (!table_insert(table, mask, row, key_of(row), key_of, nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

// Block-wide exclusive scan of one int per thread (blockDim = kBlockThreads).
__device__ __forceinline__ int block_exclusive_scan(int value, int& block_total) {
    __shared__ int warp_totals[kWarpsPerBlock];
    __shared__ int total_shared;
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int wtotal;
    int prefix = warp_exclusive_scan(value, wtotal);
    if (lane == 31) {
        warp_totals[warp] = wtotal;
    }
    __syncthreads();
    if (warp == 0) {
        int v = lane < kWarpsPerBlock ? warp_totals[lane] : 0;
        int t;
        int p = warp_exclusive_scan(v, t);
        if (lane < kWarpsPerBlock) {
            warp_totals[lane] = p;
        }
        if (lane == 0) {
            total_shared = t;
        }
    }
    __syncthreads();
    block_total = total_shared;
    int out = prefix + warp_totals[warp];
    __syncthreads();
    return out;
}

// Consumers of per-block totals add them up themselves up to this many blocks (1 M rows);
// above it scan_blocks_kernel runs first, because every block reading every total before it
// grows with the square of the block count.
constexpr int kSelfScanBlocks = 4096;

// What a scan over the per-block totals would give block `block`: the sum of the totals of
// the blocks before it, and the sum of all of them. Every block of a consumer kernel adds
// them up itself (a few KB from L2) instead of waiting for a one-block scan kernel between
// the counting kernel and itself. Call with the whole block (blockDim = kBlockThreads).
__device__ __forceinline__ void block_prefix_of(
    const int32_t* sums, int count, int block, int& before, int& total
) {
    __shared__ int partial_before[kWarpsPerBlock];
    __shared__ int partial_total[kWarpsPerBlock];
    int b = 0, t = 0;
    for (int i = threadIdx.x; i < count; i += kBlockThreads) {
        const int v = __ldg(sums + i);
        t += v;
        b += i < block ? v : 0;
    }
    b = warp_sum(b);
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) {
        partial_before[threadIdx.x >> 5] = b;
        partial_total[threadIdx.x >> 5] = t;
    }
    __syncthreads();
    before = 0;
    total = 0;
#pragma unroll
    for (int w = 0; w < kWarpsPerBlock; ++w) {
        before += partial_before[w];
        total += partial_total[w];
    }
    __syncthreads();
}

// winners of the downsampled table -> per-block counts
__global__ void mark_winners_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, int sx, int sy, int sz,
    const Slot* table, uint32_t mask, int32_t* block_sums
) {
    int active = active_ptr ? clamp_count(active_ptr, rows) : rows;
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    DownsampledKey key_of{coords, sx, sy, sz};
    int win = 0;
    if (row < active) {
        win = table_find(table, mask, key_of(row), key_of) == row;
    }
    int total;
    block_exclusive_scan(win, total);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = total;
    }
}

// Exclusive scan of `count` block sums in place (single block), total to *total_out.
// Extra blocks (blockIdx.x >= 1) scan column (blockIdx.x - 1) of a [count, columns]
// histogram in place and leave the column totals in hist_totals.
__global__ void scan_blocks_kernel(
    int32_t* block_sums, int count, int32_t* total_out, int32_t* second_out,
    const int32_t* second_value_ptr, int second_cap,
    int32_t* hist, int columns, int32_t* hist_totals
) {
    int carry = 0;
    if (blockIdx.x == 0) {
        if (block_sums == nullptr) {
            return;
        }
        for (int base = 0; base < count; base += kBlockThreads) {
            int i = base + threadIdx.x;
            int v = i < count ? block_sums[i] : 0;
            int total;
            int p = block_exclusive_scan(v, total);
            if (i < count) {
                block_sums[i] = carry + p;
            }
            carry += total;
        }
        if (threadIdx.x == 0) {
            if (total_out != nullptr) {
                *total_out = carry;
            }
            if (second_out != nullptr && second_value_ptr != nullptr) {
                second_out[0] = clamp_count(second_value_ptr, second_cap);
            }
        }
        return;
    }
    int column = blockIdx.x - 1;
    for (int base = 0; base < count; base += kBlockThreads) {
        int i = base + threadIdx.x;
        int v = i < count ? hist[static_cast<size_t>(i) * columns + column] : 0;
        int total;
        int p = block_exclusive_scan(v, total);
        if (i < count) {
            hist[static_cast<size_t>(i) * columns + column] = carry + p;
        }
        carry += total;
    }
    if (threadIdx.x == 0) {
        hist_totals[column] = carry;
    }
}

// stable compaction of the winners: out_coords in first-seen order; block_sums are the
// per-block winner counts of mark_winners_kernel, *count_out receives their total
__global__ void compact_winners_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, int sx, int sy, int sz,
    const Slot* table, uint32_t mask, const int32_t* block_sums, int prescanned, int32_t* count_out,
    int32_t* out_coords, int out_capacity, int32_t* status
) {
    // prescanned: scan_blocks_kernel has turned block_sums into offsets and written the total
    int before, all;
    if (prescanned) {
        before = block_sums[blockIdx.x];
    } else {
        block_prefix_of(block_sums, gridDim.x, blockIdx.x, before, all);
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            *count_out = all;
        }
    }
    int active = active_ptr ? clamp_count(active_ptr, rows) : rows;
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    DownsampledKey key_of{coords, sx, sy, sz};
    int win = 0;
    Coord key{0, 0, 0, 0};
    if (row < active) {
        key = key_of(row);
        win = table_find(table, mask, key, key_of) == row;
    }
    int total;
    int pos = block_exclusive_scan(win, total) + before;
    if (win) {
        if (pos < out_capacity) {
            store_coord(out_coords, pos, key);
        } else {
            raise_status(status, LAT_STATUS_EDGE_OVERFLOW);
        }
    }
}

// (ox, oy, oz) is the spatial offset of the lane's kernel id, computed once per pass
// (the integer divisions in KernelGeometry::offset are too slow for the row loop)
__device__ __forceinline__ bool candidate_of(
    const MapParams& p, Coord out, int ox, int oy, int oz, Coord& cand
) {
    if (p.rule == static_cast<int>(MapRule::Forward)) {
        cand = {out.b, out.x * p.sx + ox - p.px, out.y * p.sy + oy - p.py,
                out.z * p.sz + oz - p.pz};
        return true;
    }
    int tx = out.x + p.px - ox, ty = out.y + p.py - oy, tz = out.z + p.pz - oz;
    int qx = floor_div(tx, p.sx), qy = floor_div(ty, p.sy), qz = floor_div(tz, p.sz);
    if (qx * p.sx != tx || qy * p.sy != ty || qz * p.sz != tz) {
        return false;
    }
    cand = {out.b, qx, qy, qz};
    return true;
}

// one warp per 32 output rows, lane = kernel offset (in passes of 32)
__global__ void __launch_bounds__(kBlockThreads) map_count_kernel(MapParams p) {
    extern __shared__ int smem_hist[];  // [kWarpsPerBlock][K] when block_hist
    __shared__ int warp_edges[kWarpsPerBlock];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int n_out = clamp_count(p.out_count_ptr, p.out_count_cap);
    int row0 = blockIdx.x * kRowsPerBlock + warp * 32;
    PlainKey key_of{p.coords};
    int K = p.geo.volume;

    Coord mine{0, 0, 0, 0};
    if (row0 + lane < n_out) {
        mine = load_coord(p.out_coords, row0 + lane);
    }
    int edges = 0;
    for (int pass = 0; pass < p.words; ++pass) {
        int k = pass * 32 + lane;
        int k_hits = 0;
        int ox = 0, oy = 0, oz = 0;
        if (k < K) {
            p.geo.offset(k, ox, oy, oz);
        }
        for (int j = 0; j < 32; ++j) {
            int row = row0 + j;
            if (row >= n_out) {
                break;
            }
            Coord out{__shfl_sync(0xffffffffu, mine.b, j), __shfl_sync(0xffffffffu, mine.x, j),
                      __shfl_sync(0xffffffffu, mine.y, j), __shfl_sync(0xffffffffu, mine.z, j)};
            bool hit = false;
            Coord cand;
            if (k < K && candidate_of(p, out, ox, oy, oz, cand)) {
                hit = table_find(p.table, p.table_mask, cand, key_of) >= 0;
            }
            unsigned m = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) {
                p.masks[static_cast<size_t>(row) * p.words + pass] = static_cast<int>(m);
                edges += __popc(m);
            }
            k_hits += hit;
        }
        if (p.block_hist != nullptr && k < K) {
            smem_hist[warp * K + k] = k_hits;
        }
    }
    if (lane == 0) {
        warp_edges[warp] = edges;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int w = 0; w < kWarpsPerBlock; ++w) {
            total += warp_edges[w];
        }
        p.block_sums[blockIdx.x] = total;
    }
    if (p.block_hist != nullptr) {
        for (int k = threadIdx.x; k < K; k += kBlockThreads) {
            int total = 0;
            for (int w = 0; w < kWarpsPerBlock; ++w) {
                total += smem_hist[w * K + k];
            }
            p.block_hist[static_cast<size_t>(blockIdx.x) * K + k] = total;
        }
    }
}

__global__ void __launch_bounds__(kBlockThreads) map_fill_kernel(MapParams p) {
    extern __shared__ int smem_dyn[];  // [kWarpsPerBlock][K] per-warp list cursors
    __shared__ int warp_edge_base[kWarpsPerBlock];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int n_out = clamp_count(p.out_count_ptr, p.out_count_cap);
    int row0 = blockIdx.x * kRowsPerBlock + warp * 32;
    int my_row = row0 + lane;
    PlainKey key_of{p.coords};
    int K = p.geo.volume;
    bool lists = p.kernel_edge_ids != nullptr;
    int total_edges = __ldg(p.counts);

    int my_masks[kMaxMaskWords];
    int my_degree = 0;
#pragma unroll
    for (int w = 0; w < kMaxMaskWords; ++w) {
        my_masks[w] = 0;
        if (w < p.words && my_row < n_out) {
            my_masks[w] = p.masks[static_cast<size_t>(my_row) * p.words + w];
            my_degree += __popc(static_cast<unsigned>(my_masks[w]));
        }
    }
    int wtotal;
    int my_start = warp_exclusive_scan(my_degree, wtotal);
    if (lane == 0) {
        warp_edge_base[warp] = wtotal;
    }
    int* warp_kbase = smem_dyn;           // [kWarpsPerBlock][K]
    if (lists) {
        // per-offset hit counts of this warp's 32 rows (lane = offset)
        for (int pass = 0; pass < p.words; ++pass) {
            int k = pass * 32 + lane;
            int count = 0;
            for (int j = 0; j < 32; ++j) {
                int m = 0;
#pragma unroll
                for (int w = 0; w < kMaxMaskWords; ++w) {
                    if (w == pass) {
                        m = __shfl_sync(0xffffffffu, my_masks[w], j);
                    }
                }
                count += (static_cast<unsigned>(m) >> lane) & 1u;
            }
            if (k < K) {
                warp_kbase[warp * K + k] = count;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = p.block_sums[blockIdx.x];
        for (int w = 0; w < kWarpsPerBlock; ++w) {
            int t = warp_edge_base[w];
            warp_edge_base[w] = run;
            run += t;
        }
    }
    if (lists) {
        for (int k = threadIdx.x; k < K; k += kBlockThreads) {
            // start of list k = totals of the lists before it
            int start = 0;
            for (int q = 0; q < k; ++q) {
                start += __ldg(p.hist_totals + q);
            }
            if (blockIdx.x == 0) {
                p.kernel_row_offsets[k] = start;
                if (k == K - 1) {
                    p.kernel_row_offsets[K] = start + __ldg(p.hist_totals + k);
                }
            }
            int run = start + p.block_hist[static_cast<size_t>(blockIdx.x) * K + k];
            for (int w = 0; w < kWarpsPerBlock; ++w) {
                int t = warp_kbase[w * K + k];
                warp_kbase[w * K + k] = run;
                run += t;
            }
        }
    }
    __syncthreads();
    my_start += warp_edge_base[warp];
    if (my_row < n_out) {
        p.row_offsets[my_row] = my_start;
    } else if (my_row <= p.out_capacity) {
        if (my_row == n_out || p.tail_is_total) {
            p.row_offsets[my_row] = total_edges;
        }
    }

    for (int pass = 0; pass < p.words; ++pass) {
        int k = pass * 32 + lane;
        int k_cursor = (lists && k < K) ? warp_kbase[warp * K + k] : 0;
        int ox = 0, oy = 0, oz = 0;
        if (k < K) {
            p.geo.offset(k, ox, oy, oz);
        }
        for (int j = 0; j < 32; ++j) {
            int row = row0 + j;
            if (row >= n_out) {
                break;
            }
            int m = 0;
            int before = 0;  // hits of this row in earlier words
#pragma unroll
            for (int w = 0; w < kMaxMaskWords; ++w) {
                int v = (w <= pass) ? __shfl_sync(0xffffffffu, my_masks[w], j) : 0;
                if (w == pass) {
                    m = v;
                } else if (w < pass) {
                    before += __popc(static_cast<unsigned>(v));
                }
            }
            if (m == 0) {
                continue;
            }
            int start = __shfl_sync(0xffffffffu, my_start, j);
            bool hit = (static_cast<unsigned>(m) >> lane) & 1u;
            if (hit) {
                Coord out = load_coord(p.out_coords, row);
                Coord cand;
                candidate_of(p, out, ox, oy, oz, cand);
                int in_row = table_find(p.table, p.table_mask, cand, key_of);
                int pos = start + before + __popc(static_cast<unsigned>(m) & lanemask_lt());
                if (pos < p.edge_capacity) {
                    p.in_rows[pos] = in_row;
                    p.out_rows[pos] = row;
                    p.kernel_ids[pos] = k;
                    if (lists) {
                        p.kernel_edge_ids[k_cursor] = pos;
                    }
                } else {
                    raise_status(p.status, LAT_STATUS_EDGE_OVERFLOW);
                }
                ++k_cursor;
            }
        }
    }
}

// ---- single-pass kernel map (K <= 32) --------------------------------------------------
//
// One block per 256 output rows (tiles taken in ticket order), one warp per 32 rows.
//  1. probe, lane = output row: the K candidates of a row are K independent bucket reads,
//     scanned by tag only; the hit rows wait in shared memory. For the forward rule the
//     candidate is `row base + offset`, so its two linear hash forms are the row's forms
//     (computed once per row) plus a per-offset constant from shared memory.
//  2. verify, lane = output row: each tag hit is compared with the coordinate it stands
//     for; a false tag match (one in 2^32) falls back to the exact table lookup.
//  3. the block learns where its edges start from a decoupled look-back over the tiles
//     before it: it publishes its own edge count, then one warp sums its predecessors'
//     counts 32 tiles at a time until it meets one that already knows its prefix.
//  4. write, lane = output row: edges in (output row asc, kernel id asc) order.
constexpr unsigned long long kTileAggregate = 1ull << 62;
constexpr unsigned long long kTilePrefix = 2ull << 62;
constexpr unsigned long long kTileValueMask = (1ull << 62) - 1;

__global__ void __launch_bounds__(kBlockThreads, 5) map_single_pass_kernel(
    MapParams p, unsigned long long* tile_status, int* ticket, int num_tiles
) {
    extern __shared__ int s_hits[];            // [256][K]
    __shared__ int2 s_offset_hash[32];         // forward rule: linear hash forms of the offsets
    __shared__ int4 s_offset[32];              // kernel offsets by id
    __shared__ int s_tile;
    __shared__ int s_base;
    __shared__ int s_failed;
    __shared__ int warp_total[kWarpsPerBlock];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K = p.geo.volume;
    if (threadIdx.x == 0) {
        s_tile = atomicAdd(ticket, 1);
        s_failed = 0;
    }
    int ox = 0, oy = 0, oz = 0;
    if (lane < K) {
        p.geo.offset(lane, ox, oy, oz);
    }
    if (warp == 0) {
        s_offset[lane] = make_int4(ox, oy, oz, 0);
        uint32_t u_off, t_off;
        hash_linear(Coord{0, ox, oy, oz}, u_off, t_off);
        s_offset_hash[lane] = make_int2(static_cast<int>(u_off), static_cast<int>(t_off));
    }
    __syncthreads();
    const int tile = s_tile;
    if (tile >= num_tiles) {
        return;
    }
    const int n_out = clamp_count(p.out_count_ptr, p.out_count_cap);
    const int row0 = tile * kRowsPerBlock + warp * 32;
    const int my_row = row0 + lane;
    const bool forward = p.rule == static_cast<int>(MapRule::Forward);
    PlainKey key_of{p.coords};

    Coord mine{0, 0, 0, 0};
    if (my_row < n_out) {
        mine = load_coord(p.out_coords, my_row);
    }
    // 1. probe, lane = output row: K independent bucket reads per lane
    uint32_t u_row = 0, t_row = 0;  // linear hash forms of this row's base coordinate
    const int z_row = mine.z * p.sz - p.pz;
    if (forward) {
        hash_linear(Coord{mine.b, mine.x * p.sx - p.px, mine.y * p.sy - p.py, z_row}, u_row, t_row);
    }
    unsigned my_mask = 0;
    unsigned my_overflow = 0;  // offsets whose first bucket was full without a tag match
    int* warp_hits = s_hits + warp * 32 * K;
    int* my_hits = warp_hits + lane * K;
    const bool row_live = my_row < n_out;
    // Column probing: with the forward rule and a z extent of at most five voxels, the KZ
    // candidates of one (x, y) column of the footprint lie in at most two z-groups of the
    // table's hash, the group of the first and the group of the last: two bucket reads (one
    // when the groups coincide) answer the column.
    auto probe_columns = [&](auto kz_tag) {
        constexpr int KZ = decltype(kz_tag)::value;
        const int columns = K / KZ;
#pragma unroll 1
        for (int c = 0; c < columns; ++c) {
            const int k0 = c * KZ;
            const uint32_t u_col = u_row + static_cast<uint32_t>(s_offset_hash[k0].x);
            const int z_first = z_row + s_offset[k0].z;
            const int z_last = z_row + s_offset[k0 + KZ - 1].z;
            const uint32_t base_a =
                hash_finalize(u_col + hash_z_term(z_first)) & p.table_mask & ~(kBucketSlots - 1);
            const uint32_t base_b =
                hash_finalize(u_col + hash_z_term(z_last)) & p.table_mask & ~(kBucketSlots - 1);
            const bool two = (z_first >> kHashZShift) != (z_last >> kHashZShift);
            const Bucket a = load_bucket_if(p.table, base_a, row_live);
            const Bucket b = load_bucket_if(p.table, base_b, row_live && two);
#pragma unroll
            for (int j = 0; j < KZ; ++j) {
                const int k = k0 + j;
                const bool in_a = ((z_row + s_offset[k].z) >> kHashZShift) == (z_first >> kHashZShift);
                const uint32_t tag = t_row + static_cast<uint32_t>(s_offset_hash[k].y);
                const int found_a = scan_bucket_tags(a, tag);
                const int found_b = scan_bucket_tags(b, tag);
                const int found = row_live ? (in_a ? found_a : found_b) : -1;
                my_mask |= found >= 0 ? (1u << k) : 0u;
                my_overflow |= found == -2 ? (1u << k) : 0u;
                if (found >= 0) {
                    my_hits[k] = found;
                }
            }
        }
    };
    const int z_span = (p.geo.kz - 1) * p.geo.dz;
    if (row0 >= n_out) {
        // nothing to probe
    } else if (forward && z_span <= 4 && p.geo.kz == 3) {
        probe_columns(std::integral_constant<int, 3>{});
    } else if (forward && z_span <= 4 && p.geo.kz == 2) {
        probe_columns(std::integral_constant<int, 2>{});
    } else if (forward && p.geo.kz == 1) {
        probe_columns(std::integral_constant<int, 1>{});
    } else {
#pragma unroll 3
        for (int k = 0; k < K; ++k) {
            bool live = row_live;
            uint32_t index = 0, tag = 0;
            if (forward) {
                const int2 h = s_offset_hash[k];
                index = hash_finalize(u_row + static_cast<uint32_t>(h.x) + hash_z_term(z_row + s_offset[k].z));
                tag = t_row + static_cast<uint32_t>(h.y);
            } else if (live) {
                const int4 off = s_offset[k];
                Coord cand;
                live = candidate_of(p, mine, off.x, off.y, off.z, cand);
                hash_coord(cand, index, tag);
            }
            int found = -1;
            if (live) {
                const Bucket bucket = load_bucket(p.table, index & p.table_mask & ~(kBucketSlots - 1));
                found = scan_bucket_tags(bucket, tag);
            }
            my_mask |= found >= 0 ? (1u << k) : 0u;
            my_overflow |= found == -2 ? (1u << k) : 0u;
            if (found >= 0) {
                my_hits[k] = found;
            }
        }
    }
    __syncwarp();

    // 2. verify this lane's row, four hits at a time (their coordinate loads overlap)
    {
        unsigned bits = my_mask;
        while (bits != 0) {
            int ks[4];
            Coord got[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                ks[u] = bits != 0 ? __ffs(bits) - 1 : -1;
                bits &= bits - 1;   // 0 stays 0
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (ks[u] >= 0) {
                    got[u] = key_of(warp_hits[lane * K + ks[u]]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (ks[u] < 0) {
                    continue;
                }
                const int k = ks[u];
                const int4 off = s_offset[k];
                Coord expect;
                candidate_of(p, mine, off.x, off.y, off.z, expect);
                if (!(got[u] == expect)) {
                    const int exact = table_find(p.table, p.table_mask, expect, key_of);
                    if (exact >= 0) {
                        warp_hits[lane * K + k] = exact;
                    } else {
                        my_mask &= ~(1u << k);
                    }
                }
            }
        }
    }
    // candidates that ran past their first bucket take the exact lookup (rare at this
    // load factor), here rather than in the probe loop where one lane would hold up 32
    while (my_overflow != 0) {
        const int k = __ffs(my_overflow) - 1;
        my_overflow &= my_overflow - 1;
        const int4 off = s_offset[k];
        Coord expect;
        candidate_of(p, mine, off.x, off.y, off.z, expect);
        const int exact = table_find(p.table, p.table_mask, expect, key_of);
        if (exact >= 0) {
            warp_hits[lane * K + k] = exact;
            my_mask |= 1u << k;
        }
    }
    if (p.masks != nullptr && my_row < p.out_capacity) {
        p.masks[my_row] = static_cast<int>(my_mask);
    }

    // 3. where this tile's edges start
    int wtotal;
    int my_start = warp_exclusive_scan(__popc(my_mask), wtotal);
    if (lane == 0) {
        warp_total[warp] = wtotal;
    }
    __syncthreads();
    if (warp == 0) {
        int block_total;
        const int warp_start = warp_exclusive_scan(lane < kWarpsPerBlock ? warp_total[lane] : 0, block_total);
        if (lane < kWarpsPerBlock) {
            warp_total[lane] = warp_start;
        }
        volatile unsigned long long* status = tile_status;
        long long exclusive = 0;
        bool failed = false;
        if (tile > 0) {
            if (lane == 0) {
                status[tile] = kTileAggregate | static_cast<unsigned long long>(block_total);
            }
            const long long start = clock64();
            int top = tile - 1;  // nearest predecessor not summed yet
            while (true) {
                const int t = top - lane;
                unsigned long long v = 2ull << 62;  // before tile 0 stands a virtual tile with prefix 0
                if (t >= 0) {
                    v = status[t];
                }
                const unsigned ready = __ballot_sync(0xffffffffu, v != 0);
                const unsigned prefix = __ballot_sync(0xffffffffu, (v >> 63) != 0);
                const int nearest = prefix != 0 ? __ffs(prefix) - 1 : 31;
                const unsigned need = nearest >= 31 ? 0xffffffffu : ((2u << nearest) - 1u);
                if ((ready & need) != need) {
                    // the warp gives up as one (a lane left behind would hang the next ballot)
                    if (__any_sync(0xffffffffu, clock64() - start > p.wait_budget)) {
                        failed = true;
                        break;
                    }
                    continue;
                }
                long long part = lane <= nearest ? static_cast<long long>(v & kTileValueMask) : 0;
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
                status[tile] = kTilePrefix | static_cast<unsigned long long>(exclusive + block_total);
                if (tile == num_tiles - 1) {
                    p.counts[0] = static_cast<int>(exclusive + block_total);
                    p.counts[1] = n_out;
                }
            }
            s_base = static_cast<int>(exclusive);
        }
    }
    __syncthreads();
    if (s_failed) {
        return;
    }

    // 4. write this lane's row
    my_start += s_base + warp_total[warp];
    const int total_after = my_start + __popc(my_mask);  // == E for rows at and beyond n_out
    if (my_row < n_out) {
        p.row_offsets[my_row] = my_start;
    } else if (my_row <= p.out_capacity) {
        if (my_row == n_out || p.tail_is_total) {
            p.row_offsets[my_row] = total_after;
        }
    }
    if (total_after > p.edge_capacity) {
        if (my_mask != 0) {
            raise_status(p.status, LAT_STATUS_EDGE_OVERFLOW);
        }
    }
    if (wtotal <= 4 * 32) {
        // few edges per row: each lane walks its own row's hits
        unsigned bits = my_mask;
        int pos = my_start;
        while (bits != 0) {
            const int k = __ffs(bits) - 1;
            bits &= bits - 1;
            if (pos < p.edge_capacity) {
                p.in_rows[pos] = warp_hits[lane * K + k];
                p.out_rows[pos] = my_row;
                p.kernel_ids[pos] = k;
            }
            ++pos;
        }
    } else {
        // many edges per row: one row at a time, lane = kernel offset, contiguous stores
        for (int j = 0; j < 32; ++j) {
            const unsigned m = __shfl_sync(0xffffffffu, my_mask, j);
            const int start = __shfl_sync(0xffffffffu, my_start, j);
            if ((m >> lane) & 1u) {
                const int pos = start + __popc(m & lanemask_lt());
                if (pos < p.edge_capacity) {
                    p.in_rows[pos] = warp_hits[j * K + lane];
                    p.out_rows[pos] = row0 + j;
                    p.kernel_ids[pos] = lane;
                }
            }
        }
    }
}

// rows of the identity output support: a copy of the active input rows, zero after
__global__ void copy_active_coords_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, int32_t* out_coords
) {
    int active = clamp_count(active_ptr, rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) {
        return;
    }
    int4 v = make_int4(0, 0, 0, 0);
    if (row < active) {
        v = reinterpret_cast<const int4*>(coords)[row];
    }
    reinterpret_cast<int4*>(out_coords)[row] = v;
}

__global__ void store_clamped_kernel(const int32_t* src, int cap, int32_t* dst) {
    dst[0] = clamp_count(src, cap);
}

// closed-form transposed / generative map: edge e = in*K + k
__global__ void direct_transposed_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, KernelGeometry geo,
    int sx, int sy, int sz, int px, int py, int pz,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts
) {
    int active = clamp_count(active_ptr, rows);
    int K = geo.volume;
    long long capacity = static_cast<long long>(rows) * K;
    long long total = static_cast<long long>(active) * K;
    long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (e == 0) {
        counts[0] = static_cast<int>(total);
        counts[1] = static_cast<int>(total);
    }
    if (e > capacity) {
        return;
    }
    if (e == capacity) {
        row_offsets[e] = (e == total) ? static_cast<int>(total) : 0;
        return;
    }
    if (e < total) {
        int in_row = static_cast<int>(e / K);
        int k = static_cast<int>(e - static_cast<long long>(in_row) * K);
        int ox, oy, oz;
        geo.offset(k, ox, oy, oz);
        Coord c = load_coord(coords, in_row);
        in_rows[e] = in_row;
        out_rows[e] = static_cast<int>(e);
        kernel_ids[e] = k;
        row_offsets[e] = static_cast<int>(e);
        store_coord(out_coords, static_cast<int>(e),
                    {c.b, c.x * sx + ox - px, c.y * sy + oy - py, c.z * sz + oz - pz});
    } else {
        in_rows[e] = 0;
        out_rows[e] = 0;
        kernel_ids[e] = 0;
        row_offsets[e] = (e == total) ? static_cast<int>(total) : 0;
        store_coord(out_coords, static_cast<int>(e), {0, 0, 0, 0});
    }
}

// candidate outputs of the overlapping transposed map, id = in*K + k
struct TransposedCandidateKey {
    const int32_t* coords;
    KernelGeometry geo;
    int sx, sy, sz, px, py, pz;
    __device__ __forceinline__ Coord operator()(int id) const {
        int in_row = id / geo.volume;
        int k = id - in_row * geo.volume;
        int ox, oy, oz;
        geo.offset(k, ox, oy, oz);
        Coord c = load_coord(coords, in_row);
        return {c.b, c.x * sx + ox - px, c.y * sy + oy - py, c.z * sz + oz - pz};
    }
};

__global__ void insert_candidates_kernel(
    TransposedCandidateKey key_of, const int32_t* active_ptr, int rows, Slot* table,
    uint32_t mask, int32_t* status
) {
    int active = clamp_count(active_ptr, rows);
    long long total = static_cast<long long>(active) * key_of.geo.volume;
    long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (id >= total) {
        return;
    }
    if (!table_insert(table, mask, static_cast<int>(id), key_of(static_cast<int>(id)), key_of,
                      nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

__global__ void mark_candidate_winners_kernel(
    TransposedCandidateKey key_of, const int32_t* active_ptr, int rows, const Slot* table,
    uint32_t mask, int32_t* block_sums
) {
    int active = clamp_count(active_ptr, rows);
    long long total = static_cast<long long>(active) * key_of.geo.volume;
    long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    int win = 0;
    if (id < total) {
        win = table_find(table, mask, key_of(static_cast<int>(id)), key_of) ==
              static_cast<int>(id);
    }
    int t;
    block_exclusive_scan(win, t);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = t;
    }
}

__global__ void compact_candidates_kernel(
    TransposedCandidateKey key_of, const int32_t* active_ptr, int rows, const Slot* table,
    uint32_t mask, const int32_t* block_offsets, int32_t* out_coords, int out_capacity
) {
    int active = clamp_count(active_ptr, rows);
    long long total = static_cast<long long>(active) * key_of.geo.volume;
    long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    int win = 0;
    Coord key{0, 0, 0, 0};
    if (id < total) {
        key = key_of(static_cast<int>(id));
        win = table_find(table, mask, key, key_of) == static_cast<int>(id);
    }
    int t;
    int pos = block_exclusive_scan(win, t) + block_offsets[blockIdx.x];
    if (win && pos < out_capacity) {
        store_coord(out_coords, pos, key);
    }
}

// target-restricted transposed map of a kernel_size == stride conv
__global__ void target_transposed_count_kernel(
    const int32_t* coords, const Slot* table, uint32_t mask, const int32_t* target,
    const int32_t* target_active_ptr, int target_rows, int sx, int sy, int sz,
    int lox, int loy, int loz, int32_t* hit_rows, int32_t* block_sums
) {
    int active = clamp_count(target_active_ptr, target_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int hit = 0;
    if (row < active) {
        Coord t = load_coord(target, row);
        Coord parent{t.b, floor_div(t.x - lox, sx), floor_div(t.y - loy, sy),
                     floor_div(t.z - loz, sz)};
        int in_row = table_find(table, mask, parent, PlainKey{coords});
        hit = in_row >= 0;
        hit_rows[row] = in_row;
    }
    int total;
    block_exclusive_scan(hit, total);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = total;
    }
}

__global__ void target_transposed_fill_kernel(
    const int32_t* target, const int32_t* target_active_ptr, int target_rows,
    int sx, int sy, int sz, int lox, int loy, int loz,
    const int32_t* hit_rows, const int32_t* block_sums, int prescanned, int32_t* counts,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* row_masks
) {
    int active = clamp_count(target_active_ptr, target_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int in_row = -1;
    if (row < active) {
        in_row = hit_rows[row];
    }
    // block_sums: the per-block hit counts of target_transposed_count_kernel, or (prescanned)
    // what scan_blocks_kernel made of them, with the counts already written
    int before, edges;
    if (prescanned) {
        before = block_sums[blockIdx.x];
        edges = counts[0];
    } else {
        block_prefix_of(block_sums, gridDim.x, blockIdx.x, before, edges);
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            counts[0] = edges;
            counts[1] = active;
        }
    }
    int total;
    int pos = block_exclusive_scan(in_row >= 0, total) + before;
    if (row < active) {
        row_offsets[row] = pos;
        if (in_row >= 0) {
            Coord t = load_coord(target, row);
            int ox = t.x - lox - floor_div(t.x - lox, sx) * sx;
            int oy = t.y - loy - floor_div(t.y - loy, sy) * sy;
            int oz = t.z - loz - floor_div(t.z - loz, sz) * sz;
            int k = (ox * sy + oy) * sz + oz;
            in_rows[pos] = in_row;
            out_rows[pos] = row;
            kernel_ids[pos] = k;
            if (row_masks != nullptr) {
                row_masks[row] = static_cast<int>(1u << (k & 31));
            }
        } else if (row_masks != nullptr) {
            row_masks[row] = 0;
        }
    } else if (row <= target_rows) {
        row_offsets[row] = edges;
        if (row_masks != nullptr && row < target_rows) {
            row_masks[row] = 0;
        }
    }
}

// ---- grouped view (generic stable counting sort of edge ids by group id) ---------

constexpr int kChunkEdges = 1024;  // edges per warp-chunk of the multisplit

// few groups (<= kMultisplitGroups): per-chunk histograms, column scans, stable ranks
constexpr int kMultisplitGroups = 1024;

__global__ void grouped_hist_kernel(
    const int32_t* group_ids, const int32_t* counts, int edge_capacity, int groups,
    int32_t* chunk_hist
) {
    extern __shared__ int smem_counts[];  // [warps][groups]
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int warps = blockDim.x >> 5;
    int edges = clamp_count(counts, edge_capacity);
    int chunk = blockIdx.x * warps + warp;
    int* mine = smem_counts + warp * groups;
    for (int g = lane; g < groups; g += 32) {
        mine[g] = 0;
    }
    __syncwarp();
    int begin = chunk * kChunkEdges;
    for (int i = begin + lane; i < begin + kChunkEdges && i < edges; i += 32) {
        int g = group_ids[i];
        if (g >= 0 && g < groups) {
            atomicAdd(&mine[g], 1);
        }
    }
    __syncwarp();
    if (begin < edges) {
        for (int g = lane; g < groups; g += 32) {
            chunk_hist[static_cast<size_t>(chunk) * groups + g] = mine[g];
        }
    }
}

__global__ void grouped_scatter_kernel(
    const int32_t* group_ids, const int32_t* counts, int edge_capacity, int groups,
    const int32_t* chunk_hist, const int32_t* hist_totals, int32_t* row_offsets,
    int32_t* edge_ids
) {
    extern __shared__ int smem_cursor[];  // [warps][groups]
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int warps = blockDim.x >> 5;
    int edges = clamp_count(counts, edge_capacity);
    int chunk = blockIdx.x * warps + warp;
    int* cursor = smem_cursor + warp * groups;
    int begin = chunk * kChunkEdges;
    // list starts: prefix of the totals (each warp recomputes; groups is small)
    int run = 0;
    for (int base = 0; base < groups; base += 32) {
        int g = base + lane;
        int v = g < groups ? __ldg(hist_totals + g) : 0;
        int total;
        int pre = warp_exclusive_scan(v, total);
        if (g < groups) {
            int start = run + pre;
            cursor[g] = start + (begin < edges
                                     ? chunk_hist[static_cast<size_t>(chunk) * groups + g]
                                     : 0);
            if (chunk == 0) {
                row_offsets[g] = start;
                if (g == groups - 1) {
                    row_offsets[groups] = start + v;
                }
            }
        }
        run += total;
    }
    __syncwarp();
    for (int base = begin; base < begin + kChunkEdges && base < edges; base += 32) {
        int i = base + lane;
        int g = (i < edges) ? group_ids[i] : -1;
        bool valid = g >= 0 && g < groups;
        unsigned peers = __match_any_sync(0xffffffffu, valid ? g : -1 - lane);
        int rank = __popc(peers & lanemask_lt());
        if (valid) {
            edge_ids[cursor[g] + rank] = i;
        }
        __syncwarp();
        if (valid && rank == 0) {
            cursor[g] += __popc(peers);
        }
        __syncwarp();
    }
}

// many groups (input rows): count, scan, fill with cursors, then sort each group
__global__ void grouped_count_kernel(
    const int32_t* group_ids, const int32_t* counts, int edge_capacity, int groups,
    int32_t* degrees
) {
    int edges = clamp_count(counts, edge_capacity);
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < edges) {
        int g = group_ids[i];
        if (g >= 0 && g < groups) {
            atomicAdd(&degrees[g], 1);
        }
    }
}

__global__ void grouped_block_sums_kernel(const int32_t* degrees, int groups, int32_t* sums) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    int total;
    block_exclusive_scan(i < groups ? degrees[i] : 0, total);
    if (threadIdx.x == 0) {
        sums[blockIdx.x] = total;
    }
}

__global__ void grouped_offsets_kernel(
    const int32_t* degrees, int groups, const int32_t* sums, const int32_t* total,
    int32_t* row_offsets, int32_t* cursors
) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    int t;
    int pos = block_exclusive_scan(i < groups ? degrees[i] : 0, t) + sums[blockIdx.x];
    if (i < groups) {
        row_offsets[i] = pos;
        cursors[i] = pos;
    } else if (i == groups) {
        row_offsets[i] = *total;
    }
}

__global__ void grouped_fill_kernel(
    const int32_t* group_ids, const int32_t* counts, int edge_capacity, int groups,
    int32_t* cursors, int32_t* edge_ids
) {
    int edges = clamp_count(counts, edge_capacity);
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < edges) {
        int g = group_ids[i];
        if (g >= 0 && g < groups) {
            edge_ids[atomicAdd(&cursors[g], 1)] = i;
        }
    }
}

// ascending edge id inside every group (the cursor fill above is unordered)
__global__ void grouped_sort_kernel(const int32_t* row_offsets, int groups, int32_t* edge_ids) {
    int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) {
        return;
    }
    int begin = row_offsets[g];
    int end = row_offsets[g + 1];
    for (int i = begin + 1; i < end; ++i) {
        int v = edge_ids[i];
        int j = i - 1;
        while (j >= begin && edge_ids[j] > v) {
            edge_ids[j + 1] = edge_ids[j];
            --j;
        }
        edge_ids[j + 1] = v;
    }
}

// ---- implicit-GEMM view, lookup, alignment ----------------------------------------

__global__ void __launch_bounds__(kBlockThreads) igemm_view_kernel(
    const int32_t* source_coords, const Slot* table, uint32_t mask,
    const int32_t* source_active_ptr, int source_rows, const int32_t* output_coords,
    const int32_t* output_active_ptr, int output_rows, const int32_t* offsets, int K,
    int words, int sx, int sy, int sz, int px, int py, int pz, int32_t* out_in_map,
    int32_t* row_masks
) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= output_rows) {
        return;
    }
    int source_active = clamp_count(source_active_ptr, source_rows);
    int output_active = clamp_count(output_active_ptr, output_rows);
    PlainKey key_of{source_coords};
    Coord out = load_coord(output_coords, row);
    for (int pass = 0; pass < words; ++pass) {
        int k = pass * 32 + lane;
        int found = -1;
        if (k < K && row < output_active) {
            Coord cand{out.b, out.x * sx + __ldg(offsets + 3 * k) - px,
                       out.y * sy + __ldg(offsets + 3 * k + 1) - py,
                       out.z * sz + __ldg(offsets + 3 * k + 2) - pz};
            found = table_find(table, mask, cand, key_of);
            if (found >= source_active) {
                found = -1;
            }
        }
        unsigned m = __ballot_sync(0xffffffffu, found >= 0);
        if (k < K) {
            out_in_map[static_cast<size_t>(row) * K + k] = found;
        }
        if (lane == 0) {
            row_masks[static_cast<size_t>(row) * words + pass] = static_cast<int>(m);
        }
    }
}

__global__ void lookup_kernel(
    const int32_t* coords, const Slot* table, uint32_t mask, const int32_t* queries,
    int query_rows, const int32_t* query_active_ptr, int32_t* out_rows
) {
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= query_rows) {
        return;
    }
    int active = query_active_ptr ? clamp_count(query_active_ptr, query_rows) : query_rows;
    int found = -1;
    if (row < active) {
        found = table_find(table, mask, load_coord(queries, row), PlainKey{coords});
    }
    out_rows[row] = found;
}

// alignment pass over lhs rows: keep flag (+ matching rhs row) and block counts
__global__ void align_lhs_count_kernel(
    const int32_t* lhs, const int32_t* lhs_active_ptr, int lhs_rows, const int32_t* rhs,
    const Slot* rhs_table, uint32_t rhs_mask, int inner, int32_t* match, int32_t* block_sums
) {
    int active = clamp_count(lhs_active_ptr, lhs_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int keep = 0;
    if (row < active) {
        int m = table_find(rhs_table, rhs_mask, load_coord(lhs, row), PlainKey{rhs});
        match[row] = m;
        keep = inner ? (m >= 0) : 1;
    }
    int t;
    block_exclusive_scan(keep, t);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = t;
    }
}

__global__ void align_lhs_fill_kernel(
    const int32_t* lhs, const int32_t* lhs_active_ptr, int lhs_rows, int inner,
    const int32_t* match, const int32_t* block_offsets, int32_t* out_coords,
    int32_t* out_lhs, int32_t* out_rhs
) {
    int active = clamp_count(lhs_active_ptr, lhs_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int keep = 0, m = -1;
    if (row < active) {
        m = match[row];
        keep = inner ? (m >= 0) : 1;
    }
    int t;
    int pos = block_exclusive_scan(keep, t) + block_offsets[blockIdx.x];
    if (keep) {
        reinterpret_cast<int4*>(out_coords)[pos] = reinterpret_cast<const int4*>(lhs)[row];
        out_lhs[pos] = row;
        out_rhs[pos] = m;
    }
}

// outer join tail: rhs rows absent from lhs, appended after `base` rows
__global__ void align_rhs_count_kernel(
    const int32_t* rhs, const int32_t* rhs_active_ptr, int rhs_rows, const int32_t* lhs,
    const Slot* lhs_table, uint32_t lhs_mask, int32_t* absent, int32_t* block_sums
) {
    int active = clamp_count(rhs_active_ptr, rhs_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int keep = 0;
    if (row < active) {
        keep = table_find(lhs_table, lhs_mask, load_coord(rhs, row), PlainKey{lhs}) < 0;
        absent[row] = keep;
    }
    int t;
    block_exclusive_scan(keep, t);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = t;
    }
}

__global__ void align_rhs_fill_kernel(
    const int32_t* rhs, const int32_t* rhs_active_ptr, int rhs_rows, const int32_t* absent,
    const int32_t* block_offsets, const int32_t* base_ptr, int32_t* out_coords,
    int32_t* out_lhs, int32_t* out_rhs, int32_t* out_count, const int32_t* tail_total
) {
    int active = clamp_count(rhs_active_ptr, rhs_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    int keep = row < active ? absent[row] : 0;
    int t;
    int base = *base_ptr;
    int pos = block_exclusive_scan(keep, t) + block_offsets[blockIdx.x] + base;
    if (keep) {
        reinterpret_cast<int4*>(out_coords)[pos] = reinterpret_cast<const int4*>(rhs)[row];
        out_lhs[pos] = -1;
        out_rhs[pos] = row;
    }
    if (row == 0) {
        out_count[0] = base + *tail_total;
    }
}

// right join: one output row per active rhs row
__global__ void align_right_kernel(
    const int32_t* rhs, const int32_t* rhs_active_ptr, int rhs_rows, const int32_t* lhs,
    const Slot* lhs_table, uint32_t lhs_mask, int32_t* out_coords, int32_t* out_lhs,
    int32_t* out_rhs, int32_t* out_count
) {
    int active = clamp_count(rhs_active_ptr, rhs_rows);
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row == 0) {
        out_count[0] = active;
    }
    if (row >= rhs_rows) {
        return;
    }
    if (row < active) {
        Coord c = load_coord(rhs, row);
        store_coord(out_coords, row, c);
        out_lhs[row] = table_find(lhs_table, lhs_mask, c, PlainKey{lhs});
        out_rhs[row] = row;
    } else {
        store_coord(out_coords, row, {0, 0, 0, 0});
        out_lhs[row] = -1;
        out_rhs[row] = -1;
    }
}

inline int blocks_for(long long count, int threads = kBlockThreads) {
    return static_cast<int>((count + threads - 1) / threads);
}

inline int fill_grid(size_t count) {
    size_t blocks = (count + 1023) / 1024;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

cudaError_t fill_i32(int32_t* data, size_t count, int value, cudaStream_t stream) {
    if (count == 0) {
        return cudaSuccess;
    }
    if (value == 0 || value == -1) {
        return cudaMemsetAsync(data, value == 0 ? 0 : 0xFF, count * sizeof(int32_t), stream);
    }
    fill_i32_kernel<<<fill_grid(count), 256, 0, stream>>>(data, count, value);
    return cudaGetLastError();
}

// The three edge arrays are zero beyond the edge count (the reference's contract for
// its statically sized outputs). Only that tail is written, after the count is known:
// a map over N rows has capacity N * K, of which a sparse cloud uses a few per cent.
__global__ void zero_edge_tails_kernel(
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, size_t capacity, const int32_t* counts,
    int count_cap
) {
    const size_t edges = static_cast<size_t>(clamp_count(counts, count_cap));
    const size_t quads = (capacity + 3) / 4;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t quad = edges / 4 + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
         quad < quads; quad += stride) {
        const size_t first = quad * 4;
        if (first >= edges && first + 4 <= capacity) {
            const int4 zero = make_int4(0, 0, 0, 0);
            reinterpret_cast<int4*>(in_rows)[quad] = zero;
            reinterpret_cast<int4*>(out_rows)[quad] = zero;
            reinterpret_cast<int4*>(kernel_ids)[quad] = zero;
        } else {
            for (size_t i = first > edges ? first : edges; i < first + 4 && i < capacity; ++i) {
                in_rows[i] = 0;
                out_rows[i] = 0;
                kernel_ids[i] = 0;
            }
        }
    }
}

cudaError_t zero_edge_tails(
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, size_t capacity, const int32_t* counts,
    cudaStream_t stream
) {
    if (capacity == 0) {
        return cudaSuccess;
    }
    const uintptr_t bits = reinterpret_cast<uintptr_t>(in_rows) | reinterpret_cast<uintptr_t>(out_rows) |
                           reinterpret_cast<uintptr_t>(kernel_ids);
    if (bits % 16 != 0) {
        // unaligned caller buffers: clear everything up front instead (the map kernels
        // then overwrite the live part); callers order this before the map themselves
        return cudaErrorInvalidValue;
    }
    const int count_cap = static_cast<int>(std::min<size_t>(capacity, 0x7fffffff));
    const size_t quads = (capacity + 3) / 4;
    const int blocks = static_cast<int>(std::min<size_t>((quads + 255) / 256, 148 * 8));
    zero_edge_tails_kernel<<<blocks, 256, 0, stream>>>(in_rows, out_rows, kernel_ids, capacity, counts,
                                                       count_cap);
    return cudaGetLastError();
}

cudaError_t clear_table(Slot* slots, size_t capacity, cudaStream_t stream) {
    return cudaMemsetAsync(slots, 0xFF, capacity * sizeof(Slot), stream);
}

struct SourceTable {
    Slot* slots;
    uint32_t mask;
};

// build the first-row table of rows [0, active) of `coords`
int build_source_table(
    Workspace& ws, const int32_t* coords, int rows, const int32_t* active_rows,
    int32_t* status, bool flag_duplicates, cudaStream_t stream, SourceTable& table
) {
    int capacity = table_slots(rows);
    table.slots = ws.take<Slot>(capacity);
    table.mask = static_cast<uint32_t>(capacity - 1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the coordinate table.");
    }
    LAT_CUDA_CHECK(clear_table(table.slots, capacity, stream));
    if (rows > 0) {
        insert_rows_kernel<<<blocks_for(rows), kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, table.slots, table.mask, status, flag_duplicates ? 1 : 0);
        LAT_LAUNCH_CHECK();
    }
    return LAT_OK;
}

// the first-row table of `coords`: the caller's prebuilt one (lat_build_coord_table over the
// same coords / active_rows) or a fresh one in the workspace
int acquire_source_table(
    Workspace& ws, const int32_t* coords, int rows, const int32_t* active_rows, int32_t* status,
    cudaStream_t stream, const void* prebuilt, SourceTable& table
) {
    if (prebuilt == nullptr) {
        return build_source_table(ws, coords, rows, active_rows, status, false, stream, table);
    }
    if (reinterpret_cast<uintptr_t>(prebuilt) % 32 != 0) {
        return fail(LAT_INVALID_ARGUMENT, "source_table must be a 32-byte aligned device buffer.");
    }
    table.slots = const_cast<Slot*>(static_cast<const Slot*>(prebuilt));
    table.mask = static_cast<uint32_t>(table_slots(rows) - 1);
    return LAT_OK;
}

struct MapOutputs {
    int32_t* in_rows;
    int32_t* out_rows;
    int32_t* kernel_ids;
    int32_t* row_offsets;
    int32_t* counts;
    int32_t* row_masks;
    int32_t* kernel_row_offsets;
    int32_t* kernel_edge_ids;
};

// count -> scan -> fill over `out_capacity` output rows whose coordinates are given
int run_map(
    Workspace& ws, const int32_t* coords, const SourceTable& table,
    const int32_t* out_coords, const int32_t* out_count_ptr, int out_capacity,
    int offsets_capacity, KernelGeometry geo, lat_triple stride, lat_triple padding,
    MapRule rule, bool tail_is_total, const MapOutputs& o, int32_t* status, cudaStream_t stream
) {
    int K = geo.volume;
    int words = (K + 31) / 32;
    if (words > kMaxMaskWords) {
        return fail(LAT_INVALID_ARGUMENT, "kernel volume above 352 offsets is not supported.");
    }
    size_t edge_capacity = static_cast<size_t>(out_capacity) * K;
    // one extra row so that row_offsets[out_capacity] is written by the fill kernel
    int nblocks = std::max(1, blocks_for(static_cast<long long>(out_capacity) + 1, kRowsPerBlock));
    bool lists = o.kernel_edge_ids != nullptr && o.kernel_row_offsets != nullptr;
    int32_t* masks = o.row_masks != nullptr
                         ? o.row_masks
                         : ws.take<int32_t>(static_cast<size_t>(std::max(out_capacity, 1)) * words);
    int32_t* block_sums = ws.take<int32_t>(nblocks);
    int32_t* block_hist = lists ? ws.take<int32_t>(static_cast<size_t>(nblocks) * K) : nullptr;
    int32_t* hist_totals = lists ? ws.take<int32_t>(K) : nullptr;
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
    }

    // 16-byte aligned edge arrays get only their tail zeroed, after the map; others are
    // cleared whole here
    const bool tail_only =
        (reinterpret_cast<uintptr_t>(o.in_rows) | reinterpret_cast<uintptr_t>(o.out_rows) |
         reinterpret_cast<uintptr_t>(o.kernel_ids)) % 16 == 0;
    if (!tail_only) {
        LAT_CUDA_CHECK(fill_i32(o.in_rows, edge_capacity, 0, stream));
        LAT_CUDA_CHECK(fill_i32(o.out_rows, edge_capacity, 0, stream));
        LAT_CUDA_CHECK(fill_i32(o.kernel_ids, edge_capacity, 0, stream));
    }
    LAT_CUDA_CHECK(fill_i32(o.row_offsets, static_cast<size_t>(offsets_capacity) + 1, 0, stream));
    if (o.row_masks != nullptr) {
        LAT_CUDA_CHECK(fill_i32(o.row_masks, static_cast<size_t>(out_capacity) * words, 0, stream));
    }
    if (lists) {
        LAT_CUDA_CHECK(fill_i32(o.kernel_edge_ids, edge_capacity, -1, stream));
    }

    MapParams p{};
    p.wait_budget = wait_budget_cycles();
    p.coords = coords;
    p.table = table.slots;
    p.table_mask = table.mask;
    p.out_coords = out_coords;
    p.out_count_ptr = out_count_ptr;
    p.out_capacity = out_capacity;
    p.out_count_cap = out_capacity;
    p.geo = geo;
    p.sx = stride.x, p.sy = stride.y, p.sz = stride.z;
    p.px = padding.x, p.py = padding.y, p.pz = padding.z;
    p.rule = static_cast<int>(rule);
    p.words = words;
    p.masks = masks;
    p.block_sums = block_sums;
    p.block_hist = block_hist;
    p.in_rows = o.in_rows;
    p.out_rows = o.out_rows;
    p.kernel_ids = o.kernel_ids;
    p.row_offsets = o.row_offsets;
    p.counts = o.counts;
    p.kernel_row_offsets = lists ? o.kernel_row_offsets : nullptr;
    p.kernel_edge_ids = lists ? o.kernel_edge_ids : nullptr;
    p.hist_totals = hist_totals;
    p.tail_is_total = tail_is_total ? 1 : 0;
    p.edge_capacity = static_cast<int>(std::min<size_t>(edge_capacity, 0x7fffffff));
    p.status = status;

    if (!lists && K <= 32) {
        // single pass: probe once, look back for the tile prefix, write
        unsigned long long* tile_status = ws.take<unsigned long long>(nblocks);
        int* ticket = ws.take<int>(1);
        if (!ws.ok) {
            return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
        }
        LAT_CUDA_CHECK(cudaMemsetAsync(tile_status, 0, sizeof(unsigned long long) * nblocks, stream));
        LAT_CUDA_CHECK(cudaMemsetAsync(ticket, 0, sizeof(int), stream));
        p.masks = o.row_masks;  // optional output; no scratch copy needed
        size_t smem = sizeof(int) * kRowsPerBlock * K;
        map_single_pass_kernel<<<nblocks, kBlockThreads, smem, stream>>>(p, tile_status, ticket, nblocks);
        LAT_LAUNCH_CHECK();
        if (tail_only) {
            LAT_CUDA_CHECK(zero_edge_tails(o.in_rows, o.out_rows, o.kernel_ids, edge_capacity, o.counts, stream));
            count_launch();
        }
        return LAT_OK;
    }
    size_t count_smem = lists ? sizeof(int) * kWarpsPerBlock * K : 0;
    map_count_kernel<<<nblocks, kBlockThreads, count_smem, stream>>>(p);
    LAT_LAUNCH_CHECK();
    scan_blocks_kernel<<<lists ? K + 1 : 1, kBlockThreads, 0, stream>>>(
        block_sums, nblocks, o.counts, o.counts + 1, out_count_ptr, out_capacity, block_hist, K,
        hist_totals);
    LAT_LAUNCH_CHECK();
    size_t fill_smem = lists ? sizeof(int) * kWarpsPerBlock * K : 0;
    map_fill_kernel<<<nblocks, kBlockThreads, fill_smem, stream>>>(p);
    LAT_LAUNCH_CHECK();
    if (tail_only) {
        LAT_CUDA_CHECK(zero_edge_tails(o.in_rows, o.out_rows, o.kernel_ids, edge_capacity, o.counts, stream));
        count_launch();
    }
    return LAT_OK;
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_relation_workspace_bytes(int32_t rows, int32_t out_rows, int32_t kernel_count) {
    size_t K = static_cast<size_t>(std::max(kernel_count, 1));
    size_t words = (K + 31) / 32;
    size_t r = static_cast<size_t>(std::max(rows, 1));
    size_t o = static_cast<size_t>(std::max(out_rows, 1));
    size_t total = 0;
    total += align_up(sizeof(Slot) * table_slots(r));              // source table
    total += align_up(sizeof(Slot) * table_slots(std::max(r, o)));     // second table
    total += align_up(sizeof(int32_t) * o * words);                  // masks
    size_t nblocks = (std::max(o, r * 1) + kRowsPerBlock) / kRowsPerBlock + 2;
    total += 3 * align_up(sizeof(int32_t) * nblocks);                // block sums
    total += align_up(sizeof(int32_t) * nblocks * K);                // per-block offset hist
    total += align_up(sizeof(int32_t) * K) + 4 * 256;
    total += align_up(sizeof(unsigned long long) * nblocks) + 256;      // tile status + ticket
    total += align_up(sizeof(int32_t) * o);                          // hit rows / flags
    return total;
}

static int validate_relation_args(
    const int32_t* coords, int32_t rows, const int32_t* active_rows, lat_triple kernel_size,
    lat_triple stride, lat_triple padding, lat_triple dilation
) {
    LAT_REQUIRE(rows >= 0, "coords must have shape (N, 4).");
    LAT_REQUIRE(coords != nullptr || rows == 0, "coords must have shape (N, 4).");
    LAT_REQUIRE(active_rows != nullptr, "active_rows must have shape (1,) and int32 dtype.");
    LAT_REQUIRE(kernel_size.x > 0 && kernel_size.y > 0 && kernel_size.z > 0,
                "kernel_size values must be positive.");
    LAT_REQUIRE(stride.x > 0 && stride.y > 0 && stride.z > 0, "stride values must be positive.");
    LAT_REQUIRE(padding.x >= 0 && padding.y >= 0 && padding.z >= 0,
                "padding values must be non-negative.");
    LAT_REQUIRE(dilation.x > 0 && dilation.y > 0 && dilation.z > 0,
                "dilation values must be positive.");
    long long volume = 1LL * kernel_size.x * kernel_size.y * kernel_size.z;
    LAT_REQUIRE(volume * std::max(rows, 1) <= 0x7fffffffLL,
                "rows * kernel volume exceeds the int32 edge capacity.");
    return LAT_OK;
}

size_t lat_coord_table_bytes(int32_t rows) {
    return align_up(sizeof(Slot) * static_cast<size_t>(table_slots(std::max(rows, 1))));
}

int lat_build_coord_table(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    void* table, size_t table_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0 && (coords != nullptr || rows == 0), "coords must have shape (N, 4).");
    LAT_REQUIRE(active_rows != nullptr, "active_rows must have shape (1,) and int32 dtype.");
    LAT_REQUIRE(table != nullptr && reinterpret_cast<uintptr_t>(table) % 32 == 0,
                "table must be a 32-byte aligned device buffer.");
    LAT_REQUIRE(table_bytes >= lat_coord_table_bytes(rows), "table is smaller than lat_coord_table_bytes.");
    Workspace ws(table, table_bytes);
    SourceTable built;
    return build_source_table(ws, coords, rows, active_rows, status, false, as_stream(stream_ptr), built);
}

int lat_build_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    const void* source_table,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    int rc = validate_relation_args(coords, rows, active_rows, kernel_size, stride, padding, dilation);
    if (rc != LAT_OK) {
        return rc;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    KernelGeometry geo = make_geometry(kernel_size, dilation);
    Workspace ws(workspace, workspace_bytes);
    MapOutputs o{in_rows, out_rows, kernel_ids, row_offsets, counts, row_masks,
                 kernel_row_offsets, kernel_edge_ids};
    if (rows == 0) {
        LAT_CUDA_CHECK(fill_i32(row_offsets, 1, 0, stream));
        LAT_CUDA_CHECK(fill_i32(counts, 2, 0, stream));
        if (kernel_row_offsets != nullptr) {
            LAT_CUDA_CHECK(fill_i32(kernel_row_offsets, geo.volume + 1, 0, stream));
        }
        return LAT_OK;
    }
    SourceTable table;
    rc = acquire_source_table(ws, coords, rows, active_rows, status, stream, source_table, table);
    if (rc != LAT_OK) {
        return rc;
    }
    bool identity = stride.x == 1 && stride.y == 1 && stride.z == 1 && padding.x == 0 &&
                    padding.y == 0 && padding.z == 0;
    int32_t* out_count = ws.take<int32_t>(1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
    }
    if (identity) {
        copy_active_coords_kernel<<<blocks_for(rows), kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, out_coords);
        LAT_LAUNCH_CHECK();
        store_clamped_kernel<<<1, 1, 0, stream>>>(active_rows, rows, out_count);
        LAT_LAUNCH_CHECK();
    } else {
        int capacity = table_slots(rows);
        Slot* table2 = ws.take<Slot>(capacity);
        int nblocks = blocks_for(rows);
        int32_t* sums = ws.take<int32_t>(nblocks);
        if (!ws.ok) {
            return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
        }
        uint32_t mask2 = static_cast<uint32_t>(capacity - 1);
        LAT_CUDA_CHECK(clear_table(table2, capacity, stream));
        LAT_CUDA_CHECK(fill_i32(out_coords, static_cast<size_t>(rows) * 4, 0, stream));
        insert_downsampled_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, stride.x, stride.y, stride.z, table2, mask2, status);
        LAT_LAUNCH_CHECK();
        mark_winners_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, stride.x, stride.y, stride.z, table2, mask2, sums);
        LAT_LAUNCH_CHECK();
        const int prescanned = nblocks > kSelfScanBlocks ? 1 : 0;
        if (prescanned) {
            scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
                sums, nblocks, out_count, nullptr, nullptr, 0, nullptr, 0, nullptr);
            LAT_LAUNCH_CHECK();
        }
        compact_winners_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, stride.x, stride.y, stride.z, table2, mask2, sums, prescanned,
            out_count, out_coords, rows, status);
        LAT_LAUNCH_CHECK();
    }
    return run_map(ws, coords, table, out_coords, out_count, rows, rows, geo, stride, padding,
                   MapRule::Forward, false, o, status, stream);
}

int lat_build_submanifold_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    const void* source_table,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream
) {
    return lat_build_kernel_relation(
        coords, rows, active_rows, kernel_size, {1, 1, 1}, {0, 0, 0}, dilation, in_rows,
        out_rows, kernel_ids, row_offsets, out_coords, counts, row_masks, kernel_row_offsets,
        kernel_edge_ids, source_table, workspace, workspace_bytes, status, stream);
}

int lat_build_target_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    const int32_t* target_coords, int32_t target_rows, const int32_t* target_active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    int rc = validate_relation_args(coords, rows, active_rows, kernel_size, stride, padding, dilation);
    if (rc != LAT_OK) {
        return rc;
    }
    LAT_REQUIRE(target_rows >= 0 && (target_coords != nullptr || target_rows == 0),
                "coords must have shape (N, 4).");
    LAT_REQUIRE(target_active_rows != nullptr,
                "active_rows must have shape (1,) and int32 dtype.");
    cudaStream_t stream = as_stream(stream_ptr);
    KernelGeometry geo = make_geometry(kernel_size, dilation);
    LAT_REQUIRE(1LL * geo.volume * std::max(target_rows, 1) <= 0x7fffffffLL,
                "rows * kernel volume exceeds the int32 edge capacity.");
    Workspace ws(workspace, workspace_bytes);
    MapOutputs o{in_rows, out_rows, kernel_ids, row_offsets, counts, row_masks,
                 kernel_row_offsets, kernel_edge_ids};
    SourceTable table;
    rc = build_source_table(ws, coords, rows, active_rows, status, false, stream, table);
    if (rc != LAT_OK) {
        return rc;
    }
    if (target_rows == 0) {
        LAT_CUDA_CHECK(fill_i32(row_offsets, 1, 0, stream));
        LAT_CUDA_CHECK(fill_i32(counts, 2, 0, stream));
        if (kernel_row_offsets != nullptr) {
            LAT_CUDA_CHECK(fill_i32(kernel_row_offsets, geo.volume + 1, 0, stream));
        }
        return LAT_OK;
    }
    return run_map(ws, coords, table, target_coords, target_active_rows, target_rows,
                   target_rows, geo, stride, padding, MapRule::Forward, true, o, status, stream);
}

static bool direct_transposed(KernelGeometry geo, lat_triple stride) {
    // stride must exceed the offset extent on every axis
    // (coordinates/relations.cpp:107-126)
    int ex = (geo.kx - 1) * geo.dx, ey = (geo.ky - 1) * geo.dy, ez = (geo.kz - 1) * geo.dz;
    return stride.x > ex && stride.y > ey && stride.z > ez;
}

int lat_build_transposed_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    int rc = validate_relation_args(coords, rows, active_rows, kernel_size, stride, padding, dilation);
    if (rc != LAT_OK) {
        return rc;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    KernelGeometry geo = make_geometry(kernel_size, dilation);
    long long capacity = 1LL * rows * geo.volume;
    if (direct_transposed(geo, stride)) {
        direct_transposed_kernel<<<blocks_for(capacity + 1), kBlockThreads, 0, stream>>>(
            coords, active_rows, rows, geo, stride.x, stride.y, stride.z, padding.x, padding.y,
            padding.z, in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts);
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    // overlapping outputs: dedupe candidates in first-seen (in-major, k-minor) order,
    // then gather per output row in (k asc) order through the source table
    Workspace ws(workspace, workspace_bytes);
    SourceTable table;
    rc = build_source_table(ws, coords, rows, active_rows, status, true, stream, table);
    if (rc != LAT_OK) {
        return rc;
    }
    int cap2 = table_slots(capacity);
    Slot* table2 = ws.take<Slot>(cap2);
    int nblocks = std::max(1, blocks_for(capacity));
    int32_t* sums = ws.take<int32_t>(nblocks);
    int32_t* out_count = ws.take<int32_t>(1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
    }
    uint32_t mask2 = static_cast<uint32_t>(cap2 - 1);
    TransposedCandidateKey key_of{coords, geo, stride.x, stride.y, stride.z,
                                  padding.x, padding.y, padding.z};
    LAT_CUDA_CHECK(clear_table(table2, cap2, stream));
    LAT_CUDA_CHECK(fill_i32(out_coords, static_cast<size_t>(capacity) * 4, 0, stream));
    insert_candidates_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        key_of, active_rows, rows, table2, mask2, status);
    LAT_LAUNCH_CHECK();
    mark_candidate_winners_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        key_of, active_rows, rows, table2, mask2, sums);
    LAT_LAUNCH_CHECK();
    scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
        sums, nblocks, out_count, nullptr, nullptr, 0, nullptr, 0, nullptr);
    LAT_LAUNCH_CHECK();
    compact_candidates_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        key_of, active_rows, rows, table2, mask2, sums, out_coords, static_cast<int>(capacity));
    LAT_LAUNCH_CHECK();
    // The edge arrays are rows*K long (every (in, k) pair yields exactly one edge when
    // the input coordinates are unique), not out_capacity*K, hence no run_map here.
    {
        int K = geo.volume;
        int words = (K + 31) / 32;
        if (words > kMaxMaskWords) {
            return fail(LAT_INVALID_ARGUMENT, "kernel volume above 352 offsets is not supported.");
        }
        int out_capacity = static_cast<int>(capacity);
        int mblocks = std::max(1, blocks_for(static_cast<long long>(out_capacity) + 1, kRowsPerBlock));
        int32_t* masks = ws.take<int32_t>(static_cast<size_t>(out_capacity) * words);
        int32_t* block_sums = ws.take<int32_t>(mblocks);
        if (!ws.ok) {
            return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
        }
        LAT_CUDA_CHECK(fill_i32(in_rows, capacity, 0, stream));
        LAT_CUDA_CHECK(fill_i32(out_rows, capacity, 0, stream));
        LAT_CUDA_CHECK(fill_i32(kernel_ids, capacity, 0, stream));
        LAT_CUDA_CHECK(fill_i32(row_offsets, capacity + 1, 0, stream));
        MapParams p{};
        p.wait_budget = wait_budget_cycles();
        p.coords = coords;
        p.table = table.slots;
        p.table_mask = table.mask;
        p.out_coords = out_coords;
        p.out_count_ptr = out_count;
        p.out_capacity = out_capacity;
        p.out_count_cap = out_capacity;
        p.geo = geo;
        p.sx = stride.x, p.sy = stride.y, p.sz = stride.z;
        p.px = padding.x, p.py = padding.y, p.pz = padding.z;
        p.rule = static_cast<int>(MapRule::TransposedGather);
        p.words = words;
        p.masks = masks;
        p.block_sums = block_sums;
        p.in_rows = in_rows;
        p.out_rows = out_rows;
        p.kernel_ids = kernel_ids;
        p.row_offsets = row_offsets;
        p.counts = counts;
        p.edge_capacity = out_capacity;
        p.status = status;
        map_count_kernel<<<mblocks, kBlockThreads, 0, stream>>>(p);
        LAT_LAUNCH_CHECK();
        scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
            block_sums, mblocks, counts, counts + 1, out_count, out_capacity, nullptr, 0, nullptr);
        LAT_LAUNCH_CHECK();
        map_fill_kernel<<<mblocks, kBlockThreads, 0, stream>>>(p);
        LAT_LAUNCH_CHECK();
    }
    return LAT_OK;
}

int lat_build_generative_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    (void)workspace, (void)workspace_bytes, (void)status;
    int rc = validate_relation_args(coords, rows, active_rows, kernel_size, stride, {0, 0, 0},
                                    {1, 1, 1});
    if (rc != LAT_OK) {
        return rc;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    KernelGeometry geo = make_geometry(kernel_size, {1, 1, 1});
    long long capacity = 1LL * rows * geo.volume;
    direct_transposed_kernel<<<blocks_for(capacity + 1), kBlockThreads, 0, stream>>>(
        coords, active_rows, rows, geo, stride.x, stride.y, stride.z, 0, 0, 0, in_rows, out_rows,
        kernel_ids, row_offsets, out_coords, counts);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_build_target_transposed_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    const int32_t* target_coords, int32_t target_rows, const int32_t* target_active_rows,
    lat_triple stride,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* counts, int32_t* row_masks, const void* source_table,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    int rc = validate_relation_args(coords, rows, active_rows, stride, stride, {0, 0, 0}, {1, 1, 1});
    if (rc == LAT_OK && row_masks != nullptr && 1LL * stride.x * stride.y * stride.z > 32) {
        rc = fail(LAT_INVALID_ARGUMENT, "row masks need a kernel volume of at most 32.");
    }
    if (rc != LAT_OK) {
        return rc;
    }
    LAT_REQUIRE(target_rows >= 0 && (target_coords != nullptr || target_rows == 0),
                "coords must have shape (N, 4).");
    LAT_REQUIRE(target_active_rows != nullptr,
                "active_rows must have shape (1,) and int32 dtype.");
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    SourceTable table;
    rc = acquire_source_table(ws, coords, rows, active_rows, status, stream, source_table, table);
    if (rc != LAT_OK) {
        return rc;
    }
    int nblocks = std::max(1, blocks_for(static_cast<long long>(target_rows) + 1));
    int32_t* hit_rows = ws.take<int32_t>(std::max(target_rows, 1));
    int32_t* sums = ws.take<int32_t>(nblocks);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the kernel map.");
    }
    // odd kernel sizes are centred, even ones start at zero (coordinates/offsets.cpp:11-45)
    int lox = (stride.x & 1) ? -(stride.x / 2) : 0;
    int loy = (stride.y & 1) ? -(stride.y / 2) : 0;
    int loz = (stride.z & 1) ? -(stride.z / 2) : 0;
    LAT_CUDA_CHECK(fill_i32(in_rows, target_rows, 0, stream));
    LAT_CUDA_CHECK(fill_i32(out_rows, target_rows, 0, stream));
    LAT_CUDA_CHECK(fill_i32(kernel_ids, target_rows, 0, stream));
    target_transposed_count_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        coords, table.slots, table.mask, target_coords, target_active_rows, target_rows,
        stride.x, stride.y, stride.z, lox, loy, loz, hit_rows, sums);
    LAT_LAUNCH_CHECK();
    const int prescanned = nblocks > kSelfScanBlocks ? 1 : 0;
    if (prescanned) {
        scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
            sums, nblocks, counts, counts + 1, target_active_rows, target_rows, nullptr, 0, nullptr);
        LAT_LAUNCH_CHECK();
    }
    target_transposed_fill_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        target_coords, target_active_rows, target_rows, stride.x, stride.y, stride.z, lox, loy,
        loz, hit_rows, sums, prescanned, counts, in_rows, out_rows, kernel_ids, row_offsets, row_masks);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_grouped_view_workspace_bytes(int32_t edge_capacity, int32_t group_count) {
    size_t e = static_cast<size_t>(std::max(edge_capacity, 1));
    size_t g = static_cast<size_t>(std::max(group_count, 1));
    if (group_count <= kMultisplitGroups) {
        size_t chunks = (e + kChunkEdges - 1) / kChunkEdges + 8;
        return align_up(sizeof(int32_t) * chunks * g) + align_up(sizeof(int32_t) * g) + 1024;
    }
    size_t nblocks = (g + kBlockThreads) / kBlockThreads + 1;
    return 2 * align_up(sizeof(int32_t) * (g + 1)) + align_up(sizeof(int32_t) * nblocks) + 1024;
}

int lat_build_relation_grouped_view(
    const int32_t* group_ids, int32_t edge_capacity, const int32_t* counts, int32_t group_count,
    int32_t* row_offsets, int32_t* edge_ids,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    (void)status;
    LAT_REQUIRE(edge_capacity >= 0 && group_count >= 0, "grouped view sizes must be non-negative.");
    LAT_REQUIRE(counts != nullptr, "counts must have shape (2,) and int32 dtype.");
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    LAT_CUDA_CHECK(fill_i32(edge_ids, edge_capacity, -1, stream));
    LAT_CUDA_CHECK(fill_i32(row_offsets, static_cast<size_t>(group_count) + 1, 0, stream));
    if (edge_capacity == 0 || group_count == 0) {
        return LAT_OK;
    }
    if (group_count <= kMultisplitGroups) {
        int chunks = (edge_capacity + kChunkEdges - 1) / kChunkEdges;
        // warps per block limited by shared memory (groups ints per warp)
        int warps = std::max(1, std::min(8, static_cast<int>(40960 / (sizeof(int) * group_count))));
        int blocks = (chunks + warps - 1) / warps;
        int32_t* hist = ws.take<int32_t>(static_cast<size_t>(blocks) * warps * group_count);
        int32_t* totals = ws.take<int32_t>(group_count);
        if (!ws.ok) {
            return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the grouped view.");
        }
        size_t smem = sizeof(int) * warps * group_count;
        LAT_CUDA_CHECK(fill_i32(hist, static_cast<size_t>(blocks) * warps * group_count, 0, stream));
        grouped_hist_kernel<<<blocks, warps * 32, smem, stream>>>(
            group_ids, counts, edge_capacity, group_count, hist);
        LAT_LAUNCH_CHECK();
        scan_blocks_kernel<<<group_count + 1, kBlockThreads, 0, stream>>>(
            nullptr, blocks * warps, nullptr, nullptr, nullptr, 0, hist, group_count, totals);
        LAT_LAUNCH_CHECK();
        grouped_scatter_kernel<<<blocks, warps * 32, smem, stream>>>(
            group_ids, counts, edge_capacity, group_count, hist, totals, row_offsets, edge_ids);
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    int nblocks = blocks_for(static_cast<long long>(group_count) + 1);
    int32_t* degrees = ws.take<int32_t>(static_cast<size_t>(group_count) + 1);
    int32_t* cursors = ws.take<int32_t>(static_cast<size_t>(group_count) + 1);
    int32_t* sums = ws.take<int32_t>(nblocks);
    int32_t* total = ws.take<int32_t>(1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the grouped view.");
    }
    LAT_CUDA_CHECK(fill_i32(degrees, static_cast<size_t>(group_count) + 1, 0, stream));
    grouped_count_kernel<<<blocks_for(edge_capacity), kBlockThreads, 0, stream>>>(
        group_ids, counts, edge_capacity, group_count, degrees);
    LAT_LAUNCH_CHECK();
    grouped_block_sums_kernel<<<nblocks, kBlockThreads, 0, stream>>>(degrees, group_count, sums);
    LAT_LAUNCH_CHECK();
    scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
        sums, nblocks, total, nullptr, nullptr, 0, nullptr, 0, nullptr);
    LAT_LAUNCH_CHECK();
    grouped_offsets_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        degrees, group_count, sums, total, row_offsets, cursors);
    LAT_LAUNCH_CHECK();
    grouped_fill_kernel<<<blocks_for(edge_capacity), kBlockThreads, 0, stream>>>(
        group_ids, counts, edge_capacity, group_count, cursors, edge_ids);
    LAT_LAUNCH_CHECK();
    grouped_sort_kernel<<<blocks_for(group_count), kBlockThreads, 0, stream>>>(
        row_offsets, group_count, edge_ids);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_implicit_gemm_view_workspace_bytes(int32_t source_rows) {
    return align_up(sizeof(Slot) * table_slots(source_rows)) + 1024;
}

int lat_build_relation_implicit_gemm_view(
    const int32_t* source_coords, int32_t source_rows, const int32_t* source_active_rows,
    const int32_t* output_coords, int32_t output_rows, const int32_t* output_active_rows,
    const int32_t* offsets, int32_t kernel_count, lat_triple stride, lat_triple padding,
    int32_t* out_in_map, int32_t* row_masks,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(source_rows >= 0 && output_rows >= 0 && kernel_count > 0,
                "implicit GEMM view sizes must be non-negative.");
    LAT_REQUIRE(source_active_rows != nullptr && output_active_rows != nullptr,
                "active_rows must have shape (1,) and int32 dtype.");
    cudaStream_t stream = as_stream(stream_ptr);
    int words = (kernel_count + 31) / 32;
    if (output_rows == 0) {
        return LAT_OK;
    }
    Workspace ws(workspace, workspace_bytes);
    int capacity = table_slots(source_rows);
    Slot* table = ws.take<Slot>(capacity);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the implicit GEMM view.");
    }
    uint32_t mask = static_cast<uint32_t>(capacity - 1);
    LAT_CUDA_CHECK(clear_table(table, capacity, stream));
    if (source_rows > 0) {
        // the reference hashes every source row and filters hits by the active count
        // afterwards (coordinates/cpu/relation_views_detail.h:122-169)
        insert_all_rows_kernel<<<blocks_for(source_rows), kBlockThreads, 0, stream>>>(
            source_coords, source_rows, table, mask, status);
        LAT_LAUNCH_CHECK();
    }
    igemm_view_kernel<<<blocks_for(output_rows, kWarpsPerBlock), kBlockThreads, 0, stream>>>(
        source_coords, table, mask, source_active_rows, source_rows, output_coords,
        output_active_rows, output_rows, offsets, kernel_count, words, stride.x, stride.y,
        stride.z, padding.x, padding.y, padding.z, out_in_map, row_masks);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_coord_set_workspace_bytes(int32_t rows) {
    size_t r = static_cast<size_t>(std::max(rows, 1));
    return align_up(sizeof(Slot) * table_slots(r)) +
           align_up(sizeof(int32_t) * ((r + kBlockThreads) / kBlockThreads + 1)) + 1024;
}

int lat_downsample_coords(
    const int32_t* coords, int32_t rows, lat_triple stride,
    int32_t* out_coords, int32_t* count,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0, "coords must have shape (N, 4).");
    LAT_REQUIRE(stride.x > 0 && stride.y > 0 && stride.z > 0, "stride values must be positive.");
    cudaStream_t stream = as_stream(stream_ptr);
    if (rows == 0) {
        LAT_CUDA_CHECK(fill_i32(count, 1, 0, stream));
        return LAT_OK;
    }
    Workspace ws(workspace, workspace_bytes);
    int capacity = table_slots(rows);
    Slot* table = ws.take<Slot>(capacity);
    int nblocks = blocks_for(rows);
    int32_t* sums = ws.take<int32_t>(nblocks);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the coordinate set.");
    }
    uint32_t mask = static_cast<uint32_t>(capacity - 1);
    LAT_CUDA_CHECK(clear_table(table, capacity, stream));
    LAT_CUDA_CHECK(fill_i32(out_coords, static_cast<size_t>(rows) * 4, 0, stream));
    insert_downsampled_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        coords, nullptr, rows, stride.x, stride.y, stride.z, table, mask, status);
    LAT_LAUNCH_CHECK();
    mark_winners_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        coords, nullptr, rows, stride.x, stride.y, stride.z, table, mask, sums);
    LAT_LAUNCH_CHECK();
    const int prescanned = nblocks > kSelfScanBlocks ? 1 : 0;
    if (prescanned) {
        scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
            sums, nblocks, count, nullptr, nullptr, 0, nullptr, 0, nullptr);
        LAT_LAUNCH_CHECK();
    }
    compact_winners_kernel<<<nblocks, kBlockThreads, 0, stream>>>(
        coords, nullptr, rows, stride.x, stride.y, stride.z, table, mask, sums, prescanned, count,
        out_coords, rows, status);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_lookup_coords(
    const int32_t* coords, int32_t rows, const int32_t* queries, int32_t query_rows,
    int32_t* out_rows,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0 && query_rows >= 0, "coords must have shape (N, 4).");
    cudaStream_t stream = as_stream(stream_ptr);
    if (query_rows == 0) {
        return LAT_OK;
    }
    Workspace ws(workspace, workspace_bytes);
    int capacity = table_slots(rows);
    Slot* table = ws.take<Slot>(capacity);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the coordinate set.");
    }
    uint32_t mask = static_cast<uint32_t>(capacity - 1);
    LAT_CUDA_CHECK(clear_table(table, capacity, stream));
    if (rows > 0) {
        insert_all_rows_kernel<<<blocks_for(rows), kBlockThreads, 0, stream>>>(
            coords, rows, table, mask, status);
        LAT_LAUNCH_CHECK();
    }
    lookup_kernel<<<blocks_for(query_rows), kBlockThreads, 0, stream>>>(
        coords, table, mask, queries, query_rows, nullptr, out_rows);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_sparse_alignment_workspace_bytes(int32_t lhs_rows, int32_t rhs_rows) {
    size_t l = static_cast<size_t>(std::max(lhs_rows, 1));
    size_t r = static_cast<size_t>(std::max(rhs_rows, 1));
    return align_up(sizeof(Slot) * table_slots(l)) +
           align_up(sizeof(Slot) * table_slots(r)) + align_up(sizeof(int32_t) * l) +
           align_up(sizeof(int32_t) * r) +
           2 * align_up(sizeof(int32_t) * ((std::max(l, r) + kBlockThreads) / kBlockThreads + 1)) +
           2048;
}

int lat_build_sparse_alignment(
    const int32_t* lhs_coords, int32_t lhs_rows, const int32_t* lhs_active_rows,
    const int32_t* rhs_coords, int32_t rhs_rows, const int32_t* rhs_active_rows,
    int32_t join,
    int32_t* out_coords, int32_t* out_count, int32_t* out_lhs_rows, int32_t* out_rhs_rows,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(lhs_rows >= 0 && rhs_rows >= 0, "coords must have shape (N, 4).");
    LAT_REQUIRE(lhs_active_rows != nullptr && rhs_active_rows != nullptr,
                "active_rows must have shape (1,) and int32 dtype.");
    LAT_REQUIRE(join >= LAT_JOIN_INNER && join <= LAT_JOIN_OUTER,
                "join must be 'inner', 'left', 'right', or 'outer'.");
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    int out_capacity = join == LAT_JOIN_RIGHT
                           ? rhs_rows
                           : (join == LAT_JOIN_OUTER ? lhs_rows + rhs_rows : lhs_rows);
    SourceTable lhs_table, rhs_table;
    int rc = build_source_table(ws, lhs_coords, lhs_rows, lhs_active_rows, status, false, stream,
                                lhs_table);
    if (rc != LAT_OK) {
        return rc;
    }
    rc = build_source_table(ws, rhs_coords, rhs_rows, rhs_active_rows, status, false, stream,
                            rhs_table);
    if (rc != LAT_OK) {
        return rc;
    }
    if (join == LAT_JOIN_RIGHT) {
        align_right_kernel<<<std::max(1, blocks_for(rhs_rows)), kBlockThreads, 0, stream>>>(
            rhs_coords, rhs_active_rows, rhs_rows, lhs_coords, lhs_table.slots, lhs_table.mask,
            out_coords, out_lhs_rows, out_rhs_rows, out_count);
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    LAT_CUDA_CHECK(fill_i32(out_coords, static_cast<size_t>(out_capacity) * 4, 0, stream));
    LAT_CUDA_CHECK(fill_i32(out_lhs_rows, out_capacity, -1, stream));
    LAT_CUDA_CHECK(fill_i32(out_rhs_rows, out_capacity, -1, stream));
    int lblocks = std::max(1, blocks_for(lhs_rows));
    int rblocks = std::max(1, blocks_for(rhs_rows));
    int32_t* match = ws.take<int32_t>(std::max(lhs_rows, 1));
    int32_t* absent = ws.take<int32_t>(std::max(rhs_rows, 1));
    int32_t* lsums = ws.take<int32_t>(lblocks);
    int32_t* rsums = ws.take<int32_t>(rblocks);
    int32_t* rtotal = ws.take<int32_t>(1);
    int32_t* ltotal = ws.take<int32_t>(1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the alignment.");
    }
    int inner = join == LAT_JOIN_INNER;
    align_lhs_count_kernel<<<lblocks, kBlockThreads, 0, stream>>>(
        lhs_coords, lhs_active_rows, lhs_rows, rhs_coords, rhs_table.slots, rhs_table.mask, inner,
        match, lsums);
    LAT_LAUNCH_CHECK();
    scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
        lsums, lblocks, join == LAT_JOIN_OUTER ? ltotal : out_count, nullptr, nullptr, 0, nullptr,
        0, nullptr);
    LAT_LAUNCH_CHECK();
    align_lhs_fill_kernel<<<lblocks, kBlockThreads, 0, stream>>>(
        lhs_coords, lhs_active_rows, lhs_rows, inner, match, lsums, out_coords, out_lhs_rows,
        out_rhs_rows);
    LAT_LAUNCH_CHECK();
    if (join == LAT_JOIN_OUTER) {
        align_rhs_count_kernel<<<rblocks, kBlockThreads, 0, stream>>>(
            rhs_coords, rhs_active_rows, rhs_rows, lhs_coords, lhs_table.slots, lhs_table.mask,
            absent, rsums);
        LAT_LAUNCH_CHECK();
        scan_blocks_kernel<<<1, kBlockThreads, 0, stream>>>(
            rsums, rblocks, rtotal, nullptr, nullptr, 0, nullptr, 0, nullptr);
        LAT_LAUNCH_CHECK();
        align_rhs_fill_kernel<<<rblocks, kBlockThreads, 0, stream>>>(
            rhs_coords, rhs_active_rows, rhs_rows, absent, rsums, ltotal, out_coords,
            out_lhs_rows, out_rhs_rows, out_count, rtotal);
        LAT_LAUNCH_CHECK();
    }
    return LAT_OK;
}

} // extern "C"
