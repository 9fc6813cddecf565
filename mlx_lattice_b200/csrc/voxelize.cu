// Point -> voxel front end on the coordinate hash table.
//
// lat_sparse_quantize: voxel coordinate of every active point, (batch, floor((p - origin)
// / voxel_size)) in float32 arithmetic; the unique voxels in first-seen point order, the
// voxel row of every point and the points per voxel. Same machinery as the strided
// output support: a table keyed by the voxel coordinate keeps the lowest point row of
// each voxel (the "winner"), winners are compacted stably, and every point then looks its
// voxel up. Integer atomics only; the result does not depend on scheduling.
//
// lat_voxelize_features: per-voxel sum or mean of float32 point features, accumulated in
// ascending point order with one fused multiply-add per term (the order and rounding of
// the reference's sequential loop): the points of a voxel come from the stable grouped
// view of the inverse rows, one warp per voxel, lanes across channels.
//
// lat_build_point_voxel_map / lat_interpolate_point_features: the way back. Every point
// gets eight (voxel row, weight) slots: the nearest voxel centre with weight 1, or the
// eight corners of its cell with trilinear weights; corners that are not voxels stay
// (-1, 0). Interpolation is the weighted sum over the slots in slot order.
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kVoxThreads = 256;

struct PointKey {
    const float* points;
    const int32_t* batch;
    float vx, vy, vz;
    float ox, oy, oz;
    __device__ __forceinline__ Coord operator()(int row) const {
        const float* p = points + static_cast<size_t>(row) * 3;
        // (p - origin) / voxel_size, each operation rounded to float32, then floor
        const float x = floorf(__fdiv_rn(__fsub_rn(p[0], ox), vx));
        const float y = floorf(__fdiv_rn(__fsub_rn(p[1], oy), vy));
        const float z = floorf(__fdiv_rn(__fsub_rn(p[2], oz), vz));
        return {batch != nullptr ? batch[row] : 0, static_cast<int>(x), static_cast<int>(y),
                static_cast<int>(z)};
    }
};

__global__ void __launch_bounds__(kVoxThreads) quantize_insert_kernel(
    PointKey key_of, const int32_t* active_ptr, int rows, Slot* table, uint32_t mask, int32_t* status
) {
    const int active = active_ptr != nullptr ? clamp_count(active_ptr, rows) : rows;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row < active && !table_insert(table, mask, row, key_of(row), key_of, nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

// block-wide exclusive scan of one int per thread
__device__ __forceinline__ int vox_block_scan(int value, int& block_total) {
    __shared__ int warp_totals[kVoxThreads / 32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int wtotal;
    const int prefix = warp_exclusive_scan(value, wtotal);
    if (lane == 31) {
        warp_totals[warp] = wtotal;
    }
    __syncthreads();
    int before = 0;
    int total = 0;
    for (int w = 0; w < kVoxThreads / 32; ++w) {
        if (w < warp) {
            before += warp_totals[w];
        }
        total += warp_totals[w];
    }
    block_total = total;
    __syncthreads();
    return before + prefix;
}

__global__ void __launch_bounds__(kVoxThreads) quantize_mark_kernel(
    PointKey key_of, const int32_t* active_ptr, int rows, const Slot* table, uint32_t mask,
    int32_t* winner_of, int32_t* block_sums
) {
    const int active = active_ptr != nullptr ? clamp_count(active_ptr, rows) : rows;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    int win = 0;
    if (row < active) {
        const int winner = table_find(table, mask, key_of(row), key_of);
        winner_of[row] = winner;
        win = winner == row;
    }
    int total;
    vox_block_scan(win, total);
    if (threadIdx.x == 0) {
        block_sums[blockIdx.x] = total;
    }
}

// exclusive scan of the block sums in place (one block), total to *count
__global__ void __launch_bounds__(kVoxThreads) quantize_scan_kernel(
    int32_t* block_sums, int blocks, int32_t* count
) {
    __shared__ int carry;
    if (threadIdx.x == 0) {
        carry = 0;
    }
    __syncthreads();
    for (int first = 0; first < blocks; first += kVoxThreads) {
        const int i = first + threadIdx.x;
        const int v = i < blocks ? block_sums[i] : 0;
        int total;
        const int prefix = vox_block_scan(v, total);
        const int base = carry;
        if (i < blocks) {
            block_sums[i] = base + prefix;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry = base + total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        count[0] = carry;
    }
}

__global__ void __launch_bounds__(kVoxThreads) quantize_compact_kernel(
    PointKey key_of, const int32_t* active_ptr, int rows, const int32_t* winner_of,
    const int32_t* block_offsets, int32_t* out_coords, int32_t* voxel_of_winner
) {
    const int active = active_ptr != nullptr ? clamp_count(active_ptr, rows) : rows;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const int win = row < active && winner_of[row] == row;
    int total;
    const int pos = vox_block_scan(win, total) + block_offsets[blockIdx.x];
    if (win) {
        store_coord(out_coords, pos, key_of(row));
        voxel_of_winner[row] = pos;
    }
}

__global__ void __launch_bounds__(kVoxThreads) quantize_inverse_kernel(
    const int32_t* active_ptr, int rows, const int32_t* winner_of, const int32_t* voxel_of_winner,
    int32_t* inverse_rows, int32_t* voxel_counts
) {
    const int active = active_ptr != nullptr ? clamp_count(active_ptr, rows) : rows;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) {
        return;
    }
    int voxel = -1;
    if (row < active) {
        voxel = voxel_of_winner[winner_of[row]];
        atomicAdd(voxel_counts + voxel, 1);
    }
    inverse_rows[row] = voxel;
}

// one warp per voxel, lanes across channels, points in ascending order
__global__ void __launch_bounds__(kVoxThreads) voxel_reduce_kernel(
    const float* values, const int32_t* row_offsets, const int32_t* point_ids,
    const int32_t* voxel_counts, int point_rows, int voxel_rows, int channels, int mean, float* out
) {
    const int lane = threadIdx.x & 31;
    const int voxel = blockIdx.x * (kVoxThreads / 32) + (threadIdx.x >> 5);
    if (voxel >= voxel_rows) {
        return;
    }
    const int begin = row_offsets[voxel];
    const int end = row_offsets[voxel + 1];
    const float scale = mean != 0 ? __fdiv_rn(1.0f, static_cast<float>(max(voxel_counts[voxel], 1))) : 1.0f;
    for (int c0 = 0; c0 < channels; c0 += 32) {
        const int c = c0 + lane;
        float acc = 0.0f;
        for (int e = begin; e < end; ++e) {
            const int point = point_ids[e];
            if (c < channels && point >= 0 && point < point_rows) {
                acc = fmaf(values[static_cast<size_t>(point) * channels + c], scale, acc);
            }
        }
        if (c < channels) {
            out[static_cast<size_t>(voxel) * channels + c] = acc;
        }
    }
}

// few channels: one thread per output element (a warp per voxel would idle most lanes);
// same order and arithmetic
__global__ void __launch_bounds__(kVoxThreads) voxel_reduce_narrow_kernel(
    const float* values, const int32_t* row_offsets, const int32_t* point_ids,
    const int32_t* voxel_counts, int point_rows, long long elements, int channels, int mean, float* out
) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= elements) {
        return;
    }
    const int voxel = static_cast<int>(i / channels);
    const int c = static_cast<int>(i - static_cast<long long>(voxel) * channels);
    const int begin = row_offsets[voxel];
    const int end = row_offsets[voxel + 1];
    const float scale = mean != 0 ? __fdiv_rn(1.0f, static_cast<float>(max(voxel_counts[voxel], 1))) : 1.0f;
    float acc = 0.0f;
    for (int e = begin; e < end; ++e) {
        const int point = point_ids[e];
        if (point >= 0 && point < point_rows) {
            acc = fmaf(values[static_cast<size_t>(point) * channels + c], scale, acc);
        }
    }
    out[i] = acc;
}

// inverse rows outside [0, voxel_rows) take no part (the reference skips them): they are
// mapped to one extra trailing group that nobody reads
__global__ void voxel_group_ids_kernel(
    const int32_t* inverse_rows, const int32_t* active_ptr, int point_rows, int voxel_rows,
    int32_t* group_ids, int32_t* counts
) {
    const int active = clamp_count(active_ptr, point_rows);
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row == 0) {
        counts[0] = active;
        counts[1] = voxel_rows;
    }
    if (row < point_rows) {
        const int v = inverse_rows[row];
        group_ids[row] = (v >= 0 && v < voxel_rows) ? v : voxel_rows;
    }
}

struct PointFrame {
    const float* points;
    const int32_t* batch;
    float vx, vy, vz;
    float ox, oy, oz;
    // (p - origin) / voxel_size per axis, float32
    __device__ __forceinline__ void position(int row, float (&pos)[3]) const {
        const float* p = points + static_cast<size_t>(row) * 3;
        pos[0] = __fdiv_rn(__fsub_rn(p[0], ox), vx);
        pos[1] = __fdiv_rn(__fsub_rn(p[1], oy), vy);
        pos[2] = __fdiv_rn(__fsub_rn(p[2], oz), vz);
    }
};

__global__ void __launch_bounds__(kVoxThreads) voxel_table_insert_kernel(
    const int32_t* coords, const int32_t* active_ptr, int rows, Slot* table, uint32_t mask, int32_t* status
) {
    const int active = clamp_count(active_ptr, rows);
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    PlainKey key_of{coords};
    if (row < active && !table_insert(table, mask, row, key_of(row), key_of, nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

// one thread per (point, slot)
__global__ void __launch_bounds__(kVoxThreads) point_voxel_map_kernel(
    PointFrame frame, const int32_t* point_active_ptr, int point_rows, const int32_t* voxel_coords,
    const Slot* table, uint32_t mask, int linear, int32_t* rows_out, float* weights_out
) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(point_rows) * 8) {
        return;
    }
    const int point = static_cast<int>(i >> 3);
    const int corner = static_cast<int>(i & 7);
    int row = -1;
    float weight = 0.0f;
    if (point < clamp_count(point_active_ptr, point_rows)) {
        float pos[3];
        frame.position(point, pos);
        const int b = frame.batch != nullptr ? frame.batch[point] : 0;
        PlainKey key_of{voxel_coords};
        if (linear == 0) {
            if (corner == 0) {
                const Coord query{b, static_cast<int>(floorf(__fadd_rn(pos[0], 0.5f))),
                                  static_cast<int>(floorf(__fadd_rn(pos[1], 0.5f))),
                                  static_cast<int>(floorf(__fadd_rn(pos[2], 0.5f)))};
                row = table_find(table, mask, query, key_of);
                weight = row >= 0 ? 1.0f : 0.0f;
            }
        } else {
            const float lower[3] = {floorf(pos[0]), floorf(pos[1]), floorf(pos[2])};
            const float frac[3] = {__fsub_rn(pos[0], lower[0]), __fsub_rn(pos[1], lower[1]),
                                   __fsub_rn(pos[2], lower[2])};
            const int dx = corner & 1, dy = (corner >> 1) & 1, dz = (corner >> 2) & 1;
            const Coord query{b, static_cast<int>(lower[0]) + dx, static_cast<int>(lower[1]) + dy,
                              static_cast<int>(lower[2]) + dz};
            row = table_find(table, mask, query, key_of);
            if (row >= 0) {
                const float wx = dx == 0 ? __fsub_rn(1.0f, frac[0]) : frac[0];
                const float wy = dy == 0 ? __fsub_rn(1.0f, frac[1]) : frac[1];
                const float wz = dz == 0 ? __fsub_rn(1.0f, frac[2]) : frac[2];
                weight = __fmul_rn(__fmul_rn(wx, wy), wz);
            }
        }
    }
    rows_out[i] = row;
    weights_out[i] = weight;
}

// one thread per output element; slots in order, one fused multiply-add each
__global__ void __launch_bounds__(kVoxThreads) point_interpolate_kernel(
    const float* values, const int32_t* rows, const float* weights, long long elements, int voxel_rows,
    int channels, float* out
) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= elements) {
        return;
    }
    const long long point = i / channels;
    const int c = static_cast<int>(i - point * channels);
    float acc = 0.0f;
#pragma unroll
    for (int corner = 0; corner < 8; ++corner) {
        const int voxel = rows[point * 8 + corner];
        if (voxel >= 0 && voxel < voxel_rows) {
            acc = fmaf(values[static_cast<size_t>(voxel) * channels + c], weights[point * 8 + corner], acc);
        }
    }
    out[i] = acc;
}

inline int vox_blocks(long long count) { return static_cast<int>((count + kVoxThreads - 1) / kVoxThreads); }

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_sparse_quantize_workspace_bytes(int32_t rows) {
    const size_t r = static_cast<size_t>(std::max(rows, 1));
    return align_up(sizeof(Slot) * table_slots(static_cast<long long>(r))) + 2 * align_up(sizeof(int32_t) * r) +
           align_up(sizeof(int32_t) * (r / kVoxThreads + 2)) + 1024;
}

int lat_sparse_quantize(
    const float* points, const int32_t* batch_indices, int32_t rows, const int32_t* active_rows,
    lat_float_triple voxel_size, lat_float_triple origin,
    int32_t* out_coords, int32_t* count, int32_t* inverse_rows, int32_t* voxel_counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0, "points must have shape (N, 3).");
    LAT_REQUIRE(voxel_size.x > 0.0f && voxel_size.y > 0.0f && voxel_size.z > 0.0f,
                "voxel_size values must be positive.");
    LAT_REQUIRE(count != nullptr, "count is required.");
    LAT_REQUIRE(rows == 0 || (points != nullptr && out_coords != nullptr && inverse_rows != nullptr &&
                              voxel_counts != nullptr),
                "points, coords, inverse_rows and voxel_counts are required.");
    cudaStream_t stream = as_stream(stream_ptr);
    LAT_CUDA_CHECK(cudaMemsetAsync(count, 0, sizeof(int32_t), stream));
    if (rows == 0) {
        return LAT_OK;
    }
    Workspace ws(workspace, workspace_bytes);
    const int capacity = table_slots(rows);
    Slot* table = ws.take<Slot>(capacity);
    int32_t* winner_of = ws.take<int32_t>(rows);
    int32_t* voxel_of_winner = ws.take<int32_t>(rows);
    const int blocks = vox_blocks(rows);
    int32_t* sums = ws.take<int32_t>(blocks + 1);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the quantization.");
    }
    const uint32_t mask = static_cast<uint32_t>(capacity - 1);
    PointKey key_of{points, batch_indices, voxel_size.x, voxel_size.y, voxel_size.z,
                    origin.x, origin.y, origin.z};
    LAT_CUDA_CHECK(cudaMemsetAsync(table, 0xFF, sizeof(Slot) * capacity, stream));
    LAT_CUDA_CHECK(cudaMemsetAsync(out_coords, 0, sizeof(int32_t) * 4 * rows, stream));
    LAT_CUDA_CHECK(cudaMemsetAsync(voxel_counts, 0, sizeof(int32_t) * rows, stream));
    quantize_insert_kernel<<<blocks, kVoxThreads, 0, stream>>>(key_of, active_rows, rows, table, mask, status);
    LAT_LAUNCH_CHECK();
    quantize_mark_kernel<<<blocks, kVoxThreads, 0, stream>>>(key_of, active_rows, rows, table, mask,
                                                             winner_of, sums);
    LAT_LAUNCH_CHECK();
    quantize_scan_kernel<<<1, kVoxThreads, 0, stream>>>(sums, blocks, count);
    LAT_LAUNCH_CHECK();
    quantize_compact_kernel<<<blocks, kVoxThreads, 0, stream>>>(key_of, active_rows, rows, winner_of, sums,
                                                                out_coords, voxel_of_winner);
    LAT_LAUNCH_CHECK();
    quantize_inverse_kernel<<<blocks, kVoxThreads, 0, stream>>>(active_rows, rows, winner_of, voxel_of_winner,
                                                                inverse_rows, voxel_counts);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_voxelize_features_workspace_bytes(int32_t point_rows, int32_t voxel_rows) {
    const size_t p = static_cast<size_t>(std::max(point_rows, 1));
    const size_t v = static_cast<size_t>(std::max(voxel_rows, 1));
    return 2 * align_up(sizeof(int32_t) * p) + align_up(sizeof(int32_t) * (v + 2)) + 256 +
           lat_grouped_view_workspace_bytes(point_rows, voxel_rows + 1) + 1024;
}

int lat_voxelize_features(
    const float* values, const int32_t* inverse_rows, const int32_t* voxel_counts,
    const int32_t* active_rows, int32_t point_rows, int32_t voxel_rows, int32_t channels,
    int32_t mean, float* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(point_rows >= 0 && voxel_rows >= 0 && channels >= 0, "feats must have shape (N, C).");
    LAT_REQUIRE(active_rows != nullptr, "active_rows must have shape (1,) and int32 dtype.");
    cudaStream_t stream = as_stream(stream_ptr);
    if (voxel_rows == 0 || channels == 0) {
        return LAT_OK;
    }
    LAT_REQUIRE(out != nullptr && voxel_counts != nullptr, "out and voxel_counts are required.");
    if (point_rows == 0) {
        LAT_CUDA_CHECK(cudaMemsetAsync(out, 0, sizeof(float) * voxel_rows * channels, stream));
        return LAT_OK;
    }
    LAT_REQUIRE(values != nullptr && inverse_rows != nullptr, "feats and inverse_rows are required.");
    Workspace ws(workspace, workspace_bytes);
    int32_t* group_ids = ws.take<int32_t>(point_rows);
    int32_t* point_ids = ws.take<int32_t>(point_rows);
    int32_t* row_offsets = ws.take<int32_t>(static_cast<size_t>(voxel_rows) + 2);
    int32_t* counts = ws.take<int32_t>(2);
    const size_t view_bytes = lat_grouped_view_workspace_bytes(point_rows, voxel_rows + 1);
    void* view_ws = ws.take<char>(view_bytes);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the voxel reduction.");
    }
    voxel_group_ids_kernel<<<vox_blocks(point_rows), kVoxThreads, 0, stream>>>(
        inverse_rows, active_rows, point_rows, voxel_rows, group_ids, counts);
    LAT_LAUNCH_CHECK();
    int rc = lat_build_relation_grouped_view(group_ids, point_rows, counts, voxel_rows + 1, row_offsets,
                                             point_ids, view_ws, view_bytes, status, stream_ptr);
    if (rc != LAT_OK) {
        return rc;
    }
    if (channels < 16) {
        const long long elements = static_cast<long long>(voxel_rows) * channels;
        voxel_reduce_narrow_kernel<<<vox_blocks(elements), kVoxThreads, 0, stream>>>(
            values, row_offsets, point_ids, voxel_counts, point_rows, elements, channels, mean, out);
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    const int warps_per_block = kVoxThreads / 32;
    voxel_reduce_kernel<<<(voxel_rows + warps_per_block - 1) / warps_per_block, kVoxThreads, 0, stream>>>(
        values, row_offsets, point_ids, voxel_counts, point_rows, voxel_rows, channels, mean, out);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

size_t lat_point_voxel_map_workspace_bytes(int32_t voxel_rows) {
    return align_up(sizeof(Slot) * table_slots(std::max(voxel_rows, 1))) + 1024;
}

int lat_build_point_voxel_map(
    const float* points, const int32_t* batch_indices, int32_t point_rows,
    const int32_t* point_active_rows, const int32_t* voxel_coords, int32_t voxel_rows,
    const int32_t* voxel_active_rows, lat_float_triple voxel_size, lat_float_triple origin,
    int32_t linear, int32_t* rows_out, float* weights_out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(point_rows >= 0 && voxel_rows >= 0, "points must have shape (N, 3).");
    LAT_REQUIRE(voxel_size.x > 0.0f && voxel_size.y > 0.0f && voxel_size.z > 0.0f,
                "voxel_size values must be positive.");
    LAT_REQUIRE(point_active_rows != nullptr && voxel_active_rows != nullptr,
                "active_rows must have shape (1,) and int32 dtype.");
    if (point_rows == 0) {
        return LAT_OK;
    }
    LAT_REQUIRE(points != nullptr && rows_out != nullptr && weights_out != nullptr &&
                    (voxel_coords != nullptr || voxel_rows == 0),
                "points, voxel_coords, rows and weights are required.");
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    const int capacity = table_slots(std::max(voxel_rows, 1));
    Slot* table = ws.take<Slot>(capacity);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the point-voxel map.");
    }
    const uint32_t mask = static_cast<uint32_t>(capacity - 1);
    LAT_CUDA_CHECK(cudaMemsetAsync(table, 0xFF, sizeof(Slot) * capacity, stream));
    if (voxel_rows > 0) {
        voxel_table_insert_kernel<<<vox_blocks(voxel_rows), kVoxThreads, 0, stream>>>(
            voxel_coords, voxel_active_rows, voxel_rows, table, mask, status);
        LAT_LAUNCH_CHECK();
    }
    PointFrame frame{points, batch_indices, voxel_size.x, voxel_size.y, voxel_size.z,
                     origin.x, origin.y, origin.z};
    point_voxel_map_kernel<<<vox_blocks(static_cast<long long>(point_rows) * 8), kVoxThreads, 0, stream>>>(
        frame, point_active_rows, point_rows, voxel_coords, table, mask, linear, rows_out, weights_out);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_interpolate_point_features(
    const float* values, const int32_t* rows, const float* weights, int32_t point_rows,
    int32_t voxel_rows, int32_t channels, float* out, void* stream_ptr
) {
    LAT_REQUIRE(point_rows >= 0 && voxel_rows >= 0 && channels >= 0,
                "voxel_feats must have shape (N, C).");
    if (point_rows == 0 || channels == 0) {
        return LAT_OK;
    }
    LAT_REQUIRE(rows != nullptr && weights != nullptr && out != nullptr && (values != nullptr || voxel_rows == 0),
                "voxel_feats, rows, weights and out are required.");
    const long long elements = static_cast<long long>(point_rows) * channels;
    point_interpolate_kernel<<<vox_blocks(elements), kVoxThreads, 0, as_stream(stream_ptr)>>>(
        values, rows, weights, elements, voxel_rows, channels, out);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"
