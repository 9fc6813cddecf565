// Sparse pooling (gather-reduce over the output CSR) and per-batch global pooling.
// Bandwidth-bound: one warp per output row, lanes across channels, so every gathered
// input row is read as contiguous 128-byte segments. float32 only, like the reference
// (pooling/validation.cpp:20-24).
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kPoolWarps = 8;

template <int Reduce>
__global__ void __launch_bounds__(kPoolWarps * 32) sparse_pool_kernel(
    const float* feats, long long feat_stride, int in_capacity, int channels,
    const int32_t* in_rows, int edge_capacity, const int32_t* row_offsets,
    const int32_t* counts, int out_capacity, float* out, int32_t* status
) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * kPoolWarps + (threadIdx.x >> 5);
    if (row >= out_capacity) {
        return;
    }
    int n_out = min(max(__ldg(counts + 1), 0), out_capacity);
    const float identity = Reduce == LAT_REDUCE_MAX ? -INFINITY : 0.0f;
    int begin = 0, end = 0;
    if (row < n_out) {
        begin = __ldg(row_offsets + row);
        end = __ldg(row_offsets + row + 1);
    }
    // pooling/cpu/algorithms.cpp:236-241: scale = 1 / max(degree, 1), applied last
    float scale = 1.0f / static_cast<float>(max(end - begin, 1));
    for (int c0 = 0; c0 < channels; c0 += 128) {
        float acc[4] = {identity, identity, identity, identity};
        for (int e = begin; e < end; ++e) {
            if (e < 0 || e >= edge_capacity) {
                continue;
            }
            int in_row = __ldg(in_rows + e);
            if (in_row < 0 || in_row >= in_capacity) {
                raise_status(status, LAT_STATUS_BAD_INDEX);
                continue;
            }
            const float* x = feats + static_cast<size_t>(in_row) * feat_stride + c0 + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (c0 + lane + 32 * j < channels) {
                    float v = __ldg(x + 32 * j);
                    acc[j] = Reduce == LAT_REDUCE_MAX ? fmaxf(acc[j], v) : acc[j] + v;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int c = c0 + lane + 32 * j;
            if (c < channels) {
                float v = acc[j];
                if (Reduce == LAT_REDUCE_AVG && row < n_out) {
                    v *= scale;
                }
                out[static_cast<size_t>(row) * channels + c] = v;
            }
        }
    }
}

// one block per (batch, 32-channel group); warps stride over the batch's rows and
// their partial results are combined in a fixed order (no float atomics)
template <int Reduce>
__global__ void __launch_bounds__(256) global_pool_kernel(
    const float* feats, int rows, int channels, const int32_t* batch_offsets, float* out
) {
    __shared__ float partial[8][32];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int batch = blockIdx.x;
    int c = blockIdx.y * 32 + lane;
    int begin = min(max(__ldg(batch_offsets + batch), 0), rows);
    int end = min(max(__ldg(batch_offsets + batch + 1), begin), rows);
    float acc = Reduce == LAT_REDUCE_MAX ? -INFINITY : 0.0f;
    if (c < channels) {
        for (int r = begin + warp; r < end; r += 8) {
            float v = __ldg(feats + static_cast<size_t>(r) * channels + c);
            acc = Reduce == LAT_REDUCE_MAX ? fmaxf(acc, v) : acc + v;
        }
    }
    partial[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && c < channels) {
        float total = partial[0][lane];
        for (int w = 1; w < 8; ++w) {
            total = Reduce == LAT_REDUCE_MAX ? fmaxf(total, partial[w][lane])
                                             : total + partial[w][lane];
        }
        if (Reduce == LAT_REDUCE_AVG) {
            // ops/pool.py:226-231: sums / max(count, 1); an empty batch stays 0
            total = total / static_cast<float>(max(end - begin, 1));
        }
        out[static_cast<size_t>(batch) * channels + c] = total;
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

int lat_sparse_pool_features(
    const float* feats, int32_t in_capacity, int32_t channels, int64_t feat_row_stride,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* row_offsets, const int32_t* counts,
    int32_t input_exclusive, int32_t reduce, int32_t out_capacity, int32_t n_kernels,
    float* out, int32_t* status, void* stream_ptr
) {
    (void)out_rows, (void)kernel_ids, (void)input_exclusive, (void)n_kernels;
    LAT_REQUIRE(channels > 0 && in_capacity >= 0, "feats must have shape (N, C).");
    LAT_REQUIRE(out_capacity >= 0 && edge_capacity >= 0,
                "out_capacity must be non-negative.");
    LAT_REQUIRE(reduce >= LAT_REDUCE_SUM && reduce <= LAT_REDUCE_AVG,
                "reduce must be 'sum', 'max', or 'avg'.");
    LAT_REQUIRE(counts != nullptr && row_offsets != nullptr,
                "counts must have shape (2,) and int32 dtype.");
    if (out_capacity == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    int blocks = (out_capacity + kPoolWarps - 1) / kPoolWarps;
    if (reduce == LAT_REDUCE_SUM) {
        sparse_pool_kernel<LAT_REDUCE_SUM><<<blocks, kPoolWarps * 32, 0, stream>>>(
            feats, feat_row_stride, in_capacity, channels, in_rows, edge_capacity, row_offsets,
            counts, out_capacity, out, status);
    } else if (reduce == LAT_REDUCE_MAX) {
        sparse_pool_kernel<LAT_REDUCE_MAX><<<blocks, kPoolWarps * 32, 0, stream>>>(
            feats, feat_row_stride, in_capacity, channels, in_rows, edge_capacity, row_offsets,
            counts, out_capacity, out, status);
    } else {
        sparse_pool_kernel<LAT_REDUCE_AVG><<<blocks, kPoolWarps * 32, 0, stream>>>(
            feats, feat_row_stride, in_capacity, channels, in_rows, edge_capacity, row_offsets,
            counts, out_capacity, out, status);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_global_pool(
    const float* feats, int32_t rows, int32_t channels, const int32_t* batch_offsets,
    int32_t batches, int32_t reduce, float* out, void* stream_ptr
) {
    LAT_REQUIRE(channels > 0 && rows >= 0, "feats must have shape (N, C).");
    LAT_REQUIRE(batches >= 0 && batch_offsets != nullptr,
                "batch_counts metadata is required for global pooling.");
    LAT_REQUIRE(reduce >= LAT_REDUCE_SUM && reduce <= LAT_REDUCE_AVG,
                "mode must be 'sum', 'max', or 'avg'.");
    if (batches == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    dim3 grid(batches, (channels + 31) / 32);
    if (reduce == LAT_REDUCE_SUM) {
        global_pool_kernel<LAT_REDUCE_SUM><<<grid, 256, 0, stream>>>(
            feats, rows, channels, batch_offsets, out);
    } else if (reduce == LAT_REDUCE_MAX) {
        global_pool_kernel<LAT_REDUCE_MAX><<<grid, 256, 0, stream>>>(
            feats, rows, channels, batch_offsets, out);
    } else {
        global_pool_kernel<LAT_REDUCE_AVG><<<grid, 256, 0, stream>>>(
            feats, rows, channels, batch_offsets, out);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"
