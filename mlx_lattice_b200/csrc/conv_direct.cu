// CUDA-core route of the sparse-conv contraction: exact float32 arithmetic in the
// reference's own summation order (edges of an output row in CSR order, input
// channels ascending; convolution/cpu/algorithms.cpp:206-238, cpu/quantized.cpp:94-138).
// It serves float32 features (1e-5 parity needs true fp32 products), channel counts
// the tensor-core route does not tile, and kernel volumes above 32.
//
// Two kernels: `prepare_weights` rewrites any accepted weight form -- kernel-major,
// dense 5-D, or packed int4/int8 with per-group scale and bias -- into float32
// (K, C_in, C_out) in the caller's workspace (w = code*scale + bias evaluated in
// float32 like the reference); `direct_conv` gives one warp per output row, lanes
// across output channels.
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void prepare_float_weights_kernel(
    const T* weights, int layout, int K, int c_in, int c_out, float* out
) {
    size_t total = static_cast<size_t>(K) * c_in * c_out;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i >= total) {
        return;
    }
    int co = static_cast<int>(i % c_out);
    size_t rest = i / c_out;
    int ci = static_cast<int>(rest % c_in);
    int k = static_cast<int>(rest / c_in);
    size_t src = layout == LAT_WEIGHT_KERNEL_MAJOR
                     ? i
                     : (static_cast<size_t>(co) * K + k) * c_in + ci;  // (C_out, K, C_in)
    out[i] = to_float<T>(weights[src]);
}

template <typename T>
__global__ void prepare_quantized_weights_kernel(
    const uint32_t* packed, const T* scales, const T* biases, int K, int c_in, int c_out,
    int storage, int group_size, int bits, float* out
) {
    size_t total = static_cast<size_t>(K) * c_in * c_out;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i >= total) {
        return;
    }
    int co = static_cast<int>(i % c_out);
    size_t rest = i / c_out;
    int ci = static_cast<int>(rest % c_in);
    int k = static_cast<int>(rest / c_in);
    int words = storage * bits / 32;
    int groups = storage / group_size;
    int bit = ci * bits;
    uint32_t word = packed[(static_cast<size_t>(k) * words + (bit >> 5)) * c_out + co];
    uint32_t code = (word >> (bit & 31)) & ((1u << bits) - 1u);
    size_t q = (static_cast<size_t>(k) * groups + ci / group_size) * c_out + co;
    // code*scale + bias as one fused multiply-add, which is what optimising C++
    // compilers make of the reference's scalar expression on FMA hardware
    out[i] = fmaf(static_cast<float>(code), to_float<T>(scales[q]), to_float<T>(biases[q]));
}

constexpr int kDirectWarps = 8;
constexpr int kMaxOutPerLane = 8;  // C_out <= 256 per pass

template <typename T>
__global__ void __launch_bounds__(kDirectWarps * 32) direct_conv_kernel(
    const T* feats, long long feat_stride, int in_capacity, const float* weights, int K,
    int c_in, int c_out, const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity,
    const int32_t* counts, const int32_t* row_offsets, int out_capacity, const T* bias, T* out,
    int32_t* status
) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * kDirectWarps + (threadIdx.x >> 5);
    if (row >= out_capacity) {
        return;
    }
    int edge_total = min(max(__ldg(counts), 0), edge_capacity);
    int n_out = min(max(__ldg(counts + 1), 0), out_capacity);
    T* out_row = out + static_cast<size_t>(row) * c_out;
    for (int co0 = 0; co0 < c_out; co0 += 32 * kMaxOutPerLane) {
        float acc[kMaxOutPerLane];
#pragma unroll
        for (int j = 0; j < kMaxOutPerLane; ++j) {
            acc[j] = 0.0f;
        }
        if (row < n_out) {
            int begin = __ldg(row_offsets + row);
            int end = __ldg(row_offsets + row + 1);
            for (int e = begin; e < end; ++e) {
                if (e < 0 || e >= edge_total) {
                    continue;
                }
                int in_row = __ldg(in_rows + e);
                int k = __ldg(kernel_ids + e);
                if (in_row < 0 || k < 0) {
                    continue;
                }
                if (in_row >= in_capacity || k >= K) {
                    raise_status(status, LAT_STATUS_BAD_INDEX);
                    continue;
                }
                const T* x = feats + static_cast<size_t>(in_row) * feat_stride;
                const float* w = weights + static_cast<size_t>(k) * c_in * c_out + co0 + lane;
                for (int c0 = 0; c0 < c_in; c0 += 32) {
                    float xv = (c0 + lane < c_in) ? to_float<T>(x[c0 + lane]) : 0.0f;
                    int lim = min(32, c_in - c0);
                    for (int c = 0; c < lim; ++c) {
                        float v = __shfl_sync(0xffffffffu, xv, c);
                        const float* wc = w + static_cast<size_t>(c0 + c) * c_out;
#pragma unroll
                        for (int j = 0; j < kMaxOutPerLane; ++j) {
                            if (co0 + lane + 32 * j < c_out) {
                                acc[j] = fmaf(v, __ldg(wc + 32 * j), acc[j]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kMaxOutPerLane; ++j) {
            int co = co0 + lane + 32 * j;
            if (co < c_out) {
                T y = from_float<T>(acc[j]);
                if (bias != nullptr) {
                    y = from_float<T>(to_float<T>(y) + to_float<T>(bias[co]));
                }
                out_row[co] = y;
            }
        }
    }
}

// Narrow layers (C_in <= 8, C_out <= 32: a network's stem): one thread per output row
// with all output channels in registers and the fp32 weights in shared memory. A warp
// per row (the general kernel) leaves such a layer bound by its chain of dependent
// loads; here 32 rows per warp are in flight. Same fp32 summation order: edges
// ascending, input channels ascending, one fma per (edge, c_in, c_out).
constexpr int kNarrowMaxIn = 8;
constexpr int kNarrowMaxOut = 32;

template <typename T>
__global__ void __launch_bounds__(256) direct_conv_narrow_kernel(
    const T* feats, long long feat_stride, int in_capacity, const float* weights, int K,
    int c_in, int c_out, const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity,
    const int32_t* counts, const int32_t* row_offsets, int out_capacity, const T* bias, T* out,
    int32_t* status
) {
    extern __shared__ float w_smem[];  // [K * c_in][c_out + 1]: the pad spreads rows over banks
    const int pitch = c_out + 1;
    for (int i = threadIdx.x; i < K * c_in * c_out; i += blockDim.x) {
        w_smem[(i / c_out) * pitch + i % c_out] = weights[i];
    }
    __syncthreads();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= out_capacity) {
        return;
    }
    const int edge_total = min(max(__ldg(counts), 0), edge_capacity);
    const int n_out = min(max(__ldg(counts + 1), 0), out_capacity);
    float acc[kNarrowMaxOut];
#pragma unroll
    for (int j = 0; j < kNarrowMaxOut; ++j) {
        acc[j] = 0.0f;
    }
    if (row < n_out) {
        const int begin = max(__ldg(row_offsets + row), 0);
        const int end = min(__ldg(row_offsets + row + 1), edge_total);
        for (int e = begin; e < end; ++e) {
            const int in_row = __ldg(in_rows + e);
            const int k = __ldg(kernel_ids + e);
            if (in_row < 0 || k < 0) {
                continue;
            }
            if (in_row >= in_capacity || k >= K) {
                raise_status(status, LAT_STATUS_BAD_INDEX);
                continue;
            }
            const T* x = feats + static_cast<size_t>(in_row) * feat_stride;
            for (int c = 0; c < c_in; ++c) {
                const float v = to_float<T>(x[c]);
                const float* w = w_smem + (k * c_in + c) * pitch;
#pragma unroll
                for (int j = 0; j < kNarrowMaxOut; ++j) {
                    if (j < c_out) {
                        acc[j] = fmaf(v, w[j], acc[j]);
                    }
                }
            }
        }
    }
    T* out_row = out + static_cast<size_t>(row) * c_out;
    T y[kNarrowMaxOut];
#pragma unroll
    for (int j = 0; j < kNarrowMaxOut; ++j) {
        y[j] = from_float<T>(acc[j]);
        if (bias != nullptr && j < c_out) {
            y[j] = from_float<T>(to_float<T>(y[j]) + to_float<T>(bias[j]));
        }
    }
    if (sizeof(T) == 2 && (c_out & 7) == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
        // rows are 16-byte multiples: eight half values per store
#pragma unroll
        for (int j = 0; j < kNarrowMaxOut; j += 8) {
            if (j < c_out) {
                *reinterpret_cast<uint4*>(out_row + j) = *reinterpret_cast<const uint4*>(&y[j]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < kNarrowMaxOut; ++j) {
            if (j < c_out) {
                out_row[j] = y[j];
            }
        }
    }
}

inline int blocks_for(size_t count, int threads) {
    return static_cast<int>((count + threads - 1) / threads);
}

} // namespace

size_t direct_conv_workspace_bytes(int n_kernels, int in_channels, int out_channels) {
    return align_up(sizeof(float) * static_cast<size_t>(std::max(n_kernels, 1)) *
                    std::max(in_channels, 1) * std::max(out_channels, 1));
}

// Runs the CUDA-core route. Exactly one of (weights) or (packed, scales, biases) is set.
int run_direct_conv(
    int dtype, const void* feats, int in_capacity, int in_channels, long long feat_stride,
    const void* weights, int weight_layout, const uint32_t* packed, const void* scales,
    const void* biases, int storage_in_channels, int group_size, int bits, int out_channels,
    const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity, const int32_t* counts,
    const int32_t* row_offsets, int out_capacity, int n_kernels, const void* bias, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, cudaStream_t stream
) {
    Workspace ws(workspace, workspace_bytes);
    size_t total = static_cast<size_t>(n_kernels) * in_channels * out_channels;
    float* w32 = ws.take<float>(total);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the convolution.");
    }
    if (out_capacity == 0) {
        return LAT_OK;
    }
    int prep_blocks = blocks_for(total, 256);
    if (packed != nullptr) {
        if (dtype == LAT_F32) {
            prepare_quantized_weights_kernel<float><<<prep_blocks, 256, 0, stream>>>(
                packed, static_cast<const float*>(scales), static_cast<const float*>(biases),
                n_kernels, in_channels, out_channels, storage_in_channels, group_size, bits, w32);
        } else {
            prepare_quantized_weights_kernel<__half><<<prep_blocks, 256, 0, stream>>>(
                packed, static_cast<const __half*>(scales), static_cast<const __half*>(biases),
                n_kernels, in_channels, out_channels, storage_in_channels, group_size, bits, w32);
        }
    } else if (dtype == LAT_F32) {
        prepare_float_weights_kernel<float><<<prep_blocks, 256, 0, stream>>>(
            static_cast<const float*>(weights), weight_layout, n_kernels, in_channels,
            out_channels, w32);
    } else {
        prepare_float_weights_kernel<__half><<<prep_blocks, 256, 0, stream>>>(
            static_cast<const __half*>(weights), weight_layout, n_kernels, in_channels,
            out_channels, w32);
    }
    LAT_LAUNCH_CHECK();
    const size_t narrow_smem = sizeof(float) * static_cast<size_t>(n_kernels) * in_channels * (out_channels + 1);
    if (in_channels <= kNarrowMaxIn && out_channels <= kNarrowMaxOut && narrow_smem <= 48 * 1024) {
        const int narrow_blocks = blocks_for(out_capacity, 256);
        if (dtype == LAT_F32) {
            direct_conv_narrow_kernel<float><<<narrow_blocks, 256, narrow_smem, stream>>>(
                static_cast<const float*>(feats), feat_stride, in_capacity, w32, n_kernels,
                in_channels, out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
                out_capacity, static_cast<const float*>(bias), static_cast<float*>(out), status);
        } else {
            direct_conv_narrow_kernel<__half><<<narrow_blocks, 256, narrow_smem, stream>>>(
                static_cast<const __half*>(feats), feat_stride, in_capacity, w32, n_kernels,
                in_channels, out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
                out_capacity, static_cast<const __half*>(bias), static_cast<__half*>(out), status);
        }
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    int blocks = blocks_for(out_capacity, kDirectWarps);
    if (dtype == LAT_F32) {
        direct_conv_kernel<float><<<blocks, kDirectWarps * 32, 0, stream>>>(
            static_cast<const float*>(feats), feat_stride, in_capacity, w32, n_kernels,
            in_channels, out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
            out_capacity, static_cast<const float*>(bias), static_cast<float*>(out), status);
    } else {
        direct_conv_kernel<__half><<<blocks, kDirectWarps * 32, 0, stream>>>(
            static_cast<const __half*>(feats), feat_stride, in_capacity, w32, n_kernels,
            in_channels, out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
            out_capacity, static_cast<const __half*>(bias), static_cast<__half*>(out), status);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // namespace lat
