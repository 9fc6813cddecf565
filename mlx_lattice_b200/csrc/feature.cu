// Pointwise feature operators of the inference path: linear / quantized linear
// (x @ W.T with float32 accumulation), inference batch-norm with optional fused ReLU,
// and ReLU. They stand in for the third-party array ops the reference calls
// (mlx_lattice/ops/feature.py:33-56,166-187, ops/_quantized.py:8-38).
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

constexpr int kRowsPerBlock = 32;
constexpr int kThreads = 256;

// Block: 32 rows staged in shared memory; thread t owns output channel(s) t, t+256, ...
// and keeps its weight row in registers/L1 across the 32 rows.
template <typename T, bool Quantized>
__global__ void __launch_bounds__(kThreads) linear_kernel(
    const T* feats, int rows, int c_in, const T* weight, const uint32_t* packed,
    const T* scales, const T* biases, int storage, int group_size, int bits, int c_out,
    const T* bias, T* out
) {
    extern __shared__ float x_tile[];  // [kRowsPerBlock][c_in]
    int row0 = blockIdx.x * kRowsPerBlock;
    int valid = min(kRowsPerBlock, rows - row0);
    for (int i = threadIdx.x; i < kRowsPerBlock * c_in; i += kThreads) {
        int r = i / c_in;
        int c = i - r * c_in;
        x_tile[i] = r < valid ? to_float<T>(feats[static_cast<size_t>(row0 + r) * c_in + c]) : 0.0f;
    }
    __syncthreads();
    int words = Quantized ? storage * bits / 32 : 0;
    int groups = Quantized ? storage / group_size : 0;
    for (int co = threadIdx.x; co < c_out; co += kThreads) {
        float acc[kRowsPerBlock];
#pragma unroll
        for (int r = 0; r < kRowsPerBlock; ++r) {
            acc[r] = 0.0f;
        }
        for (int ci = 0; ci < c_in; ++ci) {
            float w;
            if (Quantized) {
                int bit = ci * bits;
                uint32_t word = __ldg(packed + static_cast<size_t>(co) * words + (bit >> 5));
                uint32_t code = (word >> (bit & 31)) & ((1u << bits) - 1u);
                size_t q = static_cast<size_t>(co) * groups + ci / group_size;
                w = fmaf(static_cast<float>(code), to_float<T>(scales[q]), to_float<T>(biases[q]));
            } else {
                w = to_float<T>(weight[static_cast<size_t>(co) * c_in + ci]);
            }
#pragma unroll
            for (int r = 0; r < kRowsPerBlock; ++r) {
                acc[r] = fmaf(x_tile[r * c_in + ci], w, acc[r]);
            }
        }
        for (int r = 0; r < valid; ++r) {
            T y = from_float<T>(acc[r]);
            if (bias != nullptr) {
                y = from_float<T>(to_float<T>(y) + to_float<T>(bias[co]));
            }
            out[static_cast<size_t>(row0 + r) * c_out + co] = y;
        }
    }
}

// Few output channels (a classification head): one thread per row with every output in
// registers and the fp32 weight matrix in shared memory (all lanes read the same weight:
// a broadcast). Same summation order as linear_kernel: input channels ascending.
constexpr int kNarrowOut = 32;

template <typename T, bool Quantized>
__global__ void __launch_bounds__(kThreads) linear_narrow_kernel(
    const T* feats, int rows, int c_in, const T* weight, const uint32_t* packed,
    const T* scales, const T* biases, int storage, int group_size, int bits, int c_out,
    const T* bias, T* out
) {
    extern __shared__ float w_tile[];  // [c_in][c_out]
    const int words = Quantized ? storage * bits / 32 : 0;
    const int groups = Quantized ? storage / group_size : 0;
    for (int i = threadIdx.x; i < c_in * c_out; i += kThreads) {
        const int ci = i / c_out;
        const int co = i - ci * c_out;
        float w;
        if (Quantized) {
            const int bit = ci * bits;
            const uint32_t word = __ldg(packed + static_cast<size_t>(co) * words + (bit >> 5));
            const uint32_t code = (word >> (bit & 31)) & ((1u << bits) - 1u);
            const size_t q = static_cast<size_t>(co) * groups + ci / group_size;
            w = fmaf(static_cast<float>(code), to_float<T>(scales[q]), to_float<T>(biases[q]));
        } else {
            w = to_float<T>(weight[static_cast<size_t>(co) * c_in + ci]);
        }
        w_tile[i] = w;
    }
    __syncthreads();
    const int row = blockIdx.x * kThreads + threadIdx.x;
    float acc[kNarrowOut];
#pragma unroll
    for (int j = 0; j < kNarrowOut; ++j) {
        acc[j] = 0.0f;
    }
    if (row < rows) {
        const T* x = feats + static_cast<size_t>(row) * c_in;
        if (sizeof(T) == 2 && (c_in & 7) == 0 && reinterpret_cast<uintptr_t>(feats) % 16 == 0) {
            // eight half values per load
            for (int c0 = 0; c0 < c_in; c0 += 8) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + c0));
                const T* v8 = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float v = to_float<T>(v8[u]);
                    const float* w = w_tile + (c0 + u) * c_out;
                    if ((c_out & 3) == 0) {
                        // four weights per shared-memory read (rows of w_tile stay 16-byte aligned)
#pragma unroll
                        for (int j = 0; j < kNarrowOut; j += 4) {
                            if (j < c_out) {
                                const float4 w4 = *reinterpret_cast<const float4*>(w + j);
                                acc[j] = fmaf(v, w4.x, acc[j]);
                                acc[j + 1] = fmaf(v, w4.y, acc[j + 1]);
                                acc[j + 2] = fmaf(v, w4.z, acc[j + 2]);
                                acc[j + 3] = fmaf(v, w4.w, acc[j + 3]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < kNarrowOut; ++j) {
                            if (j < c_out) {
                                acc[j] = fmaf(v, w[j], acc[j]);
                            }
                        }
                    }
                }
            }
        } else {
            for (int ci = 0; ci < c_in; ++ci) {
                const float v = to_float<T>(x[ci]);
                const float* w = w_tile + ci * c_out;
#pragma unroll
                for (int j = 0; j < kNarrowOut; ++j) {
                    if (j < c_out) {
                        acc[j] = fmaf(v, w[j], acc[j]);
                    }
                }
            }
        }
    }
    // the block's output rows are one contiguous range: stage them in shared memory (the
    // weights are no longer needed) and write 16 bytes per thread
    __syncthreads();
    T* y_tile = reinterpret_cast<T*>(w_tile);  // [kThreads][c_out]
#pragma unroll
    for (int j = 0; j < kNarrowOut; ++j) {
        if (j < c_out) {
            T value = from_float<T>(acc[j]);
            if (bias != nullptr) {
                value = from_float<T>(to_float<T>(value) + to_float<T>(bias[j]));
            }
            y_tile[threadIdx.x * c_out + j] = value;
        }
    }
    __syncthreads();
    const int first_row = blockIdx.x * kThreads;
    const int valid_rows = min(kThreads, rows - first_row);
    const size_t bytes = static_cast<size_t>(valid_rows) * c_out * sizeof(T);
    char* dst = reinterpret_cast<char*>(out + static_cast<size_t>(first_row) * c_out);
    const char* src = reinterpret_cast<const char*>(y_tile);
    if (reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
        const size_t vectors = bytes / 16;
        for (size_t i = threadIdx.x; i < vectors; i += kThreads) {
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        }
        for (size_t i = vectors * 16 + threadIdx.x * sizeof(T); i < bytes; i += kThreads * sizeof(T)) {
            *reinterpret_cast<T*>(dst + i) = *reinterpret_cast<const T*>(src + i);
        }
    } else {
        for (size_t i = threadIdx.x * sizeof(T); i < bytes; i += kThreads * sizeof(T)) {
            *reinterpret_cast<T*>(dst + i) = *reinterpret_cast<const T*>(src + i);
        }
    }
}

template <typename T>
__global__ void batch_norm_relu_kernel(
    const T* feats, long long rows, int channels, const T* weight, const T* bias,
    const T* mean, const T* var, float eps, int apply_relu, T* out
) {
    long long total = rows * channels;
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (; i < total; i += stride) {
        int c = static_cast<int>(i % channels);
        float x = to_float<T>(feats[i]);
        float m = mean != nullptr ? to_float<T>(mean[c]) : 0.0f;
        float v = var != nullptr ? to_float<T>(var[c]) : 1.0f;
        float y = (x - m) * (1.0f / sqrtf(v + eps));
        if (weight != nullptr) {
            y *= to_float<T>(weight[c]);
        }
        if (bias != nullptr) {
            y += to_float<T>(bias[c]);
        }
        if (apply_relu) {
            y = fmaxf(y, 0.0f);
        }
        out[i] = from_float<T>(y);
    }
}

template <typename T>
__global__ void relu_kernel(const T* feats, long long total, T* out) {
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (; i < total; i += stride) {
        out[i] = from_float<T>(fmaxf(to_float<T>(feats[i]), 0.0f));
    }
}

// Pointwise activations of mlx_lattice/ops/feature.py:59-129, evaluated in float32 and cast
// once. p0 / p1: negative slope (leaky ReLU); beta and threshold (softplus).
enum Activation {
    kSigmoid = 0, kSilu = 1, kTanh = 2, kGeluErf = 3, kGeluTanh = 4, kGeluFast = 5,
    kLeakyRelu = 6, kSoftplus = 7,
};

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int Op> __device__ __forceinline__ float activate(float x, float p0, float p1) {
    switch (Op) {
        case kSigmoid: return sigmoid_f(x);
        case kSilu: return x * sigmoid_f(x);
        case kTanh: return tanhf(x);
        case kGeluErf: return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
        case kGeluTanh: return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        case kGeluFast: return x * sigmoid_f(1.702f * x);
        case kLeakyRelu: return x >= 0.0f ? x : x * p0;
        default: {
            const float scaled = x * p0;
            return scaled > p1 ? x : log1pf(expf(scaled)) / p0;
        }
    }
}

template <typename T, int Op>
__global__ void activation_kernel(const T* feats, long long total, float p0, float p1, T* out) {
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (; i < total; i += stride) {
        out[i] = from_float<T>(activate<Op>(to_float<T>(feats[i]), p0, p1));
    }
}

template <typename T, int Op>
void launch_activation(const void* feats, long long total, float p0, float p1, void* out,
                       int grid, cudaStream_t stream) {
    activation_kernel<T, Op><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(feats), total, p0, p1, static_cast<T*>(out));
}

template <typename T>
void dispatch_activation(int op, const void* feats, long long total, float p0, float p1, void* out,
                         int grid, cudaStream_t stream) {
    switch (op) {
        case kSigmoid: return launch_activation<T, kSigmoid>(feats, total, p0, p1, out, grid, stream);
        case kSilu: return launch_activation<T, kSilu>(feats, total, p0, p1, out, grid, stream);
        case kTanh: return launch_activation<T, kTanh>(feats, total, p0, p1, out, grid, stream);
        case kGeluErf: return launch_activation<T, kGeluErf>(feats, total, p0, p1, out, grid, stream);
        case kGeluTanh: return launch_activation<T, kGeluTanh>(feats, total, p0, p1, out, grid, stream);
        case kGeluFast: return launch_activation<T, kGeluFast>(feats, total, p0, p1, out, grid, stream);
        case kLeakyRelu: return launch_activation<T, kLeakyRelu>(feats, total, p0, p1, out, grid, stream);
        default: return launch_activation<T, kSoftplus>(feats, total, p0, p1, out, grid, stream);
    }
}

// Row-wise normalisations (mlx_lattice/ops/feature.py:196-225, which call the array
// library's fused layer_norm / rms_norm): one warp per row, statistics in float32 over
// the channels (mean, then the biased variance about it; or the mean square), then
// (x - mean) * rsqrt(var + eps) * weight + bias, or x * rsqrt(ms + eps) * weight.
template <typename T, bool Rms>
__global__ void __launch_bounds__(256) row_norm_kernel(
    const T* feats, long long rows, int channels, const T* weight, const T* bias, float eps, T* out
) {
    const int lane = threadIdx.x & 31;
    const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
    for (long long row = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
         row < rows; row += warps) {
        const T* x = feats + row * channels;
        float mean = 0.0f;
        if (!Rms) {
            float sum = 0.0f;
            for (int c = lane; c < channels; c += 32) {
                sum += to_float<T>(x[c]);
            }
            for (int delta = 16; delta > 0; delta >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, delta);
            }
            mean = sum / static_cast<float>(channels);
        }
        float squares = 0.0f;
        for (int c = lane; c < channels; c += 32) {
            const float d = to_float<T>(x[c]) - mean;
            squares = fmaf(d, d, squares);
        }
        for (int delta = 16; delta > 0; delta >>= 1) {
            squares += __shfl_xor_sync(0xffffffffu, squares, delta);
        }
        const float scale = rsqrtf(squares / static_cast<float>(channels) + eps);
        T* y = out + row * channels;
        for (int c = lane; c < channels; c += 32) {
            float v = (to_float<T>(x[c]) - mean) * scale;
            if (weight != nullptr) {
                v *= to_float<T>(weight[c]);
            }
            if (bias != nullptr) {
                v += to_float<T>(bias[c]);
            }
            y[c] = from_float<T>(v);
        }
    }
}

inline int elementwise_grid(long long total) {
    long long blocks = (total + 255) / 256;
    return static_cast<int>(std::max(1LL, std::min(blocks, 148LL * 32)));
}

template <typename T, bool Quantized>
int launch_linear(
    const void* feats, int rows, int c_in, const void* weight, const uint32_t* packed,
    const void* scales, const void* biases, int storage, int group_size, int bits, int c_out,
    const void* bias, void* out, cudaStream_t stream
) {
    if (c_out <= kNarrowOut && sizeof(float) * c_in * c_out <= 48 * 1024) {
        // shared memory holds the fp32 weights, then the block's output rows
        const size_t w_bytes = std::max(sizeof(float) * c_in * c_out, sizeof(T) * kThreads * c_out);
        linear_narrow_kernel<T, Quantized><<<(rows + kThreads - 1) / kThreads, kThreads, w_bytes, stream>>>(
            static_cast<const T*>(feats), rows, c_in, static_cast<const T*>(weight), packed,
            static_cast<const T*>(scales), static_cast<const T*>(biases), storage, group_size, bits,
            c_out, static_cast<const T*>(bias), static_cast<T*>(out));
        LAT_LAUNCH_CHECK();
        return LAT_OK;
    }
    size_t smem = sizeof(float) * kRowsPerBlock * c_in;
    if (smem > 48 * 1024) {
        LAT_CUDA_CHECK(cudaFuncSetAttribute(
            linear_kernel<T, Quantized>, cudaFuncAttributeMaxDynamicSharedMemorySize,
            static_cast<int>(smem)));
    }
    int blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    linear_kernel<T, Quantized><<<blocks, kThreads, smem, stream>>>(
        static_cast<const T*>(feats), rows, c_in, static_cast<const T*>(weight), packed,
        static_cast<const T*>(scales), static_cast<const T*>(biases), storage, group_size, bits,
        c_out, static_cast<const T*>(bias), static_cast<T*>(out));
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

int lat_linear(
    int32_t dtype, const void* feats, int32_t rows, int32_t in_channels,
    const void* weight, int32_t out_channels, const void* bias, void* out, void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "convolution supports float32 and float16 tensors.");
    LAT_REQUIRE(rows >= 0 && in_channels > 0 && out_channels > 0,
                "weight input channels must match x.channels.");
    LAT_REQUIRE(in_channels <= 1536, "linear supports at most 1536 input channels.");
    if (rows == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    if (dtype == LAT_F32) {
        return launch_linear<float, false>(feats, rows, in_channels, weight, nullptr, nullptr,
                                           nullptr, 0, 1, 0, out_channels, bias, out, stream);
    }
    return launch_linear<__half, false>(feats, rows, in_channels, weight, nullptr, nullptr,
                                        nullptr, 0, 1, 0, out_channels, bias, out, stream);
}

int lat_quantized_linear(
    int32_t dtype, const void* feats, int32_t rows, int32_t in_channels,
    const uint32_t* packed, const void* scales, const void* biases,
    int32_t out_channels, int32_t storage_in_channels, int32_t group_size, int32_t bits,
    const void* bias, void* out, void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "convolution supports float32 and float16 tensors.");
    LAT_REQUIRE(bits == 4 || bits == 8, "quantized weight bits must be 4 or 8.");
    LAT_REQUIRE(group_size == 32 || group_size == 64 || group_size == 128,
                "quantized weight group_size must be 32, 64, or 128.");
    LAT_REQUIRE(rows >= 0 && in_channels > 0 && out_channels > 0 &&
                    storage_in_channels >= in_channels && storage_in_channels % group_size == 0,
                "features must have shape (N, quantized_weight.in_channels).");
    LAT_REQUIRE(in_channels <= 1536, "linear supports at most 1536 input channels.");
    if (rows == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    if (dtype == LAT_F32) {
        return launch_linear<float, true>(feats, rows, in_channels, nullptr, packed, scales,
                                          biases, storage_in_channels, group_size, bits,
                                          out_channels, bias, out, stream);
    }
    return launch_linear<__half, true>(feats, rows, in_channels, nullptr, packed, scales, biases,
                                       storage_in_channels, group_size, bits, out_channels, bias,
                                       out, stream);
}

int lat_batch_norm_relu(
    int32_t dtype, const void* feats, int64_t rows, int32_t channels,
    const void* weight, const void* bias, const void* mean, const void* var, float eps,
    int32_t apply_relu, void* out, void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "batch_norm supports float32 and float16 tensors.");
    LAT_REQUIRE(eps > 0.0f, "eps must be positive.");
    LAT_REQUIRE(rows >= 0 && channels > 0, "feats must have shape (N, C).");
    if (rows == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    int grid = elementwise_grid(rows * channels);
    if (dtype == LAT_F32) {
        batch_norm_relu_kernel<float><<<grid, 256, 0, stream>>>(
            static_cast<const float*>(feats), rows, channels, static_cast<const float*>(weight),
            static_cast<const float*>(bias), static_cast<const float*>(mean),
            static_cast<const float*>(var), eps, apply_relu, static_cast<float*>(out));
    } else {
        batch_norm_relu_kernel<__half><<<grid, 256, 0, stream>>>(
            static_cast<const __half*>(feats), rows, channels, static_cast<const __half*>(weight),
            static_cast<const __half*>(bias), static_cast<const __half*>(mean),
            static_cast<const __half*>(var), eps, apply_relu, static_cast<__half*>(out));
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_relu(int32_t dtype, const void* feats, int64_t elements, void* out, void* stream_ptr) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "relu supports float32 and float16 tensors.");
    LAT_REQUIRE(elements >= 0, "feats must have shape (N, C).");
    if (elements == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    int grid = elementwise_grid(elements);
    if (dtype == LAT_F32) {
        relu_kernel<float><<<grid, 256, 0, stream>>>(
            static_cast<const float*>(feats), elements, static_cast<float*>(out));
    } else {
        relu_kernel<__half><<<grid, 256, 0, stream>>>(
            static_cast<const __half*>(feats), elements, static_cast<__half*>(out));
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_row_norm(
    int32_t dtype, int32_t rms, const void* feats, int64_t rows, int32_t channels,
    const void* weight, const void* bias, float eps, void* out, void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "normalisation supports float32 and float16 tensors.");
    LAT_REQUIRE(eps > 0.0f, "eps must be positive.");
    LAT_REQUIRE(rows >= 0 && channels > 0, "feats must have shape (N, C).");
    LAT_REQUIRE(!rms || bias == nullptr, "rms_norm has no bias.");
    if (rows == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((rows + 7) / 8, 148LL * 16)));
    if (dtype == LAT_F32) {
        auto* x = static_cast<const float*>(feats);
        auto* w = static_cast<const float*>(weight);
        auto* b = static_cast<const float*>(bias);
        auto* y = static_cast<float*>(out);
        if (rms) {
            row_norm_kernel<float, true><<<grid, 256, 0, stream>>>(x, rows, channels, w, b, eps, y);
        } else {
            row_norm_kernel<float, false><<<grid, 256, 0, stream>>>(x, rows, channels, w, b, eps, y);
        }
    } else {
        auto* x = static_cast<const __half*>(feats);
        auto* w = static_cast<const __half*>(weight);
        auto* b = static_cast<const __half*>(bias);
        auto* y = static_cast<__half*>(out);
        if (rms) {
            row_norm_kernel<__half, true><<<grid, 256, 0, stream>>>(x, rows, channels, w, b, eps, y);
        } else {
            row_norm_kernel<__half, false><<<grid, 256, 0, stream>>>(x, rows, channels, w, b, eps, y);
        }
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_activation(
    int32_t dtype, int32_t op, const void* feats, int64_t elements, float p0, float p1, void* out,
    void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "activations support float32 and float16 tensors.");
    LAT_REQUIRE(op >= kSigmoid && op <= kSoftplus, "unknown activation.");
    LAT_REQUIRE(elements >= 0, "feats must have shape (N, C).");
    LAT_REQUIRE(op != kSoftplus || p0 > 0.0f, "beta must be positive.");
    if (elements == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    int grid = elementwise_grid(elements);
    if (dtype == LAT_F32) {
        dispatch_activation<float>(op, feats, elements, p0, p1, out, grid, stream);
    } else {
        dispatch_activation<__half>(op, feats, elements, p0, p1, out, grid, stream);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"
