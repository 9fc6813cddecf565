// Error plumbing, runtime queries and the dispatch of the two convolution routes.
#include <algorithm>
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace lat {

namespace {
thread_local std::string g_last_error;
std::atomic<long long> g_launches{0};
std::atomic<long long> g_wait_budget{4000000000LL};  // about two seconds of SM clocks
}

long long wait_budget_cycles() { return g_wait_budget.load(std::memory_order_relaxed); }

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const std::string& message) { g_last_error = message; }

int fail(int code, const std::string& message) {
    g_last_error = message;
    return code;
}

// conv_direct.cu
size_t direct_conv_workspace_bytes(int n_kernels, int in_channels, int out_channels);
int run_direct_conv(
    int dtype, const void* feats, int in_capacity, int in_channels, long long feat_stride,
    const void* weights, int weight_layout, const uint32_t* packed, const void* scales,
    const void* biases, int storage_in_channels, int group_size, int bits, int out_channels,
    const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity, const int32_t* counts,
    const int32_t* row_offsets, int out_capacity, int n_kernels, const void* bias, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, cudaStream_t stream);

// conv_tc.cu
bool tc_conv_supported(int dtype, int n_kernels, int in_channels, int out_channels,
                       int quantized_bits, int group_size);
size_t tc_conv_workspace_bytes(int n_kernels, int in_channels, int out_channels);
int run_tc_conv(
    const void* feats, int in_capacity, int in_channels, long long feat_stride,
    const void* feats2, int feats2_channels, long long feat2_stride,
    const void* weights, int weight_layout, const uint32_t* packed, const void* scales,
    const void* biases, int storage_in_channels, int group_size, int bits, int out_channels,
    const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity, const int32_t* counts,
    const int32_t* row_offsets, int out_capacity, int n_kernels, const void* bias,
    const int32_t* row_order, const void* plan, void* out, void* workspace,
    size_t workspace_bytes, int32_t* status, cudaStream_t stream);

int run_tc_conv_plan(
    const void* feats, int in_channels, long long feat_stride, const void* feats2, int split,
    long long feat2_stride, const void* weights,
    long long w_stride_k, long long w_stride_co, int n_kernels, int out_channels, int out_capacity,
    const void* bias, const int32_t* row_order, const void* plan, void* out, int32_t* status,
    cudaStream_t stream);

int run_stage_quantized_weights(
    const uint32_t* packed, const void* scales, const void* biases, int n_kernels, int in_channels,
    int out_channels, int storage_in_channels, int group_size, int bits, void* out, cudaStream_t stream);

} // namespace lat

using namespace lat;

extern "C" {

const char* lat_version(void) { return "0.1.0+b200"; }

const char* lat_last_error(void) { return g_last_error.c_str(); }

long long lat_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int lat_set_wait_budget_cycles(int64_t cycles) {
    LAT_REQUIRE(cycles > 0, "the wait budget must be a positive number of clock cycles.");
    g_wait_budget.store(cycles, std::memory_order_relaxed);
    return LAT_OK;
}

int64_t lat_wait_budget_cycles(void) { return wait_budget_cycles(); }

int lat_capabilities(int32_t* has_sm100, int32_t* device_count) {
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    int ok = 0;
    for (int d = 0; d < count; ++d) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, d) == cudaSuccess && prop.major == 10) {
            ok = 1;
        }
    }
    if (has_sm100 != nullptr) {
        *has_sm100 = ok;
    }
    if (device_count != nullptr) {
        *device_count = count;
    }
    return LAT_OK;
}

int lat_kernel_offsets_host(lat_triple kernel_size, lat_triple dilation, int32_t* offsets_host) {
    LAT_REQUIRE(kernel_size.x > 0 && kernel_size.y > 0 && kernel_size.z > 0,
                "kernel_size values must be positive.");
    LAT_REQUIRE(dilation.x > 0 && dilation.y > 0 && dilation.z > 0,
                "dilation values must be positive.");
    LAT_REQUIRE(offsets_host != nullptr, "offsets buffer is required.");
    KernelGeometry geo = make_geometry(kernel_size, dilation);
    for (int k = 0; k < geo.volume; ++k) {
        int ox, oy, oz;
        geo.offset(k, ox, oy, oz);
        offsets_host[3 * k] = ox;
        offsets_host[3 * k + 1] = oy;
        offsets_host[3 * k + 2] = oz;
    }
    return LAT_OK;
}

size_t lat_sparse_conv_workspace_bytes(int32_t n_kernels, int32_t in_channels, int32_t out_channels) {
    return std::max(direct_conv_workspace_bytes(n_kernels, in_channels, out_channels),
                    tc_conv_workspace_bytes(n_kernels, in_channels, out_channels)) + 256;
}

int lat_conv_uses_tensor_cores(int32_t dtype, int32_t n_kernels, int32_t in_channels,
                               int32_t out_channels, int32_t quantized_bits, int32_t group_size) {
    return tc_conv_supported(dtype, n_kernels, in_channels, out_channels, quantized_bits,
                             group_size) ? 1 : 0;
}

static int validate_conv_common(
    int32_t dtype, const void* feats, int32_t in_capacity, int32_t in_channels,
    int32_t out_channels, const int32_t* in_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* counts, const int32_t* row_offsets,
    int32_t out_capacity, int32_t n_kernels, void* out
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16,
                "convolution supports float32 and float16 tensors.");
    LAT_REQUIRE(in_capacity >= 0 && in_channels > 0 && (feats != nullptr || in_capacity == 0),
                "feats must have shape (N, C).");
    LAT_REQUIRE(out_channels > 0, "weight output channels must be positive.");
    LAT_REQUIRE(out_capacity >= 0, "out_capacity must be non-negative.");
    LAT_REQUIRE(n_kernels > 0, "n_kernels must be positive.");
    LAT_REQUIRE(edge_capacity >= 0 && (edge_capacity == 0 || (in_rows && kernel_ids)),
                "in_rows, out_rows and kernel_ids must have the same length.");
    LAT_REQUIRE(counts != nullptr, "counts must have shape (2,) and int32 dtype.");
    LAT_REQUIRE(row_offsets != nullptr, "row_offsets must have length out_capacity + 1.");
    LAT_REQUIRE(out != nullptr || out_capacity == 0, "output buffer is required.");
    return LAT_OK;
}

int lat_sparse_conv_features(
    int32_t dtype, const void* feats, int32_t in_capacity, int32_t in_channels,
    int64_t feat_row_stride, const void* feats2, int32_t feats2_channels, int64_t feats2_row_stride,
    const void* weights, int32_t weight_layout, lat_triple kernel_shape, int32_t out_channels,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* counts, const int32_t* row_offsets,
    int32_t out_capacity, int32_t n_kernels,
    const void* bias, const int32_t* row_order, const void* plan, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    (void)out_rows;
    int rc = validate_conv_common(dtype, feats, in_capacity, in_channels, out_channels, in_rows,
                                  kernel_ids, edge_capacity, counts, row_offsets, out_capacity,
                                  n_kernels, out);
    if (rc != LAT_OK) {
        return rc;
    }
    LAT_REQUIRE(weights != nullptr, "weights are required.");
    LAT_REQUIRE(weight_layout == LAT_WEIGHT_KERNEL_MAJOR || weight_layout == LAT_WEIGHT_DENSE_5D ||
                    weight_layout == LAT_WEIGHT_OUT_MAJOR,
                "mapped convolution weight must have shape (K, C_in, C_out) or "
                "(C_out, Kx, Ky, Kz, C_in).");
    LAT_REQUIRE(weight_layout != LAT_WEIGHT_OUT_MAJOR ||
                    tc_conv_supported(dtype, n_kernels, in_channels, out_channels, 0, 0),
                "(K, C_out, C_in) weights are taken by the tensor-core route only.");
    if (weight_layout == LAT_WEIGHT_DENSE_5D) {
        LAT_REQUIRE(kernel_shape.x * kernel_shape.y * kernel_shape.z == n_kernels,
                    "weight kernel rows must match the convolution kernel.");
    }
    cudaStream_t stream = as_stream(stream_ptr);
    if (tc_conv_supported(dtype, n_kernels, in_channels, out_channels, 0, 0)) {
        return run_tc_conv(feats, in_capacity, in_channels, feat_row_stride, feats2,
                           feats2_channels, feats2_row_stride, weights, weight_layout, nullptr, nullptr, nullptr, in_channels, 0, 0,
                           out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
                           out_capacity, n_kernels, bias, row_order, plan, out, workspace,
                           workspace_bytes, status, stream);
    }
    LAT_REQUIRE(feats2 == nullptr, "a second feature source needs the tensor-core route and a gather plan.");
    return run_direct_conv(dtype, feats, in_capacity, in_channels, feat_row_stride, weights,
                           weight_layout, nullptr, nullptr, nullptr, in_channels, 0, 0,
                           out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
                           out_capacity, n_kernels, bias, out, workspace, workspace_bytes, status,
                           stream);
}

int lat_linear_uses_tensor_cores(int32_t dtype, int32_t in_channels, int32_t out_channels) {
    return tc_conv_supported(dtype, 1, in_channels, out_channels, 0, 0) ? 1 : 0;
}

int lat_linear_tensor_cores(
    const void* feats, int32_t rows, int32_t in_channels, int64_t feat_row_stride,
    const void* weight, int32_t out_channels, const void* bias, const void* plan, void* out,
    int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0 && (feats != nullptr || rows == 0), "feats must have shape (N, C).");
    LAT_REQUIRE(tc_conv_supported(LAT_F16, 1, in_channels, out_channels, 0, 0),
                "the tensor-core linear needs float16, C_in a multiple of 32 and C_out a multiple of "
                "16 up to 256.");
    LAT_REQUIRE(weight != nullptr && reinterpret_cast<uintptr_t>(weight) % 16 == 0,
                "weight (C_out, C_in) must be a 16-byte aligned device array.");
    LAT_REQUIRE(feat_row_stride >= in_channels && feat_row_stride % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(feats) % 16 == 0,
                "feature rows must be 16-byte aligned for the tensor-core route.");
    LAT_REQUIRE(plan != nullptr && (out != nullptr || rows == 0), "plan and output buffer are required.");
    // x @ W.T is the convolution over the identity relation with a single kernel offset
    return run_tc_conv_plan(feats, in_channels, feat_row_stride, nullptr, in_channels, 0, weight,
                            static_cast<long long>(out_channels) * in_channels, in_channels, 1,
                            out_channels, rows, bias, nullptr, plan, out, status, as_stream(stream_ptr));
}

int lat_dequantize_conv_weights(
    const uint32_t* packed, const void* scales, const void* biases, int32_t n_kernels,
    int32_t in_channels, int32_t out_channels, int32_t storage_in_channels, int32_t group_size,
    int32_t bits, void* out, void* stream_ptr
) {
    LAT_REQUIRE(bits == 4 || bits == 8, "quantized convolution supports only 4 or 8 bits.");
    LAT_REQUIRE(group_size == 32 || group_size == 64 || group_size == 128,
                "quantized convolution group_size must be 32, 64, or 128.");
    LAT_REQUIRE(n_kernels > 0 && in_channels > 0 && out_channels > 0, "weight shape must be positive.");
    LAT_REQUIRE(storage_in_channels >= in_channels && storage_in_channels % group_size == 0,
                "packed storage channels must be divisible by group_size.");
    LAT_REQUIRE(packed != nullptr && scales != nullptr && biases != nullptr && out != nullptr,
                "packed weight, scales, biases and the output buffer are required.");
    return run_stage_quantized_weights(packed, scales, biases, n_kernels, in_channels, out_channels,
                                       storage_in_channels, group_size, bits, out, as_stream(stream_ptr));
}

int lat_sparse_quantized_conv_features(
    int32_t dtype, const void* feats, int32_t in_capacity, int64_t feat_row_stride,
    const void* feats2, int32_t feats2_channels, int64_t feats2_row_stride,
    const uint32_t* packed, const void* scales, const void* biases,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* counts, const int32_t* row_offsets,
    int32_t out_capacity, int32_t n_kernels, int32_t in_channels, int32_t out_channels,
    int32_t storage_in_channels, int32_t group_size, int32_t bits,
    const void* bias, const int32_t* row_order, const void* plan, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    (void)out_rows;
    int rc = validate_conv_common(dtype, feats, in_capacity, in_channels, out_channels, in_rows,
                                  kernel_ids, edge_capacity, counts, row_offsets, out_capacity,
                                  n_kernels, out);
    if (rc != LAT_OK) {
        return rc;
    }
    // messages follow native/features/convolution/quantized.cpp:57-118
    LAT_REQUIRE(bits == 4 || bits == 8, "quantized convolution supports only 4 or 8 bits.");
    LAT_REQUIRE(group_size == 32 || group_size == 64 || group_size == 128,
                "quantized convolution group_size must be 32, 64, or 128.");
    LAT_REQUIRE(storage_in_channels >= in_channels && storage_in_channels % group_size == 0,
                "packed storage channels must be divisible by group_size.");
    LAT_REQUIRE(packed != nullptr && scales != nullptr && biases != nullptr,
                "packed weight, scales and biases are required.");
    cudaStream_t stream = as_stream(stream_ptr);
    if (tc_conv_supported(dtype, n_kernels, in_channels, out_channels, bits, group_size)) {
        return run_tc_conv(feats, in_capacity, in_channels, feat_row_stride, feats2,
                           feats2_channels, feats2_row_stride, nullptr, 0, packed,
                           scales, biases, storage_in_channels, group_size, bits, out_channels,
                           in_rows, kernel_ids, edge_capacity, counts, row_offsets, out_capacity,
                           n_kernels, bias, row_order, plan, out, workspace, workspace_bytes, status,
                           stream);
    }
    LAT_REQUIRE(feats2 == nullptr, "a second feature source needs the tensor-core route and a gather plan.");
    return run_direct_conv(dtype, feats, in_capacity, in_channels, feat_row_stride, nullptr, 0,
                           packed, scales, biases, storage_in_channels, group_size, bits,
                           out_channels, in_rows, kernel_ids, edge_capacity, counts, row_offsets,
                           out_capacity, n_kernels, bias, out, workspace, workspace_bytes, status,
                           stream);
}

} // extern "C"
