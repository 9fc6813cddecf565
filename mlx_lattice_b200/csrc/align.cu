// Feature movement after a sparse alignment: channel concatenation and elementwise
// binary operators of two feature matrices read through row maps (-1 = the row is absent
// on that side). The reference composes these from array ops
// (mlx_lattice/ops/tensor.py:89-147 `gather_aligned_features` + `sparse_binary_op`,
// tensor.py:228-249 `sparse_cat_aligned`): gather both sides, fill the missing rows, then
// concatenate or combine. Here each is one pass: every output element is written once
// and nothing is staged in HBM. Both are HBM-bound (read both sides once, write once).
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kAlignThreads = 256;

inline int align_grid(long long items) {
    long long blocks = (items + kAlignThreads - 1) / kAlignThreads;
    return static_cast<int>(std::max(1LL, std::min(blocks, 148LL * 16)));
}

// One thread per Chunk-byte piece of an output row; rows are byte strings here, so the
// kernel serves every element type. Missing rows give zero bytes.
template <typename Chunk>
__global__ void __launch_bounds__(kAlignThreads) concat_rows_kernel(
    const Chunk* lhs, const int32_t* lhs_rows, int lhs_capacity, int lhs_chunks,
    const Chunk* rhs, const int32_t* rhs_rows, int rhs_capacity, int rhs_chunks,
    long long rows_out, Chunk* out, int32_t* status
) {
    const int row_chunks = lhs_chunks + rhs_chunks;
    const long long total = rows_out * row_chunks;
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += step) {
        const long long row = i / row_chunks;
        const int c = static_cast<int>(i - row * row_chunks);
        const bool left = c < lhs_chunks;
        const int32_t* map = left ? lhs_rows : rhs_rows;
        const int capacity = left ? lhs_capacity : rhs_capacity;
        long long src = map != nullptr ? __ldg(map + row) : row;
        Chunk value{};
        if (src >= capacity) {
            raise_status(status, LAT_STATUS_BAD_INDEX);
        } else if (src >= 0) {
            value = left ? lhs[src * lhs_chunks + c] : rhs[src * rhs_chunks + (c - lhs_chunks)];
        }
        out[i] = value;
    }
}

enum BinaryOp { kAdd = 0, kSub = 1, kMul = 2, kMaximum = 3, kMinimum = 4 };

// the operators in the element type itself (one rounding, like an array op in that dtype);
// maximum / minimum propagate NaN
template <int Op> __device__ __forceinline__ float apply_op(float a, float b) {
    if (Op == kAdd) return a + b;
    if (Op == kSub) return a - b;
    if (Op == kMul) return a * b;
    if (a != a) return a;
    if (b != b) return b;
    return Op == kMaximum ? fmaxf(a, b) : fminf(a, b);
}

template <int Op> __device__ __forceinline__ __half apply_op(__half a, __half b) {
    if (Op == kAdd) return __hadd(a, b);
    if (Op == kSub) return __hsub(a, b);
    if (Op == kMul) return __hmul(a, b);
    return Op == kMaximum ? __hmax_nan(a, b) : __hmin_nan(a, b);
}

template <typename T> __device__ __forceinline__ T fill_value(float v);
template <> __device__ __forceinline__ float fill_value<float>(float v) { return v; }
template <> __device__ __forceinline__ __half fill_value<__half>(float v) { return __float2half_rn(v); }

// One thread per Vec consecutive channels of an output row (Vec * sizeof(T) = 16 bytes on
// the aligned route, one element otherwise).
template <typename T, int Op, int Vec>
__global__ void __launch_bounds__(kAlignThreads) binary_rows_kernel(
    const T* lhs, const int32_t* lhs_rows, int lhs_capacity, float lhs_fill,
    const T* rhs, const int32_t* rhs_rows, int rhs_capacity, float rhs_fill,
    long long rows_out, int channels, T* out, int32_t* status
) {
    struct alignas(sizeof(T) * Vec) Pack { T v[Vec]; };
    const int row_packs = channels / Vec;
    const long long total = rows_out * row_packs;
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    const T left_fill = fill_value<T>(lhs_fill);
    const T right_fill = fill_value<T>(rhs_fill);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += step) {
        const long long row = i / row_packs;
        const int c = static_cast<int>(i - row * row_packs);
        long long l = lhs_rows != nullptr ? __ldg(lhs_rows + row) : row;
        long long r = rhs_rows != nullptr ? __ldg(rhs_rows + row) : row;
        if (l >= lhs_capacity || r >= rhs_capacity) {
            raise_status(status, LAT_STATUS_BAD_INDEX);
            l = l >= lhs_capacity ? -1 : l;
            r = r >= rhs_capacity ? -1 : r;
        }
        Pack a, b, y;
#pragma unroll
        for (int u = 0; u < Vec; ++u) {
            a.v[u] = left_fill;
            b.v[u] = right_fill;
        }
        if (l >= 0) {
            a = reinterpret_cast<const Pack*>(lhs)[l * row_packs + c];
        }
        if (r >= 0) {
            b = reinterpret_cast<const Pack*>(rhs)[r * row_packs + c];
        }
#pragma unroll
        for (int u = 0; u < Vec; ++u) {
            y.v[u] = apply_op<Op>(a.v[u], b.v[u]);
        }
        reinterpret_cast<Pack*>(out)[i] = y;
    }
}

template <typename T, int Op>
int launch_binary(
    const void* lhs, const int32_t* lhs_rows, int lhs_capacity, float lhs_fill,
    const void* rhs, const int32_t* rhs_rows, int rhs_capacity, float rhs_fill,
    long long rows_out, int channels, void* out, int32_t* status, cudaStream_t stream
) {
    constexpr int kWide = 16 / sizeof(T);
    const bool wide = channels % kWide == 0 &&
                      (reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs) |
                       reinterpret_cast<uintptr_t>(out)) % 16 == 0;
    if (wide) {
        binary_rows_kernel<T, Op, kWide><<<align_grid(rows_out * (channels / kWide)), kAlignThreads, 0, stream>>>(
            static_cast<const T*>(lhs), lhs_rows, lhs_capacity, lhs_fill, static_cast<const T*>(rhs),
            rhs_rows, rhs_capacity, rhs_fill, rows_out, channels, static_cast<T*>(out), status);
    } else {
        binary_rows_kernel<T, Op, 1><<<align_grid(rows_out * channels), kAlignThreads, 0, stream>>>(
            static_cast<const T*>(lhs), lhs_rows, lhs_capacity, lhs_fill, static_cast<const T*>(rhs),
            rhs_rows, rhs_capacity, rhs_fill, rows_out, channels, static_cast<T*>(out), status);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

template <typename T, typename... Args> int dispatch_binary(int op, Args... args) {
    switch (op) {
        case kAdd: return launch_binary<T, kAdd>(args...);
        case kSub: return launch_binary<T, kSub>(args...);
        case kMul: return launch_binary<T, kMul>(args...);
        case kMaximum: return launch_binary<T, kMaximum>(args...);
        default: return launch_binary<T, kMinimum>(args...);
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

int lat_concat_aligned_features(
    int32_t element_bytes, const void* lhs, const int32_t* lhs_rows, int32_t lhs_capacity,
    int32_t lhs_channels, const void* rhs, const int32_t* rhs_rows, int32_t rhs_capacity,
    int32_t rhs_channels, int64_t rows_out, void* out, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(element_bytes == 2 || element_bytes == 4, "features must be float16 or float32.");
    LAT_REQUIRE(lhs_channels >= 0 && rhs_channels >= 0 && lhs_channels + rhs_channels > 0,
                "feats must have shape (N, C).");
    LAT_REQUIRE(rows_out >= 0 && lhs_capacity >= 0 && rhs_capacity >= 0, "row counts must be non-negative.");
    LAT_REQUIRE(lhs_rows != nullptr || rows_out <= lhs_capacity, "lhs has fewer rows than the output.");
    LAT_REQUIRE(rhs_rows != nullptr || rows_out <= rhs_capacity, "rhs has fewer rows than the output.");
    if (rows_out == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    const long long lhs_bytes = static_cast<long long>(lhs_channels) * element_bytes;
    const long long rhs_bytes = static_cast<long long>(rhs_channels) * element_bytes;
    const uintptr_t bases = reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs) |
                            reinterpret_cast<uintptr_t>(out);
    if (lhs_bytes % 16 == 0 && rhs_bytes % 16 == 0 && bases % 16 == 0) {
        const int lc = static_cast<int>(lhs_bytes / 16), rc = static_cast<int>(rhs_bytes / 16);
        concat_rows_kernel<uint4><<<align_grid(rows_out * (lc + rc)), kAlignThreads, 0, stream>>>(
            static_cast<const uint4*>(lhs), lhs_rows, lhs_capacity, lc, static_cast<const uint4*>(rhs),
            rhs_rows, rhs_capacity, rc, rows_out, static_cast<uint4*>(out), status);
    } else if (element_bytes == 4) {
        concat_rows_kernel<uint32_t><<<align_grid(rows_out * (lhs_channels + rhs_channels)), kAlignThreads, 0, stream>>>(
            static_cast<const uint32_t*>(lhs), lhs_rows, lhs_capacity, lhs_channels,
            static_cast<const uint32_t*>(rhs), rhs_rows, rhs_capacity, rhs_channels, rows_out,
            static_cast<uint32_t*>(out), status);
    } else {
        concat_rows_kernel<uint16_t><<<align_grid(rows_out * (lhs_channels + rhs_channels)), kAlignThreads, 0, stream>>>(
            static_cast<const uint16_t*>(lhs), lhs_rows, lhs_capacity, lhs_channels,
            static_cast<const uint16_t*>(rhs), rhs_rows, rhs_capacity, rhs_channels, rows_out,
            static_cast<uint16_t*>(out), status);
    }
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

int lat_binary_aligned_features(
    int32_t dtype, int32_t op, const void* lhs, const int32_t* lhs_rows, int32_t lhs_capacity,
    float lhs_fill, const void* rhs, const int32_t* rhs_rows, int32_t rhs_capacity, float rhs_fill,
    int64_t rows_out, int32_t channels, void* out, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(dtype == LAT_F32 || dtype == LAT_F16, "features must be float16 or float32.");
    LAT_REQUIRE(op >= kAdd && op <= kMinimum, "unknown sparse binary op.");
    LAT_REQUIRE(channels > 0, "feats must have shape (N, C).");
    LAT_REQUIRE(rows_out >= 0 && lhs_capacity >= 0 && rhs_capacity >= 0, "row counts must be non-negative.");
    LAT_REQUIRE(lhs_rows != nullptr || rows_out <= lhs_capacity, "lhs has fewer rows than the output.");
    LAT_REQUIRE(rhs_rows != nullptr || rows_out <= rhs_capacity, "rhs has fewer rows than the output.");
    if (rows_out == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    if (dtype == LAT_F32) {
        return dispatch_binary<float>(op, lhs, lhs_rows, lhs_capacity, lhs_fill, rhs, rhs_rows,
                                      rhs_capacity, rhs_fill, static_cast<long long>(rows_out),
                                      channels, out, status, stream);
    }
    return dispatch_binary<__half>(op, lhs, lhs_rows, lhs_capacity, lhs_fill, rhs, rhs_rows,
                                   rhs_capacity, rhs_fill, static_cast<long long>(rows_out),
                                   channels, out, status, stream);
}

} // extern "C"
