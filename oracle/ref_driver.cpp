// Test infrastructure only -- never linked into or called by the shipped library.
//
// A plain-C entry layer over the reference project's own CPU algorithm files
// (compiled unmodified from the reference checkout against the header stand-ins in
// shim/). Every function wraps caller-owned host buffers as arrays, fills the shape
// structs the way the reference factory layer does, and calls the reference CPU
// eval function. Callers size the outputs with the capacities the reference
// factories use:
//   forward / submanifold map   edges N*K, row_offsets N+1, out_coords N x 4
//                               (native/features/coordinates/relations.cpp:540-581)
//   target map                  edges Nt*K, row_offsets Nt+1, out_coords 1 x 4 dummy
//                               (relations.cpp:672-722)
//   transposed / generative     edges N*K, row_offsets N*K+1, out_coords N*K x 4
//                               (relations.cpp:599-670)
//   grouped view                offsets G+1, edge_ids = edge capacity
//                               (relations.cpp:438-459)
//   implicit-GEMM view          out_in_map Nout x K, row_masks Nout x ceil(K/32)
//                               (relations.cpp:498-538)
#include <array>
#include <cstdint>
#include <exception>
#include <vector>

#include "features/convolution/cpu/algorithms.h"
#include "features/coordinates/api.h"
#include "features/coordinates/cpu/algorithms.h"
#include "features/pooling/cpu/algorithms.h"

namespace {

namespace mx = mlx::core;
using mlx_lattice::Triple;

mx::Stream host_stream() { return mx::Stream{}; }

Triple triple(const int* values) { return {values[0], values[1], values[2]}; }

mx::array i32(const void* data, mx::Shape shape) {
    return mx::array(const_cast<void*>(data), std::move(shape), mx::int32);
}

mx::Dtype feature_dtype(int is_half) {
    return is_half != 0 ? mx::float16 : mx::float32;
}

template <typename Fn> int guarded(Fn fn) {
    try {
        fn();
        return 0;
    } catch (const std::exception&) {
        return 1;
    }
}

} // namespace

extern "C" {

// kernel_offsets: native/features/coordinates/offsets.cpp:11-45.
int ref_kernel_offsets(const int* kernel_size, const int* dilation, int* out) {
    return guarded([&] {
        auto offsets =
            mlx_lattice::kernel_offsets(triple(kernel_size), triple(dilation));
        for (std::size_t k = 0; k < offsets.size(); ++k) {
            out[3 * k] = offsets[k][0];
            out[3 * k + 1] = offsets[k][1];
            out[3 * k + 2] = offsets[k][2];
        }
    });
}

// Forward (op = 0) or transposed (op = 1) generic relation:
// native/features/coordinates/cpu/relation_algorithms.cpp:4-50.
int ref_generic_kernel_relation(
    int op,
    const int* stride,
    const int* padding,
    int direct,
    const int32_t* coords,
    int rows,
    const int32_t* offsets,
    int kernel_count,
    int active_rows,
    int edge_capacity,
    int out_capacity,
    int32_t* in_rows,
    int32_t* out_rows,
    int32_t* kernel_ids,
    int32_t* row_offsets,
    int32_t* out_coords,
    int32_t* counts
) {
    return guarded([&] {
        int32_t active = active_rows;
        std::vector<mx::array> inputs{
            i32(coords, {rows, 4}),
            i32(offsets, {kernel_count, 3}),
            i32(&active, {1}),
        };
        std::vector<mx::array> outputs{
            i32(in_rows, {edge_capacity}),
            i32(out_rows, {edge_capacity}),
            i32(kernel_ids, {edge_capacity}),
            i32(row_offsets, {out_capacity + 1}),
            i32(out_coords, {out_capacity, 4}),
            i32(counts, {2}),
        };
        mlx_lattice::coords::cpu::eval_generic_kernel_relation(
            op == 0 ? mlx_lattice::CoordRelationOp::Forward
                    : mlx_lattice::CoordRelationOp::Transposed,
            triple(stride),
            triple(padding),
            direct != 0,
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Explicit-target relation: cpu/relation_algorithms.cpp:52-80.
int ref_target_kernel_relation(
    const int* stride,
    const int* padding,
    const int32_t* coords,
    int rows,
    const int32_t* offsets,
    int kernel_count,
    int active_rows,
    const int32_t* target_coords,
    int target_rows,
    int target_active_rows,
    int32_t* in_rows,
    int32_t* out_rows,
    int32_t* kernel_ids,
    int32_t* row_offsets,
    int32_t* counts
) {
    return guarded([&] {
        int32_t active = active_rows;
        int32_t target_active = target_active_rows;
        int32_t dummy_coords[4] = {0, 0, 0, 0};
        auto edge_capacity = target_rows * kernel_count;
        std::vector<mx::array> inputs{
            i32(coords, {rows, 4}),
            i32(offsets, {kernel_count, 3}),
            i32(&active, {1}),
            i32(target_coords, {target_rows, 4}),
            i32(&target_active, {1}),
        };
        std::vector<mx::array> outputs{
            i32(in_rows, {edge_capacity}),
            i32(out_rows, {edge_capacity}),
            i32(kernel_ids, {edge_capacity}),
            i32(row_offsets, {target_rows + 1}),
            i32(dummy_coords, {1, 4}),
            i32(counts, {2}),
        };
        mlx_lattice::coords::cpu::eval_target_kernel_relation(
            triple(stride), triple(padding), host_stream(), inputs, outputs
        );
    });
}

// Generative relation: cpu/relation_algorithms.cpp:82-107.
int ref_generative_kernel_relation(
    const int* stride,
    const int32_t* coords,
    int rows,
    const int32_t* offsets,
    int kernel_count,
    int active_rows,
    int32_t* in_rows,
    int32_t* out_rows,
    int32_t* kernel_ids,
    int32_t* row_offsets,
    int32_t* out_coords,
    int32_t* counts
) {
    return guarded([&] {
        int32_t active = active_rows;
        auto pair_count = rows * kernel_count;
        std::vector<mx::array> inputs{
            i32(coords, {rows, 4}),
            i32(offsets, {kernel_count, 3}),
            i32(&active, {1}),
        };
        std::vector<mx::array> outputs{
            i32(in_rows, {pair_count}),
            i32(out_rows, {pair_count}),
            i32(kernel_ids, {pair_count}),
            i32(row_offsets, {pair_count + 1}),
            i32(out_coords, {pair_count, 4}),
            i32(counts, {2}),
        };
        mlx_lattice::coords::cpu::eval_generative_kernel_relation(
            triple(stride), host_stream(), inputs, outputs
        );
    });
}

// Grouped (CSR) view of edge ids by group id: cpu/relation_algorithms.cpp:109-125.
int ref_relation_grouped_view(
    const int32_t* group_ids,
    int edge_capacity,
    const int32_t* counts,
    int group_count,
    int32_t* row_offsets,
    int32_t* edge_ids
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            i32(group_ids, {edge_capacity}),
            i32(counts, {2}),
        };
        std::vector<mx::array> outputs{
            i32(row_offsets, {group_count + 1}),
            i32(edge_ids, {edge_capacity}),
        };
        mlx_lattice::coords::cpu::eval_relation_grouped_view(
            {edge_capacity, group_count}, host_stream(), inputs, outputs
        );
    });
}

// out_in_map + row masks: cpu/relation_algorithms.cpp:145-163.
int ref_relation_implicit_gemm_view(
    const int32_t* source_coords,
    int source_rows,
    int source_active,
    const int32_t* output_coords,
    int output_rows,
    int output_active,
    const int32_t* offsets,
    int kernel_count,
    const int* stride,
    const int* padding,
    int32_t* out_in_map,
    int32_t* row_masks
) {
    return guarded([&] {
        int32_t src_active = source_active;
        int32_t out_active = output_active;
        auto mask_words = (kernel_count + 31) / 32;
        std::vector<mx::array> inputs{
            i32(source_coords, {source_rows, 4}),
            i32(&src_active, {1}),
            i32(output_coords, {output_rows, 4}),
            i32(&out_active, {1}),
            i32(offsets, {kernel_count, 3}),
        };
        std::vector<mx::array> outputs{
            i32(out_in_map, {output_rows, kernel_count}),
            i32(row_masks, {output_rows, mask_words}),
        };
        mlx_lattice::coords::cpu::eval_relation_implicit_gemm_view(
            {source_rows,
             output_rows,
             kernel_count,
             mask_words,
             mlx_lattice::CoordRelationOp::Forward,
             triple(stride),
             triple(padding)},
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Downsample set op (first-seen unique floor_div): cpu/set_algorithms.cpp:4-37.
int ref_downsample_coords(
    const int32_t* coords,
    int rows,
    const int* stride,
    int32_t* out_coords,
    int32_t* count
) {
    return guarded([&] {
        std::vector<mx::array> inputs{i32(coords, {rows, 4})};
        std::vector<mx::array> outputs{
            i32(out_coords, {rows, 4}),
            i32(count, {1}),
        };
        mlx_lattice::coords::cpu::eval_set_coords(
            mlx_lattice::CoordSetOp::Downsample,
            triple(stride),
            host_stream(),
            inputs,
            outputs
        );
    });
}

// First-row lookup of query coords: cpu/set_algorithms.cpp:39-56.
int ref_lookup_coords(
    const int32_t* coords,
    int rows,
    const int32_t* queries,
    int query_rows,
    int32_t* out_rows
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            i32(coords, {rows, 4}),
            i32(queries, {query_rows, 4}),
        };
        std::vector<mx::array> outputs{i32(out_rows, {query_rows})};
        mlx_lattice::coords::cpu::eval_lookup_coords(
            host_stream(), inputs, outputs
        );
    });
}

// Sparse alignment (join 0 inner, 1 left, 2 right, 3 outer):
// cpu/set_algorithms.cpp:58-88. Output capacity as native/features/coordinates/
// lookup.cpp sizes it is passed in by the caller.
int ref_sparse_alignment(
    int join,
    const int32_t* lhs_coords,
    int lhs_rows,
    int lhs_active,
    const int32_t* rhs_coords,
    int rhs_rows,
    int rhs_active,
    int output_rows,
    int32_t* out_coords,
    int32_t* out_count,
    int32_t* out_lhs_rows,
    int32_t* out_rhs_rows
) {
    return guarded([&] {
        int32_t lhs_n = lhs_active;
        int32_t rhs_n = rhs_active;
        std::vector<mx::array> inputs{
            i32(lhs_coords, {lhs_rows, 4}),
            i32(&lhs_n, {1}),
            i32(rhs_coords, {rhs_rows, 4}),
            i32(&rhs_n, {1}),
        };
        std::vector<mx::array> outputs{
            i32(out_coords, {output_rows, 4}),
            i32(out_count, {1}),
            i32(out_lhs_rows, {output_rows}),
            i32(out_rhs_rows, {output_rows}),
        };
        mlx_lattice::coords::cpu::eval_sparse_alignment(
            static_cast<mlx_lattice::SparseJoinOp>(join),
            {lhs_rows, rhs_rows, output_rows},
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Float sparse conv forward: native/features/convolution/cpu/algorithms.cpp:706-722.
// weight_layout 0: (K, C_in, C_out) kernel-major; 1: (C_out, Kx, Ky, Kz, C_in).
// Shape fill as native/features/convolution/primitive.cpp:446-457.
int ref_sparse_conv(
    int is_half,
    const void* feats,
    int in_capacity,
    int in_channels,
    const void* weights,
    int weight_layout,
    int kernel_x,
    int kernel_y,
    int kernel_z,
    int out_channels,
    const int32_t* in_rows,
    const int32_t* out_rows,
    const int32_t* kernel_ids,
    int edge_capacity,
    const int32_t* counts,
    const int32_t* row_offsets,
    int out_capacity,
    int n_kernels,
    void* out
) {
    return guarded([&] {
        auto dtype = feature_dtype(is_half);
        auto weight_shape =
            weight_layout == 0
                ? mx::Shape{n_kernels, in_channels, out_channels}
                : mx::Shape{
                      out_channels, kernel_x, kernel_y, kernel_z, in_channels};
        std::vector<mx::array> inputs{
            mx::array(
                const_cast<void*>(feats), {in_capacity, in_channels}, dtype
            ),
            mx::array(const_cast<void*>(weights), weight_shape, dtype),
            i32(in_rows, {edge_capacity}),
            i32(out_rows, {edge_capacity}),
            i32(kernel_ids, {edge_capacity}),
            i32(counts, {2}),
            i32(row_offsets, {out_capacity + 1}),
        };
        std::vector<mx::array> outputs{
            mx::array(out, {out_capacity, out_channels}, dtype),
        };
        mlx_lattice::SparseConvShape shape{
            in_capacity,
            out_capacity,
            n_kernels,
            in_channels,
            out_channels,
            weight_layout,
            kernel_x,
            kernel_y,
            kernel_z,
            0,
        };
        mlx_lattice::backend::cpu::conv::eval(
            shape, host_stream(), inputs, outputs
        );
    });
}

// Quantized sparse conv forward:
// native/features/convolution/cpu/quantized.cpp:144-166. Input order as
// native/features/convolution/quantized.cpp:174-189.
int ref_sparse_quantized_conv(
    int is_half,
    const void* feats,
    int in_capacity,
    const uint32_t* packed,
    const void* scales,
    const void* biases,
    const int32_t* in_rows,
    const int32_t* out_rows,
    const int32_t* kernel_ids,
    int edge_capacity,
    const int32_t* counts,
    const int32_t* row_offsets,
    int out_capacity,
    int n_kernels,
    int in_channels,
    int out_channels,
    int storage_in_channels,
    int group_size,
    int bits,
    void* out
) {
    return guarded([&] {
        auto dtype = feature_dtype(is_half);
        auto words = storage_in_channels * bits / 32;
        auto groups = storage_in_channels / group_size;
        std::vector<mx::array> inputs{
            mx::array(
                const_cast<void*>(feats), {in_capacity, in_channels}, dtype
            ),
            mx::array(
                const_cast<uint32_t*>(packed),
                {n_kernels, words, out_channels},
                mx::uint32
            ),
            mx::array(
                const_cast<void*>(scales),
                {n_kernels, groups, out_channels},
                dtype
            ),
            mx::array(
                const_cast<void*>(biases),
                {n_kernels, groups, out_channels},
                dtype
            ),
            i32(in_rows, {edge_capacity}),
            i32(out_rows, {edge_capacity}),
            i32(kernel_ids, {edge_capacity}),
            i32(counts, {2}),
            i32(row_offsets, {out_capacity + 1}),
        };
        std::vector<mx::array> outputs{
            mx::array(out, {out_capacity, out_channels}, dtype),
        };
        mlx_lattice::QuantizedSparseConvShape shape{
            in_capacity,
            out_capacity,
            n_kernels,
            in_channels,
            out_channels,
            storage_in_channels,
            group_size,
            bits,
        };
        mlx_lattice::backend::cpu::conv::eval_quantized(
            shape, host_stream(), inputs, outputs
        );
    });
}

// Sparse pooling forward (reduce 0 sum, 1 max, 2 avg), float32 only:
// native/features/pooling/cpu/algorithms.cpp:181-244.
int ref_sparse_pool(
    int reduce,
    const float* feats,
    int in_capacity,
    int channels,
    const int32_t* in_rows,
    const int32_t* out_rows,
    const int32_t* kernel_ids,
    int edge_capacity,
    const int32_t* row_offsets,
    const int32_t* counts,
    int input_exclusive,
    int out_capacity,
    int n_kernels,
    float* out
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            mx::array(
                const_cast<float*>(feats), {in_capacity, channels}, mx::float32
            ),
            i32(in_rows, {edge_capacity}),
            i32(out_rows, {edge_capacity}),
            i32(kernel_ids, {edge_capacity}),
            i32(row_offsets, {out_capacity + 1}),
            i32(counts, {2}),
        };
        std::vector<mx::array> outputs{
            mx::array(out, {out_capacity, channels}, mx::float32),
        };
        mlx_lattice::SparsePoolShape shape{
            in_capacity,
            out_capacity,
            n_kernels,
            channels,
            input_exclusive != 0,
        };
        mlx_lattice::backend::cpu::pool::eval(
            static_cast<mlx_lattice::PoolReduceOp>(reduce),
            shape,
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Point -> voxel quantization (first-seen unique voxel per point, inverse rows, points
// per voxel): cpu/quantization_algorithms.cpp:4-30 -> cpu/quantization_detail.h:87-125.
// Outputs sized like the reference factory: coords points x 4, count 1, inverse points,
// voxel_counts points.
int ref_sparse_quantize(
    const float* points,
    const int32_t* batch_indices,
    int rows,
    const int32_t* active_rows,
    const float* voxel_size,
    const float* origin,
    int32_t* out_coords,
    int32_t* count,
    int32_t* inverse_rows,
    int32_t* voxel_counts
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            mx::array(const_cast<float*>(points), {rows, 3}, mx::float32),
            i32(batch_indices, {rows}),
            i32(active_rows, {1}),
        };
        std::vector<mx::array> outputs{
            i32(out_coords, {rows, 4}),
            i32(count, {1}),
            i32(inverse_rows, {rows}),
            i32(voxel_counts, {rows}),
        };
        mlx_lattice::QuantizationSpec spec{
            {voxel_size[0], voxel_size[1], voxel_size[2]},
            {origin[0], origin[1], origin[2]},
        };
        mlx_lattice::coords::cpu::eval_sparse_quantize(
            spec, host_stream(), inputs, outputs
        );
    });
}

// Per-voxel sum / mean of point features in point order:
// cpu/quantization_algorithms.cpp:32-62 -> cpu/quantization_detail.h:138-166.
int ref_voxelize_features(
    const float* values,
    const int32_t* inverse_rows,
    const int32_t* voxel_counts,
    const int32_t* active_rows,
    int point_rows,
    int voxel_rows,
    int channels,
    int mean,
    float* out
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            mx::array(const_cast<float*>(values), {point_rows, channels}, mx::float32),
            i32(inverse_rows, {point_rows}),
            i32(voxel_counts, {voxel_rows}),
            i32(active_rows, {1}),
        };
        std::vector<mx::array> outputs{
            mx::array(out, {voxel_rows, channels}, mx::float32),
        };
        mlx_lattice::coords::cpu::eval_voxelize_features(
            mean != 0 ? mlx_lattice::VoxelReduceOp::Mean : mlx_lattice::VoxelReduceOp::Sum,
            mlx_lattice::VoxelFeatureShape{point_rows, voxel_rows, channels},
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Point -> voxel interpolation slots (nearest or trilinear):
// cpu/quantization_algorithms.cpp -> cpu/quantization_detail.h:203-315.
int ref_point_voxel_map(
    const float* points,
    const int32_t* batch_indices,
    int point_rows,
    const int32_t* point_active_rows,
    const int32_t* voxel_coords,
    int voxel_rows,
    const int32_t* voxel_active_rows,
    const float* voxel_size,
    const float* origin,
    int linear,
    int32_t* rows,
    float* weights
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            mx::array(const_cast<float*>(points), {point_rows, 3}, mx::float32),
            i32(batch_indices, {point_rows}),
            i32(point_active_rows, {1}),
            i32(voxel_coords, {voxel_rows, 4}),
            i32(voxel_active_rows, {1}),
        };
        std::vector<mx::array> outputs{
            i32(rows, {point_rows, 8}),
            mx::array(weights, {point_rows, 8}, mx::float32),
        };
        mlx_lattice::QuantizationSpec spec{
            {voxel_size[0], voxel_size[1], voxel_size[2]},
            {origin[0], origin[1], origin[2]},
        };
        mlx_lattice::coords::cpu::eval_point_voxel_map(
            spec,
            linear != 0 ? mlx_lattice::PointVoxelInterpolationOp::Linear
                        : mlx_lattice::PointVoxelInterpolationOp::Nearest,
            mlx_lattice::PointVoxelMapShape{point_rows, voxel_rows},
            host_stream(),
            inputs,
            outputs
        );
    });
}

// Weighted sum of voxel features over a point's slots:
// cpu/quantization_detail.h:317-346.
int ref_interpolate_point_features(
    const float* values,
    const int32_t* rows,
    const float* weights,
    int point_rows,
    int voxel_rows,
    int channels,
    float* out
) {
    return guarded([&] {
        std::vector<mx::array> inputs{
            mx::array(const_cast<float*>(values), {voxel_rows, channels}, mx::float32),
            i32(rows, {point_rows, 8}),
            mx::array(const_cast<float*>(weights), {point_rows, 8}, mx::float32),
        };
        std::vector<mx::array> outputs{
            mx::array(out, {point_rows, channels}, mx::float32),
        };
        mlx_lattice::coords::cpu::eval_interpolate_point_features(
            mlx_lattice::VoxelFeatureShape{point_rows, voxel_rows, channels},
            host_stream(),
            inputs,
            outputs
        );
    });
}

} // extern "C"
