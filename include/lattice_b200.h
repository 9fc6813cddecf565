/*
 * lattice_b200 -- C ABI of the sm_100a sparse-convolution inference path.
 *
 * Every entry point replaces one function of the reference project's native
 * extension (`mlx_lattice._ext`, built from native/bindings) for the hot path
 * coordinate hash -> kernel map -> sparse-conv contraction -> sparse pooling.
 * The citation on each declaration names the reference interface it stands in
 * for (paths relative to the reference checkout).
 *
 * Conventions
 *  - All array arguments are DEVICE pointers on the current CUDA device unless a
 *    parameter name ends in `_host`. Arrays are dense row-major.
 *  - Static capacities + device-side counts, exactly like the reference: outputs
 *    are sized by the worst case, `counts[2] = {edge_count, out_count}` and
 *    `active_rows[1]` live on the device, and no call reads them back. Nothing
 *    here synchronises the stream, so calls can be captured into a CUDA graph.
 *  - `stream` is a `cudaStream_t` passed as `void*` (NULL = default stream).
 *  - Scratch memory is caller-provided: ask `lat_*_workspace_bytes`, pass a
 *    256-byte-aligned device buffer of at least that size. The library never
 *    allocates device memory in these calls.
 *  - Return value: LAT_OK or an error code; `lat_last_error()` returns the
 *    message of the last failing call on the calling thread (the reference
 *    throws std::invalid_argument / std::runtime_error with the same texts).
 *  - Device-side problems that can only be seen while a kernel runs (hash table
 *    full, more edges than capacity, a wait that gave up) never trap: the kernel
 *    records a bit in the caller's `status` word (device int32, may be NULL) and
 *    returns. Read it back after synchronising.
 */
#ifndef LATTICE_B200_H
#define LATTICE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lat_triple {
    int32_t x, y, z;
} lat_triple;

typedef struct lat_float_triple {
    float x, y, z;
} lat_float_triple;

enum {
    LAT_OK = 0,
    LAT_INVALID_ARGUMENT = 1, /* contract violation (reference: std::invalid_argument) */
    LAT_CUDA_ERROR = 2,       /* a CUDA runtime call or launch failed */
    LAT_UNSUPPORTED = 3,      /* no sm_100 device (reference: std::runtime_error) */
    LAT_WORKSPACE_TOO_SMALL = 4,
};

/* bits of the device status word */
enum {
    LAT_STATUS_HASH_FULL = 1,      /* probe sequence exhausted the table */
    LAT_STATUS_EDGE_OVERFLOW = 2,  /* more edges/rows than the output capacity */
    LAT_STATUS_BAD_INDEX = 4,      /* row id or kernel id outside its range */
    LAT_STATUS_WAIT_TIMEOUT = 8,   /* a bounded in-kernel wait gave up */
    LAT_STATUS_DUPLICATE_INPUT = 16 /* overlapping transposed map met duplicate input coords */
};

enum { LAT_F32 = 0, LAT_F16 = 1 };
enum { LAT_REDUCE_SUM = 0, LAT_REDUCE_MAX = 1, LAT_REDUCE_AVG = 2 };
/* weight layouts of lat_sparse_conv_features: (K, C_in, C_out); (C_out, Kx, Ky, Kz, C_in);
 * (K, C_out, C_in) as lat_dequantize_conv_weights writes it (tensor-core route only) */
enum { LAT_WEIGHT_KERNEL_MAJOR = 0, LAT_WEIGHT_DENSE_5D = 1, LAT_WEIGHT_OUT_MAJOR = 2 };
enum { LAT_JOIN_INNER = 0, LAT_JOIN_LEFT = 1, LAT_JOIN_RIGHT = 2, LAT_JOIN_OUTER = 3 };

/* native/bindings/runtime.cpp:27-38 (`version`, `capabilities`). */
const char* lat_version(void);
int lat_capabilities(int32_t* has_sm100, int32_t* device_count);
const char* lat_last_error(void);
/* Number of CUDA kernels this library has launched in the process so far (no
 * reference counterpart; used by the benchmark to report its launch count). */
long long lat_launch_count(void);
/* Clock budget (SM cycles, default 4e9, about two seconds) after which a bounded wait
 * inside a kernel (an mbarrier of the tensor-core pipeline, the look-back of the
 * single-pass kernel map) gives up: the kernel then sets LAT_STATUS_WAIT_TIMEOUT in the
 * status word, every role leaves its loop, tensor memory is freed and the launch
 * returns. No reference counterpart (the reference's kernels do not wait on each
 * other). Process-wide; takes effect for launches made after the call. */
int lat_set_wait_budget_cycles(int64_t cycles);
int64_t lat_wait_budget_cycles(void);

/* native/features/coordinates/offsets.cpp:11-45 (`kernel_offsets`): host helper,
 * writes kernel_volume x 3 int32 to a HOST buffer, x-major / z-fastest. */
int lat_kernel_offsets_host(lat_triple kernel_size, lat_triple dilation, int32_t* offsets_host);

/* ---- kernel maps -------------------------------------------------------- */

/* Scratch for any relation builder below. `rows` = source capacity,
 * `out_rows` = output-row capacity of the map (rows for forward/submanifold,
 * target rows for target maps, rows*K for transposed/generative). */
size_t lat_relation_workspace_bytes(int32_t rows, int32_t out_rows, int32_t kernel_count);

/* The first-row-wins coordinate table every builder below starts from (the
 * reference's GPU builders fill one per call: scratch of coord_hash_capacity(rows),
 * native/features/coordinates/relations.cpp:95-105 and :555, inserted by
 * coordinates/metal/hash.metal:7-41) as a buffer the caller may keep:
 * lat_build_coord_table fills `table` (32-byte aligned, lat_coord_table_bytes(rows)
 * bytes) from coords [rows, 4] and active_rows [1]. A builder that takes
 * `source_table` accepts such a buffer made from the same (coords, rows,
 * active_rows) and skips its own table build; NULL builds one in the workspace.
 * One coordinate set usually feeds several builders (submanifold, strided,
 * transposed). The buffer's layout is private to the library. */
size_t lat_coord_table_bytes(int32_t rows);
int lat_build_coord_table(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    void* table, size_t table_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:414-479 (`build_kernel_relation`) ->
 * make_kernel_relation, native/features/coordinates/relations.cpp:540-581;
 * algorithm native/features/coordinates/cpu/relation_build_detail.h:3-41.
 * Output capacities: in_rows/out_rows/kernel_ids [rows*K], row_offsets [rows+1],
 * out_coords [rows,4], counts [2]. Optional (may be NULL): row_masks
 * [rows, ceil(K/32)] (bit k of an output row's mask = offset k present),
 * kernel_row_offsets [K+1] + kernel_edge_ids [rows*K] (the per-offset pair lists
 * of relations.cpp:461-476 built in the same pass). */
int lat_build_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    const void* source_table /* optional, lat_build_coord_table of `coords` */,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:480-508 (`build_submanifold_kernel_relation`) ->
 * relations.cpp:583-597: the forward map with stride 1 and padding 0; outputs are
 * the input rows themselves (out_coords is a copy of the active input rows). */
int lat_build_submanifold_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    const void* source_table /* optional, lat_build_coord_table of `coords` */,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:546-589 (`build_target_kernel_relation`) ->
 * relations.cpp:672-722; algorithm cpu/relation_build_detail.h:43-80.
 * Edge arrays [target_rows*K], row_offsets [target_rows+1]; counts =
 * {E, target_active}. The caller's target coords are the relation's out coords. */
int lat_build_target_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    const int32_t* target_coords, int32_t target_rows, const int32_t* target_active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* counts,
    int32_t* row_masks, int32_t* kernel_row_offsets, int32_t* kernel_edge_ids,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:509-545 (`build_transposed_kernel_relation`) ->
 * relations.cpp:632-670; algorithm cpu/relation_build_detail.h:122-196. All edge
 * and output arrays have capacity rows*K (row_offsets rows*K+1, out_coords
 * [rows*K,4]). Uses the closed form when stride exceeds the offset extent on
 * every axis (relations.cpp:107-126), else the deduplicating form. */
int lat_build_transposed_kernel_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride, lat_triple padding, lat_triple dilation,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp (`build_generative_relation`) ->
 * relations.cpp:599-630; algorithm cpu/relation_build_detail.h:82-120. */
int lat_build_generative_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    lat_triple kernel_size, lat_triple stride,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* out_coords, int32_t* counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* A superset entry (no reference counterpart as one call): the transposed map of
 * a k = stride conv restricted to a caller-given fine support. For target row t:
 * in = first_row(floor(t / stride)), kernel id from t - stride*floor(t/stride).
 * It equals the reference composition conv_transpose3d (mlx_lattice/ops/conv.py:
 * 153-182) followed by sparse_cat_aligned(join='right') (mlx_lattice/ops/
 * tensor.py:228-249) and is what `coordinates=` on the transposed op maps to.
 * Requires kernel_size == stride, padding 0, dilation 1. Capacities as for the
 * target map with K = 1 edge per target row at most: edge arrays [target_rows]. */
int lat_build_target_transposed_relation(
    const int32_t* coords, int32_t rows, const int32_t* active_rows,
    const int32_t* target_coords, int32_t target_rows, const int32_t* target_active_rows,
    lat_triple stride,
    int32_t* in_rows, int32_t* out_rows, int32_t* kernel_ids, int32_t* row_offsets,
    int32_t* counts, int32_t* row_masks /* optional [target_rows, 1] */,
    const void* source_table /* optional, lat_build_coord_table of `coords` */,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* relations.cpp:438-459 (`make_relation_grouped_view`), algorithm
 * cpu/relation_views_detail.h:84-120: CSR of edge ids by group id, ascending edge
 * id inside a group, -1 fill. row_offsets [group_count+1], edge_ids [edge_capacity]. */
size_t lat_grouped_view_workspace_bytes(int32_t edge_capacity, int32_t group_count);
int lat_build_relation_grouped_view(
    const int32_t* group_ids, int32_t edge_capacity, const int32_t* counts, int32_t group_count,
    int32_t* row_offsets, int32_t* edge_ids,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:590-627 (`build_relation_implicit_gemm_view`) ->
 * relations.cpp:498-538; algorithm cpu/relation_views_detail.h:122-169.
 * out_in_map [output_rows, K] (-1 = empty), row_masks [output_rows, ceil(K/32)].
 * `offsets` is a DEVICE array [K,3]. */
size_t lat_implicit_gemm_view_workspace_bytes(int32_t source_rows);
int lat_build_relation_implicit_gemm_view(
    const int32_t* source_coords, int32_t source_rows, const int32_t* source_active_rows,
    const int32_t* output_coords, int32_t output_rows, const int32_t* output_active_rows,
    const int32_t* offsets, int32_t kernel_count, lat_triple stride, lat_triple padding,
    int32_t* out_in_map, int32_t* row_masks,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- coordinate sets ---------------------------------------------------- */

/* native/bindings/coords.cpp:132-160 (`downsample_coords`): unique
 * floor(coord/stride) rows in first-seen order; out_coords [rows,4], count [1]. */
size_t lat_coord_set_workspace_bytes(int32_t rows);
int lat_downsample_coords(
    const int32_t* coords, int32_t rows, lat_triple stride,
    int32_t* out_coords, int32_t* count,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:176-190 (`lookup_coords`): first row of each query
 * coordinate among ALL `rows` source rows, -1 when absent. out_rows [query_rows]. */
int lat_lookup_coords(
    const int32_t* coords, int32_t rows, const int32_t* queries, int32_t query_rows,
    int32_t* out_rows,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* No counterpart in the reference. The same lookup as lat_lookup_coords for callers
 * that must not allocate and have no workspace to lend (a host that freezes its device
 * memory after start-up, a latency-critical loop): the hash table lives in a fixed
 * 2 MiB __device__ array inside the library instead. At most
 * lat_lookup_coords_static_max_rows() (262144) source rows; more is an
 * LAT_INVALID_ARGUMENT. The array is shared by all calls: calls that overlap on the
 * GPU race, so serialise them. The first call on a device looks up the array's address;
 * make it before any stream capture. */
int32_t lat_lookup_coords_static_max_rows(void);
int lat_lookup_coords_static(
    const int32_t* coords, int32_t rows, const int32_t* queries, int32_t query_rows,
    int32_t* out_rows, int32_t* status, void* stream);

/* native/bindings/coords.cpp:191-222 (`build_sparse_alignment`) ->
 * native/features/coordinates/lookup.cpp:111-146; algorithm
 * cpu/set_neighbors_detail.h:59-136. Output capacity: lhs_rows (inner, left),
 * rhs_rows (right), lhs_rows + rhs_rows (outer). */
size_t lat_sparse_alignment_workspace_bytes(int32_t lhs_rows, int32_t rhs_rows);
int lat_build_sparse_alignment(
    const int32_t* lhs_coords, int32_t lhs_rows, const int32_t* lhs_active_rows,
    const int32_t* rhs_coords, int32_t rhs_rows, const int32_t* rhs_active_rows,
    int32_t join,
    int32_t* out_coords, int32_t* out_count, int32_t* out_lhs_rows, int32_t* out_rhs_rows,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- feature contraction ------------------------------------------------ */

/* native/bindings/convolution.cpp:90-146 (`sparse_conv_features`) ->
 * native/features/convolution/api.cpp:119-246; arithmetic
 * native/features/convolution/cpu/algorithms.cpp:180-302.
 * feats [in_capacity, in_channels] with row stride `feat_row_stride` (elements),
 * weights either (K, C_in, C_out) or (C_out, Kx, Ky, Kz, C_in) contiguous, out
 * [out_capacity, out_channels]; rows >= counts[1] are zero (plus `bias` when given). dtype LAT_F32 or
 * LAT_F16 for feats, weights and out alike; accumulation is float32. The
 * grouped-view arguments of the reference call are not read by the forward pass
 * and are therefore not part of this signature. Optional `bias` [out_channels]
 * (feature dtype) is added after the final cast (mlx_lattice/ops/conv.py:460-469),
 * optional `row_order` [out_capacity] is a permutation of output rows that the
 * tensor-core route uses to form its 256-row tiles (any permutation is valid),
 * optional `plan` is the gather plan built by lat_build_conv_plan over this relation
 * and this `row_order` (the tensor-core route then reads it instead of the relation
 * arrays; other routes ignore it). Optional `feats2` [in_capacity, feats2_channels] (row
 * stride `feats2_row_stride`, NULL = none) supplies the LAST feats2_channels of the
 * in_channels input channels, `feats` the first in_channels - feats2_channels: the
 * convolution then reads the channel concatenation of two tensors over the same rows
 * (mlx_lattice/ops/tensor.py `sparse_cat_aligned` followed by a convolution) without the
 * concatenated tensor being written. Tensor-core route with a plan only; the channel
 * split must be a multiple of 8. */
size_t lat_sparse_conv_workspace_bytes(int32_t n_kernels, int32_t in_channels, int32_t out_channels);
int lat_sparse_conv_features(
    int32_t dtype, const void* feats, int32_t in_capacity, int32_t in_channels,
    int64_t feat_row_stride, const void* feats2, int32_t feats2_channels, int64_t feats2_row_stride,
    const void* weights, int32_t weight_layout, lat_triple kernel_shape, int32_t out_channels,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* counts, const int32_t* row_offsets,
    int32_t out_capacity, int32_t n_kernels,
    const void* bias, const int32_t* row_order, const void* plan, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/convolution.cpp:12-89 (`sparse_quantized_conv_features`) ->
 * native/features/convolution/quantized.cpp:198-268; arithmetic
 * native/features/convolution/cpu/quantized.cpp:54-140. packed (K, S*bits/32,
 * C_out) uint32, scales/biases (K, S/group, C_out) in the feature dtype, S =
 * storage_in_channels; w = code*scale + bias, float32 accumulation, one cast.
 * The three sorted-plan arrays of the reference call may be empty there and are
 * replaced here by the optional `row_order`. `bias`/`row_order` as above. */
int lat_sparse_quantized_conv_features(
    int32_t dtype, const void* feats, int32_t in_capacity, int64_t feat_row_stride,
    const void* feats2, int32_t feats2_channels, int64_t feats2_row_stride,
    const uint32_t* packed, const void* scales, const void* biases,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* counts, const int32_t* row_offsets,
    int32_t out_capacity, int32_t n_kernels, int32_t in_channels, int32_t out_channels,
    int32_t storage_in_channels, int32_t group_size, int32_t bits,
    const void* bias, const int32_t* row_order, const void* plan, void* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* The fp16 weights a packed convolution weight stands for, as (K, C_out, C_in): w =
 * code*scale + bias evaluated in float32 and rounded once (the decode rule of
 * native/features/convolution/cpu/quantized.cpp:54-62, 107-131). The tensor-core route
 * of lat_sparse_quantized_conv_features makes this array in its workspace on every call;
 * a caller that keeps it (weights are constants of an inference network) passes it to
 * lat_sparse_conv_features with LAT_WEIGHT_OUT_MAJOR instead and gets the same bits
 * without the per-call conversion. fp16 scales/biases only. */
int lat_dequantize_conv_weights(
    const uint32_t* packed, const void* scales, const void* biases, int32_t n_kernels,
    int32_t in_channels, int32_t out_channels, int32_t storage_in_channels, int32_t group_size,
    int32_t bits, void* out, void* stream);

/* Gather plan of the tensor-core route for one relation (no reference counterpart;
 * it takes the place of the per-call walk over the relation that the reference's
 * implicit-GEMM view, native/features/coordinates/cpu/relations.cpp, prepares on the
 * host side). The output rows in `row_order` (natural order when NULL) are cut into
 * 256-row tiles; per tile the plan holds the mask of kernel offsets its rows use and,
 * per used offset, the input row of each tile row (-1 = none), and it lists the tiles by
 * falling number of used offsets, the order in which the convolution hands them to its
 * thread blocks. Build it once per
 * relation after `row_order`, then pass `plan` together with the same `row_order` to
 * the convolutions over that relation. kernel_count <= 32. Optional `row_masks`
 * [out_capacity] (bit k = the row has an edge at offset k, as the kernel-map builders and
 * lat_build_relation_implicit_gemm_view write them) spares the builder a walk over the
 * edges; they must describe the same relation. */
size_t lat_conv_plan_bytes(int32_t out_capacity, int32_t kernel_count);
int lat_build_conv_plan(
    const int32_t* in_rows, const int32_t* kernel_ids, int32_t edge_capacity,
    const int32_t* counts, const int32_t* row_offsets, int32_t in_capacity,
    int32_t out_capacity, int32_t kernel_count, const int32_t* row_order, const int32_t* row_masks,
    void* plan, size_t plan_bytes, int32_t* status, void* stream);

/* 1 when the tensor-core (tcgen05) route serves this shape, 0 when the CUDA-core
 * route does. Informational; both routes give results inside the tolerance. */
int lat_conv_uses_tensor_cores(int32_t dtype, int32_t n_kernels, int32_t in_channels,
                               int32_t out_channels, int32_t quantized_bits, int32_t group_size);

/* Row permutation that groups output rows with equal offset masks (the idea of
 * the sorted view, mlx_lattice/core/relations/views.py:467-510, as a native
 * product). row_masks [rows, 1] with bits [0, kernel_count) (K <= 32); rows at or
 * beyond counts[1] come last. row_order [rows]. */
size_t lat_mask_order_workspace_bytes(int32_t rows);
int lat_build_mask_row_order(
    const int32_t* row_masks, int32_t rows, int32_t kernel_count, const int32_t* counts,
    int32_t* row_order,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- point -> voxel front end (the step before the path) ------------------ */

/* native/bindings/coords.cpp:294-325 (`sparse_quantize`) ->
 * native/features/coordinates/quantization.cpp; arithmetic
 * native/features/coordinates/cpu/quantization_detail.h:67-125. points [rows,3]
 * float32, batch_indices [rows] int32 (NULL = all zero), active_rows [1] (NULL =
 * rows). Voxel coordinate = (batch, floor((p - origin) / voxel_size)) in float32.
 * out_coords [rows,4] holds the unique voxels in first-seen point order (zero
 * tail), count [1] their number, inverse_rows [rows] the voxel row of each point
 * (-1 at and beyond active_rows), voxel_counts [rows] the points per voxel (zero
 * tail). */
size_t lat_sparse_quantize_workspace_bytes(int32_t rows);
int lat_sparse_quantize(
    const float* points, const int32_t* batch_indices, int32_t rows, const int32_t* active_rows,
    lat_float_triple voxel_size, lat_float_triple origin,
    int32_t* out_coords, int32_t* count, int32_t* inverse_rows, int32_t* voxel_counts,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:326-352 (`voxelize_features`); arithmetic
 * cpu/quantization_detail.h:127-166. values [point_rows, channels] float32; out
 * [voxel_rows, channels] = per-voxel sum (mean = 0) or mean (sum of value *
 * 1/max(count,1)) over the points p < active_rows[0] with inverse_rows[p] in
 * [0, voxel_rows), accumulated in ascending point order. */
size_t lat_voxelize_features_workspace_bytes(int32_t point_rows, int32_t voxel_rows);
int lat_voxelize_features(
    const float* values, const int32_t* inverse_rows, const int32_t* voxel_counts,
    const int32_t* active_rows, int32_t point_rows, int32_t voxel_rows, int32_t channels,
    int32_t mean, float* out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp:353-395 (`build_point_voxel_map`); arithmetic
 * cpu/quantization_detail.h:203-315. rows_out / weights_out [point_rows, 8]: for
 * `linear` = 0 slot 0 holds the voxel at floor(position + 0.5) with weight 1, for
 * `linear` = 1 slot c holds the cell corner (c & 1, c >> 1 & 1, c >> 2 & 1) above
 * floor(position) with its trilinear weight; absent voxels and points at or beyond
 * point_active_rows are (-1, 0). Voxel rows at or beyond voxel_active_rows are not
 * looked up; duplicates resolve to the first row. */
size_t lat_point_voxel_map_workspace_bytes(int32_t voxel_rows);
int lat_build_point_voxel_map(
    const float* points, const int32_t* batch_indices, int32_t point_rows,
    const int32_t* point_active_rows, const int32_t* voxel_coords, int32_t voxel_rows,
    const int32_t* voxel_active_rows, lat_float_triple voxel_size, lat_float_triple origin,
    int32_t linear, int32_t* rows_out, float* weights_out,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* native/bindings/coords.cpp (`interpolate_point_features`); arithmetic
 * cpu/quantization_detail.h:317-346: out [point_rows, channels] = sum over the eight
 * slots, in slot order, of values[row] * weight (float32). */
int lat_interpolate_point_features(
    const float* values, const int32_t* rows, const float* weights, int32_t point_rows,
    int32_t voxel_rows, int32_t channels, float* out, void* stream);

/* ---- pooling and pointwise feature ops ---------------------------------- */

/* native/bindings/pooling.cpp:17-72 (`sparse_pool_features`) ->
 * native/features/pooling/api.cpp:8-38; arithmetic
 * native/features/pooling/cpu/algorithms.cpp:181-244. float32 only, like the
 * reference. Rows >= counts[1] hold the identity (0, or -inf for max). */
int lat_sparse_pool_features(
    const float* feats, int32_t in_capacity, int32_t channels, int64_t feat_row_stride,
    const int32_t* in_rows, const int32_t* out_rows, const int32_t* kernel_ids,
    int32_t edge_capacity, const int32_t* row_offsets, const int32_t* counts,
    int32_t input_exclusive, int32_t reduce, int32_t out_capacity, int32_t n_kernels,
    float* out, int32_t* status, void* stream);

/* mlx_lattice/ops/pool.py:197-236 (`global_sum_pool` / `global_avg_pool` /
 * `global_max_pool`): per-batch reduction over contiguous row ranges given by
 * `batch_offsets` (DEVICE int32 [batches+1], prefix sums of batch_counts).
 * feats float32 [rows, channels]; out float32 [batches, channels]. */
int lat_global_pool(
    const float* feats, int32_t rows, int32_t channels, const int32_t* batch_offsets,
    int32_t batches, int32_t reduce, float* out, void* stream);

/* The same `linear` (mlx_lattice/ops/feature.py:33-51) on the tensor cores, for float16
 * rows with C_in a multiple of 32 and C_out a multiple of 16 up to 256
 * (lat_linear_uses_tensor_cores): x @ W.T is the tcgen05 convolution over the identity
 * relation with one kernel offset. `plan` is lat_build_identity_conv_plan(rows) in a
 * buffer of lat_conv_plan_bytes(rows, 1) bytes; it depends on `rows` only and can be
 * kept. weight (C_out, C_in) float16, 16-byte aligned; float32 accumulation, one cast,
 * optional bias [C_out] added after it. */
int lat_linear_uses_tensor_cores(int32_t dtype, int32_t in_channels, int32_t out_channels);
int lat_build_identity_conv_plan(int32_t rows, void* plan, size_t plan_bytes, void* stream);
int lat_linear_tensor_cores(
    const void* feats, int32_t rows, int32_t in_channels, int64_t feat_row_stride,
    const void* weight, int32_t out_channels, const void* bias, const void* plan, void* out,
    int32_t* status, void* stream);

/* mlx_lattice/ops/feature.py:33-51 (`linear`, x @ W.T + b) and the pointwise
 * branch of conv3d (mlx_lattice/ops/conv.py:79-82,347-355). weight (C_out, C_in). */
int lat_linear(
    int32_t dtype, const void* feats, int32_t rows, int32_t in_channels,
    const void* weight, int32_t out_channels, const void* bias, void* out, void* stream);

/* mlx_lattice/ops/_quantized.py:8-38 (`quantized_matmul`, transpose=True): packed
 * (C_out, S*bits/32) uint32, scales/biases (C_out, S/group). */
int lat_quantized_linear(
    int32_t dtype, const void* feats, int32_t rows, int32_t in_channels,
    const uint32_t* packed, const void* scales, const void* biases,
    int32_t out_channels, int32_t storage_in_channels, int32_t group_size, int32_t bits,
    const void* bias, void* out, void* stream);

/* mlx_lattice/ops/feature.py:166-187 (`batch_norm` with running statistics) with
 * an optional fused ReLU (`relu`, feature.py:54-56). Any of weight/bias/mean/var
 * may be NULL. Evaluated in float32, cast once. */
int lat_batch_norm_relu(
    int32_t dtype, const void* feats, int64_t elements_rows, int32_t channels,
    const void* weight, const void* bias, const void* mean, const void* var, float eps,
    int32_t apply_relu, void* out, void* stream);

/* feature.py:54-56 (`relu`). */
int lat_relu(int32_t dtype, const void* feats, int64_t elements, void* out, void* stream);

/* mlx_lattice/ops/feature.py:196-225 (`layer_norm`, `rms_norm`): per row over the
 * channels, rms = 0: (x - mean) * rsqrt(var + eps) * weight + bias with the biased
 * variance; rms = 1: x * rsqrt(mean(x^2) + eps) * weight (bias must be NULL). weight and
 * bias [channels] may be NULL. Statistics in float32, cast once. */
int lat_row_norm(
    int32_t dtype, int32_t rms, const void* feats, int64_t rows, int32_t channels,
    const void* weight, const void* bias, float eps, void* out, void* stream);

/* mlx_lattice/ops/feature.py:59-129: op 0 sigmoid, 1 silu, 2 tanh, 3 gelu (erf form),
 * 4 gelu (tanh approximation), 5 gelu (x * sigmoid(1.702 x)), 6 leaky_relu (p0 = negative
 * slope), 7 softplus (p0 = beta > 0, p1 = threshold: x where beta x > threshold, else
 * log(1 + exp(beta x)) / beta). Evaluated in float32, cast once. */
int lat_activation(
    int32_t dtype, int32_t op, const void* feats, int64_t elements, float p0, float p1, void* out,
    void* stream);

/* Channel concatenation of two feature matrices read through row maps
 * (mlx_lattice/ops/tensor.py:228-249 `sparse_cat_aligned`, which gathers each side with
 * `gather_aligned_features`, tensor.py:89-109, and concatenates): out [rows_out,
 * lhs_channels + rhs_channels]; row r takes lhs[lhs_rows[r]] and rhs[rhs_rows[r]], zeros
 * where the map holds -1. A NULL map is the identity (tensors that share coordinates).
 * element_bytes = 2 or 4. */
int lat_concat_aligned_features(
    int32_t element_bytes, const void* lhs, const int32_t* lhs_rows, int32_t lhs_capacity,
    int32_t lhs_channels, const void* rhs, const int32_t* rhs_rows, int32_t rhs_capacity,
    int32_t rhs_channels, int64_t rows_out, void* out, int32_t* status, void* stream);

/* tensor.py:112-147 (`sparse_binary_op`) after the alignment is known: out[r] =
 * op(lhs[lhs_rows[r]] or lhs_fill, rhs[rhs_rows[r]] or rhs_fill), evaluated in the
 * element type; op: 0 add, 1 sub, 2 mul, 3 maximum, 4 minimum (tensor.py:285-296).
 * NULL maps are the identity. */
int lat_binary_aligned_features(
    int32_t dtype, int32_t op, const void* lhs, const int32_t* lhs_rows, int32_t lhs_capacity,
    float lhs_fill, const void* rhs, const int32_t* rhs_rows, int32_t rhs_capacity, float rhs_fill,
    int64_t rows_out, int32_t channels, void* out, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LATTICE_B200_H */
