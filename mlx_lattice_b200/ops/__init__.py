from mlx_lattice_b200.core.coords.builders import (
    build_generative_relation,
    build_kernel_relation,
    build_submanifold_kernel_relation,
    build_target_kernel_relation,
    build_target_transposed_relation,
    build_transposed_kernel_relation,
    kernel_offsets,
)
from mlx_lattice_b200.ops.conv import (
    conv3d,
    conv_transpose3d,
    generative_conv_transpose3d,
    subm_conv3d,
)
from mlx_lattice_b200.ops.feature import (
    batch_norm,
    dropout,
    gelu,
    layer_norm,
    leaky_relu,
    linear,
    relu,
    rms_norm,
    sigmoid,
    silu,
    softplus,
    tanh,
)
from mlx_lattice_b200.ops.pool import (
    avg_pool3d,
    global_avg_pool,
    global_max_pool,
    global_sum_pool,
    max_pool3d,
    pool3d,
    sum_pool3d,
)
from mlx_lattice_b200.ops.quantization import (
    build_point_voxel_map,
    devoxelize,
    interpolate_point_features,
    sparse_quantize,
    voxelize,
    voxelize_with_quantization,
)
from mlx_lattice_b200.ops.tensor import (
    align_sparse,
    sparse_add,
    sparse_binary_op,
    sparse_cat_aligned,
    sparse_collate,
    sparse_maximum,
    sparse_minimum,
    sparse_mul,
    sparse_sub,
)

__all__ = [
    'dropout', 'gelu', 'layer_norm', 'leaky_relu', 'rms_norm', 'sigmoid', 'silu', 'softplus', 'tanh',
    'align_sparse', 'sparse_add', 'sparse_binary_op', 'sparse_maximum', 'sparse_minimum', 'sparse_mul',
    'sparse_sub',
    'avg_pool3d', 'batch_norm', 'build_generative_relation', 'build_point_voxel_map', 'devoxelize',
    'interpolate_point_features', 'build_kernel_relation',
    'build_submanifold_kernel_relation', 'build_target_kernel_relation',
    'build_target_transposed_relation', 'build_transposed_kernel_relation', 'conv3d',
    'conv_transpose3d', 'generative_conv_transpose3d', 'global_avg_pool', 'global_max_pool',
    'global_sum_pool', 'kernel_offsets', 'linear', 'max_pool3d', 'pool3d', 'relu',
    'sparse_cat_aligned', 'sparse_collate', 'sparse_quantize', 'subm_conv3d', 'sum_pool3d',
    'voxelize', 'voxelize_with_quantization',
]
