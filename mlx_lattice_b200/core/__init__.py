from mlx_lattice_b200.core.coords import (
    CoordinateManager,
    CoordinateMapKey,
    build_generative_relation,
    build_kernel_relation,
    build_submanifold_kernel_relation,
    build_target_kernel_relation,
    build_target_transposed_relation,
    build_transposed_kernel_relation,
    kernel_offsets,
)
from mlx_lattice_b200.core.quantized import (
    QuantizedWeight,
    dequantize_weight,
    quantize_weight,
)
from mlx_lattice_b200.core.relations import KernelRelation, KernelSpec
from mlx_lattice_b200.core.tensor import SparseTensor

__all__ = [
    'CoordinateManager',
    'CoordinateMapKey',
    'KernelRelation',
    'KernelSpec',
    'QuantizedWeight',
    'SparseTensor',
    'build_generative_relation',
    'build_kernel_relation',
    'build_submanifold_kernel_relation',
    'build_target_kernel_relation',
    'build_target_transposed_relation',
    'build_transposed_kernel_relation',
    'dequantize_weight',
    'kernel_offsets',
    'quantize_weight',
]
