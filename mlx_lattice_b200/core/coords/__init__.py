from mlx_lattice_b200.core.coords.builders import (
    build_generative_relation,
    build_kernel_relation,
    build_relation_implicit_gemm_view,
    build_submanifold_kernel_relation,
    build_target_kernel_relation,
    build_target_transposed_relation,
    build_transposed_kernel_relation,
    kernel_offsets,
)
from mlx_lattice_b200.core.coords.manager import CoordinateManager, CoordinateMapKey
from mlx_lattice_b200.core.coords.validation import validate_coords

__all__ = [
    'CoordinateManager',
    'CoordinateMapKey',
    'build_generative_relation',
    'build_kernel_relation',
    'build_relation_implicit_gemm_view',
    'build_submanifold_kernel_relation',
    'build_target_kernel_relation',
    'build_target_transposed_relation',
    'build_transposed_kernel_relation',
    'kernel_offsets',
    'validate_coords',
]
