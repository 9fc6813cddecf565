"""ctypes binding of ``liblattice_b200.so``.

There is no CPU fallback: importing the operators without the built library, or
calling them without an sm_100 GPU, raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

_PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_PACKAGE_DIR, 'liblattice_b200.so')

LAT_OK = 0
LAT_INVALID_ARGUMENT = 1
LAT_CUDA_ERROR = 2
LAT_UNSUPPORTED = 3
LAT_WORKSPACE_TOO_SMALL = 4

STATUS_BITS = {
    1: 'coordinate hash table is full',
    2: 'more edges or rows than the output capacity',
    4: 'row id or kernel id outside its range',
    8: 'a bounded in-kernel wait gave up',
    16: 'overlapping transposed relation met duplicate input coordinates',
}


class Triple(ctypes.Structure):
    _fields_ = [('x', c_int32), ('y', c_int32), ('z', c_int32)]


class FloatTriple(ctypes.Structure):
    _fields_ = [('x', c_float), ('y', c_float), ('z', c_float)]


P = c_void_p
I = c_int32

# name -> (restype, argtypes); mirrors include/lattice_b200.h one to one
SIGNATURES = {
    'lat_version': (c_char_p, []),
    'lat_last_error': (c_char_p, []),
    'lat_launch_count': (ctypes.c_longlong, []),
    'lat_set_wait_budget_cycles': (I, [c_int64]),
    'lat_wait_budget_cycles': (c_int64, []),
    'lat_capabilities': (I, [POINTER(c_int32), POINTER(c_int32)]),
    'lat_kernel_offsets_host': (I, [Triple, Triple, P]),
    'lat_relation_workspace_bytes': (c_size_t, [I, I, I]),
    'lat_coord_table_bytes': (c_size_t, [I]),
    'lat_build_coord_table': (I, [P, I, P, P, c_size_t, P, P]),
    'lat_build_kernel_relation': (
        I, [P, I, P, Triple, Triple, Triple, Triple, P, P, P, P, P, P, P, P, P, P, P, c_size_t, P, P]),
    'lat_build_submanifold_kernel_relation': (
        I, [P, I, P, Triple, Triple, P, P, P, P, P, P, P, P, P, P, P, c_size_t, P, P]),
    'lat_build_target_kernel_relation': (
        I, [P, I, P, P, I, P, Triple, Triple, Triple, Triple, P, P, P, P, P, P, P, P, P,
            c_size_t, P, P]),
    'lat_build_transposed_kernel_relation': (
        I, [P, I, P, Triple, Triple, Triple, Triple, P, P, P, P, P, P, P, c_size_t, P, P]),
    'lat_build_generative_relation': (
        I, [P, I, P, Triple, Triple, P, P, P, P, P, P, P, c_size_t, P, P]),
    'lat_build_target_transposed_relation': (
        I, [P, I, P, P, I, P, Triple, P, P, P, P, P, P, P, P, c_size_t, P, P]),
    'lat_grouped_view_workspace_bytes': (c_size_t, [I, I]),
    'lat_build_relation_grouped_view': (I, [P, I, P, I, P, P, P, c_size_t, P, P]),
    'lat_implicit_gemm_view_workspace_bytes': (c_size_t, [I]),
    'lat_build_relation_implicit_gemm_view': (
        I, [P, I, P, P, I, P, P, I, Triple, Triple, P, P, P, c_size_t, P, P]),
    'lat_coord_set_workspace_bytes': (c_size_t, [I]),
    'lat_downsample_coords': (I, [P, I, Triple, P, P, P, c_size_t, P, P]),
    'lat_lookup_coords': (I, [P, I, P, I, P, P, c_size_t, P, P]),
    'lat_lookup_coords_static_max_rows': (I, []),
    'lat_lookup_coords_static': (I, [P, I, P, I, P, P, P]),
    'lat_sparse_alignment_workspace_bytes': (c_size_t, [I, I]),
    'lat_build_sparse_alignment': (I, [P, I, P, P, I, P, I, P, P, P, P, P, c_size_t, P, P]),
    'lat_sparse_conv_workspace_bytes': (c_size_t, [I, I, I]),
    'lat_sparse_conv_features': (
        I, [I, P, I, I, c_int64, P, I, c_int64, P, I, Triple, I, P, P, P, I, P, P, I, I, P, P, P, P, P,
            c_size_t, P, P]),
    'lat_sparse_quantized_conv_features': (
        I, [I, P, I, c_int64, P, I, c_int64, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, P, P, P, P, P,
            c_size_t, P, P]),
    'lat_dequantize_conv_weights': (I, [P, P, P, I, I, I, I, I, I, P, P]),
    'lat_conv_plan_bytes': (c_size_t, [I, I]),
    'lat_build_conv_plan': (I, [P, P, I, P, P, I, I, I, P, P, P, c_size_t, P, P]),
    'lat_conv_uses_tensor_cores': (I, [I, I, I, I, I, I]),
    'lat_mask_order_workspace_bytes': (c_size_t, [I]),
    'lat_build_mask_row_order': (I, [P, I, I, P, P, P, c_size_t, P, P]),
    'lat_sparse_quantize_workspace_bytes': (c_size_t, [I]),
    'lat_sparse_quantize': (I, [P, P, I, P, FloatTriple, FloatTriple, P, P, P, P, P, c_size_t, P, P]),
    'lat_voxelize_features_workspace_bytes': (c_size_t, [I, I]),
    'lat_voxelize_features': (I, [P, P, P, P, I, I, I, I, P, P, c_size_t, P, P]),
    'lat_point_voxel_map_workspace_bytes': (c_size_t, [I]),
    'lat_build_point_voxel_map': (I, [P, P, I, P, P, I, P, FloatTriple, FloatTriple, I, P, P, P, c_size_t, P, P]),
    'lat_interpolate_point_features': (I, [P, P, P, I, I, I, P, P]),
    'lat_sparse_pool_features': (
        I, [P, I, I, c_int64, P, P, P, I, P, P, I, I, I, I, P, P, P]),
    'lat_global_pool': (I, [P, I, I, P, I, I, P, P]),
    'lat_linear': (I, [I, P, I, I, P, I, P, P, P]),
    'lat_linear_uses_tensor_cores': (I, [I, I, I]),
    'lat_build_identity_conv_plan': (I, [I, P, c_size_t, P]),
    'lat_linear_tensor_cores': (I, [P, I, I, c_int64, P, I, P, P, P, P, P]),
    'lat_quantized_linear': (I, [I, P, I, I, P, P, P, I, I, I, I, P, P, P]),
    'lat_batch_norm_relu': (I, [I, P, c_int64, I, P, P, P, P, c_float, I, P, P]),
    'lat_relu': (I, [I, P, c_int64, P, P]),
    'lat_activation': (I, [I, I, P, c_int64, c_float, c_float, P, P]),
    'lat_row_norm': (I, [I, I, P, c_int64, I, P, P, c_float, P, P]),
    'lat_concat_aligned_features': (I, [I, P, P, I, I, P, P, I, I, c_int64, P, P, P]),
    'lat_binary_aligned_features': (
        I, [I, I, P, P, I, c_float, P, P, I, c_float, c_int64, I, P, P, P]),
}

_lib = None


def library_present() -> bool:
    return os.path.exists(LIBRARY_PATH)


def load() -> ctypes.CDLL:
    """Load the library and declare every signature. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not library_present():
        raise RuntimeError(
            f'{LIBRARY_PATH} is not built; run `python -m mlx_lattice_b200.build`. '
            'This package has no CPU fallback.'
        )
    lib = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().lat_last_error().decode()


def check(code: int) -> None:
    """Translate a status code into the exception the reference would raise."""
    if code == LAT_OK:
        return
    message = last_error()
    if code == LAT_INVALID_ARGUMENT:
        raise ValueError(message)
    raise RuntimeError(message)
