"""Test infrastructure only -- ctypes access to ``oracle/_ref/liblattice_ref.so``.

That library is the reference project's own CPU code (compiled unmodified by
``oracle/Makefile``). The functions here size the output buffers exactly as the
reference factory layer does (``native/features/coordinates/relations.cpp:72-89,
540-722``) and return numpy arrays. Nothing in the shipped package imports this
module; it is the checker used by tests, the smoke check and the CPU-baseline leg
of the benchmark.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, '_ref', 'liblattice_ref.so')
_lib = None


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(
                f'{_LIB_PATH} is missing; run `make -C oracle` where the '
                'reference checkout is present.'
            )
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


class _Ptr(ctypes.c_void_p):
    """A pointer argument that keeps its numpy buffer alive for the call."""


def _p(array: np.ndarray) -> ctypes.c_void_p:
    pointer = _Ptr(array.ctypes.data)
    pointer._keepalive = array
    return pointer


def _t(values: int | Sequence[int]) -> np.ndarray:
    if isinstance(values, (int, np.integer)):
        values = (int(values),) * 3
    out = np.asarray(values, dtype=np.int32)
    assert out.shape == (3,)
    return np.ascontiguousarray(out)


def _i32(array) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(array, dtype=np.int32))


def _check(status: int, name: str) -> None:
    if status != 0:
        raise ValueError(f'reference {name} raised an exception')


def kernel_offsets(kernel_size, dilation=1) -> np.ndarray:
    """``kernel_offsets`` of ``native/features/coordinates/offsets.cpp:11-45``."""
    ks, dil = _t(kernel_size), _t(dilation)
    out = np.zeros((int(np.prod(ks)), 3), dtype=np.int32)
    _check(lib().ref_kernel_offsets(_p(ks), _p(dil), _p(out)), 'kernel_offsets')
    return out


def can_use_direct_transposed(offsets: np.ndarray, stride) -> bool:
    """Restates ``relations.cpp:107-126`` (the factory layer needs real MLX)."""
    stride = _t(stride)
    if len(offsets) == 0:
        return False
    extent = offsets.max(axis=0) - offsets.min(axis=0)
    return bool(np.all(stride > extent))


def _relation_dict(in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts):
    return {
        'in_rows': in_rows,
        'out_rows': out_rows,
        'kernel_ids': kernel_ids,
        'row_offsets': row_offsets,
        'out_coords': out_coords,
        'counts': counts,
    }


def _add_views(rel: dict, in_capacity: int, kernel_count: int) -> dict:
    """Input CSR and kernel CSR views (``relations.cpp:461-476``)."""
    rel['in_row_offsets'], rel['in_edge_ids'] = grouped_view(
        rel['in_rows'], rel['counts'], in_capacity
    )
    rel['kernel_row_offsets'], rel['kernel_edge_ids'] = grouped_view(
        rel['kernel_ids'], rel['counts'], kernel_count
    )
    return rel


def build_kernel_relation(
    coords, active_rows=None, kernel_size=3, stride=1, padding=0, dilation=1
) -> dict:
    """Forward relation (``make_kernel_relation``, ``relations.cpp:540-581``)."""
    coords = _i32(coords)
    rows = coords.shape[0]
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    active = rows if active_rows is None else int(active_rows)
    cap = rows * k
    rel = _relation_dict(
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(rows + 1, np.int32),
        np.zeros((rows, 4), np.int32),
        np.zeros(2, np.int32),
    )
    _check(
        lib().ref_generic_kernel_relation(
            0, _p(_t(stride)), _p(_t(padding)), 0, _p(coords), rows,
            _p(offsets), k, active, cap, rows,
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            _p(rel['row_offsets']), _p(rel['out_coords']), _p(rel['counts']),
        ),
        'build_kernel_relation',
    )
    return _add_views(rel, rows, k)


def build_submanifold_kernel_relation(
    coords, active_rows=None, kernel_size=3, dilation=1
) -> dict:
    return build_kernel_relation(coords, active_rows, kernel_size, 1, 0, dilation)


def build_transposed_kernel_relation(
    coords, active_rows=None, kernel_size=2, stride=2, padding=0, dilation=1
) -> dict:
    """``make_transposed_kernel_relation`` (``relations.cpp:632-670``)."""
    coords = _i32(coords)
    rows = coords.shape[0]
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    active = rows if active_rows is None else int(active_rows)
    cap = rows * k
    direct = can_use_direct_transposed(offsets, stride)
    rel = _relation_dict(
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap + 1, np.int32),
        np.zeros((cap, 4), np.int32),
        np.zeros(2, np.int32),
    )
    _check(
        lib().ref_generic_kernel_relation(
            1, _p(_t(stride)), _p(_t(padding)), int(direct), _p(coords), rows,
            _p(offsets), k, active, cap, cap,
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            _p(rel['row_offsets']), _p(rel['out_coords']), _p(rel['counts']),
        ),
        'build_transposed_kernel_relation',
    )
    return _add_views(rel, rows, k)


def build_generative_relation(
    coords, active_rows=None, kernel_size=2, stride=2
) -> dict:
    """``make_generative_relation`` (``relations.cpp:599-630``)."""
    coords = _i32(coords)
    rows = coords.shape[0]
    offsets = kernel_offsets(kernel_size, 1)
    k = offsets.shape[0]
    active = rows if active_rows is None else int(active_rows)
    cap = rows * k
    rel = _relation_dict(
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap + 1, np.int32),
        np.zeros((cap, 4), np.int32),
        np.zeros(2, np.int32),
    )
    _check(
        lib().ref_generative_kernel_relation(
            _p(_t(stride)), _p(coords), rows, _p(offsets), k, active,
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            _p(rel['row_offsets']), _p(rel['out_coords']), _p(rel['counts']),
        ),
        'build_generative_relation',
    )
    return _add_views(rel, rows, k)


def build_target_kernel_relation(
    coords,
    target_coords,
    active_rows=None,
    target_active_rows=None,
    kernel_size=3,
    stride=1,
    padding=0,
    dilation=1,
) -> dict:
    """``make_target_kernel_relation`` (``relations.cpp:672-722``); the relation
    reports the caller's target coords as ``out_coords`` (``relations.cpp:53-70``)."""
    coords = _i32(coords)
    target = _i32(target_coords)
    rows, target_rows = coords.shape[0], target.shape[0]
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    active = rows if active_rows is None else int(active_rows)
    target_active = (
        target_rows if target_active_rows is None else int(target_active_rows)
    )
    cap = target_rows * k
    rel = _relation_dict(
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(cap, np.int32),
        np.zeros(target_rows + 1, np.int32),
        target,
        np.zeros(2, np.int32),
    )
    _check(
        lib().ref_target_kernel_relation(
            _p(_t(stride)), _p(_t(padding)), _p(coords), rows, _p(offsets), k,
            active, _p(target), target_rows, target_active,
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            _p(rel['row_offsets']), _p(rel['counts']),
        ),
        'build_target_kernel_relation',
    )
    return _add_views(rel, rows, k)


def grouped_view(group_ids, counts, group_count: int):
    group_ids, counts = _i32(group_ids), _i32(counts)
    cap = group_ids.shape[0]
    row_offsets = np.zeros(group_count + 1, np.int32)
    edge_ids = np.zeros(cap, np.int32)
    _check(
        lib().ref_relation_grouped_view(
            _p(group_ids), cap, _p(counts), group_count,
            _p(row_offsets), _p(edge_ids),
        ),
        'relation_grouped_view',
    )
    return row_offsets, edge_ids


def implicit_gemm_view(
    source_coords, source_active, output_coords, output_active, offsets,
    stride=1, padding=0,
):
    src, out, offsets = _i32(source_coords), _i32(output_coords), _i32(offsets)
    k = offsets.shape[0]
    words = (k + 31) // 32
    out_in_map = np.zeros((out.shape[0], k), np.int32)
    row_masks = np.zeros((out.shape[0], words), np.int32)
    _check(
        lib().ref_relation_implicit_gemm_view(
            _p(src), src.shape[0], int(source_active), _p(out), out.shape[0],
            int(output_active), _p(offsets), k, _p(_t(stride)), _p(_t(padding)),
            _p(out_in_map), _p(row_masks),
        ),
        'relation_implicit_gemm_view',
    )
    return out_in_map, row_masks


def downsample_coords(coords, stride):
    coords = _i32(coords)
    out = np.zeros_like(coords)
    count = np.zeros(1, np.int32)
    _check(
        lib().ref_downsample_coords(
            _p(coords), coords.shape[0], _p(_t(stride)), _p(out), _p(count)
        ),
        'downsample_coords',
    )
    return out, count


def sparse_quantize(points, batch_indices=None, active_rows=None, voxel_size=1.0, origin=0.0):
    """``eval_sparse_quantize`` (``cpu/quantization_algorithms.cpp``): coords (N, 4),
    count (1,), inverse rows (N,), points per voxel (N,)."""
    points = np.ascontiguousarray(points, np.float32).reshape(-1, 3)
    rows = points.shape[0]
    batch = np.zeros(rows, np.int32) if batch_indices is None else _i32(batch_indices)
    active = np.asarray([rows if active_rows is None else int(np.asarray(active_rows).ravel()[0])], np.int32)
    vs = np.ascontiguousarray(np.broadcast_to(np.asarray(voxel_size, np.float32), (3,)))
    og = np.ascontiguousarray(np.broadcast_to(np.asarray(origin, np.float32), (3,)))
    coords = np.zeros((rows, 4), np.int32)
    count = np.zeros(1, np.int32)
    inverse = np.zeros(rows, np.int32)
    voxel_counts = np.zeros(rows, np.int32)
    _check(
        lib().ref_sparse_quantize(
            _p(points), _p(batch), rows, _p(active), _p(vs), _p(og), _p(coords), _p(count),
            _p(inverse), _p(voxel_counts)
        ),
        'sparse_quantize',
    )
    return coords, count, inverse, voxel_counts


def voxelize_features(values, inverse_rows, voxel_counts, active_rows, reduction='mean'):
    """``eval_voxelize_features``: (voxel rows, C) float32, voxel rows = len(voxel_counts)."""
    values = np.ascontiguousarray(values, np.float32)
    inverse, voxel_counts = _i32(inverse_rows), _i32(voxel_counts)
    active = np.asarray([int(np.asarray(active_rows).ravel()[0])], np.int32)
    out = np.zeros((voxel_counts.shape[0], values.shape[1]), np.float32)
    _check(
        lib().ref_voxelize_features(
            _p(values), _p(inverse), _p(voxel_counts), _p(active), values.shape[0],
            voxel_counts.shape[0], values.shape[1], 1 if reduction == 'mean' else 0, _p(out)
        ),
        'voxelize_features',
    )
    return out


def point_voxel_map(points, batch_indices, point_active, voxel_coords, voxel_active,
                    voxel_size=1.0, origin=0.0, interpolation='linear'):
    """``eval_point_voxel_map``: rows (P, 8) int32 and weights (P, 8) float32."""
    points = np.ascontiguousarray(points, np.float32).reshape(-1, 3)
    rows = points.shape[0]
    batch = np.zeros(rows, np.int32) if batch_indices is None else _i32(batch_indices)
    voxel_coords = _i32(voxel_coords).reshape(-1, 4)
    p_active = np.asarray([rows if point_active is None else int(np.asarray(point_active).ravel()[0])], np.int32)
    v_active = np.asarray([voxel_coords.shape[0] if voxel_active is None
                           else int(np.asarray(voxel_active).ravel()[0])], np.int32)
    vs = np.ascontiguousarray(np.broadcast_to(np.asarray(voxel_size, np.float32), (3,)))
    og = np.ascontiguousarray(np.broadcast_to(np.asarray(origin, np.float32), (3,)))
    out_rows = np.zeros((rows, 8), np.int32)
    weights = np.zeros((rows, 8), np.float32)
    _check(
        lib().ref_point_voxel_map(
            _p(points), _p(batch), rows, _p(p_active), _p(voxel_coords), voxel_coords.shape[0],
            _p(v_active), _p(vs), _p(og), 1 if interpolation == 'linear' else 0, _p(out_rows),
            _p(weights)
        ),
        'point_voxel_map',
    )
    return out_rows, weights


def interpolate_point_features(values, rows, weights):
    """``eval_interpolate_point_features``: (P, C) float32."""
    values = np.ascontiguousarray(values, np.float32)
    rows, weights = _i32(rows), np.ascontiguousarray(weights, np.float32)
    out = np.zeros((rows.shape[0], values.shape[1]), np.float32)
    _check(
        lib().ref_interpolate_point_features(
            _p(values), _p(rows), _p(weights), rows.shape[0], values.shape[0], values.shape[1], _p(out)
        ),
        'interpolate_point_features',
    )
    return out


def lookup_coords(coords, queries):
    coords, queries = _i32(coords), _i32(queries)
    out = np.zeros(queries.shape[0], np.int32)
    _check(
        lib().ref_lookup_coords(
            _p(coords), coords.shape[0], _p(queries), queries.shape[0], _p(out)
        ),
        'lookup_coords',
    )
    return out


_JOINS = {'inner': 0, 'left': 1, 'right': 2, 'outer': 3}


def sparse_alignment(lhs_coords, lhs_active, rhs_coords, rhs_active, join):
    """Output capacity per ``native/features/coordinates/lookup.cpp:95-146``."""
    lhs, rhs = _i32(lhs_coords), _i32(rhs_coords)
    capacity = {
        'inner': lhs.shape[0],
        'left': lhs.shape[0],
        'right': rhs.shape[0],
        'outer': lhs.shape[0] + rhs.shape[0],
    }[join]
    coords = np.zeros((capacity, 4), np.int32)
    count = np.zeros(1, np.int32)
    lhs_rows = np.zeros(capacity, np.int32)
    rhs_rows = np.zeros(capacity, np.int32)
    _check(
        lib().ref_sparse_alignment(
            _JOINS[join], _p(lhs), lhs.shape[0], int(lhs_active), _p(rhs),
            rhs.shape[0], int(rhs_active), capacity,
            _p(coords), _p(count), _p(lhs_rows), _p(rhs_rows),
        ),
        'sparse_alignment',
    )
    return coords, count, lhs_rows, rhs_rows


def _weight_geometry(weights: np.ndarray, n_kernels: int):
    if weights.ndim == 3:
        return 0, (n_kernels, 1, 1), weights.shape[1], weights.shape[2]
    if weights.ndim == 5:
        return 1, tuple(weights.shape[1:4]), weights.shape[4], weights.shape[0]
    raise ValueError('weights must be (K, Cin, Cout) or (Cout, Kx, Ky, Kz, Cin)')


def sparse_conv(feats, weights, rel: dict, out_capacity: int, n_kernels: int):
    """Float conv forward through ``backend::cpu::conv::eval``."""
    feats = np.ascontiguousarray(feats)
    weights = np.ascontiguousarray(weights)
    assert feats.dtype == weights.dtype and feats.dtype in (np.float32, np.float16)
    layout, (kx, ky, kz), c_in, c_out = _weight_geometry(weights, n_kernels)
    assert feats.shape[1] == c_in
    out = np.zeros((out_capacity, c_out), feats.dtype)
    _check(
        lib().ref_sparse_conv(
            int(feats.dtype == np.float16), _p(feats), feats.shape[0], c_in,
            _p(weights), layout, kx, ky, kz, c_out,
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            rel['in_rows'].shape[0], _p(rel['counts']), _p(rel['row_offsets']),
            out_capacity, n_kernels, _p(out),
        ),
        'sparse_conv',
    )
    return out


def sparse_quantized_conv(
    feats, packed, scales, biases, rel: dict, out_capacity: int, n_kernels: int,
    in_channels: int, out_channels: int, storage_in_channels: int,
    group_size: int, bits: int,
):
    """Quantized conv forward through ``backend::cpu::conv::eval_quantized``."""
    feats = np.ascontiguousarray(feats)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales)
    biases = np.ascontiguousarray(biases)
    assert feats.dtype == scales.dtype == biases.dtype
    assert feats.shape[1] == in_channels
    out = np.zeros((out_capacity, out_channels), feats.dtype)
    _check(
        lib().ref_sparse_quantized_conv(
            int(feats.dtype == np.float16), _p(feats), feats.shape[0],
            _p(packed), _p(scales), _p(biases),
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            rel['in_rows'].shape[0], _p(rel['counts']), _p(rel['row_offsets']),
            out_capacity, n_kernels, in_channels, out_channels,
            storage_in_channels, group_size, bits, _p(out),
        ),
        'sparse_quantized_conv',
    )
    return out


_REDUCE = {'sum': 0, 'max': 1, 'avg': 2}


def sparse_pool(
    feats, rel: dict, *, input_exclusive: bool, reduce: str,
    out_capacity: int, n_kernels: int,
):
    feats = np.ascontiguousarray(feats, dtype=np.float32)
    out = np.zeros((out_capacity, feats.shape[1]), np.float32)
    _check(
        lib().ref_sparse_pool(
            _REDUCE[reduce], _p(feats), feats.shape[0], feats.shape[1],
            _p(rel['in_rows']), _p(rel['out_rows']), _p(rel['kernel_ids']),
            rel['in_rows'].shape[0], _p(rel['row_offsets']), _p(rel['counts']),
            int(input_exclusive), out_capacity, n_kernels, _p(out),
        ),
        'sparse_pool',
    )
    return out
