"""Test infrastructure only -- a numpy restatement of the reference CPU route.

Each function follows one function of the reference project (cited by file:line,
paths relative to the reference checkout). It exists so that parity can be checked
on machines where the compiled reference (``oracle/_ref``) is absent, and to state
the algorithm in one readable place. It is pinned against the reference's own
known-answer tests (``tests/golden/reference_kats.json``) and against outputs of the
compiled reference (``tests/golden/*.npz``) by ``tests/test_oracle.py``.

Parity status: kernel maps, views, float conv, quantized conv and pooling are
pinned by the reference's own tests and by the compiled reference. The affine
quantizer (``quantize_affine``) and ``quantized_matmul`` restate the published
algorithm of the third-party MLX library (mlx 0.31.2, not present here): their
code selection is PARITY UNPINNED; only the packed storage format and the decode
rule are pinned (``native/features/convolution/cpu/quantized.cpp:54-62,107-131``).

Nothing in the shipped package imports this module.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np

# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #


def triple(values) -> tuple[int, int, int]:
    if isinstance(values, (int, np.integer)):
        return (int(values),) * 3
    out = tuple(int(v) for v in values)
    if len(out) != 3:
        raise ValueError('expected an int or three ints')
    return out


def kernel_offsets(kernel_size, dilation=1) -> np.ndarray:
    """``native/features/coordinates/offsets.cpp:11-45``: x-major, z-fastest; odd
    sizes are centred, even sizes start at 0; scaled by dilation."""
    ks, dil = triple(kernel_size), triple(dilation)
    axes = []
    for size in ks:
        if size % 2 == 1:
            axes.append(range(-(size // 2), size // 2 + 1))
        else:
            axes.append(range(size))
    out = [
        (x * dil[0], y * dil[1], z * dil[2])
        for x in axes[0]
        for y in axes[1]
        for z in axes[2]
    ]
    return np.asarray(out, dtype=np.int32).reshape(-1, 3)


def _keys(*coord_sets: np.ndarray) -> list[np.ndarray]:
    """Map (b,x,y,z) rows of several arrays to comparable scalar ids.

    Mixed-radix int64 packing when the value ranges allow it, else a dense rank
    from a row-wise unique. Equal rows get equal ids across all inputs.
    """
    stacked = [np.asarray(c, dtype=np.int64).reshape(-1, 4) for c in coord_sets]
    total = np.concatenate(stacked, axis=0)
    if total.shape[0] == 0:
        return [np.zeros(0, np.int64) for _ in stacked]
    lo = total.min(axis=0)
    span = total.max(axis=0) - lo + 1
    bits = sum(int(s).bit_length() for s in span)
    if bits <= 62:
        out = []
        for c in stacked:
            key = np.zeros(c.shape[0], np.int64)
            for axis in range(4):
                key = key * int(span[axis]) + (c[:, axis] - lo[axis])
            out.append(key)
        return out
    _, inverse = np.unique(total, axis=0, return_inverse=True)
    inverse = inverse.reshape(-1).astype(np.int64)
    out, start = [], 0
    for c in stacked:
        out.append(inverse[start : start + c.shape[0]])
        start += c.shape[0]
    return out


def _first_rows(source_keys: np.ndarray):
    """``first_row_map`` (``cpu/quantization_detail.h:394-402``): key -> first row."""
    uniq, first = np.unique(source_keys, return_index=True)
    return uniq, first.astype(np.int32)


def _lookup(uniq: np.ndarray, first: np.ndarray, query_keys: np.ndarray) -> np.ndarray:
    if uniq.shape[0] == 0:
        return np.full(query_keys.shape, -1, np.int32)
    pos = np.searchsorted(uniq, query_keys)
    pos = np.minimum(pos, uniq.shape[0] - 1)
    hit = uniq[pos] == query_keys
    return np.where(hit, first[pos], -1).astype(np.int32)


def downsample_values(coords: np.ndarray, stride) -> np.ndarray:
    """``floor_div`` + ``downsample_values`` (``cpu/quantization_detail.h:3-31``):
    unique (b, floor(x/sx), floor(y/sy), floor(z/sz)) in first-seen order."""
    s = triple(stride)
    q = np.asarray(coords, dtype=np.int64).reshape(-1, 4).copy()
    for axis in range(3):
        q[:, axis + 1] = np.floor_divide(q[:, axis + 1], s[axis])
    (keys,) = _keys(q)
    _, first = np.unique(keys, return_index=True)
    return q[np.sort(first)].astype(np.int32)


def sparse_quantize(points, batch_indices=None, active_rows=None, voxel_size=1.0, origin=0.0):
    """``write_sparse_quantization`` (``cpu/quantization_detail.h:87-125``) with
    ``voxel_coord_for_point`` (``:67-85``): voxel = (batch, floor((p - origin) / size)) in
    float32; unique voxels in first-seen point order, the voxel row of every active
    point (-1 beyond), points per voxel."""
    points = np.asarray(points, np.float32).reshape(-1, 3)
    rows = points.shape[0]
    batch = np.zeros(rows, np.int32) if batch_indices is None else np.asarray(batch_indices, np.int32)
    active = rows if active_rows is None else min(int(np.asarray(active_rows).ravel()[0]), rows)
    vs = np.broadcast_to(np.asarray(voxel_size, np.float32), (3,))
    og = np.broadcast_to(np.asarray(origin, np.float32), (3,))
    cells = np.floor((points[:active] - og[None, :]) / vs[None, :]).astype(np.int64)
    q = np.concatenate([batch[:active, None].astype(np.int64), cells], axis=1)
    coords = np.zeros((rows, 4), np.int32)
    inverse = np.full(rows, -1, np.int32)
    counts = np.zeros(rows, np.int32)
    if active > 0:
        (keys,) = _keys(q)
        _, first, inv = np.unique(keys, return_index=True, return_inverse=True)
        order = np.argsort(first, kind='stable')          # unique ids in first-seen order
        rank = np.empty_like(order)
        rank[order] = np.arange(order.shape[0])
        voxel = rank[inv.reshape(-1)]
        n = order.shape[0]
        coords[:n] = q[np.sort(first)].astype(np.int32)
        inverse[:active] = voxel
        counts[:n] = np.bincount(voxel, minlength=n)
    else:
        n = 0
    return coords, np.asarray([n], np.int32), inverse, counts


def voxelize_features(values, inverse_rows, voxel_counts, active_rows, reduction='mean'):
    """``write_voxel_features`` (``cpu/quantization_detail.h:138-166``): float32 running
    sum per voxel in point order of value * scale, scale = 1 / max(count, 1) for the mean.
    (The compiled reference fuses the multiply-add; this restatement rounds the product,
    so it agrees to a few ulp, not bitwise.)"""
    values = np.asarray(values, np.float32)
    inverse = np.asarray(inverse_rows, np.int32)
    counts = np.asarray(voxel_counts, np.int32)
    active = min(int(np.asarray(active_rows).ravel()[0]), values.shape[0])
    out = np.zeros((counts.shape[0], values.shape[1]), np.float32)
    scale = np.float32(1.0) / np.maximum(counts, 1).astype(np.float32) if reduction == 'mean' else None
    for p in range(active):
        v = inverse[p]
        if v < 0 or v >= counts.shape[0]:
            continue
        term = values[p] * scale[v] if scale is not None else values[p]
        out[v] = out[v] + term
    return out


def point_voxel_map(points, batch_indices, point_active, voxel_coords, voxel_active,
                    voxel_size=1.0, origin=0.0, interpolation='linear'):
    """``write_nearest_point_voxel_map`` / ``write_linear_point_voxel_map``
    (``cpu/quantization_detail.h:203-315``): eight (voxel row, weight) slots per point;
    positions (p - origin) / size in float32; nearest = floor(position + 0.5) in slot 0 with
    weight 1; linear = the eight corners above floor(position) with weights
    (wx * wy) * wz, w = 1 - frac or frac; absent voxels and inactive points stay (-1, 0)."""
    points = np.asarray(points, np.float32).reshape(-1, 3)
    rows = points.shape[0]
    batch = np.zeros(rows, np.int32) if batch_indices is None else np.asarray(batch_indices, np.int32)
    voxel_coords = np.asarray(voxel_coords, np.int32).reshape(-1, 4)
    p_active = rows if point_active is None else min(int(np.asarray(point_active).ravel()[0]), rows)
    v_active = voxel_coords.shape[0] if voxel_active is None else min(
        int(np.asarray(voxel_active).ravel()[0]), voxel_coords.shape[0])
    vs = np.broadcast_to(np.asarray(voxel_size, np.float32), (3,))
    og = np.broadcast_to(np.asarray(origin, np.float32), (3,))
    out_rows = np.full((rows, 8), -1, np.int32)
    weights = np.zeros((rows, 8), np.float32)
    pos = (points[:p_active] - og[None, :]) / vs[None, :]
    if interpolation == 'nearest':
        cell = np.floor(pos + np.float32(0.5)).astype(np.int64)
        q = np.concatenate([batch[:p_active, None].astype(np.int64), cell], axis=1)
        found = lookup_coords(voxel_coords[:v_active], q.astype(np.int32))
        out_rows[:p_active, 0] = found
        weights[:p_active, 0] = (found >= 0).astype(np.float32)
        return out_rows, weights
    lower = np.floor(pos)
    frac = (pos - lower).astype(np.float32)
    lower = lower.astype(np.int64)
    for corner in range(8):
        d = np.asarray([corner & 1, (corner >> 1) & 1, (corner >> 2) & 1])
        q = np.concatenate([batch[:p_active, None].astype(np.int64), lower + d[None, :]], axis=1)
        found = lookup_coords(voxel_coords[:v_active], q.astype(np.int32))
        w = [np.where(d[a] == 0, np.float32(1.0) - frac[:, a], frac[:, a]).astype(np.float32) for a in range(3)]
        weight = ((w[0] * w[1]).astype(np.float32) * w[2]).astype(np.float32)
        out_rows[:p_active, corner] = found
        weights[:p_active, corner] = np.where(found >= 0, weight, np.float32(0.0))
    return out_rows, weights


def interpolate_point_features(values, rows, weights):
    """``write_point_features`` (``cpu/quantization_detail.h:317-346``): running float32
    sum over the eight slots in order of value * weight (the compiled reference fuses the
    multiply-add; this restatement rounds the product)."""
    values = np.asarray(values, np.float32)
    rows = np.asarray(rows, np.int32)
    weights = np.asarray(weights, np.float32)
    out = np.zeros((rows.shape[0], values.shape[1]), np.float32)
    for corner in range(8):
        r = rows[:, corner]
        ok = (r >= 0) & (r < values.shape[0])
        term = values[np.where(ok, r, 0)] * weights[:, corner, None]
        out = np.where(ok[:, None], out + term, out).astype(np.float32)
    return out


def downsample_coords(coords, stride):
    """Set-op form (``cpu/set_algorithms.cpp:4-37``): zero-padded (N, 4) buffer
    with the unique rows as prefix, and the count."""
    coords = np.asarray(coords, np.int32).reshape(-1, 4)
    values = downsample_values(coords, stride)
    out = np.zeros_like(coords)
    out[: values.shape[0]] = values
    return out, np.asarray([values.shape[0]], np.int32)


def _candidates(out_coords: np.ndarray, offsets, stride, padding) -> np.ndarray:
    """``kernel_input_coord`` (``cpu/relation_views_detail.h:1-13``)."""
    s, p = triple(stride), triple(padding)
    out = np.asarray(out_coords, dtype=np.int64).reshape(-1, 1, 4)
    off = np.asarray(offsets, dtype=np.int64).reshape(1, -1, 3)
    cand = np.empty((out.shape[0], off.shape[1], 4), np.int64)
    cand[:, :, 0] = out[:, :, 0]
    for axis in range(3):
        cand[:, :, axis + 1] = (
            out[:, :, axis + 1] * s[axis] + off[:, :, axis] - p[axis]
        )
    return cand


def _map_rows(in_rows, out_rows, kernel_ids, edge_capacity, out_capacity, offsets_capacity=None):
    """``write_map_rows`` (``cpu/relation_views_detail.h:15-50``): zero-filled
    tails and a CSR by output row of ``out_capacity + 1`` entries (rows past the
    last edge repeat E). ``out_capacity`` is the row count the reference passes --
    N_out for forward / transposed / generative maps, the full target capacity for
    target maps -- and the array itself (``offsets_capacity + 1`` long) is zero
    beyond it (``cpu/common_detail.h:125-129``)."""
    e = in_rows.shape[0]
    rel = {
        'in_rows': np.zeros(edge_capacity, np.int32),
        'out_rows': np.zeros(edge_capacity, np.int32),
        'kernel_ids': np.zeros(edge_capacity, np.int32),
    }
    rel['in_rows'][:e] = in_rows
    rel['out_rows'][:e] = out_rows
    rel['kernel_ids'][:e] = kernel_ids
    degree = np.bincount(out_rows, minlength=out_capacity)[:out_capacity]
    row_offsets = np.zeros(out_capacity + 1, np.int64)
    np.cumsum(degree, out=row_offsets[1:])
    full = np.zeros((out_capacity if offsets_capacity is None else offsets_capacity) + 1, np.int32)
    full[: out_capacity + 1] = row_offsets
    rel['row_offsets'] = full
    return rel


def grouped_view(group_ids, counts, group_count: int):
    """``write_relation_grouped_view`` (``cpu/relation_views_detail.h:84-120``):
    stable counting sort of edge ids by group, -1 fill."""
    group_ids = np.asarray(group_ids, np.int32)
    cap = group_ids.shape[0]
    e = int(np.clip(counts[0], 0, cap))
    g = group_ids[:e]
    valid = (g >= 0) & (g < group_count)
    edges = np.arange(e, dtype=np.int32)[valid]
    g = g[valid]
    offsets = np.zeros(group_count + 1, np.int64)
    np.cumsum(np.bincount(g, minlength=group_count)[:group_count], out=offsets[1:])
    edge_ids = np.full(cap, -1, np.int32)
    order = np.argsort(g, kind='stable')
    edge_ids[: order.shape[0]] = edges[order]
    return offsets.astype(np.int32), edge_ids


def _with_views(rel: dict, in_capacity: int, kernel_count: int) -> dict:
    """``make_kernel_relation_views`` (``relations.cpp:461-476``)."""
    rel['in_row_offsets'], rel['in_edge_ids'] = grouped_view(
        rel['in_rows'], rel['counts'], in_capacity
    )
    rel['kernel_row_offsets'], rel['kernel_edge_ids'] = grouped_view(
        rel['kernel_ids'], rel['counts'], kernel_count
    )
    return rel


# --------------------------------------------------------------------------- #
# kernel maps
# --------------------------------------------------------------------------- #


def build_kernel_relation(
    coords, active_rows=None, kernel_size=3, stride=1, padding=0, dilation=1
) -> dict:
    """``write_kernel_relation`` (``cpu/relation_build_detail.h:3-41``) with the
    capacities of ``make_kernel_relation`` (``relations.cpp:540-581``)."""
    coords = np.asarray(coords, dtype=np.int32).reshape(-1, 4)
    rows = coords.shape[0]
    active = rows if active_rows is None else min(int(active_rows), rows)
    values = coords[:active]
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    s, p = triple(stride), triple(padding)
    identity = s == (1, 1, 1) and p == (0, 0, 0)
    out_values = values if identity else downsample_values(values, s)
    cand = _candidates(out_values, offsets, s, p)
    src_keys, cand_keys = _keys(values, cand.reshape(-1, 4))
    uniq, first = _first_rows(src_keys)
    hit_rows = _lookup(uniq, first, cand_keys).reshape(-1, k)
    out_idx, k_idx = np.nonzero(hit_rows >= 0)
    rel = _map_rows(
        hit_rows[out_idx, k_idx],
        out_idx.astype(np.int32),
        k_idx.astype(np.int32),
        rows * k,
        out_values.shape[0],
        rows,
    )
    rel['out_coords'] = np.zeros((rows, 4), np.int32)
    rel['out_coords'][: out_values.shape[0]] = out_values
    rel['counts'] = np.asarray([out_idx.shape[0], out_values.shape[0]], np.int32)
    return _with_views(rel, rows, k)


def build_submanifold_kernel_relation(
    coords, active_rows=None, kernel_size=3, dilation=1
) -> dict:
    """``make_submanifold_kernel_relation`` (``relations.cpp:583-597``)."""
    return build_kernel_relation(coords, active_rows, kernel_size, 1, 0, dilation)


def build_target_kernel_relation(
    coords, target_coords, active_rows=None, target_active_rows=None,
    kernel_size=3, stride=1, padding=0, dilation=1,
) -> dict:
    """``write_target_kernel_relation`` (``cpu/relation_build_detail.h:43-80``)."""
    coords = np.asarray(coords, dtype=np.int32).reshape(-1, 4)
    target = np.asarray(target_coords, dtype=np.int32).reshape(-1, 4)
    rows, target_rows = coords.shape[0], target.shape[0]
    active = rows if active_rows is None else min(int(active_rows), rows)
    target_active = (
        target_rows
        if target_active_rows is None
        else min(int(target_active_rows), target_rows)
    )
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    cand = _candidates(target[:target_active], offsets, stride, padding)
    src_keys, cand_keys = _keys(coords[:active], cand.reshape(-1, 4))
    uniq, first = _first_rows(src_keys)
    hit_rows = _lookup(uniq, first, cand_keys).reshape(-1, k)
    out_idx, k_idx = np.nonzero(hit_rows >= 0)
    rel = _map_rows(
        hit_rows[out_idx, k_idx],
        out_idx.astype(np.int32),
        k_idx.astype(np.int32),
        target_rows * k,
        target_rows,
    )
    rel['out_coords'] = target
    rel['counts'] = np.asarray([out_idx.shape[0], target_active], np.int32)
    return _with_views(rel, rows, k)


def can_use_direct_transposed(offsets: np.ndarray, stride) -> bool:
    """``can_use_direct_transposed_relation`` (``relations.cpp:107-126``)."""
    if len(offsets) == 0:
        return False
    extent = offsets.max(axis=0) - offsets.min(axis=0)
    return bool(np.all(np.asarray(triple(stride)) > extent))


def build_transposed_kernel_relation(
    coords, active_rows=None, kernel_size=2, stride=2, padding=0, dilation=1
) -> dict:
    """``write_transposed_kernel_relation`` (``cpu/relation_build_detail.h:122-196``)
    and ``write_map`` (``cpu/relation_views_detail.h:52-82``)."""
    coords = np.asarray(coords, dtype=np.int32).reshape(-1, 4)
    rows = coords.shape[0]
    active = rows if active_rows is None else min(int(active_rows), rows)
    offsets = kernel_offsets(kernel_size, dilation)
    k = offsets.shape[0]
    s, p = triple(stride), triple(padding)
    cap = rows * k
    values = coords[:active].astype(np.int64)
    out = np.empty((active, k, 4), np.int64)
    out[:, :, 0] = values[:, None, 0]
    for axis in range(3):
        out[:, :, axis + 1] = (
            values[:, None, axis + 1] * s[axis] + offsets[None, :, axis] - p[axis]
        )
    out = out.reshape(-1, 4)
    in_rows = np.repeat(np.arange(active, dtype=np.int32), k)
    kernel_ids = np.tile(np.arange(k, dtype=np.int32), active)
    if can_use_direct_transposed(offsets, s):
        out_rows = np.arange(active * k, dtype=np.int32)
        out_values = out
    else:
        (keys,) = _keys(out)
        uniq, first = np.unique(keys, return_index=True)
        order = np.sort(first)                      # first-seen output order
        rank_of_first = np.empty(uniq.shape[0], np.int64)
        rank_of_first[np.argsort(first, kind='stable')] = np.arange(uniq.shape[0])
        out_rows = rank_of_first[np.searchsorted(uniq, keys)].astype(np.int32)
        out_values = out[order]
        sort = np.lexsort((in_rows, kernel_ids, out_rows))
        in_rows, kernel_ids, out_rows = in_rows[sort], kernel_ids[sort], out_rows[sort]
    rel = _map_rows(in_rows, out_rows, kernel_ids, cap, out_values.shape[0], cap)
    rel['out_coords'] = np.zeros((cap, 4), np.int32)
    rel['out_coords'][: out_values.shape[0]] = out_values
    rel['counts'] = np.asarray([in_rows.shape[0], out_values.shape[0]], np.int32)
    return _with_views(rel, rows, k)


def build_generative_relation(
    coords, active_rows=None, kernel_size=2, stride=2
) -> dict:
    """``write_generative_relation`` (``cpu/relation_build_detail.h:82-120``)."""
    coords = np.asarray(coords, dtype=np.int32).reshape(-1, 4)
    rows = coords.shape[0]
    active = rows if active_rows is None else min(int(active_rows), rows)
    offsets = kernel_offsets(kernel_size, 1)
    k = offsets.shape[0]
    s = triple(stride)
    cap = rows * k
    values = coords[:active].astype(np.int64)
    out = np.empty((active, k, 4), np.int64)
    out[:, :, 0] = values[:, None, 0]
    for axis in range(3):
        out[:, :, axis + 1] = values[:, None, axis + 1] * s[axis] + offsets[None, :, axis]
    rel = _map_rows(
        np.repeat(np.arange(active, dtype=np.int32), k),
        np.arange(active * k, dtype=np.int32),
        np.tile(np.arange(k, dtype=np.int32), active),
        cap,
        active * k,
        cap,
    )
    rel['out_coords'] = np.zeros((cap, 4), np.int32)
    rel['out_coords'][: active * k] = out.reshape(-1, 4)
    rel['counts'] = np.asarray([active * k, active * k], np.int32)
    return _with_views(rel, rows, k)


def implicit_gemm_view(
    source_coords, source_active, output_coords, output_active, offsets,
    stride=1, padding=0,
):
    """``write_relation_implicit_gemm_view`` (``cpu/relation_views_detail.h:122-169``):
    the first-row map covers ALL source rows; hits at rows >= source_active are
    dropped afterwards."""
    src = np.asarray(source_coords, np.int32).reshape(-1, 4)
    out = np.asarray(output_coords, np.int32).reshape(-1, 4)
    offsets = np.asarray(offsets, np.int32).reshape(-1, 3)
    k = offsets.shape[0]
    words = (k + 31) // 32
    source_active = int(np.clip(source_active, 0, src.shape[0]))
    output_active = int(np.clip(output_active, 0, out.shape[0]))
    out_in_map = np.full((out.shape[0], k), -1, np.int32)
    row_masks = np.zeros((out.shape[0], words), np.uint32)
    cand = _candidates(out[:output_active], offsets, stride, padding)
    src_keys, cand_keys = _keys(src, cand.reshape(-1, 4))
    uniq, first = _first_rows(src_keys)
    hit = _lookup(uniq, first, cand_keys).reshape(-1, k)
    hit = np.where(hit >= source_active, -1, hit)
    out_in_map[:output_active] = hit
    for kernel in range(k):
        bit = np.uint32(1) << np.uint32(kernel % 32)
        row_masks[:output_active, kernel // 32] |= np.where(
            hit[:, kernel] >= 0, bit, np.uint32(0)
        )
    return out_in_map, row_masks.view(np.int32)


def sorted_implicit_gemm_view(out_in_map: np.ndarray, row_masks: np.ndarray):
    """``KernelRelation.require_sorted_implicit_gemm``
    (``mlx_lattice/core/relations/views.py:467-510``): rows argsorted by the signed
    int32 mask (ties in ascending row order -- the tie rule of the third-party
    argsort is not pinned by the reference), the K-major map, and four 16-row
    sub-tile masks per 64-row tile."""
    if row_masks.shape[1] != 1:
        raise ValueError('sorted implicit GEMM view currently supports K <= 32.')
    masks = row_masks[:, 0]
    order = np.argsort(masks, kind='stable').astype(np.int32)
    sorted_map = out_in_map[order]
    n = out_in_map.shape[0]
    tiles = (n + 63) // 64
    padded = np.zeros(tiles * 64, np.int32)
    padded[:n] = masks[order]
    tile_masks = np.bitwise_or.reduce(padded.reshape(tiles, 4, 16), axis=2)
    return sorted_map, np.ascontiguousarray(sorted_map.T), order, tile_masks.reshape(-1)


def lookup_coords(coords, queries) -> np.ndarray:
    """``lookup_values`` (``cpu/set_neighbors_detail.h:45-57``)."""
    src_keys, q_keys = _keys(coords, queries)
    uniq, first = _first_rows(src_keys)
    return _lookup(uniq, first, q_keys)


def sparse_alignment(lhs_coords, lhs_active, rhs_coords, rhs_active, join: str):
    """``alignment_values`` / ``write_sparse_alignment``
    (``cpu/set_neighbors_detail.h:59-136``); capacities from
    ``native/features/coordinates/lookup.cpp:111-146``."""
    lhs = np.asarray(lhs_coords, np.int32).reshape(-1, 4)
    rhs = np.asarray(rhs_coords, np.int32).reshape(-1, 4)
    capacity = {
        'inner': lhs.shape[0],
        'left': lhs.shape[0],
        'right': rhs.shape[0],
        'outer': lhs.shape[0] + rhs.shape[0],
    }[join]
    la = min(int(lhs_active), lhs.shape[0])
    ra = min(int(rhs_active), rhs.shape[0])
    l, r = lhs[:la], rhs[:ra]
    lk, rk = _keys(l, r)
    lu, lf = _first_rows(lk)
    ru, rf = _first_rows(rk)
    if join == 'right':
        coords, lrows, rrows = r, _lookup(lu, lf, rk), np.arange(ra, dtype=np.int32)
    else:
        match = _lookup(ru, rf, lk)
        keep = match >= 0 if join == 'inner' else np.ones(la, bool)
        coords, lrows, rrows = l[keep], np.arange(la, dtype=np.int32)[keep], match[keep]
        if join == 'outer':
            extra = _lookup(lu, lf, rk) < 0
            coords = np.concatenate([coords, r[extra]])
            lrows = np.concatenate([lrows, np.full(int(extra.sum()), -1, np.int32)])
            rrows = np.concatenate([rrows, np.arange(ra, dtype=np.int32)[extra]])
    n = coords.shape[0]
    out_coords = np.zeros((capacity, 4), np.int32)
    out_coords[:n] = coords
    out_l = np.full(capacity, -1, np.int32)
    out_r = np.full(capacity, -1, np.int32)
    out_l[:n], out_r[:n] = lrows, rrows
    return out_coords, np.asarray([n], np.int32), out_l, out_r


def gather_aligned_features(feats, rows, fill: float = 0.0) -> np.ndarray:
    """``gather_aligned_features`` (``mlx_lattice/ops/tensor.py:89-109``): rows < 0 give
    the fill value in every channel, in the feature dtype."""
    feats = np.asarray(feats)
    rows = np.asarray(rows, np.int32)
    gathered = feats[np.maximum(rows, 0)]
    return np.where((rows >= 0)[:, None], gathered, feats.dtype.type(fill))


def concat_aligned_features(lhs, lhs_rows, rhs, rhs_rows) -> np.ndarray:
    """The feature half of ``sparse_cat_aligned`` (``ops/tensor.py:228-249``)."""
    return np.concatenate(
        [gather_aligned_features(lhs, lhs_rows), gather_aligned_features(rhs, rhs_rows)], axis=1)


def binary_aligned_features(lhs, lhs_rows, rhs, rhs_rows, op: str,
                            lhs_fill: float = 0.0, rhs_fill: float = 0.0) -> np.ndarray:
    """The feature half of ``sparse_binary_op`` (``ops/tensor.py:112-147``) with
    ``_apply_binary_op`` (``tensor.py:285-296``), evaluated in the feature dtype."""
    a = gather_aligned_features(lhs, lhs_rows, lhs_fill)
    b = gather_aligned_features(rhs, rhs_rows, rhs_fill)
    with np.errstate(all='ignore'):
        return {
            'add': lambda: a + b, 'sub': lambda: a - b, 'mul': lambda: a * b,
            'maximum': lambda: np.maximum(a, b), 'minimum': lambda: np.minimum(a, b),
        }[op]()


def row_norm(feats, weight=None, bias=None, eps: float = 1e-5, rms: bool = False) -> np.ndarray:
    """``layer_norm`` / ``rms_norm`` of ``mlx_lattice/ops/feature.py:196-225`` in float64:
    biased variance over the channels of each row."""
    x = np.asarray(feats, np.float64)
    if rms:
        y = x / np.sqrt(np.mean(x * x, axis=1, keepdims=True) + eps)
    else:
        mean = x.mean(axis=1, keepdims=True)
        y = (x - mean) / np.sqrt(((x - mean) ** 2).mean(axis=1, keepdims=True) + eps)
    if weight is not None:
        y = y * np.asarray(weight, np.float64)
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y


def activation(feats, name: str, **params) -> np.ndarray:
    """Pointwise activations of ``mlx_lattice/ops/feature.py:59-129`` in float64, for
    comparison within a rounding tolerance of the feature dtype."""
    import math

    x = np.asarray(feats, np.float64)
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))  # noqa: E731
    erf = np.vectorize(math.erf)
    if name == 'sigmoid':
        return sig(x)
    if name == 'silu':
        return x * sig(x)
    if name == 'tanh':
        return np.tanh(x)
    if name == 'gelu':
        form = params.get('approximate', 'none')
        if form in ('none', 'precise'):
            return 0.5 * x * (1.0 + erf(x * 0.7071067811865476))
        if form == 'tanh':
            return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
        return x * sig(1.702 * x)
    if name == 'leaky_relu':
        return np.where(x >= 0, x, x * params.get('negative_slope', 0.01))
    if name == 'softplus':
        beta, threshold = params.get('beta', 1.0), params.get('threshold', 20.0)
        with np.errstate(over='ignore'):
            return np.where(x * beta > threshold, x, np.log1p(np.exp(x * beta)) / beta)
    raise ValueError(name)


# --------------------------------------------------------------------------- #
# feature contraction
# --------------------------------------------------------------------------- #


def _kernel_major(weights: np.ndarray) -> np.ndarray:
    """(K, C_in, C_out) view of either weight layout; dense-5D kernel id is
    ``(ix*Ky + iy)*Kz + iz`` (``convolution/cpu/algorithms.cpp:113-150``)."""
    if weights.ndim == 3:
        return weights
    c_out, kx, ky, kz, c_in = weights.shape
    return weights.transpose(1, 2, 3, 4, 0).reshape(kx * ky * kz, c_in, c_out)


def _edges(rel: dict, out_capacity: int):
    e = min(int(rel['counts'][0]), rel['in_rows'].shape[0])
    n_out = min(int(rel['counts'][1]), out_capacity)
    # edges are consumed through the output CSR (row_offsets), rows < n_out only
    end = int(rel['row_offsets'][n_out]) if n_out > 0 else 0
    end = min(end, e)
    return rel['in_rows'][:end], rel['out_rows'][:end], rel['kernel_ids'][:end], n_out


def sparse_conv(feats, weights, rel: dict, out_capacity: int, n_kernels: int):
    """``eval_dense_channels_typed`` / ``eval_typed``
    (``convolution/cpu/algorithms.cpp:180-302``). fp32 accumulation, one final
    cast, for float32 and for float16 with square C in {16,32,64}; the generic
    float16 route re-rounds the accumulator to float16 after every multiply-add
    (``:229-235``), reproduced here with a sequential loop."""
    feats = np.asarray(feats)
    w = _kernel_major(np.asarray(weights))
    c_in, c_out = w.shape[1], w.shape[2]
    in_rows, out_rows, kernel_ids, n_out = _edges(rel, out_capacity)
    dtype = feats.dtype
    square = c_in == c_out and c_in in (16, 32, 64)
    out = np.zeros((out_capacity, c_out), np.float32)
    if dtype == np.float32 or square:
        x32, w32 = feats.astype(np.float32), w.astype(np.float32)
        for kernel in range(n_kernels):
            sel = kernel_ids == kernel
            if not sel.any():
                continue
            contrib = x32[in_rows[sel]] @ w32[kernel]
            np.add.at(out, out_rows[sel], contrib)
        return out.astype(dtype)
    # lossy float16 route: per output row, edges in CSR order, ci outer, co inner
    acc = np.zeros((out_capacity, c_out), np.float16)
    row_offsets = rel['row_offsets']
    degree = np.diff(row_offsets[: n_out + 1])
    for step in range(int(degree.max()) if n_out else 0):
        rows = np.nonzero(degree > step)[0]
        e = row_offsets[rows] + step
        x = feats[in_rows[e]].astype(np.float32)
        wk = w[kernel_ids[e]].astype(np.float32)          # (rows, C_in, C_out)
        for ci in range(c_in):
            cur = acc[rows].astype(np.float32) + x[:, ci : ci + 1] * wk[:, ci, :]
            acc[rows] = cur.astype(np.float16)
    return acc


def unpack_codes(packed: np.ndarray, bits: int, channels: int) -> np.ndarray:
    """``unpack`` (``convolution/cpu/quantized.cpp:54-62``): packed is
    (K, words, C_out) uint32, channel ci sits in word ``(ci*bits)>>5`` at shift
    ``(ci*bits)&31``. Returns codes (K, channels, C_out)."""
    packed = np.asarray(packed, np.uint32)
    ci = np.arange(channels)
    word = (ci * bits) >> 5
    shift = ((ci * bits) & 31).astype(np.uint32)
    mask = np.uint32((1 << bits) - 1)
    return (packed[:, word, :] >> shift[None, :, None]) & mask


def dequantize_spatial(packed, scales, biases, in_channels, group_size, bits):
    """``code*scale + bias`` in float32 with group ``ci // group_size``
    (``convolution/cpu/quantized.cpp:107-131``). Returns (K, C_in, C_out) float32."""
    codes = unpack_codes(packed, bits, in_channels).astype(np.float32)
    group = np.arange(in_channels) // group_size
    s = np.asarray(scales).astype(np.float32)[:, group, :]
    b = np.asarray(biases).astype(np.float32)[:, group, :]
    return codes * s + b


def sparse_quantized_conv(
    feats, packed, scales, biases, rel: dict, out_capacity: int, n_kernels: int,
    in_channels: int, out_channels: int, storage_in_channels: int,
    group_size: int, bits: int,
):
    """``eval_typed`` of ``convolution/cpu/quantized.cpp:64-140``: float32
    dequantisation and accumulation, one final cast to the feature dtype."""
    feats = np.asarray(feats)
    w = dequantize_spatial(packed, scales, biases, in_channels, group_size, bits)
    in_rows, out_rows, kernel_ids, n_out = _edges(rel, out_capacity)
    keep = (kernel_ids >= 0) & (kernel_ids < n_kernels) & (in_rows >= 0)
    in_rows, out_rows, kernel_ids = in_rows[keep], out_rows[keep], kernel_ids[keep]
    out = np.zeros((out_capacity, out_channels), np.float32)
    x32 = feats.astype(np.float32)
    for kernel in range(n_kernels):
        sel = kernel_ids == kernel
        if sel.any():
            np.add.at(out, out_rows[sel], x32[in_rows[sel]] @ w[kernel])
    return out.astype(feats.dtype)


def sparse_pool(
    feats, rel: dict, *, input_exclusive: bool, reduce: str,
    out_capacity: int, n_kernels: int,
):
    """``pool::eval`` (``pooling/cpu/algorithms.cpp:181-244``): float32 only; rows
    past N_out keep the reduction identity (0, or -inf for max)."""
    feats = np.asarray(feats, np.float32)
    n_out = min(int(rel['counts'][1]), out_capacity)
    end = int(rel['row_offsets'][n_out]) if n_out else 0
    in_rows, out_rows = rel['in_rows'][:end], rel['out_rows'][:end]
    if reduce == 'max':
        out = np.full((out_capacity, feats.shape[1]), -np.inf, np.float32)
        np.maximum.at(out, out_rows, feats[in_rows])
        return out
    out = np.zeros((out_capacity, feats.shape[1]), np.float32)
    # the reference adds edges of a row in CSR order; do the same per step so the
    # float32 rounding sequence is identical
    degree = np.diff(rel['row_offsets'][: n_out + 1])
    for step in range(int(degree.max()) if n_out else 0):
        rows = np.nonzero(degree > step)[0]
        out[rows] += feats[in_rows[rel['row_offsets'][rows] + step]]
    if reduce == 'avg':
        scale = (1.0 / np.maximum(degree, 1).astype(np.float32)).astype(np.float32)
        out[:n_out] *= scale[:, None]
    return out


def input_exclusive(kernel_size, stride, dilation=1) -> bool:
    """``_input_exclusive`` (``mlx_lattice/ops/pool.py:271-280``)."""
    return all(
        s >= (k - 1) * d + 1
        for s, k, d in zip(triple(stride), triple(kernel_size), triple(dilation))
    )


def global_pool(feats, batch_counts: Sequence[int], mode: str) -> np.ndarray:
    """``_stack_batch_reductions`` (``mlx_lattice/ops/pool.py:197-236``): per-batch
    sum / avg / max over contiguous batch row ranges; avg of an empty batch is 0.
    Arithmetic in float32 (the reference rejects other dtypes)."""
    feats = np.asarray(feats, np.float32)
    out = np.zeros((len(batch_counts), feats.shape[1]), np.float32)
    start = 0
    for b, count in enumerate(batch_counts):
        rows = feats[start : start + count]
        start += count
        if mode == 'max':
            if count == 0:
                raise ValueError('global_max_pool does not support empty batches.')
            out[b] = rows.max(axis=0)
        else:
            total = rows.sum(axis=0, dtype=np.float32)
            out[b] = total / np.float32(max(count, 1)) if mode == 'avg' else total
    return out


def linear(feats, weight, bias=None):
    """``linear`` (``mlx_lattice/ops/feature.py:33-51``): ``x @ W.T (+ bias)`` with
    float32 accumulation and one cast to the feature dtype."""
    feats = np.asarray(feats)
    out = feats.astype(np.float32) @ np.asarray(weight).astype(np.float32).T
    out = out.astype(feats.dtype)
    if bias is not None:
        out = (out.astype(np.float32) + np.asarray(bias).astype(np.float32)).astype(
            feats.dtype
        )
    return out


def relu(feats):
    """``relu`` (``mlx_lattice/ops/feature.py:54-56``)."""
    return np.maximum(feats, np.asarray(0, feats.dtype))


def batch_norm(feats, weight=None, bias=None, mean=None, var=None, eps=1e-5):
    """``batch_norm`` with running statistics (``mlx_lattice/ops/feature.py:166-187``):
    ``(x - mean) * rsqrt(var + eps) * weight + bias`` evaluated in float32 and
    cast once to the feature dtype."""
    feats = np.asarray(feats)
    x = feats.astype(np.float32)
    c = feats.shape[1]
    mean = np.zeros(c, np.float32) if mean is None else np.asarray(mean).astype(np.float32)
    var = np.ones(c, np.float32) if var is None else np.asarray(var).astype(np.float32)
    y = (x - mean) * (1.0 / np.sqrt(var + np.float32(eps))).astype(np.float32)
    if weight is not None:
        y = y * np.asarray(weight).astype(np.float32)
    if bias is not None:
        y = y + np.asarray(bias).astype(np.float32)
    return y.astype(feats.dtype)


# --------------------------------------------------------------------------- #
# affine quantizer (third-party algorithm, parity unpinned)
# --------------------------------------------------------------------------- #


def quantize_affine(rows: np.ndarray, group_size: int, bits: int):
    """Per-group affine quantisation of a (R, S) matrix along its last axis,
    restating the published ``mode='affine'`` rule of mlx 0.31.2 that
    ``mlx_lattice/core/quantized.py:164-169`` calls: with ``n = 2^bits - 1``,
    ``scale = max((max - min)/n, 1e-7)`` signed towards the larger-magnitude edge,
    the edge is snapped so that it is an exact multiple of the scale, ``bias`` is
    that edge, codes are ``clip(round((w - bias)/scale), 0, n)``. Returns codes
    (R, S) uint32, scales and biases (R, S/group) float32. PARITY UNPINNED."""
    rows = np.asarray(rows, np.float32)
    r, s = rows.shape
    assert s % group_size == 0
    g = rows.reshape(r, s // group_size, group_size)
    n_bins = np.float32((1 << bits) - 1)
    w_max, w_min = g.max(axis=2), g.min(axis=2)
    mask = np.abs(w_min) > np.abs(w_max)
    scales = np.maximum((w_max - w_min) / n_bins, np.float32(1e-7)).astype(np.float32)
    scales = np.where(mask, scales, -scales).astype(np.float32)
    edge = np.where(mask, w_min, w_max).astype(np.float32)
    q0 = np.rint(edge / scales).astype(np.float32)
    safe_q0 = np.where(q0 == 0, np.float32(1), q0)
    scales = np.where(q0 != 0, edge / safe_q0, scales).astype(np.float32)
    biases = np.where(q0 == 0, np.float32(0), edge).astype(np.float32)
    codes = np.rint((g - biases[:, :, None]) / scales[:, :, None])
    codes = np.clip(codes, 0, n_bins).astype(np.uint32).reshape(r, s)
    return codes, scales, biases


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """Little-endian packing of codes along the last axis into uint32 words."""
    r, s = codes.shape
    per = 32 // bits
    grouped = codes.reshape(r, s // per, per).astype(np.uint64)
    shifts = (np.arange(per) * bits).astype(np.uint64)
    return (grouped << shifts).sum(axis=2).astype(np.uint32)


def quantize_weight(weight: np.ndarray, group_size: int = 32, bits: int = 4) -> dict:
    """``quantize_weight`` (``mlx_lattice/core/quantized.py:124-187``): rows are
    (K*C_out, C_in) padded to the group size; spatial layouts are stored as
    packed (K, words, C_out), scales/biases (K, groups, C_out); linear weights as
    (1, C_out, words) and (1, C_out, groups). Scales and biases are cast to the
    weight dtype."""
    weight = np.asarray(weight)
    dtype = weight.dtype
    if weight.ndim == 2:
        c_out, c_in = weight.shape
        rows, layout, ks = weight, 'linear', (1, 1, 1)
    elif weight.ndim == 3:
        k, c_in, c_out = weight.shape
        rows, layout, ks = weight.transpose(0, 2, 1).reshape(k * c_out, c_in), 'kernel_major', (k, 1, 1)
    elif weight.ndim == 5:
        c_out, kx, ky, kz, c_in = weight.shape
        rows = weight.transpose(1, 2, 3, 0, 4).reshape(kx * ky * kz * c_out, c_in)
        layout, ks = 'dense_5d', (kx, ky, kz)
    else:
        raise ValueError('unsupported weight rank')
    storage = -(-c_in // group_size) * group_size
    rows = np.pad(rows.astype(np.float32), [(0, 0), (0, storage - c_in)])
    codes, scales, biases = quantize_affine(rows, group_size, bits)
    packed = pack_codes(codes, bits)
    kernel_rows = ks[0] * ks[1] * ks[2]
    packed = packed.reshape(kernel_rows, c_out, -1)
    scales = scales.astype(dtype).reshape(kernel_rows, c_out, -1)
    biases = biases.astype(dtype).reshape(kernel_rows, c_out, -1)
    if kernel_rows > 1:
        packed = np.ascontiguousarray(packed.transpose(0, 2, 1))
        scales = np.ascontiguousarray(scales.transpose(0, 2, 1))
        biases = np.ascontiguousarray(biases.transpose(0, 2, 1))
    return {
        'weight': packed, 'scales': scales, 'biases': biases,
        'group_size': group_size, 'bits': bits, 'in_channels': c_in,
        'out_channels': c_out, 'kernel_size': ks, 'layout': layout,
        'storage_in_channels': storage,
    }


def dequantize_weight(q: dict) -> np.ndarray:
    """``dequantize_weight`` (``mlx_lattice/core/quantized.py:190-223``)."""
    kernel_rows = int(np.prod(q['kernel_size']))
    packed, scales, biases = q['weight'], q['scales'], q['biases']
    if kernel_rows > 1:
        w = dequantize_spatial(
            packed, scales, biases, q['in_channels'], q['group_size'], q['bits']
        )                                            # (K, C_in, C_out)
        w = w.astype(scales.dtype)
        if q['layout'] == 'kernel_major':
            return w
        kx, ky, kz = q['kernel_size']
        return w.reshape(kx, ky, kz, q['in_channels'], q['out_channels']).transpose(
            4, 0, 1, 2, 3
        )
    spatial = dequantize_spatial(
        packed.transpose(0, 2, 1), scales.transpose(0, 2, 1),
        biases.transpose(0, 2, 1), q['in_channels'], q['group_size'], q['bits'],
    )                                                # (1, C_in, C_out)
    return spatial[0].T.astype(scales.dtype)


def quantized_matmul(feats, q: dict):
    """``quantized_matmul`` (``mlx_lattice/ops/_quantized.py:8-38``): the
    third-party ``mx.quantized_matmul(transpose=True)`` restated as float32
    dequantise (``code*scale + bias``), float32 accumulate, one cast. PARITY
    UNPINNED against the third-party kernel."""
    feats = np.asarray(feats)
    w = dequantize_weight(q).astype(np.float32)       # (C_out, C_in)
    return (feats.astype(np.float32) @ w.T).astype(feats.dtype)
