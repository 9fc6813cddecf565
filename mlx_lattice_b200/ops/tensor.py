"""Tensor assembly helpers (``mlx_lattice/ops/tensor.py:15-64,228-249``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.coords.alignment import SparseAlignment
from mlx_lattice_b200.core.tensor import SparseTensor
from mlx_lattice_b200.core.types import triple

__all__ = ['sparse_cat_aligned', 'sparse_collate']


def sparse_collate(
    coords: Sequence[torch.Tensor], feats: Sequence[torch.Tensor], *, stride=1
) -> SparseTensor:
    """Collate unbatched ``(N_i, 3)`` coords / ``(N_i, C)`` feats into one tensor
    with a prepended batch column and ``batch_counts`` metadata."""
    if len(coords) != len(feats):
        raise ValueError('coords and feats batch sizes must match.')
    if not coords:
        raise ValueError('expected at least one sparse tensor batch.')
    batched_coords, batched_feats = [], []
    dtype = coords[0].dtype
    for batch, (c, f) in enumerate(zip(coords, feats, strict=True)):
        if c.ndim != 2 or c.shape[1] != 3:
            raise ValueError('collated coords must have shape (N, 3).')
        if c.dtype not in (torch.int32, torch.int64):
            raise ValueError('collated coords must be int32 or int64.')
        if c.dtype != dtype:
            raise ValueError('collated coords must share a dtype.')
        if f.ndim != 2:
            raise ValueError('collated feats must have shape (N, C).')
        if c.shape[0] != f.shape[0]:
            raise ValueError('collated coords and feats must have matching rows.')
        col = torch.full((c.shape[0], 1), batch, dtype=c.dtype, device=c.device)
        batched_coords.append(torch.cat([col, c], dim=1))
        batched_feats.append(f)
    return SparseTensor(
        torch.cat(batched_coords, dim=0).contiguous(),
        torch.cat(batched_feats, dim=0).contiguous(),
        stride=triple(stride, name='stride'),
        batch_counts=tuple(int(c.shape[0]) for c in coords),
    )


def _require_compatible(lhs: SparseTensor, rhs: SparseTensor) -> None:
    if lhs.stride != rhs.stride:
        raise ValueError('sparse tensor strides must match.')
    if lhs.coords.dtype != rhs.coords.dtype:
        raise ValueError('sparse tensor coordinate dtypes must match.')


def align_sparse(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseAlignment:
    """Coordinate-value alignment of two sparse tensors (``ops/tensor.py:67-86``): the joined
    support and, per joined row, the row of each operand (-1 where it has none)."""
    _require_compatible(lhs, rhs)
    coords, active, lhs_rows, rhs_rows = _ext.build_sparse_alignment(
        lhs.coords, lhs.active_rows, rhs.coords, rhs.active_rows, join
    )
    return SparseAlignment(coords, active, lhs_rows, rhs_rows)


def sparse_cat_aligned(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseTensor:
    """Concatenate the channels of two sparse tensors after coordinate-value
    alignment; tensors that share coordinate identity are concatenated directly
    (``ops/tensor.py:228-249``). One gather-and-concatenate kernel either way; for tensors
    of one coordinate identity that kernel runs only when ``feats`` of the result is read
    (a tensor-core convolution reads the two parts in place instead)."""
    _require_compatible(lhs, rhs)
    if lhs.same_coords(rhs):
        return lhs.replace(feats=(lhs.feats, rhs.feats))
    alignment = align_sparse(lhs, rhs, join=join)
    return SparseTensor(
        alignment.coords,
        _ext.concat_aligned_features(lhs.feats, alignment.lhs_rows, rhs.feats, alignment.rhs_rows),
        lhs.stride,
        coord_manager=lhs.coord_manager,
        active_rows=alignment.active_rows,
    )


def sparse_binary_op(
    lhs: SparseTensor, rhs: SparseTensor, op: str, *, join: str = 'outer',
    lhs_fill: float = 0.0, rhs_fill: float = 0.0,
) -> SparseTensor:
    """Elementwise ``add / sub / mul / maximum / minimum`` after coordinate-value alignment
    (``ops/tensor.py:112-147``); rows one operand lacks take its fill value. Operands that
    share coordinate identity are combined row by row without an alignment."""
    _require_compatible(lhs, rhs)
    if lhs.channels != rhs.channels:
        raise ValueError('sparse binary operands must have matching channels.')
    if lhs.same_coords(rhs):
        return lhs.replace(feats=_ext.binary_aligned_features(lhs.feats, None, rhs.feats, None, op))
    alignment = align_sparse(lhs, rhs, join=join)
    return SparseTensor(
        alignment.coords,
        _ext.binary_aligned_features(
            lhs.feats, alignment.lhs_rows, rhs.feats, alignment.rhs_rows, op, lhs_fill, rhs_fill
        ),
        lhs.stride,
        coord_manager=lhs.coord_manager,
        active_rows=alignment.active_rows,
    )


def sparse_add(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'outer') -> SparseTensor:
    """``ops/tensor.py:150-157``; the residual connection of a sparse ResNet block."""
    return sparse_binary_op(lhs, rhs, 'add', join=join)


def sparse_sub(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'outer') -> SparseTensor:
    return sparse_binary_op(lhs, rhs, 'sub', join=join)


def sparse_mul(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseTensor:
    return sparse_binary_op(lhs, rhs, 'mul', join=join)


def sparse_maximum(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseTensor:
    return sparse_binary_op(lhs, rhs, 'maximum', join=join)


def sparse_minimum(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseTensor:
    return sparse_binary_op(lhs, rhs, 'minimum', join=join)
