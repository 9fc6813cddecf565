"""Tensor assembly helpers (``mlx_lattice/ops/tensor.py:15-64,228-249``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200 import _ext
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


def _gather_aligned(feats: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    gathered = feats.index_select(0, rows.clamp(min=0).long())
    return gathered * (rows >= 0).to(feats.dtype)[:, None]


def sparse_cat_aligned(lhs: SparseTensor, rhs: SparseTensor, *, join: str = 'inner') -> SparseTensor:
    """Concatenate the channels of two sparse tensors after coordinate-value
    alignment; tensors that share coordinate identity are concatenated directly."""
    if lhs.stride != rhs.stride:
        raise ValueError('sparse tensors must have matching stride.')
    if lhs.coords.dtype != rhs.coords.dtype:
        raise ValueError('sparse tensors must have matching coordinate dtype.')
    if lhs.same_coords(rhs):
        return lhs.replace(feats=torch.cat([lhs.feats, rhs.feats], dim=1))
    coords, active, lhs_rows, rhs_rows = _ext.build_sparse_alignment(
        lhs.coords, lhs.active_rows, rhs.coords, rhs.active_rows, join
    )
    return SparseTensor(
        coords,
        torch.cat([_gather_aligned(lhs.feats, lhs_rows), _gather_aligned(rhs.feats, rhs_rows)], dim=1),
        lhs.stride,
        coord_manager=lhs.coord_manager,
        active_rows=active,
    )
