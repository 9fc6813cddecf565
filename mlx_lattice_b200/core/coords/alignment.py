"""Coordinate-value alignment of two sparse supports
(``mlx_lattice/core/coords/alignment.py:14-57``)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True, slots=True)
class SparseAlignment:
    """``coords`` is the joined support; ``lhs_rows`` / ``rhs_rows`` name, for every joined
    row, the row of the left and right tensor that holds it (-1 = missing under the join)."""

    coords: torch.Tensor
    active_rows: torch.Tensor
    lhs_rows: torch.Tensor
    rhs_rows: torch.Tensor

    def __post_init__(self) -> None:
        if self.coords.ndim != 2 or self.coords.shape[1] != 4:
            raise ValueError('coords must have shape (N, 4).')
        if self.coords.dtype not in (torch.int32, torch.int64):
            raise ValueError('coords must be int32 or int64.')
        if tuple(self.active_rows.shape) != (1,) or self.active_rows.dtype != torch.int32:
            raise ValueError('active_rows must have shape (1,) and int32 dtype.')
        rows = (int(self.coords.shape[0]),)
        if tuple(self.lhs_rows.shape) != rows:
            raise ValueError('lhs_rows must have shape (N,).')
        if tuple(self.rhs_rows.shape) != rows:
            raise ValueError('rhs_rows must have shape (N,).')
        if self.lhs_rows.dtype != torch.int32 or self.rhs_rows.dtype != torch.int32:
            raise ValueError('alignment rows must be int32.')

    @property
    def capacity(self) -> int:
        return int(self.coords.shape[0])

    @property
    def active_count(self) -> torch.Tensor:
        return self.active_rows
