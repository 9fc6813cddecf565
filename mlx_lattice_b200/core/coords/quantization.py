"""Point-to-voxel quantization metadata (``mlx_lattice/core/coords/quantization.py``,
the sparse_quantize / voxelize_features part)."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.coords.validation import validate_coords


@dataclass(frozen=True, slots=True)
class SparseQuantization:
    """Sparse voxel coordinates plus point-to-voxel metadata (``:16-61``).

    ``coords`` stores unique voxel coordinates in ``(batch, x, y, z)`` order,
    ``inverse_rows`` maps each input point row to its voxel row, ``counts`` stores the
    number of active point rows accumulated into each voxel.
    """

    coords: torch.Tensor
    active_rows: torch.Tensor
    inverse_rows: torch.Tensor
    counts: torch.Tensor

    def __post_init__(self) -> None:
        validate_coords(self.coords)
        if self.coords.dtype != torch.int32:
            raise ValueError('quantized coords must be int32.')
        if tuple(self.active_rows.shape) != (1,) or self.active_rows.dtype != torch.int32:
            raise ValueError('active_rows must have shape (1,) and int32 dtype.')
        rows = self.coords.shape[0]
        if tuple(self.inverse_rows.shape) != (rows,) or self.inverse_rows.dtype != torch.int32:
            raise ValueError('inverse_rows must have shape (N,) and int32 dtype.')
        if tuple(self.counts.shape) != (rows,) or self.counts.dtype != torch.int32:
            raise ValueError('counts must have shape (N,) and int32 dtype.')

    @property
    def capacity(self) -> int:
        return int(self.coords.shape[0])

    @property
    def active_count(self) -> torch.Tensor:
        return self.active_rows


@dataclass(frozen=True, slots=True)
class PointVoxelMap:
    """Fixed-width point-to-voxel interpolation rows and weights (``:64-89``): both
    ``(N, 8)``; linear interpolation uses up to eight voxel rows per point, nearest one."""

    rows: torch.Tensor
    weights: torch.Tensor

    def __post_init__(self) -> None:
        if self.rows.ndim != 2 or self.rows.shape[1] != 8 or self.rows.dtype != torch.int32:
            raise ValueError('rows must have shape (N, 8) and int32 dtype.')
        if self.weights.shape != self.rows.shape:
            raise ValueError('weights must have the same shape as rows.')
        if self.weights.dtype != torch.float32:
            raise ValueError('weights must be float32.')

    @property
    def point_count(self) -> int:
        return int(self.rows.shape[0])


def _validate_points(points: torch.Tensor) -> None:
    if points.ndim != 2 or points.shape[1] != 3:
        raise ValueError('points must have shape (N, 3).')
    if points.dtype != torch.float32:
        raise ValueError('points must be float32.')


def _batch_indices(value: torch.Tensor | None, rows: int, device) -> torch.Tensor:
    if value is None:
        return torch.zeros(rows, dtype=torch.int32, device=device)
    if tuple(value.shape) != (rows,) or value.dtype != torch.int32:
        raise ValueError('batch_indices must have shape (N,) and int32 dtype.')
    return value


def _active_rows(value: torch.Tensor | None, rows: int, device) -> torch.Tensor:
    if value is None:
        return torch.full((1,), int(rows), dtype=torch.int32, device=device)
    if tuple(value.shape) != (1,) or value.dtype != torch.int32:
        raise ValueError('active_rows must have shape (1,) and int32 dtype.')
    return value


def _float_triple(value: float | Sequence[float], name: str) -> tuple[float, float, float]:
    if isinstance(value, (int, float)):
        values = (float(value), float(value), float(value))
    else:
        raw = tuple(float(item) for item in value)
        if len(raw) != 3:
            raise ValueError(f'{name} must contain exactly 3 values.')
        values = (raw[0], raw[1], raw[2])
    if name == 'voxel_size' and any(item <= 0.0 for item in values):
        raise ValueError('voxel_size values must be positive.')
    return values


def _validate_reduction(value: str) -> str:
    if value in ('sum', 'mean'):
        return value
    raise ValueError("reduction must be 'sum' or 'mean'.")


def sparse_quantize(
    points: torch.Tensor,
    voxel_size: float | Sequence[float] = 1.0,
    *,
    batch_indices: torch.Tensor | None = None,
    origin: float | Sequence[float] = 0.0,
    active_rows: torch.Tensor | None = None,
) -> SparseQuantization:
    """Voxelize floating-point points into sparse integer coordinates (``:92-117``)."""
    _validate_points(points)
    rows = int(points.shape[0])
    batches = _batch_indices(batch_indices, rows, points.device)
    point_rows = _active_rows(active_rows, rows, points.device)
    native = _ext.sparse_quantize(
        points, batches, point_rows, _float_triple(voxel_size, 'voxel_size'),
        _float_triple(origin, 'origin'),
    )
    return SparseQuantization(*native)


def voxelize_features(
    feats: torch.Tensor,
    quantization: SparseQuantization,
    *,
    active_rows: torch.Tensor | None = None,
    reduction: str = 'mean',
) -> torch.Tensor:
    """Aggregate point features into voxels using quantization data (``:120-145``)."""
    if feats.ndim != 2:
        raise ValueError('feats must have shape (N, C).')
    if feats.dtype != torch.float32:
        raise ValueError('voxelize currently supports float32 features.')
    if feats.shape[0] != quantization.capacity:
        raise ValueError('feats and quantization metadata must share rows.')
    point_rows = _active_rows(active_rows, int(feats.shape[0]), feats.device)
    return _ext.voxelize_features(
        feats, quantization.inverse_rows, quantization.counts, point_rows,
        _validate_reduction(reduction),
    )


def _validate_interpolation(value: str) -> str:
    if value in ('nearest', 'linear'):
        return value
    raise ValueError("interpolation must be 'nearest' or 'linear'.")


def build_point_voxel_map(
    points: torch.Tensor,
    voxel_coords: torch.Tensor,
    voxel_active_rows: torch.Tensor,
    voxel_size: float | Sequence[float] = 1.0,
    *,
    batch_indices: torch.Tensor | None = None,
    point_active_rows: torch.Tensor | None = None,
    origin: float | Sequence[float] = 0.0,
    interpolation: str = 'linear',
) -> PointVoxelMap:
    """Build fixed-width interpolation rows from points to voxel centers (``:148-189``)."""
    _validate_points(points)
    validate_coords(voxel_coords)
    if voxel_coords.dtype != torch.int32:
        raise ValueError('voxel_coords must be int32.')
    rows = int(points.shape[0])
    batches = _batch_indices(batch_indices, rows, points.device)
    point_rows = _active_rows(point_active_rows, rows, points.device)
    if tuple(voxel_active_rows.shape) != (1,) or voxel_active_rows.dtype != torch.int32:
        raise ValueError('voxel_active_rows must have shape (1,) and int32 dtype.')
    native = _ext.build_point_voxel_map(
        points, batches, point_rows, voxel_coords, voxel_active_rows,
        _float_triple(voxel_size, 'voxel_size'), _float_triple(origin, 'origin'),
        _validate_interpolation(interpolation),
    )
    return PointVoxelMap(*native)


def interpolate_point_features(voxel_feats: torch.Tensor, point_voxel_map: PointVoxelMap) -> torch.Tensor:
    """Interpolate voxel features back to point rows (``:192-208``)."""
    if voxel_feats.ndim != 2:
        raise ValueError('voxel_feats must have shape (N, C).')
    if voxel_feats.dtype != torch.float32:
        raise ValueError('point interpolation currently supports float32.')
    return _ext.interpolate_point_features(voxel_feats, point_voxel_map.rows, point_voxel_map.weights)
