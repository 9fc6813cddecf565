"""Sparse feature tensor (``mlx_lattice/core/tensor.py:17-267``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200.core.coords import CoordinateManager, CoordinateMapKey, validate_coords
from mlx_lattice_b200.core.types import Triple, triple


class SparseTensor:
    """Sparse feature tensor indexed by batched integer coordinates.

    ``coords`` is ``(N, 4)`` ordered ``(batch, x, y, z)``, ``feats`` is ``(N, C)``
    in the same row order; both are CUDA tensors. ``active_rows`` (int32 ``(1,)``
    on the device) records the valid prefix of the static-capacity buffers. A
    ``CoordinateManager`` owns the coordinate array and a ``CoordinateMapKey``
    names it; feature-only operations keep that identity so relations are reused.

    ``feats`` may also be given as a pair of tensors over the same rows (the result of a
    channel concatenation that has not been written yet): ``feat_parts`` then returns the
    pair, which a tensor-core convolution reads in place, and ``feats`` writes and caches
    the concatenated array on first access.
    """

    __slots__ = (
        'coords', '_feats', '_parts', 'stride', 'coord_key', 'coord_manager', 'batch_counts',
        'active_rows',
    )

    def __init__(
        self,
        coords: torch.Tensor,
        feats: torch.Tensor,
        stride: int | Sequence[int] = 1,
        *,
        coord_key: CoordinateMapKey | None = None,
        coord_manager: CoordinateManager | None = None,
        batch_counts: Sequence[int] | None = None,
        active_rows: torch.Tensor | None = None,
    ) -> None:
        normalized_stride = triple(stride, name='stride')
        validate_coords(coords)
        if coord_key is None:
            manager = CoordinateManager() if coord_manager is None else coord_manager
            key = manager.insert_coords(coords, normalized_stride, active_rows)
            owned, active = coords, manager.active_rows(key)
        else:
            if coord_manager is None:
                raise ValueError('coord_manager is required when coord_key is set.')
            if not coord_manager.owns(coord_key):
                raise ValueError('coord_key does not belong to coord_manager.')
            if coord_key.stride != normalized_stride:
                raise ValueError('stride must match coord_key stride.')
            owned = coord_manager.coords(coord_key)
            if coords is not owned:
                raise ValueError('coords must be the manager-owned array for coord_key.')
            manager, key = coord_manager, coord_key
            active = (
                coord_manager.active_rows(coord_key)
                if active_rows is None
                else _active_rows(active_rows)
            )
        parts = None
        if isinstance(feats, (tuple, list)):
            parts = tuple(feats)
            if len(parts) != 2 or any(part.ndim != 2 for part in parts):
                raise ValueError('feature parts must be two arrays of shape (N, C).')
            if parts[0].shape[0] != parts[1].shape[0] or parts[0].dtype != parts[1].dtype:
                raise ValueError('feature parts must share row count and dtype.')
            rows = int(parts[0].shape[0])
        else:
            if feats.ndim != 2:
                raise ValueError('feats must have shape (N, C).')
            rows = int(feats.shape[0])
        if owned.shape[0] != rows:
            raise ValueError('coords and feats must have the same row count.')
        counts = None
        if batch_counts is not None:
            counts = tuple(int(v) for v in batch_counts)
            if any(v < 0 for v in counts):
                raise ValueError('batch_counts must be non-negative.')
            if sum(counts) != owned.shape[0]:
                raise ValueError('batch_counts must cover all sparse rows.')
        self.coords = owned
        self._feats = None if parts is not None else feats
        self._parts = parts
        self.stride = normalized_stride
        self.coord_key = key
        self.coord_manager = manager
        self.batch_counts = counts
        self.active_rows = active

    @property
    def feats(self) -> torch.Tensor:
        if self._feats is None:
            from mlx_lattice_b200 import _ext

            self._feats = _ext.concat_aligned_features(self._parts[0], None, self._parts[1], None)
            self._parts = None
        return self._feats

    @feats.setter
    def feats(self, value: torch.Tensor) -> None:
        self._feats = value
        self._parts = None

    @property
    def feat_parts(self):
        """The two tensors whose channel concatenation is ``feats``, while it is unwritten."""
        return self._parts

    @property
    def capacity(self) -> int:
        return int(self.coords.shape[0])

    @property
    def active_count(self) -> torch.Tensor:
        return self.active_rows

    @property
    def channels(self) -> int:
        if self._parts is not None:
            return int(self._parts[0].shape[1] + self._parts[1].shape[1])
        return int(self._feats.shape[1])

    @property
    def shape(self) -> tuple[int, int]:
        return (self.capacity, self.channels)

    @property
    def dtype(self) -> torch.dtype:
        return self._parts[0].dtype if self._parts is not None else self._feats.dtype

    @property
    def batch_indices(self) -> torch.Tensor:
        return self.coords[:, 0]

    def astype(self, dtype: torch.dtype) -> 'SparseTensor':
        return self.replace(feats=self.feats.to(dtype))

    def replace(
        self,
        *,
        coords: torch.Tensor | None = None,
        feats: torch.Tensor | None = None,
        stride: int | Sequence[int] | None = None,
    ) -> 'SparseTensor':
        """Replacing only ``feats`` keeps the coordinate identity; new coords or a
        new stride register a new key and drop batch metadata (``tensor.py:162-190``)."""
        next_coords = self.coords if coords is None else coords
        next_stride = self.stride if stride is None else triple(stride, name='stride')
        reuse = next_coords is self.coords and next_stride == self.stride
        return SparseTensor(
            next_coords,
            self.feats if feats is None else feats,
            next_stride,
            coord_key=self.coord_key if reuse else None,
            coord_manager=self.coord_manager,
            batch_counts=self.batch_counts if reuse else None,
            active_rows=self.active_rows if reuse else None,
        )

    def same_coords(self, other: 'SparseTensor') -> bool:
        return self.coord_manager is other.coord_manager and self.coord_key == other.coord_key


def _active_rows(value: torch.Tensor) -> torch.Tensor:
    if tuple(value.shape) != (1,) or value.dtype != torch.int32:
        raise ValueError('active_rows must have shape (1,) and int32 dtype.')
    return value
