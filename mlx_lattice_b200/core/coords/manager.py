"""Coordinate identity and relation cache (``mlx_lattice/core/coords/manager.py``)."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass, field
from itertools import count

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.coords.builders import (
    build_generative_relation,
    build_kernel_relation,
    build_submanifold_kernel_relation,
    build_target_kernel_relation,
    build_target_transposed_relation,
    build_transposed_kernel_relation,
)
from mlx_lattice_b200.core.coords.validation import validate_coords
from mlx_lattice_b200.core.relations import KernelRelation, KernelSpec
from mlx_lattice_b200.core.types import Triple, triple

_manager_ids = count()


@dataclass(frozen=True, slots=True)
class CoordinateMapKey:
    """Opaque coordinate identity key owned by a ``CoordinateManager``."""

    id: int
    stride: Triple
    manager_id: int


@dataclass(slots=True)
class CoordinateManager:
    """Owns coordinate arrays and caches sparse relations by identity, keyed by
    ``(key, target key, KernelSpec, kind)`` (``manager.py:43-305``)."""

    _manager_id: int = field(default_factory=lambda: next(_manager_ids), init=False)
    _next_id: int = 0
    _coords: dict = field(default_factory=dict)
    _identity_keys: dict = field(default_factory=dict)
    _default_identity_keys: dict = field(default_factory=dict)
    _active_rows: dict = field(default_factory=dict)
    _kernel_relations: dict = field(default_factory=dict)
    _coord_tables: dict = field(default_factory=dict)

    def insert_coords(
        self,
        coords: torch.Tensor,
        stride: int | Sequence[int] = 1,
        active_rows: torch.Tensor | None = None,
    ) -> CoordinateMapKey:
        """Register a coordinate array by object identity and stride."""
        validate_coords(coords)
        normalized = triple(stride, name='stride')
        if active_rows is None:
            default_key = (id(coords), normalized)
            if default_key in self._default_identity_keys:
                return self._default_identity_keys[default_key]
            active = torch.full((1,), int(coords.shape[0]), dtype=torch.int32, device=coords.device)
        else:
            active = active_rows
        cache_key = (id(coords), id(active), normalized)
        if cache_key in self._identity_keys:
            return self._identity_keys[cache_key]
        key = CoordinateMapKey(self._next_id, normalized, self._manager_id)
        self._next_id += 1
        self._coords[key] = coords
        self._active_rows[key] = active
        self._identity_keys[cache_key] = key
        if active_rows is None:
            self._default_identity_keys[(id(coords), normalized)] = key
        return key

    def owns(self, key: CoordinateMapKey) -> bool:
        return key.manager_id == self._manager_id and key in self._coords

    def coords(self, key: CoordinateMapKey) -> torch.Tensor:
        if not self.owns(key):
            raise ValueError('coordinate key does not belong to this manager.')
        return self._coords[key]

    def active_rows(self, key: CoordinateMapKey) -> torch.Tensor:
        if not self.owns(key):
            raise ValueError('coordinate key does not belong to this manager.')
        return self._active_rows[key]

    def coord_table(self, key: CoordinateMapKey) -> torch.Tensor:
        """The first-row coordinate table of a key, built once and handed to every
        builder that starts from these coordinates (submanifold, strided, transposed)."""
        if key not in self._coord_tables:
            self._coord_tables[key] = _ext.build_coord_table(
                self.coords(key), self.active_rows(key)
            )
        return self._coord_tables[key]

    def _cached(self, cache_key, build) -> KernelRelation:
        if cache_key not in self._kernel_relations:
            self._kernel_relations[cache_key] = build()
        return self._kernel_relations[cache_key]

    def kernel_relation(
        self, key, *, kernel_size=3, stride=1, padding=0, dilation=1
    ) -> KernelRelation:
        spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
        return self._cached(
            (key, None, spec, 'forward'),
            lambda: build_kernel_relation(
                self.coords(key),
                active_rows=self.active_rows(key),
                kernel_size=spec.size,
                stride=spec.stride,
                padding=spec.padding,
                dilation=spec.dilation,
                source_table=self.coord_table(key),
            ),
        )

    def submanifold_kernel_relation(self, key, *, kernel_size=3, dilation=1) -> KernelRelation:
        spec = KernelSpec(size=kernel_size, stride=1, padding=0, dilation=dilation)
        return self._cached(
            (key, key, spec, 'submanifold'),
            lambda: build_submanifold_kernel_relation(
                self.coords(key),
                active_rows=self.active_rows(key),
                kernel_size=spec.size,
                dilation=spec.dilation,
                source_table=self.coord_table(key),
            ),
        )

    def transposed_kernel_relation(
        self, key, *, kernel_size=2, stride=2, padding=0, dilation=1
    ) -> KernelRelation:
        spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
        return self._cached(
            (key, None, spec, 'transpose'),
            lambda: build_transposed_kernel_relation(
                self.coords(key),
                active_rows=self.active_rows(key),
                kernel_size=spec.size,
                stride=spec.stride,
                padding=spec.padding,
                dilation=spec.dilation,
            ),
        )

    def generative_relation(self, key, *, kernel_size=2, stride=2) -> KernelRelation:
        spec = KernelSpec(size=kernel_size, stride=stride)
        return self._cached(
            (key, None, spec, 'generative'),
            lambda: build_generative_relation(
                self.coords(key),
                active_rows=self.active_rows(key),
                kernel_size=spec.size,
                stride=spec.stride,
            ),
        )

    def target_kernel_relation(
        self, key, target_key, *, kernel_size=3, stride=1, padding=0, dilation=1
    ) -> KernelRelation:
        if not self.owns(key) or not self.owns(target_key):
            raise ValueError('input and target coordinate keys must belong to this manager.')
        spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
        return self._cached(
            (key, target_key, spec, 'target'),
            lambda: build_target_kernel_relation(
                self.coords(key),
                self.coords(target_key),
                active_rows=self.active_rows(key),
                target_active_rows=self.active_rows(target_key),
                kernel_size=spec.size,
                stride=spec.stride,
                padding=spec.padding,
                dilation=spec.dilation,
            ),
        )

    def target_transposed_relation(self, key, target_key, *, stride=2) -> KernelRelation:
        """Transposed ``kernel_size == stride`` relation onto an existing fine support."""
        if not self.owns(key) or not self.owns(target_key):
            raise ValueError('input and target coordinate keys must belong to this manager.')
        spec = KernelSpec(size=stride, stride=stride)
        return self._cached(
            (key, target_key, spec, 'target_transpose'),
            lambda: build_target_transposed_relation(
                self.coords(key),
                self.coords(target_key),
                active_rows=self.active_rows(key),
                target_active_rows=self.active_rows(target_key),
                stride=spec.stride,
                source_table=self.coord_table(key),
            ),
        )
