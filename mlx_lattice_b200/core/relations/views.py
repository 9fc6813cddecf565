"""Kernel relation container (``mlx_lattice/core/relations/views.py:258-510``).

A relation stores the contract arrays ``(in_rows, out_rows, kernel_ids)`` with
device-side ``counts = [E, N_out]`` plus execution views. The reference evaluates
its arrays lazily (unused views are never computed); here the input CSR, the
per-offset pair lists, the implicit-GEMM view and the mask-sorted row order are
built on first access for the same effect.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Literal

import torch

from mlx_lattice_b200.core.types import Triple

RelationKind = Literal['forward', 'target', 'submanifold', 'transposed', 'generative']
_KINDS = ('forward', 'target', 'submanifold', 'transposed', 'generative')


@dataclass(frozen=True, slots=True)
class RelationEdges:
    in_rows: torch.Tensor
    out_rows: torch.Tensor
    kernel_ids: torch.Tensor

    @property
    def capacity(self) -> int:
        return int(self.in_rows.shape[0])


@dataclass(frozen=True, slots=True)
class RelationCSRView:
    row_offsets: torch.Tensor
    edge_ids: torch.Tensor | None = None


@dataclass(frozen=True, slots=True)
class RelationImplicitGemmView:
    out_in_map: torch.Tensor
    row_masks: torch.Tensor

    def __post_init__(self) -> None:
        if self.out_in_map.ndim != 2:
            raise ValueError('out_in_map must have shape (Nout, K).')
        if self.row_masks.ndim != 2:
            raise ValueError('row_masks must have shape (Nout, M).')
        if int(self.row_masks.shape[0]) != int(self.out_in_map.shape[0]):
            raise ValueError('row_masks must have one row per out_in_map row.')
        if int(self.row_masks.shape[1]) != (int(self.out_in_map.shape[1]) + 31) // 32:
            raise ValueError('row_masks must have ceil(K / 32) words per output row.')


@dataclass(frozen=True, slots=True)
class RelationSortedImplicitGemmView:
    sorted_out_in_map: torch.Tensor
    sorted_kv_out_in_map: torch.Tensor
    reorder_rows: torch.Tensor
    tile_masks: torch.Tensor


@dataclass(frozen=True, slots=True)
class SparseRelationContract:
    counts: torch.Tensor
    kernel_offsets: tuple[Triple, ...]
    out_coords: torch.Tensor | None = None
    n_in_capacity: int | None = None
    n_out_capacity: int | None = None
    n_kernels: int | None = None
    source_coords: torch.Tensor | None = None
    source_active_rows: torch.Tensor | None = None
    target_coords: torch.Tensor | None = None
    target_active_rows: torch.Tensor | None = None
    stride: Triple = (1, 1, 1)
    padding: Triple = (0, 0, 0)
    kind: RelationKind = 'forward'

    def __post_init__(self) -> None:
        if tuple(self.counts.shape) != (2,) or self.counts.dtype != torch.int32:
            raise ValueError('counts must have shape (2,) and int32 dtype.')
        if self.kind not in _KINDS:
            raise ValueError(
                "relation kind must be 'forward', 'target', "
                "'submanifold', 'transposed', or 'generative'."
            )

    @property
    def edge_count(self) -> torch.Tensor:
        return self.counts[:1]

    @property
    def out_count(self) -> torch.Tensor:
        return self.counts[1:2]


class KernelRelation:
    """Sparse kernel relation with execution-oriented views."""

    def __init__(
        self,
        in_rows: torch.Tensor,
        out_rows: torch.Tensor,
        kernel_ids: torch.Tensor,
        *,
        row_offsets: torch.Tensor,
        counts: torch.Tensor,
        kernel_offsets: tuple[Triple, ...] = (),
        out_coords: torch.Tensor | None = None,
        n_in_capacity: int | None = None,
        n_out_capacity: int | None = None,
        n_kernels: int | None = None,
        source_coords: torch.Tensor | None = None,
        source_active_rows: torch.Tensor | None = None,
        target_coords: torch.Tensor | None = None,
        target_active_rows: torch.Tensor | None = None,
        stride: Triple = (1, 1, 1),
        padding: Triple = (0, 0, 0),
        kind: RelationKind = 'forward',
        in_row_offsets: torch.Tensor | None = None,
        in_edge_ids: torch.Tensor | None = None,
        kernel_row_offsets: torch.Tensor | None = None,
        kernel_edge_ids: torch.Tensor | None = None,
        row_masks: torch.Tensor | None = None,
    ) -> None:
        if n_out_capacity is None and out_coords is not None:
            n_out_capacity = int(out_coords.shape[0])
        if n_kernels is None and kernel_offsets:
            n_kernels = len(kernel_offsets)
        if n_out_capacity is not None and int(row_offsets.shape[0]) != n_out_capacity + 1:
            raise ValueError('row_offsets must have length n_out_capacity + 1.')
        self.contract = SparseRelationContract(
            counts=counts,
            kernel_offsets=tuple((int(x), int(y), int(z)) for x, y, z in kernel_offsets),
            out_coords=out_coords,
            n_in_capacity=n_in_capacity,
            n_out_capacity=n_out_capacity,
            n_kernels=n_kernels,
            source_coords=source_coords,
            source_active_rows=source_active_rows,
            target_coords=target_coords,
            target_active_rows=target_active_rows,
            stride=tuple(int(v) for v in stride),
            padding=tuple(int(v) for v in padding),
            kind=kind,
        )
        self.edges = RelationEdges(in_rows, out_rows, kernel_ids)
        self.output_csr = RelationCSRView(row_offsets)
        self._input_csr = (
            None if in_row_offsets is None else RelationCSRView(in_row_offsets, in_edge_ids)
        )
        self._kernel_csr = (
            None
            if kernel_row_offsets is None
            else RelationCSRView(kernel_row_offsets, kernel_edge_ids)
        )
        self.row_masks = row_masks
        self.implicit_gemm: RelationImplicitGemmView | None = None
        self.sorted_implicit_gemm: RelationSortedImplicitGemmView | None = None
        self._row_order: torch.Tensor | None = None
        self._conv_plan: torch.Tensor | None = None

    # -- contract ------------------------------------------------------------
    @property
    def edge_capacity(self) -> int:
        return self.edges.capacity

    @property
    def counts(self) -> torch.Tensor:
        return self.contract.counts

    @property
    def edge_count(self) -> torch.Tensor:
        return self.contract.edge_count

    @property
    def out_count(self) -> torch.Tensor:
        return self.contract.out_count

    @property
    def kernel_offsets(self) -> tuple[Triple, ...]:
        return self.contract.kernel_offsets

    @property
    def out_coords(self) -> torch.Tensor | None:
        return self.contract.out_coords

    @property
    def n_in_capacity(self) -> int | None:
        return self.contract.n_in_capacity

    @property
    def n_out_capacity(self) -> int | None:
        return self.contract.n_out_capacity

    @property
    def n_kernels(self) -> int | None:
        return self.contract.n_kernels

    # -- views ---------------------------------------------------------------
    @property
    def row_offsets(self) -> torch.Tensor:
        return self.output_csr.row_offsets

    @property
    def input_csr(self) -> RelationCSRView:
        if self._input_csr is None:
            from mlx_lattice_b200 import _ext

            offsets, edges = _ext.build_relation_grouped_view(
                self.edges.in_rows, self.counts, int(self.n_in_capacity or 0)
            )
            self._input_csr = RelationCSRView(offsets, edges)
        return self._input_csr

    @property
    def kernel_csr(self) -> RelationCSRView:
        if self._kernel_csr is None:
            from mlx_lattice_b200 import _ext

            offsets, edges = _ext.build_relation_grouped_view(
                self.edges.kernel_ids, self.counts, int(self.n_kernels or 0)
            )
            self._kernel_csr = RelationCSRView(offsets, edges)
        return self._kernel_csr

    @property
    def in_row_offsets(self) -> torch.Tensor:
        return self.input_csr.row_offsets

    @property
    def in_edge_ids(self) -> torch.Tensor:
        return self.input_csr.edge_ids

    @property
    def kernel_row_offsets(self) -> torch.Tensor:
        return self.kernel_csr.row_offsets

    @property
    def kernel_edge_ids(self) -> torch.Tensor:
        return self.kernel_csr.edge_ids

    out_view = property(lambda self: self.output_csr)
    in_view = property(lambda self: self.input_csr)
    kernel_view = property(lambda self: self.kernel_csr)

    def require_implicit_gemm(self) -> RelationImplicitGemmView:
        """Return or lazily build the dense output-row by offset map."""
        if self.implicit_gemm is None:
            from mlx_lattice_b200.core.coords.builders import (
                build_relation_implicit_gemm_view,
            )

            self.implicit_gemm = build_relation_implicit_gemm_view(self)
        return self.implicit_gemm

    def require_sorted_implicit_gemm(self) -> RelationSortedImplicitGemmView:
        """Mask-sorted view (``views.py:467-510``): rows ordered by offset mask, the
        K-major map, and per-64-row-tile masks (four 16-row sub-tile words)."""
        if self.sorted_implicit_gemm is not None:
            return self.sorted_implicit_gemm
        view = self.require_implicit_gemm()
        if view.row_masks.shape[1] != 1:
            raise ValueError('sorted implicit GEMM view currently supports K <= 32.')
        masks = view.row_masks[:, 0]
        if self.n_kernels is not None and self.n_kernels <= 31:
            # the native stable radix sort of the masks; every row takes part, as in the
            # reference's argsort (masks of at most 31 bits sort alike signed and unsigned)
            from mlx_lattice_b200 import _ext

            every_row = torch.tensor([0, int(masks.shape[0])], dtype=torch.int32, device=masks.device)
            order = _ext.build_mask_row_order(view.row_masks, every_row, self.n_kernels)
        else:
            order = torch.argsort(masks, stable=True).to(torch.int32)
        sorted_map = view.out_in_map[order.long()]
        n = int(view.out_in_map.shape[0])
        tiles = (n + 63) // 64
        padded = torch.zeros(tiles * 64, dtype=torch.int32, device=masks.device)
        padded[:n] = masks[order.long()]
        groups = padded.view(tiles, 4, 16)
        tile_masks = groups[:, :, 0].clone()
        for i in range(1, 16):
            tile_masks |= groups[:, :, i]
        self.sorted_implicit_gemm = RelationSortedImplicitGemmView(
            sorted_out_in_map=sorted_map,
            sorted_kv_out_in_map=sorted_map.t().contiguous(),
            reorder_rows=order,
            tile_masks=tile_masks.reshape(-1),
        )
        return self.sorted_implicit_gemm

    def require_row_order(self) -> torch.Tensor | None:
        """Row permutation for the tensor-core tiles (rows grouped by offset mask);
        None when the relation carries no single-word row masks."""
        if self._row_order is None and self.row_masks is not None and self.row_masks.shape[1] == 1:
            from mlx_lattice_b200 import _ext

            self._row_order = _ext.build_mask_row_order(
                self.row_masks, self.counts, int(self.n_kernels or 32)
            )
        return self._row_order

    def require_conv_plan(self) -> torch.Tensor | None:
        """Gather plan of the tensor-core convolution over this relation, built once
        and shared by every convolution that consumes the relation; None when the
        relation has more than 32 kernel offsets or no static capacities."""
        if self._conv_plan is None:
            if self.n_kernels is None or self.n_kernels > 32 or self.n_out_capacity is None:
                return None
            if self.n_in_capacity is None:
                return None
            from mlx_lattice_b200 import _ext

            self._conv_plan = _ext.build_conv_plan(
                self.edges.in_rows, self.edges.kernel_ids, self.counts,
                self.output_csr.row_offsets, int(self.n_in_capacity), int(self.n_out_capacity),
                int(self.n_kernels), self.require_row_order(),
                self.row_masks if self.row_masks is not None and self.row_masks.shape[1] == 1 else None,
            )
        return self._conv_plan
