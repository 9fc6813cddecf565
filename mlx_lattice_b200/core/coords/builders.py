"""Relation builders (``mlx_lattice/core/coords/builders.py:42-306``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.coords.validation import validate_coords
from mlx_lattice_b200.core.relations import (
    KernelRelation,
    KernelSpec,
    RelationImplicitGemmView,
)
from mlx_lattice_b200.core.types import Triple, triple


def kernel_offsets(
    kernel_size: int | Sequence[int], dilation: int | Sequence[int] = 1
) -> tuple[Triple, ...]:
    """Spatial offsets of a dense 3D footprint, x-major / z-fastest; odd sizes are
    centred, even sizes start at 0 (``builders.py:130-153``)."""
    kernel = triple(kernel_size, name='kernel_size')
    rate = triple(dilation, name='dilation')
    _require_positive(kernel, 'kernel_size')
    _require_positive(rate, 'dilation')
    axes = []
    for size in kernel:
        if size % 2 == 1:
            axes.append(range(-(size // 2), size // 2 + 1))
        else:
            axes.append(range(size))
    return tuple(
        (int(x * rate[0]), int(y * rate[1]), int(z * rate[2]))
        for x in axes[0]
        for y in axes[1]
        for z in axes[2]
    )


def _active_rows(value: torch.Tensor | None, coords: torch.Tensor) -> torch.Tensor:
    if value is not None:
        if tuple(value.shape) != (1,) or value.dtype != torch.int32:
            raise ValueError('active_rows must have shape (1,) and int32 dtype.')
        return value
    return torch.full((1,), int(coords.shape[0]), dtype=torch.int32, device=coords.device)


def _require_positive(values: Triple, name: str) -> None:
    if any(value <= 0 for value in values):
        raise ValueError(f'{name} values must be positive.')


def _require_nonnegative(values: Triple, name: str) -> None:
    if any(value < 0 for value in values):
        raise ValueError(f'{name} values must be non-negative.')


def _relation(base, masks, lists, **meta) -> KernelRelation:
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = base
    explicit_out = meta.pop('out_coords', None)
    k_offsets, k_edges = lists if lists is not None else (None, None)
    return KernelRelation(
        in_rows,
        out_rows,
        kernel_ids,
        row_offsets=row_offsets,
        counts=counts,
        out_coords=out_coords if explicit_out is None else explicit_out,
        kernel_row_offsets=k_offsets,
        kernel_edge_ids=k_edges,
        row_masks=masks,
        **meta,
    )


def build_kernel_relation(
    coords: torch.Tensor,
    active_rows: torch.Tensor | None = None,
    kernel_size: int | Sequence[int] = 3,
    stride: int | Sequence[int] = 1,
    padding: int | Sequence[int] = 0,
    dilation: int | Sequence[int] = 1,
    *,
    source_table: torch.Tensor | None = None,
) -> KernelRelation:
    """Forward sparse convolution / pooling relation (``builders.py:156-191``).
    ``source_table`` is an optional ``_ext.build_coord_table(coords, active_rows)``."""
    validate_coords(coords)
    spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
    offsets = kernel_offsets(spec.size, spec.dilation)
    source_active = _active_rows(active_rows, coords)
    base, masks, lists = _ext.build_kernel_relation_base(
        coords, source_active, spec.size, spec.stride, spec.padding, spec.dilation,
        want_masks=True, want_kernel_lists=False, source_table=source_table,
    )
    return _relation(
        base, masks, lists,
        kernel_offsets=offsets,
        n_in_capacity=int(coords.shape[0]),
        source_coords=coords,
        source_active_rows=source_active,
        stride=spec.stride,
        padding=spec.padding,
        kind='forward',
    )


def build_submanifold_kernel_relation(
    coords: torch.Tensor,
    active_rows: torch.Tensor | None = None,
    kernel_size: int | Sequence[int] = 3,
    dilation: int | Sequence[int] = 1,
    *,
    source_table: torch.Tensor | None = None,
) -> KernelRelation:
    """Submanifold relation whose output support is ``coords`` (``builders.py:194-233``).
    ``source_table`` is an optional ``_ext.build_coord_table(coords, active_rows)``."""
    validate_coords(coords)
    spec = KernelSpec(size=kernel_size, stride=1, padding=0, dilation=dilation)
    if not all(value % 2 == 1 for value in spec.size):
        raise ValueError(
            'submanifold relations require odd kernels, stride=1, '
            'padding=0, and positive dilation.'
        )
    offsets = kernel_offsets(spec.size, spec.dilation)
    source_active = _active_rows(active_rows, coords)
    base, masks, lists = _ext.build_kernel_relation_base(
        coords, source_active, spec.size, spec.stride, spec.padding, spec.dilation,
        want_masks=True, want_kernel_lists=False, source_table=source_table,
    )
    return _relation(
        base, masks, lists,
        kernel_offsets=offsets,
        n_in_capacity=int(coords.shape[0]),
        out_coords=coords,
        source_coords=coords,
        source_active_rows=source_active,
        target_coords=coords,
        target_active_rows=source_active,
        stride=spec.stride,
        padding=spec.padding,
        kind='submanifold',
    )


def build_target_kernel_relation(
    coords: torch.Tensor,
    target_coords: torch.Tensor,
    *,
    active_rows: torch.Tensor | None = None,
    target_active_rows: torch.Tensor | None = None,
    kernel_size: int | Sequence[int] = 3,
    stride: int | Sequence[int] = 1,
    padding: int | Sequence[int] = 0,
    dilation: int | Sequence[int] = 1,
) -> KernelRelation:
    """Relation from source coords to explicit target coords (``builders.py:82-127``)."""
    validate_coords(coords)
    validate_coords(target_coords)
    if coords.dtype != target_coords.dtype:
        raise ValueError('coordinate arrays must have matching dtype.')
    spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
    offsets = kernel_offsets(spec.size, spec.dilation)
    source_active = _active_rows(active_rows, coords)
    target_active = _active_rows(target_active_rows, target_coords)
    base, masks, lists = _ext.build_target_kernel_relation_base(
        coords, source_active, target_coords, target_active, spec.size, spec.stride,
        spec.padding, spec.dilation, want_masks=True, want_kernel_lists=False,
    )
    return _relation(
        base, masks, lists,
        kernel_offsets=offsets,
        n_in_capacity=int(coords.shape[0]),
        out_coords=target_coords,
        source_coords=coords,
        source_active_rows=source_active,
        target_coords=target_coords,
        target_active_rows=target_active,
        stride=spec.stride,
        padding=spec.padding,
        kind='target',
    )


def build_transposed_kernel_relation(
    coords: torch.Tensor,
    active_rows: torch.Tensor | None = None,
    kernel_size: int | Sequence[int] = 2,
    stride: int | Sequence[int] = 2,
    padding: int | Sequence[int] = 0,
    dilation: int | Sequence[int] = 1,
) -> KernelRelation:
    """Sparse transpose-convolution relation (``builders.py:270-306``)."""
    validate_coords(coords)
    kernel = triple(kernel_size, name='kernel_size')
    step = triple(stride, name='stride')
    pad = triple(padding, name='padding')
    rate = triple(dilation, name='dilation')
    _require_positive(kernel, 'kernel_size')
    _require_positive(step, 'stride')
    _require_nonnegative(pad, 'padding')
    _require_positive(rate, 'dilation')
    offsets = kernel_offsets(kernel, rate)
    source_active = _active_rows(active_rows, coords)
    base = _ext.build_transposed_kernel_relation_base(
        coords, source_active, kernel, step, pad, rate
    )
    return _relation(
        base, None, None,
        kernel_offsets=offsets,
        n_in_capacity=int(coords.shape[0]),
        source_coords=coords,
        source_active_rows=source_active,
        stride=step,
        padding=pad,
        kind='transposed',
    )


def build_generative_relation(
    coords: torch.Tensor,
    active_rows: torch.Tensor | None = None,
    kernel_size: int | Sequence[int] = 2,
    stride: int | Sequence[int] = 2,
) -> KernelRelation:
    """Generative transpose-convolution relation (``builders.py:236-267``)."""
    validate_coords(coords)
    kernel = triple(kernel_size, name='kernel_size')
    step = triple(stride, name='stride')
    _require_positive(kernel, 'kernel_size')
    _require_positive(step, 'stride')
    offsets = kernel_offsets(kernel)
    source_active = _active_rows(active_rows, coords)
    base = _ext.build_generative_relation_base(coords, source_active, kernel, step)
    return _relation(
        base, None, None,
        kernel_offsets=offsets,
        n_in_capacity=int(coords.shape[0]),
        source_coords=coords,
        source_active_rows=source_active,
        stride=step,
        kind='generative',
    )


def build_target_transposed_relation(
    coords: torch.Tensor,
    target_coords: torch.Tensor,
    *,
    active_rows: torch.Tensor | None = None,
    target_active_rows: torch.Tensor | None = None,
    stride: int | Sequence[int] = 2,
    source_table: torch.Tensor | None = None,
) -> KernelRelation:
    """Transposed relation of a ``kernel_size == stride`` conv restricted to a given
    fine support. Equals ``conv_transpose3d`` followed by a right-join alignment to
    the target rows (``mlx_lattice/ops/conv.py:153-182``,
    ``mlx_lattice/ops/tensor.py:228-249``) without materialising the 8x output."""
    validate_coords(coords)
    validate_coords(target_coords)
    step = triple(stride, name='stride')
    _require_positive(step, 'stride')
    source_active = _active_rows(active_rows, coords)
    target_active = _active_rows(target_active_rows, target_coords)
    base, masks = _ext.build_target_transposed_relation_base(
        coords, source_active, target_coords, target_active, step, want_masks=True,
        source_table=source_table,
    )
    return _relation(
        base, masks, None,
        kernel_offsets=kernel_offsets(step),
        n_in_capacity=int(coords.shape[0]),
        out_coords=target_coords,
        source_coords=coords,
        source_active_rows=source_active,
        target_coords=target_coords,
        target_active_rows=target_active,
        stride=step,
        kind='transposed',
    )


def build_relation_implicit_gemm_view(relation: KernelRelation) -> RelationImplicitGemmView:
    """Dense output-to-input map of a relation (``builders.py:42-79``)."""
    contract = relation.contract
    if contract.kind not in ('forward', 'target', 'submanifold'):
        raise ValueError(
            'implicit GEMM view currently supports forward, target, and '
            'submanifold relations.'
        )
    if (
        contract.source_coords is None
        or contract.source_active_rows is None
        or contract.out_coords is None
    ):
        raise ValueError('kernel relation is missing coordinate context for implicit GEMM.')
    output_active = (
        contract.target_active_rows
        if contract.kind in ('target', 'submanifold')
        else contract.out_count
    )
    if output_active is None:
        raise ValueError('kernel relation is missing output activity for implicit GEMM.')
    offsets = torch.tensor(
        contract.kernel_offsets, dtype=torch.int32, device=contract.source_coords.device
    ).reshape(-1, 3)
    out_in_map, row_masks = _ext.build_relation_implicit_gemm_view(
        contract.source_coords,
        contract.source_active_rows,
        contract.out_coords,
        output_active.contiguous(),
        offsets,
        contract.stride,
        contract.padding,
    )
    return RelationImplicitGemmView(out_in_map, row_masks=row_masks)
