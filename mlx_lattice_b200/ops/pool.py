"""Sparse pooling operators (``mlx_lattice/ops/pool.py:27-280``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core import KernelSpec, SparseTensor
from mlx_lattice_b200.ops._relation_exec import sparse_pool_features_from_relation

__all__ = [
    'avg_pool3d', 'global_avg_pool', 'global_max_pool', 'global_sum_pool', 'max_pool3d',
    'pool3d', 'sum_pool3d',
]


def pool3d(x: SparseTensor, *, mode='sum', kernel_size=2, stride=2, padding=0, dilation=1) -> SparseTensor:
    """Local sparse pooling over a forward kernel relation; float32 features only,
    like the reference (``ops/pool.py:27-54,155-191``)."""
    spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
    if x.feats.dtype != torch.float32:
        raise ValueError('pooling currently supports float32 tensors.')
    if x.coords.dtype != torch.int32:
        raise ValueError('CUDA sparse pooling requires int32 coordinates.')
    if mode not in ('sum', 'max', 'avg'):
        raise ValueError("mode must be 'sum', 'max', or 'avg'.")
    relation = x.coord_manager.kernel_relation(
        x.coord_key, kernel_size=spec.size, stride=spec.stride, padding=spec.padding,
        dilation=spec.dilation,
    )
    feats = sparse_pool_features_from_relation(
        x.feats, relation, input_exclusive=_input_exclusive(spec), mode=mode
    )
    return SparseTensor(
        relation.out_coords,
        feats,
        stride=tuple(a * b for a, b in zip(x.stride, spec.stride)),
        coord_manager=x.coord_manager,
        active_rows=relation.out_count,
    )


def sum_pool3d(x: SparseTensor, *, kernel_size=2, stride=2, padding=0, dilation=1) -> SparseTensor:
    return pool3d(x, mode='sum', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


def max_pool3d(x: SparseTensor, *, kernel_size=2, stride=2, padding=0, dilation=1) -> SparseTensor:
    return pool3d(x, mode='max', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


def avg_pool3d(x: SparseTensor, *, kernel_size=2, stride=2, padding=0, dilation=1) -> SparseTensor:
    return pool3d(x, mode='avg', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


def global_sum_pool(x: SparseTensor) -> torch.Tensor:
    return _global(x, 'sum')


def global_avg_pool(x: SparseTensor) -> torch.Tensor:
    """Per-batch mean; empty batches give zero rows (``ops/pool.py:120-129``)."""
    return _global(x, 'avg')


def global_max_pool(x: SparseTensor) -> torch.Tensor:
    return _global(x, 'max')


def _global(x: SparseTensor, mode: str) -> torch.Tensor:
    if x.feats.dtype != torch.float32:
        raise ValueError('pooling currently supports float32 tensors.')
    if x.batch_counts is None:
        raise ValueError('batch_counts metadata is required for global pooling.')
    counts = x.batch_counts
    if mode == 'max' and any(count == 0 for count in counts):
        raise ValueError('global_max_pool does not support empty batches.')
    offsets = [0]
    for count in counts:
        offsets.append(offsets[-1] + count)
    batch_offsets = torch.tensor(offsets, dtype=torch.int32, device=x.feats.device)
    return _ext.global_pool(x.feats, batch_offsets, mode)


def _input_exclusive(spec: KernelSpec) -> bool:
    return all(
        stride >= (size - 1) * dilation + 1
        for stride, size, dilation in zip(spec.stride, spec.size, spec.dilation, strict=True)
    )
