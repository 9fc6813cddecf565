"""Pooling modules (``mlx_lattice/nn/pool.py``)."""

from __future__ import annotations

import torch

from mlx_lattice_b200.core import KernelSpec, SparseTensor
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.ops import global_avg_pool, global_max_pool, global_sum_pool, pool3d

__all__ = ['AvgPool3d', 'GlobalAvgPool', 'GlobalMaxPool', 'GlobalSumPool', 'MaxPool3d',
           'Pool3d', 'SumPool3d']


class Pool3d(Module):
    def __init__(self, *, mode='sum', kernel_size=2, stride=2, padding=0, dilation=1) -> None:
        self.mode = mode
        self.spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return pool3d(
            x, mode=self.mode, kernel_size=self.spec.size, stride=self.spec.stride,
            padding=self.spec.padding, dilation=self.spec.dilation,
        )


class SumPool3d(Pool3d):
    def __init__(self, *, kernel_size=2, stride=2, padding=0, dilation=1) -> None:
        super().__init__(mode='sum', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


class MaxPool3d(Pool3d):
    def __init__(self, *, kernel_size=2, stride=2, padding=0, dilation=1) -> None:
        super().__init__(mode='max', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


class AvgPool3d(Pool3d):
    def __init__(self, *, kernel_size=2, stride=2, padding=0, dilation=1) -> None:
        super().__init__(mode='avg', kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation)


class GlobalSumPool(Module):
    def __call__(self, x: SparseTensor) -> torch.Tensor:
        return global_sum_pool(x)


class GlobalAvgPool(Module):
    def __call__(self, x: SparseTensor) -> torch.Tensor:
        return global_avg_pool(x)


class GlobalMaxPool(Module):
    def __call__(self, x: SparseTensor) -> torch.Tensor:
        return global_max_pool(x)
