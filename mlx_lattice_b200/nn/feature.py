"""Feature modules (``mlx_lattice/nn/feature.py:36-177``)."""

from __future__ import annotations

import math

import torch

from mlx_lattice_b200.core import SparseTensor
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.ops import feature as F

__all__ = ['BatchNorm', 'Linear', 'ReLU']


class Linear(Module):
    def __init__(self, input_dims: int, output_dims: int, bias: bool = True) -> None:
        scale = math.sqrt(1.0 / input_dims)
        self.weight = (torch.rand((output_dims, input_dims)) * 2 - 1) * scale
        self.bias = (torch.rand((output_dims,)) * 2 - 1) * scale if bias else None

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.linear(x, self.weight, self.bias)


class ReLU(Module):
    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.relu(x)


class BatchNorm(Module):
    """Inference batch normalisation with running statistics
    (``nn/feature.py:153-177``, evaluation branch). ``fuse_relu`` folds a following
    ReLU into the same pass."""

    def __init__(self, num_features: int, eps: float = 1e-5, affine: bool = True,
                 fuse_relu: bool = False) -> None:
        self.eps = eps
        self.fuse_relu = fuse_relu
        self.weight = torch.ones(num_features) if affine else None
        self.bias = torch.zeros(num_features) if affine else None
        self.running_mean = torch.zeros(num_features)
        self.running_var = torch.ones(num_features)

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.batch_norm(
            x, weight=self.weight, bias=self.bias, mean=self.running_mean,
            var=self.running_var, eps=self.eps, fuse_relu=self.fuse_relu,
        )
