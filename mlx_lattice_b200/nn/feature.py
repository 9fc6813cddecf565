"""Feature modules (``mlx_lattice/nn/feature.py:36-177``)."""

from __future__ import annotations

import math

import torch

from mlx_lattice_b200.core import SparseTensor
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.ops import feature as F

__all__ = [
    'BatchNorm', 'Dropout', 'GELU', 'LayerNorm', 'LeakyReLU', 'Linear', 'RMSNorm', 'ReLU', 'SiLU',
    'Sigmoid', 'Softplus', 'Tanh',
]


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


class Sigmoid(Module):
    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.sigmoid(x)


class SiLU(Module):
    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.silu(x)


class Tanh(Module):
    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.tanh(x)


class GELU(Module):
    """``approx``: ``'none'`` / ``'precise'`` / ``'tanh'`` / ``'fast'`` (``nn/feature.py:88-96``)."""

    def __init__(self, approx: str = 'none') -> None:
        self.approx = approx

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.gelu(x, approximate=self.approx)


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01) -> None:
        self.negative_slope = negative_slope

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.leaky_relu(x, negative_slope=self.negative_slope)


class Softplus(Module):
    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.softplus(x)


class Dropout(Module):
    """Inference module: features pass unchanged (``nn/feature.py:134-145``, evaluation)."""

    def __init__(self, p: float = 0.5) -> None:
        if p < 0 or p >= 1:
            raise ValueError('p must satisfy 0 <= p < 1.')
        self.p = p

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.dropout(x, p=self.p, training=False)


class LayerNorm(Module):
    def __init__(self, dims: int, eps: float = 1e-5, affine: bool = True, bias: bool = True) -> None:
        self.eps = eps
        self.weight = torch.ones(dims) if affine else None
        self.bias = torch.zeros(dims) if affine and bias else None

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.layer_norm(x, weight=self.weight, bias=self.bias, eps=self.eps)


class RMSNorm(Module):
    def __init__(self, dims: int, eps: float = 1e-5) -> None:
        self.eps = eps
        self.weight = torch.ones(dims)

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.rms_norm(x, weight=self.weight, eps=self.eps)
