"""Pointwise feature operators (``mlx_lattice/ops/feature.py:33-56,166-187``)."""

from __future__ import annotations

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core import QuantizedWeight, SparseTensor
from mlx_lattice_b200.ops._quantized import quantized_matmul

__all__ = [
    'batch_norm', 'dropout', 'gelu', 'layer_norm', 'leaky_relu', 'linear', 'relu', 'rms_norm', 'sigmoid',
    'silu', 'softplus', 'tanh',
]


def linear(x: SparseTensor, weight, bias: torch.Tensor | None = None) -> SparseTensor:
    """Dense ``(C_out, C_in)`` or packed linear projection; coordinates preserved."""
    _check_bias(bias, x.feats.dtype)
    if isinstance(weight, QuantizedWeight):
        if bias is not None and bias.shape[0] != weight.out_channels:
            raise ValueError('bias channels must match output channels.')
        return x.replace(feats=quantized_matmul(x.feats, weight, bias))
    if weight.ndim != 2:
        raise ValueError('weight must have shape (C_out, C_in).')
    if weight.shape[1] != x.channels:
        raise ValueError('weight input channels must match x.channels.')
    if weight.dtype != x.feats.dtype:
        raise ValueError('convolution weights must match feature dtype.')
    if bias is not None and bias.shape[0] != weight.shape[0]:
        raise ValueError('bias channels must match output channels.')
    return x.replace(feats=_ext.linear(x.feats, weight, bias))


def relu(x: SparseTensor) -> SparseTensor:
    return x.replace(feats=_ext.relu(x.feats))


def sigmoid(x: SparseTensor) -> SparseTensor:
    return x.replace(feats=_ext.activation(x.feats, 'sigmoid'))


def silu(x: SparseTensor) -> SparseTensor:
    return x.replace(feats=_ext.activation(x.feats, 'silu'))


def tanh(x: SparseTensor) -> SparseTensor:
    return x.replace(feats=_ext.activation(x.feats, 'tanh'))


def gelu(x: SparseTensor, *, approximate: str = 'none') -> SparseTensor:
    """``'none'`` / ``'precise'``: the erf formula; ``'tanh'``: the tanh approximation;
    ``'fast'``: ``x * sigmoid(1.702 x)`` (``ops/feature.py:64-93``)."""
    forms = {'none': 'gelu_erf', 'precise': 'gelu_erf', 'tanh': 'gelu_tanh', 'fast': 'gelu_fast'}
    if approximate not in forms:
        raise ValueError("approximate must be 'none', 'precise', 'tanh', or 'fast'.")
    return x.replace(feats=_ext.activation(x.feats, forms[approximate]))


def leaky_relu(x: SparseTensor, *, negative_slope: float = 0.01) -> SparseTensor:
    return x.replace(feats=_ext.activation(x.feats, 'leaky_relu', float(negative_slope)))


def softplus(x: SparseTensor, *, beta: float = 1.0, threshold: float = 20.0) -> SparseTensor:
    """``x`` where ``beta * x > threshold``, else ``log(1 + exp(beta x)) / beta``
    (``ops/feature.py:112-129``)."""
    if beta <= 0:
        raise ValueError('beta must be positive.')
    return x.replace(feats=_ext.activation(x.feats, 'softplus', float(beta), float(threshold)))


def dropout(x: SparseTensor, *, p: float = 0.5, training: bool = True) -> SparseTensor:
    """Inference form of ``ops/feature.py:132-150``: the features pass unchanged when
    ``training`` is false or ``p`` is zero. Sampling a mask is training work and is not
    part of this package."""
    if p < 0 or p >= 1:
        raise ValueError('p must satisfy 0 <= p < 1.')
    if training and p != 0:
        raise ValueError('dropout in training mode is not available on the inference path.')
    return x.replace(feats=x.feats)


def layer_norm(x: SparseTensor, *, weight=None, bias=None, eps: float = 1e-5) -> SparseTensor:
    """Layer normalisation of every sparse row over its channels (``ops/feature.py:196-210``)."""
    if eps <= 0:
        raise ValueError('eps must be positive.')
    return x.replace(feats=_ext.row_norm(x.feats, weight, bias, eps, rms=False))


def rms_norm(x: SparseTensor, *, weight=None, eps: float = 1e-5) -> SparseTensor:
    """RMS normalisation of every sparse row (``ops/feature.py:214-225``)."""
    if eps <= 0:
        raise ValueError('eps must be positive.')
    return x.replace(feats=_ext.row_norm(x.feats, weight, None, eps, rms=True))


def batch_norm(
    x: SparseTensor, *, weight=None, bias=None, mean=None, var=None, eps: float = 1e-5,
    fuse_relu: bool = False,
) -> SparseTensor:
    """Per-channel normalisation with given (running) statistics. ``fuse_relu``
    (an addition to the reference signature) applies ReLU in the same pass."""
    if eps <= 0:
        raise ValueError('eps must be positive.')
    if mean is None or var is None:
        raise ValueError(
            'batch statistics over active rows are a training-path feature; '
            'pass running mean and var.'
        )
    for name, vector in (('mean', mean), ('var', var), ('weight', weight), ('bias', bias)):
        if vector is not None and tuple(vector.shape) != (x.channels,):
            raise ValueError(f'{name} must have shape (C,).')
        if vector is not None and vector.dtype != x.feats.dtype:
            raise ValueError(f'{name} dtype must match features.')
    return x.replace(
        feats=_ext.batch_norm_relu(x.feats, weight, bias, mean, var, eps, fuse_relu)
    )


def _check_bias(bias, dtype) -> None:
    if bias is None:
        return
    if bias.ndim != 1:
        raise ValueError('bias must have shape (C_out,).')
    if bias.dtype != dtype:
        raise ValueError('bias dtype must match output features.')
