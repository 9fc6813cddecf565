"""Packed-weight matrix multiply (``mlx_lattice/ops/_quantized.py:8-38``)."""

from __future__ import annotations

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.quantized import QuantizedWeight


def quantized_matmul(feats: torch.Tensor, weight: QuantizedWeight, bias=None) -> torch.Tensor:
    """``feats @ dequantize(weight).T`` with float32 accumulation."""
    if weight.kernel_size != (1, 1, 1):
        raise ValueError('quantized matmul requires a pointwise weight.')
    if feats.ndim != 2 or feats.shape[1] != weight.in_channels:
        raise ValueError('features must have shape (N, quantized_weight.in_channels).')
    if feats.dtype != weight.scales.dtype:
        raise ValueError('features must match quantized scale dtype.')
    return _ext.quantized_linear(
        feats,
        weight.weight[0],
        weight.scales[0],
        weight.biases[0],
        weight.out_channels,
        weight.storage_in_channels,
        weight.group_size,
        weight.bits,
        bias,
    )
