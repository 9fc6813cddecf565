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
    if (feats.dtype == torch.float16 and feats.is_cuda and feats.shape[0] >= 4096
            and weight.in_channels % 32 == 0 and weight.out_channels % 16 == 0
            and 16 <= weight.out_channels <= 256):
        # the tensor cores take fp16 operands: the codes are converted once and kept
        return _ext.linear(feats, _kept_fp16_matrix(weight), bias)
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


def _kept_fp16_matrix(weight: QuantizedWeight) -> torch.Tensor:
    """The dequantised ``(C_out, C_in)`` fp16 matrix of a packed pointwise weight, made once
    and kept on the packed array (a later in-place change of the codes, scales or biases
    makes a new one). code * scale + bias in float32, rounded once."""
    from mlx_lattice_b200.core.quantized import dequantize_weight

    versions = (weight.weight._version, weight.scales._version, weight.biases._version,
                weight.scales.data_ptr(), weight.biases.data_ptr())
    kept = getattr(weight.weight, '_lattice_fp16_matrix', None)
    if kept is None or kept[0] != versions:
        dense = dequantize_weight(weight).to(torch.float16)
        if weight.layout == 'kernel_major':      # (1, C_in, C_out)
            matrix = dense.reshape(weight.in_channels, weight.out_channels).t()
        else:                                    # (C_out, C_in) or (C_out, 1, 1, 1, C_in)
            matrix = dense.reshape(weight.out_channels, weight.in_channels)
        kept = (versions, matrix.contiguous())
        weight.weight._lattice_fp16_matrix = kept
    return kept[1]
