"""Sparse convolution modules (``mlx_lattice/nn/conv.py:49-308``)."""

from __future__ import annotations

import math
from collections.abc import Sequence

import torch

from mlx_lattice_b200.core import KernelSpec, SparseTensor
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.ops import conv3d, conv_transpose3d, subm_conv3d

__all__ = ['Conv3d', 'ConvTranspose3d', 'SubmConv3d']


def _init_kernel_params(module, in_channels, out_channels, spec: KernelSpec, bias: bool) -> None:
    """``U(+-sqrt(1 / (C_in * K)))`` dense 5-D weight, zero bias (``conv.py:294-308``)."""
    scale = math.sqrt(1.0 / (in_channels * spec.volume))
    module.weight = (torch.rand((out_channels, *spec.size, in_channels)) * 2 - 1) * scale
    module.bias = torch.zeros((out_channels,)) if bias else None


class Conv3d(Module):
    """Sparse 3D convolution; weight ``(C_out, Kx, Ky, Kz, C_in)``."""

    def __init__(self, in_channels, out_channels, *, kernel_size=3, stride=1, padding=0,
                 dilation=1, bias=True) -> None:
        self.spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
        _init_kernel_params(self, in_channels, out_channels, self.spec, bias)

    def __call__(self, x: SparseTensor, *, coordinates=None) -> SparseTensor:
        return conv3d(
            x, self.weight, self.bias, kernel_size=self.spec.size, stride=self.spec.stride,
            padding=self.spec.padding, dilation=self.spec.dilation, coordinates=coordinates,
        )

    def to_quantized(self, group_size: int | None = None, bits: int | None = None):
        from mlx_lattice_b200.nn.quantized_conv import QuantizedConv3d

        return QuantizedConv3d.from_conv(self, group_size=group_size, bits=4 if bits is None else bits)


class SubmConv3d(Module):
    """Submanifold sparse convolution preserving coordinate identity."""

    def __init__(self, in_channels, out_channels, *, kernel_size=3, dilation=1, bias=True) -> None:
        self.spec = KernelSpec(size=kernel_size, stride=1, padding=0, dilation=dilation)
        _init_kernel_params(self, in_channels, out_channels, self.spec, bias)

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return subm_conv3d(
            x, self.weight, self.bias, kernel_size=self.spec.size, dilation=self.spec.dilation
        )

    def to_quantized(self, group_size: int | None = None, bits: int | None = None):
        from mlx_lattice_b200.nn.quantized_conv import QuantizedSubmConv3d

        return QuantizedSubmConv3d.from_conv(self, group_size=group_size, bits=4 if bits is None else bits)


class ConvTranspose3d(Module):
    """Sparse transpose convolution. ``coordinates=`` (an addition to the reference
    call) restricts the output to an existing fine support."""

    def __init__(self, in_channels, out_channels, *, kernel_size=2, stride=2, padding=0,
                 dilation=1, bias=True) -> None:
        self.spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
        _init_kernel_params(self, in_channels, out_channels, self.spec, bias)

    def __call__(self, x: SparseTensor, *, coordinates: SparseTensor | None = None) -> SparseTensor:
        return conv_transpose3d(
            x, self.weight, self.bias, kernel_size=self.spec.size, stride=self.spec.stride,
            padding=self.spec.padding, dilation=self.spec.dilation, coordinates=coordinates,
        )

    def to_quantized(self, group_size: int | None = None, bits: int | None = None):
        from mlx_lattice_b200.nn.quantized_conv import QuantizedConvTranspose3d

        return QuantizedConvTranspose3d.from_conv(self, group_size=group_size, bits=4 if bits is None else bits)
