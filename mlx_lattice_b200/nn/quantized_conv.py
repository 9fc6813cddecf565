"""Weight-quantized sparse convolution modules
(``mlx_lattice/nn/quantized_conv.py:37-375``): packed int4/int8 affine weights,
floating-point activations. Module fields: ``weight, scales, biases, group_size,
bits, in_channels, out_channels[, bias]``."""

from __future__ import annotations

from mlx_lattice_b200.core import QuantizedWeight, SparseTensor, quantize_weight
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.nn.conv import Conv3d, ConvTranspose3d, SubmConv3d
from mlx_lattice_b200.ops import conv3d, conv_transpose3d, subm_conv3d

__all__ = ['QuantizedConv3d', 'QuantizedConvTranspose3d', 'QuantizedSubmConv3d']


class _QuantizedConvBase(Module):
    def _assign_quantized(self, weight, group_size, bits) -> None:
        q = quantize_weight(weight, group_size=group_size, bits=bits)
        self.weight, self.scales, self.biases = q.weight, q.scales, q.biases
        self.group_size, self.bits = q.group_size, q.bits
        self.in_channels, self.out_channels = q.in_channels, q.out_channels

    def _quantized_weight(self) -> QuantizedWeight:
        return QuantizedWeight(
            self.weight, self.scales, self.biases, self.group_size, self.bits,
            self.in_channels, self.out_channels, self.spec.size, 'dense_5d',
        )

    def _copy_from(self, source, group_size, bits) -> None:
        self.spec = source.spec
        self._assign_quantized(source.weight, group_size, bits)
        self.bias = source.bias

    def to(self, device=None, dtype=None):
        """Scales and biases follow the activation dtype; packed codes stay int."""
        return super().to(device, dtype)


class QuantizedConv3d(_QuantizedConvBase):
    def __init__(self, in_channels, out_channels, *, kernel_size=3, stride=1, padding=0,
                 dilation=1, bias=True, group_size=None, bits=4) -> None:
        self._copy_from(
            Conv3d(in_channels, out_channels, kernel_size=kernel_size, stride=stride,
                   padding=padding, dilation=dilation, bias=bias),
            group_size, bits,
        )

    def __call__(self, x: SparseTensor, *, coordinates=None) -> SparseTensor:
        return conv3d(
            x, self._quantized_weight(), self.bias, kernel_size=self.spec.size,
            stride=self.spec.stride, padding=self.spec.padding, dilation=self.spec.dilation,
            coordinates=coordinates,
        )

    @classmethod
    def from_conv(cls, source: Conv3d, group_size=None, bits=4):
        out = cls.__new__(cls)
        out._copy_from(source, group_size, bits)
        return out


class QuantizedSubmConv3d(_QuantizedConvBase):
    def __init__(self, in_channels, out_channels, *, kernel_size=3, dilation=1, bias=True,
                 group_size=None, bits=4) -> None:
        self._copy_from(
            SubmConv3d(in_channels, out_channels, kernel_size=kernel_size, dilation=dilation,
                       bias=bias),
            group_size, bits,
        )

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return subm_conv3d(
            x, self._quantized_weight(), self.bias, kernel_size=self.spec.size,
            dilation=self.spec.dilation,
        )

    @classmethod
    def from_conv(cls, source: SubmConv3d, group_size=None, bits=4):
        out = cls.__new__(cls)
        out._copy_from(source, group_size, bits)
        return out


class QuantizedConvTranspose3d(_QuantizedConvBase):
    def __init__(self, in_channels, out_channels, *, kernel_size=2, stride=2, padding=0,
                 dilation=1, bias=True, group_size=None, bits=4) -> None:
        self._copy_from(
            ConvTranspose3d(in_channels, out_channels, kernel_size=kernel_size, stride=stride,
                            padding=padding, dilation=dilation, bias=bias),
            group_size, bits,
        )

    def __call__(self, x: SparseTensor, *, coordinates=None) -> SparseTensor:
        return conv_transpose3d(
            x, self._quantized_weight(), self.bias, kernel_size=self.spec.size,
            stride=self.spec.stride, padding=self.spec.padding, dilation=self.spec.dilation,
            coordinates=coordinates,
        )

    @classmethod
    def from_conv(cls, source: ConvTranspose3d, group_size=None, bits=4):
        out = cls.__new__(cls)
        out._copy_from(source, group_size, bits)
        return out
