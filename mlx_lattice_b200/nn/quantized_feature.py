"""Weight-quantized linear module (``mlx_lattice/nn/quantized_feature.py:14-100``)."""

from __future__ import annotations

from mlx_lattice_b200.core import QuantizedWeight, SparseTensor, quantize_weight
from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.ops import feature as F

__all__ = ['QuantizedLinear']


class QuantizedLinear(Module):
    def __init__(self, input_dims, output_dims, bias=True, group_size=None, bits=4,
                 mode='affine') -> None:
        if mode != 'affine':
            raise ValueError("QuantizedLinear supports only mode='affine'.")
        from mlx_lattice_b200.nn.feature import Linear

        source = Linear(input_dims, output_dims, bias=bias)
        self._assign_quantized(source.weight, group_size, bits)
        self.bias = source.bias

    def __call__(self, x: SparseTensor) -> SparseTensor:
        return F.linear(x, self._quantized_weight(), self.bias)

    @classmethod
    def from_linear(cls, linear, group_size=None, bits=4, mode='affine'):
        if mode != 'affine':
            raise ValueError("QuantizedLinear supports only mode='affine'.")
        out = cls.__new__(cls)
        out._assign_quantized(linear.weight, group_size, bits)
        out.bias = linear.bias
        return out

    def _assign_quantized(self, weight, group_size, bits) -> None:
        q = quantize_weight(weight, group_size=group_size, bits=bits)
        self.weight, self.scales, self.biases = q.weight, q.scales, q.biases
        self.group_size, self.bits = q.group_size, q.bits
        self.input_dims, self.output_dims = q.in_channels, q.out_channels

    def _quantized_weight(self) -> QuantizedWeight:
        return QuantizedWeight(
            self.weight, self.scales, self.biases, self.group_size, self.bits,
            self.input_dims, self.output_dims, (1, 1, 1), 'linear',
        )
