"""Packed affine INT4/INT8 inference weights (``mlx_lattice/core/quantized.py``).

Storage format (pinned by the reference's own decoder,
``native/features/convolution/cpu/quantized.cpp:54-62``): spatial weights are
``weight (K, S*bits/32, C_out)`` uint32 with channel ``ci`` in word ``(ci*bits)>>5``
at shift ``(ci*bits)&31`` and ``scales/biases (K, S/group, C_out)``; linear weights
are ``(1, C_out, S*bits/32)`` and ``(1, C_out, S/group)``. ``S`` is ``C_in`` rounded
up to the group size. The code selection itself comes from a third-party routine in
the reference (``mx.quantize(mode='affine')``); ``quantize_weight`` restates that
published rule with torch tensor ops. It runs once at set-up, not on the hot path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

import torch

from mlx_lattice_b200.core.types import Triple

QuantizedWeightLayout = Literal['linear', 'kernel_major', 'dense_5d']

__all__ = ['QuantizedWeight', 'QuantizedWeightLayout', 'dequantize_weight', 'quantize_weight']


def _volume(size: Triple) -> int:
    return size[0] * size[1] * size[2]


@dataclass(frozen=True, slots=True)
class QuantizedWeight:
    """Packed codes plus per-group ``scales`` and ``biases``; logical values are
    ``scale * code + bias``."""

    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    group_size: int
    bits: int
    in_channels: int
    out_channels: int
    kernel_size: Triple
    layout: QuantizedWeightLayout

    def __post_init__(self) -> None:
        if self.bits not in (4, 8):
            raise ValueError('quantized weight bits must be 4 or 8.')
        if self.group_size not in (32, 64, 128):
            raise ValueError('quantized weight group_size must be 32, 64, or 128.')
        if self.weight.dtype not in (torch.uint32, torch.int32) or self.weight.ndim != 3:
            raise ValueError('packed weight must be a three-dimensional uint32 array.')
        if self.scales.dtype not in (torch.float16, torch.float32):
            raise ValueError('quantized scales must be float16 or float32.')
        if self.biases.dtype != self.scales.dtype:
            raise ValueError('quantized biases must match scales dtype.')
        if self.scales.ndim != 3 or self.biases.shape != self.scales.shape:
            raise ValueError('scales and biases must have shape (K, C_out, G).')
        if self.in_channels <= 0 or self.out_channels <= 0:
            raise ValueError('quantized weight channels must be positive.')
        if any(size <= 0 for size in self.kernel_size):
            raise ValueError('quantized weight kernel dimensions must be positive.')
        if self.weight.shape[0] != _volume(self.kernel_size):
            raise ValueError('packed weight kernel rows do not match kernel_size.')
        if self.is_pointwise:
            if self.weight.shape[1] != self.out_channels:
                raise ValueError('pointwise packed weight output channels do not match.')
            if tuple(self.scales.shape[:2]) != tuple(self.weight.shape[:2]):
                raise ValueError('pointwise weight and quantization rows must match.')
        else:
            if self.weight.shape[2] != self.out_channels:
                raise ValueError('spatial packed weight output channels do not match.')
            if self.scales.shape[0] != self.weight.shape[0] or (
                self.scales.shape[2] != self.out_channels
            ):
                raise ValueError('spatial weight and quantization rows must match.')
        if self.storage_in_channels % self.group_size != 0:
            raise ValueError('packed storage channels must be divisible by group_size.')
        group_dim = 2 if self.is_pointwise else 1
        if self.scales.shape[group_dim] != self.storage_in_channels // self.group_size:
            raise ValueError('quantization group count does not match storage.')
        if self.storage_in_channels < self.in_channels:
            raise ValueError('packed storage channels cannot be smaller than logical channels.')

    @property
    def storage_in_channels(self) -> int:
        packed_dim = 2 if self.is_pointwise else 1
        return int(self.weight.shape[packed_dim]) * 32 // self.bits

    @property
    def is_pointwise(self) -> bool:
        return _volume(self.kernel_size) == 1

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.scales, self.biases))


def _weight_rows(weight: torch.Tensor):
    if weight.ndim == 2:
        c_out, c_in = (int(v) for v in weight.shape)
        return weight, 'linear', (1, 1, 1), c_in, c_out
    if weight.ndim == 3:
        k, c_in, c_out = (int(v) for v in weight.shape)
        return weight.permute(0, 2, 1).reshape(k * c_out, c_in), 'kernel_major', (k, 1, 1), c_in, c_out
    if weight.ndim == 5:
        c_out, kx, ky, kz, c_in = (int(v) for v in weight.shape)
        rows = weight.permute(1, 2, 3, 0, 4).reshape(kx * ky * kz * c_out, c_in)
        return rows, 'dense_5d', (kx, ky, kz), c_in, c_out
    raise ValueError(
        'weight must have shape (C_out, C_in), (K, C_in, C_out), '
        'or (C_out, Kx, Ky, Kz, C_in).'
    )


def quantize_affine(rows: torch.Tensor, group_size: int, bits: int):
    """Per-group affine codes of a (R, S) float32 matrix: ``n = 2^bits - 1``, scale
    ``max((max-min)/n, 1e-7)`` signed towards the larger-magnitude edge, the edge
    snapped to a multiple of the scale and used as bias, codes
    ``clip(round((w - bias)/scale), 0, n)``. Returns (codes int64, scales, biases)."""
    r, s = rows.shape
    g = rows.reshape(r, s // group_size, group_size)
    n_bins = float((1 << bits) - 1)
    w_max, w_min = g.amax(dim=2), g.amin(dim=2)
    mask = w_min.abs() > w_max.abs()
    scales = torch.clamp((w_max - w_min) / n_bins, min=1e-7)
    scales = torch.where(mask, scales, -scales)
    edge = torch.where(mask, w_min, w_max)
    q0 = torch.round(edge / scales)
    safe_q0 = torch.where(q0 == 0, torch.ones_like(q0), q0)
    scales = torch.where(q0 != 0, edge / safe_q0, scales)
    biases = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    codes = torch.round((g - biases[:, :, None]) / scales[:, :, None])
    codes = codes.clamp(0, n_bins).to(torch.int64).reshape(r, s)
    return codes, scales, biases


def _pack(codes: torch.Tensor, bits: int) -> torch.Tensor:
    r, s = codes.shape
    per = 32 // bits
    shifts = torch.arange(per, device=codes.device, dtype=torch.int64) * bits
    words = (codes.reshape(r, s // per, per) << shifts).sum(dim=2)
    # keep the low 32 bits; stored as int32 (bit pattern of the uint32 word)
    words = torch.where(words >= (1 << 31), words - (1 << 32), words)
    return words.to(torch.int32)


def quantize_weight(
    weight: torch.Tensor, *, group_size: int | None = None, bits: int = 4
) -> QuantizedWeight:
    """Pack a linear or sparse-convolution weight (``quantized.py:124-187``).
    ``group_size=None`` chooses 64 for ``C_in >= 64`` and 32 otherwise."""
    if weight.dtype not in (torch.float16, torch.float32):
        raise ValueError('weight quantization supports float16 and float32.')
    if bits not in (4, 8):
        raise ValueError('weight quantization supports only 4 or 8 bits.')
    rows, layout, kernel_size, c_in, c_out = _weight_rows(weight)
    if group_size is None:
        group_size = 64 if c_in >= 64 else 32
    elif group_size not in (32, 64, 128):
        raise ValueError('group_size must be 32, 64, or 128.')
    storage = -(-c_in // group_size) * group_size
    rows32 = rows.to(torch.float32)
    if storage != c_in:
        rows32 = torch.nn.functional.pad(rows32, (0, storage - c_in))
    codes, scales, biases = quantize_affine(rows32.contiguous(), group_size, bits)
    kernel_rows = _volume(kernel_size)
    packed = _pack(codes, bits).reshape(kernel_rows, c_out, -1)
    scales = scales.to(weight.dtype).reshape(kernel_rows, c_out, -1)
    biases = biases.to(weight.dtype).reshape(kernel_rows, c_out, -1)
    if kernel_rows > 1:
        packed = packed.permute(0, 2, 1).contiguous()
        scales = scales.permute(0, 2, 1).contiguous()
        biases = biases.permute(0, 2, 1).contiguous()
    return QuantizedWeight(
        weight=packed, scales=scales, biases=biases, group_size=group_size, bits=bits,
        in_channels=c_in, out_channels=c_out, kernel_size=kernel_size, layout=layout,
    )


def dequantize_weight(weight: QuantizedWeight) -> torch.Tensor:
    """Logical float weight in the layout recorded by ``weight.layout``
    (``quantized.py:190-223``); padded storage channels are sliced away."""
    kernel_rows = _volume(weight.kernel_size)
    packed, scales, biases = weight.weight, weight.scales, weight.biases
    if not weight.is_pointwise:
        packed, scales, biases = (t.permute(0, 2, 1) for t in (packed, scales, biases))
    rows = kernel_rows * weight.out_channels
    words = packed.reshape(rows, -1).to(torch.int64) & 0xFFFFFFFF
    per = 32 // weight.bits
    shifts = torch.arange(per, device=words.device, dtype=torch.int64) * weight.bits
    codes = ((words[:, :, None] >> shifts) & ((1 << weight.bits) - 1)).reshape(rows, -1)
    s = scales.reshape(rows, -1).to(torch.float32).repeat_interleave(weight.group_size, dim=1)
    b = biases.reshape(rows, -1).to(torch.float32).repeat_interleave(weight.group_size, dim=1)
    values = (codes.to(torch.float32) * s + b)[:, : weight.in_channels].to(scales.dtype)
    if weight.layout == 'linear':
        return values.reshape(weight.out_channels, weight.in_channels)
    mapped = values.reshape(kernel_rows, weight.out_channels, weight.in_channels)
    if weight.layout == 'kernel_major':
        return mapped.permute(0, 2, 1).contiguous()
    return mapped.reshape(
        *weight.kernel_size, weight.out_channels, weight.in_channels
    ).permute(3, 0, 1, 2, 4).contiguous()
