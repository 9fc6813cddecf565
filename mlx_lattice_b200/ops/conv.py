"""Sparse convolution operators (``mlx_lattice/ops/conv.py:34-211``)."""

from __future__ import annotations

from collections.abc import Sequence

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core import (
    CoordinateMapKey,
    KernelSpec,
    QuantizedWeight,
    SparseTensor,
)
from mlx_lattice_b200.core.types import Triple
from mlx_lattice_b200.ops._quantized import quantized_matmul
from mlx_lattice_b200.ops._relation_exec import (
    sparse_conv_features_from_relation,
    sparse_quantized_conv_features_from_relation,
)

__all__ = ['conv3d', 'conv_transpose3d', 'generative_conv_transpose3d', 'subm_conv3d']


def conv3d(
    x: SparseTensor,
    weight: torch.Tensor | QuantizedWeight,
    bias: torch.Tensor | None = None,
    *,
    kernel_size: int | Sequence[int] = 3,
    stride: int | Sequence[int] = 1,
    padding: int | Sequence[int] = 0,
    dilation: int | Sequence[int] = 1,
    coordinates: SparseTensor | CoordinateMapKey | torch.Tensor | None = None,
) -> SparseTensor:
    """Sparse 3D convolution. The pointwise case without explicit target
    coordinates is a feature matrix multiply that keeps the input coordinates;
    other shapes build (or reuse) a kernel relation. ``coordinates`` fixes the
    output support (``ops/conv.py:34-110``)."""
    spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
    output_stride = _mul_stride(x.stride, spec.stride)
    if coordinates is None and spec.is_pointwise:
        return x.replace(feats=_pointwise_features(x, weight, bias))
    if coordinates is not None:
        target_key = _target_key(x, coordinates, output_stride)
        reuse_input = target_key == x.coord_key
        return _relation_conv(
            x, _target_weight(weight, spec), bias, spec,
            map_kind='forward' if reuse_input else 'target',
            output_stride=target_key.stride,
            reuse_input_coords=reuse_input,
            target_key=target_key,
        )
    return _relation_conv(x, weight, bias, spec, map_kind='forward', output_stride=output_stride)


def subm_conv3d(
    x: SparseTensor,
    weight: torch.Tensor | QuantizedWeight,
    bias: torch.Tensor | None = None,
    *,
    kernel_size: int | Sequence[int] = 3,
    dilation: int | Sequence[int] = 1,
) -> SparseTensor:
    """Submanifold convolution: odd kernel, stride 1, output support = input
    support, coordinate identity preserved (``ops/conv.py:112-146``)."""
    spec = KernelSpec(size=kernel_size, stride=1, padding=0, dilation=dilation)
    if any(value % 2 == 0 for value in spec.size):
        raise ValueError('subm_conv3d requires odd kernel_size values.')
    if spec.size == (1, 1, 1) and spec.dilation == (1, 1, 1):
        return x.replace(feats=_pointwise_features(x, weight, bias))
    return _relation_conv(
        x, weight, bias, spec, map_kind='submanifold', output_stride=x.stride,
        reuse_input_coords=True,
    )


def conv_transpose3d(
    x: SparseTensor,
    weight: torch.Tensor | QuantizedWeight,
    bias: torch.Tensor | None = None,
    *,
    kernel_size: int | Sequence[int] = 2,
    stride: int | Sequence[int] = 2,
    padding: int | Sequence[int] = 0,
    dilation: int | Sequence[int] = 1,
    coordinates: SparseTensor | None = None,
) -> SparseTensor:
    """Sparse transpose convolution (``ops/conv.py:153-182``). The output sparse
    stride is ``x.stride / stride``.

    ``coordinates`` is an addition to the reference signature: a sparse tensor (on
    the output stride, same manager) whose support the output is restricted to.
    The result equals ``sparse_cat_aligned``-style right alignment of the plain
    transposed output to that support, computed without the ``K``-times larger
    intermediate; it needs ``kernel_size == stride``, ``padding == 0``,
    ``dilation == 1`` (every fine cell then has exactly one parent and offset)."""
    spec = KernelSpec(size=kernel_size, stride=stride, padding=padding, dilation=dilation)
    output_stride = _div_stride(x.stride, spec.stride)
    if coordinates is None:
        return _relation_conv(x, weight, bias, spec, map_kind='transposed', output_stride=output_stride)
    if not isinstance(coordinates, SparseTensor):
        raise ValueError('coordinates must be a SparseTensor for transposed convolution.')
    if coordinates.stride != output_stride:
        raise ValueError('target coordinates must use the convolution output stride.')
    if spec.size != spec.stride or spec.padding != (0, 0, 0) or spec.dilation != (1, 1, 1):
        raise ValueError(
            'target-restricted transposed convolution requires kernel_size == stride, '
            'padding == 0 and dilation == 1.'
        )
    if coordinates.coord_manager is x.coord_manager:
        target_key = coordinates.coord_key
    else:
        target_key = x.coord_manager.insert_coords(
            coordinates.coords, coordinates.stride, coordinates.active_rows
        )
    return _relation_conv(
        x, weight, bias, spec, map_kind='target_transposed', output_stride=output_stride,
        target_key=target_key,
    )


def generative_conv_transpose3d(
    x: SparseTensor,
    weight: torch.Tensor | QuantizedWeight,
    bias: torch.Tensor | None = None,
    *,
    kernel_size: int | Sequence[int] = 2,
    stride: int | Sequence[int] = 2,
) -> SparseTensor:
    """Generative transpose convolution (``ops/conv.py:189-211``)."""
    spec = KernelSpec(size=kernel_size, stride=stride)
    return _relation_conv(
        x, weight, bias, spec, map_kind='generative',
        output_stride=_div_stride(x.stride, spec.stride),
    )


# -- execution policy (ops/conv.py:217-262) ------------------------------------


def _relation_conv(
    x: SparseTensor,
    weight,
    bias,
    spec: KernelSpec,
    *,
    map_kind: str,
    output_stride: Triple,
    reuse_input_coords: bool = False,
    target_key: CoordinateMapKey | None = None,
) -> SparseTensor:
    _validate_feature_dtype(x, weight)
    if x.coords.dtype != torch.int32:
        raise ValueError('CUDA sparse convolution requires int32 coordinates.')
    _validate_weight_for_kernel(x, weight, spec.volume)
    _validate_bias(bias, weight, x.dtype)
    relation = _kernel_relation(x, spec, map_kind, target_key=target_key)
    if relation.n_out_capacity is None or relation.n_kernels is None:
        raise ValueError('kernel relation is missing static shape metadata.')
    run = (sparse_quantized_conv_features_from_relation if isinstance(weight, QuantizedWeight)
           else sparse_conv_features_from_relation)
    feats = run(x.feat_parts or x.feats, weight, relation, bias)
    if reuse_input_coords:
        return x.replace(feats=feats)
    if relation.out_coords is None:
        raise ValueError('kernel relation is missing output coordinates.')
    if target_key is not None and map_kind in ('target', 'target_transposed'):
        return SparseTensor(
            x.coord_manager.coords(target_key),
            feats,
            stride=output_stride,
            coord_key=target_key,
            coord_manager=x.coord_manager,
            active_rows=x.coord_manager.active_rows(target_key),
        )
    return SparseTensor(
        relation.out_coords,
        feats,
        stride=output_stride,
        coord_manager=x.coord_manager,
        active_rows=relation.out_count,
    )


def _kernel_relation(x, spec: KernelSpec, map_kind: str, *, target_key=None):
    manager, key = x.coord_manager, x.coord_key
    if map_kind == 'forward':
        return manager.kernel_relation(
            key, kernel_size=spec.size, stride=spec.stride, padding=spec.padding,
            dilation=spec.dilation,
        )
    if map_kind == 'submanifold':
        return manager.submanifold_kernel_relation(
            key, kernel_size=spec.size, dilation=spec.dilation
        )
    if map_kind == 'transposed':
        return manager.transposed_kernel_relation(
            key, kernel_size=spec.size, stride=spec.stride, padding=spec.padding,
            dilation=spec.dilation,
        )
    if map_kind == 'generative':
        return manager.generative_relation(key, kernel_size=spec.size, stride=spec.stride)
    if map_kind == 'target':
        if target_key is None:
            raise ValueError('target_key is required for target relations.')
        return manager.target_kernel_relation(
            key, target_key, kernel_size=spec.size, stride=spec.stride, padding=spec.padding,
            dilation=spec.dilation,
        )
    if map_kind == 'target_transposed':
        if target_key is None:
            raise ValueError('target_key is required for target relations.')
        return manager.target_transposed_relation(key, target_key, stride=spec.stride)
    raise ValueError(
        "map_kind must be 'forward', 'submanifold', 'transposed', "
        "'generative', or 'target'."
    )


def _target_key(x: SparseTensor, coordinates, output_stride: Triple) -> CoordinateMapKey:
    if isinstance(coordinates, SparseTensor):
        if coordinates.stride != output_stride:
            raise ValueError('target coordinates must use the convolution output stride.')
        if coordinates.coord_manager is x.coord_manager:
            return coordinates.coord_key
        return x.coord_manager.insert_coords(
            coordinates.coords, coordinates.stride, coordinates.active_rows
        )
    if isinstance(coordinates, CoordinateMapKey):
        if not x.coord_manager.owns(coordinates):
            raise ValueError('target coordinate key must belong to x.coord_manager.')
        if coordinates.stride != output_stride:
            raise ValueError('target coordinate key must use the convolution output stride.')
        return coordinates
    return x.coord_manager.insert_coords(coordinates, output_stride)


def _pointwise_features(x: SparseTensor, weight, bias) -> torch.Tensor:
    _validate_feature_dtype(x.feats, weight)
    _validate_bias(bias, weight, x.dtype)
    if isinstance(weight, QuantizedWeight):
        return quantized_matmul(x.feats, weight, bias)
    return _ext.linear(x.feats, _pointwise_weight_matrix(x, weight), bias)


def _target_weight(weight, spec: KernelSpec):
    if isinstance(weight, QuantizedWeight):
        return weight
    if not spec.is_pointwise or weight.ndim != 2:
        return weight
    return weight.t().unsqueeze(0).contiguous()


# -- validation (ops/conv.py:372-469) --------------------------------------------


def _validate_feature_dtype(feats: torch.Tensor, weight) -> None:
    if feats.dtype not in (torch.float32, torch.float16):
        raise ValueError('convolution supports float32 and float16 tensors.')
    weight_dtype = weight.scales.dtype if isinstance(weight, QuantizedWeight) else weight.dtype
    if weight_dtype != feats.dtype:
        raise ValueError('convolution weights must match feature dtype.')


def _pointwise_weight_matrix(x: SparseTensor, weight: torch.Tensor) -> torch.Tensor:
    if weight.ndim == 2:
        if weight.shape[1] != x.channels:
            raise ValueError('weight input channels must match x.channels.')
        return weight
    if weight.ndim == 5 and tuple(weight.shape[1:4]) == (1, 1, 1):
        if weight.shape[4] != x.channels:
            raise ValueError('weight input channels must match x.channels.')
        return weight[:, 0, 0, 0, :]
    if weight.ndim == 3 and weight.shape[0] == 1:
        if weight.shape[1] != x.channels:
            raise ValueError('weight input channels must match x.channels.')
        return weight[0].t()
    raise ValueError(
        'pointwise weight must have shape (C_out, C_in), '
        '(C_out, 1, 1, 1, C_in), or (1, C_in, C_out).'
    )


def _validate_weight_for_kernel(x: SparseTensor, weight, kernel_rows: int) -> None:
    if isinstance(weight, QuantizedWeight):
        if weight.in_channels != x.channels:
            raise ValueError('quantized weight input channels must match x.channels.')
        if weight.kernel_size[0] * weight.kernel_size[1] * weight.kernel_size[2] != kernel_rows:
            raise ValueError('quantized weight kernel rows must match the convolution kernel.')
        return
    if weight.ndim == 3:
        if weight.shape[1] != x.channels:
            raise ValueError('weight input channels must match x.channels.')
        if weight.shape[0] != kernel_rows:
            raise ValueError('weight kernel rows must match the convolution kernel.')
        return
    if weight.ndim != 5:
        raise ValueError(
            'mapped convolution weight must have shape (K, C_in, C_out) '
            'or (C_out, Kx, Ky, Kz, C_in).'
        )
    if weight.shape[4] != x.channels:
        raise ValueError('weight input channels must match x.channels.')
    if int(weight.shape[1] * weight.shape[2] * weight.shape[3]) != kernel_rows:
        raise ValueError('weight kernel rows must match the convolution kernel.')


def _validate_bias(bias, weight, dtype) -> None:
    if bias is None:
        return
    if bias.ndim != 1:
        raise ValueError('bias must have shape (C_out,).')
    if isinstance(weight, QuantizedWeight):
        c_out = weight.out_channels
    elif weight.ndim == 3:
        c_out = int(weight.shape[2])
    else:
        c_out = int(weight.shape[0])
    if bias.shape[0] != c_out:
        raise ValueError('bias channels must match output channels.')
    if bias.dtype != dtype:
        raise ValueError('bias dtype must match output features.')


def _mul_stride(lhs: Triple, rhs: Triple) -> Triple:
    return (lhs[0] * rhs[0], lhs[1] * rhs[1], lhs[2] * rhs[2])


def _div_stride(lhs: Triple, rhs: Triple) -> Triple:
    out = []
    for left, right in zip(lhs, rhs, strict=True):
        if left % right != 0:
            raise ValueError('transpose stride must divide the input tensor stride.')
        out.append(left // right)
    return (out[0], out[1], out[2])
