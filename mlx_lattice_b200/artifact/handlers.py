"""Run-time pieces of the artifact graph: the execution context that resolves value
names and weight names, IR value types against Python types, the dtype policy, and the
two operations that need more than a call of the bound function.

Follows ``mlx_lattice/artifact/bindings.py:150-300`` (context, quantised payloads, dtype
policy, value-type table) and ``mlx_lattice/artifact/ops.py:371-425`` (global pooling of a
tensor that lost its ``batch_counts``).
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.artifact.manifest import IRNode
from mlx_lattice_b200.core import QuantizedWeight, SparseTensor
from mlx_lattice_b200.core.coords.alignment import SparseAlignment
from mlx_lattice_b200.core.coords.quantization import PointVoxelMap, SparseQuantization
from mlx_lattice_b200.core.relations import KernelRelation

QUANTIZED_SUFFIXES = ('weight', 'scales', 'biases', 'attrs')
_LAYOUTS = ('linear', 'kernel_major', 'dense_5d')          # layout id = position

# IR value type -> (Python type, label used in error texts, structural fields)
_VALUE_TYPES: dict[str, tuple[Any, str, dict[str, str]]] = {
    'any': (object, 'object', {}),
    'sparse_tensor': (SparseTensor, 'SparseTensor', {}),
    'dense_tensor': (torch.Tensor, 'a dense tensor', {}),
    'relation': (KernelRelation, 'KernelRelation', {}),
    'alignment': (SparseAlignment, 'SparseAlignment', {
        'coords': 'dense_tensor', 'active_rows': 'dense_tensor',
        'lhs_rows': 'dense_tensor', 'rhs_rows': 'dense_tensor'}),
    'quantization': (SparseQuantization, 'SparseQuantization', {
        'coords': 'dense_tensor', 'active_rows': 'dense_tensor',
        'inverse_rows': 'dense_tensor', 'counts': 'dense_tensor'}),
    'point_voxel_map': (PointVoxelMap, 'PointVoxelMap', {
        'rows': 'dense_tensor', 'weights': 'dense_tensor'}),
    'bytes': (bytes, 'bytes', {}),
}


def layout_id(layout: str) -> int:
    if layout not in _LAYOUTS:
        raise ValueError(f'unknown quantized weight layout: {layout!r}.')
    return _LAYOUTS.index(layout)


def validate_value_type(name: str, expected: str, value: Any) -> None:
    if expected not in _VALUE_TYPES:
        raise ValueError(f'unsupported IR value type: {expected!r}.')
    python_type, label, _ = _VALUE_TYPES[expected]
    if python_type is not object and not isinstance(value, python_type):
        raise ValueError(f'graph value {name!r} must be {label}.')


def field_value(value: Any, field: Any, node_id: str = 'value.field') -> Any:
    """``value.field``: a public structural field of a typed graph value."""
    if not isinstance(field, str):
        raise ValueError(f'{node_id}.attributes.field must be a string.')
    for python_type, _, fields in _VALUE_TYPES.values():
        if fields and isinstance(value, python_type) and field in fields:
            return getattr(value, field)
    raise ValueError(f'field {field!r} is not supported for {type(value).__name__}.')


def _cast(value: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return value.to(dtype) if value.dtype in (torch.float16, torch.float32) else value


def apply_dtype_policy(value: Any, policy: str) -> Any:
    """``preserve`` keeps dtypes; ``fp32`` / ``fp16`` / ``fp16_inference`` cast float16 and
    float32 features and dense tensors (``bindings.py:246-262``)."""
    if policy == 'preserve':
        return value
    if policy not in ('fp32', 'fp16', 'fp16_inference'):
        raise ValueError(f'unsupported dtype policy: {policy!r}.')
    dtype = torch.float32 if policy == 'fp32' else torch.float16
    if isinstance(value, SparseTensor):
        return value if value.feats.dtype == dtype else value.replace(feats=_cast(value.feats, dtype))
    if isinstance(value, torch.Tensor):
        return _cast(value, dtype)
    return value


def quantized_payload_names(weights: Mapping[str, torch.Tensor]) -> set[str]:
    """Names of the tensors that belong to complete packed-weight payloads."""
    names: set[str] = set()
    for name in weights:
        if name.endswith('.attrs'):
            prefix = name[: -len('.attrs')]
            if all(f'{prefix}.{suffix}' in weights for suffix in QUANTIZED_SUFFIXES):
                names.update(f'{prefix}.{suffix}' for suffix in QUANTIZED_SUFFIXES)
    return names


@dataclass(slots=True)
class ExecutionContext:
    values: dict[str, Any]
    weights: Mapping[str, torch.Tensor]
    quantized: dict[str, QuantizedWeight]
    batch_size: int | None = None

    def value(self, name: str) -> Any:
        if name not in self.values:
            raise ValueError(f'missing graph value {name!r}.')
        return self.values[name]

    def input_value(self, ref: str | tuple[str, ...], *, sequence: bool = False) -> Any:
        if isinstance(ref, str):
            value = self.value(ref)
            return (value,) if sequence else value
        values = tuple(self.value(name) for name in ref)
        if sequence:
            return values
        if len(values) != 1:
            raise ValueError('expected a single graph value reference.')
        return values[0]

    def array(self, name: str) -> torch.Tensor:
        if name not in self.weights:
            raise ValueError(f'missing lattice weight {name!r}.')
        return self.weights[name]

    def parameter(self, name: str, kind: str) -> Any:
        if kind == 'optional_array':
            return None if name == '' else self.array(name)
        if kind == 'quantized_weight' or (
            kind == 'array_or_quantized_weight' and f'{name}.attrs' in self.weights
        ):
            return self.quantized_weight(name)
        return self.array(name)

    def quantized_weight(self, prefix: str) -> QuantizedWeight:
        if prefix not in self.quantized:
            self.quantized[prefix] = decode_quantized_weight(prefix, self.weights)
        return self.quantized[prefix]


def decode_quantized_weight(prefix: str, weights: Mapping[str, torch.Tensor]) -> QuantizedWeight:
    """The four tensors ``<prefix>.weight/.scales/.biases/.attrs`` as a ``QuantizedWeight``;
    ``attrs`` = int32 ``[layout id, group_size, bits, C_in, C_out, kx, ky, kz]``
    (written by ``mlx_lattice/artifact/builder.py:307-330``)."""
    for suffix in QUANTIZED_SUFFIXES:
        if f'{prefix}.{suffix}' not in weights:
            raise ValueError(f'missing lattice weight {prefix}.{suffix!r}.')
    attrs = weights[f'{prefix}.attrs']
    if attrs.ndim != 1:
        raise ValueError(f'quantized parameter {prefix!r} metadata must be a vector.')
    raw = [int(v) for v in attrs.tolist()]
    if len(raw) != 8:
        raise ValueError(f'quantized parameter {prefix!r} has invalid metadata.')
    layout, group_size, bits, c_in, c_out, kx, ky, kz = raw
    if not 0 <= layout < len(_LAYOUTS):
        raise ValueError(f'unknown quantized weight layout id: {layout}.')
    return QuantizedWeight(
        weights[f'{prefix}.weight'], weights[f'{prefix}.scales'], weights[f'{prefix}.biases'],
        group_size, bits, c_in, c_out, (kx, ky, kz), _LAYOUTS[layout],
    )


def infer_batch_size(values: Mapping[str, Any]) -> int | None:
    for value in values.values():
        if isinstance(value, SparseTensor) and value.batch_counts is not None:
            return len(value.batch_counts)
    return None


def _pool_by_batch_column(x: SparseTensor, batch_size: int, mode: str) -> torch.Tensor:
    """Per-batch sum / mean of a tensor without ``batch_counts``: rows are grouped by their
    batch column (stable, so sums run in row order), inactive rows fall into a spare group,
    and the grouped rows go through the library's segmented pooling kernel."""
    if batch_size <= 0:
        raise ValueError('batch_size must be positive.')
    rows = torch.arange(x.coords.shape[0], device=x.coords.device)
    batch = x.coords[:, 0].long().clamp(0, batch_size - 1)
    batch = torch.where(rows < x.active_rows[0], batch, torch.full_like(batch, batch_size))
    order = torch.argsort(batch, stable=True)
    counts = torch.bincount(batch, minlength=batch_size + 1)[:batch_size]
    offsets = torch.zeros(batch_size + 1, dtype=torch.int32, device=x.coords.device)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return _ext.global_pool(x.feats[order].contiguous(), offsets, mode)


def global_pool_handler(context: ExecutionContext, node: IRNode, binding) -> dict[str, Any]:
    """``pool.global_*``: the bound function when the tensor carries ``batch_counts`` (always
    for max), else pooling by batch column with the batch size of the graph inputs."""
    ref = node.inputs['input']
    if not isinstance(ref, str):
        raise ValueError('expected a single graph value reference.')
    x = context.value(ref)
    if not isinstance(x, SparseTensor):
        raise ValueError(f'graph value {ref!r} is not a SparseTensor.')
    if x.batch_counts is not None or node.op == 'pool.global_max':
        return {'output': binding.function(x)}
    if context.batch_size is None:
        raise ValueError(
            f'{node.id} requires batch_counts metadata or a sparse graph '
            'input with known batch_counts.'
        )
    if x.feats.dtype != torch.float32:
        raise ValueError('pooling currently supports float32 tensors.')
    return {'output': _pool_by_batch_column(x, context.batch_size, node.op.removeprefix('pool.global_'))}
