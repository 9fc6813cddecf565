"""The lattice IR manifest: the JSON half of a model artifact.

Mirrors the reference's stable artifact contract (``contract/lattice_contract/
manifest.py:9-210``): schema version ``0.1``, coordinate order ``batch, x, y, z``,
row-major features, the ``mlx-lattice`` weight layout, four dtype policies, typed
graph inputs/outputs and a topologically ordered node list. A node's ``support``
object is folded into its attributes the way the reference does
(``manifest.py:258-271``): ``target`` becomes the ``coordinates`` attribute.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

CURRENT_SCHEMA_VERSION = '0.1'

IR_VALUE_TYPES = (
    'any', 'sparse_tensor', 'dense_tensor', 'relation', 'coordinate_set', 'alignment',
    'quantization', 'point_voxel_map', 'coordinate_ordering', 'sparse_occupancy',
    'occupancy_expansion', 'bytes',
)
DTYPE_POLICIES = ('preserve', 'fp32', 'fp16', 'fp16_inference')
COORDINATE_ORDER = ('batch', 'x', 'y', 'z')
FEATURE_LAYOUT = ('row', 'channel')
WEIGHT_LAYOUT = 'mlx-lattice'

_SUPPORT_TRIPLES = ('kernel_size', 'stride', 'padding', 'dilation')
_SUPPORT_STRINGS = ('target', 'mode', 'join')
# support field -> attribute name it turns into
_SUPPORT_ATTRIBUTE = {'target': 'coordinates'}


@dataclass(frozen=True, slots=True)
class IRSparseSupport:
    kind: str
    kernel_size: tuple[int, int, int] | None = None
    stride: tuple[int, int, int] | None = None
    padding: tuple[int, int, int] | None = None
    dilation: tuple[int, int, int] | None = None
    target: str | None = None
    mode: str | None = None
    join: str | None = None


@dataclass(frozen=True, slots=True)
class IRTensorSpec:
    name: str
    type: str


@dataclass(frozen=True, slots=True)
class IRNode:
    id: str
    op: str
    inputs: dict[str, str | tuple[str, ...]]
    outputs: dict[str, str]
    parameters: dict[str, str] = field(default_factory=dict)
    attributes: dict[str, Any] = field(default_factory=dict)
    support: IRSparseSupport | None = None


@dataclass(frozen=True, slots=True)
class IRManifest:
    schema_version: str
    producer: dict[str, str]
    runtime: dict[str, str]
    inputs: tuple[IRTensorSpec, ...]
    outputs: tuple[IRTensorSpec, ...]
    nodes: tuple[IRNode, ...]
    dtype_policy: str = 'preserve'
    coordinate_order: tuple[str, ...] = COORDINATE_ORDER
    feature_layout: tuple[str, ...] = FEATURE_LAYOUT
    weight_layout: str = WEIGHT_LAYOUT


def value_refs(ref: str | tuple[str, ...]) -> tuple[str, ...]:
    return (ref,) if isinstance(ref, str) else tuple(ref)


class _Object:
    """A decoded JSON object together with its path, for error texts."""

    def __init__(self, raw: Any, path: str) -> None:
        if not isinstance(raw, Mapping):
            raise ValueError(f'{path} must be an object.')
        self.raw, self.path = raw, path

    def _where(self, name: str) -> str:
        return name if self.path in ('', 'manifest') else f'{self.path}.{name}'

    def string(self, name: str, default: str | None = None) -> str:
        value = self.raw.get(name, default)
        if not isinstance(value, str):
            raise ValueError(f'{self._where(name)} must be a string.')
        return value

    def optional_string(self, name: str) -> str | None:
        return self.string(name) if name in self.raw else None

    def items(self, name: str) -> list:
        value = self.raw.get(name)
        if not isinstance(value, list):
            raise ValueError(f'{name} must be a list.')
        return value

    def strings(self, name: str, default: tuple[str, ...]) -> tuple[str, ...]:
        value = self.raw.get(name, default)
        if not isinstance(value, (list, tuple)) or not all(isinstance(v, str) for v in value):
            raise ValueError(f'{name} must be a list of strings.')
        return tuple(value)

    def string_map(self, name: str) -> dict[str, str]:
        child = _Object(self.raw.get(name, {}), self._where(name))
        for key, value in child.raw.items():
            if not isinstance(key, str) or not isinstance(value, str):
                raise ValueError(f'{child.path} must map strings to strings.')
        return dict(child.raw)

    def optional_triple(self, name: str) -> tuple[int, int, int] | None:
        if name not in self.raw:
            return None
        value = self.raw[name]
        if isinstance(value, bool):
            value = None
        if isinstance(value, int):
            return (value, value, value)
        if not isinstance(value, (list, tuple)) or len(value) != 3:
            raise ValueError(f'{self._where(name)} must be an int or a sequence of 3 ints.')
        return (int(value[0]), int(value[1]), int(value[2]))


def _tensor_spec(raw: Any, path: str) -> IRTensorSpec:
    data = _Object(raw, path)
    name, value_type = data.string('name'), data.string('type')
    if value_type not in IR_VALUE_TYPES:
        raise ValueError(f'{path}.type is not a supported lattice IR value type.')
    return IRTensorSpec(name, value_type)


def _support(raw: Any, path: str) -> IRSparseSupport:
    data = _Object(raw, path)
    fields: dict[str, Any] = {'kind': data.string('kind')}
    for name in _SUPPORT_TRIPLES:
        fields[name] = data.optional_triple(name)
    for name in _SUPPORT_STRINGS:
        fields[name] = data.optional_string(name)
    return IRSparseSupport(**fields)


def _node(raw: Any, path: str) -> IRNode:
    data = _Object(raw, path)
    attributes = dict(_Object(data.raw.get('attributes', {}), f'{path}.attributes').raw)
    support = _support(data.raw['support'], f'{path}.support') if 'support' in data.raw else None
    if support is not None:
        for name in _SUPPORT_TRIPLES + _SUPPORT_STRINGS:
            value = getattr(support, name)
            if value is not None:
                attributes[_SUPPORT_ATTRIBUTE.get(name, name)] = value
    inputs: dict[str, str | tuple[str, ...]] = {}
    for port, ref in _Object(data.raw.get('inputs', {}), f'{path}.inputs').raw.items():
        if not isinstance(port, str):
            raise ValueError(f'{path}.inputs must map strings to value refs.')
        if isinstance(ref, str):
            inputs[port] = ref
        elif isinstance(ref, (list, tuple)) and all(isinstance(item, str) for item in ref):
            inputs[port] = tuple(ref)
        else:
            raise ValueError(f'{path}.inputs.{port} must be a string or list of strings.')
    return IRNode(
        id=data.string('id'),
        op=data.string('op'),
        inputs=inputs,
        outputs=data.string_map('outputs'),
        parameters=data.string_map('parameters'),
        attributes=attributes,
        support=support,
    )


def _check_graph(manifest: IRManifest) -> None:
    """Every value is defined once, before its first use (``manifest.py:325-347``)."""
    values: set[str] = set()
    node_ids: set[str] = set()

    def define(seen: set[str], name: str, label: str) -> None:
        if name in seen:
            raise ValueError(f'duplicate {label}: {name!r}.')
        seen.add(name)

    for spec in manifest.inputs:
        define(values, spec.name, 'graph value')
    for node in manifest.nodes:
        define(node_ids, node.id, 'node id')
        if not node.outputs:
            raise ValueError(f'node {node.id!r} must define outputs.')
        for ref in node.inputs.values():
            for name in value_refs(ref):
                if name not in values:
                    raise ValueError(f'node {node.id!r} references unknown input {name!r}.')
        for name in node.outputs.values():
            define(values, name, 'graph value')
    for spec in manifest.outputs:
        if spec.name not in values:
            raise ValueError(f'unknown manifest output {spec.name!r}.')


def manifest_from_dict(raw: Mapping[str, Any]) -> IRManifest:
    """Validated manifest from decoded JSON (``manifest.py:118-181``)."""
    data = _Object(raw, 'manifest')
    schema_version = data.string('schema_version')
    if schema_version != CURRENT_SCHEMA_VERSION:
        raise ValueError(
            f'unsupported lattice IR schema_version {schema_version!r}; '
            f'expected {CURRENT_SCHEMA_VERSION!r}.'
        )
    coordinate_order = data.strings('coordinate_order', COORDINATE_ORDER)
    if coordinate_order != COORDINATE_ORDER:
        raise ValueError("coordinate_order must be ['batch', 'x', 'y', 'z'].")
    feature_layout = data.strings('feature_layout', FEATURE_LAYOUT)
    if feature_layout != FEATURE_LAYOUT:
        raise ValueError("feature_layout must be ['row', 'channel'].")
    weight_layout = data.string('weight_layout', WEIGHT_LAYOUT)
    if weight_layout != WEIGHT_LAYOUT:
        raise ValueError("weight_layout must be 'mlx-lattice'.")
    dtype_policy = data.string('dtype_policy', 'preserve')
    if dtype_policy not in DTYPE_POLICIES:
        raise ValueError('dtype_policy must be preserve, fp32, fp16, or fp16_inference.')
    manifest = IRManifest(
        schema_version=schema_version,
        producer=data.string_map('producer'),
        runtime=data.string_map('runtime'),
        inputs=tuple(_tensor_spec(v, f'inputs[{i}]') for i, v in enumerate(data.items('inputs'))),
        outputs=tuple(_tensor_spec(v, f'outputs[{i}]') for i, v in enumerate(data.items('outputs'))),
        nodes=tuple(_node(v, f'nodes[{i}]') for i, v in enumerate(data.items('nodes'))),
        dtype_policy=dtype_policy,
        coordinate_order=coordinate_order,
        feature_layout=feature_layout,
        weight_layout=weight_layout,
    )
    _check_graph(manifest)
    return manifest


def load_manifest(path: str | Path) -> IRManifest:
    with Path(path).open('r', encoding='utf-8') as file:
        return manifest_from_dict(json.load(file))


def _jsonable(value: Any) -> Any:
    if isinstance(value, tuple):
        return [_jsonable(item) for item in value]
    if isinstance(value, list):
        return [_jsonable(item) for item in value]
    if isinstance(value, dict):
        return {key: _jsonable(item) for key, item in value.items()}
    return value


def manifest_to_dict(manifest: IRManifest) -> dict[str, Any]:
    """JSON-serialisable form (``manifest.py:184-210``); loading it again gives an equal
    manifest (support-derived attributes are written in both places, as the reference does)."""
    nodes = []
    for node in manifest.nodes:
        raw: dict[str, Any] = {
            'id': node.id,
            'op': node.op,
            'inputs': {k: v if isinstance(v, str) else list(v) for k, v in node.inputs.items()},
            'outputs': dict(node.outputs),
        }
        if node.parameters:
            raw['parameters'] = dict(node.parameters)
        if node.attributes:
            raw['attributes'] = _jsonable(dict(node.attributes))
        if node.support is not None:
            support: dict[str, Any] = {'kind': node.support.kind}
            for name in _SUPPORT_TRIPLES:
                if getattr(node.support, name) is not None:
                    support[name] = list(getattr(node.support, name))
            for name in _SUPPORT_STRINGS:
                if getattr(node.support, name) is not None:
                    support[name] = getattr(node.support, name)
            raw['support'] = support
        nodes.append(raw)
    return {
        'schema_version': manifest.schema_version,
        'producer': dict(manifest.producer),
        'runtime': dict(manifest.runtime),
        'coordinate_order': list(manifest.coordinate_order),
        'feature_layout': list(manifest.feature_layout),
        'weight_layout': manifest.weight_layout,
        'dtype_policy': manifest.dtype_policy,
        'inputs': [{'name': s.name, 'type': s.type} for s in manifest.inputs],
        'outputs': [{'name': s.name, 'type': s.type} for s in manifest.outputs],
        'nodes': nodes,
    }
