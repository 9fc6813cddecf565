"""``LatticeModel``: an executable graph loaded from a lattice artifact.

No generated code runs: every node is checked against the operation table and then
dispatched through the public ``mlx_lattice_b200.ops`` surface, as the reference's model
does through ``mlx_lattice.ops`` (``mlx_lattice/artifact/model.py:29-68``). Construction
validates the whole manifest statically (ports, parameter names, attribute names, value
types, weights present); a call validates every node's outputs against its declared type.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

import torch

from mlx_lattice_b200.artifact.handlers import (
    QUANTIZED_SUFFIXES, ExecutionContext, apply_dtype_policy, decode_quantized_weight,
    infer_batch_size, quantized_payload_names, validate_value_type,
)
from mlx_lattice_b200.artifact.manifest import IRManifest, IRNode, value_refs
from mlx_lattice_b200.artifact.registry import OperationBinding, node_inputs, validate_node

# the version of the reference's public interface this package mirrors; a manifest's
# ``runtime.version`` specifier is evaluated against it
REFERENCE_RUNTIME_VERSION = '0.2.1'
_RUNTIME_NAME = 'mlx-lattice'
_COMPARISONS = ('>=', '<=', '==', '!=', '>', '<')      # two-character operators first


def _version_tuple(text: str) -> tuple[int, ...]:
    numbers = []
    for part in text.split('.'):
        digits = ''
        for char in part:
            if not char.isdigit():
                break
            digits += char
        if not digits:
            break
        numbers.append(int(digits))
    if not numbers:
        raise ValueError(f'unsupported runtime version value: {text!r}.')
    return tuple(numbers)


def version_satisfies(version: str, specifier: str) -> bool:
    """Comma-separated ``>= <= == != > <`` clauses, compared as zero-padded integer tuples
    (``model.py:158-226``); a bare version means equality."""
    have = _version_tuple(version)
    for clause in (item.strip() for item in specifier.split(',')):
        if not clause:
            continue
        operator = next((op for op in _COMPARISONS if clause.startswith(op)), None)
        wanted = clause[len(operator):].strip() if operator else clause
        if operator is None and clause[0].isdigit():
            operator = '=='
        if operator is None or not wanted:
            raise ValueError(f'unsupported runtime version specifier: {clause!r}.')
        want = _version_tuple(wanted)
        width = max(len(have), len(want))
        left = have + (0,) * (width - len(have))
        right = want + (0,) * (width - len(want))
        holds = {
            '==': left == right, '!=': left != right, '>=': left >= right,
            '>': left > right, '<=': left <= right, '<': left < right,
        }[operator]
        if not holds:
            return False
    return True


def _check_runtime(manifest: IRManifest) -> None:
    name = manifest.runtime.get('name')
    if name not in (None, '', _RUNTIME_NAME):
        raise ValueError(f"manifest runtime.name must be 'mlx-lattice', got {name!r}.")
    specifier = manifest.runtime.get('version')
    if specifier in (None, ''):
        return
    if not version_satisfies(REFERENCE_RUNTIME_VERSION, specifier):
        raise ValueError(
            f'manifest runtime.version {specifier!r} is not compatible '
            f'with mlx-lattice runtime {REFERENCE_RUNTIME_VERSION!r}.'
        )


def _check_types(node_id: str, path: str, value_name: str, expected: str, actual: str) -> None:
    if expected == 'any' or actual == 'any' or expected == actual:
        return
    raise ValueError(
        f'{node_id}.{path} expects {expected!r} but graph value {value_name!r} has type {actual!r}.'
    )


def _check_weight(node_id: str, name: str, kind: str, weights: Mapping[str, torch.Tensor]) -> None:
    if kind in ('quantized_weight', 'array_or_quantized_weight'):
        keys = [f'{name}.{suffix}' for suffix in QUANTIZED_SUFFIXES]
        if all(key in weights for key in keys):
            return
        if kind == 'quantized_weight':
            missing = [key for key in keys if key not in weights]
            raise ValueError(f'{node_id}.parameters has missing quantized weight tensors: {missing}.')
    if name not in weights:
        raise ValueError(f'{node_id}.parameters missing weight {name!r}.')


def _check_manifest(manifest: IRManifest, weights: Mapping[str, torch.Tensor]) -> list[OperationBinding]:
    types = {spec.name: spec.type for spec in manifest.inputs}
    bindings = []
    for node in manifest.nodes:
        binding = validate_node(node)
        bindings.append(binding)
        for port, ref in node_inputs(binding, node).items():
            for value_name in value_refs(ref):
                if value_name in types:
                    _check_types(node.id, f'inputs.{port}', value_name,
                                 binding.input_types.get(port, 'any'), types[value_name])
        for name in binding.value_attributes:
            if name in node.attributes:
                ref = node.attributes[name]
                if ref not in types:
                    raise ValueError(
                        f'{node.id}.attributes.{name} references unknown graph value {ref!r}.'
                    )
                _check_types(node.id, f'attributes.{name}', ref,
                             binding.value_attribute_types.get(name, 'any'), types[ref])
        for name, weight_name in node.parameters.items():
            _check_weight(node.id, weight_name, binding.parameter(name).kind, weights)
        for port, value_name in node.outputs.items():
            types[value_name] = binding.output_types.get(port, 'any')
    for spec in manifest.outputs:
        if spec.name not in types:
            raise ValueError(f'unknown manifest output {spec.name!r}.')
        _check_types('manifest', f'outputs.{spec.name}', spec.name, spec.type, types[spec.name])
    return bindings


def _arguments(binding: OperationBinding, context: ExecutionContext, node: IRNode) -> dict[str, Any]:
    kwargs: dict[str, Any] = {}
    inputs = node_inputs(binding, node)
    for port, argument in binding.inputs.items():
        kwargs[argument] = context.input_value(
            inputs[port], sequence=port in binding.sequence_inputs
        )
    for name, weight_name in node.parameters.items():
        item = binding.parameter(name)
        kwargs[item.argument] = context.parameter(weight_name, item.kind)
    for name, argument in binding.attributes.items():
        if name in node.attributes:
            kwargs[argument] = node.attributes[name]
    for name, argument in binding.value_attributes.items():
        if name in node.attributes:
            kwargs[argument] = context.value(node.attributes[name])
    return kwargs


class LatticeModel:
    """Executable in-memory graph of a lattice artifact (``model.py:29-68``).

    ``weights`` maps artifact names to tensors; packed payloads (``<name>.weight``,
    ``.scales``, ``.biases``, ``.attrs``) keep their dtypes under every dtype policy, other
    float tensors follow the policy. Weights stay where they are unless ``device`` is given
    (or ``to`` is called): then they move there once; the metadata vectors stay on the host.
    """

    def __init__(self, manifest: IRManifest, weights: Mapping[str, torch.Tensor],
                 device: torch.device | str | None = None) -> None:
        _check_runtime(manifest)
        packed = quantized_payload_names(weights)
        self.manifest = manifest
        self.weights: dict[str, torch.Tensor] = {
            name: value if name in packed else apply_dtype_policy(value, manifest.dtype_policy)
            for name, value in weights.items()
        }
        self._bindings = _check_manifest(manifest, self.weights)
        self._quantized: dict = {}
        for node, binding in zip(manifest.nodes, self._bindings):
            for name, weight_name in node.parameters.items():
                if f'{weight_name}.attrs' in packed and binding.parameter(name).kind != 'array':
                    # decode (and so validate) every packed payload now, not at the first call
                    decode_quantized_weight(weight_name, self.weights)
        if device is not None:
            self.to(device)

    def to(self, device: torch.device | str) -> 'LatticeModel':
        target = torch.device(device)
        self.weights = {
            # the metadata vector is read on the host; it stays there
            name: value if name.endswith('.attrs') else value.to(target)
            for name, value in self.weights.items()
        }
        self._quantized = {}
        return self

    def __call__(self, *inputs: Any, **named: Any) -> Any:
        manifest = self.manifest
        values = self._bind_inputs(inputs, dict(named))
        context = ExecutionContext(values, self.weights, self._quantized, infer_batch_size(values))
        for node, binding in zip(manifest.nodes, self._bindings):
            if binding.handler is not None:
                outputs = binding.handler(context, node, binding)
            else:
                outputs = {'output': binding.function(**_arguments(binding, context, node))}
            self._check_outputs(node, binding, outputs)
            for port, value in outputs.items():
                context.values[node.outputs[port]] = apply_dtype_policy(value, manifest.dtype_policy)
        results = []
        for spec in manifest.outputs:
            validate_value_type(spec.name, spec.type, context.values[spec.name])
            results.append(context.values[spec.name])
        return results[0] if len(results) == 1 else tuple(results)

    def _bind_inputs(self, inputs: tuple, named: dict[str, Any]) -> dict[str, Any]:
        specs = self.manifest.inputs
        if len(inputs) > len(specs):
            raise ValueError('too many positional graph inputs.')
        values: dict[str, Any] = {}
        for position, spec in enumerate(specs):
            if position < len(inputs):
                value = inputs[position]
            elif spec.name in named:
                value = named.pop(spec.name)
            else:
                raise ValueError(f'missing graph input {spec.name!r}.')
            validate_value_type(spec.name, spec.type, value)
            values[spec.name] = apply_dtype_policy(value, self.manifest.dtype_policy)
        if named:
            raise ValueError(f'unknown graph inputs: {sorted(named)}.')
        return values

    @staticmethod
    def _check_outputs(node: IRNode, binding: OperationBinding, outputs: Mapping[str, Any]) -> None:
        missing, extra = set(node.outputs) - set(outputs), set(outputs) - set(node.outputs)
        if missing:
            raise ValueError(f'{node.id}.artifact_outputs missing required keys: {sorted(missing)}.')
        if extra:
            raise ValueError(f'{node.id}.artifact_outputs has unsupported keys: {sorted(extra)}.')
        for port, value in outputs.items():
            validate_value_type(f'{node.id}.outputs.{port}', binding.output_types.get(port, 'any'), value)
