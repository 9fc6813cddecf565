"""A small graph writer: emits a manifest and its weight mapping node by node.

The reference's producer side (``mlx_lattice/artifact/builder.py``) walks MLX modules;
this writer covers what the loader needs on this side: building artifacts for tests and
exporting the networks of ``mlx_lattice_b200.workloads`` in the reference's format, with
packed weights stored the way ``builder.py:307-330`` stores them.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

import torch

from mlx_lattice_b200.artifact.handlers import layout_id
from mlx_lattice_b200.artifact.manifest import IRManifest, manifest_from_dict
from mlx_lattice_b200.artifact.registry import operation_binding
from mlx_lattice_b200.core import QuantizedWeight

RUNTIME = {'name': 'mlx-lattice', 'version': '>=0.2.1,<0.3'}


class GraphWriter:
    def __init__(self, inputs: Mapping[str, str], *, dtype_policy: str = 'preserve',
                 producer: Mapping[str, str] | None = None) -> None:
        self.inputs = dict(inputs)
        self.dtype_policy = dtype_policy
        self.producer = dict(producer or {'name': 'mlx-lattice-b200'})
        self.nodes: list[dict[str, Any]] = []
        self.weights: dict[str, torch.Tensor] = {}
        self._types = dict(inputs)

    def _unique(self, name: str) -> str:
        taken = lambda n: n in self.weights or f'{n}.attrs' in self.weights  # noqa: E731
        candidate, index = name, 1
        while taken(candidate):
            candidate, index = f'{name}_{index}', index + 1
        return candidate

    def add_parameter(self, name: str, value: torch.Tensor | QuantizedWeight) -> str:
        """Store a dense tensor under a unique name, or a packed weight as the four tensors
        ``<name>.weight/.scales/.biases/.attrs``; returns the name to put in ``parameters``."""
        key = self._unique(name)
        if isinstance(value, QuantizedWeight):
            codes = value.weight.detach().cpu()
            # the reference stores packed codes as uint32; this package keeps the same bits as int32
            self.weights[f'{key}.weight'] = codes.view(torch.uint32) if codes.dtype == torch.int32 else codes
            self.weights[f'{key}.scales'] = value.scales.detach().cpu()
            self.weights[f'{key}.biases'] = value.biases.detach().cpu()
            self.weights[f'{key}.attrs'] = torch.tensor(
                [layout_id(value.layout), value.group_size, value.bits, value.in_channels,
                 value.out_channels, *value.kernel_size], dtype=torch.int32)
        else:
            self.weights[key] = value.detach().cpu()
        return key

    def add(self, op: str, inputs: Mapping[str, str | tuple[str, ...]], *,
            node_id: str | None = None, output: str | None = None,
            parameters: Mapping[str, torch.Tensor | QuantizedWeight | None] | None = None,
            attributes: Mapping[str, Any] | None = None) -> str:
        """Append a node; returns the name of its output value."""
        binding = operation_binding(op)
        node_id = node_id or f'n{len(self.nodes)}'
        output = output or node_id
        node: dict[str, Any] = {
            'id': node_id, 'op': op,
            'inputs': {k: v if isinstance(v, str) else list(v) for k, v in inputs.items()},
            'outputs': {'output': output},
        }
        stored = {
            name: self.add_parameter(f'{node_id}.{name}', value)
            for name, value in (parameters or {}).items() if value is not None
        }
        if stored:
            node['parameters'] = stored
        if attributes:
            node['attributes'] = {
                k: list(v) if isinstance(v, tuple) else v for k, v in attributes.items() if v is not None
            }
        self.nodes.append(node)
        self._types[output] = binding.output_type
        return output

    def manifest(self, outputs: Mapping[str, str] | None = None) -> IRManifest:
        """``outputs``: value name -> IR type (default: the last node's output)."""
        if outputs is None:
            last = self.nodes[-1]['outputs']['output']
            outputs = {last: self._types[last]}
        return manifest_from_dict({
            'schema_version': '0.1',
            'producer': self.producer,
            'runtime': dict(RUNTIME),
            'dtype_policy': self.dtype_policy,
            'inputs': [{'name': k, 'type': v} for k, v in self.inputs.items()],
            'outputs': [{'name': k, 'type': v} for k, v in outputs.items()],
            'nodes': self.nodes,
        })
