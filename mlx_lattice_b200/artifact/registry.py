"""Which lattice IR operations this runtime executes, and how a node's ports,
parameters and attributes become the arguments of a public ``ops`` function.

Two families, as in the reference (``mlx_lattice/artifact/ops.py:38-300``):

* the stable semantic names persisted artifacts use (``sparse.conv3d``,
  ``sparse.quantized_subm_conv3d``, ``feature.linear``, ``feature.batch_norm``,
  ``pool.global_avg`` ...), port ``input`` bound to the function's first argument;
* one generic ``ops.<function>`` route per public function of ``mlx_lattice_b200.ops``,
  derived from its signature: a required graph-valued argument is an input port, a
  defaulted graph-valued argument is a value attribute (the name of another graph
  value), every other argument is a JSON attribute; weights are parameters.

Operations of the reference that lie outside this package's path (occupancy, ordering,
neighbour-search and coordinate-set ops) are not registered and are
rejected at load time with the reference's message, ``unsupported lattice IR op``.
"""

from __future__ import annotations

import inspect
from collections.abc import Callable, Mapping
from dataclasses import dataclass, field
from typing import Any

from mlx_lattice_b200 import ops
from mlx_lattice_b200.artifact.manifest import IRNode

# annotation fragment -> IR value type (annotations are strings in this package)
_ANNOTATION_TYPES = (
    ('SparseTensor', 'sparse_tensor'),
    ('SparseAlignment', 'alignment'),
    ('KernelRelation', 'relation'),
    ('PointVoxelMap', 'point_voxel_map'),
    ('SparseQuantization', 'quantization'),
    ('torch.Tensor', 'dense_tensor'),
)
_WEIGHT_KINDS = ('array', 'optional_array', 'quantized_weight', 'array_or_quantized_weight')

# persisted tensor arguments of the public functions (``lattice_op_hints`` in the
# reference: mlx_lattice/ops/conv.py:29-33, ops/feature.py:29-32 and :158-165)
_CONV_HINTS = {'weight': ('required', 'array_or_quantized_weight'), 'bias': ('optional', 'array')}
_PARAMETER_HINTS: dict[str, dict[str, tuple[str, str]]] = {
    'conv3d': _CONV_HINTS,
    'subm_conv3d': _CONV_HINTS,
    'conv_transpose3d': _CONV_HINTS,
    'generative_conv_transpose3d': _CONV_HINTS,
    'linear': _CONV_HINTS,
    'batch_norm': {name: ('optional', 'array') for name in ('weight', 'bias', 'mean', 'var')},
    'layer_norm': {name: ('optional', 'array') for name in ('weight', 'bias')},
    'rms_norm': {'weight': ('optional', 'array')},
}
_VALUE_ATTRIBUTE_HINTS = {'conv3d': {'coordinates': 'any'}, 'conv_transpose3d': {'coordinates': 'sparse_tensor'}}


@dataclass(frozen=True, slots=True)
class ParameterBinding:
    argument: str
    kind: str = 'array'


@dataclass(frozen=True, slots=True)
class OperationBinding:
    name: str
    function: Callable[..., Any]
    inputs: Mapping[str, str]                                  # port -> argument
    parameters: Mapping[str, ParameterBinding] = field(default_factory=dict)
    optional_parameters: Mapping[str, ParameterBinding] = field(default_factory=dict)
    attributes: Mapping[str, str] = field(default_factory=dict)
    value_attributes: Mapping[str, str] = field(default_factory=dict)
    input_types: Mapping[str, str] = field(default_factory=dict)
    value_attribute_types: Mapping[str, str] = field(default_factory=dict)
    sequence_inputs: frozenset[str] = frozenset()
    output_type: str = 'any'
    handler: Callable[..., Any] | None = None

    @property
    def output_types(self) -> dict[str, str]:
        return {'output': self.output_type}

    def parameter(self, name: str) -> ParameterBinding | None:
        return self.parameters.get(name) or self.optional_parameters.get(name)


_OPS: dict[str, OperationBinding] = {}


def _annotation_type(annotation: Any) -> str:
    text = annotation if isinstance(annotation, str) else getattr(annotation, '__name__', '')
    for fragment, value_type in _ANNOTATION_TYPES:
        if fragment in text:
            return value_type
    return 'any'


def _is_sequence(annotation: Any) -> bool:
    return isinstance(annotation, str) and annotation.startswith('Sequence[')


def _return_type(function: Callable[..., Any]) -> str:
    annotation = inspect.signature(function).return_annotation
    if annotation is inspect.Signature.empty:
        return 'any'
    text = annotation if isinstance(annotation, str) else getattr(annotation, '__name__', '')
    if text.startswith('tuple'):
        return 'any'
    return _annotation_type(text)


def register(binding: OperationBinding) -> None:
    if binding.name in _OPS:
        raise ValueError(f'duplicate lattice operation binding: {binding.name}.')
    for item in (*binding.parameters.values(), *binding.optional_parameters.values()):
        if item.kind not in _WEIGHT_KINDS:
            raise ValueError(f'unsupported IR parameter kind: {item.kind!r}.')
    _OPS[binding.name] = binding


def public_ops() -> dict[str, Callable[..., Any]]:
    return {name: getattr(ops, name) for name in ops.__all__ if inspect.isfunction(getattr(ops, name))}


def _generic_binding(name: str, function: Callable[..., Any]) -> OperationBinding:
    hints = _PARAMETER_HINTS.get(name, {})
    value_hints = _VALUE_ATTRIBUTE_HINTS.get(name, {})
    inputs, attributes, value_attributes = {}, {}, {}
    input_types, value_types, sequences = {}, {}, set()
    required, optional = {}, {}
    for arg, parameter in inspect.signature(function).parameters.items():
        if parameter.kind in (inspect.Parameter.VAR_POSITIONAL, inspect.Parameter.VAR_KEYWORD):
            continue
        if arg in hints:
            need, kind = hints[arg]
            (required if need == 'required' else optional)[arg] = ParameterBinding(arg, kind)
            continue
        value_type = _annotation_type(parameter.annotation)
        if arg in value_hints:
            value_attributes[arg] = arg
            if value_hints[arg] != 'any':
                value_types[arg] = value_hints[arg]
        elif value_type == 'any':
            attributes[arg] = arg
        elif parameter.default is inspect.Parameter.empty:
            inputs[arg] = arg
            input_types[arg] = value_type
            if _is_sequence(parameter.annotation):
                sequences.add(arg)
        else:
            value_attributes[arg] = arg
            value_types[arg] = value_type
    return OperationBinding(
        name=f'ops.{name}', function=function, inputs=inputs, parameters=required,
        optional_parameters=optional, attributes=attributes, value_attributes=value_attributes,
        input_types=input_types, value_attribute_types=value_types,
        sequence_inputs=frozenset(sequences), output_type=_return_type(function),
    )


_KERNEL_ATTRS = ('kernel_size', 'stride', 'padding', 'dilation')


def _semantic(
    name: str, function_name: str, *, weight: str | None = None, bias: bool = False,
    attributes: tuple[str, ...] = (), value_attributes: Mapping[str, str] | None = None,
    optional: tuple[str, ...] = (), handler: Callable[..., Any] | None = None,
) -> None:
    """One stable artifact name: port ``input`` is the function's first argument."""
    function = public_ops()[function_name]
    first = next(iter(inspect.signature(function).parameters))
    required = {} if weight is None else {'weight': ParameterBinding('weight', weight)}
    optionals = {arg: ParameterBinding(arg, 'array') for arg in optional}
    if bias:
        optionals['bias'] = ParameterBinding('bias', 'array')
    typed = {k: v for k, v in (value_attributes or {}).items() if v != 'any'}
    register(OperationBinding(
        name=name, function=function, inputs={'input': first}, parameters=required,
        optional_parameters=optionals, attributes={a: a for a in attributes},
        value_attributes={a: a for a in (value_attributes or {})},
        input_types={'input': 'sparse_tensor'}, value_attribute_types=typed,
        output_type=_return_type(function), handler=handler,
    ))


def _register_all() -> None:
    from mlx_lattice_b200.artifact.handlers import field_value, global_pool_handler

    register(OperationBinding(
        name='value.field', function=field_value, inputs={'input': 'value'},
        attributes={'field': 'field'}, output_type='any',
        handler=lambda context, node, binding: {
            'output': field_value(context.input_value(node.inputs['input']), node.attributes.get('field'), node.id)
        },
    ))
    for prefix, weight in (('', 'array'), ('quantized_', 'quantized_weight')):
        # the transposed convolution accepts a target support here (an extension of the
        # reference's signature); artifacts written by the reference never set it
        _semantic(f'sparse.{prefix}conv3d', 'conv3d', weight=weight, bias=True,
                  attributes=_KERNEL_ATTRS, value_attributes={'coordinates': 'any'})
        _semantic(f'sparse.{prefix}subm_conv3d', 'subm_conv3d', weight=weight, bias=True,
                  attributes=('kernel_size', 'dilation'))
        _semantic(f'sparse.{prefix}conv_transpose3d', 'conv_transpose3d', weight=weight, bias=True,
                  attributes=_KERNEL_ATTRS, value_attributes={'coordinates': 'sparse_tensor'})
        _semantic(f'sparse.{prefix}generative_conv_transpose3d', 'generative_conv_transpose3d',
                  weight=weight, bias=True, attributes=('kernel_size', 'stride'))
        _semantic(f'feature.{prefix}linear', 'linear', weight=weight, bias=True)
    add = public_ops()['sparse_add']
    register(OperationBinding(
        name='sparse.add', function=add, inputs={'lhs': 'lhs', 'rhs': 'rhs'},
        attributes={'join': 'join'}, input_types={'lhs': 'sparse_tensor', 'rhs': 'sparse_tensor'},
        output_type=_return_type(add),
    ))
    _semantic('feature.relu', 'relu')
    _semantic('feature.sigmoid', 'sigmoid')
    _semantic('feature.silu', 'silu')
    _semantic('feature.tanh', 'tanh')
    _semantic('feature.gelu', 'gelu', attributes=('approximate',))
    _semantic('feature.leaky_relu', 'leaky_relu', attributes=('negative_slope',))
    _semantic('feature.softplus', 'softplus', attributes=('beta', 'threshold'))
    _semantic('feature.dropout', 'dropout', attributes=('p', 'training'))
    _semantic('feature.batch_norm', 'batch_norm', optional=('weight', 'bias', 'mean', 'var'),
              attributes=('eps', 'fuse_relu'))
    _semantic('feature.layer_norm', 'layer_norm', optional=('weight', 'bias'), attributes=('eps',))
    _semantic('feature.rms_norm', 'rms_norm', optional=('weight',), attributes=('eps',))
    for mode in ('sum', 'avg', 'max'):
        _semantic(f'pool.global_{mode}', f'global_{mode}_pool', handler=global_pool_handler)
    for name, function in public_ops().items():
        register(_generic_binding(name, function))


def operation_binding(name: str) -> OperationBinding:
    if not _OPS:
        _register_all()
    try:
        return _OPS[name]
    except KeyError as exc:
        raise ValueError(f'unsupported lattice IR op for this runtime: {name!r}.') from exc


def iter_operation_bindings() -> tuple[OperationBinding, ...]:
    if not _OPS:
        _register_all()
    return tuple(_OPS.values())


def _require_keys(actual: Mapping[str, Any], expected: set[str], path: str) -> None:
    missing, extra = expected - set(actual), set(actual) - expected
    if missing:
        raise ValueError(f'{path} missing required keys: {sorted(missing)}.')
    if extra:
        raise ValueError(f'{path} has unsupported keys: {sorted(extra)}.')


def _check_json(value: Any, path: str) -> None:
    if value is None or isinstance(value, (str, int, float, bool)):
        return
    if isinstance(value, (list, tuple)):
        for index, item in enumerate(value):
            _check_json(item, f'{path}[{index}]')
    elif isinstance(value, dict):
        for key, item in value.items():
            if not isinstance(key, str):
                raise ValueError(f'{path} keys must be strings.')
            _check_json(item, f'{path}.{key}')
    else:
        raise ValueError(f'{path} must be JSON-compatible.')


def node_inputs(binding: OperationBinding, node: IRNode) -> Mapping[str, Any]:
    """The node's inputs by the binding's port names. A module node is written with the
    single port ``input`` whatever its operation (``mlx_lattice/artifact/builder.py:244-251``),
    also for the pooling modules whose operation is a generic ``ops.<function>`` route with
    the port ``x``: ``input`` is accepted for the only port of such a route."""
    if len(binding.inputs) == 1 and set(node.inputs) == {'input'} and 'input' not in binding.inputs:
        return {next(iter(binding.inputs)): node.inputs['input']}
    return node.inputs


def validate_node(node: IRNode) -> OperationBinding:
    """Ports, parameter names and attribute names of a node against its binding
    (``mlx_lattice/artifact/registry.py:205-246``)."""
    binding = operation_binding(node.op)
    _require_keys(node_inputs(binding, node), set(binding.inputs), f'{node.id}.inputs')
    _require_keys(node.outputs, {'output'}, f'{node.id}.outputs')
    missing = set(binding.parameters) - set(node.parameters)
    extra = set(node.parameters) - set(binding.parameters) - set(binding.optional_parameters)
    if missing:
        raise ValueError(f'{node.id}.parameters missing required keys: {sorted(missing)}.')
    if extra:
        raise ValueError(f'{node.id}.parameters has unsupported keys: {sorted(extra)}.')
    unknown = set(node.attributes) - set(binding.attributes) - set(binding.value_attributes)
    if unknown:
        raise ValueError(f'{node.id}.attributes has unsupported keys: {sorted(unknown)}.')
    for name in binding.value_attributes:
        if name in node.attributes and not isinstance(node.attributes[name], str):
            raise ValueError(f'{node.id}.attributes.{name} must be a graph value name.')
    for name in binding.attributes:
        if name in node.attributes:
            _check_json(node.attributes[name], f'{node.id}.attributes.{name}')
    return binding
