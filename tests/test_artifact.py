"""Artifact loader, host side: manifest contract, the safetensors container, the operation
table and the static validation of a model against its weights. The cases mirror the
reference's own artifact tests (``tests/artifact/test_lattice_artifact.py:68-430``) with the
same manifests and the same error texts; nothing here launches a kernel."""

import json

import numpy as np
import pytest
import torch

from mlx_lattice_b200 import artifact
from mlx_lattice_b200.artifact.model import version_satisfies
from mlx_lattice_b200.artifact.tensors_file import load_tensors, save_tensors
from mlx_lattice_b200.core import quantize_weight


def _raw_manifest():
    # tests/artifact/test_lattice_artifact.py:68-115
    return {
        'schema_version': '0.1',
        'producer': {'name': 'test'},
        'runtime': {'name': 'mlx-lattice', 'version': '>=0.2.1,<0.3'},
        'inputs': [{'name': 'input', 'type': 'sparse_tensor'}],
        'outputs': [{'name': 'logits', 'type': 'dense_tensor'}],
        'nodes': [
            {'id': 'conv', 'op': 'sparse.conv3d', 'inputs': {'input': 'input'},
             'outputs': {'output': 'conv'}, 'parameters': {'weight': 'conv.weight'},
             'support': {'kind': 'forward', 'kernel_size': [3, 1, 1], 'stride': [1, 1, 1],
                         'padding': [0, 0, 0], 'dilation': [1, 1, 1]}},
            {'id': 'relu', 'op': 'feature.relu', 'inputs': {'input': 'conv'},
             'outputs': {'output': 'relu'}},
            {'id': 'linear', 'op': 'feature.linear', 'inputs': {'input': 'relu'},
             'outputs': {'output': 'projected'},
             'parameters': {'weight': 'linear.weight', 'bias': 'linear.bias'}},
            {'id': 'pool', 'op': 'pool.global_avg', 'inputs': {'input': 'projected'},
             'outputs': {'output': 'logits'}},
        ],
    }


def _weights():
    return {
        'conv.weight': torch.tensor([1.0, 2.0, 3.0]).reshape(1, 3, 1, 1, 1),
        'linear.weight': torch.tensor([[2.0], [3.0]]),
        'linear.bias': torch.tensor([1.0, -1.0]),
    }


def test_manifest_round_trip_and_support_attributes():
    manifest = artifact.manifest_from_dict(_raw_manifest())
    conv = manifest.nodes[0]
    assert conv.support.kind == 'forward' and conv.support.kernel_size == (3, 1, 1)
    assert conv.attributes['kernel_size'] == (3, 1, 1) and conv.attributes['dilation'] == (1, 1, 1)
    assert manifest.dtype_policy == 'preserve'
    assert manifest.coordinate_order == ('batch', 'x', 'y', 'z')
    again = artifact.manifest_from_dict(json.loads(json.dumps(artifact.manifest_to_dict(manifest))))
    assert artifact.manifest_to_dict(again) == artifact.manifest_to_dict(manifest)
    target = artifact.manifest_from_dict({
        'schema_version': '0.1', 'inputs': [{'name': 'a', 'type': 'sparse_tensor'},
                                            {'name': 't', 'type': 'dense_tensor'}],
        'outputs': [{'name': 'o', 'type': 'sparse_tensor'}],
        'nodes': [{'id': 'c', 'op': 'sparse.conv3d', 'inputs': {'input': 'a'}, 'outputs': {'output': 'o'},
                   'parameters': {'weight': 'w'}, 'support': {'kind': 'target', 'target': 't', 'kernel_size': 3}}],
    })
    assert target.nodes[0].attributes == {'kernel_size': (3, 3, 3), 'coordinates': 't'}


@pytest.mark.parametrize('edit, message', [
    (lambda m: m.update(schema_version='9'), 'unsupported lattice IR schema_version'),
    (lambda m: m.update(coordinate_order=['x', 'y', 'z', 'batch']), 'coordinate_order must be'),
    (lambda m: m.update(feature_layout=['channel', 'row']), 'feature_layout must be'),
    (lambda m: m.update(weight_layout='other'), "weight_layout must be 'mlx-lattice'"),
    (lambda m: m.update(dtype_policy='bf16'), 'dtype_policy must be'),
    (lambda m: m.update(inputs='input'), 'inputs must be a list'),
    (lambda m: m['inputs'].append({'name': 'input', 'type': 'sparse_tensor'}), 'duplicate graph value'),
    (lambda m: m['inputs'][0].update(type='tensor'), 'not a supported lattice IR value type'),
    (lambda m: m['nodes'][1].update(id='conv'), 'duplicate node id'),
    (lambda m: m['nodes'][1].update(outputs={}), 'must define outputs'),
    (lambda m: m['nodes'][1].update(inputs={'input': 'nowhere'}), 'references unknown input'),
    (lambda m: m['nodes'][2].update(outputs={'output': 'conv'}), 'duplicate graph value'),
    (lambda m: m['outputs'][0].update(name='nothing'), 'unknown manifest output'),
    (lambda m: m['nodes'][0]['support'].update(kernel_size=[3, 1]), 'sequence of 3 ints'),
    (lambda m: m['nodes'][0].update(inputs={'input': 5}), 'must be a string or list of strings'),
    (lambda m: m['nodes'][0].update(parameters={'weight': 3}), 'must map strings to strings'),
])
def test_manifest_rejects_contract_violations(edit, message):
    raw = _raw_manifest()
    edit(raw)
    with pytest.raises(ValueError, match=message):
        artifact.manifest_from_dict(raw)


def test_runtime_compatibility():
    # tests/artifact/test_lattice_artifact.py:197-245
    for runtime in ({'name': 'mlx-lattice', 'version': '>=0.2.1,<0.3.0'}, {}):
        raw = _raw_manifest()
        raw['runtime'] = runtime
        model = artifact.LatticeModel(artifact.manifest_from_dict(raw), _weights())
        assert model.manifest.runtime == runtime
    for runtime, message in (
        ({'name': 'other-runtime', 'version': '>=0.2.1,<0.3'}, r'runtime\.name'),
        ({'name': 'mlx-lattice', 'version': '>=999.0'}, r'runtime\.version'),
        ({'name': 'mlx-lattice', 'version': '~=0.2'}, 'unsupported runtime version specifier'),
    ):
        raw = _raw_manifest()
        raw['runtime'] = runtime
        with pytest.raises(ValueError, match=message):
            artifact.LatticeModel(artifact.manifest_from_dict(raw), _weights())
    assert version_satisfies('0.2.1', '0.2.1') and version_satisfies('0.2.1', '==0.2.1.0')
    assert version_satisfies('0.2.1rc1', '>=0.2, !=0.2.0, <=0.2.1')
    assert not version_satisfies('0.2.1', '>0.2.1') and not version_satisfies('0.2.1', '<0.2.1')


def _single(op, inputs, outputs, *, node_inputs, attributes=None, out_type='sparse_tensor'):
    node = {'id': 'node', 'op': op, 'inputs': node_inputs, 'outputs': {'output': outputs}}
    if attributes:
        node['attributes'] = attributes
    return artifact.manifest_from_dict({
        'schema_version': '0.1', 'inputs': [{'name': k, 'type': v} for k, v in inputs.items()],
        'outputs': [{'name': outputs, 'type': out_type}], 'nodes': [node],
    })


def test_model_static_validation_messages():
    # tests/artifact/test_lattice_artifact.py:248-356
    with pytest.raises(ValueError, match='unsupported lattice IR op'):
        artifact.LatticeModel(_single('custom.bad', {'input': 'sparse_tensor'}, 'output',
                                      node_inputs={'input': 'input'}), {})
    with pytest.raises(ValueError, match='unknown graph value'):
        artifact.LatticeModel(_single(
            'ops.voxelize', {'points': 'dense_tensor', 'feats': 'dense_tensor'}, 'voxels',
            node_inputs={'points': 'points', 'feats': 'feats'},
            attributes={'batch_indices': 'missing'}), {})
    with pytest.raises(ValueError, match=r"expects 'dense_tensor'"):
        artifact.LatticeModel(_single('ops.voxelize', {'input': 'sparse_tensor'}, 'output',
                                      node_inputs={'points': 'input', 'feats': 'input'}), {})
    bad_map = artifact.manifest_from_dict({
        'schema_version': '0.1',
        'inputs': [{'name': n, 'type': 'dense_tensor'} for n in ('points', 'feats', 'bad_map')],
        'outputs': [{'name': 'sampled', 'type': 'dense_tensor'}],
        'nodes': [
            {'id': 'voxelize', 'op': 'ops.voxelize', 'inputs': {'points': 'points', 'feats': 'feats'},
             'outputs': {'output': 'voxels'}},
            {'id': 'sample', 'op': 'ops.devoxelize', 'inputs': {'points': 'points', 'voxels': 'voxels'},
             'outputs': {'output': 'sampled'}, 'attributes': {'point_voxel_map': 'bad_map'}},
        ],
    })
    with pytest.raises(ValueError, match=r"expects 'point_voxel_map'"):
        artifact.LatticeModel(bad_map, {})
    manifest = artifact.manifest_from_dict(_raw_manifest())
    with pytest.raises(ValueError, match='missing weight'):
        artifact.LatticeModel(manifest, {})
    raw = _raw_manifest()
    raw['outputs'][0]['type'] = 'sparse_tensor'
    with pytest.raises(ValueError, match=r"outputs\.logits expects 'sparse_tensor'"):
        artifact.LatticeModel(artifact.manifest_from_dict(raw), _weights())
    for edit, message in (
        (lambda n: n.update(inputs={'x': 'input'}), r'conv\.inputs missing required keys'),
        (lambda n: n['inputs'].update(extra='input'), r'conv\.inputs has unsupported keys'),
        (lambda n: n.update(outputs={'result': 'conv'}), r'conv\.outputs missing required keys'),
        (lambda n: n.update(parameters={}), r'conv\.parameters missing required keys'),
        (lambda n: n['parameters'].update(scale='conv.weight'), r'conv\.parameters has unsupported keys'),
        (lambda n: n.update(attributes={'groups': 2}), r'conv\.attributes has unsupported keys'),
        (lambda n: n.update(attributes={'coordinates': 3}), 'must be a graph value name'),
    ):
        raw = _raw_manifest()
        edit(raw['nodes'][0])
        with pytest.raises(ValueError, match=message):
            artifact.LatticeModel(artifact.manifest_from_dict(raw), _weights())


def test_module_style_node_on_a_generic_route():
    """A pooling module is exported as ``ops.max_pool3d`` with the port ``input``."""
    manifest = _single('ops.max_pool3d', {'x0': 'sparse_tensor'}, 'pooled', node_inputs={'input': 'x0'},
                       attributes={'kernel_size': [2, 2, 2], 'stride': [2, 2, 2]})
    artifact.LatticeModel(manifest, {})
    with pytest.raises(ValueError, match=r"expects 'sparse_tensor'"):
        artifact.LatticeModel(_single('ops.max_pool3d', {'x0': 'dense_tensor'}, 'pooled',
                                      node_inputs={'input': 'x0'}), {})
    with pytest.raises(ValueError, match='inputs missing required keys'):
        artifact.LatticeModel(_single('ops.sparse_cat_aligned', {'x0': 'sparse_tensor'}, 'y',
                                      node_inputs={'input': 'x0'}), {})


def _quantized_linear_artifact():
    dense = torch.from_numpy(np.random.default_rng(0).normal(size=(8, 64)).astype(np.float16))
    writer = artifact.GraphWriter({'input': 'sparse_tensor'})
    writer.add('feature.quantized_linear', {'input': 'input'}, node_id='head', output='output',
               parameters={'weight': quantize_weight(dense, group_size=32, bits=4),
                           'bias': torch.zeros(8, dtype=torch.float32)})
    return writer


def test_quantized_payload_layout_policy_and_completeness():
    # tests/artifact/test_lattice_artifact.py:391-430, builder.py:307-330
    writer = _quantized_linear_artifact()
    prefix = 'head.weight'
    assert sorted(writer.weights) == ['head.bias'] + [f'{prefix}.{s}' for s in ('attrs', 'biases', 'scales', 'weight')]
    assert writer.weights[f'{prefix}.attrs'].dtype == torch.int32
    assert writer.weights[f'{prefix}.attrs'].tolist() == [0, 32, 4, 64, 8, 1, 1, 1]
    raw = artifact.manifest_to_dict(writer.manifest())
    assert raw['runtime'] == {'name': 'mlx-lattice', 'version': '>=0.2.1,<0.3'}
    raw['dtype_policy'] = 'fp16'
    model = artifact.LatticeModel(artifact.manifest_from_dict(raw), writer.weights)
    assert model.weights[f'{prefix}.weight'].dtype == torch.uint32
    assert model.weights[f'{prefix}.scales'].dtype == writer.weights[f'{prefix}.scales'].dtype
    assert model.weights[f'{prefix}.biases'].dtype == writer.weights[f'{prefix}.biases'].dtype
    assert model.weights['head.bias'].dtype == torch.float16
    weights = dict(writer.weights)
    del weights[f'{prefix}.attrs']
    with pytest.raises(ValueError, match='missing quantized weight'):
        artifact.LatticeModel(writer.manifest(), weights)
    weights = dict(writer.weights)
    weights[f'{prefix}.attrs'] = torch.tensor([7, 32, 4, 64, 8, 1, 1, 1], dtype=torch.int32)
    with pytest.raises(ValueError, match='unknown quantized weight layout id'):
        artifact.LatticeModel(writer.manifest(), weights)
    weights[f'{prefix}.attrs'] = torch.tensor([0, 32, 4, 64], dtype=torch.int32)
    with pytest.raises(ValueError, match='invalid metadata'):
        artifact.LatticeModel(writer.manifest(), weights)


def test_safetensors_container_round_trip_and_foreign_reader(tmp_path):
    rng = np.random.default_rng(1)
    tensors = {
        'codes': torch.from_numpy(rng.integers(0, 2 ** 32, size=(3, 4, 5), dtype=np.uint32)),
        'attrs': torch.tensor([0, 32, 4, 64, 8, 1, 1, 1], dtype=torch.int32),
        'half': torch.from_numpy(rng.normal(size=(7, 3)).astype(np.float16)),
        'single': torch.from_numpy(rng.normal(size=(2, 2, 2)).astype(np.float32)),
        'brain': torch.from_numpy(rng.normal(size=(5,)).astype(np.float32)).to(torch.bfloat16),
        'scalar': torch.tensor(3.5),
        'empty': torch.zeros((0, 4), dtype=torch.float16),
        'flags': torch.tensor([True, False]),
    }
    path = tmp_path / 'weights.safetensors'
    save_tensors(path, tensors, metadata={'format': 'pt'})
    loaded = load_tensors(path)
    assert sorted(loaded) == sorted(tensors)
    for name, value in tensors.items():
        assert loaded[name].dtype == value.dtype and loaded[name].shape == value.shape, name
        assert loaded[name].numpy(force=True).tobytes() == value.numpy(force=True).tobytes() \
            if value.dtype != torch.bfloat16 else torch.equal(loaded[name], value), name
    header_bytes = int.from_bytes(path.read_bytes()[:8], 'little')
    assert header_bytes % 8 == 0
    # the public safetensors package reads this file and writes files this reader reads
    st = pytest.importorskip('safetensors.numpy')
    from safetensors import safe_open

    with safe_open(str(path), framework='np') as foreign:
        assert sorted(foreign.keys()) == sorted(tensors)
        assert foreign.metadata() == {'format': 'pt'}
        for name in ('codes', 'attrs', 'half', 'single', 'scalar', 'empty', 'flags'):
            assert np.array_equal(foreign.get_tensor(name), tensors[name].numpy()), name
    other = tmp_path / 'foreign.safetensors'
    st.save_file({k: v.numpy() for k, v in tensors.items() if k != 'brain'}, str(other))
    back = load_tensors(other)
    for name, value in tensors.items():
        if name != 'brain':
            assert torch.equal(back[name], value), name
    for damage, message in ((b'\x01', 'truncated'), (b'\xff' * 16, 'invalid header length'),
                            ((2).to_bytes(8, 'little') + b'[]', 'tensor mapping')):
        broken = tmp_path / 'broken.safetensors'
        broken.write_bytes(damage)
        with pytest.raises(ValueError, match=message):
            load_tensors(broken)


def test_artifact_directory_checks(tmp_path):
    with pytest.raises(ValueError, match='does not exist'):
        artifact.load_lattice_artifact(tmp_path / 'nothing')
    with pytest.raises(ValueError, match='missing manifest.json'):
        artifact.load_lattice_artifact(tmp_path)
    (tmp_path / 'manifest.json').write_text(json.dumps(_raw_manifest()))
    with pytest.raises(ValueError, match='missing weights.safetensors'):
        artifact.load_lattice_artifact(tmp_path)
    with pytest.raises(ValueError, match='missing weight'):
        artifact.save_lattice_model(tmp_path / 'out', artifact.manifest_from_dict(_raw_manifest()), {})
    artifact.save_lattice_model(tmp_path / 'out', artifact.manifest_from_dict(_raw_manifest()), _weights())
    loaded = artifact.load_lattice_artifact(tmp_path / 'out')
    assert isinstance(loaded, artifact.LatticeArtifact)
    assert artifact.manifest_to_dict(loaded.manifest) == artifact.manifest_to_dict(
        artifact.manifest_from_dict(_raw_manifest()))
    for name, value in _weights().items():
        assert torch.equal(loaded.weights[name], value)
    assert isinstance(loaded.model(), artifact.LatticeModel)


def test_operation_table_covers_the_public_ops_and_keeps_tensors_out_of_attributes():
    # tests/artifact/test_lattice_artifact.py:474-540
    from mlx_lattice_b200 import ops

    names = {binding.name for binding in artifact.iter_operation_bindings()}
    for name in ops.__all__:
        assert f'ops.{name}' in names, name
    for name in ('sparse.conv3d', 'sparse.subm_conv3d', 'sparse.conv_transpose3d',
                 'sparse.generative_conv_transpose3d', 'feature.linear', 'feature.relu',
                 'feature.batch_norm', 'pool.global_sum', 'pool.global_avg', 'pool.global_max',
                 'value.field'):
        assert name in names
        if name.startswith('sparse.') or name == 'feature.linear':
            family, op = name.split('.')
            quantized = artifact.operation_binding(f'{family}.quantized_{op}')
            assert quantized.parameters['weight'].kind == 'quantized_weight'
            assert artifact.operation_binding(name).parameters['weight'].kind == 'array'
    for binding in artifact.iter_operation_bindings():
        for tensor_argument in ('weight', 'bias', 'mean', 'var'):
            assert tensor_argument not in binding.attributes, binding.name
    assert artifact.operation_binding('ops.conv3d').parameters['weight'].kind == 'array_or_quantized_weight'
