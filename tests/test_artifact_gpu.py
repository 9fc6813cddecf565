"""Artifact models on the GPU: the reference's own manifest cases with their known
answers (``tests/artifact/test_lattice_artifact.py:167-195`` and ``:431-470``), the dtype
policy, packed payloads through a directory on disk, and the MinkUNet workload exported
as an artifact against the same network assembled from the operators directly."""

import numpy as np
import pytest
import torch

from mlx_lattice_b200 import artifact, synthetic, workloads
from test_artifact import _raw_manifest, _weights

pytestmark = pytest.mark.gpu


def _input(cuda, dtype=torch.float32):
    from mlx_lattice_b200.core import SparseTensor

    coords = torch.tensor([[0, 0, 0, 0], [0, 1, 0, 0], [0, 2, 0, 0]], dtype=torch.int32, device=cuda)
    feats = torch.tensor([[1.0], [2.0], [3.0]], dtype=dtype, device=cuda)
    return SparseTensor(coords, feats, batch_counts=(3,))


def test_reference_manifest_known_answer(cuda, tmp_path):
    """conv (3,1,1) with taps 1,2,3 over features 1,2,3 -> 8,14,8; ReLU; linear [[2],[3]] +
    [1,-1] -> (17,23),(29,41),(17,23); global average -> (21, 29). The convolution output
    has no batch_counts, so the pooling node groups rows by their batch column."""
    from mlx_lattice_b200 import ops

    manifest = artifact.manifest_from_dict(_raw_manifest())
    model = artifact.LatticeModel(manifest, _weights(), device=cuda)
    x = _input(cuda)
    got = model(x)
    assert got.shape == (1, 2) and got.dtype == torch.float32
    assert got.tolist() == [[21.0, 29.0]]
    w = {k: v.to(cuda) for k, v in _weights().items()}
    direct = ops.linear(ops.relu(ops.conv3d(x, w['conv.weight'], kernel_size=(3, 1, 1))),
                        w['linear.weight'], w['linear.bias'])
    assert direct.feats.tolist() == [[17.0, 23.0], [29.0, 41.0], [17.0, 23.0]]
    assert torch.equal(model(input=x), got)
    artifact.save_lattice_model(tmp_path, manifest, _weights())
    loaded = artifact.load_lattice_model(tmp_path)
    assert all(v.is_cuda for v in loaded.weights.values())
    assert torch.equal(loaded(x), got)
    with pytest.raises(ValueError, match='too many positional'):
        model(x, x)
    with pytest.raises(ValueError, match="missing graph input 'input'"):
        model()
    with pytest.raises(ValueError, match='unknown graph inputs'):
        model(x, other=x)
    with pytest.raises(ValueError, match="graph value 'input' must be SparseTensor"):
        model(x.feats)


def test_pooling_by_batch_column_matches_batch_counts(cuda):
    """Three clouds with interleaved rows, trailing inactive rows and an empty batch."""
    from mlx_lattice_b200.artifact.handlers import _pool_by_batch_column
    from mlx_lattice_b200.core import SparseTensor

    rng = np.random.default_rng(3)
    coords = rng.integers(-20, 20, size=(5000, 4)).astype(np.int32)
    coords[:, 0] = rng.choice([0, 1, 3], size=5000)
    feats = rng.normal(size=(5000, 24)).astype(np.float32)
    active = 4321
    x = SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda),
                     active_rows=torch.tensor([active], dtype=torch.int32, device=cuda))
    for mode in ('sum', 'avg'):
        got = _pool_by_batch_column(x, 4, mode).cpu().numpy()
        want = np.zeros((4, 24), np.float32)
        for b in range(4):
            rows = feats[:active][coords[:active, 0] == b]
            if rows.shape[0]:
                total = np.zeros(24, np.float32)
                for row in rows:                      # row order, float32 accumulation
                    total += row
                want[b] = total if mode == 'sum' else total / np.float32(rows.shape[0])
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
        assert not got[2].any()


def test_target_convolution_and_value_attributes(cuda):
    # tests/artifact/test_lattice_artifact.py:431-470
    from mlx_lattice_b200 import ops

    manifest = artifact.manifest_from_dict({
        'schema_version': '0.1',
        'inputs': [{'name': 'input', 'type': 'sparse_tensor'}, {'name': 'target', 'type': 'dense_tensor'}],
        'outputs': [{'name': 'output', 'type': 'sparse_tensor'}],
        'nodes': [{'id': 'target_conv', 'op': 'sparse.conv3d', 'inputs': {'input': 'input'},
                   'outputs': {'output': 'output'}, 'parameters': {'weight': 'conv.weight'},
                   'support': {'kind': 'target', 'target': 'target', 'kernel_size': [3, 1, 1]}}],
    })
    model = artifact.LatticeModel(manifest, _weights(), device=cuda)
    x = _input(cuda)
    target = torch.tensor([[0, 1, 0, 0], [0, 3, 0, 0]], dtype=torch.int32, device=cuda)
    got = model(x, target)
    want = ops.conv3d(x, _weights()['conv.weight'].to(cuda), kernel_size=(3, 1, 1), coordinates=target)
    assert torch.equal(got.coords, want.coords) and torch.equal(got.coords, target)
    assert got.feats.tolist() == want.feats.tolist() == [[14.0], [3.0]]


def test_fp16_policy_casts_values_and_dense_weights(cuda):
    # tests/artifact/test_lattice_artifact.py:359-388
    manifest = artifact.manifest_from_dict({
        'schema_version': '0.1', 'dtype_policy': 'fp16',
        'inputs': [{'name': 'input', 'type': 'sparse_tensor'}],
        'outputs': [{'name': 'output', 'type': 'sparse_tensor'}],
        'nodes': [{'id': 'linear', 'op': 'feature.linear', 'inputs': {'input': 'input'},
                   'outputs': {'output': 'output'},
                   'parameters': {'weight': 'linear.weight', 'bias': 'linear.bias'}}],
    })
    model = artifact.LatticeModel(manifest, _weights(), device=cuda)
    assert model.weights['linear.weight'].dtype == torch.float16
    assert model.weights['linear.bias'].dtype == torch.float16
    got = model(_input(cuda))
    assert got.feats.dtype == torch.float16
    assert got.feats.tolist() == [[3.0, 2.0], [5.0, 5.0], [7.0, 8.0]]


def test_minkunet_artifact_equals_the_direct_network(cuda, tmp_path):
    """The int4 MinkUNet exported to manifest.json + weights.safetensors, loaded back from
    disk and run: bitwise equal to the network assembled from the operators, in both decoder
    forms (target support named on the transposed convolution, and the reference's form:
    transposed convolution followed by a right-join concatenation)."""
    from mlx_lattice_b200.core import SparseTensor

    quantized = workloads.quantize_all(workloads.minkunet_dense_weights(11))
    net = workloads.MinkUNet(quantized, cuda)
    coords = torch.from_numpy(synthetic.lidar_batch(5, 2, 6000)).to(cuda)
    feats = torch.from_numpy(
        np.random.default_rng(5).normal(size=(coords.shape[0], 4)).astype(np.float16)).to(cuda)

    def fresh():
        return SparseTensor(coords, feats, batch_counts=(6000, 6000))

    want = net(fresh())
    for target_support in (True, False):
        manifest, weights = workloads.minkunet_artifact(quantized, target_support=target_support)
        root = tmp_path / f'unet_{int(target_support)}'
        artifact.save_lattice_artifact(root, manifest, weights)
        stored = artifact.load_lattice_artifact(root)
        assert stored.weights['stem.weight.weight'].dtype == torch.uint32
        assert stored.weights['stem.weight.attrs'].tolist() == [2, 32, 4, 4, 32, 3, 3, 3]
        model = artifact.load_lattice_model(root, device=cuda)
        got = model(fresh())
        assert torch.equal(got.coords, want.coords)
        if target_support:
            assert torch.equal(got.feats, want.feats)
        else:
            # same sums; the unfused decoder materialises the 8x transposed output first
            scale = float(want.feats.float().abs().max())
            assert float((got.feats.float() - want.feats.float()).abs().max()) <= 2e-3 * scale
        assert torch.equal(model(fresh()).feats, got.feats)


def test_point_cloud_graph_with_structured_fields(cuda):
    """voxelize -> convolution -> devoxelize as one artifact: generic ``ops.*`` routes, a
    defaulted graph-valued argument passed by name, and ``value.field`` projections."""
    from mlx_lattice_b200 import ops

    rng = np.random.default_rng(8)
    points = torch.from_numpy((rng.random((4000, 3)) * 12).astype(np.float32)).to(cuda)
    feats = torch.from_numpy(rng.normal(size=(4000, 16)).astype(np.float32)).to(cuda)
    batch = torch.from_numpy(rng.integers(0, 2, size=4000).astype(np.int32)).to(cuda)
    weight = torch.from_numpy((rng.normal(size=(16, 3, 3, 3, 16)) * 0.1).astype(np.float32))

    g = artifact.GraphWriter({'points': 'dense_tensor', 'feats': 'dense_tensor', 'batch': 'dense_tensor'})
    quant = g.add('ops.sparse_quantize', {'points': 'points'}, node_id='quant',
                  attributes={'voxel_size': 0.5, 'batch_indices': 'batch'})
    voxels = g.add('ops.voxelize_with_quantization', {'quantization': quant, 'feats': 'feats'}, node_id='voxels')
    conv = g.add('sparse.subm_conv3d', {'input': voxels}, node_id='conv', parameters={'weight': weight},
                 attributes={'kernel_size': 3})
    g.add('ops.devoxelize', {'points': 'points', 'voxels': conv}, node_id='sampled',
          attributes={'voxel_size': 0.5, 'batch_indices': 'batch', 'interpolation': 'nearest'})
    g.add('value.field', {'input': quant}, node_id='inverse', attributes={'field': 'inverse_rows'})
    manifest = g.manifest({'sampled': 'dense_tensor', 'inverse': 'dense_tensor'})
    model = artifact.LatticeModel(manifest, g.weights, device=cuda)
    sampled, inverse = model(points, feats, batch)

    q = ops.sparse_quantize(points, 0.5, batch_indices=batch)
    v = ops.voxelize_with_quantization(q, feats)
    y = ops.subm_conv3d(v, weight.to(cuda), kernel_size=3)
    want = ops.devoxelize(points, y, 0.5, batch_indices=batch, interpolation='nearest')
    assert torch.equal(inverse, q.inverse_rows)
    assert torch.equal(sampled, want)
    bad = artifact.GraphWriter({'points': 'dense_tensor'})
    quant = bad.add('ops.sparse_quantize', {'points': 'points'}, node_id='quant')
    bad.add('value.field', {'input': quant}, node_id='f', attributes={'field': 'secret'})
    with pytest.raises(ValueError, match="field 'secret' is not supported for SparseQuantization"):
        artifact.LatticeModel(bad.manifest(), {})(points)
