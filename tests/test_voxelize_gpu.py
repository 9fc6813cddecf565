"""Point -> voxel front end on the GPU against the oracle: voxel coordinates, first-seen
order, inverse rows and counts bit-exact; voxel features bit-exact against the compiled
reference (same fused multiply-add, same order) and within 1e-5 of the restatement."""

import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KATS = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden',
                                   'reference_kats.json')))


def _dev(array, cuda):
    return torch.from_numpy(np.ascontiguousarray(array)).to(cuda)


def _cloud(seed, rows, batches):
    rng = np.random.default_rng(seed)
    points = (rng.normal(size=(rows, 3)) * 9.0).astype(np.float32)
    points[::7] = np.round(points[::7])          # points on cell boundaries
    points[5::11] = points[4::11][: points[5::11].shape[0]]   # exact duplicates
    batch = np.sort(rng.integers(0, batches, size=rows)).astype(np.int32)
    return points, batch


def test_reference_known_answers(cuda):
    from mlx_lattice_b200 import ops

    kat = KATS['quantize_ordered']
    q = ops.sparse_quantize(_dev(np.asarray(kat['points'], np.float32), cuda), kat['voxel_size'],
                            batch_indices=_dev(np.asarray(kat['batches'], np.int32), cuda))
    n = kat['active_rows'][0]
    assert q.capacity == 5 and q.active_count is q.active_rows
    assert q.active_rows.tolist() == kat['active_rows']
    assert q.coords[:n].tolist() == kat['coords']
    assert q.inverse_rows.tolist() == kat['inverse_rows']
    assert q.counts[:n].tolist() == kat['counts']

    kat = KATS['quantize_origin_active']
    q = ops.sparse_quantize(_dev(np.asarray(kat['points'], np.float32), cuda), kat['voxel_size'],
                            origin=kat['origin'],
                            active_rows=_dev(np.asarray(kat['point_active'], np.int32), cuda))
    assert q.active_rows.tolist() == kat['active_rows']
    assert q.coords[: kat['active_rows'][0]].tolist() == kat['coords']
    assert q.inverse_rows.tolist() == kat['inverse_rows']
    assert q.counts.tolist() == kat['counts']

    kat = KATS['voxelize_mean_sum']
    points = _dev(np.asarray(kat['points'], np.float32), cuda)
    feats = _dev(np.asarray(kat['feats'], np.float32), cuda)
    mean = ops.voxelize(points, feats, voxel_size=1.0, reduction='mean')
    total = ops.voxelize(points, feats, voxel_size=1.0, reduction='sum')
    n = int(mean.active_rows.item())
    assert mean.coords[:n].tolist() == kat['coords'] and mean.stride == (1, 1, 1)
    assert np.allclose(mean.feats[:n].cpu().numpy(), kat['mean'])
    assert np.allclose(total.feats[:n].cpu().numpy(), kat['sum'])


@pytest.mark.parametrize('rows,batches,active', [(50000, 4, None), (20000, 1, 17500), (1, 1, None),
                                                  (3000, 3, 0)])
def test_sparse_quantize_matches_oracle(cuda, oracle, rows, batches, active):
    from mlx_lattice_b200 import _ext

    points, batch = _cloud(rows + batches, rows, batches)
    size, origin = (0.5, 0.75, 1.25), (0.1, -0.3, 2.0)
    active_np = None if active is None else np.asarray([active], np.int32)
    want = oracle.sparse_quantize(points, batch, active_np, size, origin)
    active_dev = _dev(np.asarray([rows if active is None else active], np.int32), cuda)
    got = _ext.sparse_quantize(_dev(points, cuda), _dev(batch, cuda), active_dev, size, origin)
    for g, w, name in zip(got, want, ('coords', 'count', 'inverse_rows', 'counts')):
        assert np.array_equal(g.cpu().numpy(), w), name
    _ext.check_status(cuda)


@pytest.mark.parametrize('channels', [1, 4, 40])
@pytest.mark.parametrize('mode', ['mean', 'sum'])
def test_voxelize_features_matches_oracle(cuda, oracle, restatement, channels, mode):
    from mlx_lattice_b200 import _ext

    rows = 30000
    points, batch = _cloud(channels, rows, 2)
    coords, count, inverse, counts = oracle.sparse_quantize(points, batch, None, 1.5, 0.0)
    rng = np.random.default_rng(channels * 3 + 1)
    feats = rng.normal(size=(rows, channels)).astype(np.float32)
    active = np.asarray([rows - 500], np.int32)
    want = oracle.voxelize_features(feats, inverse, counts, active, mode)
    got = _ext.voxelize_features(_dev(feats, cuda), _dev(inverse, cuda), _dev(counts, cuda),
                                 _dev(active, cuda), mode).cpu().numpy()
    if oracle is restatement:
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    else:
        assert np.array_equal(got, want)   # same fused multiply-adds in the same order
    n = int(count[0])
    assert not got[n:].any()
    _ext.check_status(cuda)


def test_voxelize_feeds_the_convolution(cuda, oracle):
    """points -> voxelize -> subm_conv3d: the front end's tensor is a regular input of the
    path (coordinates unique, active_rows respected)."""
    from mlx_lattice_b200 import ops

    points, batch = _cloud(9, 20000, 2)
    rng = np.random.default_rng(10)
    feats = rng.normal(size=(20000, 4)).astype(np.float32)
    x = ops.voxelize(_dev(points, cuda), _dev(feats, cuda), 1.0, batch_indices=_dev(batch, cuda))
    n = int(x.active_rows.item())
    weight = (rng.normal(size=(8, 3, 3, 3, 4)) * 0.1).astype(np.float32)
    y = ops.subm_conv3d(x, _dev(weight, cuda), kernel_size=3)
    coords, count, inverse, counts = oracle.sparse_quantize(points, batch, None, 1.0, 0.0)
    vox = oracle.voxelize_features(feats, inverse, counts, np.asarray([20000], np.int32), 'mean')
    rel = oracle.build_submanifold_kernel_relation(coords, n)
    want = oracle.sparse_conv(vox, weight, rel, coords.shape[0], 27)
    got = y.feats.cpu().numpy()
    scale = np.abs(want).max()
    assert np.abs(got[:n] - want[:n]).max() <= 1e-5 * scale
    assert not got[n:].any()


def test_argument_errors(cuda):
    from mlx_lattice_b200 import ops

    points = torch.zeros((4, 3), dtype=torch.float32, device=cuda)
    with pytest.raises(ValueError, match='points must have shape'):
        ops.sparse_quantize(torch.zeros((4, 2), dtype=torch.float32, device=cuda))
    with pytest.raises(ValueError, match='points must be float32'):
        ops.sparse_quantize(points.double())
    with pytest.raises(ValueError, match='voxel_size values must be positive'):
        ops.sparse_quantize(points, 0.0)
    with pytest.raises(ValueError, match='batch_indices must have shape'):
        ops.sparse_quantize(points, batch_indices=torch.zeros(3, dtype=torch.int32, device=cuda))
    with pytest.raises(ValueError, match="reduction must be 'sum' or 'mean'"):
        ops.voxelize(points, torch.zeros((4, 2), device=cuda), reduction='max')
    with pytest.raises(ValueError, match='matching rows'):
        ops.voxelize(points, torch.zeros((3, 2), device=cuda))


def test_devoxelize_known_answers(cuda):
    from mlx_lattice_b200 import ops
    from mlx_lattice_b200.core import SparseTensor

    for name, mode in (('devoxelize_nearest', 'nearest'), ('devoxelize_linear', 'linear'),
                       ('interpolate_linear_quarter', 'linear')):
        kat = KATS[name]
        voxels = SparseTensor(_dev(np.asarray(kat['coords'], np.int32), cuda),
                              _dev(np.asarray(kat['feats'], np.float32), cuda))
        got = ops.devoxelize(_dev(np.asarray(kat['points'], np.float32), cuda), voxels, interpolation=mode)
        assert np.allclose(got.cpu().numpy(), kat['out']), name
    kat = KATS['point_map_active_rows']
    coords = _dev(np.asarray(kat['coords'], np.int32), cuda)
    feats = _dev(np.asarray(kat['feats'], np.float32), cuda)
    point_map = ops.build_point_voxel_map(
        _dev(np.asarray(kat['points'], np.float32), cuda), coords,
        _dev(np.asarray(kat['voxel_active'], np.int32), cuda),
        point_active_rows=_dev(np.asarray(kat['point_active'], np.int32), cuda), interpolation='nearest')
    assert point_map.point_count == 2
    assert np.allclose(ops.interpolate_point_features(feats, point_map).cpu().numpy(), kat['out'])


@pytest.mark.parametrize('mode', ['nearest', 'linear'])
def test_point_voxel_map_matches_oracle(cuda, oracle, restatement, mode):
    from mlx_lattice_b200 import _ext

    rng = np.random.default_rng(51)
    voxels = np.unique(rng.integers(-12, 12, size=(30000, 4)).astype(np.int32), axis=0)
    voxels[:, 0] = np.abs(voxels[:, 0]) % 3
    voxels = np.concatenate([voxels, voxels[:500]])            # duplicates: first row wins
    voxels = voxels[rng.permutation(voxels.shape[0])]
    points = rng.uniform(-13, 13, size=(40000, 3)).astype(np.float32)
    points[::9] = np.round(points[::9])
    batch = rng.integers(0, 3, size=40000).astype(np.int32)
    p_active, v_active = [39000], [voxels.shape[0] - 100]
    size, origin = (1.0, 0.5, 2.0), (0.25, 0.0, -0.5)
    want_rows, want_weights = oracle.point_voxel_map(points, batch, p_active, voxels, v_active, size,
                                                     origin, mode)
    got_rows, got_weights = _ext.build_point_voxel_map(
        _dev(points, cuda), _dev(batch, cuda), _dev(np.asarray(p_active, np.int32), cuda),
        _dev(voxels, cuda), _dev(np.asarray(v_active, np.int32), cuda), size, origin, mode)
    assert np.array_equal(got_rows.cpu().numpy(), want_rows)
    assert np.array_equal(got_weights.cpu().numpy(), want_weights)
    feats = rng.normal(size=(voxels.shape[0], 6)).astype(np.float32)
    want = oracle.interpolate_point_features(feats, want_rows, want_weights)
    got = _ext.interpolate_point_features(_dev(feats, cuda), got_rows, got_weights).cpu().numpy()
    if oracle is restatement:
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    else:
        assert np.array_equal(got, want)
    _ext.check_status(cuda)


def test_voxelize_then_devoxelize_round_trip(cuda):
    """Nearest devoxelisation of mean-voxelised features returns, for every point, the mean of
    its own voxel: the voxel centre convention (floor on the way in, floor(x + 0.5) on the way
    back) differs by half a cell, so points are sampled at their voxel's integer corner."""
    from mlx_lattice_b200 import ops

    rng = np.random.default_rng(8)
    cells = rng.integers(0, 40, size=(20000, 3))
    points = _dev(cells.astype(np.float32), cuda)              # points on integer positions
    feats = _dev(rng.normal(size=(20000, 3)).astype(np.float32), cuda)
    x = ops.voxelize(points, feats, 1.0, reduction='mean')
    back = ops.devoxelize(points, x, 1.0, interpolation='nearest')
    quant = ops.sparse_quantize(points, 1.0)
    assert torch.equal(back, x.feats[quant.inverse_rows.long()])
