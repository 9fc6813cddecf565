"""Pins the CPU oracle: the numpy restatement (and the compiled reference when its
library is present) against (1) the known-answer vectors of the reference's own
tests and (2) outputs of the compiled reference stored in tests/golden."""

import json
import os

import numpy as np
import pytest

from oracle import reference, restatement

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
KATS = json.load(open(os.path.join(GOLDEN, 'reference_kats.json')))
BACKENDS = [restatement] + ([reference] if reference.available() else [])
IDS = ['restatement'] + (['compiled_reference'] if reference.available() else [])

LINE = np.asarray(KATS['line3'], np.int32)


@pytest.fixture(scope='module')
def golden():
    return np.load(os.path.join(GOLDEN, 'reference_outputs.npz'))


def _rel(golden, prefix):
    return {k.split('.', 1)[1]: golden[k] for k in golden.files if k.startswith(prefix + '.')}


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_known_answer_relations(backend):
    kat = KATS['forward_k311']
    assert backend.kernel_offsets((3, 1, 1)).tolist() == kat['offsets']
    rel = backend.build_kernel_relation(LINE, None, kernel_size=(3, 1, 1))
    e = kat['counts'][0]
    assert rel['counts'].tolist() == kat['counts']
    for key in ('in_rows', 'out_rows', 'kernel_ids', 'in_edge_ids', 'kernel_edge_ids'):
        assert rel[key][:e].tolist() == kat[key], key
    for key in ('row_offsets', 'in_row_offsets', 'kernel_row_offsets'):
        assert rel[key].tolist() == kat[key], key

    kat = KATS['target_k311']
    rel = backend.build_target_kernel_relation(LINE, np.asarray(kat['target'], np.int32),
                                               kernel_size=(3, 1, 1))
    assert rel['counts'].tolist() == kat['counts']
    for key in ('in_rows', 'out_rows', 'kernel_ids'):
        assert rel[key][:4].tolist() == kat[key]
    assert rel['row_offsets'].tolist() == kat['row_offsets']

    kat = KATS['strided_k1_s2']
    rel = backend.build_kernel_relation(np.asarray(kat['coords'], np.int32), None,
                                        kernel_size=1, stride=2)
    assert rel['counts'].tolist() == kat['counts']
    assert rel['out_coords'][:2].tolist() == kat['out_coords']
    assert rel['in_rows'][:2].tolist() == kat['in_rows']

    kat = KATS['generative_k211_s211']
    coords = np.asarray(kat['coords'], np.int32)
    gen = backend.build_generative_relation(coords, None, kernel_size=(2, 1, 1), stride=(2, 1, 1))
    tr = backend.build_transposed_kernel_relation(coords, None, kernel_size=(2, 1, 1), stride=(2, 1, 1))
    for rel in (gen, tr):
        assert rel['counts'].tolist() == kat['counts']
        assert rel['out_coords'][:2].tolist() == kat['out_coords']

    kat = KATS['igemm_view_k311']
    offs = backend.kernel_offsets((3, 1, 1))
    m, masks = backend.implicit_gemm_view(LINE, 3, LINE, 3, offs)
    assert m.tolist() == kat['out_in_map'] and masks.tolist() == kat['row_masks']
    target = np.asarray(KATS['target_k311']['target'], np.int32)
    m, masks = backend.implicit_gemm_view(LINE, 3, target, 2, offs)
    assert m.tolist() == kat['target_out_in_map'] and masks.tolist() == kat['target_row_masks']


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_known_answer_features(backend):
    kat = KATS['conv_k311']
    rel = backend.build_kernel_relation(LINE, None, kernel_size=(3, 1, 1))
    feats = np.asarray(kat['feats'], np.float32)
    w = np.asarray(kat['weight_dense5d_1x3x1x1x1'], np.float32).reshape(1, 3, 1, 1, 1)
    assert backend.sparse_conv(feats, w, rel, 3, 3).tolist() == kat['out']
    half = backend.sparse_conv(feats.astype(np.float16), w.astype(np.float16), rel, 3, 3)
    assert half.dtype == np.float16 and half.tolist() == kat['out']
    assert backend.sparse_conv(feats, np.ones_like(w), rel, 3, 3).tolist() == kat['ones_weight_out']
    trel = backend.build_target_kernel_relation(
        LINE, np.asarray(KATS['target_k311']['target'], np.int32), kernel_size=(3, 1, 1))
    assert backend.sparse_conv(feats, w, trel, 2, 3).tolist() == kat['target_out']

    kat = KATS['strided_conv_k1_s2']
    coords = np.asarray(KATS['strided_k1_s2']['coords'], np.int32)
    rel = backend.build_kernel_relation(coords, None, kernel_size=1, stride=2)
    out = backend.sparse_conv(np.asarray(kat['feats'], np.float32),
                              np.ones((1, 1, 1, 1, 1), np.float32), rel, 4, 1)
    assert out[:2].tolist() == kat['out'] and not out[2:].any()

    kat = KATS['transpose_k211_s211']
    coords = np.asarray(KATS['generative_k211_s211']['coords'], np.int32)
    rel = backend.build_transposed_kernel_relation(coords, None, kernel_size=(2, 1, 1), stride=(2, 1, 1))
    w = np.asarray(kat['weight'], np.float32).reshape(1, 2, 1, 1, 1)
    assert backend.sparse_conv(np.asarray(kat['feats'], np.float32), w, rel, 2, 2).tolist() == kat['out']

    kat = KATS['pool_k311_s1']
    rel = backend.build_kernel_relation(LINE, None, kernel_size=(3, 1, 1))
    feats = np.asarray(kat['feats'], np.float32)
    for mode in ('sum', 'max', 'avg'):
        out = backend.sparse_pool(feats, rel, input_exclusive=False, reduce=mode,
                                  out_capacity=3, n_kernels=3)
        assert out.tolist() == kat[mode]

    kat = KATS['pointwise']
    out = restatement.linear(np.asarray(kat['feats'], np.float32), np.asarray(kat['weight'], np.float32),
                             np.asarray(kat['bias'], np.float32))
    assert out.tolist() == kat['out']


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_relations_match_compiled_reference_outputs(backend, golden):
    g = golden
    cases = [
        ('subm_lidar', lambda: backend.build_submanifold_kernel_relation(g['in_lidar'])),
        ('subm_sphere', lambda: backend.build_submanifold_kernel_relation(g['in_sphere'])),
        ('k3s2_sphere', lambda: backend.build_kernel_relation(g['in_sphere'], None, 3, 2, 0, 1)),
        ('k2s2_dup', lambda: backend.build_kernel_relation(g['in_dup'], 1000, 2, 2, 0, 1)),
        ('k3s2p1_lidar', lambda: backend.build_kernel_relation(g['in_lidar'], None, 3, 2, 1, 1)),
        ('tr_k2s2', lambda: backend.build_transposed_kernel_relation(g['in_sphere'][:400], 350, 2, 2, 0, 1)),
        ('tr_k3s2p1', lambda: backend.build_transposed_kernel_relation(g['in_sphere'][:400], None, 3, 2, 1, 1)),
        ('gen_k2s2', lambda: backend.build_generative_relation(g['in_lidar'][:300], None, 2, 2)),
        ('target_k2s2', lambda: backend.build_target_kernel_relation(
            g['in_sphere'], g['in_target'], 2000, 500, 2, 2, 0, 1)),
    ]
    for prefix, build in cases:
        want = _rel(g, prefix)
        got = build()
        for key, value in want.items():
            assert np.array_equal(got[key], value), (prefix, key)
    coords, count = backend.downsample_coords(g['in_sphere'], 2)
    assert np.array_equal(coords, g['downsample.coords']) and np.array_equal(count, g['downsample.count'])
    m, masks = backend.implicit_gemm_view(g['in_sphere'], 2000, g['in_sphere'], 2200,
                                          backend.kernel_offsets(3))
    assert np.array_equal(m, g['igemm.out_in_map']) and np.array_equal(masks, g['igemm.row_masks'])
    for join in ('inner', 'left', 'right', 'outer'):
        res = backend.sparse_alignment(g['in_sphere'][:1500], 1400, g['in_dup'], 1100, join)
        for name, value in zip(('coords', 'count', 'lhs_rows', 'rhs_rows'), res):
            assert np.array_equal(value, g[f'align_{join}.{name}']), (join, name)


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_features_match_compiled_reference_outputs(backend, golden):
    g = golden
    rel = _rel(g, 'subm_sphere')
    n = g['in_sphere'].shape[0]

    def rel_err(a, b):
        b = b.astype(np.float64)
        return np.abs(a.astype(np.float64) - b).max() / np.abs(b).max()

    # float32: 1e-5 relative (summation order may differ in the restatement)
    assert rel_err(backend.sparse_conv(g['in_feats32'], g['in_w32'], rel, n, 27), g['conv32']) <= 1e-5
    # float16, 32 -> 64 channels: the reference route that re-rounds every multiply-add
    assert rel_err(backend.sparse_conv(g['in_feats16'], g['in_w16'], rel, n, 27), g['conv16']) <= 2e-3
    for bits in (4, 8):
        q = restatement.quantize_weight(g['in_w16'], 32, bits)
        # the quantiser itself is deterministic: same packed arrays as when the fixture was made
        assert np.array_equal(q['weight'], g[f'q{bits}.weight'])
        assert np.array_equal(q['scales'], g[f'q{bits}.scales'])
        assert np.array_equal(q['biases'], g[f'q{bits}.biases'])
        got = backend.sparse_quantized_conv(
            g['in_feats16'], q['weight'], q['scales'], q['biases'], rel, n, 27, 32, 64, 32, 32, bits)
        assert rel_err(got, g[f'qconv{bits}']) <= 1e-3
    prel = _rel(g, 'k3s2_sphere')
    for mode in ('sum', 'max', 'avg'):
        got = backend.sparse_pool(g['in_feats32'], prel, input_exclusive=False, reduce=mode,
                                  out_capacity=n, n_kernels=27)
        assert np.array_equal(got, g[f'pool_{mode}']), mode


def test_quantizer_roundtrip_and_package_agreement():
    """Affine quantiser: reconstruction error within one quantisation step, packed format decodes
    with the reference's rule, and the package's torch quantiser emits the same arrays."""
    import torch

    from mlx_lattice_b200.core import dequantize_weight, quantize_weight

    rng = np.random.default_rng(5)
    for shape in ((48, 40), (27, 40, 16), (24, 3, 3, 3, 64)):
        for bits in (4, 8):
            for dtype in (np.float16, np.float32):
                w = (rng.normal(size=shape) * 0.05).astype(dtype)
                q = restatement.quantize_weight(w, 32, bits)
                deq = restatement.dequantize_weight(q).astype(np.float32)
                groups_step = (np.abs(w).max() * 2) / (2 ** bits - 1)
                assert np.abs(deq - w.astype(np.float32)).max() <= groups_step + 1e-3
                pq = quantize_weight(torch.from_numpy(w), group_size=32, bits=bits)
                assert np.array_equal(pq.weight.numpy().view(np.uint32), q['weight'])
                assert np.array_equal(pq.scales.numpy(), q['scales'])
                assert np.array_equal(pq.biases.numpy(), q['biases'])
                assert pq.storage_in_channels == q['storage_in_channels']
                assert np.array_equal(dequantize_weight(pq).numpy(), restatement.dequantize_weight(q))


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_quantization_matches_compiled_reference_outputs(backend, golden):
    g = golden
    active = np.asarray([5500], np.int32)
    got = backend.sparse_quantize(g['in_points'], g['in_point_batch'], active, (0.5, 1.0, 2.0),
                                  (0.25, -0.5, 0.0))
    for name, value in zip(('coords', 'count', 'inverse', 'counts'), got):
        assert np.array_equal(value, g[f'quantize.{name}']), name
    for mode in ('mean', 'sum'):
        vox = backend.voxelize_features(g['in_point_feats'], got[2], got[3], active, mode)
        assert np.allclose(vox, g[f'voxelize_{mode}'], rtol=1e-5, atol=1e-6), mode


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_known_answer_quantization(backend):
    """Point -> voxel front end against the reference's own known answers."""
    kat = KATS['quantize_ordered']
    coords, count, inverse, counts = backend.sparse_quantize(
        np.asarray(kat['points'], np.float32), np.asarray(kat['batches'], np.int32), None,
        kat['voxel_size'], 0.0)
    n = kat['active_rows'][0]
    assert count.tolist() == kat['active_rows']
    assert coords[:n].tolist() == kat['coords'] and not coords[n:].any()
    assert inverse.tolist() == kat['inverse_rows']
    assert counts[:n].tolist() == kat['counts']

    kat = KATS['quantize_origin_active']
    coords, count, inverse, counts = backend.sparse_quantize(
        np.asarray(kat['points'], np.float32), None, np.asarray(kat['point_active'], np.int32),
        kat['voxel_size'], kat['origin'])
    n = kat['active_rows'][0]
    assert count.tolist() == kat['active_rows']
    assert coords[:n].tolist() == kat['coords']
    assert inverse.tolist() == kat['inverse_rows']
    assert counts.tolist() == kat['counts']

    kat = KATS['voxelize_mean_sum']
    points = np.asarray(kat['points'], np.float32)
    feats = np.asarray(kat['feats'], np.float32)
    coords, count, inverse, counts = backend.sparse_quantize(points, None, None, 1.0, 0.0)
    n = int(count[0])
    assert coords[:n].tolist() == kat['coords']
    active = np.asarray([points.shape[0]], np.int32)
    mean = backend.voxelize_features(feats, inverse, counts, active, 'mean')
    total = backend.voxelize_features(feats, inverse, counts, active, 'sum')
    assert np.allclose(mean[:n], kat['mean']) and np.allclose(total[:n], kat['sum'])
    assert not mean[n:].any() and not total[n:].any()


@pytest.mark.skipif(not reference.available(), reason='compiled reference not built')
def test_quantization_restatement_matches_compiled_reference():
    rng = np.random.default_rng(41)
    points = (rng.normal(size=(20000, 3)) * 7.0).astype(np.float32)
    batch = rng.integers(0, 3, size=20000).astype(np.int32)
    active = np.asarray([19000], np.int32)
    got = restatement.sparse_quantize(points, batch, active, (0.5, 0.25, 1.0), (0.1, -0.3, 2.0))
    want = reference.sparse_quantize(points, batch, active, (0.5, 0.25, 1.0), (0.1, -0.3, 2.0))
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    feats = rng.normal(size=(20000, 5)).astype(np.float32)
    for mode in ('mean', 'sum'):
        g = restatement.voxelize_features(feats[:3000], got[2][:3000], got[3], np.asarray([3000], np.int32), mode)
        w = reference.voxelize_features(feats[:3000], want[2][:3000], want[3], np.asarray([3000], np.int32), mode)
        assert np.allclose(g, w, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize('backend', BACKENDS, ids=IDS)
def test_known_answer_devoxelize(backend):
    """Point-voxel map and interpolation against the reference's own known answers."""
    for name, mode in (('devoxelize_nearest', 'nearest'), ('devoxelize_linear', 'linear'),
                       ('point_map_active_rows', 'nearest'), ('interpolate_linear_quarter', 'linear')):
        kat = KATS[name]
        coords = np.asarray(kat['coords'], np.int32)
        rows, weights = backend.point_voxel_map(
            np.asarray(kat['points'], np.float32), None, kat.get('point_active'), coords,
            kat.get('voxel_active'), 1.0, 0.0, mode)
        out = backend.interpolate_point_features(np.asarray(kat['feats'], np.float32), rows, weights)
        assert np.allclose(out, kat['out']), name


@pytest.mark.skipif(not reference.available(), reason='compiled reference not built')
def test_point_voxel_map_restatement_matches_compiled_reference():
    rng = np.random.default_rng(43)
    voxels = np.unique(rng.integers(-6, 6, size=(3000, 4)).astype(np.int32), axis=0)
    voxels[:, 0] = np.abs(voxels[:, 0]) % 2
    voxels = voxels[rng.permutation(voxels.shape[0])]
    points = (rng.uniform(-7, 7, size=(5000, 3))).astype(np.float32)
    points[::9] = np.round(points[::9])
    batch = rng.integers(0, 2, size=5000).astype(np.int32)
    feats = rng.normal(size=(voxels.shape[0], 3)).astype(np.float32)
    for mode in ('nearest', 'linear'):
        got = restatement.point_voxel_map(points, batch, [4800], voxels, [voxels.shape[0] - 7],
                                          (1.0, 0.5, 2.0), (0.25, 0.0, -0.5), mode)
        want = reference.point_voxel_map(points, batch, [4800], voxels, [voxels.shape[0] - 7],
                                         (1.0, 0.5, 2.0), (0.25, 0.0, -0.5), mode)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), mode
        g = restatement.interpolate_point_features(feats, *got)
        w = reference.interpolate_point_features(feats, *want)
        assert np.allclose(g, w, rtol=1e-5, atol=1e-6)
