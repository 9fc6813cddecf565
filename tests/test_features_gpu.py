"""Sparse-conv contraction, pooling and pointwise feature ops on the GPU against
the oracle. Tolerances are the parity contract's: fp16 activations
max|y - ref| <= 2e-3 * max|ref|; fp32 <= 1e-5 relative."""

import numpy as np
import pytest
import torch

from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu

FP16_TOL = 2e-3
FP32_TOL = 1e-5


def _dev(array, cuda):
    return torch.from_numpy(np.ascontiguousarray(array)).to(cuda)


def _rel_dev(rel, cuda):
    return {k: _dev(v, cuda) for k, v in rel.items()}


def _max_rel_err(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    scale = np.abs(want).max()
    return np.abs(got - want).max() / (scale if scale > 0 else 1.0)


def _plan(cuda, r, in_capacity, out_capacity, n_kernels, row_order):
    from mlx_lattice_b200 import _ext

    return _ext.build_conv_plan(r['in_rows'], r['kernel_ids'], r['counts'], r['row_offsets'],
                                in_capacity, out_capacity, n_kernels, row_order)


def _conv(cuda, feats, weights, rel, out_capacity, n_kernels, bias=None, row_order=None,
          with_plan=False):
    from mlx_lattice_b200 import _ext

    r = _rel_dev(rel, cuda)
    order = None if row_order is None else _dev(row_order, cuda)
    plan = _plan(cuda, r, feats.shape[0], out_capacity, n_kernels, order) if with_plan else None
    if with_plan:
        return _ext.sparse_conv_features(
            _dev(feats, cuda), _dev(weights, cuda), r['in_rows'], r['out_rows'], r['kernel_ids'],
            r['counts'], r['row_offsets'], out_capacity=out_capacity, n_kernels=n_kernels,
            bias=None if bias is None else _dev(bias, cuda), row_order=order,
            plan=plan).cpu().numpy()
    out = _ext.sparse_conv_features(
        _dev(feats, cuda), _dev(weights, cuda), r['in_rows'], r['out_rows'], r['kernel_ids'],
        r['counts'], r['row_offsets'], out_capacity=out_capacity, n_kernels=n_kernels,
        bias=None if bias is None else _dev(bias, cuda),
        row_order=None if row_order is None else _dev(row_order, cuda))
    return out.cpu().numpy()


def _qconv(cuda, feats, q, rel, out_capacity, n_kernels, row_order=None, with_plan=False):
    from mlx_lattice_b200 import _ext

    r = _rel_dev(rel, cuda)
    if with_plan:
        order = None if row_order is None else _dev(row_order, cuda)
        plan = _plan(cuda, r, feats.shape[0], out_capacity, n_kernels, order)
        return _ext.sparse_quantized_conv_features(
            _dev(feats, cuda), _dev(q['weight'].view(np.int32), cuda), _dev(q['scales'], cuda),
            _dev(q['biases'], cuda), r['in_rows'], r['out_rows'], r['kernel_ids'], r['counts'],
            r['row_offsets'], None, None, None, out_capacity, n_kernels, q['in_channels'],
            q['out_channels'], q['storage_in_channels'], q['group_size'], q['bits'],
            row_order=order, plan=plan).cpu().numpy()
    out = _ext.sparse_quantized_conv_features(
        _dev(feats, cuda), _dev(q['weight'].view(np.int32), cuda), _dev(q['scales'], cuda),
        _dev(q['biases'], cuda), r['in_rows'], r['out_rows'], r['kernel_ids'], r['counts'],
        r['row_offsets'], None, None, None, out_capacity, n_kernels, q['in_channels'],
        q['out_channels'], q['storage_in_channels'], q['group_size'], q['bits'],
        row_order=None if row_order is None else _dev(row_order, cuda))
    return out.cpu().numpy()


@pytest.fixture(scope='module')
def sphere(oracle):
    coords = synthetic.sphere_plane_batch(0, 1, 20000, 96)
    return coords, oracle.build_submanifold_kernel_relation(coords)


def test_reference_known_answer_conv(cuda, oracle):
    # tests/ops/test_conv.py:44-62 of the reference: 3-point line, K=(3,1,1)
    coords = np.array([[0, 0, 0, 0], [0, 1, 0, 0], [0, 2, 0, 0]], np.int32)
    rel = oracle.build_kernel_relation(coords, None, kernel_size=(3, 1, 1))
    feats = np.array([[1.0], [2.0], [3.0]], np.float32)
    weights = np.array([[[1.0]], [[2.0]], [[3.0]]], np.float32)
    assert _conv(cuda, feats, weights, rel, 3, 3).ravel().tolist() == [8.0, 14.0, 8.0]
    half = _conv(cuda, feats.astype(np.float16), weights.astype(np.float16), rel, 3, 3)
    assert half.dtype == np.float16 and half.ravel().tolist() == [8.0, 14.0, 8.0]


@pytest.mark.parametrize('c_in,c_out', [(32, 32), (5, 7), (16, 48), (64, 20)])
def test_float32_conv(cuda, oracle, sphere, c_in, c_out):
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(c_in * 100 + c_out)
    feats = rng.normal(size=(n, c_in)).astype(np.float32)
    w5 = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float32)
    want = oracle.sparse_conv(feats, w5, rel, n, 27)
    got = _conv(cuda, feats, w5, rel, n, 27)
    assert _max_rel_err(got, want) <= FP32_TOL
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    wk = np.ascontiguousarray(w5.transpose(1, 2, 3, 4, 0).reshape(27, c_in, c_out))
    assert np.array_equal(_conv(cuda, feats, wk, rel, n, 27), got)


@pytest.mark.parametrize('c_in,c_out', [(32, 32), (64, 64), (32, 64), (64, 128), (96, 96),
                                        (128, 256), (256, 256), (8, 24), (4, 32), (32, 20)])
def test_float16_conv(cuda, oracle, sphere, c_in, c_out):
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(c_in * 1000 + c_out)
    feats = rng.normal(size=(n, c_in)).astype(np.float16)
    w5 = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float16)
    # square 16/32/64 channels: the reference accumulates in float32; other shapes
    # re-round to float16 after every multiply-add, for which the reference's own
    # parity tolerance is 2e-2 (tests/cases/conv_cases.py:17)
    square = c_in == c_out and c_in in (16, 32, 64)
    want = oracle.sparse_conv(feats, w5, rel, n, 27)
    got = _conv(cuda, feats, w5, rel, n, 27)
    assert _max_rel_err(got, want) <= (FP16_TOL if square else 2e-2)
    exact = oracle.sparse_conv(feats.astype(np.float32), w5.astype(np.float32), rel, n, 27)
    assert _max_rel_err(got, exact) <= FP16_TOL


@pytest.mark.parametrize('bits', [4, 8])
@pytest.mark.parametrize('c_in,c_out', [(32, 32), (64, 128), (96, 96), (128, 64), (256, 256), (40, 16)])
def test_quantized_conv_float16(cuda, oracle, restatement, sphere, bits, c_in, c_out):
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(bits * 7 + c_in + c_out)
    feats = rng.normal(size=(n, c_in)).astype(np.float16)
    w5 = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float16)
    q = restatement.quantize_weight(w5, 32, bits)
    want = oracle.sparse_quantized_conv(
        feats, q['weight'], q['scales'], q['biases'], rel, n, 27, c_in, c_out,
        q['storage_in_channels'], 32, bits)
    got = _qconv(cuda, feats, q, rel, n, 27)
    assert _max_rel_err(got, want) <= FP16_TOL


@pytest.mark.parametrize('c_in,c_out', [(32, 32), (64, 128), (128, 64), (96, 48), (256, 256), (32, 16),
                                        (64, 16), (128, 48), (192, 240)])
def test_conv_with_gather_plan(cuda, oracle, restatement, sphere, c_in, c_out):
    """The plan-driven tensor-core kernel: same bits as the relation-walking one, in
    natural row order and under a permutation, fp16 and packed int4 weights."""
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(c_in * 31 + c_out)
    feats = rng.normal(size=(n, c_in)).astype(np.float16)
    w5 = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float16)
    bias = rng.normal(size=c_out).astype(np.float16)
    exact = oracle.sparse_conv(feats.astype(np.float32), w5.astype(np.float32), rel, n, 27)
    base = _conv(cuda, feats, w5, rel, n, 27)
    got = _conv(cuda, feats, w5, rel, n, 27, with_plan=True)
    assert _max_rel_err(got, exact) <= FP16_TOL
    assert np.array_equal(got, base)
    order = np.random.default_rng(9).permutation(n).astype(np.int32)
    assert np.array_equal(_conv(cuda, feats, w5, rel, n, 27, row_order=order, with_plan=True), base)
    with_bias = _conv(cuda, feats, w5, rel, n, 27, bias=bias, with_plan=True)
    assert np.array_equal(with_bias, _conv(cuda, feats, w5, rel, n, 27, bias=bias))
    q = restatement.quantize_weight(w5, 32, 4)
    want = oracle.sparse_quantized_conv(
        feats, q['weight'], q['scales'], q['biases'], rel, n, 27, c_in, c_out,
        q['storage_in_channels'], 32, 4)
    got_q = _qconv(cuda, feats, q, rel, n, 27, row_order=order, with_plan=True)
    assert _max_rel_err(got_q, want) <= FP16_TOL
    assert np.array_equal(got_q, _qconv(cuda, feats, q, rel, n, 27))


def test_gather_plan_from_row_masks(cuda, oracle, sphere):
    """The plan builder given the relation's row masks (what the kernel map writes) makes
    the plan it makes from a walk over the edges: same convolution bits."""
    from mlx_lattice_b200 import _ext

    coords, rel = sphere
    n = coords.shape[0]
    r = _rel_dev(rel, cuda)
    e = int(rel['counts'][0])
    masks = np.zeros((n, 1), np.int32)
    np.bitwise_or.at(masks[:, 0], rel['out_rows'][:e], (1 << rel['kernel_ids'][:e]).astype(np.int32))
    order = _dev(np.random.default_rng(3).permutation(n).astype(np.int32), cuda)
    rng = np.random.default_rng(41)
    feats = _dev(rng.normal(size=(n, 64)).astype(np.float16), cuda)
    w5 = _dev((rng.normal(size=(64, 3, 3, 3, 64)) * 0.05).astype(np.float16), cuda)
    outs = []
    for row_masks in (None, _dev(masks, cuda)):
        plan = _ext.build_conv_plan(r['in_rows'], r['kernel_ids'], r['counts'], r['row_offsets'], n, n, 27,
                                    order, row_masks)
        outs.append(_ext.sparse_conv_features(
            feats, w5, r['in_rows'], r['out_rows'], r['kernel_ids'], r['counts'], r['row_offsets'],
            out_capacity=n, n_kernels=27, row_order=order, plan=plan))
    assert torch.equal(outs[0], outs[1])
    _ext.check_status()
    with pytest.raises(ValueError, match='row_masks must hold one int32 word per output row'):
        _ext.build_conv_plan(r['in_rows'], r['kernel_ids'], r['counts'], r['row_offsets'], n, n, 27, order,
                             _dev(masks[:-1], cuda))


def test_gather_plan_layout(cuda, oracle, sphere):
    """The plan buffer as the header describes it: per tile (mask, first vector), the closing
    entry (tiles in use, vector total), the tile order (every tile once, by falling number
    of used offsets, equal counts in tile order), and the row vectors in gather order."""
    from mlx_lattice_b200 import _ext

    coords, rel = sphere
    n = coords.shape[0]
    active = n - 300                                   # some tiles at the end use no offset
    rel = oracle.build_submanifold_kernel_relation(coords, active)
    r = _rel_dev(rel, cuda)
    order = np.random.default_rng(21).permutation(n).astype(np.int32)
    plan = _ext.build_conv_plan(r['in_rows'], r['kernel_ids'], r['counts'], r['row_offsets'], n, n, 27,
                                _dev(order, cuda)).cpu().numpy()
    _ext.check_status()
    tiles = (n + 255) // 256
    info_bytes = -(-(tiles + 1) * 8 // 256) * 256
    order_bytes = -(-tiles * 4 // 256) * 256
    info = plan[:(tiles + 1) * 8].view(np.int32).reshape(tiles + 1, 2)
    tile_order = plan[info_bytes:info_bytes + tiles * 4].view(np.int32)
    vectors = plan[info_bytes + order_bytes:].view(np.int32)
    # expected masks from the relation
    e = int(rel['counts'][0])
    row_masks = np.zeros(n, np.int64)
    np.bitwise_or.at(row_masks, rel['out_rows'][:e], np.int64(1) << rel['kernel_ids'][:e].astype(np.int64))
    padded = np.zeros(tiles * 256, np.int64)
    padded[:n] = row_masks[order]
    masks = np.bitwise_or.reduce(padded.reshape(tiles, 256), axis=1)
    counts = np.array([bin(int(m)).count('1') for m in masks])
    assert np.array_equal(info[:tiles, 0].astype(np.int64), masks)
    assert np.array_equal(info[:tiles, 1], np.concatenate([[0], np.cumsum(counts)[:-1]]))
    assert info[tiles, 0] == int((counts > 0).sum()) and info[tiles, 1] == int(counts.sum())
    assert np.array_equal(tile_order, np.argsort(-counts, kind='stable'))
    # row vectors: tile row r sits at (r % 32) * 8 + r / 32
    in_of = {}
    for edge in range(e):
        in_of[(int(rel['out_rows'][edge]), int(rel['kernel_ids'][edge]))] = int(rel['in_rows'][edge])
    slot = lambda row: (row % 32) * 8 + row // 32
    rng = np.random.default_rng(2)
    for tile in rng.choice(tiles, size=6, replace=False):
        used = [k for k in range(27) if (int(masks[tile]) >> k) & 1]
        for o, k in enumerate(used):
            vector = vectors[(info[tile, 1] + o) * 256:(info[tile, 1] + o + 1) * 256]
            for row in range(0, 256, 7):
                position = tile * 256 + row
                want = in_of.get((int(order[position]), k), -1) if position < n else -1
                assert vector[slot(row)] == want


def test_gather_plan_strided_and_padding_rows(cuda, oracle, restatement):
    """k=2, s=2 relation whose output capacity exceeds the live rows: plan tiles beyond
    the live rows are empty and their output rows are zero."""
    coords = synthetic.sphere_plane_batch(1, 2, 15000, 128)
    n = coords.shape[0]
    rel = oracle.build_kernel_relation(coords, None, kernel_size=2, stride=2)
    n_out = int(rel['counts'][1])
    rng = np.random.default_rng(12)
    feats = rng.normal(size=(n, 64)).astype(np.float16)
    w5 = (rng.normal(size=(128, 2, 2, 2, 64)) * 0.05).astype(np.float16)
    q = restatement.quantize_weight(w5, 32, 4)
    base = _qconv(cuda, feats, q, rel, n, 8)
    got = _qconv(cuda, feats, q, rel, n, 8, with_plan=True)
    assert np.array_equal(got, base)
    assert not got[n_out:].any()
    order = np.random.default_rng(6).permutation(n).astype(np.int32)
    assert np.array_equal(_qconv(cuda, feats, q, rel, n, 8, row_order=order, with_plan=True), base)


@pytest.mark.parametrize('bits', [4, 8])
def test_in_register_dequant_route(cuda, oracle, restatement, sphere, bits, monkeypatch):
    """LAT_TC_DEQUANT=register keeps the codes packed until the tensor-core kernel's
    producers convert them in registers (code * scale + bias, fp16 fma)."""
    monkeypatch.setenv('LAT_TC_DEQUANT', 'register')
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(100 + bits)
    for c_in, c_out in ((64, 64), (128, 96), (32, 48)):
        feats = rng.normal(size=(n, c_in)).astype(np.float16)
        w5 = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float16)
        q = restatement.quantize_weight(w5, 32, bits)
        want = oracle.sparse_quantized_conv(
            feats, q['weight'], q['scales'], q['biases'], rel, n, 27, c_in, c_out,
            q['storage_in_channels'], 32, bits)
        order = np.random.default_rng(4).permutation(n).astype(np.int32)
        got = _qconv(cuda, feats, q, rel, n, 27, row_order=order)
        assert _max_rel_err(got, want) <= FP16_TOL
        # a plan is accepted and ignored on this route
        assert np.array_equal(_qconv(cuda, feats, q, rel, n, 27, row_order=order, with_plan=True), got)


def test_gather_plan_edge_shapes(cuda, oracle):
    """Plans over tiny and empty relations, and capacities that are not tile multiples."""
    rng = np.random.default_rng(77)
    for rows, active in ((1, 1), (5, 5), (257, 257), (300, 0), (513, 100)):
        coords = np.zeros((rows, 4), np.int32)
        coords[:, 1] = np.arange(rows) % 23
        coords[:, 2] = np.arange(rows) // 23
        rel = oracle.build_submanifold_kernel_relation(coords, active)
        feats = rng.normal(size=(rows, 32)).astype(np.float16)
        w5 = (rng.normal(size=(32, 3, 3, 3, 32)) * 0.1).astype(np.float16)
        want = oracle.sparse_conv(feats.astype(np.float32), w5.astype(np.float32), rel, rows, 27)
        got = _conv(cuda, feats, w5, rel, rows, 27, with_plan=True)
        assert got.shape == (rows, 32)
        assert _max_rel_err(got, want) <= FP16_TOL
        assert not got[active:].any()
        assert np.array_equal(got, _conv(cuda, feats, w5, rel, rows, 27))


def test_quantized_conv_float32_and_group64(cuda, oracle, restatement, sphere):
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(3)
    feats = rng.normal(size=(n, 64)).astype(np.float32)
    w5 = (rng.normal(size=(32, 3, 3, 3, 64)) * 0.05).astype(np.float32)
    q = restatement.quantize_weight(w5, 64, 4)
    want = oracle.sparse_quantized_conv(
        feats, q['weight'], q['scales'], q['biases'], rel, n, 27, 64, 32, 64, 64, 4)
    assert _max_rel_err(_qconv(cuda, feats, q, rel, n, 27), want) <= FP32_TOL


def test_strided_quantized_conv_config1_shape(cuda, oracle, restatement):
    """k=2, s=2, int4 g32, 64 -> 128 on a sphere+plane cloud: padding rows are zero."""
    coords = synthetic.sphere_plane_batch(1, 2, 15000, 128)
    n = coords.shape[0]
    rel = oracle.build_kernel_relation(coords, None, kernel_size=2, stride=2)
    n_out = int(rel['counts'][1])
    rng = np.random.default_rng(11)
    feats = rng.normal(size=(n, 64)).astype(np.float16)
    w5 = (rng.normal(size=(128, 2, 2, 2, 64)) * 0.05).astype(np.float16)
    q = restatement.quantize_weight(w5, 32, 4)
    want = oracle.sparse_quantized_conv(
        feats, q['weight'], q['scales'], q['biases'], rel, n, 8, 64, 128, 64, 32, 4)
    got = _qconv(cuda, feats, q, rel, n, 8)
    assert _max_rel_err(got, want) <= FP16_TOL
    assert not got[n_out:].any()
    order = np.random.default_rng(5).permutation(n).astype(np.int32)
    assert np.array_equal(_qconv(cuda, feats, q, rel, n, 8, row_order=order), got)


def test_bias_and_determinism(cuda, oracle, sphere):
    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(17)
    feats = rng.normal(size=(n, 32)).astype(np.float16)
    w5 = (rng.normal(size=(64, 3, 3, 3, 32)) * 0.05).astype(np.float16)
    bias = rng.normal(size=64).astype(np.float16)
    plain = _conv(cuda, feats, w5, rel, n, 27)
    with_bias = _conv(cuda, feats, w5, rel, n, 27, bias=bias)
    assert np.array_equal(with_bias, (plain.astype(np.float32) + bias.astype(np.float32)).astype(np.float16))
    assert np.array_equal(_conv(cuda, feats, w5, rel, n, 27), plain)


@pytest.mark.parametrize('reduce', ['sum', 'max', 'avg'])
def test_sparse_pool(cuda, oracle, reduce):
    from mlx_lattice_b200 import _ext

    coords = synthetic.lidar_batch(3, 2, 12000)
    n = coords.shape[0]
    rng = np.random.default_rng(23)
    for spec in (dict(kernel_size=3, stride=2), dict(kernel_size=2, stride=2)):
        rel = oracle.build_kernel_relation(coords, None, **spec)
        volume = spec['kernel_size'] ** 3
        for channels in (96, 7, 130):
            feats = rng.normal(size=(n, channels)).astype(np.float32)
            want = oracle.sparse_pool(feats, rel, input_exclusive=False, reduce=reduce,
                                      out_capacity=n, n_kernels=volume)
            r = _rel_dev(rel, cuda)
            got = _ext.sparse_pool_features(
                _dev(feats, cuda), r['in_rows'], r['out_rows'], r['kernel_ids'], r['row_offsets'],
                r['counts'], False, reduce, n, volume).cpu().numpy()
            assert np.array_equal(got, want)
    with pytest.raises(ValueError, match='pooling currently supports float32'):
        _ext.sparse_pool_features(
            _dev(feats.astype(np.float16), cuda), r['in_rows'], r['out_rows'], r['kernel_ids'],
            r['row_offsets'], r['counts'], False, reduce, n, volume)


def test_global_pool_linear_batchnorm(cuda, restatement):
    from mlx_lattice_b200 import _ext

    rng = np.random.default_rng(29)
    counts = (4000, 0, 2500, 1)
    rows = sum(counts)
    feats = rng.normal(size=(rows, 192)).astype(np.float32)
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=cuda)
    for mode in ('sum', 'avg'):
        got = _ext.global_pool(_dev(feats, cuda), offsets, mode).cpu().numpy()
        want = restatement.global_pool(feats, counts, mode)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    nonempty = (4000, 2500, 1)
    offs2 = torch.tensor(np.concatenate([[0], np.cumsum(nonempty)]), dtype=torch.int32, device=cuda)
    got = _ext.global_pool(_dev(feats[: sum(nonempty)], cuda), offs2, 'max').cpu().numpy()
    assert np.array_equal(got, restatement.global_pool(feats[: sum(nonempty)], nonempty, 'max'))

    x16 = rng.normal(size=(5000, 96)).astype(np.float16)
    w = (rng.normal(size=(192, 96)) * 0.1).astype(np.float16)
    b = rng.normal(size=192).astype(np.float16)
    got = _ext.linear(_dev(x16, cuda), _dev(w, cuda), _dev(b, cuda)).cpu().numpy()
    assert _max_rel_err(got, restatement.linear(x16, w, b)) <= FP16_TOL
    for bits in (4, 8):
        q = restatement.quantize_weight(w, 32, bits)
        got = _ext.quantized_linear(
            _dev(x16, cuda), _dev(q['weight'][0].view(np.int32), cuda), _dev(q['scales'][0], cuda),
            _dev(q['biases'][0], cuda), 192, 96, 32, bits).cpu().numpy()
        assert _max_rel_err(got, restatement.quantized_matmul(x16, q)) <= FP16_TOL
    # few output channels (a head): the one-thread-per-row kernel
    wn = (rng.normal(size=(20, 96)) * 0.1).astype(np.float16)
    bn = rng.normal(size=20).astype(np.float16)
    got = _ext.linear(_dev(x16, cuda), _dev(wn, cuda), _dev(bn, cuda)).cpu().numpy()
    assert _max_rel_err(got, restatement.linear(x16, wn, bn)) <= FP16_TOL
    for bits in (4, 8):
        q = restatement.quantize_weight(wn, 32, bits)
        got = _ext.quantized_linear(
            _dev(x16, cuda), _dev(q['weight'][0].view(np.int32), cuda), _dev(q['scales'][0], cuda),
            _dev(q['biases'][0], cuda), 20, 96, 32, bits).cpu().numpy()
        assert _max_rel_err(got, restatement.quantized_matmul(x16, q)) <= FP16_TOL
    xn = rng.normal(size=(3001, 24)).astype(np.float32)
    wn32 = rng.normal(size=(7, 24)).astype(np.float32)
    got = _ext.linear(_dev(xn, cuda), _dev(wn32, cuda)).cpu().numpy()
    assert _max_rel_err(got, restatement.linear(xn, wn32)) <= FP32_TOL
    x32 = rng.normal(size=(3000, 20)).astype(np.float32)
    w32 = rng.normal(size=(33, 20)).astype(np.float32)
    got = _ext.linear(_dev(x32, cuda), _dev(w32, cuda)).cpu().numpy()
    assert _max_rel_err(got, restatement.linear(x32, w32)) <= FP32_TOL

    mean = (rng.normal(size=96) * 0.1).astype(np.float16)
    var = rng.uniform(0.5, 1.5, size=96).astype(np.float16)
    gamma = np.ones(96, np.float16)
    beta = np.zeros(96, np.float16)
    want = restatement.relu(restatement.batch_norm(x16, gamma, beta, mean, var, 1e-5))
    got = _ext.batch_norm_relu(
        _dev(x16, cuda), _dev(gamma, cuda), _dev(beta, cuda), _dev(mean, cuda), _dev(var, cuda),
        1e-5, True).cpu().numpy()
    assert _max_rel_err(got, want) <= FP16_TOL
    assert np.array_equal(_ext.relu(_dev(x16, cuda)).cpu().numpy(), restatement.relu(x16))


@pytest.mark.parametrize('c_first,c_second,c_out', [(128, 128, 128), (64, 64, 64), (32, 32, 32),
                                                   (32, 64, 32), (64, 32, 48), (8, 24, 16)])
def test_two_source_conv_equals_conv_of_concatenation(cuda, oracle, sphere, c_first, c_second, c_out):
    """A convolution that reads the channel concatenation of two tensors in place
    (`feats2`) gives the bits of the same convolution over the written concatenation,
    and stays within the fp16 tolerance of the oracle."""
    from mlx_lattice_b200 import _ext

    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(c_first * 31 + c_second)
    first = rng.normal(size=(n, c_first)).astype(np.float16)
    second = rng.normal(size=(n, c_second)).astype(np.float16)
    both = np.concatenate([first, second], axis=1)
    w5 = (rng.normal(size=(c_out, 3, 3, 3, c_first + c_second)) * 0.05).astype(np.float16)
    r = _rel_dev(rel, cuda)
    plan = _plan(cuda, r, n, n, 27, None)
    args = (r['in_rows'], r['out_rows'], r['kernel_ids'], r['counts'], r['row_offsets'])
    joined = _ext.sparse_conv_features(_dev(both, cuda), _dev(w5, cuda), *args, out_capacity=n,
                                       n_kernels=27, plan=plan).cpu().numpy()
    # the second source as a strided view: rows of a wider array
    wide = _dev(np.concatenate([second, second], axis=1), cuda)[:, :c_second]
    in_place = _ext.sparse_conv_features(_dev(first, cuda), _dev(w5, cuda), *args, out_capacity=n,
                                         n_kernels=27, plan=plan, feats2=wide).cpu().numpy()
    assert np.array_equal(in_place, joined)
    exact = oracle.sparse_conv(both.astype(np.float32), w5.astype(np.float32), rel, n, 27)
    assert _max_rel_err(in_place, exact) <= FP16_TOL
    _ext.check_status(cuda)


def test_two_source_conv_needs_a_plan(cuda, sphere):
    from mlx_lattice_b200 import _ext

    coords, rel = sphere
    n = coords.shape[0]
    r = _rel_dev(rel, cuda)
    feats = torch.zeros((n, 32), dtype=torch.float16, device=cuda)
    weights = torch.zeros((32, 3, 3, 3, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(ValueError, match='second feature source'):
        _ext.sparse_conv_features(feats, weights, r['in_rows'], r['out_rows'], r['kernel_ids'],
                                  r['counts'], r['row_offsets'], out_capacity=n, n_kernels=27,
                                  feats2=feats)


def test_kept_fp16_weights_give_the_bits_of_the_packed_call(cuda, restatement, sphere):
    """ops.subm_conv3d converts a packed weight to fp16 once and keeps the result; the bits
    equal those of lat_sparse_quantized_conv_features, which converts on every call."""
    from mlx_lattice_b200 import _ext, ops
    from mlx_lattice_b200.core import QuantizedWeight, SparseTensor

    coords, rel = sphere
    n = coords.shape[0]
    rng = np.random.default_rng(77)
    feats = rng.normal(size=(n, 64)).astype(np.float16)
    q = restatement.quantize_weight((rng.normal(size=(128, 3, 3, 3, 64)) * 0.05).astype(np.float16), 32, 4)
    direct = _qconv(cuda, feats, q, rel, n, 27, with_plan=True)
    weight = QuantizedWeight(_dev(q['weight'].view(np.int32), cuda), _dev(q['scales'], cuda),
                             _dev(q['biases'], cuda), 32, 4, 64, 128, (3, 3, 3), 'dense_5d')
    x = SparseTensor(_dev(coords, cuda), _dev(feats, cuda))
    first = ops.subm_conv3d(x, weight, kernel_size=3).feats
    kept = weight.weight._lattice_fp16[1]
    second = ops.subm_conv3d(x, weight, kernel_size=3).feats
    assert weight.weight._lattice_fp16[1] is kept          # converted once
    assert np.array_equal(first.cpu().numpy(), direct) and torch.equal(first, second)
    weight.scales.mul_(2)                                  # an in-place change makes a new copy
    third = ops.subm_conv3d(x, weight, kernel_size=3).feats
    assert weight.weight._lattice_fp16[1] is not kept and not torch.equal(third, first)
    _ext.check_status(cuda)


def test_bad_vector_arguments_raise_before_any_launch(cuda, sphere):
    """Optional per-channel vectors reach the kernels as bare pointers; wrong device, dtype,
    length or layout is a ValueError in the wrapper, never a device fault."""
    from mlx_lattice_b200 import _ext

    coords, rel = sphere
    n = coords.shape[0]
    r = _rel_dev(rel, cuda)
    feats = torch.zeros((n, 32), dtype=torch.float16, device=cuda)
    weights = torch.zeros((32, 3, 3, 3, 32), dtype=torch.float16, device=cuda)
    args = (r['in_rows'], r['out_rows'], r['kernel_ids'], r['counts'], r['row_offsets'])
    before = _ext.launch_count()
    for bias in (torch.zeros(32, dtype=torch.float16),                       # host memory
                 torch.zeros(32, dtype=torch.float32, device=cuda),          # dtype
                 torch.zeros(31, dtype=torch.float16, device=cuda),          # too short
                 torch.zeros((32, 1), dtype=torch.float16, device=cuda)):    # shape
        with pytest.raises(ValueError, match='bias'):
            _ext.sparse_conv_features(feats, weights, *args, out_capacity=n, n_kernels=27, bias=bias)
        with pytest.raises(ValueError, match='bias'):
            _ext.linear(feats, torch.zeros((32, 32), dtype=torch.float16, device=cuda), bias)
    with pytest.raises(ValueError, match='row_order'):
        _ext.sparse_conv_features(feats, weights, *args, out_capacity=n, n_kernels=27,
                                  row_order=torch.zeros(n - 1, dtype=torch.int32, device=cuda))
    with pytest.raises(ValueError, match='plan'):
        _ext.sparse_conv_features(feats, weights, *args, out_capacity=n, n_kernels=27,
                                  plan=torch.zeros(64, dtype=torch.uint8, device=cuda))
    good = torch.ones(32, dtype=torch.float16, device=cuda)
    for name in ('weight', 'bias', 'mean', 'var'):
        vectors = {'weight': good, 'bias': good, 'mean': good, 'var': good}
        vectors[name] = torch.ones(64, dtype=torch.float16, device=cuda)[::2]   # strided view: made contiguous
        _ext.batch_norm_relu(feats, vectors['weight'], vectors['bias'], vectors['mean'], vectors['var'], 1e-5, False)
        vectors[name] = torch.ones(33, dtype=torch.float16, device=cuda)
        with pytest.raises(ValueError, match=name):
            _ext.batch_norm_relu(feats, vectors['weight'], vectors['bias'], vectors['mean'], vectors['var'], 1e-5, False)
    with pytest.raises(ValueError, match='linear weight'):
        _ext.linear(feats, torch.zeros((32, 16), dtype=torch.float16, device=cuda))
    assert _ext.launch_count() == before + 4      # only the four valid batch_norm calls launched
    _ext.check_status(cuda)


@pytest.mark.parametrize('c_in,c_out', [(96, 192), (32, 16), (256, 256), (64, 48)])
def test_linear_on_the_tensor_cores(cuda, restatement, c_in, c_out):
    """float16 matrices of at least 4096 rows whose shapes the tcgen05 tiles cover run as the
    convolution over the identity relation; same tolerance as every fp16 contraction, also
    for rows of a wider array, a bias, and a packed weight converted once."""
    from mlx_lattice_b200 import _ext, ops
    from mlx_lattice_b200.core import QuantizedWeight, SparseTensor

    assert _ext._lib().lat_linear_uses_tensor_cores(1, c_in, c_out) == 1
    rng = np.random.default_rng(c_in + c_out)
    rows = 4096 + 777
    x = rng.normal(size=(rows, c_in)).astype(np.float16)
    w = (rng.normal(size=(c_out, c_in)) * 0.1).astype(np.float16)
    b = rng.normal(size=c_out).astype(np.float16)
    before = _ext.launch_count()
    got = _ext.linear(_dev(x, cuda), _dev(w, cuda), _dev(b, cuda)).cpu().numpy()
    assert _max_rel_err(got, restatement.linear(x, w, b)) <= FP16_TOL
    wide = _dev(np.concatenate([x, x], axis=1), cuda)[:, :c_in]
    assert np.array_equal(_ext.linear(wide, _dev(w, cuda), _dev(b, cuda)).cpu().numpy(), got)
    small = _ext.linear(_dev(x[:4000], cuda), _dev(w, cuda), _dev(b, cuda)).cpu().numpy()   # CUDA cores
    assert _max_rel_err(small, got[:4000]) <= FP16_TOL
    q = restatement.quantize_weight(w, 32, 8)
    weight = QuantizedWeight(_dev(q['weight'].view(np.int32), cuda), _dev(q['scales'], cuda),
                             _dev(q['biases'], cuda), 32, 8, c_in, c_out, (1, 1, 1), 'linear')
    coords = np.zeros((rows, 4), np.int32)
    coords[:, 1] = np.arange(rows)
    y = ops.linear(SparseTensor(_dev(coords, cuda), _dev(x, cuda)), weight).feats.cpu().numpy()
    assert _max_rel_err(y, restatement.quantized_matmul(x, q)) <= FP16_TOL
    assert hasattr(weight.weight, '_lattice_fp16_matrix')
    assert _ext.launch_count() > before
    _ext.check_status(cuda)
