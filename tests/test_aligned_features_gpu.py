"""Channel concatenation and elementwise binary operators through a sparse alignment:
the GPU kernels against the numpy restatement of the reference's array-op composition,
bit for bit, over the four joins, both feature dtypes, wide and odd channel counts, fill
values, NaN propagation and operands that share their coordinates."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

JOINS = ('inner', 'left', 'right', 'outer')
OPS = ('add', 'sub', 'mul', 'maximum', 'minimum')


def _clouds(seed=0, n_lhs=3000, n_rhs=2600):
    rng = np.random.default_rng(seed)
    pool = rng.integers(-12, 12, size=(5000, 4)).astype(np.int32)
    pool[:, 0] = rng.integers(0, 2, size=5000)
    pool = np.unique(pool, axis=0)
    rng.shuffle(pool)
    lhs = pool[rng.choice(pool.shape[0], n_lhs, replace=False)]
    rhs = pool[rng.choice(pool.shape[0], n_rhs, replace=False)]
    return lhs, rhs


def _tensor(cuda, coords, feats, active=None):
    from mlx_lattice_b200.core import SparseTensor

    kwargs = {}
    if active is not None:
        kwargs['active_rows'] = torch.tensor([active], dtype=torch.int32, device=cuda)
    return SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda), **kwargs)


def _same_bits(got: torch.Tensor, want: np.ndarray) -> bool:
    """Equal bit for bit wherever the result is a number; NaN in the same places (the
    payload of a NaN is not part of the contract)."""
    got = got.cpu().numpy()
    nan = np.isnan(want)
    if got.shape != want.shape or got.dtype != want.dtype or not np.array_equal(np.isnan(got), nan):
        return False
    return got[~nan].tobytes() == want[~nan].tobytes()


@pytest.mark.parametrize('dtype', [np.float16, np.float32])
@pytest.mark.parametrize('channels', [(32, 64), (3, 5), (8, 7), (1, 1)])
def test_cat_aligned_all_joins(cuda, oracle, restatement, dtype, channels):
    from mlx_lattice_b200 import _ext, ops

    lhs_c, rhs_c = _clouds(1)
    rng = np.random.default_rng(2)
    lhs_f = rng.normal(size=(lhs_c.shape[0], channels[0])).astype(dtype)
    rhs_f = rng.normal(size=(rhs_c.shape[0], channels[1])).astype(dtype)
    la, ra = 2900, 2600
    for join in JOINS:
        coords, count, lrows, rrows = oracle.sparse_alignment(lhs_c, la, rhs_c, ra, join)
        want = restatement.concat_aligned_features(lhs_f, lrows, rhs_f, rrows)
        got = ops.sparse_cat_aligned(_tensor(cuda, lhs_c, lhs_f, la), _tensor(cuda, rhs_c, rhs_f, ra), join=join)
        assert got.active_rows.tolist() == count.tolist()
        assert np.array_equal(got.coords.cpu().numpy(), coords)
        assert _same_bits(got.feats, want), join
    _ext.check_status()
    shared = _tensor(cuda, lhs_c, lhs_f)
    other = shared.replace(feats=torch.from_numpy(rng.normal(size=(lhs_c.shape[0], channels[1])).astype(dtype)).to(cuda))
    got = ops.sparse_cat_aligned(shared, other)
    assert got.same_coords(shared)
    assert torch.equal(got.feats, torch.cat([shared.feats, other.feats], dim=1))


@pytest.mark.parametrize('dtype', [np.float16, np.float32])
@pytest.mark.parametrize('channels', [64, 5])
def test_binary_ops_all_joins_and_fills(cuda, oracle, restatement, dtype, channels):
    from mlx_lattice_b200 import _ext, ops

    lhs_c, rhs_c = _clouds(3)
    rng = np.random.default_rng(4)
    lhs_f = (rng.normal(size=(lhs_c.shape[0], channels)) * 40).astype(dtype)
    rhs_f = (rng.normal(size=(rhs_c.shape[0], channels)) * 0.03).astype(dtype)
    lhs_f[5, 0], rhs_f[7, channels - 1] = np.nan, np.inf
    lhs_t, rhs_t = _tensor(cuda, lhs_c, lhs_f), _tensor(cuda, rhs_c, rhs_f)
    for join in JOINS:
        _, count, lrows, rrows = oracle.sparse_alignment(lhs_c, lhs_c.shape[0], rhs_c, rhs_c.shape[0], join)
        for op in OPS:
            for fills in ((0.0, 0.0), (1.5, -2.25)):
                want = restatement.binary_aligned_features(lhs_f, lrows, rhs_f, rrows, op, *fills)
                got = ops.sparse_binary_op(lhs_t, rhs_t, op, join=join, lhs_fill=fills[0], rhs_fill=fills[1])
                assert got.active_rows.tolist() == count.tolist()
                assert _same_bits(got.feats, want), (join, op, fills)
    _ext.check_status()
    # the named forms and their default joins (ops/tensor.py:150-197)
    for name, op, join in (('sparse_add', 'add', 'outer'), ('sparse_sub', 'sub', 'outer'),
                           ('sparse_mul', 'mul', 'inner'), ('sparse_maximum', 'maximum', 'inner'),
                           ('sparse_minimum', 'minimum', 'inner')):
        got = getattr(ops, name)(lhs_t, rhs_t)
        want = ops.sparse_binary_op(lhs_t, rhs_t, op, join=join)
        assert torch.equal(got.coords, want.coords)
        assert _same_bits(got.feats, want.feats.cpu().numpy())
    # shared coordinates: no alignment, row by row
    other = lhs_t.replace(feats=torch.from_numpy((rng.normal(size=lhs_f.shape)).astype(dtype)).to(cuda))
    got = ops.sparse_add(lhs_t, other)
    assert got.same_coords(lhs_t)
    with np.errstate(all='ignore'):
        assert _same_bits(got.feats, lhs_f + other.feats.cpu().numpy())


def test_residual_block_through_the_artifact_route(cuda):
    """``sparse.add`` as persisted artifacts name it: conv -> add(input) with shared
    coordinates equals the operator composition."""
    from mlx_lattice_b200 import artifact, ops

    lhs_c, _ = _clouds(5)
    rng = np.random.default_rng(6)
    feats = rng.normal(size=(lhs_c.shape[0], 16)).astype(np.float32)
    weight = torch.from_numpy((rng.normal(size=(16, 3, 3, 3, 16)) * 0.1).astype(np.float32))
    g = artifact.GraphWriter({'input': 'sparse_tensor'})
    conv = g.add('sparse.subm_conv3d', {'input': 'input'}, node_id='conv',
                 parameters={'weight': weight}, attributes={'kernel_size': 3})
    g.add('sparse.add', {'lhs': conv, 'rhs': 'input'}, node_id='residual', attributes={'join': 'outer'})
    model = artifact.LatticeModel(g.manifest(), g.weights, device=cuda)
    x = _tensor(cuda, lhs_c, feats)
    got = model(x)
    want = ops.sparse_add(ops.subm_conv3d(x, weight.to(cuda), kernel_size=3), x)
    assert torch.equal(got.feats, want.feats) and got.same_coords(x)


def test_argument_errors(cuda):
    from mlx_lattice_b200 import ops

    lhs_c, rhs_c = _clouds(7)
    a = _tensor(cuda, lhs_c, np.zeros((lhs_c.shape[0], 4), np.float32))
    b = _tensor(cuda, rhs_c, np.zeros((rhs_c.shape[0], 5), np.float32))
    with pytest.raises(ValueError, match='matching channels'):
        ops.sparse_add(a, b)
    with pytest.raises(ValueError, match='unknown sparse binary op'):
        ops.sparse_binary_op(a, a, 'pow')
    with pytest.raises(ValueError, match='join must be'):
        ops.sparse_cat_aligned(a, b, join='cross')
    c = _tensor(cuda, rhs_c, np.zeros((rhs_c.shape[0], 4), np.float16))
    with pytest.raises(ValueError, match='matching feature dtype'):
        ops.sparse_add(a, c)


ACTIVATIONS = [
    ('sigmoid', {}), ('silu', {}), ('tanh', {}), ('gelu', {}), ('gelu', {'approximate': 'precise'}),
    ('gelu', {'approximate': 'tanh'}), ('gelu', {'approximate': 'fast'}),
    ('leaky_relu', {}), ('leaky_relu', {'negative_slope': 0.2}),
    ('softplus', {}), ('softplus', {'beta': 2.5, 'threshold': 6.0}),
]


@pytest.mark.parametrize('dtype', [np.float16, np.float32])
@pytest.mark.parametrize('name, params', ACTIVATIONS)
def test_activations(cuda, restatement, dtype, name, params):
    """Against the float64 restatement: |error| <= 4 eps max(|result|, |input|) of the
    feature dtype. The evaluation is float32 with the device's expf / tanhf / erff and one
    cast; the input term covers the cancellation in 1 + erf(x / sqrt 2) for negative x, which
    the reference's float formula has too."""
    from mlx_lattice_b200 import ops

    lhs_c, _ = _clouds(9, n_lhs=1500)
    rng = np.random.default_rng(10)
    feats = (rng.normal(size=(lhs_c.shape[0], 24)) * 4).astype(dtype)
    feats[:8, 0] = [0.0, -0.0, 30.0, -30.0, 7.99, 8.01, 1e-4, -1e-4]
    x = _tensor(cuda, lhs_c, feats)
    got = getattr(ops, name)(x, **params)
    assert got.same_coords(x) and got.feats.dtype == x.feats.dtype
    want = restatement.activation(feats, name, **params)
    eps = float(np.finfo(dtype).eps)
    tolerance = 4 * eps * np.maximum(np.abs(want), np.abs(feats.astype(np.float64))) + float(np.finfo(dtype).tiny)
    assert np.all(np.abs(got.feats.cpu().numpy().astype(np.float64) - want) <= tolerance)


def test_activation_arguments_and_inference_dropout(cuda):
    from mlx_lattice_b200 import ops

    lhs_c, _ = _clouds(11, n_lhs=100)
    x = _tensor(cuda, lhs_c, np.ones((100, 4), np.float32))
    with pytest.raises(ValueError, match="approximate must be"):
        ops.gelu(x, approximate='quick')
    with pytest.raises(ValueError, match='beta must be positive'):
        ops.softplus(x, beta=0.0)
    with pytest.raises(ValueError, match='0 <= p < 1'):
        ops.dropout(x, p=1.0)
    with pytest.raises(ValueError, match='training mode'):
        ops.dropout(x, p=0.5, training=True)
    assert torch.equal(ops.dropout(x, p=0.5, training=False).feats, x.feats)
    assert torch.equal(ops.dropout(x, p=0.0).feats, x.feats)


@pytest.mark.parametrize('dtype', [np.float16, np.float32])
@pytest.mark.parametrize('channels', [1, 20, 64, 100])
def test_layer_norm_and_rms_norm(cuda, restatement, dtype, channels):
    """Against the float64 restatement within 8 eps of the feature dtype times the scale of
    the normalised row (float32 statistics, one cast)."""
    from mlx_lattice_b200 import ops

    lhs_c, _ = _clouds(12, n_lhs=700)
    rng = np.random.default_rng(13)
    feats = (rng.normal(size=(700, channels)) * 3 + 1.5).astype(dtype)
    weight = rng.normal(size=channels).astype(dtype)
    bias = rng.normal(size=channels).astype(dtype)
    x = _tensor(cuda, lhs_c, feats)
    w, b = torch.from_numpy(weight).to(cuda), torch.from_numpy(bias).to(cuda)
    eps = float(np.finfo(dtype).eps)
    cases = [
        (ops.layer_norm(x), restatement.row_norm(feats)),
        (ops.layer_norm(x, weight=w, bias=b, eps=1e-3), restatement.row_norm(feats, weight, bias, 1e-3)),
        (ops.rms_norm(x), restatement.row_norm(feats, rms=True)),
        (ops.rms_norm(x, weight=w, eps=1e-2), restatement.row_norm(feats, weight, None, 1e-2, rms=True)),
    ]
    for got, want in cases:
        assert got.same_coords(x) and got.feats.dtype == x.feats.dtype
        scale = np.abs(want).max(axis=1, keepdims=True) + 1.0
        assert np.all(np.abs(got.feats.cpu().numpy().astype(np.float64) - want) <= 8 * eps * scale)
    with pytest.raises(ValueError, match='eps must be positive'):
        ops.layer_norm(x, eps=0.0)
    with pytest.raises(ValueError, match=r'weight must have shape'):
        ops.rms_norm(x, weight=torch.ones(channels + 1, dtype=x.feats.dtype, device=cuda))


def test_feature_modules_call_their_operators(cuda):
    from mlx_lattice_b200 import nn, ops

    lhs_c, _ = _clouds(14, n_lhs=300)
    feats = np.random.default_rng(15).normal(size=(300, 16)).astype(np.float32)
    x = _tensor(cuda, lhs_c, feats)
    pairs = [
        (nn.Sigmoid(), ops.sigmoid(x)), (nn.SiLU(), ops.silu(x)), (nn.Tanh(), ops.tanh(x)),
        (nn.GELU('tanh'), ops.gelu(x, approximate='tanh')), (nn.LeakyReLU(0.3), ops.leaky_relu(x, negative_slope=0.3)),
        (nn.Softplus(), ops.softplus(x)), (nn.Dropout(0.4), x),
        (nn.LayerNorm(16).to(cuda), ops.layer_norm(x, weight=torch.ones(16, device=cuda), bias=torch.zeros(16, device=cuda))),
        (nn.RMSNorm(16).to(cuda), ops.rms_norm(x, weight=torch.ones(16, device=cuda))),
    ]
    for module, want in pairs:
        assert torch.equal(module(x).feats, want.feats), type(module).__name__
