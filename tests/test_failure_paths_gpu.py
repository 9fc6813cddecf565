"""Run-time problems never trap: counts and row ranges read from device memory are
clamped to the static capacities, a kernel that meets a problem sets a bit of the
status word and returns, and every in-kernel wait has a clock budget. None of these
cases feeds a kernel an index outside its arrays."""

import numpy as np
import pytest
import torch

from conftest import relation_to_numpy
from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu


def _dev(array, cuda):
    return torch.from_numpy(np.ascontiguousarray(array)).to(cuda)


@pytest.fixture(scope='module')
def cloud(oracle):
    coords = synthetic.sphere_plane_batch(0, 1, 20000, 96)
    return coords, oracle.build_submanifold_kernel_relation(coords)


@pytest.mark.parametrize('dtype,c_in,c_out', [(np.float16, 64, 64), (np.float32, 16, 16)])
def test_counts_beyond_the_capacities_are_clamped(cuda, cloud, dtype, c_in, c_out):
    """counts = (edges, rows) is device data: values above the capacities (or negative) read
    as the capacity (or zero), on the tensor-core and the CUDA-core route alike."""
    from mlx_lattice_b200 import _ext

    coords, rel = cloud
    n = coords.shape[0]
    rng = np.random.default_rng(3)
    feats = _dev(rng.normal(size=(n, c_in)).astype(dtype), cuda)
    weights = _dev((rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(dtype), cuda)
    r = {k: _dev(v, cuda) for k, v in rel.items()}
    edge_capacity = int(r['in_rows'].shape[0])

    def conv(counts):
        c = torch.tensor(counts, dtype=torch.int32, device=cuda)
        return _ext.sparse_conv_features(feats, weights, r['in_rows'], r['out_rows'], r['kernel_ids'],
                                         c, r['row_offsets'], out_capacity=n, n_kernels=27)

    at_capacity = conv([edge_capacity, n])
    assert torch.equal(conv([edge_capacity + 123456, n + 77]), at_capacity)
    assert torch.equal(conv([2 ** 31 - 1, 2 ** 31 - 1]), at_capacity)
    nothing = conv([0, 0])
    assert not nothing.any()
    assert torch.equal(conv([-5, -3]), nothing)
    pooled = _ext.sparse_pool_features(
        feats.float(), r['in_rows'], r['out_rows'], r['kernel_ids'], r['row_offsets'],
        torch.tensor([edge_capacity + 9, n + 9], dtype=torch.int32, device=cuda), False, 'max', n, 27)
    assert torch.equal(pooled, _ext.sparse_pool_features(
        feats.float(), r['in_rows'], r['out_rows'], r['kernel_ids'], r['row_offsets'],
        torch.tensor([edge_capacity, n], dtype=torch.int32, device=cuda), False, 'max', n, 27))
    _ext.check_status(cuda)


def test_active_rows_outside_the_capacity_are_clamped(cuda, cloud):
    from mlx_lattice_b200 import _ext

    coords, _ = cloud
    n = coords.shape[0]
    device_coords = _dev(coords, cuda)

    def build(active):
        rows = torch.tensor([active], dtype=torch.int32, device=cuda)
        return relation_to_numpy(_ext.build_kernel_relation(device_coords, rows, 3, 1, 0, 1))

    whole, beyond = build(n), build(n + 1000)
    for key in whole:
        assert np.array_equal(whole[key], beyond[key]), key
    empty, negative = build(0), build(-4)
    assert empty['counts'].tolist() == [0, 0]
    for key in empty:
        assert np.array_equal(empty[key], negative[key]), key
    _ext.check_status(cuda)


def test_duplicate_inputs_of_an_overlapping_transposed_map_set_the_status_bit(cuda):
    """kernel 3, stride 2 transposed (neighbouring inputs write the same output voxels) over a
    coordinate list with a repeated row: the builder cannot keep one edge per (output,
    offset), says so in the status word, returns, and the next call is clean."""
    from mlx_lattice_b200 import _ext, _native

    coords = np.array([[0, 1, 1, 1], [0, 2, 1, 1], [0, 1, 1, 1], [0, 5, 5, 5]], np.int32)
    rows = torch.tensor([4], dtype=torch.int32, device=cuda)
    _ext.build_transposed_kernel_relation(_dev(coords, cuda), rows, 3, 2, 0, 1)
    with pytest.raises(RuntimeError, match=_native.STATUS_BITS[16]):
        _ext.check_status(cuda)
    _ext.check_status(cuda)   # the word was cleared
    unique = np.array([[0, 1, 1, 1], [0, 2, 1, 1], [0, 5, 5, 5]], np.int32)
    _ext.build_transposed_kernel_relation(_dev(unique, cuda), torch.tensor([3], dtype=torch.int32, device=cuda),
                                          3, 2, 0, 1)
    _ext.check_status(cuda)


def test_a_wait_that_runs_out_of_budget_returns_with_the_status_bit(cuda, cloud, oracle):
    """With the clock budget of the in-kernel waits cut to a few cycles, a convolution whose
    epilogue has to wait for a whole tile of MMAs gives up: LAT_STATUS_WAIT_TIMEOUT, every
    role drains, tensor memory is freed, the launch returns; with the budget restored the
    same call gives the right answer."""
    from mlx_lattice_b200 import _ext, _native

    coords, rel = cloud
    n = coords.shape[0]
    rng = np.random.default_rng(11)
    feats = _dev(rng.normal(size=(n, 256)).astype(np.float16), cuda)
    weights = _dev((rng.normal(size=(256, 3, 3, 3, 256)) * 0.05).astype(np.float16), cuda)
    r = {k: _dev(v, cuda) for k, v in rel.items()}
    plan = _ext.build_conv_plan(r['in_rows'], r['kernel_ids'], r['counts'], r['row_offsets'], n, n, 27, None)

    def conv():
        return _ext.sparse_conv_features(feats, weights, r['in_rows'], r['out_rows'], r['kernel_ids'],
                                         r['counts'], r['row_offsets'], out_capacity=n, n_kernels=27,
                                         plan=plan)

    good = conv()
    _ext.check_status(cuda)
    lib = _native.load()
    default = int(lib.lat_wait_budget_cycles())
    assert default > 10 ** 9
    with pytest.raises(ValueError):
        _native.check(lib.lat_set_wait_budget_cycles(0))
    try:
        _native.check(lib.lat_set_wait_budget_cycles(8))
        conv()
        with pytest.raises(RuntimeError, match=_native.STATUS_BITS[8]):
            _ext.check_status(cuda)
    finally:
        _native.check(lib.lat_set_wait_budget_cycles(default))
    assert int(lib.lat_wait_budget_cycles()) == default
    assert torch.equal(conv(), good)
    _ext.check_status(cuda)
