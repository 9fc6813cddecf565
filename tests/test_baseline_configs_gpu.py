"""The five benchmark configurations at their stated generators and sizes, GPU path (through
the C ABI) against the oracle: config 0 exactly, both 1,000,000-coordinate kernel maps
of config 2 exactly, one whole cloud of config 1. Configs 3 and 4 (one whole cloud each)
are the full-size cases of tests/test_network_gpu.py. Bars: kernel maps bit-exact in
native order and after canonical sorting; fp32 <= 1e-5, fp16 <= 2e-3 of max|ref|."""

import numpy as np
import pytest
import torch

from conftest import RELATION_KEYS, canonical_edges, canonical_pair_lists, relation_to_numpy
from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu


def _max_rel_err(got, want):
    want = np.asarray(want, np.float64)
    return np.abs(np.asarray(got, np.float64) - want).max() / max(np.abs(want).max(), 1e-30)


def test_config0_subm_conv_fp32_50k(cuda, oracle):
    """50,000 unique voxels on 4 spheres + 2 planes in a 256^3 grid, float32, weight
    (32,3,3,3,32) ~ N(0, 0.05), no bias, batch 1: subm_conv3d against the reference CPU route."""
    from mlx_lattice_b200 import _ext, ops
    from mlx_lattice_b200.core import SparseTensor

    coords = synthetic.sphere_plane_batch(0, 1, 50000, 256)
    assert coords.shape == (50000, 4) and np.unique(coords, axis=0).shape[0] == 50000
    rng = np.random.default_rng(0)
    feats = rng.normal(size=(50000, 32)).astype(np.float32)
    weight = (rng.normal(size=(32, 3, 3, 3, 32)) * 0.05).astype(np.float32)
    x = SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda))
    got = ops.subm_conv3d(x, torch.from_numpy(weight).to(cuda), kernel_size=3).feats.cpu().numpy()
    _ext.check_status()
    rel = oracle.build_submanifold_kernel_relation(coords)
    want = oracle.sparse_conv(feats, weight, rel, 50000, 27)
    assert _max_rel_err(got, want) <= 1e-5


@pytest.mark.parametrize('stride', [1, 2], ids=['submanifold', 'stride2'])
def test_config2_kernel_maps_one_million_coords(cuda, oracle, stride):
    """1,000,000 LiDAR-like coordinates over 8 clouds: the kernel_size=3 submanifold map and
    the kernel_size=3 stride=2 map against the reference's single-thread builder, every
    array bit-exact in native order; pairs also after canonical sorting."""
    from mlx_lattice_b200 import _ext

    coords = synthetic.lidar_batch(2, 8, 125000)
    n = coords.shape[0]
    assert n == 1000000
    device_coords = torch.from_numpy(coords).to(cuda)
    active = torch.tensor([n], dtype=torch.int32, device=cuda)
    got = relation_to_numpy(_ext.build_kernel_relation(device_coords, active, 3, stride, 0, 1))
    _ext.check_status()
    want = (oracle.build_submanifold_kernel_relation(coords) if stride == 1
            else oracle.build_kernel_relation(coords, None, kernel_size=3, stride=2))
    for key in RELATION_KEYS + ('out_coords', 'in_row_offsets', 'in_edge_ids',
                                'kernel_row_offsets', 'kernel_edge_ids'):
        assert np.array_equal(got[key], want[key]), key
    assert np.array_equal(canonical_edges(got), canonical_edges(want))
    for mine, theirs in zip(canonical_pair_lists(got, 27), canonical_pair_lists(want, 27)):
        assert np.array_equal(mine, theirs)


def test_config1_strided_int4_conv_one_whole_cloud(cuda, oracle, restatement):
    """One cloud of config 1 at its full size: 200,000 sphere+plane voxels in a 512^3 grid,
    fp16 features, QuantizedConv3d int4 affine group 32, 64 -> 128, kernel_size=2 stride=2."""
    from mlx_lattice_b200 import _ext, ops
    from mlx_lattice_b200.core import QuantizedWeight, SparseTensor

    coords = synthetic.sphere_plane_batch(1, 1, 200000, 512)
    n = coords.shape[0]
    assert n == 200000
    rng = np.random.default_rng(1)
    feats = rng.normal(size=(n, 64)).astype(np.float16)
    dense = (rng.normal(size=(128, 2, 2, 2, 64)) * 0.05).astype(np.float16)
    q = restatement.quantize_weight(dense, 32, 4)
    weight = QuantizedWeight(
        torch.from_numpy(q['weight'].view(np.int32)).to(cuda), torch.from_numpy(q['scales']).to(cuda),
        torch.from_numpy(q['biases']).to(cuda), 32, 4, 64, 128, (2, 2, 2), 'dense_5d')
    x = SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda))
    y = ops.conv3d(x, weight, kernel_size=2, stride=2)
    got = y.feats.cpu().numpy()
    _ext.check_status()
    rel = oracle.build_kernel_relation(coords, None, kernel_size=2, stride=2)
    n_out = int(rel['counts'][1])
    assert int(y.active_rows.item()) == n_out
    assert np.array_equal(y.coords.cpu().numpy()[:n_out], rel['out_coords'][:n_out])
    want = oracle.sparse_quantized_conv(feats, q['weight'], q['scales'], q['biases'], rel, n, 8,
                                        64, 128, q['storage_in_channels'], 32, 4)
    assert _max_rel_err(got, want) <= 2e-3
    assert not got[n_out:].any()
