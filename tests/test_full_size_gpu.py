"""The benchmark configurations at their full sizes, checked through properties that do
not need the CPU oracle to finish a million-row case: an independent sort-and-search
construction of the kernel map in torch, exact scaling of a convolution by powers of two,
equality of a batch-sharded run with the joint run, determinism, and a sampled comparison
with the reference arithmetic on a few thousand output rows."""

import numpy as np
import pytest
import torch

from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu


def _keys(coords: torch.Tensor) -> torch.Tensor:
    """Order-preserving int64 key of (b, x, y, z) rows (values within +-2^14 here)."""
    c = coords.long()
    return ((c[:, 0] * 40000 + (c[:, 1] + 20000)) * 40000 + (c[:, 2] + 20000)) * 40000 + (c[:, 3] + 20000)


def _first_row_lookup(coords: torch.Tensor, queries: torch.Tensor) -> torch.Tensor:
    """Row of the first occurrence of each query coordinate, -1 when absent (torch only)."""
    keys = _keys(coords)
    order = torch.argsort(keys, stable=True)
    sorted_keys = keys[order]
    q = _keys(queries)
    pos = torch.searchsorted(sorted_keys, q)
    pos = pos.clamp(max=sorted_keys.shape[0] - 1)
    found = sorted_keys[pos] == q
    return torch.where(found, order[pos], torch.full_like(pos, -1))


def test_config2_submanifold_map_one_million_coords(cuda):
    """K = 27 submanifold map over 8 x 125,000 LiDAR-like voxels against an independent
    sort-and-search construction; order, offsets and tails as the contract states."""
    from mlx_lattice_b200 import _ext

    coords = torch.from_numpy(synthetic.lidar_batch(2, 8, 125000)).to(cuda)
    n = coords.shape[0]
    active = torch.tensor([n], dtype=torch.int32, device=cuda)
    base, masks, _ = _ext.build_kernel_relation_base(coords, active, 3, 1, 0, 1, want_masks=True)
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = base
    _ext.check_status(cuda)
    edges, n_out = counts.tolist()
    assert n_out == n and torch.equal(out_coords, coords)
    offsets = torch.tensor(_ext.kernel_offsets(3), dtype=torch.int32, device=cuda)
    # independent construction: for every offset, look the shifted coordinate up
    want_in = []
    for k in range(27):
        shifted = coords.clone()
        shifted[:, 1:] += offsets[k]
        want_in.append(_first_row_lookup(coords, shifted))
    want = torch.stack(want_in, dim=1)                      # [n, 27], -1 = absent
    present = want >= 0
    assert int(present.sum()) == edges
    rows, ks = torch.nonzero(present, as_tuple=True)        # row-major: (out asc, k asc)
    assert torch.equal(out_rows[:edges].long(), rows)
    assert torch.equal(kernel_ids[:edges].long(), ks)
    assert torch.equal(in_rows[:edges].long(), want[rows, ks])
    degree = present.sum(dim=1)
    expect_offsets = torch.zeros(n + 1, dtype=torch.long, device=cuda)
    expect_offsets[1:] = torch.cumsum(degree, 0)
    assert torch.equal(row_offsets.long(), expect_offsets)
    assert not in_rows[edges:].any() and not out_rows[edges:].any() and not kernel_ids[edges:].any()
    bits = (present.long() << torch.arange(27, device=cuda)).sum(dim=1)
    assert torch.equal(masks[:, 0].long(), bits)
    # symmetry of a submanifold map: as many edges at offset k as at 26 - k
    per_offset = present.sum(dim=0)
    assert torch.equal(per_offset, per_offset.flip(0))


def test_config2_strided_map_one_million_coords(cuda):
    """K = 27, stride 2: output support = unique floor(coord / 2) in first-seen order, and
    every edge joins an input with the output cell its offset points to."""
    from mlx_lattice_b200 import _ext

    coords = torch.from_numpy(synthetic.lidar_batch(2, 8, 125000)).to(cuda)
    n = coords.shape[0]
    active = torch.tensor([n], dtype=torch.int32, device=cuda)
    base, _, _ = _ext.build_kernel_relation_base(coords, active, 3, 2, 0, 1)
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = base
    _ext.check_status(cuda)
    edges, n_out = counts.tolist()
    cells = coords.clone()
    cells[:, 1:] = torch.div(coords[:, 1:], 2, rounding_mode='floor')
    keys = _keys(cells)
    uniq, inverse = torch.unique(keys, return_inverse=True)
    first = torch.full((uniq.shape[0],), n, dtype=torch.long, device=cuda)
    first.scatter_reduce_(0, inverse, torch.arange(n, device=cuda), reduce='amin')
    order = torch.sort(first).values                         # first-seen order
    assert n_out == uniq.shape[0]
    assert torch.equal(out_coords[:n_out], cells[order])
    assert not out_coords[n_out:].any()
    offsets = torch.tensor(_ext.kernel_offsets(3), dtype=torch.int32, device=cuda)
    o, i, k = out_rows[:edges].long(), in_rows[:edges].long(), kernel_ids[:edges].long()
    expect = out_coords[o].clone()
    expect[:, 1:] = expect[:, 1:] * 2 + offsets[k]
    assert torch.equal(coords[i], expect)
    assert bool((o[1:] >= o[:-1]).all())
    same = o[1:] == o[:-1]
    assert bool((k[1:][same] > k[:-1][same]).all())
    # every (output, offset) whose input exists is an edge: count by lookup
    total = 0
    support = out_coords[:n_out]
    for kk in range(27):
        cand = support.clone()
        cand[:, 1:] = cand[:, 1:] * 2 + offsets[kk]
        total += int((_first_row_lookup(coords, cand) >= 0).sum())
    assert total == edges


def test_inputs_beyond_the_self_scan_size(cuda):
    """1,250,000 rows: more than 4096 blocks / tiles, where the strided support, the decoder
    map and the gather plan run their one-block scan kernels instead of letting every block
    add up the totals before it. Output support and decoder map against torch constructions,
    the plan through a convolution that must equal the plan-free one bit for bit."""
    from mlx_lattice_b200 import _ext

    coords = torch.from_numpy(synthetic.lidar_batch(2, 10, 125000)).to(cuda)
    n = coords.shape[0]
    assert n > 4096 * 256
    active = torch.tensor([n], dtype=torch.int32, device=cuda)
    base, _, _ = _ext.build_kernel_relation_base(coords, active, 2, 2, 0, 1)
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = base
    _ext.check_status(cuda)
    edges, n_out = counts.tolist()
    cells = coords.clone()
    cells[:, 1:] = torch.div(coords[:, 1:], 2, rounding_mode='floor')
    keys = _keys(cells)
    uniq, inverse = torch.unique(keys, return_inverse=True)
    first = torch.full((uniq.shape[0],), n, dtype=torch.long, device=cuda)
    first.scatter_reduce_(0, inverse, torch.arange(n, device=cuda), reduce='amin')
    order = torch.sort(first).values
    assert n_out == uniq.shape[0] and edges == n          # every voxel has exactly one parent
    assert torch.equal(out_coords[:n_out], cells[order])
    assert not out_coords[n_out:].any()
    # decoder map: fine row -> (parent row, child offset)
    coarse = out_coords[:n_out].contiguous()
    coarse_active = torch.tensor([n_out], dtype=torch.int32, device=cuda)
    up = _ext.build_target_transposed_relation_base(coarse, coarse_active, coords, active, 2)
    up_in, up_out, up_k, up_offsets, _, up_counts = up
    _ext.check_status(cuda)
    assert up_counts.tolist() == [n, n]
    assert torch.equal(up_out.long(), torch.arange(n, device=cuda))
    assert torch.equal(up_offsets.long(), torch.arange(n + 1, device=cuda))
    assert torch.equal(up_in.long(), _first_row_lookup(coarse, cells))
    child = coords[:, 1:] - 2 * cells[:, 1:]
    assert torch.equal(up_k.long(), ((child[:, 0] * 2 + child[:, 1]) * 2 + child[:, 2]).long())
    # gather plan with more than 4096 tiles
    rng = np.random.default_rng(8)
    feats = torch.from_numpy(rng.normal(size=(n, 32)).astype(np.float16)).to(cuda)
    weights = torch.from_numpy((rng.normal(size=(8, 32, 32)) * 0.1).astype(np.float16)).to(cuda)
    plan = _ext.build_conv_plan(in_rows, kernel_ids, counts, row_offsets, n, n, 8)
    with_plan = _ext.sparse_conv_features(feats, weights, in_rows, out_rows, kernel_ids, counts, row_offsets,
                                          out_capacity=n, n_kernels=8, plan=plan)
    without = _ext.sparse_conv_features(feats, weights, in_rows, out_rows, kernel_ids, counts, row_offsets,
                                        out_capacity=n, n_kernels=8)
    _ext.check_status(cuda)
    assert torch.equal(with_plan, without)
    assert not with_plan[n_out:].any()


def _layer(cuda, c_in, c_out, seed):
    from mlx_lattice_b200.core import quantize_weight

    rng = np.random.default_rng(seed)
    dense = (rng.normal(size=(c_out, 3, 3, 3, c_in)) * 0.05).astype(np.float16)
    q = quantize_weight(torch.from_numpy(dense), group_size=32, bits=4)
    from mlx_lattice_b200.workloads import quantized_to

    return quantized_to(q, cuda)


def test_config4_layer_properties_at_full_size(cuda, restatement):
    """One int4 3x3x3 submanifold convolution over the full 8 x 120,000-voxel input:
    bitwise determinism, exact scaling by two, equality of batch shards with the joint run
    (what the multi-GPU partition relies on), and 2,000 sampled rows against the reference
    arithmetic evaluated on the host from the GPU's own (already verified) map."""
    from mlx_lattice_b200 import ops
    from mlx_lattice_b200.core import SparseTensor, dequantize_weight

    coords_np = synthetic.lidar_batch(4, 8, 120000)
    n = coords_np.shape[0]
    rng = np.random.default_rng(4)
    feats_np = rng.normal(size=(n, 64)).astype(np.float16)
    weight = _layer(cuda, 64, 64, 5)
    coords = torch.from_numpy(coords_np).to(cuda)
    feats = torch.from_numpy(feats_np).to(cuda)
    counts = (120000,) * 8

    x = SparseTensor(coords, feats, batch_counts=counts)
    y = ops.subm_conv3d(x, weight, kernel_size=3).feats
    y_again = ops.subm_conv3d(SparseTensor(coords, feats, batch_counts=counts), weight, kernel_size=3).feats
    assert torch.equal(y, y_again)
    y2 = ops.subm_conv3d(SparseTensor(coords, feats * 2, batch_counts=counts), weight, kernel_size=3).feats
    # exact wherever the float16 result is a normal number (doubling a value that rounds in
    # the subnormal range may round differently)
    normal = y.abs() >= 2.0 ** -13
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert float((y2.float() - 2 * y.float()).abs().max()) <= 2.0 ** -23

    half = 4 * 120000
    lo = ops.subm_conv3d(SparseTensor(coords[:half], feats[:half], batch_counts=counts[:4]),
                         weight, kernel_size=3).feats
    hi_coords = coords[half:].clone()
    hi = ops.subm_conv3d(SparseTensor(hi_coords, feats[half:], batch_counts=counts[4:]),
                         weight, kernel_size=3).feats
    assert torch.equal(torch.cat([lo, hi]), y)

    rel = x.coord_manager.submanifold_kernel_relation(x.coord_key, kernel_size=3)
    edges = int(rel.counts[0])
    offs = rel.output_csr.row_offsets.cpu().numpy()
    in_rows = rel.edges.in_rows[:edges].cpu().numpy()
    kernel_ids = rel.edges.kernel_ids[:edges].cpu().numpy()
    w = dequantize_weight(weight).float().cpu().numpy()          # (C_out, 3, 3, 3, C_in)
    w = w.reshape(64, 27, 64)
    sample = np.random.default_rng(6).choice(n, size=2000, replace=False)
    got = y[torch.from_numpy(sample).to(cuda)].float().cpu().numpy()
    want = np.zeros((2000, 64), np.float32)
    x32 = feats_np.astype(np.float32)
    for slot, row in enumerate(sample):
        for e in range(offs[row], offs[row + 1]):
            want[slot] += w[:, kernel_ids[e], :] @ x32[in_rows[e]]
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-3 * scale
