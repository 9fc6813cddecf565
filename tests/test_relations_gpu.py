"""Kernel maps, output supports and relation views on the GPU against the oracle.
Bit-exact: native order equals the reference order, and the canonical-sort
comparison of the parity contract is checked as well."""

import numpy as np
import pytest
import torch

from conftest import canonical_edges, canonical_pair_lists, relation_to_numpy
from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu

ALL_KEYS = ('in_rows', 'out_rows', 'kernel_ids', 'row_offsets', 'out_coords', 'counts',
            'in_row_offsets', 'in_edge_ids', 'kernel_row_offsets', 'kernel_edge_ids')


def _dev(array, cuda):
    return torch.from_numpy(np.ascontiguousarray(array)).to(cuda)


def _active(n, cuda):
    return torch.tensor([n], dtype=torch.int32, device=cuda)


def _check_relation(got, want, n_kernels, keys=ALL_KEYS):
    for key in keys:
        assert np.array_equal(got[key], want[key]), key
    assert np.array_equal(canonical_edges(got), canonical_edges(want))
    for a, b in zip(canonical_pair_lists(got, n_kernels), canonical_pair_lists(want, n_kernels)):
        assert np.array_equal(a, b)


def _clouds():
    rng = np.random.default_rng(7)
    dense = np.stack(np.meshgrid(np.arange(12), np.arange(11), np.arange(9), indexing='ij'), -1)
    dense = dense.reshape(-1, 3)[rng.permutation(12 * 11 * 9)]
    dense = np.concatenate([np.zeros((dense.shape[0], 1), np.int64), dense], axis=1).astype(np.int32)
    negative = rng.integers(-40, 40, size=(6000, 4)).astype(np.int32)
    negative[:, 0] = rng.integers(0, 3, size=6000)
    with_dups = np.concatenate([negative[:2000], negative[:500], negative[1000:1700]])
    return {
        'lidar': synthetic.lidar_batch(2, 2, 15000),
        'sphere': synthetic.sphere_plane_batch(0, 2, 12000, 128),
        'dense': dense,
        'negative': negative,
        'duplicates': with_dups,
    }


CLOUDS = _clouds()
FORWARD_SPECS = [
    dict(kernel_size=3, stride=1, padding=0, dilation=1),
    dict(kernel_size=3, stride=2, padding=0, dilation=1),
    dict(kernel_size=2, stride=2, padding=0, dilation=1),
    dict(kernel_size=3, stride=2, padding=1, dilation=1),
    dict(kernel_size=(3, 1, 2), stride=(1, 2, 1), padding=(0, 1, 0), dilation=(1, 2, 1)),
    dict(kernel_size=5, stride=1, padding=0, dilation=1),
    dict(kernel_size=(3, 3, 4), stride=3, padding=0, dilation=1),
]


def test_reference_known_answer_line(cuda, oracle):
    # tests/native/test_coordinate_primitives.py:274-342 of the reference
    from mlx_lattice_b200 import _ext

    coords = np.array([[0, 0, 0, 0], [0, 1, 0, 0], [0, 2, 0, 0]], np.int32)
    got = relation_to_numpy(_ext.build_kernel_relation(_dev(coords, cuda), _active(3, cuda), (3, 1, 1), 1, 0, 1))
    assert got['counts'].tolist() == [7, 3]
    assert got['in_rows'][:7].tolist() == [0, 1, 0, 1, 2, 1, 2]
    assert got['out_rows'][:7].tolist() == [0, 0, 1, 1, 1, 2, 2]
    assert got['kernel_ids'][:7].tolist() == [1, 2, 0, 1, 2, 0, 1]
    assert got['row_offsets'].tolist() == [0, 2, 5, 7]
    assert got['in_row_offsets'].tolist() == [0, 2, 5, 7]
    assert got['in_edge_ids'][:7].tolist() == [0, 2, 1, 3, 5, 4, 6]
    assert got['kernel_row_offsets'].tolist() == [0, 2, 5, 7]
    assert got['kernel_edge_ids'][:7].tolist() == [2, 5, 0, 3, 6, 1, 4]
    _ext.check_status()


@pytest.mark.parametrize('cloud', sorted(CLOUDS))
@pytest.mark.parametrize('spec', FORWARD_SPECS, ids=lambda s: str(s['kernel_size']) + 's' + str(s['stride']))
def test_forward_relation(cuda, oracle, cloud, spec):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS[cloud]
    n = coords.shape[0]
    got = relation_to_numpy(_ext.build_kernel_relation(
        _dev(coords, cuda), _active(n, cuda), spec['kernel_size'], spec['stride'],
        spec['padding'], spec['dilation']))
    want = oracle.build_kernel_relation(coords, None, **spec)
    volume = int(np.prod(np.broadcast_to(np.asarray(spec['kernel_size']), 3)))
    _check_relation(got, want, volume)
    _ext.check_status()


@pytest.mark.parametrize('active', [0, 1, 257, 4000])
def test_active_rows_truncate_inputs(cuda, oracle, active):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['sphere'][:6000]
    for stride in (1, 2):
        got = relation_to_numpy(_ext.build_kernel_relation(
            _dev(coords, cuda), _active(active, cuda), 3, stride, 0, 1))
        want = oracle.build_kernel_relation(coords, active, kernel_size=3, stride=stride)
        _check_relation(got, want, 27)
    _ext.check_status()


def test_submanifold_entry_point(cuda, oracle):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['lidar']
    got = relation_to_numpy(_ext.build_submanifold_kernel_relation(
        _dev(coords, cuda), _active(coords.shape[0], cuda), 3, 1))
    want = oracle.build_submanifold_kernel_relation(coords)
    _check_relation(got, want, 27)


def test_empty_and_single_row(cuda, oracle):
    from mlx_lattice_b200 import _ext

    empty = torch.zeros((0, 4), dtype=torch.int32, device=cuda)
    got = relation_to_numpy(_ext.build_kernel_relation(empty, _active(0, cuda), 3, 1, 0, 1))
    assert got['counts'].tolist() == [0, 0] and got['row_offsets'].tolist() == [0]
    assert got['kernel_row_offsets'].tolist() == [0] * 28
    one = np.array([[1, -5, 7, 2]], np.int32)
    got = relation_to_numpy(_ext.build_kernel_relation(_dev(one, cuda), _active(1, cuda), 3, 2, 1, 1))
    want = oracle.build_kernel_relation(one, None, kernel_size=3, stride=2, padding=1)
    _check_relation(got, want, 27)


@pytest.mark.parametrize('cloud', ['sphere', 'negative', 'duplicates'])
def test_target_relation(cuda, oracle, cloud):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS[cloud]
    target, count = oracle.downsample_coords(coords, 2)
    target = target[: int(count[0])]
    target = np.concatenate([target[::-1], target[:100]])  # shuffled, with duplicates
    for src_active, tgt_active in ((coords.shape[0], target.shape[0]), (3000, 1111)):
        got = relation_to_numpy(_ext.build_target_kernel_relation(
            _dev(coords, cuda), _active(src_active, cuda), _dev(target, cuda),
            _active(tgt_active, cuda), 2, 2, 0, 1))
        want = oracle.build_target_kernel_relation(
            coords, target, src_active, tgt_active, kernel_size=2, stride=2)
        _check_relation(got, want, 8)
    _ext.check_status()


@pytest.mark.parametrize('spec', [
    dict(kernel_size=2, stride=2, padding=0, dilation=1),
    dict(kernel_size=(2, 1, 2), stride=(2, 3, 4), padding=(1, 0, 0), dilation=1),
    dict(kernel_size=3, stride=2, padding=1, dilation=1),
    dict(kernel_size=3, stride=1, padding=0, dilation=1),
    dict(kernel_size=2, stride=1, padding=0, dilation=2),
], ids=str)
def test_transposed_relation(cuda, oracle, spec):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['sphere'][:3000]
    for active in (3000, 777):
        got = relation_to_numpy(_ext.build_transposed_kernel_relation(
            _dev(coords, cuda), _active(active, cuda), spec['kernel_size'], spec['stride'],
            spec['padding'], spec['dilation']))
        want = oracle.build_transposed_kernel_relation(coords, active, **spec)
        volume = int(np.prod(np.broadcast_to(np.asarray(spec['kernel_size']), 3)))
        _check_relation(got, want, volume)
    _ext.check_status()


def test_generative_relation(cuda, oracle):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['negative'][:2500]
    for ks, stride in ((2, 2), ((1, 2, 3), (2, 2, 1))):
        got = relation_to_numpy(_ext.build_generative_relation(
            _dev(coords, cuda), _active(2000, cuda), ks, stride))
        want = oracle.build_generative_relation(coords, 2000, kernel_size=ks, stride=stride)
        _check_relation(got, want, int(np.prod(np.broadcast_to(np.asarray(ks), 3))))


def test_target_transposed_equals_reference_composition(cuda, oracle):
    """conv_transpose3d (k = s = 2) followed by a right-join alignment to the fine
    support, as the reference composes it, against the fused map."""
    from mlx_lattice_b200 import _ext

    fine = CLOUDS['sphere']
    coarse_rel = oracle.build_kernel_relation(fine, None, kernel_size=2, stride=2)
    n_coarse = int(coarse_rel['counts'][1])
    coarse = coarse_rel['out_coords'][:n_coarse]
    up = oracle.build_transposed_kernel_relation(coarse, None, kernel_size=2, stride=2)
    up_coords = up['out_coords'][: int(up['counts'][1])]
    _, _, lhs_rows, _ = oracle.sparse_alignment(up_coords, up_coords.shape[0], fine, fine.shape[0], 'right')
    want_in = np.where(lhs_rows >= 0, lhs_rows // 8, -1)
    want_k = np.where(lhs_rows >= 0, lhs_rows % 8, -1)
    base = _ext.build_target_transposed_relation_base(
        _dev(coarse, cuda), _active(n_coarse, cuda), _dev(fine, cuda), _active(fine.shape[0], cuda), 2)
    in_rows, out_rows, kernel_ids, row_offsets, _, counts = (t.cpu().numpy() for t in base)
    e = int(counts[0])
    assert e == int((lhs_rows >= 0).sum()) == fine.shape[0]
    got_in = np.full(fine.shape[0], -1)
    got_k = np.full(fine.shape[0], -1)
    got_in[out_rows[:e]] = in_rows[:e]
    got_k[out_rows[:e]] = kernel_ids[:e]
    assert np.array_equal(got_in, want_in) and np.array_equal(got_k, want_k)
    assert np.array_equal(row_offsets, np.arange(fine.shape[0] + 1))


def test_prebuilt_coord_table_gives_the_same_relations(cuda, oracle):
    """One coordinate table shared by the submanifold, strided and target-transposed
    builders (what the coordinate manager does) against the oracle and against the
    builders run with their own tables; duplicates and truncated active rows included."""
    from mlx_lattice_b200 import _ext

    cases = [('duplicates', None), ('sphere', 4000), ('lidar', None), ('negative', 1)]
    for name, active in cases:
        coords = CLOUDS[name]
        n_active = coords.shape[0] if active is None else active
        dev, act = _dev(coords, cuda), _active(n_active, cuda)
        table = _ext.build_coord_table(dev, act)
        for stride in (1, 2):
            shared, masks_shared, _ = _ext.build_kernel_relation_base(
                dev, act, 3, stride, 0, 1, want_masks=True, source_table=table)
            own, masks_own, _ = _ext.build_kernel_relation_base(
                dev, act, 3, stride, 0, 1, want_masks=True)
            want = oracle.build_kernel_relation(coords, n_active, kernel_size=3, stride=stride)
            edges, n_out = shared[5].tolist()
            assert [edges, n_out] == want['counts'].tolist()
            for got_arr, own_arr, key in zip(shared, own, ALL_KEYS):
                assert torch.equal(got_arr, own_arr), key
                assert np.array_equal(got_arr.cpu().numpy(), want[key]), key
            assert torch.equal(masks_shared[:n_out], masks_own[:n_out])
    _ext.check_status()
    # the coarse level's table serves the map back onto the fine support
    fine = CLOUDS['sphere']
    down = _ext.build_kernel_relation_base(_dev(fine, cuda), _active(fine.shape[0], cuda), 2, 2, 0, 1)[0]
    n_coarse = int(down[5][1])
    coarse, coarse_act = down[4], _active(n_coarse, cuda)
    table = _ext.build_coord_table(coarse, coarse_act)
    args = (coarse, coarse_act, _dev(fine, cuda), _active(fine.shape[0], cuda), 2)
    shared = _ext.build_target_transposed_relation_base(*args, source_table=table)
    own = _ext.build_target_transposed_relation_base(*args)
    for a, b in zip(shared, own):
        assert torch.equal(a, b)
    _ext.check_status()
    with pytest.raises(ValueError):
        _ext.build_kernel_relation_base(
            _dev(fine, cuda), _active(fine.shape[0], cuda), 3, 1, 0, 1,
            source_table=table[8:])


def test_grouped_views_and_igemm_view(cuda, oracle, restatement):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['dense']
    rel = oracle.build_kernel_relation(coords, None, kernel_size=3, stride=1)
    counts = _dev(rel['counts'], cuda)
    for ids, groups in ((rel['in_rows'], coords.shape[0]), (rel['kernel_ids'], 27), (rel['out_rows'], 5)):
        offsets, edge_ids = _ext.build_relation_grouped_view(_dev(ids, cuda), counts, groups)
        want_offsets, want_ids = restatement.grouped_view(ids, rel['counts'], groups)
        assert np.array_equal(offsets.cpu().numpy(), want_offsets)
        assert np.array_equal(edge_ids.cpu().numpy(), want_ids)
    offs = np.asarray(_ext.kernel_offsets(3), np.int32)
    for src_active, out_active in ((coords.shape[0], coords.shape[0]), (700, 900)):
        out_in_map, row_masks = _ext.build_relation_implicit_gemm_view(
            _dev(coords, cuda), _active(src_active, cuda), _dev(coords, cuda),
            _active(out_active, cuda), _dev(offs, cuda), 1, 0)
        want_map, want_masks = oracle.implicit_gemm_view(coords, src_active, coords, out_active, offs)
        assert np.array_equal(out_in_map.cpu().numpy(), want_map)
        assert np.array_equal(row_masks.cpu().numpy(), want_masks)
    _ext.check_status()


def test_row_masks_and_mask_order(cuda, oracle):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['sphere']
    n = coords.shape[0]
    base, masks, _ = _ext.build_kernel_relation_base(
        _dev(coords, cuda), _active(n - 100, cuda), 3, 1, 0, 1, want_masks=True)
    offs = np.asarray(_ext.kernel_offsets(3), np.int32)
    _, want_masks = oracle.implicit_gemm_view(coords, n - 100, coords, n - 100, offs)
    assert np.array_equal(masks.cpu().numpy(), want_masks)
    order = _ext.build_mask_row_order(masks, base[5], 27).cpu().numpy()
    assert np.array_equal(np.sort(order), np.arange(n))
    keys = np.where(np.arange(n) < n - 100, want_masks[:, 0].astype(np.uint32), np.uint32(0xFFFFFFFF))
    assert np.array_equal(order, np.argsort(keys, kind='stable'))


def test_coordinate_sets(cuda, oracle, restatement):
    from mlx_lattice_b200 import _ext

    coords = CLOUDS['duplicates']
    for stride in (2, (1, 3, 2)):
        out, count = _ext.downsample_coords(_dev(coords, cuda), stride)
        want = restatement.downsample_values(coords, stride)
        assert int(count.item()) == want.shape[0]
        assert np.array_equal(out.cpu().numpy()[: want.shape[0]], want)
        assert not out.cpu().numpy()[want.shape[0]:].any()
    queries = np.concatenate([coords[::7], coords[:50] + 1000])
    got = _ext.lookup_coords(_dev(coords, cuda), _dev(queries, cuda)).cpu().numpy()
    assert np.array_equal(got, restatement.lookup_coords(coords, queries))
    lhs, rhs = CLOUDS['negative'][:4000], CLOUDS['negative'][2000:6000][::-1].copy()
    for join in ('inner', 'left', 'right', 'outer'):
        got = _ext.build_sparse_alignment(
            _dev(lhs, cuda), _active(3500, cuda), _dev(rhs, cuda), _active(3900, cuda), join)
        want = oracle.sparse_alignment(lhs, 3500, rhs, 3900, join)
        for g, w in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w), join
    _ext.check_status()


def test_invalid_arguments_raise_value_error(cuda):
    from mlx_lattice_b200 import _ext

    coords = _dev(CLOUDS['dense'][:10], cuda)
    with pytest.raises(ValueError, match='active_rows must have shape'):
        _ext.build_kernel_relation(coords, torch.zeros(2, dtype=torch.int32, device=cuda), 3, 1, 0, 1)
    with pytest.raises(ValueError, match='kernel_size values must be positive'):
        _ext.build_kernel_relation(coords, _active(10, cuda), (3, 0, 3), 1, 0, 1)
    with pytest.raises(ValueError, match='stride values must be positive'):
        _ext.build_kernel_relation(coords, _active(10, cuda), 3, 0, 0, 1)
    with pytest.raises(ValueError, match='coords must have shape'):
        _ext.build_kernel_relation(coords[:, :3], _active(10, cuda), 3, 1, 0, 1)
    with pytest.raises(RuntimeError, match='no CPU route'):
        _ext.build_kernel_relation(coords.cpu(), _active(10, cuda), 3, 1, 0, 1)


def test_sorted_implicit_gemm_view_uses_the_reference_order(cuda):
    """The mask-sorted view (mlx_lattice/core/relations/views.py:467-510): rows in the order
    of a stable argsort of their offset masks (every row, active or not), the gathered map,
    and the OR of the masks over 16-row groups -- built with the native radix sort."""
    from mlx_lattice_b200.core import SparseTensor

    coords = synthetic.lidar_batch(2, 2, 3000)
    x = SparseTensor(torch.from_numpy(coords).to(cuda),
                     torch.zeros((coords.shape[0], 4), dtype=torch.float16, device=cuda))
    relation = x.coord_manager.kernel_relation(x.coord_key, kernel_size=3, stride=2)
    view = relation.require_implicit_gemm()
    masks = view.row_masks[:, 0].cpu().numpy()
    got = relation.require_sorted_implicit_gemm()
    order = np.argsort(masks, kind='stable').astype(np.int32)
    assert np.array_equal(got.reorder_rows.cpu().numpy(), order)
    sorted_map = view.out_in_map.cpu().numpy()[order]
    assert np.array_equal(got.sorted_out_in_map.cpu().numpy(), sorted_map)
    assert np.array_equal(got.sorted_kv_out_in_map.cpu().numpy(), sorted_map.T)
    n = masks.shape[0]
    padded = np.zeros(((n + 63) // 64) * 64, np.int32)
    padded[:n] = masks[order]
    want_tiles = np.bitwise_or.reduce(padded.reshape(-1, 16), axis=1)
    assert np.array_equal(got.tile_masks.cpu().numpy(), want_tiles)
