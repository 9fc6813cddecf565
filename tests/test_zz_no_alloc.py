"""The allocation-free lookup entry point (collected last on purpose: it shares one
fixed device array between calls, so it runs after everything else).

Some callers of this library may not allocate device memory once they are running and
have no scratch buffer to lend; for them `lat_lookup_coords_static` keeps its hash
table in a fixed array inside the library. The test calls it through the C ABI twice in
a row -- the second time with a different, smaller source set, which only works if the
shared table is cleared between calls -- and expects exactly the rows the regular,
workspace-based entry point returns."""

import numpy as np
import pytest
import torch

from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu


def test_static_lookup_matches_workspace_lookup_twice(cuda):
    from mlx_lattice_b200 import _ext

    rng = np.random.default_rng(41)
    first = synthetic.lidar_batch(2, 2, 60000)
    second = synthetic.sphere_plane_batch(0, 1, 9000, 64)
    for coords in (first, second):
        queries = np.concatenate([coords[::3], coords[:200] + 5000,
                                  rng.integers(-50, 50, size=(300, 4)).astype(np.int32)])
        c = torch.from_numpy(coords).to(cuda)
        q = torch.from_numpy(np.ascontiguousarray(queries)).to(cuda)
        want = _ext.lookup_coords(c, q)
        out = torch.full((q.shape[0],), -7, dtype=torch.int32, device=cuda)
        got = _ext.lookup_coords_static(c, q, out=out)
        assert got is out
        assert torch.equal(got, want)
        assert int((want >= 0).sum()) >= coords[::3].shape[0]
    _ext.check_status()


def test_static_lookup_rejects_oversized_input(cuda):
    from mlx_lattice_b200 import _ext

    limit = _ext.lookup_coords_static_max_rows()
    assert limit == 262144
    too_many = torch.zeros((limit + 1, 4), dtype=torch.int32, device=cuda)
    with pytest.raises(ValueError, match='at most 262144 source rows'):
        _ext.lookup_coords_static(too_many, too_many[:4])


def test_static_lookup_allocates_nothing_and_handles_the_edges_of_its_range(cuda):
    """What the entry point is for: with inputs and `out` already on the device, a call
    leaves this process's device allocator untouched (the GPU-wide free figure is not
    compared: other jobs share the device). Also: a source set at the
    limit (the table then is the whole fixed array), an empty source set, and a small call
    after a large one (slots of the large call beyond the small table must not be seen)."""
    from mlx_lattice_b200 import _ext

    limit = _ext.lookup_coords_static_max_rows()
    rng = np.random.default_rng(5)
    cells = rng.permutation(128 ** 3)[:limit]
    big = np.stack([np.zeros(limit, np.int64), cells // (128 * 128), (cells // 128) % 128, cells % 128],
                   axis=1).astype(np.int32)
    big_dev = torch.from_numpy(big).to(cuda)
    queries = torch.from_numpy(np.ascontiguousarray(
        np.concatenate([big[::5], big[:1000] + 300]))).to(cuda)
    out = torch.empty(queries.shape[0], dtype=torch.int32, device=cuda)
    want = _ext.lookup_coords(big_dev, queries)
    _ext.lookup_coords_static(big_dev, queries, out=out)      # first call: address look-up
    torch.cuda.synchronize()
    allocated, reserved = torch.cuda.memory_allocated(cuda), torch.cuda.memory_reserved(cuda)
    got = _ext.lookup_coords_static(big_dev, queries, out=out)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(cuda) == allocated
    assert torch.cuda.memory_reserved(cuda) == reserved
    assert torch.equal(got, want)
    # a small source set right after the large one
    small = big_dev[:37].contiguous()
    small_out = torch.empty(queries.shape[0], dtype=torch.int32, device=cuda)
    assert torch.equal(_ext.lookup_coords_static(small, queries, out=small_out),
                       _ext.lookup_coords(small, queries))
    # no source rows at all: every query misses
    none = torch.empty((0, 4), dtype=torch.int32, device=cuda)
    assert torch.equal(_ext.lookup_coords_static(none, queries, out=small_out),
                       torch.full_like(small_out, -1))
    with pytest.raises(ValueError, match='out must be'):
        _ext.lookup_coords_static(small, queries, out=torch.empty(queries.shape[0], dtype=torch.int32))
    _ext.check_status()
