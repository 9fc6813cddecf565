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
