"""Generates tests/golden/reference_outputs.npz from the COMPILED REFERENCE
(oracle/_ref/liblattice_ref.so, i.e. the reference project's own CPU code).

Run where the reference checkout is present: `make -C oracle && python
tests/golden/make_golden.py`. The fixture pins the numpy restatement (and the GPU
path) on machines where the compiled reference is absent. Inputs are seeded and
small; every output array of the reference is stored.
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mlx_lattice_b200 import synthetic  # noqa: E402
from oracle import reference, restatement  # noqa: E402


def inputs():
    rng = np.random.default_rng(20260)
    lidar = synthetic.lidar_batch(2, 2, 1500)
    sphere = synthetic.sphere_plane_batch(0, 1, 2500, 48)
    dup = np.concatenate([sphere[:800], sphere[:200], sphere[300:500]])
    feats16 = rng.normal(size=(sphere.shape[0], 32)).astype(np.float16)
    feats32 = rng.normal(size=(sphere.shape[0], 8)).astype(np.float32)
    w16 = (rng.normal(size=(64, 3, 3, 3, 32)) * 0.05).astype(np.float16)
    w32 = (rng.normal(size=(5, 3, 3, 3, 8)) * 0.05).astype(np.float32)
    return dict(lidar=lidar, sphere=sphere, dup=dup, feats16=feats16, feats32=feats32,
                w16=w16, w32=w32)


def main() -> None:
    data = inputs()
    out = {f'in_{k}': v for k, v in data.items()}

    def put(prefix, rel):
        for key, value in rel.items():
            out[f'{prefix}.{key}'] = value

    put('subm_lidar', reference.build_submanifold_kernel_relation(data['lidar']))
    put('subm_sphere', reference.build_submanifold_kernel_relation(data['sphere']))
    put('k3s2_sphere', reference.build_kernel_relation(data['sphere'], None, 3, 2, 0, 1))
    put('k2s2_dup', reference.build_kernel_relation(data['dup'], 1000, 2, 2, 0, 1))
    put('k3s2p1_lidar', reference.build_kernel_relation(data['lidar'], None, 3, 2, 1, 1))
    put('tr_k2s2', reference.build_transposed_kernel_relation(data['sphere'][:400], 350, 2, 2, 0, 1))
    put('tr_k3s2p1', reference.build_transposed_kernel_relation(data['sphere'][:400], None, 3, 2, 1, 1))
    put('gen_k2s2', reference.build_generative_relation(data['lidar'][:300], None, 2, 2))
    target, count = reference.downsample_coords(data['sphere'], 2)
    out['downsample.coords'], out['downsample.count'] = target, count
    put('target_k2s2', reference.build_target_kernel_relation(
        data['sphere'], target[: int(count[0])][::-1].copy(), 2000, 500, 2, 2, 0, 1))
    out['in_target'] = target[: int(count[0])][::-1].copy()
    offs = reference.kernel_offsets(3)
    m, masks = reference.implicit_gemm_view(data['sphere'], 2000, data['sphere'], 2200, offs)
    out['igemm.out_in_map'], out['igemm.row_masks'] = m, masks
    for join in ('inner', 'left', 'right', 'outer'):
        res = reference.sparse_alignment(data['sphere'][:1500], 1400, data['dup'], 1100, join)
        for name, value in zip(('coords', 'count', 'lhs_rows', 'rhs_rows'), res):
            out[f'align_{join}.{name}'] = value

    rel = {k.split('.', 1)[1]: v for k, v in out.items() if k.startswith('subm_sphere.')}
    n = data['sphere'].shape[0]
    out['conv16'] = reference.sparse_conv(data['feats16'], data['w16'], rel, n, 27)
    out['conv32'] = reference.sparse_conv(data['feats32'], data['w32'], rel, n, 27)
    for bits in (4, 8):
        q = restatement.quantize_weight(data['w16'], 32, bits)
        out[f'q{bits}.weight'], out[f'q{bits}.scales'], out[f'q{bits}.biases'] = (
            q['weight'], q['scales'], q['biases'])
        out[f'qconv{bits}'] = reference.sparse_quantized_conv(
            data['feats16'], q['weight'], q['scales'], q['biases'], rel, n, 27, 32, 64, 32, 32, bits)
    prel = {k.split('.', 1)[1]: v for k, v in out.items() if k.startswith('k3s2_sphere.')}
    for mode in ('sum', 'max', 'avg'):
        out[f'pool_{mode}'] = reference.sparse_pool(
            data['feats32'], prel, input_exclusive=False, reduce=mode, out_capacity=n, n_kernels=27)
    # point -> voxel front end
    rng = np.random.default_rng(20261)
    points = (rng.normal(size=(6000, 3)) * 6.0).astype(np.float32)
    points[::5] = np.round(points[::5])
    batch = np.sort(rng.integers(0, 3, size=6000)).astype(np.int32)
    pfeats = rng.normal(size=(6000, 3)).astype(np.float32)
    out['in_points'], out['in_point_batch'], out['in_point_feats'] = points, batch, pfeats
    quant = reference.sparse_quantize(points, batch, np.asarray([5500], np.int32), (0.5, 1.0, 2.0),
                                      (0.25, -0.5, 0.0))
    for name, value in zip(('coords', 'count', 'inverse', 'counts'), quant):
        out[f'quantize.{name}'] = value
    for mode in ('mean', 'sum'):
        out[f'voxelize_{mode}'] = reference.voxelize_features(
            pfeats, quant[2], quant[3], np.asarray([5500], np.int32), mode)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'reference_outputs.npz')
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path) // 1024, 'KiB,', len(out), 'arrays')


if __name__ == '__main__':
    main()
