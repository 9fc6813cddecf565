"""Test infrastructure only -- the MinkUNet-style network composed from the CPU
oracle exactly the way the reference composes it: the decoder up-sampling is
``conv_transpose3d`` (direct transposed relation, 8 output rows per input row,
``mlx_lattice/ops/conv.py:153-182``) followed by ``sparse_cat_aligned(up, skip,
join='right')`` (``mlx_lattice/ops/tensor.py:228-249``). ``backend`` is
``oracle.reference`` (compiled reference code) or ``oracle.restatement``.
"""

from __future__ import annotations

import time

import numpy as np

from oracle import restatement


def quantized_to_numpy(q) -> dict:
    """A packed weight of the package under test (CPU tensors with ``.numpy()``) as the
    dict of numpy arrays the oracle consumes."""
    return {
        'weight': q.weight.numpy().view(np.uint32),
        'scales': q.scales.numpy(),
        'biases': q.biases.numpy(),
        'group_size': q.group_size,
        'bits': q.bits,
        'in_channels': q.in_channels,
        'out_channels': q.out_channels,
        'kernel_size': q.kernel_size,
        'layout': q.layout,
        'storage_in_channels': q.storage_in_channels,
    }


def _qconv(backend, feats, q, rel, out_capacity, n_kernels):
    return backend.sparse_quantized_conv(
        feats, q['weight'], q['scales'], q['biases'], rel, out_capacity, n_kernels,
        q['in_channels'], q['out_channels'], q['storage_in_channels'], q['group_size'], q['bits'],
    )


def minkunet_forward(backend, coords, feats, quantized: dict, layers, timings: dict | None = None):
    """``quantized`` maps layer name -> dict with numpy packed arrays (the same arrays
    the GPU path consumes). Returns (logits (N, 20) fp16)."""

    def timed(key, fn):
        start = time.perf_counter()
        out = fn()
        if timings is not None:
            timings[key] = timings.get(key, 0.0) + time.perf_counter() - start
        return out

    coords = np.asarray(coords, np.int32)
    n0 = coords.shape[0]
    level_coords = [coords]
    level_active = [n0]
    subm = {}

    def subm_rel(level):
        if level not in subm:
            subm[level] = timed('relation', lambda: backend.build_submanifold_kernel_relation(
                level_coords[level], level_active[level]))
        return subm[level]

    def subm_conv(x, name, level):
        rel = subm_rel(level)
        return timed('conv', lambda: _qconv(backend, x, quantized[name], rel, level_coords[level].shape[0], 27))

    names = [l[0] for l in layers]
    stages = sum(1 for n in names if n.startswith('down'))
    skips = [subm_conv(feats, 'stem', 0)]
    cur = skips[0]
    for i in range(1, stages + 1):
        prev = i - 1
        rel = timed('relation', lambda: backend.build_kernel_relation(
            level_coords[prev], level_active[prev], kernel_size=2, stride=2))
        cap = level_coords[prev].shape[0]
        cur = timed('conv', lambda: _qconv(backend, cur, quantized[f'down{i}'], rel, cap, 8))
        level_coords.append(rel['out_coords'])
        level_active.append(int(rel['counts'][1]))
        cur = subm_conv(cur, f'enc{i}a', i)
        cur = subm_conv(cur, f'enc{i}b', i)
        if i < stages:
            skips.append(cur)
    for i in range(stages, 0, -1):
        fine = i - 1
        rel = timed('relation', lambda: backend.build_transposed_kernel_relation(
            level_coords[i], level_active[i], kernel_size=2, stride=2))
        up_cap = level_coords[i].shape[0] * 8
        up = timed('conv', lambda: _qconv(backend, cur, quantized[f'up{i}'], rel, up_cap, 8))
        up_active = int(rel['counts'][1])
        _, _, lhs_rows, rhs_rows = timed('alignment', lambda: backend.sparse_alignment(
            rel['out_coords'], up_active, level_coords[fine], level_active[fine], 'right'))
        skip = skips[fine]
        gathered_up = np.where(lhs_rows[:, None] >= 0, up[np.maximum(lhs_rows, 0)], 0).astype(up.dtype)
        gathered_skip = np.where(rhs_rows[:, None] >= 0, skip[np.maximum(rhs_rows, 0)], 0).astype(skip.dtype)
        cur = np.concatenate([gathered_up, gathered_skip], axis=1)
        cur = subm_conv(cur, f'dec{i}a', fine)
        cur = subm_conv(cur, f'dec{i}b', fine)
    return timed('linear', lambda: restatement.quantized_matmul(cur, quantized['head']))
