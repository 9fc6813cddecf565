"""Seeded synthetic point clouds used by the benchmark and the parity tests.

They stand in for real scans: the reference's own benchmarks use closed-form
layouts (``benchmarks/mlx_lattice_bench/datasets.py:10-19,130-160``) and no public
dataset. Everything here is host-side numpy; nothing touches the GPU.

RNG convention: ``numpy.random.default_rng(seed)`` with ``seed = 20260 +
config_index + 1000 * cloud_index``.
"""

from __future__ import annotations

import numpy as np

BASE_SEED = 20260


def cloud_seed(config_index: int, cloud_index: int) -> int:
    return BASE_SEED + config_index + 1000 * cloud_index


def _dedupe_first_seen(points: np.ndarray) -> np.ndarray:
    """Unique integer rows, keeping the first occurrence order."""
    if points.shape[0] == 0:
        return points
    lo = points.min(axis=0)
    span = points.max(axis=0) - lo + 1
    key = np.zeros(points.shape[0], np.int64)
    for axis in range(points.shape[1]):
        key = key * int(span[axis]) + (points[:, axis] - lo[axis])
    _, first = np.unique(key, return_index=True)
    return points[np.sort(first)]


def sphere_plane_cloud(seed: int, grid: int, target: int) -> np.ndarray:
    """Points on the union of 4 random spheres and 2 random axis-aligned planes.

    Sphere centres ~ U(0, grid)^3, radii ~ U(30, 100) * grid / 256; plane axis
    ~ U{x, y, z}, position ~ U(0, grid). Surfaces are sampled area-proportionally,
    rounded to integers, clipped to [0, grid), deduplicated in first-seen order and
    truncated to exactly ``target`` rows. Returns int32 (target, 3).
    """
    rng = np.random.default_rng(seed)
    scale = grid / 256.0
    centres = rng.uniform(0, grid, size=(4, 3))
    radii = rng.uniform(30, 100, size=4) * scale
    plane_axis = rng.integers(0, 3, size=2)
    plane_pos = rng.uniform(0, grid, size=2)
    areas = np.concatenate([4 * np.pi * radii**2, np.full(2, float(grid) ** 2)])
    prob = areas / areas.sum()
    chunks: list[np.ndarray] = []
    have = np.zeros((0, 3), np.int64)
    while have.shape[0] < target:
        n = max(2 * target, 1024)
        which = rng.choice(6, size=n, p=prob)
        pts = np.empty((n, 3), np.float64)
        direction = rng.normal(size=(n, 3))
        direction /= np.linalg.norm(direction, axis=1, keepdims=True) + 1e-12
        flat = rng.uniform(0, grid, size=(n, 3))
        for s in range(4):
            sel = which == s
            pts[sel] = centres[s] + radii[s] * direction[sel]
        for p in range(2):
            sel = which == 4 + p
            chunk = flat[sel]
            chunk[:, plane_axis[p]] = plane_pos[p]
            pts[sel] = chunk
        ints = np.clip(np.rint(pts), 0, grid - 1).astype(np.int64)
        chunks.append(ints)
        have = _dedupe_first_seen(np.concatenate(chunks, axis=0))
    return have[:target].astype(np.int32)


def lidar_cloud(seed: int, target: int, grid: int = 1024) -> np.ndarray:
    """LiDAR-like sweep: 64 beams with elevations linspace(-25 deg, 3 deg), 2048
    azimuth steps, range ~ U(2, 70) m times (1 + 0.1 N(0,1)), voxel size 0.05 m,
    translated by +grid/2; rays that land outside [0, grid)^3 are dropped (our
    choice of how the sweep is fitted into the grid). Sweeps are repeated with
    fresh noise until ``target`` unique voxels exist; first-seen order, truncated.
    Returns int32 (target, 3).
    """
    rng = np.random.default_rng(seed)
    elev = np.deg2rad(np.linspace(-25.0, 3.0, 64))
    azim = np.linspace(0.0, 2 * np.pi, 2048, endpoint=False)
    ee, aa = np.meshgrid(elev, azim, indexing='ij')
    ee, aa = ee.reshape(-1), aa.reshape(-1)
    chunks: list[np.ndarray] = []
    have = np.zeros((0, 3), np.int64)
    while have.shape[0] < target:
        r = rng.uniform(2.0, 70.0, size=ee.shape[0])
        r = r * (1.0 + 0.1 * rng.normal(size=ee.shape[0]))
        xyz = np.stack(
            [r * np.cos(ee) * np.cos(aa), r * np.cos(ee) * np.sin(aa), r * np.sin(ee)],
            axis=1,
        )
        vox = np.floor(xyz / 0.05).astype(np.int64) + grid // 2
        keep = np.all((vox >= 0) & (vox < grid), axis=1)
        chunks.append(vox[keep])
        have = _dedupe_first_seen(np.concatenate(chunks, axis=0))
    return have[:target].astype(np.int32)


def batched(clouds: list[np.ndarray], first_batch: int = 0) -> np.ndarray:
    """Concatenate per-cloud (n, 3) voxels into batch-contiguous (N, 4) int32
    (b, x, y, z) rows, as ``sparse_collate`` does
    (``mlx_lattice/ops/tensor.py:15-64``)."""
    rows = []
    for index, cloud in enumerate(clouds):
        b = np.full((cloud.shape[0], 1), first_batch + index, np.int32)
        rows.append(np.concatenate([b, cloud.astype(np.int32)], axis=1))
    return np.ascontiguousarray(np.concatenate(rows, axis=0))


def sphere_plane_batch(config_index, batch, per_cloud, grid, first_batch=0):
    clouds = [
        sphere_plane_cloud(cloud_seed(config_index, first_batch + i), grid, per_cloud)
        for i in range(batch)
    ]
    return batched(clouds, first_batch)


def lidar_batch(config_index, batch, per_cloud, grid=1024, first_batch=0):
    clouds = [
        lidar_cloud(cloud_seed(config_index, first_batch + i), per_cloud, grid)
        for i in range(batch)
    ]
    return batched(clouds, first_batch)
