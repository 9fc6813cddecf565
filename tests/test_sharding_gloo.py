"""Batch sharding on two CPU ranks (gloo): per-shard kernel maps concatenate to the
unsharded map bit-exactly, and the global-pool all-gather assembles the (B, C) rows."""

import os
import socket

from datetime import timedelta

import numpy as np
import pytest
import torch
import torch.distributed as dist

from conftest import run_ranks
from mlx_lattice_b200 import sharding, synthetic
from oracle import restatement

CLOUDS, PER_CLOUD = 4, 1500


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=timedelta(seconds=120))
    try:
        coords = synthetic.lidar_batch(2, CLOUDS, PER_CLOUD)
        counts = (PER_CLOUD,) * CLOUDS
        row0, row1 = sharding.shard_rows(counts, world, rank)
        local = coords[row0:row1]
        rel = restatement.build_kernel_relation(local, None, kernel_size=3, stride=2)
        n_out = int(rel['counts'][1])
        # exchange shard sizes, then the maps themselves (test-only traffic)
        sizes = [None] * world
        dist.all_gather_object(sizes, (row0, n_out))
        payload = [None] * world
        keep = {k: rel[k] for k in ('in_rows', 'out_rows', 'kernel_ids', 'counts')}
        keep['out_coords'] = rel['out_coords'][:n_out]
        dist.all_gather_object(payload, keep)
        # global pool rows: one row per local cloud, gathered to (CLOUDS, C)
        feats = torch.arange(local.shape[0] * 3, dtype=torch.float32).reshape(-1, 3) + rank
        begin, end = sharding.shard_range(CLOUDS, world, rank)
        pooled = torch.stack([
            feats[i * PER_CLOUD:(i + 1) * PER_CLOUD].mean(dim=0) for i in range(end - begin)])
        gathered = sharding.gather_global_pool(pooled)
        if rank == 0:
            out_starts = np.concatenate([[0], np.cumsum([n for _, n in sizes])])[:-1].tolist()
            merged = sharding.merge_relations(payload, [r for r, _ in sizes], out_starts)
            full = restatement.build_kernel_relation(coords, None, kernel_size=3, stride=2)
            e = int(full['counts'][0])
            ok = (np.array_equal(merged['counts'], full['counts'])
                  and all(np.array_equal(merged[k], full[k][:e])
                          for k in ('in_rows', 'out_rows', 'kernel_ids'))
                  and np.array_equal(np.concatenate([p['out_coords'] for p in payload]),
                                     full['out_coords'][: int(full['counts'][1])])
                  and tuple(gathered.shape) == (CLOUDS, 3))
            results.put(bool(ok))
    finally:
        dist.destroy_process_group()


def test_shard_ranges_cover_all_clouds():
    for clouds in (1, 4, 7, 8, 16):
        for world in (1, 2, 3, 8):
            ranges = [sharding.shard_range(clouds, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == clouds
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def test_two_rank_sharding_reproduces_unsharded_maps():
    codes, results = run_ranks(_worker, 2, (_free_port(),), timeout=180)
    assert codes == [0, 0]
    assert results.get(timeout=10) is True


def _uneven_worker(rank: int, world: int, port: int, clouds: int, results) -> None:
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=timedelta(seconds=120))
    try:
        begin, end = sharding.shard_range(clouds, world, rank)
        # row b of the joint result is (b, 10 b, 100 b)
        local = torch.tensor([[b, 10.0 * b, 100.0 * b] for b in range(begin, end)],
                             dtype=torch.float32).reshape(end - begin, 3)
        gathered = sharding.gather_global_pool(local)
        want = torch.tensor([[b, 10.0 * b, 100.0 * b] for b in range(clouds)], dtype=torch.float32)
        results.put((rank, bool(torch.equal(gathered, want.reshape(clouds, 3)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('clouds,world', [(5, 2), (7, 3), (2, 3)])
def test_global_pool_gather_with_an_uneven_split(clouds, world):
    """CLOUDS % world != 0: the earlier ranks hold one cloud more (one rank may hold none);
    the gather still returns the (CLOUDS, C) rows in cloud order on every rank."""
    codes, results = run_ranks(_uneven_worker, world, (_free_port(), clouds), timeout=180)
    assert codes == [0] * world
    seen = sorted(results.get(timeout=10) for _ in range(world))
    assert seen == [(rank, True) for rank in range(world)]
