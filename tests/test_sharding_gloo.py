"""Batch sharding on two CPU ranks (gloo): per-shard kernel maps concatenate to the
unsharded map bit-exactly, and the global-pool all-gather assembles the (B, C) rows."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

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
    dist.init_process_group('gloo', rank=rank, world_size=world)
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
    ctx = mp.get_context('spawn')
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert results.get(timeout=10) is True
