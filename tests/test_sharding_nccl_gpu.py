"""Batch sharding on two GPUs (NCCL): each rank runs its clouds through the GPU path, the
global-pool rows are all-gathered, and rank 0 checks the result against the joint run on
one GPU. Skipped on a single-GPU box."""

import os
import socket

from datetime import timedelta

import numpy as np
import pytest
import torch

from conftest import run_ranks

pytestmark = pytest.mark.gpu

CLOUDS, PER_CLOUD, CHANNELS = 4, 5000, 32


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _inputs():
    from mlx_lattice_b200 import synthetic

    coords = synthetic.lidar_batch(3, CLOUDS, PER_CLOUD)
    rng = np.random.default_rng(12)
    feats = rng.normal(size=(coords.shape[0], CHANNELS)).astype(np.float32)
    weight = (rng.normal(size=(CHANNELS, 3, 3, 3, CHANNELS)) * 0.05).astype(np.float32)
    return coords, feats, weight


def _pooled(device, coords, feats, weight, counts):
    from mlx_lattice_b200 import ops
    from mlx_lattice_b200.core import SparseTensor

    x = SparseTensor(torch.from_numpy(coords).to(device), torch.from_numpy(feats).to(device),
                     batch_counts=counts)
    y = ops.subm_conv3d(x, torch.from_numpy(weight).to(device), kernel_size=3)
    return ops.global_avg_pool(y)


def _worker(rank: int, world: int, port: int, results) -> None:
    import torch.distributed as dist

    from mlx_lattice_b200 import sharding

    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    device = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device,
                            timeout=timedelta(seconds=120))
    try:
        coords, feats, weight = _inputs()
        counts = (PER_CLOUD,) * CLOUDS
        row0, row1 = sharding.shard_rows(counts, world, rank)
        begin, end = sharding.shard_range(CLOUDS, world, rank)
        local = _pooled(device, coords[row0:row1], feats[row0:row1], weight, counts[begin:end])
        gathered = sharding.gather_global_pool(local)
        torch.cuda.synchronize()
        if rank == 0:
            joint = _pooled(device, coords, feats, weight, counts)
            results.put(bool(torch.equal(gathered, joint)) and tuple(gathered.shape) == (CLOUDS, CHANNELS))
    finally:
        dist.destroy_process_group()


def test_two_gpu_shards_gather_the_joint_global_pool():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    codes, results = run_ranks(_worker, 2, (_free_port(),), timeout=300)
    assert codes == [0, 0]
    assert results.get(timeout=10) is True
