"""Batch-element sharding over the GPUs of one box.

Point clouds shard naturally: the batch index is part of every coordinate key, so no
kernel-map edge connects two batch elements and weights are replicated. Each rank
owns a contiguous range of clouds; batch ids stay global. The only exchange on the
path is the all-gather of per-cloud global-pool rows.
"""

from __future__ import annotations

import numpy as np
import torch


def shard_range(num_clouds: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) range of cloud indices owned by `rank` (earlier ranks
    take the remainder)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError('rank must lie in [0, world).')
    base, extra = divmod(num_clouds, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_rows(batch_counts, world: int, rank: int) -> tuple[int, int]:
    """Row range of a batch-contiguous tensor owned by `rank`."""
    begin, end = shard_range(len(batch_counts), world, rank)
    offsets = np.concatenate([[0], np.cumsum(batch_counts)])
    return int(offsets[begin]), int(offsets[end])


def merge_relations(shards: list[dict], row_starts: list[int], out_starts: list[int]) -> dict:
    """Concatenate per-shard kernel maps (dicts of numpy arrays with in_rows, out_rows,
    kernel_ids, counts) into the single-device map: row ids are shifted by the shard's
    first input / output row. Used to check that sharding reproduces the unsharded map."""
    in_rows, out_rows, kernel_ids = [], [], []
    for rel, row0, out0 in zip(shards, row_starts, out_starts):
        e = int(rel['counts'][0])
        in_rows.append(rel['in_rows'][:e] + row0)
        out_rows.append(rel['out_rows'][:e] + out0)
        kernel_ids.append(rel['kernel_ids'][:e])
    return {
        'in_rows': np.concatenate(in_rows),
        'out_rows': np.concatenate(out_rows),
        'kernel_ids': np.concatenate(kernel_ids),
        'counts': np.asarray([sum(int(r['counts'][0]) for r in shards),
                              sum(int(r['counts'][1]) for r in shards)], np.int32),
    }


def gather_global_pool(local_rows: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the (B_local, C) global-pool rows into (B, C) on every rank; every
    rank must hold the same B_local. NCCL on GPUs, gloo on the CPU."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_rows
    parts = [torch.empty_like(local_rows) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, local_rows.contiguous(), group=group)
    return torch.cat(parts, dim=0)
