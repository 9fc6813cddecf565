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
    """All-gather of the (B_local, C) global-pool rows into (B, C) on every rank, in rank
    order. Ranks may hold different B_local (``shard_range`` gives the earlier ranks one
    cloud more when the clouds do not divide evenly): the row counts are exchanged first
    and every rank pads its block to the largest one, because an all-gather of unequal
    blocks is undefined. NCCL on GPUs, gloo on the CPU."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_rows
    world = dist.get_world_size(group)
    if local_rows.ndim != 2:
        raise ValueError('global-pool rows must have shape (B_local, C).')
    counts = [torch.zeros(2, dtype=torch.int64, device=local_rows.device) for _ in range(world)]
    mine = torch.tensor([local_rows.shape[0], local_rows.shape[1]], dtype=torch.int64,
                        device=local_rows.device)
    dist.all_gather(counts, mine, group=group)
    sizes = [tuple(int(v) for v in c.tolist()) for c in counts]
    if any(channels != sizes[0][1] for _, channels in sizes):
        raise ValueError('every rank must hold global-pool rows of the same channel count.')
    largest = max(rows for rows, _ in sizes)
    block = local_rows.new_zeros((largest, local_rows.shape[1]))
    block[: local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(block) for _ in range(world)]
    dist.all_gather(parts, block, group=group)
    return torch.cat([part[:rows] for part, (rows, _) in zip(parts, sizes)], dim=0)
