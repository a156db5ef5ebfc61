"""Partitioning helpers for running the path on several GPUs (one process per GPU).

Windows are independent work units, scenes are independent, KNN queries are independent, so the
path shards without any exchange of per-voxel data when every rank owns whole scenes (data-parallel
training): the only collective is the sum of the three table-gradient arrays, which are ordinary
parameters.  ``shard_windows`` covers the other case, one window set split over ranks.
"""
from typing import List, Tuple

import numpy as np


def shard_windows(w_sizes, world_size: int) -> List[Tuple[int, int]]:
    """Cuts the window list into `world_size` contiguous ranges of near-equal cost (sum of w^2,
    the number of attention pairs).  -> [(first_window, end_window)] per rank; ranges are disjoint,
    ordered and cover every window; a rank may get an empty range when there are fewer windows
    than ranks."""
    w = np.asarray(w_sizes, dtype=np.int64)
    W = len(w)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    cost = np.cumsum(w * w)
    total = int(cost[-1]) if W else 0
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        c = int(np.searchsorted(cost, target, side="left")) + 1 if W else 0
        cuts.append(min(max(c, cuts[-1]), W))
    cuts.append(W)
    return [(cuts[r], cuts[r + 1]) for r in range(world_size)]


def shard_voxel_range(w_sizes, w2n, first_window: int, end_window: int) -> Tuple[int, int]:
    """Sorted-position range [begin, end) of the voxels of windows [first_window, end_window)."""
    if first_window >= end_window:
        return (0, 0)
    begin = int(w2n[first_window])
    end = int(w2n[end_window - 1]) + int(w_sizes[end_window - 1])
    return (begin, end)


def allreduce_table_grads(grads, group=None):
    """Sums the (dtq, dtk, dtv) arrays over ranks in one collective (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return grads
    flat = torch.stack([g.contiguous() for g in grads])
    dist.all_reduce(flat, group=group)
    return tuple(flat[i] for i in range(len(grads)))
