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


def all_gather_window_rows(local_rows, ranges, n2n, group=None):
    """Reassembles a per-voxel array from the pieces the ranks computed for their window ranges.

    One window set split over ranks (``shard_windows``): rank g owns the windows of its range and
    with them the voxels at sorted positions ``ranges[g] = [lo, hi)`` (``shard_voxel_range``).
    ``local_rows`` holds this rank's rows in SORTED order, shape ``[hi - lo, ...]``.  Pieces are
    disjoint, so one all-gather of the (padded) pieces followed by the un-permutation through
    ``n2n`` (sorted position -> voxel row) yields the full ``[N, ...]`` array in original voxel
    order on every rank; nothing else is exchanged.
    """
    import torch
    import torch.distributed as dist
    n2n = n2n.long()
    N = n2n.shape[0]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if len(ranges) != world:
        raise ValueError("one (lo, hi) range per rank is required")
    sizes = [hi - lo for lo, hi in ranges]
    rank = dist.get_rank(group) if world > 1 else 0
    if local_rows.shape[0] != sizes[rank]:
        raise ValueError(f"rank {rank}: expected {sizes[rank]} rows, got {local_rows.shape[0]}")
    full = torch.empty((N,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    if world == 1:
        full[n2n[ranges[0][0]:ranges[0][1]]] = local_rows
        return full
    pad = max(sizes)
    piece = torch.zeros((pad,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    piece[:sizes[rank]] = local_rows
    pieces = [torch.empty_like(piece) for _ in range(world)]
    dist.all_gather(pieces, piece, group=group)
    for (lo, hi), p, s in zip(ranges, pieces, sizes):
        if s:
            full[n2n[lo:hi]] = p[:s]
    return full


def sharded_attention(q, k, v, tq, tk, tv, sizes, w_sizes, w2n, n2n, n_coords, dout=None, group=None):
    """cRSE window attention on ONE window set split over the ranks of `group` by contiguous window
    ranges of equal pair count.  Every rank holds the full inputs, computes the windows of its range
    through the C-ABI kernels, and the per-voxel results are all-gathered; the table gradients are
    summed.  -> out [N,H,hd] (and, with `dout`, dq, dk, dv, (dtq, dtk, dtv)) identical on every rank.
    """
    import torch
    import torch.distributed as dist
    from .sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    ws_host = w_sizes.cpu().numpy()
    w2n_host = w2n.cpu().numpy()
    parts = shard_windows(ws_host, world)
    ranges = [shard_voxel_range(ws_host, w2n_host, a, b) for a, b in parts]
    a, b = parts[rank]
    lo, hi = ranges[rank]
    ws_l, w2n_l = w_sizes[a:b].contiguous(), w2n[a:b].contiguous()
    mine = n2n[lo:hi].long()
    out, lse = attn_forward_raw(q, k, v, tq, tk, tv, sizes, ws_l, w2n_l, n2n, n_coords)
    out_full = all_gather_window_rows(out[mine], ranges, n2n, group)
    if dout is None:
        return out_full
    grads = attn_backward_raw(q, k, v, tq, tk, tv, sizes, ws_l, w2n_l, n2n, n_coords, out, lse, dout)
    dq, dk, dv = (all_gather_window_rows(x[mine], ranges, n2n, group) for x in grads[:3])
    tg = allreduce_table_grads(tuple(grads[3:6]), group)
    return out_full, dq, dk, dv, tg
