"""Running the path on several GPUs (one process per GPU).

Windows are independent work units, scenes are independent, KNN queries are independent.  When every
rank owns whole scenes (data-parallel training) the only collective is the sum of the three
table-gradient arrays, which are ordinary parameters.  The other case, ONE window set split over the
ranks, is what this module does:

* ``shard_windows`` cuts the window list into contiguous ranges of equal cost;
* ``ShardPlan`` holds everything about one (window set, world size, rank) that does not change
  between calls -- ranges, the rank's slice of the window arrays, the gather index of its rows and
  the inverse index that puts gathered rows back into voxel order.  Building it reads the window
  sizes on the host once; it is cached per window set, so a step does no host synchronisation;
* ``exchange_rows`` packs any number of per-voxel arrays of a rank into ONE buffer, runs ONE
  ``all_gather_into_tensor`` (equal, padded shards) and un-permutes everything with ONE gather;
* ``sharded_attention_step`` runs forward + backward of the rank's windows in chunks so that the
  all-gather of a chunk overlaps the kernels of the next one, and sums the table gradients.

Only NCCL (gloo on CPU) collectives on the caller's buffers are used: no peer-memory loads, no
symmetric memory.
"""
import weakref
from typing import List, Optional, Sequence, Tuple

import numpy as np

TILE = 32   # voxels per tile of the attention kernels


def window_cost(w_sizes) -> np.ndarray:
    """Cost model of a window for the attention kernels: a fixed part per 32 x 32 tile pair (the
    table projections and histogram products do not depend on how full a tile is) plus a part per
    attention pair."""
    w = np.asarray(w_sizes, dtype=np.int64)
    nt = (w + TILE - 1) // TILE
    return nt * nt * 600 + w * w


def shard_windows(w_sizes, world_size: int, cost=None) -> List[Tuple[int, int]]:
    """Cuts the window list into `world_size` contiguous ranges of near-equal cost (default: the
    number of attention pairs, sum of w^2; pass ``window_cost(w_sizes)`` for the kernels' cost
    model).  -> [(first_window, end_window)] per rank; ranges are disjoint, ordered and cover every
    window; a rank may get an empty range when there are fewer windows than ranks."""
    w = np.asarray(w_sizes, dtype=np.int64)
    W = len(w)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    c = (w * w) if cost is None else np.asarray(cost, dtype=np.int64)
    if len(c) != W:
        raise ValueError("one cost per window is required")
    csum = np.cumsum(c)
    total = int(csum[-1]) if W else 0
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        x = int(np.searchsorted(csum, target, side="left")) + 1 if W else 0
        cuts.append(min(max(x, cuts[-1]), W))
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
    order on every rank; nothing else is exchanged.  (The general, uncached form; a training or
    benchmark loop uses ``ShardPlan`` + ``exchange_rows``.)
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


class ShardPlan:
    """One window set split over `world` ranks, from the point of view of `rank`.

    parts[r] = (first_window, end_window) of rank r, cut by ``window_cost``; every rank's range is
    further cut into `chunks` sub-ranges of equal cost (chunk c of every rank is exchanged together).
    For chunk c: ``chunk_windows[c]`` = this rank's (first, end) windows, ``pad[c]`` = rows of the
    largest shard of that chunk over the ranks, ``gather_idx[c]`` = int64 [pad[c]] voxel rows of this
    rank's shard in sorted order (padded with row 0).  ``slot`` = int64 [N]: for voxel row v the row of
    the gathered buffer (laid out [chunk][rank][array][pad]) that holds v, for array 0 of `A` arrays:
    ``slot_base + a * pad_of_voxel``, see ``exchange_rows``.
    """

    def __init__(self, w_sizes, w2n, n2n, world: int, rank: int, chunks: int = 1):
        import torch
        ws = w_sizes.detach().cpu().numpy().astype(np.int64)       # the one host read, at plan time
        w2 = w2n.detach().cpu().numpy().astype(np.int64)
        if not (0 <= rank < world):
            raise ValueError("rank out of range")
        chunks = max(1, int(chunks))
        self.world, self.rank, self.chunks = world, rank, chunks
        self.N = int(n2n.shape[0])
        cost = window_cost(ws)
        self.parts = shard_windows(ws, world, cost)
        dev = n2n.device
        n2n64 = n2n.long()
        # sub-ranges of every rank
        sub = []                                   # [rank][chunk] -> (a, b, lo, hi)
        for a, b in self.parts:
            cuts = shard_windows(ws[a:b], chunks, cost[a:b])
            sub.append([(a + x, a + y) + shard_voxel_range(ws, w2, a + x, a + y) for x, y in cuts])
        self.pad = [max(8, -(-max(sub[r][c][3] - sub[r][c][2] for r in range(world)) // 8) * 8)
                    for c in range(chunks)]
        self.chunk_windows = [(sub[rank][c][0], sub[rank][c][1]) for c in range(chunks)]
        self.chunk_rows = [(sub[rank][c][2], sub[rank][c][3]) for c in range(chunks)]
        self.w_sizes_chunk = [w_sizes[a:b].contiguous() for a, b in self.chunk_windows]
        self.w2n_chunk = [w2n[a:b].contiguous() for a, b in self.chunk_windows]
        self.gather_idx = []
        for c in range(chunks):
            lo, hi = self.chunk_rows[c]
            idx = torch.zeros(self.pad[c], dtype=torch.int64, device=dev)
            idx[:hi - lo] = n2n64[lo:hi]
            self.gather_idx.append(idx)
        # inverse map: sorted position -> (chunk, rank, offset); stored per voxel row as
        # slot_chunk_base (row offset of the chunk's block for ONE array) and slot_in_chunk
        pos_chunk = np.zeros(self.N, dtype=np.int64)
        pos_rank = np.zeros(self.N, dtype=np.int64)
        pos_off = np.zeros(self.N, dtype=np.int64)
        for r in range(world):
            for c in range(chunks):
                _, _, lo, hi = sub[r][c]
                pos_chunk[lo:hi] = c
                pos_rank[lo:hi] = r
                pos_off[lo:hi] = np.arange(hi - lo)
        n2n_host = n2n64.cpu().numpy()
        self._v_chunk = np.empty(self.N, dtype=np.int64)
        self._v_rank = np.empty(self.N, dtype=np.int64)
        self._v_off = np.empty(self.N, dtype=np.int64)
        self._v_chunk[n2n_host] = pos_chunk
        self._v_rank[n2n_host] = pos_rank
        self._v_off[n2n_host] = pos_off
        self._dev = dev
        self._unperm = {}      # number of arrays -> int64 [A * N] gather index into the flat gathered buffer

    def gathered_rows(self, A: int) -> int:
        """Rows of the flat gathered buffer for `A` arrays: sum over chunks of world * A * pad."""
        return sum(self.world * A * p for p in self.pad)

    def chunk_offset(self, A: int, c: int) -> int:
        return sum(self.world * A * p for p in self.pad[:c])

    def unpermute_index(self, A: int):
        """int64 [A * N]: entry a * N + v is the row of the flat gathered buffer holding array a of voxel v."""
        import torch
        if A not in self._unperm:
            pad = np.asarray(self.pad, dtype=np.int64)
            base = np.asarray([self.chunk_offset(A, c) for c in range(self.chunks)], dtype=np.int64)
            p = pad[self._v_chunk]
            first = base[self._v_chunk] + self._v_rank * A * p + self._v_off
            idx = np.concatenate([first + a * p for a in range(A)])
            self._unperm[A] = torch.from_numpy(idx).to(self._dev)
        return self._unperm[A]


_PLAN_CACHE = {}


def get_plan(w_sizes, w2n, n2n, world: int, rank: int, chunks: int = 1) -> ShardPlan:
    """The ShardPlan of this window set, built on first use and kept while the window tensors live
    (keyed by the identity and version of ``w_sizes`` / ``n2n``, like the int32 index cache of the
    attention Function)."""
    key = (id(w_sizes), w_sizes._version, id(n2n), n2n._version, world, rank, chunks)
    hit = _PLAN_CACHE.get(key)
    if hit is not None and hit[0]() is w_sizes and hit[1]() is n2n:
        return hit[2]
    plan = ShardPlan(w_sizes, w2n, n2n, world, rank, chunks)
    if len(_PLAN_CACHE) > 16:
        _PLAN_CACHE.clear()
    _PLAN_CACHE[key] = (weakref.ref(w_sizes), weakref.ref(n2n), plan)
    return plan


def gather_rows(srcs: Sequence, idx, out):
    """out[a][i] = srcs[a][idx[i]] for up to four [rows, C] arrays sharing one int64 index list
    (`out`: [A, len(idx), C], contiguous).  On CUDA tensors one launch of the library's row-gather
    kernel (torch's index_select reaches a tenth of the memory bandwidth on 160-byte rows); on CPU
    tensors (the gloo tests) torch."""
    import torch
    if not out.is_cuda:
        for a, x in enumerate(srcs):
            torch.index_select(x, 0, idx, out=out[a])
        return out
    import ctypes
    from . import _lib
    A, n, C = out.shape
    row_bytes = C * out.element_size()
    for x in srcs:
        if not x.is_contiguous() or x.dtype != out.dtype or x.shape[1] != C:
            raise ValueError("gather_rows: sources must be contiguous [rows, C] arrays of the output's dtype")
    ptrs = (ctypes.c_void_p * A)(*[x.data_ptr() for x in srcs])
    with torch.cuda.device(out.device):
        rc = _lib.lib.s3d_gather_rows(ctypes.cast(ptrs, ctypes.c_void_p), A, idx.data_ptr(), n, row_bytes,
                                      out.data_ptr(), n * row_bytes, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "s3d_gather_rows")
    return out


class RowExchange:
    """The in-flight exchange of one step: packs chunk after chunk, one collective per chunk
    (asynchronous, so it overlaps whatever the caller launches next), one un-permute at the end."""

    def __init__(self, plan: ShardPlan, A: int, C: int, dtype, group=None):
        import torch
        self.plan, self.A, self.C, self.group = plan, A, C, group
        self.flat = torch.empty((plan.gathered_rows(A), C), dtype=dtype, device=plan._dev)
        self.piece = [torch.empty((A, plan.pad[c], C), dtype=dtype, device=plan._dev) for c in range(plan.chunks)]
        self.works = []

    def send_chunk(self, c: int, arrays: Sequence):
        """arrays: `A` tensors [N, C] whose rows of this rank's chunk c are valid."""
        import torch
        import torch.distributed as dist
        plan = self.plan
        if len(arrays) != self.A:
            raise ValueError("wrong number of arrays")
        gather_rows([x.reshape(plan.N, self.C) for x in arrays], plan.gather_idx[c], self.piece[c])
        rows = plan.world * self.A * plan.pad[c]
        off = plan.chunk_offset(self.A, c)
        dst = self.flat[off:off + rows]
        if plan.world == 1:
            dst.copy_(self.piece[c].reshape(rows, self.C))
            return
        self.works.append(dist.all_gather_into_tensor(dst.reshape(-1), self.piece[c].reshape(-1),
                                                      group=self.group, async_op=True))

    def finish(self):
        """-> `A` tensors [N, C] in voxel order, identical on every rank."""
        import torch
        for w in self.works:
            w.wait()
        self.works = []
        full = torch.empty((1, self.A * self.plan.N, self.C), dtype=self.flat.dtype, device=self.flat.device)
        gather_rows([self.flat], self.plan.unpermute_index(self.A), full)
        return [full[0, a * self.plan.N:(a + 1) * self.plan.N] for a in range(self.A)]


def exchange_rows(plan: ShardPlan, arrays: Sequence, group=None):
    """All ranks end with the full per-voxel arrays: rank r contributes the rows of its windows.
    One packed buffer, one all-gather per chunk of the plan, one un-permute."""
    C = int(np.prod(arrays[0].shape[1:]))
    ex = RowExchange(plan, len(arrays), C, arrays[0].dtype, group)
    for c in range(plan.chunks):
        ex.send_chunk(c, arrays)
    return [x.reshape(arrays[0].shape) for x in ex.finish()]


def sharded_attention_step(q, k, v, tq, tk, tv, sizes, w_sizes, w2n, n2n, n_coords, dout, group=None,
                           chunks: int = 2, plan: Optional[ShardPlan] = None):
    """Forward + backward of the cRSE window attention on ONE window set split over the ranks of
    `group`.  Every rank holds the inputs of (at least) its own voxels in full-size arrays, runs its
    window range through the C-ABI kernels chunk by chunk, and the rows of out, dq, dk, dv are
    exchanged packed: the all-gather of chunk c runs while the kernels of chunk c+1 do.  The table
    gradients are summed over chunks and ranks.  -> out, dq, dk, dv [N,H,hd] and (dtq, dtk, dtv),
    identical on every rank."""
    import torch
    import torch.distributed as dist
    from .sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    if plan is None:
        plan = get_plan(w_sizes, w2n, n2n, world, rank, chunks)
    N, H, hd = q.shape
    C = H * hd
    ex = RowExchange(plan, 4, C, q.dtype, group)
    out = torch.empty_like(q)
    lse = torch.empty((N, H), dtype=torch.float32, device=q.device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    tg = None
    for c in range(plan.chunks):
        ws_c, w2n_c = plan.w_sizes_chunk[c], plan.w2n_chunk[c]
        attn_forward_raw(q, k, v, tq, tk, tv, sizes, ws_c, w2n_c, n2n, n_coords, out=out, lse=lse)
        g = attn_backward_raw(q, k, v, tq, tk, tv, sizes, ws_c, w2n_c, n2n, n_coords, out, lse, dout,
                              dq=dq, dk=dk, dv=dv)
        tg = list(g[3:6]) if tg is None else [a + b for a, b in zip(tg, g[3:6])]
        ex.send_chunk(c, (out, dq, dk, dv))
    tg = allreduce_table_grads(tuple(tg), group)
    o_f, dq_f, dk_f, dv_f = (x.view(N, H, hd) for x in ex.finish())
    return o_f, dq_f, dk_f, dv_f, tg


def sharded_attention(q, k, v, tq, tk, tv, sizes, w_sizes, w2n, n2n, n_coords, dout=None, group=None):
    """cRSE window attention on ONE window set split over the ranks of `group` (see
    ``sharded_attention_step``).  Forward only when `dout` is None -> out [N,H,hd]; otherwise
    -> out, dq, dk, dv, (dtq, dtk, dtv).  Identical on every rank; no host synchronisation after the
    first call on a window set."""
    import torch
    import torch.distributed as dist
    from .sparse_dl.attn.attn_coff import attn_forward_raw
    if dout is not None:
        return sharded_attention_step(q, k, v, tq, tk, tv, sizes, w_sizes, w2n, n2n, n_coords, dout, group)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    plan = get_plan(w_sizes, w2n, n2n, world, rank, 1)
    out, _ = attn_forward_raw(q, k, v, tq, tk, tv, sizes, plan.w_sizes_chunk[0], plan.w2n_chunk[0], n2n, n_coords)
    return exchange_rows(plan, [out], group)[0]


# ---- KNN over several GPUs ---------------------------------------------------------------------------

def shard_queries(n_query: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous, equal query ranges [(begin, end)] per rank (queries are independent; a range may
    span several scenes)."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    per = -(-n_query // world_size) if n_query else 0
    return [(min(r * per, n_query), min((r + 1) * per, n_query)) for r in range(world_size)]


def local_query_offsets(query_offset, begin: int, end: int):
    """The cumulative per-scene END offsets of the queries [begin, end) taken alone: scenes that lie
    before the range end at 0, scenes after it at end - begin, so that the kernel's scene search
    (first scene whose end is above the query number, Swin3D/src/knn/knn_cuda_kernel.cu:170-173) finds
    the same scene for a query as in the full problem.  Works on numpy arrays and torch tensors."""
    return (query_offset - begin).clip(0, end - begin)


def sharded_knn(K: int, src_xyz, query_xyz, src_offset, query_offset, group=None, knn_fn=None):
    """KNN of all queries with the query list split over the ranks of `group` in equal contiguous
    ranges; every rank holds the source points (50 k x 12 B per scene in the stress test) and its
    slice of the queries is enough.  The [Nq_r, K] index and squared-distance blocks are all-gathered
    (padded to equal size).  -> (idx int32 [Nq,K], d2 float32 [Nq,K]) on every rank, bit for bit the
    single-GPU result.  `knn_fn(K, src, query, src_offset, query_offset) -> (idx, d2)` defaults to
    the library's kernel; the CPU tests pass the oracle."""
    import torch
    import torch.distributed as dist
    if knn_fn is None:
        from .sparse_dl.knn.knn import knn_raw as knn_fn
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    Nq = query_xyz.shape[0]
    ranges = shard_queries(Nq, world)
    a, b = ranges[rank]
    qo_l = local_query_offsets(query_offset, a, b)
    idx_l, d2_l = knn_fn(K, src_xyz, query_xyz[a:b].contiguous(), src_offset, qo_l)
    if world == 1:
        return idx_l, d2_l
    pad = max(hi - lo for lo, hi in ranges)
    # one packed exchange: indices and distance bits side by side as int32 [pad, 2K]
    piece = torch.zeros((pad, 2 * K), dtype=torch.int32, device=idx_l.device)
    piece[:b - a, :K] = idx_l
    piece[:b - a, K:] = d2_l.view(torch.int32)
    full = torch.empty((world, pad, 2 * K), dtype=torch.int32, device=idx_l.device)
    dist.all_gather_into_tensor(full.view(-1), piece.view(-1), group=group)
    rows = torch.cat([full[r, :hi - lo] for r, (lo, hi) in enumerate(ranges)])
    return rows[:, :K].contiguous(), rows[:, K:].contiguous().view(torch.float32)
