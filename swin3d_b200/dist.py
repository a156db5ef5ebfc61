"""Running the path on several GPUs (one process per GPU).

Windows are independent work units, scenes are independent, KNN queries are independent.  When every
rank owns whole scenes (data-parallel training) the only collective is the sum of the three
table-gradient arrays, which are ordinary parameters.  The other case, ONE window set split over the
ranks, is what this module does:

* ``shard_windows`` cuts the window list into contiguous ranges of equal cost;
* ``ShardPlan`` holds everything about one (window set, world size, rank) that does not change
  between calls -- ranges, the rank's slice of the window arrays, the gather index of its rows and
  the scatter index of the rows it receives.  Building it reads the window sizes on the host once;
  it is cached per window set, so a step does no host synchronisation;
* ``RowExchange`` / ``exchange_rows`` work IN PLACE: the kernels write a rank's rows in voxel order;
  per chunk the rows are packed by one row-gather launch, exchanged by one asynchronous
  ``all_gather_into_tensor`` (equal, padded shards) and the other ranks' rows are put in place by one
  row-scatter launch on a side stream;
* ``sharded_attention_step`` runs forward + backward of the rank's windows in chunks; `out` leaves
  right after the forward of a chunk (it travels while the backward runs), `dq`, `dk`, `dv` after
  the backward, so only the gradients of the last chunk are exposed; the table gradients are summed.

* ``PeerResults`` / ``sharded_attention_step_p2p`` are the second way to exchange the rows: the
  result arrays of all ranks are mapped into every process (CUDA IPC) and the attention kernels store
  each row they produce to all of them (plain peer stores); nothing is packed, gathered or
  scattered, and the only collective is the all-reduce of the table gradients.

The collectives are NCCL's (gloo on CPU); peer memory is only ever written by this library's own
kernels with plain stores -- no peer loads, no bulk-copy engine and no library kernel touch it.
"""
import weakref
from typing import List, Optional, Sequence, Tuple

import numpy as np

TILE = 32   # voxels per tile of the attention kernels
ITEM_COST = 10000   # cost of a 32 x 32 tile pair in units of one attention pair (see ``window_cost``)


def window_cost(w_sizes) -> np.ndarray:
    """Cost model of a window for the attention kernels: a part per 32 x 32 tile pair (the table
    projections, histogram products and barriers of a tile pair do not depend on how full it is) plus
    a part per attention pair.  Measured on the benchmark batch, ranges cut by the tile-pair count
    alone are the best balanced (the kernels' own split over their blocks uses it too); the pair
    count only breaks ties."""
    w = np.asarray(w_sizes, dtype=np.int64)
    nt = (w + TILE - 1) // TILE
    return nt * nt * ITEM_COST + w * w


def shard_windows(w_sizes, world_size: int, cost=None, weights=None) -> List[Tuple[int, int]]:
    """Cuts the window list into `world_size` contiguous ranges of near-equal cost (default: the
    number of attention pairs, sum of w^2; pass ``window_cost(w_sizes)`` for the kernels' cost
    model), or of cost shares proportional to `weights`.  -> [(first_window, end_window)] per rank;
    ranges are disjoint, ordered and cover every window; a rank may get an empty range when there
    are fewer windows than ranks."""
    w = np.asarray(w_sizes, dtype=np.int64)
    W = len(w)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    c = (w * w) if cost is None else np.asarray(cost, dtype=np.int64)
    if len(c) != W:
        raise ValueError("one cost per window is required")
    csum = np.cumsum(c)
    total = int(csum[-1]) if W else 0
    if weights is None:
        share = np.arange(world_size + 1) / world_size
    else:
        wt = np.asarray(weights, dtype=np.float64)
        if len(wt) != world_size or (wt <= 0).any():
            raise ValueError("one positive weight per range is required")
        share = np.concatenate([[0.0], np.cumsum(wt) / wt.sum()])
    cuts = [0]
    for r in range(1, world_size):
        target = total * share[r]
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
    further cut into `chunks` sub-ranges of equal cost -- or, when `chunks` is a sequence of weights,
    of costs in those proportions: a small last chunk leaves little exchange exposed after the last
    kernel (chunk c of every rank is exchanged together).
    For chunk c: ``chunk_windows[c]`` = this rank's (first, end) windows, ``pad[c]`` = rows of the
    largest shard of that chunk over the ranks, ``gather_idx[c]`` = int64 [pad[c]] voxel rows of this
    rank's shard in sorted order (padded with row 0), ``scatter_index(c)`` = where the rows of the
    gathered block of chunk c (laid out [rank][array][pad]) belong.
    """

    def __init__(self, w_sizes, w2n, n2n, world: int, rank: int, chunks=1):
        import torch
        chunk_weights = None
        if not isinstance(chunks, int):          # a sequence of relative chunk costs, e.g. (3, 2, 1)
            chunk_weights = tuple(float(x) for x in chunks)
            chunks = len(chunk_weights)
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
            cuts = shard_windows(ws[a:b], chunks, cost[a:b], chunk_weights)
            sub.append([(a + x, a + y) + shard_voxel_range(ws, w2, a + x, a + y) for x, y in cuts])
        self.pad = [max(8, -(-max(sub[r][c][3] - sub[r][c][2] for r in range(world)) // 8) * 8)
                    for c in range(chunks)]
        self.chunk_windows = [(sub[rank][c][0], sub[rank][c][1]) for c in range(chunks)]
        self.chunk_rows = [(sub[rank][c][2], sub[rank][c][3]) for c in range(chunks)]
        self.w_sizes_chunk = [w_sizes[a:b].contiguous() for a, b in self.chunk_windows]
        self.w2n_chunk = [w2n[a:b].contiguous() for a, b in self.chunk_windows]
        # the forward runs one kernel for windows of at most TILE voxels and one for larger ones, and each
        # walks the whole list it is given: with the sizes on the host anyway, hand each kernel its own list
        self.fwd_classes = []
        for a, b in self.chunk_windows:
            small = np.nonzero(ws[a:b] <= TILE)[0] + a
            large = np.nonzero(ws[a:b] > TILE)[0] + a
            lists = []
            for cls, sel in ((1, small), (2, large)):
                if len(sel):
                    ix = torch.from_numpy(sel).to(dev)
                    lists.append((cls, w_sizes[ix].contiguous(), w2n[ix].contiguous()))
            self.fwd_classes.append(lists)
        self.gather_idx = []
        for c in range(chunks):
            lo, hi = self.chunk_rows[c]
            idx = torch.zeros(self.pad[c], dtype=torch.int64, device=dev)
            idx[:hi - lo] = n2n64[lo:hi]
            self.gather_idx.append(idx)
        self._sub = sub
        self._n2n_host = n2n64.cpu().numpy()
        self._dev = dev
        self._scatter = {}     # chunk -> int64 [world * pad] scatter index of the gathered block

    def scatter_index(self, c: int):
        """int64 [world * pad[c]]: the voxel row of entry (rank, offset) of chunk c's gathered block,
        -1 for padding and for this rank's own rows (its kernels wrote them in place)."""
        import torch
        if c not in self._scatter:
            idx = np.full((self.world, self.pad[c]), -1, dtype=np.int64)
            for r in range(self.world):
                if r != self.rank:
                    _, _, lo, hi = self._sub[r][c]
                    idx[r, :hi - lo] = self._n2n_host[lo:hi]
            self._scatter[c] = torch.from_numpy(idx.reshape(-1)).to(self._dev)
        return self._scatter[c]


_PLAN_CACHE = {}


def get_plan(w_sizes, w2n, n2n, world: int, rank: int, chunks=1) -> ShardPlan:
    """The ShardPlan of this window set, built on first use and kept while the window tensors live
    (keyed by the identity and version of ``w_sizes`` / ``n2n``, like the int32 index cache of the
    attention Function)."""
    if not isinstance(chunks, int):
        chunks = tuple(float(x) for x in chunks)
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


def scatter_rows(src, idx, block_rows: int, dsts: Sequence):
    """dsts[a][idx[i]] = src[i // block_rows][a][i % block_rows] for every i with idx[i] >= 0
    (`src`: [blocks, A, block_rows, C] contiguous, `dsts`: A contiguous [rows, C] arrays).  One launch
    of the library's row-scatter kernel on CUDA tensors, torch on CPU tensors (the gloo tests)."""
    import torch
    nb, A, br, C = src.shape
    if br != block_rows or len(dsts) != A:
        raise ValueError("scatter_rows: shape mismatch")
    if not src.is_cuda:
        keep = idx >= 0
        rows = idx[keep]
        for a, d in enumerate(dsts):
            d[rows] = src[:, a].reshape(nb * br, C)[keep]
        return
    import ctypes
    from . import _lib
    row_bytes = C * src.element_size()
    for d in dsts:
        if not d.is_contiguous() or d.dtype != src.dtype or d.shape[1] != C:
            raise ValueError("scatter_rows: destinations must be contiguous [rows, C] arrays of the source's dtype")
    ptrs = (ctypes.c_void_p * A)(*[d.data_ptr() for d in dsts])
    with torch.cuda.device(src.device):
        rc = _lib.lib.s3d_scatter_rows(src.data_ptr(), A, idx.data_ptr(), nb * br, row_bytes, br,
                                       A * br * row_bytes, br * row_bytes, ctypes.cast(ptrs, ctypes.c_void_p),
                                       torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "s3d_scatter_rows")


_SIDE_STREAMS = {}


def _side_stream(device):
    import torch
    key = (device.type, device.index)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device, priority=-1)    # ahead of the attention kernels
    return _SIDE_STREAMS[key]


def forward_of_chunk(plan: "ShardPlan", c: int, q, k, v, tq, tk, tv, sizes, n2n, n_coords, out, lse, mirrors=None):
    """The forward of this rank's windows of chunk c, one call per size class of the plan (every call
    writes only the rows of its own windows into `out` / `lse`)."""
    from .sparse_dl.attn.attn_coff import attn_forward_raw
    for cls, ws_c, w2n_c in plan.fwd_classes[c]:
        attn_forward_raw(q, k, v, tq, tk, tv, sizes, ws_c, w2n_c, n2n, n_coords, out=out, lse=lse,
                         mirrors=mirrors, window_class=cls)


class RowExchange:
    """The in-flight exchange of `A` per-voxel arrays of one step, IN PLACE: a rank's kernels wrote the
    rows of its own windows into ``arrays``; ``send_chunk(c)`` packs those of chunk c (one row-gather
    launch), starts one asynchronous all-gather and queues, on a side stream behind it, the one
    row-scatter launch that puts the other ranks' rows of that chunk into ``arrays``.  Pack and
    collective are ordered behind the kernels already launched; everything the caller launches
    afterwards overlaps them.  ``finish()`` makes the current stream wait for the scatters."""

    def __init__(self, plan: ShardPlan, arrays: Sequence, group=None):
        import torch
        self.plan, self.group = plan, group
        self.A = len(arrays)
        self.C = int(np.prod(arrays[0].shape[1:]))
        self.arrays = list(arrays)
        self.rows = [x.reshape(plan.N, self.C) for x in arrays]
        for x, r in zip(arrays, self.rows):
            if r.data_ptr() != x.data_ptr():
                raise ValueError("RowExchange: arrays must be contiguous")
        self.cuda = arrays[0].is_cuda
        self.side = _side_stream(arrays[0].device) if (self.cuda and plan.world > 1) else None
        self.keep = []         # buffers in flight

    def send_chunk(self, c: int):
        import torch
        import torch.distributed as dist
        plan = self.plan
        if plan.world == 1:
            return
        dtype, dev = self.rows[0].dtype, self.rows[0].device
        piece = torch.empty((self.A, plan.pad[c], self.C), dtype=dtype, device=dev)
        block = torch.empty((plan.world, self.A, plan.pad[c], self.C), dtype=dtype, device=dev)
        gather_rows(self.rows, plan.gather_idx[c], piece)
        work = dist.all_gather_into_tensor(block.reshape(-1), piece.reshape(-1), group=self.group, async_op=True)
        self.keep.append((piece, block))
        if self.cuda:
            with torch.cuda.stream(self.side):
                work.wait()                                   # the side stream waits, the host does not
                scatter_rows(block, plan.scatter_index(c), plan.pad[c], self.rows)
        else:
            work.wait()
            scatter_rows(block, plan.scatter_index(c), plan.pad[c], self.rows)

    def finish(self):
        """-> the `A` arrays, complete and identical on every rank."""
        import torch
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        self.keep = []          # freed in current-stream order, i.e. behind the scatters
        return self.arrays


def exchange_rows(plan: ShardPlan, arrays: Sequence, group=None):
    """All ranks end with the full per-voxel arrays: rank r contributes the rows of its windows, the
    other rows of ``arrays`` are overwritten in place.  One packed all-gather and one scatter per chunk
    of the plan."""
    ex = RowExchange(plan, arrays, group)
    for c in range(plan.chunks):
        ex.send_chunk(c)
    return ex.finish()


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
    out = torch.empty_like(q)
    lse = torch.empty((N, H), dtype=torch.float32, device=q.device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    ex_out = RowExchange(plan, (out,), group)          # leaves right after the forward of a chunk
    ex_grad = RowExchange(plan, (dq, dk, dv), group)
    tg = None
    for c in range(plan.chunks):
        ws_c, w2n_c = plan.w_sizes_chunk[c], plan.w2n_chunk[c]
        forward_of_chunk(plan, c, q, k, v, tq, tk, tv, sizes, n2n, n_coords, out, lse)
        ex_out.send_chunk(c)
        g = attn_backward_raw(q, k, v, tq, tk, tv, sizes, ws_c, w2n_c, n2n, n_coords, out, lse, dout,
                              dq=dq, dk=dk, dv=dv)
        tg = list(g[3:6]) if tg is None else [a + b for a, b in zip(tg, g[3:6])]
        ex_grad.send_chunk(c)
    tg = allreduce_table_grads(tuple(tg), group)
    ex_out.finish()
    ex_grad.finish()
    return out, dq, dk, dv, tg


class _RawCudaArray:
    """A device allocation presented through the CUDA array interface, for torch.as_tensor."""

    def __init__(self, ptr: int, shape, dtype):
        import torch
        typestr = {torch.float16: "<f2", torch.float32: "<f4"}[dtype]
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


class PeerResults:
    """Result arrays (out, dq, dk, dv) of the split step that every rank of the group can store into:
    each rank allocates `sets` x 4 arrays of `shape`, exports the allocation as a CUDA IPC handle, and
    maps the allocations of the other ranks (same node) into its own address space.  The attention
    kernels then write every row they produce to the same row on all ranks (plain peer stores over
    NVLink, from inside the kernels), so the exchange needs no packing, collective or scatter pass and
    overlaps the computation row by row.  Two sets alternate between steps: a rank may still be
    reading the results of step i while its peers already write those of step i + 1.
    At most 8 ranks (7 mirrors per kernel launch)."""

    def __init__(self, shape, dtype, device, group=None, sets: int = 2):
        import ctypes
        import torch
        import torch.distributed as dist
        from . import _lib
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if self.world - 1 > 7:
            raise ValueError("PeerResults: at most 8 ranks")
        self.sets = sets
        full = (sets, 4) + tuple(int(x) for x in shape)
        itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = int(np.prod(full)) * itemsize
        self._ptr, self.own, self._opened = None, None, []
        self.base = [None] * self.world            # address of rank r's block in this process
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        error = None
        # Every rank goes through the same collectives whatever fails locally, so that a rank without
        # CUDA IPC (or out of memory) makes ALL ranks raise instead of leaving the others waiting.
        try:
            with torch.cuda.device(device):
                # an allocation of its own (not a piece of the caching allocator's segments): exportable
                _lib.check(_lib.lib.s3d_peer_alloc(nbytes, ctypes.byref(ptr), ctypes.cast(handle, ctypes.c_void_p)),
                           "s3d_peer_alloc")
                self._ptr = ptr.value
                self.own = torch.as_tensor(_RawCudaArray(self._ptr, full, dtype), device=device)
            if self.own.data_ptr() != self._ptr:
                raise RuntimeError("PeerResults: the tensor does not alias the exported allocation")
            self.array_bytes = self.own[0, 0].numel() * itemsize
            self.base[self.rank] = self._ptr
        except Exception as e:          # noqa: BLE001 - reported to every rank below
            error = f"rank {self.rank}: {e}"
        if self.world > 1:
            infos = [None] * self.world
            dist.all_gather_object(infos, None if error else handle.raw, group=group)
            if error is None and all(h is not None for h in infos):
                try:
                    with torch.cuda.device(device):
                        for r, h in enumerate(infos):
                            if r == self.rank:
                                continue
                            buf = ctypes.create_string_buffer(h, 64)
                            peer = ctypes.c_void_p()
                            _lib.check(_lib.lib.s3d_ipc_open(ctypes.cast(buf, ctypes.c_void_p), ctypes.byref(peer)),
                                       "s3d_ipc_open")
                            self._opened.append(peer.value)
                            self.base[r] = peer.value
                except Exception as e:      # noqa: BLE001
                    error = f"rank {self.rank}: {e}"
            elif error is None:
                error = "another rank could not allocate or export its arrays"
            errors = [None] * self.world
            dist.all_gather_object(errors, error, group=group)
            error = next((e for e in errors if e), None)
        if error:
            self._release()
            raise RuntimeError(f"PeerResults unavailable ({error})")

    def _release(self):
        from . import _lib
        for p in self._opened:
            _lib.lib.s3d_ipc_close(p)
        self._opened = []
        if self._ptr is not None:
            self.own = None
            _lib.lib.s3d_peer_free(self._ptr)
            self._ptr = None

    def arrays(self, s: int):
        """This rank's (out, dq, dk, dv) of set s."""
        return tuple(self.own[s % self.sets, a] for a in range(4))

    def mirrors(self, s: int, a: int):
        """Addresses of array a of set s on the other ranks."""
        off = ((s % self.sets) * 4 + a) * self.array_bytes
        return [self.base[r] + off for r in range(self.world) if r != self.rank]

    def close(self):
        """Unmaps the other ranks' arrays and frees this rank's (collective: no rank may still be
        writing; the tensors handed out by ``arrays`` must not be used afterwards)."""
        import torch
        import torch.distributed as dist
        from . import _lib
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        for p in self._opened:
            _lib.lib.s3d_ipc_close(p)
        self._opened = []
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody maps this rank's allocation any more
        self._release()


def sharded_attention_step_p2p(q, k, v, tq, tk, tv, sizes, w_sizes, w2n, n2n, n_coords, dout, peers: PeerResults,
                               step: int, group=None, plan: Optional[ShardPlan] = None, consumed=None):
    """Forward + backward of ONE window set split over the ranks, the rows exchanged by the kernels
    themselves: every rank runs its window range once (no chunks) and its kernels store each result
    row to all ranks (``PeerResults``).  The all-reduce of the table gradients that follows on the
    same stream also orders the ranks: when it has completed, every rank's kernels have finished and
    all rows of set ``step % sets`` are in place.  `consumed`: a CUDA event after which this rank no
    longer reads the results of the previous step; the stream waits for it before the all-reduce
    (a rank that passes the all-reduce of step i lets its peers overwrite, in step i + 1, the set that
    held step i - 1).  Readers on the calling stream need no event.
    -> out, dq, dk, dv [N,H,hd] (views of this rank's arrays of that set) and (dtq, dtk, dtv)."""
    import torch
    import torch.distributed as dist
    from .sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    if plan is None:
        plan = get_plan(w_sizes, w2n, n2n, world, rank, 1)
    if plan.chunks != 1:
        raise ValueError("the peer-store step runs a rank's windows in one piece")
    N, H, hd = q.shape
    out, dq, dk, dv = peers.arrays(step)
    if out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("PeerResults were allocated for another shape or dtype")
    lse = torch.empty((N, H), dtype=torch.float32, device=q.device)
    ws_c, w2n_c = plan.w_sizes_chunk[0], plan.w2n_chunk[0]
    forward_of_chunk(plan, 0, q, k, v, tq, tk, tv, sizes, n2n, n_coords, out, lse, mirrors=peers.mirrors(step, 0))
    g = attn_backward_raw(q, k, v, tq, tk, tv, sizes, ws_c, w2n_c, n2n, n_coords, out, lse, dout,
                          dq=dq, dk=dk, dv=dv,
                          mirrors=(peers.mirrors(step, 1), peers.mirrors(step, 2), peers.mirrors(step, 3)))
    if consumed is not None:
        torch.cuda.current_stream().wait_event(consumed)
    tg = allreduce_table_grads(tuple(g[3:6]), group)
    return out, dq, dk, dv, tg


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
    if all(hi - lo == b - a for lo, hi in ranges):
        # equal ranges: the blocks are gathered straight into the results, no packing and no copy
        idx = torch.empty((Nq, K), dtype=idx_l.dtype, device=idx_l.device)
        d2 = torch.empty((Nq, K), dtype=d2_l.dtype, device=d2_l.device)
        w1 = dist.all_gather_into_tensor(idx.view(-1), idx_l.contiguous().view(-1), group=group, async_op=True)
        dist.all_gather_into_tensor(d2.view(-1), d2_l.contiguous().view(-1), group=group)
        w1.wait()
        return idx, d2
    pad = max(hi - lo for lo, hi in ranges)
    # unequal ranges, one packed exchange: indices and distance bits side by side as int32 [pad, 2K]
    piece = torch.zeros((pad, 2 * K), dtype=torch.int32, device=idx_l.device)
    piece[:b - a, :K] = idx_l
    piece[:b - a, K:] = d2_l.view(torch.int32)
    full = torch.empty((world, pad, 2 * K), dtype=torch.int32, device=idx_l.device)
    dist.all_gather_into_tensor(full.view(-1), piece.view(-1), group=group)
    rows = torch.cat([full[r, :hi - lo] for r, (lo, hi) in enumerate(ranges)])
    return rows[:, :K].contiguous(), rows[:, K:].contiguous().view(torch.float32)
