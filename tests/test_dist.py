"""CPU: window sharding and the table-gradient all-reduce on two gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from swin3d_b200.dist import (ShardPlan, local_query_offsets, shard_queries, sharded_knn, all_gather_window_rows, allreduce_table_grads, exchange_rows,
                              shard_voxel_range, shard_windows, window_cost)
from tests.helpers import make_problem


def test_shard_windows_covers_and_balances():
    rng = np.random.default_rng(0)
    w = rng.integers(1, 126, size=5000)
    for world in (1, 2, 3, 8):
        parts = shard_windows(w, world)
        assert parts[0][0] == 0 and parts[-1][1] == len(w)
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        cost = np.array([(w[a:b].astype(np.int64) ** 2).sum() for a, b in parts])
        assert cost.sum() == (w.astype(np.int64) ** 2).sum()
        assert cost.max() <= cost.sum() / world + 125 ** 2
    assert shard_windows([], 4) == [(0, 0)] * 4
    assert shard_windows([3], 2) in ([(0, 1), (1, 1)], [(0, 0), (0, 1)])
    w2n = np.cumsum(w) - w
    a, b = shard_windows(w, 2)[1]
    lo, hi = shard_voxel_range(w, w2n, a, b)
    assert lo == w[:a].sum() and hi == w.sum()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = make_problem(seed=71, n_voxels=500, grid=20, H=2, hd=8, crse="XYZ_RGB")
    out, s, mx = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n, p.n_crse)
    a, b = shard_windows(p.w_sizes, world)[rank]
    # this rank's windows only: same arrays, window list cut to [a, b)
    g = O.attn_backward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes[a:b], p.w2n[a:b], p.n2n,
                        p.n_crse, out, s, mx, p.g)
    dq, dk, dv = (torch.from_numpy(x) for x in g[:3])
    tg = allreduce_table_grads(tuple(torch.from_numpy(x) for x in g[3:]))
    for t in (dq, dk, dv):          # disjoint rows per rank: a sum reassembles the full gradient
        dist.all_reduce(t)
    if rank == 0:
        q.put([x.numpy() for x in (dq, dk, dv, *tg)])
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_window_sharding_reproduces_single_rank_gradients():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    got = q.get(timeout=240)
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    p = make_problem(seed=71, n_voxels=500, grid=20, H=2, hd=8, crse="XYZ_RGB")
    out, s, mx = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n, p.n_crse)
    ref = O.attn_backward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n, p.n_crse,
                          out, s, mx, p.g)
    for a, b in zip(got, ref):
        assert np.allclose(a, b, rtol=1e-12, atol=1e-14)


def _rank_gather(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = make_problem(seed=72, n_voxels=700, grid=22, H=2, hd=8, crse="XYZ_RGB")
    parts = shard_windows(p.w_sizes, world)
    ranges = [shard_voxel_range(p.w_sizes, p.w2n, a, b) for a, b in parts]
    a, b = parts[rank]
    lo, hi = ranges[rank]
    # forward of this rank's windows only; rows of other voxels stay whatever the buffer held
    out, s, mx = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes[a:b], p.w2n[a:b],
                                p.n2n, p.n_crse)
    n2n = torch.from_numpy(p.n2n)
    mine = n2n[lo:hi].long()
    out_t = torch.from_numpy(out)
    out_t[torch.ones(out_t.shape[0], dtype=torch.bool).index_fill_(0, mine, False)] = float("nan")
    full = all_gather_window_rows(out_t[mine], ranges, n2n)
    q.put((rank, full.numpy()))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_all_gather_of_window_shards_reassembles_the_output(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_gather, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    got = dict(q.get(timeout=240) for _ in range(world))
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    p = make_problem(seed=72, n_voxels=700, grid=22, H=2, hd=8, crse="XYZ_RGB")
    ref, _, _ = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n, p.n_crse)
    for r in range(world):                  # every rank ends with the full, identical array
        assert np.array_equal(got[r], ref)


def _rank_plan_exchange(rank, world, port, chunks, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = make_problem(seed=73, n_voxels=800, grid=22, H=2, hd=8, crse="XYZ_RGB")
    ws, w2n, n2n = torch.from_numpy(p.w_sizes), torch.from_numpy(p.w2n), torch.from_numpy(p.n2n)
    plan = ShardPlan(ws, w2n, n2n, world, rank, chunks)
    out = torch.full((p.q.shape[0], p.H, p.hd), float("nan"), dtype=torch.float64)
    twice = out.clone()
    for c in range(chunks):                     # this rank's windows only, chunk by chunk
        a, b = plan.chunk_windows[c]
        o, _, _ = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes[a:b], p.w2n[a:b],
                                 p.n2n, p.n_crse)
        lo, hi = plan.chunk_rows[c]
        rows = n2n[lo:hi].long()
        out[rows] = torch.from_numpy(o)[rows].double()
        twice[rows] = 2 * out[rows]
    full, full2 = exchange_rows(plan, [out, twice])
    q.put((rank, full.numpy(), full2.numpy()))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 2), (3, 2)])
def test_packed_exchange_of_a_shard_plan_reassembles_every_array(world, chunks):
    """ShardPlan + exchange_rows: one packed all-gather and one scatter per chunk, in place; every rank ends
    with the full arrays although it only ever computed (and holds NaN outside) its own windows."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_plan_exchange, args=(r, world, port, chunks, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    p = make_problem(seed=73, n_voxels=800, grid=22, H=2, hd=8, crse="XYZ_RGB")
    ref, _, _ = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n, p.n_crse)
    for _, full, full2 in got:
        assert np.array_equal(full, ref.astype(np.float64))
        assert np.array_equal(full2, 2 * ref.astype(np.float64))


def test_shard_plan_ranges_follow_the_kernel_cost_model():
    rng = np.random.default_rng(3)
    w = rng.integers(1, 126, size=4000)
    w2n = np.cumsum(w) - w
    n2n = rng.permutation(int(w.sum()))
    plans = [ShardPlan(torch.from_numpy(w), torch.from_numpy(w2n), torch.from_numpy(n2n), 4, r, 2) for r in range(4)]
    cost = window_cost(w)
    shares = [sum(int(cost[a:b].sum()) for a, b in pl.chunk_windows) for pl in plans]
    assert sum(shares) == int(cost.sum())
    assert max(shares) <= cost.sum() / 4 + 2 * cost.max()
    # chunk c of every rank has the same padded size, and the chunks of a rank tile its range
    assert all(pl.pad == plans[0].pad for pl in plans)
    for r, pl in enumerate(plans):
        assert pl.chunk_windows[0][0] == pl.parts[r][0] and pl.chunk_windows[-1][1] == pl.parts[r][1]
        assert pl.chunk_windows[0][1] == pl.chunk_windows[1][0]


def _oracle_knn(K, src, qry, so, qo):
    idx, d2 = O.knn(K, src.numpy(), qry.numpy(), so.numpy(), qo.numpy())
    return torch.from_numpy(idx), torch.from_numpy(d2)


def _rank_knn(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from swin3d_b200 import synthetic as S
    scenes = [S.make_knn_scene(40 + s, 300 + 37 * s, 150 + 11 * s) for s in range(3)]
    src = torch.from_numpy(np.concatenate([a for a, _ in scenes]))
    qry = torch.from_numpy(np.concatenate([b for _, b in scenes]))
    so = torch.tensor(np.cumsum([a.shape[0] for a, _ in scenes]), dtype=torch.int32)
    qo = torch.tensor(np.cumsum([b.shape[0] for _, b in scenes]), dtype=torch.int32)
    idx, d2 = sharded_knn(5, src, qry, so, qo, knn_fn=_oracle_knn)
    q.put((rank, idx.numpy(), d2.numpy()))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_query_sharded_knn_equals_the_single_rank_result_bit_for_bit(world):
    """Query ranges that cut through scenes: the clipped per-scene offsets make every rank search the
    right scene; indices and distance bits after the all-gather equal the unsplit run."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_knn, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    from swin3d_b200 import synthetic as S
    scenes = [S.make_knn_scene(40 + s, 300 + 37 * s, 150 + 11 * s) for s in range(3)]
    src = np.concatenate([a for a, _ in scenes])
    qry = np.concatenate([b for _, b in scenes])
    so = np.cumsum([a.shape[0] for a, _ in scenes]).astype(np.int32)
    qo = np.cumsum([b.shape[0] for _, b in scenes]).astype(np.int32)
    ref_idx, ref_d2 = O.knn(5, src, qry, so, qo)
    for _, idx, d2 in got:
        assert np.array_equal(idx, ref_idx)
        assert np.array_equal(d2.view(np.int32), ref_d2.view(np.int32))


def test_query_ranges_and_local_offsets():
    assert shard_queries(10, 3) == [(0, 4), (4, 8), (8, 10)]
    assert shard_queries(0, 2) == [(0, 0), (0, 0)]
    qo = np.array([5, 9, 20])
    assert local_query_offsets(qo, 4, 8).tolist() == [1, 4, 4]       # scene 0: one query, scene 1: three
    assert local_query_offsets(qo, 9, 20).tolist() == [0, 0, 11]


def test_all_gather_window_rows_single_process_unpermutes():
    n2n = torch.tensor([2, 0, 3, 1])
    rows = torch.arange(8.0).view(4, 2)
    full = all_gather_window_rows(rows, [(0, 4)], n2n)
    assert torch.equal(full[n2n], rows)
    with pytest.raises(ValueError):
        all_gather_window_rows(rows[:3], [(0, 4)], n2n)


def test_compat_aliases_resolve_reference_import_paths():
    import importlib
    import sys
    import swin3d_b200.compat as compat
    saved = {k: v for k, v in sys.modules.items() if k == "Swin3D" or k.startswith("Swin3D.")}
    for k in saved:
        del sys.modules[k]
    try:
        compat.install_as_swin3d()
        coff = importlib.import_module("Swin3D.sparse_dl.attn.attn_coff")
        knn = importlib.import_module("Swin3D.sparse_dl.knn")
        from swin3d_b200.sparse_dl.attn.attn_coff import SelfAttnAIOFunction
        from swin3d_b200.sparse_dl.knn import KNN
        assert coff.SelfAttnAIOFunction is SelfAttnAIOFunction and knn.KNN is KNN
        assert coff.PrecisionMode.HALF_NONE.value == 3 and coff.IndexMode.INDIRECT.value == 2
    finally:
        for k in [k for k in sys.modules if k == "Swin3D" or k.startswith("Swin3D.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_weighted_chunks_follow_the_given_proportions():
    rng = np.random.default_rng(4)
    w = rng.integers(1, 100, size=6000)
    w2n = np.cumsum(w) - w
    n2n = rng.permutation(int(w.sum()))
    pl = ShardPlan(torch.from_numpy(w), torch.from_numpy(w2n), torch.from_numpy(n2n), 2, 1, (3, 2, 1))
    assert pl.chunks == 3
    cost = window_cost(w)
    shares = np.array([cost[a:b].sum() for a, b in pl.chunk_windows], dtype=np.float64)
    assert np.allclose(shares / shares.sum(), [0.5, 1 / 3, 1 / 6], atol=0.01)
    assert pl.chunk_windows[0][0] == pl.parts[1][0] and pl.chunk_windows[-1][1] == pl.parts[1][1]
    with pytest.raises(ValueError):
        shard_windows(w, 3, cost, weights=(1, 0, 1))
