"""GPU: the packed row exchange of the window split (single process, world size 1) and the library's
row-gather kernel.  The multi-rank logic itself is covered on CPU by the gloo tests of test_dist.py."""
import numpy as np
import pytest

from tests import helpers  # noqa: F401

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_gather_rows_kernel_matches_index_select():
    from swin3d_b200.dist import gather_rows
    g = torch.Generator(device="cuda").manual_seed(5)
    for C, dtype in ((80, torch.float16), (160, torch.float16), (8, torch.float32)):
        srcs = [torch.randn((5000, C), device="cuda", generator=g).to(dtype) for _ in range(4)]
        idx = torch.randint(0, 5000, (7777,), device="cuda", generator=g)
        out = torch.empty((4, 7777, C), dtype=dtype, device="cuda")
        gather_rows(srcs, idx, out)
        for a in range(4):
            assert torch.equal(out[a], srcs[a].index_select(0, idx))
    src = torch.zeros((16, 80), dtype=torch.float16, device="cuda")
    out1 = torch.empty((1, 0, 80), dtype=torch.float16, device="cuda")
    gather_rows([src], idx[:0], out1)        # empty index list


@pytest.mark.parametrize("chunks", [1, 3])
def test_sharded_step_on_one_rank_equals_the_plain_calls(chunks):
    from swin3d_b200.dist import ShardPlan, sharded_attention_step
    from swin3d_b200.sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=31, n_voxels=3000, grid=30, H=4, hd=8, crse="XYZ_RGB_NORM")
    h = lambda a: dev(a).half()
    q, k, v, g = h(p.q), h(p.k), h(p.v), h(p.g)
    tabs = [h(p.tq), h(p.tk), h(p.tv)]
    ws, w2n, n2n, nc = dev(p.w_sizes), dev(p.w2n), dev(p.n2n), dev(p.n_crse)
    out, lse = attn_forward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc)
    ref = attn_backward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, out, lse, g)
    plan = ShardPlan(ws, w2n, n2n, 1, 0, chunks)
    o2, dq, dk, dv, tg = sharded_attention_step(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, g, plan=plan)
    # windows are independent and the kernels deterministic per window: bitwise equal per-voxel results
    assert torch.equal(o2, out) and torch.equal(dq, ref[0]) and torch.equal(dk, ref[1]) and torch.equal(dv, ref[2])
    for a, b in zip(tg, ref[3:6]):      # summed over chunks in a different order
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5 * float(b.abs().max()))


def test_scatter_rows_kernel_matches_indexed_assignment():
    from swin3d_b200.dist import scatter_rows
    g = torch.Generator(device="cuda").manual_seed(6)
    for C, dtype, A in ((80, torch.float16, 3), (160, torch.float16, 1), (8, torch.float32, 4)):
        blocks, br, rows = 3, 1000, 5000
        src = torch.randn((blocks, A, br, C), device="cuda", generator=g).to(dtype)
        idx = torch.randperm(rows, device="cuda", generator=g)[:blocks * br].clone()
        idx[::7] = -1                                   # padding and own rows are skipped
        dsts = [torch.full((rows, C), -3.0, dtype=dtype, device="cuda") for _ in range(A)]
        want = [d.clone() for d in dsts]
        keep = idx >= 0
        for a in range(A):
            want[a][idx[keep]] = src[:, a].reshape(blocks * br, C)[keep]
        scatter_rows(src, idx, br, dsts)
        for a in range(A):
            assert torch.equal(dsts[a], want[a])


@pytest.mark.parametrize("world,chunks", [(2, 2), (4, 3)])
def test_pack_and_scatter_of_every_rank_reassemble_the_arrays(world, chunks):
    """The exchange of `world` ranks replayed in one process: every rank packs its rows of a chunk with
    its plan's gather index, the blocks are concatenated as the all-gather would, and each rank's
    scatter index puts the other ranks' rows in place."""
    from swin3d_b200.dist import ShardPlan, gather_rows, scatter_rows
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=33, n_voxels=2500, grid=28, H=2, hd=8, crse="XYZ_RGB")
    ws, w2n, n2n = dev(p.w_sizes), dev(p.w2n), dev(p.n2n)
    N, C = p.q.shape[0], 16
    g = torch.Generator(device="cuda").manual_seed(7)
    truth = [torch.randn((N, C), device="cuda", generator=g).half() for _ in range(3)]
    plans = [ShardPlan(ws, w2n, n2n, world, r, chunks) for r in range(world)]
    mine = []
    for pl in plans:                                   # a rank only holds the rows of its own windows
        arrs = [torch.full((N, C), float("nan"), dtype=torch.float16, device="cuda") for _ in range(3)]
        for lo, hi in pl.chunk_rows:
            rows = n2n[lo:hi].long()
            for a in range(3):
                arrs[a][rows] = truth[a][rows]
        mine.append(arrs)
    for c in range(chunks):
        pad = plans[0].pad[c]
        block = torch.empty((world, 3, pad, C), dtype=torch.float16, device="cuda")
        for r, pl in enumerate(plans):
            gather_rows(mine[r], pl.gather_idx[c], block[r])
        for r, pl in enumerate(plans):
            scatter_rows(block, pl.scatter_index(c), pad, mine[r])
    for r in range(world):
        for a in range(3):
            assert torch.equal(mine[r][a], truth[a])


def _dense_block_scene():
    """A full 12^3 block (windows of up to 125 voxels: several 32-voxel tiles) and a few lonely voxels."""
    from swin3d_b200 import synthetic as S
    g = np.stack(np.meshgrid(*[np.arange(12)] * 3, indexing="ij"), -1).reshape(-1, 3)
    pts = np.concatenate([g, np.array([[40, 40, 40], [60, 3, 9], [90, 90, 90]])])
    n = len(pts)
    rng = np.random.default_rng(6)
    return S.Scene(np.concatenate([np.zeros((n, 1)), pts], 1).astype(np.int32),
                   rng.random((n, 3), dtype=np.float32) * 0.999, rng.random((n, 3), dtype=np.float32),
                   np.tile(np.array([[0, 0, 1]], dtype=np.float32), (n, 1)))


@pytest.mark.parametrize("H,hd,crse,n_vox,grid", [(4, 8, "XYZ_RGB_NORM", 3000, 30), (2, 8, "XYZ_RGB", 0, 0),
                                                  (3, 16, "XYZ", 1500, 26)])
def test_mirrored_stores_write_the_same_rows_to_every_buffer(H, hd, crse, n_vox, grid):
    """The kernels of the split step store every result row to further buffers (other GPUs' arrays in
    production; here three more buffers of this GPU): each mirror must hold exactly the rows of the
    plain call for the voxels of the processed windows and stay untouched elsewhere.  The second shape
    has windows of several 32-voxel tiles (rows written more than once by the backward)."""
    from swin3d_b200.sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    if n_vox:
        p = make_problem(seed=35, n_voxels=n_vox, grid=grid, H=H, hd=hd, crse=crse)
    else:
        p = make_problem(seed=35, H=H, hd=hd, crse=crse, scene=_dense_block_scene())
        assert p.w_sizes.max() > 64
    h = lambda a: dev(a).half()
    q, k, v, g = h(p.q), h(p.k), h(p.v), h(p.g)
    tabs = [h(p.tq), h(p.tk), h(p.tv)]
    ws, w2n, n2n, nc = dev(p.w_sizes), dev(p.w2n), dev(p.n2n), dev(p.n_crse)
    W = ws.shape[0]
    a, b = W // 3, W                                       # a window range, as a rank of a split step has
    ws_r, w2n_r = ws[a:b].contiguous(), w2n[a:b].contiguous()
    lo = int(w2n[a])
    rows = n2n[lo:].long()
    out, lse = attn_forward_raw(q, k, v, *tabs, p.sizes, ws_r, w2n_r, n2n, nc)
    ref = attn_backward_raw(q, k, v, *tabs, p.sizes, ws_r, w2n_r, n2n, nc, out, lse, g)
    fill = -7.0
    mk = lambda: [torch.full_like(q, fill) for _ in range(3)]
    m_out, m_dq, m_dk, m_dv = mk(), mk(), mk(), mk()
    out2, lse2 = attn_forward_raw(q, k, v, *tabs, p.sizes, ws_r, w2n_r, n2n, nc,
                                  mirrors=[t.data_ptr() for t in m_out])
    got = attn_backward_raw(q, k, v, *tabs, p.sizes, ws_r, w2n_r, n2n, nc, out2, lse2, g,
                            mirrors=([t.data_ptr() for t in m_dq], [t.data_ptr() for t in m_dk],
                                     [t.data_ptr() for t in m_dv]))
    torch.cuda.synchronize()
    assert torch.equal(out2[rows], out[rows])
    for x, y in zip(got[:3], ref[:3]):
        assert torch.equal(x[rows], y[rows])
    other = torch.ones(q.shape[0], dtype=torch.bool, device="cuda")
    other[rows] = False
    for mirrors, want in ((m_out, out), (m_dq, ref[0]), (m_dk, ref[1]), (m_dv, ref[2])):
        for m in mirrors:
            assert torch.equal(m[rows], want[rows])
            assert bool((m[other] == fill).all())


def _rank_p2p_step(rank, world, port, q_out):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from swin3d_b200.dist import PeerResults, sharded_attention_step_p2p
    from swin3d_b200.sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=36, n_voxels=4000, grid=40, H=4, hd=8, crse="XYZ_RGB_NORM")
    h = lambda a: dev(a).half()
    q, k, v, g = h(p.q), h(p.k), h(p.v), h(p.g)
    tabs = [h(p.tq), h(p.tk), h(p.tv)]
    ws, w2n, n2n, nc = dev(p.w_sizes), dev(p.w2n), dev(p.n2n), dev(p.n_crse)
    out, lse = attn_forward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc)
    ref = attn_backward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, out, lse, g)
    peers = PeerResults(q.shape, q.dtype, q.device)
    ok = True
    for step in range(4):                                   # both sets, each used twice
        gs = g * (1.0 + step)
        res = sharded_attention_step_p2p(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, gs, peers, step)
        torch.cuda.synchronize()
        want = attn_backward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, out, lse, gs)
        ok = ok and torch.equal(res[0], out)
        ok = ok and all(torch.equal(x, y) for x, y in zip(res[1:4], want[:3]))
        ok = ok and all(torch.allclose(x, y, rtol=1e-4, atol=1e-5 * float(y.abs().max())) for x, y in zip(res[4], want[3:6]))
    peers.close()
    q_out.put((rank, bool(ok)))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_peer_store_step_on_two_gpus_equals_the_plain_calls():
    """Two ranks, two GPUs: the kernels of each rank store its rows into both ranks' arrays; after the
    all-reduce of the table gradients every rank holds the complete out, dq, dk, dv, bit for bit the
    single-GPU result (windows are independent, the kernels deterministic per window)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    procs = [ctx.Process(target=_rank_p2p_step, args=(r, 2, port, q_out)) for r in range(2)]
    for pr in procs:
        pr.start()
    import queue
    import time
    got, deadline = {}, time.time() + 240
    while len(got) < 2 and time.time() < deadline:
        try:
            r, ok = q_out.get(timeout=2)
            got[r] = ok
        except queue.Empty:
            if any(pr.exitcode not in (None, 0) for pr in procs):      # a rank died: do not wait for the others
                break
    for pr in procs:
        pr.join(20)
        if pr.is_alive():
            pr.kill()
    assert [pr.exitcode for pr in procs] == [0, 0]
    assert got == {0: True, 1: True}


def test_peer_store_step_on_one_rank_equals_the_plain_calls():
    """World size 1 (no process group): the peer-store step allocates its arrays through the library,
    has no mirrors, and must give the plain calls' results; two steps use both array sets."""
    from swin3d_b200.dist import PeerResults, sharded_attention_step_p2p
    from swin3d_b200.sparse_dl.attn.attn_coff import attn_backward_raw, attn_forward_raw
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=37, n_voxels=2000, grid=30, H=4, hd=8, crse="XYZ_RGB_NORM")
    h = lambda a: dev(a).half()
    q, k, v, g = h(p.q), h(p.k), h(p.v), h(p.g)
    tabs = [h(p.tq), h(p.tk), h(p.tv)]
    ws, w2n, n2n, nc = dev(p.w_sizes), dev(p.w2n), dev(p.n2n), dev(p.n_crse)
    out, lse = attn_forward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc)
    ref = attn_backward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, out, lse, g)
    peers = PeerResults(q.shape, q.dtype, q.device)
    try:
        assert peers.mirrors(0, 0) == [] and peers.own.shape == (2, 4) + tuple(q.shape)
        for step in range(2):
            res = sharded_attention_step_p2p(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, g, peers, step)
            torch.cuda.synchronize()
            assert res[0].data_ptr() == peers.arrays(step)[0].data_ptr()
            assert torch.equal(res[0], out)
            for x, y in zip(res[1:4], ref[:3]):
                assert torch.equal(x, y)
            for x, y in zip(res[4], ref[3:6]):
                assert torch.allclose(x, y, rtol=1e-5, atol=1e-6 * float(y.abs().max()))
    finally:
        peers.close()
    assert peers.own is None


def test_forward_by_window_class_equals_the_mixed_call():
    """The plan hands the forward its windows in two lists (at most 32 voxels / more) with the
    matching class hint, so that neither kernel walks the other's windows: same bits as one call."""
    from swin3d_b200.dist import ShardPlan, forward_of_chunk
    from swin3d_b200.sparse_dl.attn.attn_coff import attn_forward_raw
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=38, H=4, hd=8, crse="XYZ_RGB_NORM", scene=_dense_block_scene())
    assert (p.w_sizes > 32).any() and (p.w_sizes <= 32).any()
    h = lambda a: dev(a).half()
    q, k, v = h(p.q), h(p.k), h(p.v)
    tabs = [h(p.tq), h(p.tk), h(p.tv)]
    ws, w2n, n2n, nc = dev(p.w_sizes), dev(p.w2n), dev(p.n2n), dev(p.n_crse)
    out, lse = attn_forward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc)
    plan = ShardPlan(ws, w2n, n2n, 1, 0, 1)
    assert [c for c, _, _ in plan.fwd_classes[0]] == [1, 2]
    out2 = torch.full_like(q, float("nan"))
    lse2 = torch.full((q.shape[0], p.H), float("nan"), dtype=torch.float32, device="cuda")
    forward_of_chunk(plan, 0, q, k, v, *tabs, p.sizes, n2n, nc, out2, lse2)
    torch.cuda.synchronize()
    assert torch.equal(out2, out) and torch.equal(lse2, lse)
    # a hint that is not true leaves the other class's windows untouched (documented, not an error)
    out3 = torch.full_like(q, float("nan"))
    attn_forward_raw(q, k, v, *tabs, p.sizes, ws, w2n, n2n, nc, out=out3, window_class=1)
    torch.cuda.synchronize()
    small_rows = torch.cat([n2n[int(a):int(a) + int(n)] for a, n in zip(p.w2n, p.w_sizes) if n <= 32]).long()
    assert torch.equal(out3[small_rows], out[small_rows]) and bool(torch.isnan(out3.float()).any())
