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
