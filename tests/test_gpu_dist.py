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
