"""GPU: the re-created pybind modules ``attn_cuda`` / ``knn_cuda`` under the reference's legacy call
protocol.  The reference's own ``attn_coff.py`` cannot be imported on a GPU box, so its forward and
backward sequences (microsoft/Swin3D, Swin3D/sparse_dl/attn/attn_coff.py:160-232: dtype policy, max ->
raw,sum -> raw/sum; raw = norm*sum -> exp-sum grads -> indirect backward) are restated here call by
call, on top of the shim, and compared with this repository's fused Function and with the recorded
result of the reference module (tests/golden/window_attention_reference.npz)."""
import os

import numpy as np
import pytest

from tests.helpers import rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "window_attention_reference.npz")


class _LegacyFunction(torch.autograd.Function):
    """attn_coff.py:160-232 over a module with the four pybind entry points."""

    @staticmethod
    def forward(ctx, q, k, v, tq, tk, tv, table_offsets, indices, precision, attn_module):
        ctx.precision, ctx.attn_module = precision, attn_module
        if torch.is_autocast_enabled() and precision != "HALF_NONE":
            c_dtype = torch.get_autocast_dtype("cuda")
        else:
            c_dtype = torch.float32
        c_feats = [t.type(c_dtype) for t in (q, k, v)]
        c_tabs = [t.type(c_dtype) for t in (tq, tk, tv)]
        rmax = attn_module.cal_max_coffs(c_feats, c_tabs, table_offsets, indices, 2, 3)
        raw, sums = attn_module.self_attn_forward(c_feats, c_tabs, rmax, table_offsets, indices, 2, 3)
        norm = raw / sums
        ctx.save_for_backward(sums, rmax, norm, q, k, v, tq, tk, tv, table_offsets, *indices)
        return norm

    @staticmethod
    def backward(ctx, grad):
        m = ctx.attn_module
        sums, rmax, norm = ctx.saved_tensors[:3]
        feats, tabs = ctx.saved_tensors[3:6], ctx.saved_tensors[6:9]
        table_offsets, indices = ctx.saved_tensors[9], list(ctx.saved_tensors[10:])
        if ctx.precision == "HALF_ALL":
            c_dtype = grad.dtype
        else:
            c_dtype = torch.float32
            norm, sums, grad = norm.type(torch.float32), sums.type(torch.float32), grad.type(torch.float32)
        c_feats = [t.type(c_dtype) for t in feats]
        c_tabs = [t.type(c_dtype) for t in tabs]
        raw = norm * sums
        esg = m.cal_exp_sum_grads(grad, raw, sums, c_feats[-1], tabs[2])
        g = m.self_attn_indir_backward(grad, esg, raw, sums, rmax, *c_feats, *c_tabs, table_offsets, indices, 2, 3)
        return (*g, None, None, None, None)


def _problem(seed=5, H=4, hd=8, crse="XYZ_RGB_NORM"):
    from oracle import oracle as O
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=seed, n_voxels=1500, grid=26, H=H, hd=hd, crse=crse)
    x_off, y_off, m2w, w, w2n64, w2m = O.window_offsets(p.w_sizes)
    idx = [dev(m2w), dev(w), dev(w2m), dev(w2n64), dev(p.n2n.astype(np.int64)), dev(p.n_crse)]
    offs = torch.IntTensor(p.sizes).cuda()
    return p, idx, offs


@pytest.mark.parametrize("precision,autocast", [("HALF_NONE", False), ("HALF_ALL", True), ("HALF_FORWARD", True)])
def test_legacy_protocol_over_the_shim_equals_the_fused_function(precision, autocast):
    from swin3d_b200.sparse_dl import attn_cuda
    from swin3d_b200.sparse_dl.attn.attn_coff import (IndexMode, PosEmb, PrecisionMode, SelfAttnAIOFunction,
                                                     TableDims)
    from tests.gpu_helpers import dev
    p, idx, offs = _problem()
    leaves = lambda: [dev(a).requires_grad_() for a in (p.q, p.k, p.v, p.tq, p.tk, p.tv)]
    up = dev(p.g)
    a, b = leaves(), leaves()
    with torch.autocast("cuda", dtype=torch.float16, enabled=autocast):
        y_ref = SelfAttnAIOFunction.apply(*a, offs, idx, PosEmb.SEPARATE, TableDims.D0, IndexMode.INDIRECT,
                                          PrecisionMode[precision])
        y = _LegacyFunction.apply(*b, offs, idx, precision, attn_cuda)
    assert y.dtype == y_ref.dtype and torch.equal(y, y_ref)       # the same launch behind both
    y_ref.backward(up.to(y_ref.dtype))
    y.backward(up.to(y.dtype))
    for x, r in zip(b, a):
        assert x.grad.dtype == r.grad.dtype and x.grad.shape == r.grad.shape
        # same kernels on the same values; table gradients are sums of atomics in any order
        tol = 1e-5 if x.dim() == 3 else 1e-3
        assert rel_err(x.grad.float().cpu().numpy(), r.grad.float().cpu().numpy()) < tol


def test_forward_runs_once_for_the_two_forward_calls(monkeypatch):
    from swin3d_b200.sparse_dl import attn_cuda
    from tests.gpu_helpers import dev
    p, idx, offs = _problem(seed=6)
    calls = []
    real = attn_cuda.attn_forward_raw
    monkeypatch.setattr(attn_cuda, "attn_forward_raw", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    feats = [dev(x).half() for x in (p.q, p.k, p.v)]
    tabs = [dev(x).half() for x in (p.tq, p.tk, p.tv)]
    rmax = attn_cuda.cal_max_coffs(feats, tabs, offs, idx, 2, 3)
    raw, sums = attn_cuda.self_attn_forward(feats, tabs, rmax, offs, idx, 2, 3)
    assert len(calls) == 1 and rmax.dtype == torch.float32 and rmax.shape == (p.N, p.H, 1)
    assert raw.dtype == torch.float16 and sums.shape == (p.N, p.H, 1)
    raw2, _ = attn_cuda.self_attn_forward(feats, tabs, rmax, offs, idx, 2, 3)      # no pending result: computes
    assert len(calls) == 2 and torch.equal(raw2, raw)
    with pytest.raises(NotImplementedError):
        attn_cuda.cal_max_coffs(feats, tabs, offs, idx, 1, 3)


def test_recorded_reference_call_through_the_legacy_protocol():
    from swin3d_b200.sparse_dl import attn_cuda
    from oracle import oracle as O
    d = np.load(FIX)
    c = {k[len("rgb_m0."):]: d[k] for k in d.files if k.startswith("rgb_m0.")}
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    m2w = O.window_offsets(c["call.idx.w_sizes"])[2]
    idx = [cu(m2w), cu(c["call.idx.w_sizes"]), cu(c["call.idx.w2m"]), cu(c["call.idx.w2n"]), cu(c["call.idx.n2n"]),
           cu(c["call.idx.n_crse"])]
    out = _LegacyFunction.apply(cu(c["call.q"]), cu(c["call.k"]), cu(c["call.v"]), cu(c["call.tq"]), cu(c["call.tk"]),
                                cu(c["call.tv"]), cu(c["call.table_offsets"]), idx, "HALF_NONE", attn_cuda)
    assert rel_err(out.cpu().numpy(), c["call.result"]) < 1e-4


def test_knn_cuda_shim_fills_the_callers_outputs():
    from swin3d_b200 import synthetic as S
    from swin3d_b200.sparse_dl import knn_cuda
    from swin3d_b200.sparse_dl.knn.knn import knn_raw
    from tests.gpu_helpers import dev
    src, qry = S.make_knn_scene(3, 900, 700)
    so, qo = dev(np.array([700], dtype=np.int32)), dev(np.array([900], dtype=np.int32))
    ridx = torch.cuda.IntTensor(900, 5).zero_()                   # as knn.py:14-15 allocates them
    rdist = torch.cuda.FloatTensor(900, 5).zero_() + 1e10
    knn_cuda.knn_cuda(5, dev(src), dev(qry), so, qo, ridx, rdist)
    idx, d2 = knn_raw(5, dev(src), dev(qry), so, qo)
    assert torch.equal(ridx, idx) and torch.equal(rdist, d2)
    with pytest.raises(ValueError):
        knn_cuda.knn_cuda(5, dev(src), dev(qry), so, qo, ridx.long(), rdist)
