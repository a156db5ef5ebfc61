"""CPU: the C oracle against an independent closed-form definition differentiated by torch.autograd.

The closed form (per window, per head):
    s_qk = q.k + q.sum_n Tq[n, idx_n] + k.sum_n Tk[n, idx_n];  out_q = softmax_k(s) (v_k + sum_n Tv[n, idx_n])
with idx_n the cRSE index of microsoft/Swin3D Swin3D/src/attn/attn_utils.cuh:437-453.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import make_problem, oracle_fwd_bwd, rel_err


def torch_closed_form(p):
    dt = torch.float64
    q, k, v = (torch.tensor(a, dtype=dt, requires_grad=True) for a in (p.q, p.k, p.v))
    tq, tk, tv = (torch.tensor(a, dtype=dt, requires_grad=True) for a in (p.tq, p.tk, p.tv))
    H, hd, D = p.H, p.hd, p.D
    HC = H * hd
    L = [s // HC for s in p.sizes]
    rowbase = np.concatenate([[0], np.cumsum(L)[:-1]])
    out = torch.zeros_like(q)
    T = [t.view(-1, H, hd) for t in (tq, tk, tv)]
    nc = p.n_crse
    for w in range(len(p.w_sizes)):
        n, base = int(p.w_sizes[w]), int(p.w2n[w])
        rows_v = torch.tensor(p.n2n[base:base + n].astype(np.int64))
        c = nc[base:base + n]                                    # [n, D] float32
        rel = (c[:, None, :] - c[None, :, :]).astype(np.float32)  # q - k
        idx = np.empty((n, n, D), dtype=np.int64)
        for d in range(D):
            r = rel[:, :, d] + np.float32(L[d] // 2)
            r = np.minimum(np.maximum(np.float32(0), r), np.float32(L[d]))
            i = r.astype(np.int64)
            if d == D - 1:
                i = np.minimum(i, L[d] - 1)
            idx[:, :, d] = i + rowbase[d]
        idx_t = torch.tensor(idx)
        bq = T[0][idx_t].sum(2)   # [n, n, H, hd]
        bk = T[1][idx_t].sum(2)
        bv = T[2][idx_t].sum(2)
        qw, kw, vw = q[rows_v], k[rows_v], v[rows_v]
        s = torch.einsum("qhc,khc->qkh", qw, kw) + torch.einsum("qhc,qkhc->qkh", qw, bq) + \
            torch.einsum("khc,qkhc->qkh", kw, bk)
        a = torch.softmax(s, dim=1)
        o = torch.einsum("qkh,qkhc->qhc", a, vw[None] + bv)
        out = out.index_add(0, rows_v, o)
    g = torch.tensor(p.g, dtype=dt)
    out.backward(g)
    return out.detach().numpy(), [x.grad.numpy() for x in (q, k, v, tq, tk, tv)]


@pytest.mark.parametrize("crse,hd,shift", [("XYZ", 8, 0), ("XYZ_RGB", 8, 2), ("XYZ_RGB_NORM", 16, 0)])
def test_oracle_matches_closed_form_fp64(crse, hd, shift):
    p = make_problem(seed=3, n_voxels=400, grid=20, H=2, hd=hd, crse=crse, shift=shift)
    out, lse, grads = oracle_fwd_bwd(p, np.float64)
    ref_out, ref_grads = torch_closed_form(p)
    assert rel_err(out, ref_out) < 1e-12
    for a, b in zip(grads, ref_grads):
        assert rel_err(a, b) < 1e-11


def test_oracle_fp32_close_to_fp64():
    p = make_problem(seed=4, n_voxels=400, grid=20, H=2, hd=8, crse="XYZ_RGB")
    o64, _, g64 = oracle_fwd_bwd(p, np.float64)
    o32, _, g32 = oracle_fwd_bwd(p, np.float32)
    assert rel_err(o32, o64) < 1e-5
    for a, b in zip(g32, g64):
        assert rel_err(a, b) < 1e-4


def test_crse_index_quirks():
    """idx == L is reachable (difference of exactly +L/2 after quantisation) and truncation is
    toward zero; the last dimension clamps to L-1."""
    sizes = [40 * 16, 32 * 16, 32 * 16]
    nc = np.array([[0.0, 16.0, 16.0], [3.99, 0.0, 0.0], [19.5, 8.0, -16.0]], dtype=np.float32)
    idx = O.crse_indices(nc, sizes, 2, 8, 0, 3)
    assert idx[0, 1, 1] == 32          # +16 + 16 = 32 == L survives the clamp
    assert idx[0, 1, 2] == 31          # ... but not in the last dimension
    assert idx[1, 0, 1] == 0           # -16 + 16 = 0
    assert idx[0, 1, 0] == 16          # -3.99 + 20 = 16.01 -> 16
    assert idx[1, 0, 0] == 23          # 3.99 + 20 = 23.99 -> 23 (truncation)
    assert idx[0, 2, 0] == 0           # -19.5 + 20 = 0.5 -> 0
    assert idx[2, 0, 2] == 0           # -32 + 16 clamps at 0
