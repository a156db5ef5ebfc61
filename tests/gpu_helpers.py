"""Helpers for the GPU parity tests: run the CUDA library through its C-ABI wrappers."""
import numpy as np
import torch

from swin3d_b200.sparse_dl.attn import attn_coff as C


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def cuda_fwd_bwd(p, dtype=torch.float32):
    """-> out, lse, (dq, dk, dv, dtq, dtk, dtv) as float64 numpy arrays."""
    q, k, v, g = (dev(a, dtype) for a in (p.q, p.k, p.v, p.g))
    tq, tk, tv = (dev(a, dtype) for a in (p.tq, p.tk, p.tv))
    ws, w2n, n2n = dev(p.w_sizes), dev(p.w2n), dev(p.n2n)
    nc = dev(p.n_crse)
    out, lse = C.attn_forward_raw(q, k, v, tq, tk, tv, list(p.sizes), ws, w2n, n2n, nc)
    grads = C.attn_backward_raw(q, k, v, tq, tk, tv, list(p.sizes), ws, w2n, n2n, nc, out, lse, g)
    torch.cuda.synchronize()
    f = lambda t: t.double().cpu().numpy()
    return f(out), f(lse), tuple(f(x) for x in grads)
