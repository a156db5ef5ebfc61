"""Shared problem builders for the tests (seeded, numpy on the host)."""
import numpy as np

from oracle import oracle as O
from swin3d_b200 import synthetic as S


class Problem:
    pass


def make_problem(seed=0, n_voxels=600, grid=24, ws=5, shift=0, quant=4, H=2, hd=8,
                 crse="XYZ_RGB", scene=None, feat_scale=1.0, round_fp16=False):
    """A single-layer attention problem: scene -> window grouping (oracle) -> q,k,v,tables."""
    rng = np.random.default_rng(seed + 1000)
    if scene is None:
        scene = S.make_planes_and_boxes(seed, n_voxels, grid)
    feats = S.signal_feats(scene, crse)
    n2n, n_coords, w_sizes, w2n = O.window_grouping(scene.coords, feats, ws, shift)
    p = Problem()
    p.scene, p.ws, p.shift, p.quant, p.H, p.hd, p.crse = scene, ws, shift, quant, H, hd, crse
    p.N = scene.coords.shape[0]
    p.n2n, p.w_sizes, p.w2n = n2n, w_sizes, w2n
    p.n_crse = S.quantise_signals(n_coords, quant)
    p.sizes = S.table_sizes(ws, quant, H, hd, crse)
    p.D = len(p.sizes)
    t = S.make_tables(seed + 7, p.sizes)
    q = (rng.standard_normal((p.N, H, hd)) * feat_scale * hd ** -0.5).astype(np.float32)
    k = (rng.standard_normal((p.N, H, hd)) * feat_scale).astype(np.float32)
    v = (rng.standard_normal((p.N, H, hd)) * feat_scale).astype(np.float32)
    g = rng.standard_normal((p.N, H, hd)).astype(np.float32)
    if round_fp16:
        q, k, v, g, t = (a.astype(np.float16).astype(np.float32) for a in (q, k, v, g, t))
    p.q, p.k, p.v, p.g = q, k, v, g
    p.tq, p.tk, p.tv = t[0].copy(), t[1].copy(), t[2].copy()
    return p


def oracle_fwd_bwd(p, dtype=np.float64):
    out, s, mx = O.attn_forward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n,
                                p.n2n, p.n_crse, dtype=dtype)
    grads = O.attn_backward(p.q, p.k, p.v, p.tq, p.tk, p.tv, p.sizes, p.w_sizes, p.w2n, p.n2n,
                            p.n_crse, out, s, mx, p.g, dtype=dtype)
    lse = mx.astype(np.float64) + np.log(s.astype(np.float64))
    return out, lse, grads


def rel_err(a, b):
    """max |a-b| / max |b|: the relative measure the tolerances of the tests refer to."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / (den if den > 0 else 1.0))


def table_row_errors(a, b, row_len, tol, floor_frac):
    """Per table ROW check of a table gradient (flat [rows * row_len]): for every row the largest
    deviation must stay below tol * max(largest reference entry of that row, floor_frac * largest
    entry of the whole table).  A gradient that landed in the wrong row (an alias row of the flat
    cRSE addressing, a rarely hit row) fails here even when it is invisible in a whole-tensor norm.
    -> list of offending rows (empty = pass)."""
    a = np.asarray(a, dtype=np.float64).reshape(-1, row_len)
    b = np.asarray(b, dtype=np.float64).reshape(-1, row_len)
    err = np.abs(a - b).max(1)
    ref = np.abs(b).max(1)
    floor = floor_frac * (ref.max() if ref.size and ref.max() > 0 else 1.0)
    bad = np.nonzero(err > tol * np.maximum(ref, floor))[0]
    return [(int(r), float(err[r]), float(ref[r])) for r in bad[:8]]
