"""Python face of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

* attention forward / backward, cRSE indices, KNN: ctypes calls into liboracle_swin3d.so
  (oracle/swin3d_oracle.c, a C restatement of the reference CUDA kernels' arithmetic);
* window grouping and offset building: numpy restatements of
  microsoft/Swin3D Swin3D/modules/swin3d_layers.py:713-822 and :76-150.

Only tests/, the smoke check and the benchmark's CPU-baseline legs may import this module.
Parity pin: see the header of swin3d_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_swin3d.so")


def build(force: bool = False) -> str:
    src = [os.path.join(_HERE, f) for f in ("swin3d_oracle.c", "attn_oracle_impl.inc")]
    if (force or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(s) for s in src)):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle_swin3d.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def _prep(q, k, v, tq, tk, tv, dtype):
    c = lambda a: np.ascontiguousarray(a, dtype=dtype)
    return c(q), c(k), c(v), c(tq), c(tk), c(tv)


def _idx(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def attn_forward(q, k, v, tq, tk, tv, table_sizes, w_sizes, w2n, n2n, n_coords,
                 dtype=np.float64, nthreads: int = 0):
    """-> (out_norm [N,H,hd], sum [N,H], max [N,H] float32), computed in `dtype`."""
    q, k, v, tq, tk, tv = _prep(q, k, v, tq, tk, tv, dtype)
    N, H, hd = q.shape
    ts, ws, w2, n2 = _idx(table_sizes), _idx(w_sizes), _idx(w2n), _idx(n2n)
    nc = np.ascontiguousarray(n_coords, dtype=np.float32)
    out = np.zeros_like(q)
    s = np.zeros((N, H), dtype=dtype)
    mx = np.zeros((N, H), dtype=np.float32)
    fn = lib().orc_attn_fwd_f64 if dtype == np.float64 else lib().orc_attn_fwd_f32
    rc = fn(_p(q), _p(k), _p(v), _p(tq), _p(tk), _p(tv), _p(ts), ctypes.c_int(len(ts)),
            _p(ws), _p(w2), _p(n2), _p(nc), ctypes.c_int64(N), ctypes.c_int64(len(ws)),
            ctypes.c_int(H), ctypes.c_int(hd), _p(out), _p(s), _p(mx), ctypes.c_int(nthreads))
    if rc != 0:
        raise ValueError("oracle: unsupported shape")
    return out, s, mx


def attn_backward(q, k, v, tq, tk, tv, table_sizes, w_sizes, w2n, n2n, n_coords,
                  out_norm, s, mx, gout, dtype=np.float64, nthreads: int = 0):
    """-> (dq, dk, dv, dtq, dtk, dtv) computed in `dtype`."""
    q, k, v, tq, tk, tv = _prep(q, k, v, tq, tk, tv, dtype)
    N, H, hd = q.shape
    ts, ws, w2, n2 = _idx(table_sizes), _idx(w_sizes), _idx(w2n), _idx(n2n)
    nc = np.ascontiguousarray(n_coords, dtype=np.float32)
    on = np.ascontiguousarray(out_norm, dtype=dtype)
    ss = np.ascontiguousarray(s, dtype=dtype)
    mm = np.ascontiguousarray(mx, dtype=np.float32)
    g = np.ascontiguousarray(gout, dtype=dtype)
    dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
    dtq, dtk, dtv = np.zeros_like(tq), np.zeros_like(tq), np.zeros_like(tq)
    fn = lib().orc_attn_bwd_f64 if dtype == np.float64 else lib().orc_attn_bwd_f32
    rc = fn(_p(q), _p(k), _p(v), _p(tq), _p(tk), _p(tv), _p(ts), ctypes.c_int(len(ts)),
            _p(ws), _p(w2), _p(n2), _p(nc), ctypes.c_int64(N), ctypes.c_int64(len(ws)),
            ctypes.c_int(H), ctypes.c_int(hd), _p(on), _p(ss), _p(mm), _p(g),
            _p(dq), _p(dk), _p(dv), _p(dtq), _p(dtk), _p(dtv), ctypes.c_int(nthreads))
    if rc != 0:
        raise ValueError("oracle: unsupported shape")
    return dq, dk, dv, dtq, dtk, dtv


def crse_indices(n_coords, table_sizes, H, hd, first_pos, n):
    """idx[q,k,d] int32 of one window (attn_utils.cuh:437-453)."""
    nc = np.ascontiguousarray(n_coords, dtype=np.float32)
    ts = _idx(table_sizes)
    D = nc.shape[1]
    out = np.zeros((n, n, D), dtype=np.int32)
    lib().orc_crse_indices(_p(nc), ctypes.c_int(D), _p(ts), ctypes.c_int(H * hd),
                           ctypes.c_int32(first_pos), ctypes.c_int32(n), _p(out))
    return out


def knn(K, src, query, src_offset, query_offset, fma_mode: int = 2, nthreads: int = 0):
    """Literal max-heap KNN -> (idx int32 [Nq,K], SQUARED dist float32 [Nq,K])."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    query = np.ascontiguousarray(query, dtype=np.float32)
    so, qo = _idx(src_offset), _idx(query_offset)
    Nq = query.shape[0]
    idx = np.zeros((Nq, K), dtype=np.int32)
    d2 = np.zeros((Nq, K), dtype=np.float32)
    rc = lib().orc_knn(ctypes.c_int(K), _p(src), _p(query), _p(so), _p(qo), ctypes.c_int(len(so)),
                       ctypes.c_int64(Nq), ctypes.c_int(fma_mode), _p(idx), _p(d2),
                       ctypes.c_int(nthreads))
    if rc != 0:
        raise ValueError("oracle: K out of range")
    return idx, d2


# ---- window grouping -----------------------------------------------------------------------------

def window_grouping(coords, feats, window_size: int, shift: int = 0, stride: int = 1):
    """numpy restatement of get_map_pair / get_window_mapping / get_index01
    (swin3d_layers.py:713-822) with the window order fixed to lexicographic (batch, wx, wy, wz).

    window = floor((c + shift*stride) / (ws*stride))   (MinkowskiEngine pooling, kernel = stride = ws)
    cell   = (c + shift*stride - window*ws*stride) / stride, cell_id = cx*ws^2 + cy*ws + cz
    voxels sorted by (window, cell_id)                  (torch.sort(in_map), :753)
    n_coords = [cell_xyz + local_xyz, other signals] in sorted order   (:800-804)
    -> n2n int32[N], n_coords float32[N,F], w_sizes int32[W], w2n int32[W]
    """
    coords = np.asarray(coords, dtype=np.int64)
    feats = np.asarray(feats, dtype=np.float32)
    ws = window_size
    shifted = coords[:, 1:] + shift * stride
    win = np.floor_divide(shifted, ws * stride)
    cell = (shifted - win * ws * stride) // stride
    cell_id = (cell[:, 0] * ws + cell[:, 1]) * ws + cell[:, 2]
    order = np.lexsort((cell_id, win[:, 2], win[:, 1], win[:, 0], coords[:, 0]))
    wkey = np.concatenate([coords[:, :1], win], 1)[order]
    head = np.ones(len(order), dtype=bool)
    if len(order) > 1:
        head[1:] = np.any(wkey[1:] != wkey[:-1], axis=1)
    w2n = np.flatnonzero(head).astype(np.int32)
    w_sizes = np.diff(np.append(w2n, len(order))).astype(np.int32)
    n_coords = feats[order].copy()
    n_coords[:, 0:3] = cell[order].astype(np.float32) + feats[order, 0:3]
    return order.astype(np.int32), n_coords, w_sizes, w2n


def window_offsets(w_sizes):
    """numpy restatement of sparse_self_attention(protocol='v2') (swin3d_layers.py:76-150):
    -> (x_offset, y_offset, m2w_indices, w_sizes, w2n_indices, w2m_indices), all int64."""
    w = np.asarray(w_sizes, dtype=np.int64)
    w2 = w * w
    w2n = np.cumsum(w) - w
    w2m = np.cumsum(w2) - w2
    M = int(w2.sum())
    m2w = np.repeat(np.arange(len(w), dtype=np.int64), w2)
    m_off = np.arange(M, dtype=np.int64) - w2m[m2w]
    x_off = w2n[m2w] + m_off // w[m2w]
    y_off = w2n[m2w] + m_off % w[m2w]
    return x_off, y_off, m2w, w, w2n, w2m


# ---- consumers of the KNN result -----------------------------------------------------------------

def knn_interpolate(idx, dist, src_feat):
    """numpy restatement of knn_linear_interpolation after its KNN.apply call
    (swin3d_layers.py:64-72), operation by operation: weights in fp32; per neighbour one rounded
    product (fp32) and one add whose result is rounded to the feature dtype (the reference's
    in-place ``query_feat += ...`` on a tensor of src_feat's dtype)."""
    idx = np.asarray(idx, dtype=np.int64)
    dist = np.asarray(dist, dtype=np.float32)
    src_feat = np.asarray(src_feat)
    dt = src_feat.dtype
    weight = (np.float32(1.0) / (dist + np.float32(1e-8))).astype(np.float32)
    norm = np.zeros((dist.shape[0], 1), dtype=np.float32)
    for i in range(dist.shape[1]):                      # sequential sum over the K neighbours
        norm[:, 0] = norm[:, 0] + weight[:, i]
    weight = (weight / norm).astype(np.float32)
    out = np.zeros((idx.shape[0], src_feat.shape[1]), dtype=dt)
    for i in range(idx.shape[1]):
        prod = src_feat[idx[:, i]].astype(np.float32) * weight[:, i:i + 1]
        out = (out.astype(np.float32) + prod).astype(dt)
    return out


def knn_interpolate_weights(dist):
    dist = np.asarray(dist, dtype=np.float32)
    weight = (np.float32(1.0) / (dist + np.float32(1e-8))).astype(np.float32)
    norm = np.zeros((dist.shape[0], 1), dtype=np.float32)
    for i in range(dist.shape[1]):
        norm[:, 0] = norm[:, 0] + weight[:, i]
    return (weight / norm).astype(np.float32)


def knn_interpolate_bwd(idx, dist, dout, n_src):
    """Gradient w.r.t. src_feat of knn_interpolate (autograd of the indexing + multiply,
    swin3d_layers.py:70-72), accumulated in fp64 and returned as float32 [n_src, C]."""
    idx = np.asarray(idx, dtype=np.int64)
    w = knn_interpolate_weights(dist).astype(np.float64)
    dout = np.asarray(dout).astype(np.float64)
    dsrc = np.zeros((n_src, dout.shape[1]), dtype=np.float64)
    for i in range(idx.shape[1]):
        np.add.at(dsrc, idx[:, i], dout * w[:, i:i + 1])
    return dsrc.astype(np.float32)


def knn_maxpool(idx, g):
    """max over the K neighbours of g[idx] per channel = MaxPool1d(K) over the gathered rows
    (swin3d_layers.py:302-309); -> (out, arg = source row of the first maximum)."""
    idx = np.asarray(idx, dtype=np.int64)
    g = np.asarray(g)
    gathered = g[idx]                                    # [Nq, K, C]
    first = np.argmax(gathered.astype(np.float32), axis=1)      # first maximum along K
    out = np.take_along_axis(gathered, first[:, None, :], axis=1)[:, 0, :]
    arg = np.take_along_axis(np.broadcast_to(idx[:, :, None], gathered.shape), first[:, None, :], axis=1)[:, 0, :]
    return out, arg.astype(np.int32)


def knn_maxpool_bwd(arg, dout, n_src):
    arg = np.asarray(arg, dtype=np.int64)
    dout = np.asarray(dout).astype(np.float64)
    dg = np.zeros((n_src, dout.shape[1]), dtype=np.float64)
    cols = np.broadcast_to(np.arange(dout.shape[1])[None, :], dout.shape)
    np.add.at(dg, (arg, cols), dout)
    return dg.astype(np.float32)
