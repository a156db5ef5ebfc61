"""The reference's pybind module ``Swin3D.sparse_dl.attn_cuda`` re-created over libswin3d_b200.so, for
callers that keep the reference's own ``attn_coff.py`` byte for byte (microsoft/Swin3D,
Swin3D/src/attn/attn_api.cpp:20-24; the four names ``SelfAttnAIOFunction`` calls,
Swin3D/sparse_dl/attn/attn_coff.py:180-184 and :220-225):

    cal_max_coffs(qkv_feats, qkv_tables, table_sizes, s_indices, indice_mode, pos_mode) -> T[N,H,1] f32
    self_attn_forward(qkv_feats, qkv_tables, max_coffs, table_sizes, s_indices, indice_mode, pos_mode)
        -> [raw[N,H,hd], sum[N,H,1]]
    cal_exp_sum_grads(normed_out_grads, unnormed_out_feats, exp_sum_feats, value_feats, value_table) -> T[N,H]
    self_attn_indir_backward(normed_out_grads, exp_sum_grads, unnormed_out_feats, exp_sum_feats, coff_rmax,
                             q, k, v, Tq, Tk, Tv, table_sizes, s_indices, indice_mode, pos_bias_method)
        -> [dq, dk, dv, dTq, dTk, dTv]

The library's forward is ONE fused launch that returns the normalised output and
``lse = max + log(sum)`` per (voxel, head).  The legacy protocol wants (max, raw, sum) with the caller
computing ``raw / sum`` (attn_coff.py:184) and handing ``raw = norm * sum``, ``sum`` and ``max`` back to
the backward (:219-225).  Any triple with ``raw / sum = out`` and ``max + log(sum) = lse`` serves that
protocol, so this module returns ``max := lse``, ``sum := 1``, ``raw := out``: ``cal_max_coffs`` runs
the fused forward and keeps its result for the ``self_attn_forward`` call that follows on the same
inputs (one launch per forward, not two); the backward rebuilds ``out`` and ``lse`` from what it is
given, whatever triple that is.  ``cal_exp_sum_grads`` has nothing left to do (the fused backward
computes that term itself) and returns zeros of the right shape.

Only ``indice_mode == 2`` (IndexMode.INDIRECT) with ``pos_mode == 3`` (PosEmb.SEPARATE) is implemented,
the combination ``WindowAttention`` passes (Swin3D/modules/swin3d_layers.py:554-567).
"""
import weakref
from typing import List

import torch

from .attn.attn_coff import _as_int32, _table_sizes_host, attn_backward_raw, attn_forward_raw

_INDIRECT, _SEPARATE = 2, 3

# result of the last cal_max_coffs, for the self_attn_forward that follows it
_last = {}


def _check_modes(indice_mode: int, pos_mode: int) -> None:
    if int(indice_mode) != _INDIRECT or int(pos_mode) != _SEPARATE:
        raise NotImplementedError("attn_cuda over libswin3d_b200: only indice_mode 2 (INDIRECT) with "
                                  "pos_mode 3 (SEPARATE) is implemented")


def _unpack_indices(s_indices: List[torch.Tensor]):
    if len(s_indices) != 6:
        raise ValueError("s_indices of the indirect mode: [m2w, w_elems, w2m, w2n, n2n, n_coords]")
    _, w_elems, _, w2n, n2n, n_coords = s_indices
    return _as_int32(w_elems), _as_int32(w2n), _as_int32(n2n), n_coords.to(torch.float32).contiguous()


def _sizes(table_sizes, qkv_tables, q):
    return _table_sizes_host(table_sizes, qkv_tables[0].numel(), q.shape[1], q.shape[2])


def _key(qkv_feats, qkv_tables, s_indices):
    return tuple((t.data_ptr(), t._version, tuple(t.shape), t.dtype) for t in list(qkv_feats) + list(qkv_tables)) + \
        tuple((t.data_ptr(), t._version) for t in s_indices)


def _fused_forward(qkv_feats, qkv_tables, table_sizes, s_indices):
    q, k, v = (t.contiguous() for t in qkv_feats)
    tabs = [t.to(q.dtype).contiguous().view(-1) for t in qkv_tables]
    w_sizes, w2n, n2n, n_coords = _unpack_indices(s_indices)
    return attn_forward_raw(q, k, v, *tabs, _sizes(table_sizes, qkv_tables, q), w_sizes, w2n, n2n, n_coords)


def cal_max_coffs(qkv_feats, qkv_tables, table_sizes, s_indices, indice_mode, pos_mode):
    """-> float32 [N,H,1]: the log-sum-exp of every (voxel, head) in the role of the row maximum."""
    _check_modes(indice_mode, pos_mode)
    out, lse = _fused_forward(qkv_feats, qkv_tables, table_sizes, s_indices)
    _last.clear()
    _last["key"] = _key(qkv_feats, qkv_tables, s_indices)
    _last["out"], _last["lse"] = out, lse
    _last["alive"] = [weakref.ref(t) for t in qkv_feats]
    return lse.unsqueeze(-1)


def self_attn_forward(qkv_feats, qkv_tables, max_coffs, table_sizes, s_indices, indice_mode, pos_mode):
    """-> [raw [N,H,hd], sum [N,H,1]] in the dtype of the features, with raw / sum the attention output."""
    _check_modes(indice_mode, pos_mode)
    hit = _last.get("key") == _key(qkv_feats, qkv_tables, s_indices) and \
        all(r() is t for r, t in zip(_last.get("alive", []), qkv_feats))
    if hit:
        out = _last["out"]
    else:
        out, _ = _fused_forward(qkv_feats, qkv_tables, table_sizes, s_indices)
    _last.clear()
    N, H, _ = out.shape
    return [out, torch.ones((N, H, 1), dtype=out.dtype, device=out.device)]


def cal_exp_sum_grads(normed_out_grads, unnormed_out_feats, exp_sum_feats, value_feats, value_table):
    """-> zeros [N,H]: the term this call produced in the reference is computed inside the fused backward."""
    N, H, _ = normed_out_grads.shape
    return torch.zeros((N, H), dtype=normed_out_grads.dtype, device=normed_out_grads.device)


def self_attn_indir_backward(normed_out_grads, exp_sum_grads, unnormed_out_feats, exp_sum_feats, coff_rmax,
                             query_feats, key_feats, value_feats, query_table, key_table, value_table,
                             table_sizes, s_indices, indice_mode, pos_bias_method):
    """-> [dq, dk, dv, dTq, dTk, dTv]; feature gradients in the features' dtype, table gradients in the
    tables' dtype and shape."""
    _check_modes(indice_mode, pos_bias_method)
    q = query_feats.contiguous()
    c_dtype = q.dtype
    k, v = key_feats.to(c_dtype).contiguous(), value_feats.to(c_dtype).contiguous()
    tabs = [t.to(c_dtype).contiguous().view(-1) for t in (query_table, key_table, value_table)]
    sums = exp_sum_feats.to(torch.float32)
    out = (unnormed_out_feats.to(torch.float32) / sums).to(c_dtype).contiguous()
    lse = (coff_rmax.to(torch.float32) + torch.log(sums)).reshape(q.shape[0], q.shape[1]).contiguous()
    w_sizes, w2n, n2n, n_coords = _unpack_indices(s_indices)
    sizes = _sizes(table_sizes, (query_table, key_table, value_table), q)
    dq, dk, dv, dtq, dtk, dtv = attn_backward_raw(q, k, v, *tabs, sizes, w_sizes, w2n, n2n, n_coords, out, lse,
                                                  normed_out_grads.to(c_dtype).contiguous())
    return [dq, dk, dv, dtq.to(query_table.dtype).view_as(query_table), dtk.to(key_table.dtype).view_as(key_table),
            dtv.to(value_table.dtype).view_as(value_table)]
