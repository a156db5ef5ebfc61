"""All-in-one cRSE window attention as an autograd Function.

Call-compatible with the reference's ``Swin3D.sparse_dl.attn.attn_coff.SelfAttnAIOFunction``
(microsoft/Swin3D, Swin3D/sparse_dl/attn/attn_coff.py:155-232): same positional arguments, same
enums and enum values (:20-40), same dtype policy (:172-178, :207-217), same returned gradient
tuple (six gradients, six None).  What runs underneath is one fused forward kernel and one fused
backward kernel of libswin3d_b200.so instead of the reference's four kernels plus host-side
normalisation; the forward saves (out, lse) instead of (sum, max, norm).
"""
import enum
import weakref
from typing import Any, List

import torch
from torch import Tensor
from torch.autograd.function import Function

from ... import _lib


class PosEmb(enum.Enum):
    NONE = enum.auto()
    LINEAR = enum.auto()
    SEPARATE = enum.auto()


class TableDims(enum.Enum):
    WHCD = enum.auto()
    DWHC = enum.auto()
    D0 = enum.auto()


class IndexMode(enum.Enum):
    DIRECT = enum.auto()
    INDIRECT = enum.auto()


class PrecisionMode(enum.Enum):
    HALF_ALL = enum.auto()
    HALF_FORWARD = enum.auto()
    HALF_NONE = enum.auto()


_DTYPE_CODE = {torch.float32: _lib.S3D_F32, torch.float16: _lib.S3D_F16}

# int64 index tensors arrive unchanged for every block of a stage; convert each once.
# Keyed by id() because tensors compare element-wise; the weak reference guards against id reuse.
_int32_cache = {}


def _as_int32(t: Tensor) -> Tensor:
    if t.dtype == torch.int32 and t.is_contiguous():
        return t
    key = id(t)
    hit = _int32_cache.get(key)
    if hit is not None and hit[0]() is t and hit[1] == t._version:
        return hit[2]
    conv = t.to(torch.int32).contiguous()
    _int32_cache[key] = (weakref.ref(t, lambda _r, key=key: _int32_cache.pop(key, None)),
                         t._version, conv)
    return conv


# The reference's WindowAttention builds a fresh CUDA IntTensor of table offsets on every forward
# (swin3d_layers.py:511); reading it back costs a blocking device-to-host copy per attention block.
# The offsets of a module never change (they are its table shapes), so the host copy is kept per
# (number of offsets, total table elements, heads, head_dim) and a device tensor is read only the
# first time such a module is seen.  Set ``CACHE_TABLE_OFFSETS = False`` to read every time.
CACHE_TABLE_OFFSETS = True

# PrecisionMode.HALF_FORWARD (fp16_mode=1): the reference runs the backward on fp32 casts of q, k, v,
# the tables and the gradient (attn_coff.py:207-217).  That is the default here too (generic fp32
# kernels, 1e-4 agreement with the reference's fp32 backward).  With this switch on, the backward of
# that mode instead runs the tensor-core kernels on the fp16 values the forward used (fp16 storage,
# fp32 accumulation, the 2e-2 tolerance of the fp16 modes) and returns fp32 gradients: about four
# times faster, for callers who accept fp16-mode accuracy in the backward of fp16_mode=1.
HALF_FORWARD_FAST_BACKWARD = False
_table_sizes_cache = {}


def _table_sizes_host(table_offsets, table_numel: int = -1, H: int = 0, hd: int = 0) -> List[int]:
    """Elements per signal dimension as Python ints."""
    if not isinstance(table_offsets, Tensor):
        return [int(x) for x in table_offsets]
    if not table_offsets.is_cuda:
        return [int(x) for x in table_offsets.detach().tolist()]
    key = (int(table_offsets.numel()), int(table_numel), int(H), int(hd))
    if CACHE_TABLE_OFFSETS and table_numel >= 0:
        hit = _table_sizes_cache.get(key)
        if hit is not None:
            return list(hit)
    sizes = [int(x) for x in table_offsets.detach().cpu().tolist()]      # one blocking copy
    if table_numel >= 0 and sum(sizes) == table_numel:
        _table_sizes_cache[key] = tuple(sizes)
    return sizes


def _check_inputs(q: Tensor, k: Tensor, v: Tensor, tables, indices):
    for name, t in (("query", q), ("key", k), ("value", v)):
        if not t.is_cuda:
            raise RuntimeError(f"{name}_feats must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{name}_feats must be contiguous")
        if t.dim() != 3 or t.shape != q.shape:
            raise ValueError(f"{name}_feats must have shape [N, heads, head_dim] like the query")
    for t in tables:
        if not t.is_cuda or not t.is_contiguous():
            raise RuntimeError("tables must be contiguous CUDA tensors")
    if len(indices) != 6:
        raise ValueError("IndexMode.INDIRECT takes six index tensors "
                         "[m2w, w_sizes, w2m, w2n, n2n, n_coords]")


def _aligned16(*tensors):
    """The library wants 16-byte aligned rows and tables; a view that starts in the middle of a
    storage (rare: torch allocations are 256-byte aligned) is copied."""
    return [t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format) for t in tensors]


def _pointer_array(ptrs):
    import ctypes
    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr, ctypes.cast(arr, ctypes.c_void_p)


def attn_forward_raw(q, k, v, tq, tk, tv, sizes: List[int], w_sizes, w2n, n2n, n_coords, out=None, lse=None,
                     mirrors=None, window_class: int = 0):
    """One fused forward launch.  Tensors must already have the compute dtype.  -> (out, lse).
    `out` / `lse` may be given (full-size, contiguous): only the rows of the voxels of the windows
    in `w_sizes` / `w2n` are written, so a window list can be processed in several calls.
    `mirrors`: device addresses (ints) of up to 7 further arrays of out's shape -- other GPUs' result
    arrays mapped into this process -- that receive the same rows by peer stores from the kernels.
    `window_class`: 1 / 2 = the caller guarantees that every window of this call has at most 32 voxels /
    more than 32 (a window that breaks the guarantee is not processed); 0 = any sizes."""
    import ctypes
    q, k, v, tq, tk, tv = _aligned16(q, k, v, tq, tk, tv)
    N, H, hd = q.shape
    W = w_sizes.shape[0]
    D = len(sizes)
    if n_coords.shape != (N, D):
        raise ValueError(f"n_coords must have shape [{N}, {D}]")
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((N, H), dtype=torch.float32, device=q.device)
    if out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or lse.shape != (N, H):
        raise ValueError("out / lse buffers must be contiguous and match the query")
    arr = (ctypes.c_int32 * D)(*sizes)
    with torch.cuda.device(q.device):
        st = torch.cuda.current_stream().cuda_stream
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                ctypes.cast(arr, ctypes.c_void_p), D, w_sizes.data_ptr(), w2n.data_ptr(),
                n2n.data_ptr(), n_coords.data_ptr(), N, W, H, hd, _DTYPE_CODE[q.dtype],
                out.data_ptr(), lse.data_ptr())
        if mirrors or window_class:
            keep, mp = _pointer_array(mirrors) if mirrors else (None, None)
            rc = _lib.lib.s3d_attn_fwd_mirrored(*args, len(mirrors) if mirrors else 0, mp, int(window_class), st)
        else:
            rc = _lib.lib.s3d_attn_fwd(*args, st)
    _lib.check(rc, "s3d_attn_fwd")
    return out, lse


def attn_backward_raw(q, k, v, tq, tk, tv, sizes: List[int], w_sizes, w2n, n2n, n_coords,
                      out, lse, dout, dq=None, dk=None, dv=None, mirrors=None):
    """One fused backward launch -> (dq, dk, dv, dtq, dtk, dtv); table grads are fp32 (fresh arrays,
    zeroed by the library).  `dq`, `dk`, `dv` may be given (full-size, contiguous): only the rows of
    the voxels of the windows in `w_sizes` / `w2n` are written.  `mirrors`: three equally long lists of
    device addresses, further dq, dk and dv arrays that receive the same rows (see the forward)."""
    import ctypes
    q, k, v, tq, tk, tv, out, dout = _aligned16(q, k, v, tq, tk, tv, out, dout)
    N, H, hd = q.shape
    W = w_sizes.shape[0]
    D = len(sizes)
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    for t in (dq, dk, dv):
        if t.shape != q.shape or t.dtype != q.dtype or not t.is_contiguous():
            raise ValueError("dq / dk / dv buffers must be contiguous and match the query")
    tn = sum(sizes)
    dt = torch.empty((3, tn), dtype=torch.float32, device=q.device)
    arr = (ctypes.c_int32 * D)(*sizes)
    with torch.cuda.device(q.device):
        st = torch.cuda.current_stream().cuda_stream
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                ctypes.cast(arr, ctypes.c_void_p), D, w_sizes.data_ptr(), w2n.data_ptr(),
                n2n.data_ptr(), n_coords.data_ptr(), N, W, H, hd, _DTYPE_CODE[q.dtype],
                out.data_ptr(), lse.data_ptr(), dout.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                dv.data_ptr(), dt[0].data_ptr(), dt[1].data_ptr(), dt[2].data_ptr())
        if mirrors and len(mirrors[0]):
            if not (len(mirrors) == 3 and len(mirrors[0]) == len(mirrors[1]) == len(mirrors[2])):
                raise ValueError("mirrors: three equally long address lists (dq, dk, dv)")
            keep = [_pointer_array(m) for m in mirrors]
            rc = _lib.lib.s3d_attn_bwd_mirrored(*args, len(mirrors[0]), keep[0][1], keep[1][1], keep[2][1], st)
        else:
            rc = _lib.lib.s3d_attn_bwd(*args, st)
    _lib.check(rc, "s3d_attn_bwd")
    return dq, dk, dv, dt[0], dt[1], dt[2]


class SelfAttnAIOFunction(Function):
    """Function of all-in-one self-attention (fused forward / fused backward)."""

    @staticmethod
    def forward(ctx, raw_query_feats, raw_key_feats, raw_value_feats, query_table, key_table,
                value_table, table_offsets, indices: List[Tensor], pe: PosEmb,
                table_dim: TableDims, mode: IndexMode, precision: PrecisionMode):
        assert table_dim == TableDims.D0
        if mode != IndexMode.INDIRECT or pe != PosEmb.SEPARATE:
            raise NotImplementedError(
                "only IndexMode.INDIRECT with PosEmb.SEPARATE is implemented "
                "(the combination WindowAttention passes)")
        _check_inputs(raw_query_feats, raw_key_feats, raw_value_feats,
                      (query_table, key_table, value_table), indices)
        ctx.precision = precision

        # dtype policy of the reference (attn_coff.py:172-178)
        if torch.is_autocast_enabled() and precision != PrecisionMode.HALF_NONE:
            c_dtype = (torch.get_autocast_dtype("cuda") if hasattr(torch, "get_autocast_dtype")
                       else torch.get_autocast_gpu_dtype())
        else:
            c_dtype = torch.float32
        if c_dtype not in _DTYPE_CODE:
            raise ValueError(f"compute dtype {c_dtype} is not supported (float32 or float16)")

        qkv = [t.to(c_dtype) for t in (raw_query_feats, raw_key_feats, raw_value_feats)]
        tabs = [t.to(c_dtype).contiguous() for t in (query_table, key_table, value_table)]
        sizes = _table_sizes_host(table_offsets, query_table.numel(), raw_query_feats.shape[1],
                                  raw_query_feats.shape[2])
        _, w_sizes, _, w2n, n2n, n_coords = indices
        w_sizes, w2n, n2n = _as_int32(w_sizes), _as_int32(w2n), _as_int32(n2n)
        n_coords = n_coords.to(torch.float32).contiguous()

        out, lse = attn_forward_raw(*qkv, *tabs, sizes, w_sizes, w2n, n2n, n_coords)

        ctx.sizes = sizes
        ctx.save_for_backward(out, lse, raw_query_feats, raw_key_feats, raw_value_feats,
                              query_table, key_table, value_table, w_sizes, w2n, n2n, n_coords)
        return out

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any) -> Any:
        (grad,) = grad_outputs
        (out, lse, q, k, v, tq, tk, tv, w_sizes, w2n, n2n, n_coords) = ctx.saved_tensors
        precision: PrecisionMode = ctx.precision
        # dtype policy of the reference (attn_coff.py:207-217)
        if precision == PrecisionMode.HALF_ALL:
            c_dtype = grad.dtype
        elif precision == PrecisionMode.HALF_FORWARD and HALF_FORWARD_FAST_BACKWARD and out.dtype == torch.float16:
            c_dtype = torch.float16       # opt-in: tensor-core backward on the forward's fp16 values
        else:
            c_dtype = torch.float32
        if c_dtype not in _DTYPE_CODE:
            raise ValueError(f"compute dtype {c_dtype} is not supported (float32 or float16)")
        qkv = [t.to(c_dtype) for t in (q, k, v)]
        tabs = [t.to(c_dtype).contiguous() for t in (tq, tk, tv)]
        dq, dk, dv, dtq, dtk, dtv = attn_backward_raw(
            *qkv, *tabs, ctx.sizes, w_sizes, w2n, n2n, n_coords,
            out.to(c_dtype), lse, grad.to(c_dtype).contiguous())
        grads = (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype),
                 dtq.to(tq.dtype).view_as(tq), dtk.to(tk.dtype).view_as(tk),
                 dtv.to(tv.dtype).view_as(tv))
        return (*grads, None, None, None, None, None, None)
