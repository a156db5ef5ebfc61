"""The callers either side of KNN, with the gather fused away.

Mirrors of the reference's module-level helpers (microsoft/Swin3D,
Swin3D/modules/swin3d_layers.py): ``knn_linear_interpolation`` (:53-73), ``query_knn_feature``
(:28-50), ``get_offset`` (:234-241), plus ``knn_max_pool`` for the gather + MaxPool1d(K) tail of
``GridKNNDownsample.forward`` (:302-309).  Same argument order and meaning as the reference; the
[Nq, K, C] gathered tensor of the reference is never built by the fused forms.
"""
import torch
from torch.autograd.function import Function

from ... import _lib
from .knn import KNN


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.S3D_F32
    if t.dtype == torch.float16:
        return _lib.S3D_F16
    raise ValueError(f"unsupported feature dtype {t.dtype}: float32 or float16")


def _check_feat(name: str, t: torch.Tensor):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dim() != 2:
        raise ValueError(f"{name} must be [n, C]")
    vec = 4 if t.dtype == torch.float32 else 8
    if t.shape[1] % vec:
        raise ValueError(f"{name}: channel count {t.shape[1]} must be a multiple of {vec} for {t.dtype}")


def get_offset(batch: torch.Tensor) -> torch.Tensor:
    """Cumulative scene ends (int32 [B]) from per-point batch indices; one bincount and one
    cumsum instead of the reference's per-scene Python loop with a device sync per scene."""
    return torch.cumsum(torch.bincount(batch.long()), 0).to(torch.int32)


class KNNInterpolate(Function):
    """out[q] = sum_i src_feat[idx[q,i]] * w_i with normalised inverse-distance weights."""

    @staticmethod
    def forward(ctx, src_feat, idx, dist):
        _check_feat("src_feat", src_feat)
        src_feat = src_feat.contiguous()
        idx = idx.to(torch.int32).contiguous()
        dist = dist.to(torch.float32).contiguous()
        Nq, K = idx.shape
        C = src_feat.shape[1]
        out = torch.empty((Nq, C), dtype=src_feat.dtype, device=src_feat.device)
        with torch.cuda.device(src_feat.device):
            st = torch.cuda.current_stream().cuda_stream
            rc = _lib.lib.s3d_knn_interpolate_fwd(idx.data_ptr(), dist.data_ptr(), src_feat.data_ptr(),
                                                  out.data_ptr(), Nq, K, C, _dtype_code(src_feat), st)
        _lib.check(rc, "s3d_knn_interpolate_fwd")
        ctx.save_for_backward(idx, dist)
        ctx.n_src = src_feat.shape[0]
        return out

    @staticmethod
    def backward(ctx, grad_out):
        idx, dist = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        Nq, K = idx.shape
        C = grad_out.shape[1]
        dsrc = torch.empty((ctx.n_src, C), dtype=torch.float32, device=grad_out.device)
        with torch.cuda.device(grad_out.device):
            st = torch.cuda.current_stream().cuda_stream
            rc = _lib.lib.s3d_knn_interpolate_bwd(idx.data_ptr(), dist.data_ptr(), grad_out.data_ptr(),
                                                  dsrc.data_ptr(), Nq, ctx.n_src, K, C,
                                                  _dtype_code(grad_out), st)
        _lib.check(rc, "s3d_knn_interpolate_bwd")
        return dsrc.to(grad_out.dtype), None, None


def knn_linear_interpolation(src_xyz, query_xyz, src_feat, src_offset, query_offset, K=3):
    """Drop-in for swin3d_layers.py:53-73."""
    assert src_xyz.is_contiguous() and query_xyz.is_contiguous() and src_feat.is_contiguous()
    idx, dist = KNN.apply(K, src_xyz, query_xyz, src_offset, query_offset)
    return KNNInterpolate.apply(src_feat, idx, dist)


class KNNMaxPool(Function):
    """out[q,c] = max_i g[idx[q,i], c]; the gradient goes to the row that supplied the maximum."""

    @staticmethod
    def forward(ctx, g, idx):
        _check_feat("g", g)
        g = g.contiguous()
        idx = idx.to(torch.int32).contiguous()
        Nq, K = idx.shape
        C = g.shape[1]
        out = torch.empty((Nq, C), dtype=g.dtype, device=g.device)
        arg = torch.empty((Nq, C), dtype=torch.int32, device=g.device)
        with torch.cuda.device(g.device):
            st = torch.cuda.current_stream().cuda_stream
            rc = _lib.lib.s3d_knn_maxpool_fwd(idx.data_ptr(), g.data_ptr(), out.data_ptr(),
                                              arg.data_ptr(), Nq, K, C, _dtype_code(g), st)
        _lib.check(rc, "s3d_knn_maxpool_fwd")
        ctx.save_for_backward(arg)
        ctx.n_src = g.shape[0]
        ctx.mark_non_differentiable(arg)
        return out, arg

    @staticmethod
    def backward(ctx, grad_out, _grad_arg):
        (arg,) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        Nq, C = grad_out.shape
        dg = torch.empty((ctx.n_src, C), dtype=torch.float32, device=grad_out.device)
        with torch.cuda.device(grad_out.device):
            st = torch.cuda.current_stream().cuda_stream
            rc = _lib.lib.s3d_knn_maxpool_bwd(arg.data_ptr(), grad_out.data_ptr(), dg.data_ptr(),
                                              Nq, ctx.n_src, C, _dtype_code(grad_out), st)
        _lib.check(rc, "s3d_knn_maxpool_bwd")
        return dg.to(grad_out.dtype), None


def knn_max_pool(K, src_xyz, query_xyz, g, src_offset, query_offset):
    """``MaxPool1d(K)(g[idx].transpose(1, 2))`` of GridKNNDownsample.forward (:302-309) for
    ``g = linear(norm(src_feat))`` evaluated per source row (LayerNorm and the bias-free Linear
    act row by row, so they commute with the reference's gather)."""
    idx, _ = KNN.apply(K, src_xyz, query_xyz, src_offset, query_offset)
    out, _ = KNNMaxPool.apply(g, idx)
    return out


def query_knn_feature(K, src_xyz, query_xyz, src_feat, src_offset, query_offset, return_idx=False):
    """Drop-in for swin3d_layers.py:28-50 (the unfused gather, kept for callers that need the
    [Nq, K, C] tensor itself)."""
    if query_xyz is None:
        query_xyz, query_offset = src_xyz, src_offset
    assert src_xyz.is_contiguous() and query_xyz.is_contiguous() and src_feat.is_contiguous()
    idx, _ = KNN.apply(K, src_xyz, query_xyz, src_offset, query_offset)
    m, c = query_xyz.shape[0], src_feat.shape[1]
    grouped = src_feat[idx.view(-1).long(), :].view(m, K, c)
    return (grouped, idx) if return_idx else grouped
