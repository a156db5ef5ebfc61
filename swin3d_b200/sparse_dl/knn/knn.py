"""Brute-force KNN as an autograd Function (no backward), call-compatible with the reference's
``Swin3D.sparse_dl.knn.KNN`` (microsoft/Swin3D, Swin3D/sparse_dl/knn/knn.py:9-26):
``KNN.apply(K, src_xyz, query_xyz, src_offset, query_offset) -> (idx int32 [Nq,K], dist [Nq,K])``
with ``dist`` the Euclidean distance (sqrt of the kernel's squared distance, knn.py:25).
"""
import torch
from torch.autograd.function import Function

from ... import _lib


def knn_raw(K: int, src_xyz, query_xyz, src_offset, query_offset):
    """-> (idx int32 [Nq,K], squared distance float32 [Nq,K])."""
    for name, t in (("src_xyz", src_xyz), ("query_xyz", query_xyz)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != 3:
            raise ValueError(f"{name} must be float32 [n, 3]")
    assert src_xyz.is_contiguous() and query_xyz.is_contiguous()
    if src_offset.shape != query_offset.shape:
        raise ValueError("src_offset and query_offset must have one entry per scene")
    so = src_offset.to(torch.int32).contiguous()
    qo = query_offset.to(torch.int32).contiguous()
    Nq, Ns = query_xyz.shape[0], src_xyz.shape[0]
    idx = torch.empty((Nq, K), dtype=torch.int32, device=query_xyz.device)
    d2 = torch.empty((Nq, K), dtype=torch.float32, device=query_xyz.device)
    with torch.cuda.device(query_xyz.device):
        st = torch.cuda.current_stream().cuda_stream
        rc = _lib.lib.s3d_knn(int(K), src_xyz.data_ptr(), query_xyz.data_ptr(), so.data_ptr(),
                              qo.data_ptr(), so.shape[0], Ns, Nq, idx.data_ptr(), d2.data_ptr(), st)
    _lib.check(rc, "s3d_knn")
    return idx, d2


class KNN(Function):
    @staticmethod
    def forward(ctx, K, src_xyz, query_xyz, src_offset, query_offset):
        idx, d2 = knn_raw(K, src_xyz, query_xyz, src_offset, query_offset)
        dist = torch.sqrt(d2)
        ctx.mark_non_differentiable(idx, dist)
        return idx, dist
