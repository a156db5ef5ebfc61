"""The reference's pybind module ``Swin3D.sparse_dl.knn_cuda`` re-created over libswin3d_b200.so, for
callers that keep the reference's own ``knn.py`` (microsoft/Swin3D, Swin3D/src/knn/knn_api.cpp:4-6,
called at Swin3D/sparse_dl/knn/knn.py:16-24):

    knn_cuda(K, src_xyz, query_xyz, src_offset, query_offset, ret_idx, ret_dist) -> None

fills the two pre-allocated outputs: ``ret_idx`` int32 [Nq,K], ``ret_dist`` float32 [Nq,K] with the
SQUARED distances (the caller takes the square root).  Slots without a candidate get distance 2^31
and index 0 (the reference leaves the index uninitialised).
"""
import torch

from .. import _lib


def knn_cuda(K, src_xyz, query_xyz, src_offset, query_offset, ret_idx, ret_dist) -> None:
    for name, t in (("src_xyz", src_xyz), ("query_xyz", query_xyz)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != 3 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous float32 [n, 3] tensor")
    Nq, Ns = query_xyz.shape[0], src_xyz.shape[0]
    if tuple(ret_idx.shape) != (Nq, K) or ret_idx.dtype != torch.int32 or not ret_idx.is_contiguous():
        raise ValueError("ret_idx must be a contiguous int32 [Nq, K] tensor")
    if tuple(ret_dist.shape) != (Nq, K) or ret_dist.dtype != torch.float32 or not ret_dist.is_contiguous():
        raise ValueError("ret_dist must be a contiguous float32 [Nq, K] tensor")
    if src_offset.shape != query_offset.shape:
        raise ValueError("src_offset and query_offset must have one entry per scene")
    so = src_offset.to(torch.int32).contiguous()
    qo = query_offset.to(torch.int32).contiguous()
    with torch.cuda.device(query_xyz.device):
        st = torch.cuda.current_stream().cuda_stream
        rc = _lib.lib.s3d_knn(int(K), src_xyz.data_ptr(), query_xyz.data_ptr(), so.data_ptr(), qo.data_ptr(),
                              so.shape[0], Ns, Nq, ret_idx.data_ptr(), ret_dist.data_ptr(), st)
    _lib.check(rc, "s3d_knn")
