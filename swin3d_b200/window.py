"""Host wrapper of the window builder kernel chain (s3d_window_build).

``build_windows`` produces, for one (stage, shift), what the reference's
``BasicLayer.get_index01`` (microsoft/Swin3D, Swin3D/modules/swin3d_layers.py:789-822) produces
through MinkowskiEngine: the window-sorted voxel order ``n2n_indices``, the per-window sizes and
offsets, and ``n_coords`` (cell + in-voxel position, then the colour / normal signals) in sorted
order.  Windows are emitted in lexicographic (batch, wx, wy, wz) order; the reference's order is
whatever MinkowskiEngine's pooling returns and attention does not depend on it.
"""
from dataclasses import dataclass

import torch

from . import _lib


@dataclass
class WindowIndex:
    n2n: torch.Tensor        # int32 [N]  sorted position -> voxel row
    n_coords: torch.Tensor   # float32 [N, F]  sorted order
    w_sizes: torch.Tensor    # int32 [W]
    w2n: torch.Tensor        # int32 [W]  first sorted position of each window
    num_pairs: int           # M = sum w^2
    max_window: int

    def reference_indices(self, n_crse: torch.Tensor):
        """The six-tensor list ``SelfAttnAIOFunction.apply`` takes for IndexMode.INDIRECT.
        ``m2w`` (one entry per attention pair in the reference) is never read by the fused
        kernels, so an empty tensor stands in for it; ``w2m`` is the exclusive sum of w^2."""
        w2 = self.w_sizes.to(torch.int64) ** 2
        w2m = torch.cumsum(w2, 0) - w2
        m2w = torch.empty(0, dtype=torch.int64, device=self.n2n.device)
        return [m2w, self.w_sizes, w2m, self.w2n, self.n2n, n_crse]


def build_windows(coords: torch.Tensor, feats: torch.Tensor, window_size: int, shift: int = 0,
                  stride: int = 1) -> WindowIndex:
    """coords int32 [N,4] (batch,x,y,z; multiples of ``stride``); feats float32 [N,F] with the
    in-voxel position in columns 0..2 and the other cRSE signals after it."""
    if not coords.is_cuda or not feats.is_cuda:
        raise RuntimeError("coords and feats must be CUDA tensors")
    if coords.dtype != torch.int32 or coords.dim() != 2 or coords.shape[1] != 4:
        raise ValueError("coords must be int32 [N, 4]")
    N = coords.shape[0]
    if feats.dtype != torch.float32 or feats.dim() != 2 or feats.shape[0] != N:
        raise ValueError("feats must be float32 [N, F]")
    coords = coords.contiguous()
    feats = feats.contiguous()
    F = feats.shape[1]
    dev = coords.device
    n2n = torch.empty(N, dtype=torch.int32, device=dev)
    n_coords = torch.empty((N, F), dtype=torch.float32, device=dev)
    w_sizes = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
    w2n = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
    counts = torch.empty(4, dtype=torch.int64, device=dev)
    wbytes = _lib.lib.s3d_window_build_workspace_bytes(N)
    work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        st = torch.cuda.current_stream().cuda_stream
        rc = _lib.lib.s3d_window_build(
            coords.data_ptr(), feats.data_ptr(), N, F, int(stride), int(window_size), int(shift),
            n2n.data_ptr(), n_coords.data_ptr(), w_sizes.data_ptr(), w2n.data_ptr(),
            counts.data_ptr(), work.data_ptr(), wbytes, st)
    _lib.check(rc, "s3d_window_build")
    W, M, mx, err = (int(x) for x in counts.tolist())  # the one host sync of the builder
    if err:
        raise ValueError("s3d_window_build: a batch index or window coordinate is outside the "
                         "supported key range (batch < 1024, |window index| < 16384)")
    return WindowIndex(n2n, n_coords, w_sizes[:W], w2n[:W], M, mx)


def _tensor_stride(sp) -> int:
    """Tensor stride of a MinkowskiEngine-style sparse tensor (or of any object that mimics
    ``sp.coordinate_map_key.get_tensor_stride()`` / ``sp.tensor_stride``)."""
    key = getattr(sp, "coordinate_map_key", None)
    if key is not None and hasattr(key, "get_tensor_stride"):
        s = key.get_tensor_stride()
    else:
        s = getattr(sp, "tensor_stride", 1)
    return int(s[0]) if isinstance(s, (list, tuple)) else int(s)


def get_index01(sp, local_xyz: torch.Tensor, colors: torch.Tensor, window_size: int,
                shift_size: int = 0):
    """Call-compatible replacement of ``BasicLayer.get_index01`` (Swin3D/modules/swin3d_layers.py:
    789-822) that does not go through MinkowskiEngine: ``sp`` only needs ``.C`` (int [N,4]: batch,
    x, y, z) and its tensor stride.  Returns the same 8-tuple ``WindowAttention.forward``
    (:490-500) unpacks:

        (x_offset, y_offset, m2w_indices, w_sizes, w2n_indices, n2n_indices, w2m_indices, n_coords)

    ``x_offset`` and ``y_offset`` are not read by ``WindowAttention`` and ``m2w_indices`` (one entry
    per attention pair) is not read by the fused kernels: they are None / an empty tensor.  The
    index tensors are int32, which ``SelfAttnAIOFunction`` takes as they are (the reference converts
    int64 to int32 inside every call, self_attn_aio_fwd.cu:395-400).

    ``shift_size`` (in voxels of this stage) may be given instead of building a shifted copy of
    ``sp`` as ``BasicLayer.get_shifted_sp`` does; a shifted ``sp`` with ``shift_size=0`` groups
    the same way."""
    feats = torch.cat([local_xyz, colors], dim=1).float()
    wi = build_windows(sp.C.int(), feats, window_size, shift_size, _tensor_stride(sp))
    w2 = wi.w_sizes.to(torch.int64) ** 2
    w2m = torch.cumsum(w2, 0) - w2
    m2w = torch.empty(0, dtype=torch.int64, device=wi.n2n.device)
    return (None, None, m2w, wi.w_sizes, wi.w2n, wi.n2n, w2m, wi.n_coords)
