"""CPU: the re-created pybind modules expose the names and argument lists of the reference's
``attn_cuda`` / ``knn_cuda`` (microsoft/Swin3D, Swin3D/src/attn/attn_api.cpp:20-24,
Swin3D/src/attn/self_attn_aio_fwd.h:11-26, self_attn_aio_bwd.h:9-32, Swin3D/src/knn/knn_api.cpp:4-6),
and the installer registers them under the names the reference's Python imports.  No compute."""
import inspect
import sys

import pytest

torch = pytest.importorskip("torch")


def test_names_and_argument_counts():
    from swin3d_b200.sparse_dl import attn_cuda, knn_cuda
    want = {"cal_max_coffs": 6, "self_attn_forward": 7, "cal_exp_sum_grads": 5, "self_attn_indir_backward": 15}
    for name, n in want.items():
        assert len(inspect.signature(getattr(attn_cuda, name)).parameters) == n, name
    assert list(inspect.signature(knn_cuda.knn_cuda).parameters) == ["K", "src_xyz", "query_xyz", "src_offset",
                                                                    "query_offset", "ret_idx", "ret_dist"]


def test_installer_registers_the_reference_import_names():
    from swin3d_b200 import compat
    saved = {k: sys.modules.get(k) for k in ("Swin3D.sparse_dl.attn_cuda", "Swin3D.sparse_dl.knn_cuda")}
    try:
        compat.install_pybind_modules(force=True)
        import swin3d_b200.sparse_dl.attn_cuda as a
        import swin3d_b200.sparse_dl.knn_cuda as k
        assert sys.modules["Swin3D.sparse_dl.attn_cuda"] is a and sys.modules["Swin3D.sparse_dl.knn_cuda"] is k
    finally:
        for name, mod in saved.items():
            if mod is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = mod


def test_unsupported_modes_are_rejected_before_any_device_work():
    from swin3d_b200.sparse_dl import attn_cuda
    with pytest.raises(NotImplementedError):
        attn_cuda.cal_max_coffs([], [], None, [], 1, 3)           # IndexMode.DIRECT
    with pytest.raises(NotImplementedError):
        attn_cuda.self_attn_indir_backward(*([None] * 13), 2, 1)  # PosEmb.NONE
