"""CPU: the C-ABI library loads and exports every symbol include/swin3d_b200.h declares; argument
validation that needs no device works (no compute call is made)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "swin3d_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(s3d_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ("s3d_attn_fwd", "s3d_attn_bwd", "s3d_window_build", "s3d_knn",
              "s3d_window_build_workspace_bytes", "s3d_status_string", "s3d_version",
              "s3d_debug_crse_indices", "s3d_knn_interpolate_fwd", "s3d_knn_interpolate_bwd",
              "s3d_knn_maxpool_fwd", "s3d_knn_maxpool_bwd"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from swin3d_b200 import _lib
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(raw, s), f"{s} declared in the header but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"


def test_status_strings_and_version():
    from swin3d_b200 import _lib
    assert _lib.lib.s3d_version() >= 1000
    assert _lib.lib.s3d_status_string(0) == b"ok"
    for code in (1, 2, 3, 4):
        assert len(_lib.lib.s3d_status_string(code)) > 3


def test_argument_validation_without_device():
    from swin3d_b200 import _lib
    L = _lib.lib
    sizes = (ctypes.c_int32 * 3)(320, 320, 320)
    p = ctypes.cast(sizes, ctypes.c_void_p)
    # unsupported head_dim / signal dims / dtype / bad table size: rejected before any CUDA call
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 3, None, None, None, None,
                          10, 1, 2, 7, 0, None, None, None) == 2
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 4, None, None, None, None,
                          10, 1, 2, 8, 0, None, None, None) == 2
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 3, None, None, None, None,
                          10, 1, 2, 8, 5, None, None, None) == 1
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 3, None, None, None, None,
                          10, 1, 3, 8, 0, None, None, None) == 1   # 320 % (3*8) != 0
    # null pointers with work to do
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 3, None, None, None, None,
                          10, 1, 2, 8, 0, None, None, None) == 1
    # empty problem is a no-op
    assert L.s3d_attn_fwd(None, None, None, None, None, None, p, 3, None, None, None, None,
                          0, 0, 2, 8, 0, None, None, None) == 0
    # a row or table pointer that is not 16-byte aligned is refused before any launch (the
    # addresses are never dereferenced on this path)
    ok, odd = 0x10000, 0x10004
    assert L.s3d_attn_fwd(odd, ok, ok, ok, ok, ok, p, 3, ok, ok, ok, ok, 10, 1, 2, 8, 0, ok, ok, None) == 1
    assert L.s3d_attn_fwd(ok, ok, ok, ok, odd, ok, p, 3, ok, ok, ok, ok, 10, 1, 2, 8, 0, ok, ok, None) == 1
    assert L.s3d_attn_fwd(ok, ok, ok, ok, ok, ok, p, 3, ok, ok, ok, ok, 10, 1, 2, 8, 0, odd, ok, None) == 1
    assert L.s3d_knn(65, None, None, None, None, 1, 0, 0, None, None, None) == 2
    assert L.s3d_knn(0, None, None, None, None, 1, 0, 0, None, None, None) == 2
    assert L.s3d_knn(3, None, None, None, None, 1, 0, 0, None, None, None) == 0
    assert L.s3d_knn(3, None, None, None, None, 1, 5, 5, None, None, None) == 1
    assert L.s3d_window_build(None, None, 5, 9, 1, 9, 0, None, None, None, None, None, None, 0, None) == 2
    assert L.s3d_window_build_workspace_bytes(1000) > 1000 * 24


def test_python_wrappers_reject_cpu_tensors():
    import torch
    from swin3d_b200.sparse_dl.attn.attn_coff import (SelfAttnAIOFunction, PosEmb, TableDims,
                                                      IndexMode, PrecisionMode)
    from swin3d_b200.sparse_dl.knn import KNN
    q = torch.zeros(4, 2, 8)
    t = torch.zeros(3 * 40 * 16)
    idx = [torch.zeros(0, dtype=torch.int64)] * 5 + [torch.zeros(4, 3)]
    with pytest.raises(RuntimeError, match="CUDA"):
        SelfAttnAIOFunction.apply(q, q, q, t, t, t, torch.tensor([640] * 3), idx, PosEmb.SEPARATE,
                                  TableDims.D0, IndexMode.INDIRECT, PrecisionMode.HALF_NONE)
    with pytest.raises(NotImplementedError):
        SelfAttnAIOFunction.apply(q, q, q, t, t, t, torch.tensor([640] * 3), idx, PosEmb.SEPARATE,
                                  TableDims.D0, IndexMode.DIRECT, PrecisionMode.HALF_NONE)
    with pytest.raises(RuntimeError, match="CUDA"):
        KNN.apply(3, torch.zeros(5, 3), torch.zeros(5, 3), torch.tensor([5]), torch.tensor([5]))


def test_patch_basic_layer_replaces_get_index01_and_forwards_the_window_size(monkeypatch):
    """compat.patch_basic_layer: the method keeps the reference's signature and hands the layer's
    window size to the window builder (no GPU: the builder is replaced by a recorder)."""
    from swin3d_b200 import compat, window

    class BasicLayer:                      # stands in for Swin3D.modules.swin3d_layers.BasicLayer
        window_size = 7

        def get_index01(self, sp, local_xyz, colors):
            raise AssertionError("the MinkowskiEngine path must not run")

    seen = []
    monkeypatch.setattr(window, "get_index01", lambda *a, **k: seen.append((a, k)) or "tuple")
    compat.patch_basic_layer(BasicLayer)
    assert BasicLayer().get_index01("sp", "xyz", "rgb") == "tuple"
    assert seen == [(("sp", "xyz", "rgb", 7), {})]
