"""GPU: the allocation-free window builder (s3d_window_build_static) against the ordinary entry
point (s3d_window_build), through the C-ABI, on two calls in a row.

The static entry exists for hosts that cannot allocate device memory when they need the window
sets (a frozen memory pool, a context from which no allocator may be entered); its scratch is a
fixed array inside the library.  The file name sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from swin3d_b200 import synthetic as S

pytestmark = pytest.mark.gpu

MAX_VOXELS = 131072


def _outputs(N, F):
    return dict(n2n=torch.empty(N, dtype=torch.int32, device="cuda"),
                n_coords=torch.empty((N, F), dtype=torch.float32, device="cuda"),
                w_sizes=torch.zeros(max(N, 1), dtype=torch.int32, device="cuda"),
                w2n=torch.zeros(max(N, 1), dtype=torch.int32, device="cuda"),
                counts=torch.zeros(4, dtype=torch.int64, device="cuda"))


def _call_dynamic(lib, coords, feats, ws, shift, o):
    N, F = feats.shape
    nbytes = lib.s3d_window_build_workspace_bytes(N)
    work = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.s3d_window_build(coords.data_ptr(), feats.data_ptr(), N, F, 1, ws, shift,
                              o["n2n"].data_ptr(), o["n_coords"].data_ptr(), o["w_sizes"].data_ptr(),
                              o["w2n"].data_ptr(), o["counts"].data_ptr(), work.data_ptr(), nbytes, None)
    torch.cuda.synchronize()
    return rc


def _call_static(lib, coords, feats, ws, shift, o):
    N, F = feats.shape
    rc = lib.s3d_window_build_static(coords.data_ptr(), feats.data_ptr(), N, F, 1, ws, shift,
                                     o["n2n"].data_ptr(), o["n_coords"].data_ptr(), o["w_sizes"].data_ptr(),
                                     o["w2n"].data_ptr(), o["counts"].data_ptr(), None)
    torch.cuda.synchronize()
    return rc


def _same(a, b):
    W = int(a["counts"][0])
    assert W == int(b["counts"][0]) and W > 0
    assert torch.equal(a["counts"], b["counts"])
    assert torch.equal(a["n2n"], b["n2n"])
    assert torch.equal(a["n_coords"], b["n_coords"])
    assert torch.equal(a["w_sizes"][:W], b["w_sizes"][:W])
    assert torch.equal(a["w2n"][:W], b["w2n"][:W])


def test_static_window_build_matches_dynamic_on_two_calls_in_a_row():
    from swin3d_b200 import _lib
    lib = _lib.lib
    sc = S.make_room(11, target_voxels=50_000)
    coords = torch.from_numpy(sc.coords).cuda()
    feats = torch.from_numpy(S.signal_feats(sc, "XYZ_RGB_NORM")).cuda()
    N, F = feats.shape
    assert N <= MAX_VOXELS
    refs = []
    for ws, shift in ((5, 0), (7, 3)):
        o = _outputs(N, F)
        assert _call_dynamic(lib, coords, feats, ws, shift, o) == 0
        refs.append(o)
    # two static calls back to back; the second one finds the first one's leftovers in the scratch
    outs = []
    for ws, shift in ((5, 0), (7, 3)):
        o = _outputs(N, F)
        assert _call_static(lib, coords, feats, ws, shift, o) == 0
        outs.append(o)
    _same(outs[0], refs[0])
    _same(outs[1], refs[1])
    # and once more with a smaller input after a larger one
    small = slice(0, 3000)
    o_dyn, o_sta = _outputs(3000, F), _outputs(3000, F)
    assert _call_dynamic(lib, coords[small].contiguous(), feats[small].contiguous(), 5, 2, o_dyn) == 0
    assert _call_static(lib, coords[small].contiguous(), feats[small].contiguous(), 5, 2, o_sta) == 0
    _same(o_sta, o_dyn)


def test_static_window_build_uses_no_device_memory_of_its_own():
    from swin3d_b200 import _lib
    lib = _lib.lib
    sc = S.make_planes_and_boxes(3, 4096, 64)
    coords = torch.from_numpy(sc.coords).cuda()
    feats = torch.from_numpy(S.signal_feats(sc, "XYZ_RGB")).cuda()
    o = _outputs(*feats.shape)
    assert _call_static(lib, coords, feats, 5, 0, o) == 0      # first call: address look-up
    free_before, _ = torch.cuda.mem_get_info()
    assert _call_static(lib, coords, feats, 5, 2, o) == 0
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_window_build_rejects_inputs_beyond_its_capacity():
    from swin3d_b200 import _lib
    lib = _lib.lib
    N = MAX_VOXELS + 1
    coords = torch.zeros((N, 4), dtype=torch.int32, device="cuda")
    feats = torch.zeros((N, 3), dtype=torch.float32, device="cuda")
    o = _outputs(N, 3)
    o["counts"].fill_(-7)
    rc = _call_static(lib, coords, feats, 5, 0, o)
    assert rc == 5
    assert b"capacity" in lib.s3d_status_string(rc)
    assert int(o["counts"][0]) == -7        # nothing was launched


def test_static_window_build_at_exactly_its_capacity():
    """N == S3D_WINDOW_BUILD_STATIC_MAX_VOXELS: the largest input the entry point accepts uses the
    whole static array and must agree with the ordinary entry point."""
    from swin3d_b200 import _lib
    lib = _lib.lib
    sc = S.concat_scenes([S.make_room(21, target_voxels=90_000), S.make_room(22, target_voxels=90_000)])
    assert sc.coords.shape[0] >= MAX_VOXELS
    coords = torch.from_numpy(np.ascontiguousarray(sc.coords[:MAX_VOXELS])).cuda()
    feats = torch.from_numpy(np.ascontiguousarray(S.signal_feats(sc, "XYZ_RGB_NORM")[:MAX_VOXELS])).cuda()
    N, F = feats.shape
    assert N == MAX_VOXELS
    o_dyn, o_sta = _outputs(N, F), _outputs(N, F)
    assert _call_dynamic(lib, coords, feats, 5, 2, o_dyn) == 0
    assert _call_static(lib, coords, feats, 5, 2, o_sta) == 0
    _same(o_sta, o_dyn)
