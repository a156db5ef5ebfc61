"""GPU parity: the CUDA attention kernels (through the C-ABI) against the CPU oracle.

Tolerances (relative = max|a-b| / max|b|, as the benchmark's north star states them):
fp32 outputs and gradients 1e-4; fp16 storage 2e-2; cRSE indices bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from swin3d_b200 import synthetic as S
from tests.helpers import make_problem, oracle_fwd_bwd, rel_err, table_row_errors

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
FP16_TOL = 2e-2

CASES = [
    # crse, H, hd, ws, shift
    ("XYZ", 2, 8, 5, 0),
    ("XYZ_RGB", 6, 8, 5, 0),       # the single-layer CPU-sized config: 6 heads of 8, window 5
    ("XYZ_RGB", 6, 8, 5, 2),
    ("XYZ_RGB_NORM", 10, 8, 5, 2), # Swin3D-L stage-1 head layout
    ("XYZ_RGB_NORM", 3, 16, 7, 3),
    ("XYZ_RGB", 1, 32, 5, 0),
]


@pytest.mark.parametrize("crse,H,hd,ws,shift", CASES)
def test_fp32_forward_backward_match_oracle(crse, H, hd, ws, shift):
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=11, n_voxels=1200, grid=28, ws=ws, shift=shift, H=H, hd=hd, crse=crse)
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    out, lse, grads = cuda_fwd_bwd(p, torch.float32)
    assert rel_err(out, o_ref) < FP32_TOL
    assert np.abs(lse - lse_ref).max() < 1e-4
    for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
        assert rel_err(a, b) < FP32_TOL, name
    for name, a, b in zip("dtq dtk dtv".split(), grads[3:], g_ref[3:]):     # row by row: no row may hide
        assert table_row_errors(a, b, H * hd, FP32_TOL, 1e-3) == [], name


@pytest.mark.parametrize("crse,H,hd,ws,shift", CASES[1:5])
def test_fp16_forward_backward_match_oracle(crse, H, hd, ws, shift):
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=12, n_voxels=1200, grid=28, ws=ws, shift=shift, H=H, hd=hd, crse=crse,
                     round_fp16=True)
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    out, lse, grads = cuda_fwd_bwd(p, torch.float16)
    assert rel_err(out, o_ref) < FP16_TOL
    for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
        assert rel_err(a, b) < FP16_TOL, name
    for name, a, b in zip("dtq dtk dtv".split(), grads[3:], g_ref[3:]):     # row by row: no row may hide
        assert table_row_errors(a, b, H * hd, FP16_TOL, 2e-2) == [], name


def test_config1_full_size_fp32():
    """4,096 voxels from 3 planes + 2 boxes in a 64^3 grid, C=48, 6 heads, window 5, XYZ_RGB."""
    from tests.gpu_helpers import cuda_fwd_bwd
    for shift in (0, 2):
        p = make_problem(seed=0, n_voxels=4096, grid=64, ws=5, shift=shift, H=6, hd=8, crse="XYZ_RGB")
        o_ref, _, g_ref = oracle_fwd_bwd(p, np.float64)
        out, _, grads = cuda_fwd_bwd(p, torch.float32)
        assert rel_err(out, o_ref) < FP32_TOL
        for a, b in zip(grads, g_ref):
            assert rel_err(a, b) < FP32_TOL


def test_dense_windows_up_to_full_occupancy():
    """Fully occupied 5^3 and 7^3 windows (125 and 343 voxels) plus single-voxel windows."""
    from tests.gpu_helpers import cuda_fwd_bwd
    g = np.stack(np.meshgrid(*[np.arange(7)] * 3, indexing="ij"), -1).reshape(-1, 3)
    lonely = np.array([[40, 40, 40], [60, 3, 9], [90, 90, 90]])
    pts = np.concatenate([g, lonely])
    n = len(pts)
    rng = np.random.default_rng(5)
    sc = S.Scene(np.concatenate([np.zeros((n, 1)), pts], 1).astype(np.int32),
                 rng.random((n, 3), dtype=np.float32) * 0.999, rng.random((n, 3), dtype=np.float32),
                 np.tile(np.array([[0, 0, 1]], dtype=np.float32), (n, 1)))
    for ws in (5, 7):
        p = make_problem(seed=2, ws=ws, H=2, hd=8, crse="XYZ_RGB_NORM", scene=sc)
        assert p.w_sizes.max() == ws ** 3 and p.w_sizes.min() == 1
        o_ref, _, g_ref = oracle_fwd_bwd(p, np.float64)
        out, _, grads = cuda_fwd_bwd(p, torch.float32)
        assert rel_err(out, o_ref) < FP32_TOL
        for a, b in zip(grads, g_ref):
            assert rel_err(a, b) < FP32_TOL


def test_crse_indices_bit_exact_including_clamp_quirk():
    import ctypes
    from swin3d_b200 import _lib
    from tests.gpu_helpers import dev
    p = make_problem(seed=21, n_voxels=900, grid=24, H=2, hd=8, crse="XYZ_RGB_NORM")
    nc = p.n_crse.copy()
    w = int(np.argmax(p.w_sizes))
    base, n = int(p.w2n[w]), int(p.w_sizes[w])
    # force differences of exactly +-2*quant*2 = +-16 in a colour and in the last normal dimension
    nc[base, 4], nc[base + 1, 4] = 8.0, -8.0
    nc[base, 8], nc[base + 1, 8] = 8.0, -8.0
    ref = O.crse_indices(nc, p.sizes, p.H, p.hd, base, n)
    assert ref[0, 1, 4] == 32 and ref[0, 1, 8] == 31
    out = torch.empty((n, n, p.D), dtype=torch.int32, device="cuda")
    arr = (ctypes.c_int32 * p.D)(*p.sizes)
    rc = _lib.lib.s3d_debug_crse_indices(dev(nc).data_ptr(), ctypes.cast(arr, ctypes.c_void_p), p.D,
                                         p.H, p.hd, base, n, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("dtype", ["fp32", "fp16"])
def test_index_equal_to_L_uses_next_dimension_row_zero(dtype):
    """With idx == L in a non-last dimension the flat table addressing of the reference selects
    row 0 of the next dimension; the kernels (generic fp32 path and tensor-core fp16 path, whose
    internal row numbering gives that case a private alias row) and the oracle must agree on it,
    row by row of the table gradients."""
    from tests.gpu_helpers import cuda_fwd_bwd
    half = dtype == "fp16"
    p = make_problem(seed=22, n_voxels=500, grid=20, H=2, hd=8, crse="XYZ_RGB", round_fp16=half)
    p.n_crse[::7, 3] = 8.0          # colour differences of exactly +-16: idx == L = 32 in dimension 3
    p.n_crse[3::7, 3] = -8.0
    idx = O.crse_indices(p.n_crse, p.sizes, p.H, p.hd, int(p.w2n[np.argmax(p.w_sizes)]), int(p.w_sizes.max()))
    assert (idx[:, :, 3] == 32).any()
    o_ref, _, g_ref = oracle_fwd_bwd(p, np.float64)
    out, _, grads = cuda_fwd_bwd(p, torch.float16 if half else torch.float32)
    tol = FP16_TOL if half else FP32_TOL
    assert rel_err(out, o_ref) < tol
    for a, b in zip(grads, g_ref):
        assert rel_err(a, b) < tol
    HC = p.H * p.hd
    for name, a, b in zip("dtq dtk dtv".split(), grads[3:], g_ref[3:]):
        assert table_row_errors(a, b, HC, tol, 2e-2 if half else 1e-3) == [], name
    # row 0 of dimension 4 (the row the alias stands for) carries gradient from the idx == L pairs:
    # with the dimension-3 signal flattened (no pair reaches L) it gets visibly less
    row0_dim4 = sum(p.sizes[:4]) // HC
    p2 = make_problem(seed=22, n_voxels=500, grid=20, H=2, hd=8, crse="XYZ_RGB", round_fp16=half)
    _, _, g_flat = oracle_fwd_bwd(p2, np.float64)
    r = slice(row0_dim4 * HC, (row0_dim4 + 1) * HC)
    assert np.abs(g_ref[5][r] - g_flat[5][r]).max() > 1e-3 * np.abs(g_ref[5]).max()
    assert np.abs(grads[5][r] - g_ref[5][r]).max() <= tol * np.abs(g_ref[5]).max()


def test_autograd_function_all_precision_modes():
    """The drop-in Function: gradients through torch.autograd, dtype policy of the reference."""
    from swin3d_b200.sparse_dl.attn.attn_coff import (SelfAttnAIOFunction, PosEmb, TableDims,
                                                      IndexMode, PrecisionMode)
    from tests.gpu_helpers import dev
    p = make_problem(seed=31, n_voxels=800, grid=24, H=6, hd=8, crse="XYZ_RGB", round_fp16=True)
    o_ref, _, g_ref = oracle_fwd_bwd(p, np.float64)
    x_off, y_off, m2w, ws64, w2n64, w2m = O.window_offsets(p.w_sizes)
    indices = [dev(m2w), dev(ws64), dev(w2m), dev(w2n64), dev(p.n2n.astype(np.int64)), dev(p.n_crse)]
    offsets = torch.IntTensor(p.sizes).cuda()
    for precision, autocast, tol in ((PrecisionMode.HALF_NONE, False, FP32_TOL),
                                     (PrecisionMode.HALF_NONE, True, FP32_TOL),
                                     (PrecisionMode.HALF_FORWARD, True, FP16_TOL),
                                     (PrecisionMode.HALF_ALL, True, FP16_TOL),
                                     (PrecisionMode.HALF_ALL, False, FP32_TOL)):
        q, k, v = (dev(a).requires_grad_() for a in (p.q, p.k, p.v))
        tq, tk, tv = (dev(a).requires_grad_() for a in (p.tq, p.tk, p.tv))
        with torch.autocast("cuda", dtype=torch.float16, enabled=autocast):
            out = SelfAttnAIOFunction.apply(q, k, v, tq, tk, tv, offsets, indices, PosEmb.SEPARATE,
                                            TableDims.D0, IndexMode.INDIRECT, precision)
        expect = torch.float16 if (autocast and precision != PrecisionMode.HALF_NONE) else torch.float32
        assert out.dtype == expect
        out.backward(dev(p.g).to(out.dtype))
        assert rel_err(out.detach().double().cpu().numpy(), o_ref) < tol
        for t, b in zip((q, k, v, tq, tk, tv), g_ref):
            assert t.grad is not None and t.grad.dtype == torch.float32
            assert rel_err(t.grad.double().cpu().numpy(), b) < tol


def test_half_forward_fast_backward_switch():
    """fp16_mode=1 with HALF_FORWARD_FAST_BACKWARD: the backward runs the tensor-core kernels on the
    forward's fp16 values and still returns fp32 gradients within the fp16 tolerance; off (the
    default) the backward is the fp32 one."""
    import swin3d_b200.sparse_dl.attn.attn_coff as C
    from tests.gpu_helpers import dev
    p = make_problem(seed=33, n_voxels=900, grid=24, H=6, hd=8, crse="XYZ_RGB_NORM", round_fp16=True)
    _, _, g_ref = oracle_fwd_bwd(p, np.float64)
    x_off, y_off, m2w, ws64, w2n64, w2m = O.window_offsets(p.w_sizes)
    indices = [dev(m2w), dev(ws64), dev(w2m), dev(w2n64), dev(p.n2n.astype(np.int64)), dev(p.n_crse)]
    offsets = torch.IntTensor(p.sizes).cuda()
    results = {}
    assert C.HALF_FORWARD_FAST_BACKWARD is False
    for fast in (False, True):
        C.HALF_FORWARD_FAST_BACKWARD = fast
        try:
            q, k, v = (dev(a).requires_grad_() for a in (p.q, p.k, p.v))
            tq, tk, tv = (dev(a).requires_grad_() for a in (p.tq, p.tk, p.tv))
            with torch.autocast("cuda", dtype=torch.float16):
                out = C.SelfAttnAIOFunction.apply(q, k, v, tq, tk, tv, offsets, indices, C.PosEmb.SEPARATE,
                                                  C.TableDims.D0, C.IndexMode.INDIRECT, C.PrecisionMode.HALF_FORWARD)
            out.backward(dev(p.g).half())
        finally:
            C.HALF_FORWARD_FAST_BACKWARD = False
        grads = [t.grad for t in (q, k, v, tq, tk, tv)]
        assert all(g.dtype == torch.float32 for g in grads)
        for g, b in zip(grads, g_ref):
            assert rel_err(g.double().cpu().numpy(), b) < FP16_TOL
        results[fast] = [g.clone() for g in grads]
    assert any(not torch.equal(a, b) for a, b in zip(results[False], results[True]))   # two different code paths


def test_empty_and_degenerate_inputs():
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device="cuda")
    sizes = [40 * 16] * 3
    out, lse = C.attn_forward_raw(z(0, 2, 8), z(0, 2, 8), z(0, 2, 8), z(1920), z(1920), z(1920), sizes,
                                  z(0, dt=torch.int32), z(0, dt=torch.int32), z(0, dt=torch.int32), z(0, 3))
    assert out.shape == (0, 2, 8) and lse.shape == (0, 2)
    with pytest.raises(ValueError):
        C.attn_forward_raw(z(4, 2, 12), z(4, 2, 12), z(4, 2, 12), z(2880), z(2880), z(2880), [960] * 3,
                           z(1, dt=torch.int32), z(1, dt=torch.int32), z(4, dt=torch.int32), z(4, 3))


def test_run_to_run_determinism_of_forward():
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=41, n_voxels=700, grid=22, H=2, hd=8, crse="XYZ_RGB")
    a = cuda_fwd_bwd(p)
    b = cuda_fwd_bwd(p)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for i in range(3):   # dq, dk, dv are owned by one thread each: bit-identical
        assert np.array_equal(a[2][i], b[2][i])


def _dense_scene():
    g = np.stack(np.meshgrid(*[np.arange(7)] * 3, indexing="ij"), -1).reshape(-1, 3)
    lonely = np.array([[40, 40, 40], [60, 3, 9], [90, 90, 90]])
    pts = np.concatenate([g, lonely])
    n = len(pts)
    rng = np.random.default_rng(5)
    return S.Scene(np.concatenate([np.zeros((n, 1)), pts], 1).astype(np.int32),
                   rng.random((n, 3), dtype=np.float32) * 0.999, rng.random((n, 3), dtype=np.float32),
                   np.tile(np.array([[0, 0, 1]], dtype=np.float32), (n, 1)))


@pytest.mark.parametrize("ws,crse,H", [(5, "XYZ_RGB_NORM", 10), (7, "XYZ_RGB_NORM", 2), (7, "XYZ", 4),
                                       (5, "XYZ_RGB", 6)])
def test_fp16_tensor_core_path_dense_and_tiny_windows(ws, crse, H):
    """fp16, head_dim 8: windows of 1, 125 and 343 voxels go through several query and key tiles
    of the tensor-core kernels."""
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=2, ws=ws, H=H, hd=8, crse=crse, scene=_dense_scene(), round_fp16=True)
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    out, lse, grads = cuda_fwd_bwd(p, torch.float16)
    assert rel_err(out, o_ref) < FP16_TOL
    assert np.abs(lse - lse_ref).max() < 2e-2
    for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
        assert rel_err(a, b) < FP16_TOL, name


def test_fp16_tensor_core_path_large_scores_stay_finite():
    """Scores of magnitude ~30 exercise the running-maximum rescale across key tiles."""
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=51, n_voxels=1500, grid=24, H=2, hd=8, crse="XYZ_RGB", round_fp16=True,
                     feat_scale=4.0)
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    out, lse, grads = cuda_fwd_bwd(p, torch.float16)
    assert np.isfinite(out).all() and np.isfinite(lse).all()
    assert rel_err(out, o_ref) < FP16_TOL
    assert np.abs(lse - lse_ref).max() < 5e-2


def test_room_scale_tensor_core_path_equals_generic_path():
    """A 60k-voxel room, Swin3D-L stage-1 head layout: the tensor-core kernels against the
    generic kernels of the same library (forced with s3d_debug_force_generic), same inputs."""
    import os
    from tests.gpu_helpers import cuda_fwd_bwd
    sc = S.make_room(7, target_voxels=60_000)
    p = make_problem(seed=61, ws=5, shift=2, H=10, hd=8, crse="XYZ_RGB_NORM", scene=sc, round_fp16=True)
    fast = cuda_fwd_bwd(p, torch.float16)
    _lib_force = __import__("swin3d_b200._lib", fromlist=["lib"]).lib.s3d_debug_force_generic(1)
    try:
        slow = cuda_fwd_bwd(p, torch.float16)
    finally:
        __import__("swin3d_b200._lib", fromlist=["lib"]).lib.s3d_debug_force_generic(0)
    assert rel_err(fast[0], slow[0]) < 5e-3
    assert np.abs(fast[1] - slow[1]).max() < 1e-2
    for a, b in zip(fast[2], slow[2]):
        assert rel_err(a, b) < 1.5e-2


def test_fp16_index_equal_to_L_alias_rows_and_determinism():
    """Opposite normals inside one window make idx == L reachable in a non-last dimension (the alias
    of the next dimension's row 0).  The tensor-core kernels give every dimension its own alias row,
    so outputs must match the oracle and repeat bit for bit from run to run."""
    from tests.gpu_helpers import cuda_fwd_bwd
    sc = S.make_room(7, target_voxels=20_000)
    p = make_problem(seed=61, ws=5, shift=2, H=10, hd=8, crse="XYZ_RGB_NORM", scene=sc, round_fp16=True)
    # colour differences of exactly +-16 as well (dimension 3 aliases dimension 4's row 0)
    p.n_crse[::11, 3] = 8.0
    p.n_crse[5::11, 3] = -8.0
    idx_hits = 0
    for w in np.argsort(-p.w_sizes)[:50]:
        ii = O.crse_indices(p.n_crse, p.sizes, p.H, p.hd, int(p.w2n[w]), int(p.w_sizes[w]))
        idx_hits += int((ii[:, :, 3] == 32).sum() + (ii[:, :, 6] == 32).sum())
    assert idx_hits > 0
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    a = cuda_fwd_bwd(p, torch.float16)
    b = cuda_fwd_bwd(p, torch.float16)
    assert rel_err(a[0], o_ref) < FP16_TOL
    for name, x, y in zip("dq dk dv".split(), a[2][:3], g_ref[:3]):
        assert rel_err(x, y) < FP16_TOL, name
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for i in range(3):
        assert np.array_equal(a[2][i], b[2][i])
    for i in range(3, 6):   # table gradients: fp32 atomics across blocks, order may differ
        assert rel_err(a[2][i], b[2][i]) < 1e-4


@pytest.mark.parametrize("crse,H,ws,shift", [("XYZ_RGB_NORM", 5, 5, 2), ("XYZ_RGB", 3, 5, 0), ("XYZ", 2, 7, 3),
                                             ("XYZ_RGB_NORM", 4, 7, 0), ("XYZ_RGB_NORM", 10, 7, 3), ("XYZ_RGB", 6, 5, 2)])
def test_fp16_head_dim_16_tensor_core_path(crse, H, ws, shift):
    """head_dim 16 (every stage but the first of the reference models).  Odd head counts: a block
    serves one head as two 8-channel halves; even head counts: a block serves two heads, their 16
    channels split into two planes.  Small and large windows."""
    from tests.gpu_helpers import cuda_fwd_bwd
    p = make_problem(seed=81, n_voxels=1500, grid=26, ws=ws, shift=shift, H=H, hd=16, crse=crse,
                     round_fp16=True)
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    out, lse, grads = cuda_fwd_bwd(p, torch.float16)
    assert rel_err(out, o_ref) < FP16_TOL
    assert np.abs(lse - lse_ref).max() < 2e-2
    for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
        assert rel_err(a, b) < FP16_TOL, name
    q = make_problem(seed=2, ws=ws, H=H, hd=16, crse=crse, scene=_dense_scene(), round_fp16=True)
    o_ref, _, g_ref = oracle_fwd_bwd(q, np.float64)
    out, _, grads = cuda_fwd_bwd(q, torch.float16)
    assert rel_err(out, o_ref) < FP16_TOL
    for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
        assert rel_err(a, b) < FP16_TOL, name


def test_sharded_attention_single_rank_equals_plain_call():
    """swin3d_b200.dist.sharded_attention without a process group: the window range is the whole
    list, the all-gather degenerates to the un-permutation through n2n."""
    import torch
    from swin3d_b200.dist import sharded_attention
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    p = make_problem(seed=31, n_voxels=3000, grid=40, H=4, hd=8, crse="XYZ_RGB_NORM")
    dev = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).cuda() if dt is None
                              else torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt))
    h = torch.float16
    q, k, v, g = (dev(x, h) for x in (p.q, p.k, p.v, p.g))
    tabs = [dev(x, h) for x in (p.tq, p.tk, p.tv)]
    ws, w2n, n2n = (dev(x.astype(np.int32)) for x in (p.w_sizes, p.w2n, p.n2n))
    ncr = dev(p.n_crse.astype(np.float32))
    sizes = [int(x) for x in p.sizes]
    out, dq, dk, dv, tg = sharded_attention(q, k, v, *tabs, sizes, ws, w2n, n2n, ncr, dout=g)
    o2, lse = C.attn_forward_raw(q, k, v, *tabs, sizes, ws, w2n, n2n, ncr)
    g2 = C.attn_backward_raw(q, k, v, *tabs, sizes, ws, w2n, n2n, ncr, o2, lse, g)
    assert torch.equal(out, o2)
    for a, b in zip((dq, dk, dv), g2[:3]):
        assert torch.equal(a, b)
    for a, b in zip(tg, g2[3:]):      # fp32 atomics: the order of the block flushes differs run to run
        assert float((a - b).abs().max()) <= 1e-5 * max(float(b.abs().max()), 1e-6)


def test_full_benchmark_size_properties():
    """The benchmark's full size (8 synthetic rooms, ~1 M voxels, 10 heads x 8, fp16), checked through
    properties that need no reference result:
      * value path is linear: out(v1 + v2) = out(v1) + out(v2), and with all value tables and v
        constant the output is that constant (probabilities sum to one);
      * the result does not depend on the order in which voxels are stored (a permutation of the
        rows, with n2n mapped accordingly, permutes the output rows);
      * dV sums: sum_k dV_k = sum_q dO_q when the value tables are zero (each row of p sums to one);
      * a sample of windows agrees with the CPU oracle."""
    import bench
    from swin3d_b200.window import build_windows
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    c = bench.CFG
    H, hd, ws, quant, crse = c["H"], c["hd"], c["ws"], c["quant"], c["crse"]
    sc = bench.make_batch(0, c["rooms"], c["voxels_per_room"])
    N = sc.coords.shape[0]
    assert N > 900_000
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    wi = build_windows(dev(sc.coords), dev(S.signal_feats(sc, crse)), ws, 0)
    ncr = wi.n_coords.clone()
    ncr[:, :3] *= quant
    ncr[:, 3:] *= 2 * quant
    sizes = S.table_sizes(ws, quant, H, hd, crse)
    gen = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda: torch.randn((N, H, hd), device="cuda", generator=gen).half()
    q, k, v1, v2, g = rnd() * hd ** -0.5, rnd(), rnd(), rnd(), rnd()
    tq, tk, tv = (dev(t).half() for t in S.make_tables(3, sizes))
    fwd = lambda vv, tvv, n2n=wi.n2n, qq=q, kk=k: C.attn_forward_raw(qq, kk, vv, tq, tk, tvv, sizes, wi.w_sizes, wi.w2n, n2n, ncr)
    zero_tv = torch.zeros_like(tv)
    o1, lse = fwd(v1, zero_tv)
    o2, _ = fwd(v2, zero_tv)
    o12, _ = fwd((v1.float() + v2.float()).half(), zero_tv)
    assert torch.isfinite(o1).all() and torch.isfinite(lse).all()
    lin = (o12.float() - o1.float() - o2.float()).abs().max().item()
    assert lin < 2e-2 * o12.float().abs().max().item()          # fp16 tolerance of the suite
    ones, _ = fwd(torch.full_like(v1, 0.5), zero_tv)
    assert (ones.float() - 0.5).abs().max().item() < 2e-3
    # storage-order independence
    perm = torch.randperm(N, device="cuda", generator=gen)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(N, device="cuda")
    n2n_p = inv[wi.n2n.long()].int()                             # sorted position -> row in the permuted arrays
    op, _ = C.attn_forward_raw(q[perm], k[perm], v1[perm], tq, tk, tv, sizes, wi.w_sizes, wi.w2n, n2n_p, ncr)
    of, lse_f = fwd(v1, tv)
    assert torch.equal(op, of[perm])
    # backward: column sums of p are carried by dV
    grads = C.attn_backward_raw(q, k, v1, tq, tk, zero_tv, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, o1, lse, g)
    dv_sum, g_sum = grads[2].double().sum(0), g.double().sum(0)
    assert (dv_sum - g_sum).abs().max().item() < 2e-3 * g.double().abs().sum(0).max().item()
    assert all(torch.isfinite(x).all() for x in grads)
    # a sample of windows against the oracle (the same rows, fp64 arithmetic)
    w_sizes, w2n, n2n = (x.cpu().numpy() for x in (wi.w_sizes, wi.w2n, wi.n2n))
    pick = np.linspace(0, len(w_sizes) - 1, 40).astype(np.int64)
    f64 = lambda t: t.double().cpu().numpy()
    o_ref, _, _ = O.attn_forward(f64(q), f64(k), f64(v1), f64(tq), f64(tk), f64(tv), sizes, w_sizes[pick],
                                 w2n[pick], n2n, ncr.cpu().numpy(), dtype=np.float64)
    rows = np.concatenate([n2n[w2n[w]:w2n[w] + w_sizes[w]] for w in pick])
    assert rel_err(f64(of)[rows], o_ref[rows]) < FP16_TOL
    # the BACKWARD of the same sample of windows: the library is run on exactly these windows (full-size
    # arrays, window list cut to the sample), so all six gradients are comparable with the oracle's
    o_s, s_s, m_s = O.attn_forward(f64(q), f64(k), f64(v1), f64(tq), f64(tk), f64(tv), sizes, w_sizes[pick],
                                   w2n[pick], n2n, ncr.cpu().numpy(), dtype=np.float64)
    g_ref = O.attn_backward(f64(q), f64(k), f64(v1), f64(tq), f64(tk), f64(tv), sizes, w_sizes[pick], w2n[pick],
                            n2n, ncr.cpu().numpy(), o_s, s_s, m_s, f64(g), dtype=np.float64)
    ws_s, w2n_s = dev(w_sizes[pick].astype(np.int32)), dev(w2n[pick].astype(np.int32))
    g_s = C.attn_backward_raw(q, k, v1, tq, tk, tv, sizes, ws_s, w2n_s, wi.n2n, ncr, of, lse_f, g)
    for name, a, b in zip("dq dk dv".split(), g_s[:3], g_ref[:3]):
        assert rel_err(f64(a)[rows], b[rows]) < FP16_TOL, name
    for name, a, b in zip("dtq dtk dtv".split(), g_s[3:], g_ref[3:]):
        assert rel_err(f64(a), b) < FP16_TOL, name
        assert table_row_errors(f64(a), b, H * hd, FP16_TOL, 2e-2) == [], name


def test_c_abi_calls_can_be_captured_in_a_cuda_graph():
    """s3d_attn_fwd / s3d_attn_bwd only enqueue kernels (and one memset) on the stream they are given:
    a forward + backward pair captured in a CUDA graph and replayed on new inputs gives the same
    results as direct calls."""
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    p = make_problem(seed=41, n_voxels=2500, grid=36, H=4, hd=8, crse="XYZ_RGB_NORM")
    dev = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).cuda() if dt is None
                              else torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt))
    h = torch.float16
    q, k, v, g = (dev(x, h) for x in (p.q, p.k, p.v, p.g))
    tabs = [dev(x, h) for x in (p.tq, p.tk, p.tv)]
    ws, w2n, n2n = (dev(x.astype(np.int32)) for x in (p.w_sizes, p.w2n, p.n2n))
    ncr = dev(p.n_crse.astype(np.float32))
    sizes = [int(x) for x in p.sizes]

    def run():
        out, lse = C.attn_forward_raw(q, k, v, *tabs, sizes, ws, w2n, n2n, ncr)
        return (out, lse) + tuple(C.attn_backward_raw(q, k, v, *tabs, sizes, ws, w2n, n2n, ncr, out, lse, g))

    run()                                   # warm-up outside the capture (function attributes, allocator)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            captured = run()
    # new inputs in the captured buffers, then replay
    gen = torch.Generator(device="cuda").manual_seed(9)
    q.copy_(torch.randn(q.shape, device="cuda", generator=gen).half() * 0.35)
    v.copy_(torch.randn(v.shape, device="cuda", generator=gen).half())
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in captured]
    direct = run()
    torch.cuda.synchronize()
    for name, a, b in zip("out lse dq dk dv".split(), replayed[:5], direct[:5]):
        assert torch.equal(a, b), name
    for a, b in zip(replayed[5:], direct[5:]):      # table gradients: fp32 atomics, order differs
        assert float((a - b).abs().max()) <= 1e-5 * max(float(b.abs().max()), 1e-6)


def test_tiled_kernels_work_list_overflow_falls_back_to_a_direct_walk():
    """150 heads leave one block per head pair, which then owns every tile of every window; nine
    dense 343-voxel windows give its first warp 99 work items, more than a list segment holds, so the
    kernels walk the chunk's windows directly.  Checked against the generic kernels of the library."""
    import os
    from tests.gpu_helpers import cuda_fwd_bwd
    g = np.stack(np.meshgrid(np.arange(21), np.arange(21), np.arange(7), indexing="ij"), -1).reshape(-1, 3)
    n = len(g)
    rng = np.random.default_rng(8)
    sc = S.Scene(np.concatenate([np.zeros((n, 1)), g], 1).astype(np.int32),
                 rng.random((n, 3), dtype=np.float32) * 0.999, rng.random((n, 3), dtype=np.float32),
                 np.tile(np.array([[0, 0, 1]], dtype=np.float32), (n, 1)))
    p = make_problem(seed=3, ws=7, H=150, hd=8, crse="XYZ", scene=sc, round_fp16=True)
    assert p.w_sizes.max() == 343 and len(p.w_sizes) == 9
    fast = cuda_fwd_bwd(p, torch.float16)
    _lib_force = __import__("swin3d_b200._lib", fromlist=["lib"]).lib.s3d_debug_force_generic(1)
    try:
        slow = cuda_fwd_bwd(p, torch.float16)
    finally:
        __import__("swin3d_b200._lib", fromlist=["lib"]).lib.s3d_debug_force_generic(0)
    assert rel_err(fast[0], slow[0]) < 5e-3
    for a, b in zip(fast[2], slow[2]):
        assert rel_err(a, b) < 1.5e-2


@pytest.mark.parametrize("H,hd,dtype", [(3, 8, "float32"), (1, 16, "float32"), (1, 32, "float32"), (3, 32, "float16")])
def test_generic_kernels_with_item_counts_that_do_not_fill_the_last_warp(H, hd, dtype):
    """The generic kernels deal (voxel, head) items to groups of lanes; with an odd number of items
    the groups past the end of the last warp repeat the last item without storing anything.  One
    voxel per window (the second case) is the other extreme of the item walk."""
    from tests.gpu_helpers import cuda_fwd_bwd
    tol = FP32_TOL if dtype == "float32" else FP16_TOL
    for seed, n_voxels, grid in ((31, 333, 18), (32, 7, 40), (33, 45, 18)):
        p = make_problem(seed=seed, n_voxels=n_voxels, grid=grid, H=H, hd=hd, crse="XYZ_RGB_NORM",
                         round_fp16=dtype == "float16")
        assert (p.N * H) % 2 == 1
        o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
        out, lse, grads = cuda_fwd_bwd(p, getattr(torch, dtype))
        assert rel_err(out, o_ref) < tol
        assert np.abs(lse - lse_ref).max() < (1e-4 if dtype == "float32" else 2e-2)
        # with one voxel per window dq, dk and two table gradients vanish identically (only rounding
        # of the stored output is left): measure against at least 1, the scale of the inputs
        for name, a, b in zip("dq dk dv dtq dtk dtv".split(), grads, g_ref):
            assert np.abs(a - b).max() / max(np.abs(b).max(), 1.0) < tol, name


def test_views_that_are_not_16_byte_aligned_are_copied_by_the_wrapper_and_refused_by_the_c_abi():
    import ctypes
    from swin3d_b200 import _lib
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    from tests.gpu_helpers import dev
    p = make_problem(seed=51, n_voxels=400, grid=20, H=2, hd=8, crse="XYZ", round_fp16=True)
    q, k, v, tq, tk, tv = (dev(a).half() for a in (p.q, p.k, p.v, p.tq, p.tk, p.tv))
    idx = [dev(a) for a in (p.w_sizes.astype(np.int32), p.w2n.astype(np.int32), p.n2n.astype(np.int32))]
    ncr = dev(p.n_crse)
    out0, lse0 = C.attn_forward_raw(q, k, v, tq, tk, tv, list(p.sizes), *idx, ncr)
    buf = torch.empty(q.numel() + 4, dtype=torch.float16, device="cuda")
    q_odd = buf[4:].view(q.shape)                     # starts 8 bytes into its storage
    q_odd.copy_(q)
    assert q_odd.data_ptr() % 16 == 8
    out1, lse1 = C.attn_forward_raw(q_odd, k, v, tq, tk, tv, list(p.sizes), *idx, ncr)
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    arr = (ctypes.c_int32 * 3)(*p.sizes)
    rc = _lib.lib.s3d_attn_fwd(q_odd.data_ptr(), k.data_ptr(), v.data_ptr(), tq.data_ptr(), tk.data_ptr(),
                               tv.data_ptr(), ctypes.cast(arr, ctypes.c_void_p), 3, idx[0].data_ptr(),
                               idx[1].data_ptr(), idx[2].data_ptr(), ncr.data_ptr(), p.N, len(p.w_sizes),
                               2, 8, _lib.S3D_F16, out1.data_ptr(),
                               lse1.data_ptr(), None)
    assert rc == 1
