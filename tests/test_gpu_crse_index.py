"""Bit-exact check of the cRSE index function of EVERY kernel family against the oracle
(microsoft/Swin3D, Swin3D/src/attn/attn_utils.cuh:444-450): the generic kernels (variant 0), the
tiled tensor-core kernels (variant 1) and the single-tile tensor-core kernels (variant 2)."""
import ctypes

import numpy as np
import pytest

from tests import helpers  # noqa: F401  (path set-up)

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _reference_index(cq, ck, L, last):
    """numpy restatement: fp32 subtract, add L/2, clamp to [0, (float)(L - 1e-10)] = [0, L], truncate;
    NaN goes through fmaxf(0, NaN) = 0."""
    with np.errstate(invalid="ignore", over="ignore"):
        rel = (cq.astype(np.float32) - ck.astype(np.float32)).astype(np.float32)
        rel = (rel + np.float32(L // 2)).astype(np.float32)
        rel = np.fmin(np.fmax(np.float32(0.0), rel), np.float32(np.float64(L) - 1e-10))
        idx = rel.astype(np.int64)
    if last:
        idx = np.minimum(idx, L - 1)
    return idx.astype(np.int32)


def _special_values(L):
    f = np.float32
    vals = []
    for b in range(-L - 3, 2 * L + 4):            # every integer boundary from -L to 2L, +-1 ulp
        x = f(b)
        vals += [x, np.nextafter(x, f(np.inf)), np.nextafter(x, f(-np.inf))]
    for b in range(-4, 5):                         # quarter steps and tiny values near zero
        vals += [f(b * 0.25), f(b * 1e-7), f(b * 2.0 ** -24)]
    vals += [f(np.nan), f(np.inf), f(-np.inf), f(1e30), f(-1e30), f(3e38), f(-3e38),
             f(1e-45), f(-1e-45), f(2.0 ** 31), f(2.0 ** 32), f(-2.0 ** 31), f(0.0), f(-0.0)]
    return np.array(vals, dtype=np.float32)


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("L", [32, 40, 56])
@pytest.mark.parametrize("last", [0, 1])
def test_index_function_bit_exact_on_boundary_values(variant, L, last):
    from swin3d_b200 import _lib
    vals = _special_values(L)
    rng = np.random.default_rng(5)
    other = np.concatenate([np.array([0.0, 0.25, 0.5, -0.75, L / 2, -L / 2, 1e-3], dtype=np.float32),
                            rng.uniform(-L, L, size=57).astype(np.float32)])
    cq = np.repeat(vals, other.size)
    ck = np.tile(other, vals.size)
    cq, ck = np.concatenate([cq, ck]), np.concatenate([ck, cq])     # special values on both sides
    ref = _reference_index(cq, ck, L, last)
    d_cq, d_ck = torch.from_numpy(cq).cuda(), torch.from_numpy(ck).cuda()
    out = torch.empty(cq.size, dtype=torch.int32, device="cuda")
    rc = _lib.lib.s3d_debug_crse_index_values(d_cq.data_ptr(), d_ck.data_ptr(), cq.size, L, last, variant,
                                              out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    bad = np.nonzero(got != ref)[0]
    assert bad.size == 0, (variant, L, last, cq[bad[:5]], ck[bad[:5]], got[bad[:5]], ref[bad[:5]])


@pytest.mark.parametrize("variant", [0, 1, 2])
def test_window_dump_matches_the_oracle_including_clamp_quirk(variant):
    from oracle import oracle as O
    from swin3d_b200 import _lib
    from tests.gpu_helpers import dev
    from tests.helpers import make_problem
    p = make_problem(seed=21, n_voxels=900, grid=24, H=2, hd=8, crse="XYZ_RGB_NORM")
    nc = p.n_crse.copy()
    w = int(np.argmax(p.w_sizes))
    base, n = int(p.w2n[w]), int(p.w_sizes[w])
    nc[base, 4], nc[base + 1, 4] = 8.0, -8.0       # +-16 in a colour dimension: idx == L
    nc[base, 8], nc[base + 1, 8] = 8.0, -8.0       # and in the last dimension: clamped to L - 1
    nc[base + 2, 0] = np.float32(np.nan)
    nc[base + 3, 1] = np.float32(np.inf)
    ref = O.crse_indices(nc, p.sizes, p.H, p.hd, base, n)
    assert ref[0, 1, 4] == 32 and ref[0, 1, 8] == 31
    out = torch.empty((n, n, p.D), dtype=torch.int32, device="cuda")
    arr = (ctypes.c_int32 * p.D)(*p.sizes)
    rc = _lib.lib.s3d_debug_crse_indices_variant(dev(nc).data_ptr(), ctypes.cast(arr, ctypes.c_void_p), p.D,
                                                 p.H, p.hd, base, n, variant, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), ref)
