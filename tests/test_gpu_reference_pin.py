"""GPU: the CPU oracle AND the CUDA library against the reference's own compiled CUDA kernels
(oracle/_ref/ref_swin3d_cuda.so, built from the sources of microsoft/Swin3D by
oracle/build_ref.py) on identical inputs.  Skipped when that build is absent.

fp32: 1e-4 relative; fp64 oracle vs fp64 reference: 1e-10; fp16: 2e-2; KNN indices and
distances bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.golden import make_golden_ref_gpu as G
from tests.helpers import make_problem, oracle_fwd_bwd, rel_err

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "float64": 1e-10, "float16": 2e-2}


@pytest.fixture(scope="module")
def ref():
    mod = G.load_ref()
    if mod is None:
        pytest.skip("reference kernels not built (python oracle/build_ref.py)")
    return mod


@pytest.mark.parametrize("name", list(G.ATTN_CASES))
def test_reference_kernels_vs_oracle_and_library(ref, name):
    from tests.gpu_helpers import cuda_fwd_bwd
    c = G.ATTN_CASES[name]
    p = make_problem(**c["kw"])
    r = G.run_ref_attention(ref, p, c["dtype"])
    tol = TOL[c["dtype"]]
    o_ref, lse_ref, g_ref = oracle_fwd_bwd(p, np.float64)
    assert rel_err(r["norm"], o_ref) < tol
    lse_r = r["max"].astype(np.float64)[..., 0] + np.log(r["sum"].astype(np.float64)[..., 0])
    assert np.abs(lse_r - lse_ref).max() < max(tol, 1e-10) * 10
    for key, b in zip("dq dk dv dtq dtk dtv".split(), g_ref):
        assert rel_err(r[key], b) < tol, key
    if c["dtype"] != "float64":
        out, lse, grads = cuda_fwd_bwd(p, getattr(torch, c["dtype"]))
        assert rel_err(out, r["norm"]) < tol
        for key, a in zip("dq dk dv dtq dtk dtv".split(), grads):
            assert rel_err(a, r[key]) < tol, key


@pytest.mark.parametrize("name", list(G.KNN_CASES))
def test_reference_knn_bit_exact(ref, name):
    from swin3d_b200.sparse_dl.knn.knn import knn_raw
    c = G.KNN_CASES[name]
    src, qry, so, qo = G.knn_inputs(c["seed"])
    ridx, rd2 = G.run_ref_knn(ref, c["K"], src, qry, so, qo)
    oidx, od2 = O.knn(c["K"], src, qry, so, qo, fma_mode=2)
    assert np.array_equal(rd2.view(np.uint32), od2.view(np.uint32)), "fp32 distance bits differ"
    assert np.array_equal(ridx, oidx)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    idx, d2 = knn_raw(c["K"], d(src), d(qry), d(so), d(qo))
    assert np.array_equal(idx.cpu().numpy(), ridx)
    assert np.array_equal(d2.cpu().numpy().view(np.uint32), rd2.view(np.uint32))
