"""CPU: the oracle against outputs of the reference's own compiled CUDA kernels, recorded on a
B200 by tests/golden/make_golden_ref_gpu.py and committed as tests/golden/ref_gpu_golden.npz.
Inputs are regenerated from the same seeds.  fp64: 1e-10; fp32: 1e-4; fp16: 2e-2 (the reference
computes fp16 products, sums and output accumulation in half precision); KNN bit-exact."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests.golden import make_golden_ref_gpu as G
from tests.helpers import make_problem, oracle_fwd_bwd, rel_err

PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_gpu_golden.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(PATH), reason="fixture not recorded yet")
TOL = {"float32": 1e-4, "float64": 1e-10, "float16": 2e-2}


@pytest.mark.parametrize("name", [n for n in G.GOLDEN if n in G.ATTN_CASES])
def test_oracle_matches_recorded_reference_attention(name):
    g = np.load(PATH)
    c = G.ATTN_CASES[name]
    p = make_problem(**c["kw"])
    out, lse, grads = oracle_fwd_bwd(p, np.float64)
    tol = TOL[c["dtype"]]
    assert rel_err(out, g[f"{name}.norm"]) < tol
    lse_r = g[f"{name}.max"].astype(np.float64)[..., 0] + np.log(g[f"{name}.sum"].astype(np.float64)[..., 0])
    assert np.abs(lse - lse_r).max() < max(10 * tol, 1e-9)
    for key, a in zip("dq dk dv dtq dtk dtv".split(), grads):
        assert rel_err(a, g[f"{name}.{key}"]) < tol, key


@pytest.mark.parametrize("name", [n for n in G.GOLDEN if n in G.KNN_CASES])
def test_oracle_matches_recorded_reference_knn(name):
    g = np.load(PATH)
    c = G.KNN_CASES[name]
    src, qry, so, qo = G.knn_inputs(c["seed"])
    idx, d2 = O.knn(c["K"], src, qry, so, qo)
    assert np.array_equal(idx, g[f"{name}.idx"])
    assert np.array_equal(d2.view(np.uint32), g[f"{name}.d2"].view(np.uint32))
