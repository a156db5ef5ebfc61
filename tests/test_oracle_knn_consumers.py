"""CPU: the numpy restatements of the KNN consumers against vectors produced by the reference's
own Python (tests/golden/make_golden_knn_consumers.py)."""
import os

import numpy as np
import pytest

from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "knn_consumers_reference.npz"))


def _neighbours(K):
    idx, d2 = O.knn(K, G["src"], G["qry"], G["so"], G["qo"])
    return idx, np.sqrt(d2)


@pytest.mark.parametrize("tag,K", [("k3", 3), ("k5", 5)])
def test_interpolation_fp32_matches_reference(tag, K):
    idx, dist = _neighbours(K)
    out = O.knn_interpolate(idx, dist, G[f"interp.{tag}.feat"])
    ref = G[f"interp.{tag}.f32.out"]
    # same operations in the same order: equal to the last bit except where the reference's
    # reduction over K associates differently (K = 5)
    np.testing.assert_allclose(out, ref, rtol=2e-6, atol=1e-7)
    if K == 3:
        assert np.array_equal(out, ref)
    dsrc = O.knn_interpolate_bwd(idx, dist, G[f"interp.{tag}.dout"], G["src"].shape[0])
    np.testing.assert_allclose(dsrc, G[f"interp.{tag}.f32.dsrc"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("tag,K", [("k3", 3), ("k5", 5)])
def test_interpolation_fp16_matches_reference(tag, K):
    idx, dist = _neighbours(K)
    feat = G[f"interp.{tag}.feat"].astype(np.float16)
    out = O.knn_interpolate(idx, dist, feat).astype(np.float32)
    ref = G[f"interp.{tag}.f16.out"]
    np.testing.assert_allclose(out, ref, rtol=2e-3, atol=2e-3)
    assert np.mean(out == ref) > 0.99          # per-neighbour fp16 rounding reproduced
    dout = G[f"interp.{tag}.dout"].astype(np.float16)
    dsrc = O.knn_interpolate_bwd(idx, dist, dout, G["src"].shape[0])
    ref_d = G[f"interp.{tag}.f16.dsrc"]
    assert np.max(np.abs(dsrc - ref_d)) <= 2e-2 * max(1.0, np.max(np.abs(ref_d)))


def test_coincident_points_take_the_source_row():
    idx, dist = _neighbours(3)
    assert np.all(dist[:5, 0] == 0.0)
    out = O.knn_interpolate(idx, dist, G["interp.k3.feat"])
    np.testing.assert_allclose(out[:5], G["interp.k3.feat"][idx[:5, 0]], rtol=1e-5, atol=1e-6)


def _layer_norm_linear(x, w, b, lw):
    mu = x.mean(1, keepdims=True)
    var = ((x - mu) ** 2).mean(1, keepdims=True)
    return ((x - mu) / np.sqrt(var + 1e-5) * w + b) @ lw.T


def test_maxpool_commutes_with_norm_and_linear():
    idx, _ = _neighbours(16)
    g = _layer_norm_linear(G["down.feat"].astype(np.float64), G["down.norm_w"], G["down.norm_b"], G["down.lin_w"])
    out, arg = O.knn_maxpool(idx, g.astype(np.float32))
    np.testing.assert_allclose(out, G["down.out"], rtol=1e-5, atol=1e-5)
    assert arg.shape == out.shape and np.all((arg >= 0) & (arg < g.shape[0]))
    # every arg is one of the query's neighbours
    assert np.all((arg[:, None, :] == idx[:, :, None]).any(axis=1))
    dg = O.knn_maxpool_bwd(arg, G["down.dout"], g.shape[0])
    assert np.isclose(dg.sum(), G["down.dout"].sum(), rtol=1e-5)


def test_maxpool_first_maximum_wins():
    idx = np.array([[2, 0, 1]], dtype=np.int32)
    g = np.array([[1.0, 5.0], [1.0, 5.0], [1.0, 4.0]], dtype=np.float32)
    out, arg = O.knn_maxpool(idx, g)
    assert out.tolist() == [[1.0, 5.0]] and arg.tolist() == [[2, 0]]
