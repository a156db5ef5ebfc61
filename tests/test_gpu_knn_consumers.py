"""GPU parity of the KNN consumers (through the C-ABI): inverse-distance interpolation and the
neighbourhood max-pool, against the numpy oracle, against vectors from the reference's own Python,
and against the unfused torch formulation of the reference on the same device."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "knn_consumers_reference.npz"))


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _scene():
    return _dev(G["src"]), _dev(G["qry"]), _dev(G["so"]), _dev(G["qo"])


@pytest.mark.parametrize("tag,K", [("k3", 3), ("k5", 5)])
def test_interpolation_fp32_bit_exact_vs_oracle_and_reference(tag, K):
    from swin3d_b200.sparse_dl.knn import knn_linear_interpolation
    src, qry, so, qo = _scene()
    feat = _dev(G[f"interp.{tag}.feat"]).requires_grad_(True)
    out = knn_linear_interpolation(src, qry, feat, so, qo, K=K)
    out.backward(_dev(G[f"interp.{tag}.dout"]))
    idx, d2 = O.knn(K, G["src"], G["qry"], G["so"], G["qo"])
    ref = O.knn_interpolate(idx, np.sqrt(d2), G[f"interp.{tag}.feat"])
    assert np.array_equal(out.detach().cpu().numpy(), ref)                # same operation order
    np.testing.assert_allclose(out.detach().cpu().numpy(), G[f"interp.{tag}.f32.out"], rtol=2e-6, atol=1e-7)
    # tolerance of the gradient: fp32 sums in a different order (atomics), 1e-5 relative
    np.testing.assert_allclose(feat.grad.cpu().numpy(), G[f"interp.{tag}.f32.dsrc"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("tag,K", [("k3", 3), ("k5", 5)])
def test_interpolation_fp16(tag, K):
    from swin3d_b200.sparse_dl.knn import knn_linear_interpolation
    src, qry, so, qo = _scene()
    feat = _dev(G[f"interp.{tag}.feat"]).half().requires_grad_(True)
    out = knn_linear_interpolation(src, qry, feat, so, qo, K=K)
    out.backward(_dev(G[f"interp.{tag}.dout"]).half())
    idx, d2 = O.knn(K, G["src"], G["qry"], G["so"], G["qo"])
    ref = O.knn_interpolate(idx, np.sqrt(d2), G[f"interp.{tag}.feat"].astype(np.float16))
    assert np.array_equal(out.detach().cpu().numpy(), ref)                # rounding after every neighbour
    ref_d = G[f"interp.{tag}.f16.dsrc"]
    err = np.max(np.abs(feat.grad.float().cpu().numpy() - ref_d))
    assert err <= 2e-2 * max(1.0, np.max(np.abs(ref_d)))                  # fp16 tolerance of the suite


def test_interpolation_matches_unfused_torch_on_large_input():
    """The reference's formulation (swin3d_layers.py:64-72) evaluated with torch ops on the GPU."""
    from swin3d_b200.sparse_dl.knn import KNN, KNNInterpolate
    g = torch.Generator(device="cuda").manual_seed(5)
    Ns, Nq, C, K = 20_000, 60_000, 96, 3
    src = torch.rand(Ns, 3, device="cuda", generator=g) * 10
    qry = torch.rand(Nq, 3, device="cuda", generator=g) * 10
    so = torch.tensor([Ns], dtype=torch.int32, device="cuda")
    qo = torch.tensor([Nq], dtype=torch.int32, device="cuda")
    feat = torch.randn(Ns, C, device="cuda", generator=g, requires_grad=True)
    idx, dist = KNN.apply(K, src, qry, so, qo)
    out = KNNInterpolate.apply(feat, idx, dist)
    dout = torch.randn(Nq, C, device="cuda", generator=g)
    out.backward(dout)
    mine, feat.grad = feat.grad.clone(), None
    weight = 1.0 / (dist + 1e-8)
    weight = weight / torch.sum(weight, dim=1, keepdim=True)
    ref = torch.zeros((Nq, C), dtype=feat.dtype, device="cuda")
    for i in range(K):
        ref = ref + feat[idx[:, i].long(), :] * weight[:, i].unsqueeze(-1)
    ref.backward(dout)
    # torch's own kernels may associate the sum over K and round the division differently: last-bit tolerance
    assert torch.allclose(out, ref, rtol=2e-6, atol=1e-6)
    assert torch.allclose(mine, feat.grad, rtol=1e-4, atol=1e-5)
    # linearity in the features: interpolating a constant field returns the constant
    ones = KNNInterpolate.apply(torch.ones(Ns, 8, device="cuda"), idx, dist)
    assert torch.allclose(ones, torch.ones_like(ones), atol=1e-6)


def test_interpolation_argument_errors():
    from swin3d_b200.sparse_dl.knn import KNNInterpolate
    idx = torch.zeros((4, 3), dtype=torch.int32, device="cuda")
    dist = torch.ones((4, 3), device="cuda")
    with pytest.raises(ValueError):
        KNNInterpolate.apply(torch.ones(5, 6, device="cuda"), idx, dist)        # C not a multiple of 4
    with pytest.raises(ValueError):
        KNNInterpolate.apply(torch.ones(5, 8, device="cuda").double(), idx, dist)
    empty = KNNInterpolate.apply(torch.ones(5, 8, device="cuda"), idx[:0], dist[:0])
    assert empty.shape == (0, 8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_maxpool_vs_oracle(dtype):
    from swin3d_b200.sparse_dl.knn import KNN, KNNMaxPool
    src, qry, so, qo = _scene()
    K = 16
    rng = np.random.default_rng(11)
    g_np = rng.normal(size=(G["src"].shape[0], 40)).astype(np.float32)
    g_np[:, :4] = np.round(g_np[:, :4])                    # ties: the first maximum must win
    g = _dev(g_np).to(dtype).requires_grad_(True)
    idx, _ = KNN.apply(K, src, qry, so, qo)
    out, arg = KNNMaxPool.apply(g, idx)
    dout_np = rng.normal(size=tuple(out.shape)).astype(np.float32)
    out.backward(_dev(dout_np).to(dtype))
    oidx, _ = O.knn(K, G["src"], G["qry"], G["so"], G["qo"])
    ref_out, ref_arg = O.knn_maxpool(oidx, g.detach().cpu().numpy())
    assert np.array_equal(out.detach().cpu().numpy(), ref_out)
    assert np.array_equal(arg.cpu().numpy(), ref_arg)
    ref_dg = O.knn_maxpool_bwd(ref_arg, _dev(dout_np).to(dtype).float().cpu().numpy(), g.shape[0])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.max(np.abs(g.grad.float().cpu().numpy() - ref_dg)) <= tol * max(1.0, np.max(np.abs(ref_dg)))


def test_downsample_tail_matches_reference_vectors():
    """gather + LayerNorm + Linear + MaxPool1d(16) of GridKNNDownsample.forward, evaluated as
    LayerNorm + Linear per source row followed by the fused neighbourhood max-pool."""
    from swin3d_b200.sparse_dl.knn import knn_max_pool
    src, qry, so, qo = _scene()
    feat = _dev(G["down.feat"]).requires_grad_(True)
    norm = torch.nn.LayerNorm(feat.shape[1]).cuda()
    linear = torch.nn.Linear(feat.shape[1], G["down.lin_w"].shape[0], bias=False).cuda()
    with torch.no_grad():
        norm.weight.copy_(_dev(G["down.norm_w"]))
        norm.bias.copy_(_dev(G["down.norm_b"]))
        linear.weight.copy_(_dev(G["down.lin_w"]))
    out = knn_max_pool(16, src, qry, linear(norm(feat)), so, qo)      # fp32 GEMM (TF32 is off by default)
    out.backward(_dev(G["down.dout"]))
    np.testing.assert_allclose(out.detach().cpu().numpy(), G["down.out"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(feat.grad.cpu().numpy(), G["down.dfeat"], rtol=1e-3, atol=1e-4)
