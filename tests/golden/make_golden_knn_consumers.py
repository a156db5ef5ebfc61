"""Generates tests/golden/knn_consumers_reference.npz by running the reference's own Python code
for the callers of KNN on CPU tensors:
  * knn_linear_interpolation            (Swin3D/modules/swin3d_layers.py:53-73), fp32 and fp16,
    forward and the autograd gradient w.r.t. src_feat;
  * query_knn_feature + LayerNorm + Linear(bias=False) + MaxPool1d(16), the tail of
    GridKNNDownsample.forward (swin3d_layers.py:302-309), forward and gradient w.r.t. sp.F.
Only the CUDA KNN search itself is replaced: `KNN.apply` returns the neighbours found by the C
oracle (oracle/swin3d_oracle.c: orc_knn, itself pinned bit-exactly to the reference's CUDA kernel),
with the same sqrt as Swin3D/sparse_dl/knn/knn.py:25.
Usage: python tests/golden/make_golden_knn_consumers.py [reference_root]
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from make_golden_offsets import import_reference  # noqa: E402
from oracle import oracle as O  # noqa: E402


class OracleKNN:
    """Stands in for Swin3D.sparse_dl.knn.KNN: same outputs, neighbours from the C oracle."""

    @staticmethod
    def apply(K, src_xyz, query_xyz, src_offset, query_offset):
        idx, d2 = O.knn(K, src_xyz.numpy(), query_xyz.numpy(), src_offset.numpy(), query_offset.numpy())
        # correctly rounded sqrt, as torch.sqrt on a CUDA tensor (torch's vectorised CPU sqrt is
        # 1 ulp off for some inputs)
        return torch.from_numpy(idx), torch.from_numpy(np.sqrt(d2))


def scene(rng, ns, nq):
    src = rng.uniform(0, 4, size=(ns, 3)).astype(np.float32)
    qry = rng.uniform(0, 4, size=(nq, 3)).astype(np.float32)
    return src, qry


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SWIN3D_REFERENCE")
    if not root:
        raise SystemExit("usage: python " + sys.argv[0] + " <reference_root>   (or set SWIN3D_REFERENCE)")
    layers, _ = import_reference(root)
    layers.KNN = OracleKNN
    rng = np.random.default_rng(7)
    out = {}
    # two scenes; a few queries coincide with a source point (distance 0 -> weight 1e8)
    s0, q0 = scene(rng, 150, 70)
    s1, q1 = scene(rng, 130, 50)
    q0[:5] = s0[:5]
    src = np.concatenate([s0, s1]); qry = np.concatenate([q0, q1])
    so = np.array([150, 280], dtype=np.int32); qo = np.array([70, 120], dtype=np.int32)
    out["src"], out["qry"], out["so"], out["qo"] = src, qry, so, qo
    for K, C, tag in ((3, 32, "k3"), (5, 16, "k5")):
        feat = rng.normal(size=(src.shape[0], C)).astype(np.float32)
        dout = rng.normal(size=(qry.shape[0], C)).astype(np.float32)
        out[f"interp.{tag}.feat"], out[f"interp.{tag}.dout"] = feat, dout
        for dt, name in ((torch.float32, "f32"), (torch.float16, "f16")):
            f = torch.from_numpy(feat).to(dt).requires_grad_(True)
            y = layers.knn_linear_interpolation(torch.from_numpy(src), torch.from_numpy(qry), f,
                                                torch.from_numpy(so), torch.from_numpy(qo), K=K)
            y.backward(torch.from_numpy(dout).to(y.dtype))
            out[f"interp.{tag}.{name}.out"] = y.detach().float().numpy()
            out[f"interp.{tag}.{name}.dsrc"] = f.grad.float().numpy()
    # GridKNNDownsample tail, K = 16
    K, Cin, Cout = 16, 24, 32
    torch.manual_seed(3)
    norm = torch.nn.LayerNorm(Cin)
    linear = torch.nn.Linear(Cin, Cout, bias=False)
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
        norm.bias.uniform_(-0.2, 0.2)
    pool = torch.nn.MaxPool1d(K)
    feat = torch.from_numpy(rng.normal(size=(src.shape[0], Cin)).astype(np.float32)).requires_grad_(True)
    dout = torch.from_numpy(rng.normal(size=(qry.shape[0], Cout)).astype(np.float32))
    feats = layers.query_knn_feature(K, torch.from_numpy(src), torch.from_numpy(qry), feat,
                                     torch.from_numpy(so), torch.from_numpy(qo))
    m, k, c = feats.shape
    feats = linear(norm(feats.view(m * k, c)).view(m, k, c)).transpose(1, 2).contiguous()
    y = pool(feats).squeeze(-1)
    y.backward(dout)
    out["down.feat"], out["down.dout"] = feat.detach().numpy(), dout.numpy()
    out["down.norm_w"], out["down.norm_b"] = norm.weight.detach().numpy(), norm.bias.detach().numpy()
    out["down.lin_w"] = linear.weight.detach().numpy()
    out["down.out"], out["down.dfeat"] = y.detach().numpy(), feat.grad.numpy()
    dst = os.path.join(HERE, "knn_consumers_reference.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
