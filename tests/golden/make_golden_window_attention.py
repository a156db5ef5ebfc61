"""Generates tests/golden/window_attention_reference.npz by running the reference's own
``WindowAttention`` module and its own ``SelfAttnAIOFunction`` (microsoft/Swin3D,
Swin3D/modules/swin3d_layers.py:382-575 and Swin3D/sparse_dl/attn/attn_coff.py:155-232), UNCHANGED,
on CPU tensors.

The reference's Python cannot travel to a GPU box and its CUDA extension cannot run without a GPU, so
the module is executed here with
  * MinkowskiEngine / timm replaced by stub modules (nothing of them is on this path),
  * ``Swin3D.sparse_dl.attn_cuda`` replaced by a module that implements the four pybind entry points
    the Function calls (cal_max_coffs, self_attn_forward, cal_exp_sum_grads, self_attn_indir_backward,
    Swin3D/src/attn/attn_api.cpp:20-24) with the C oracle of this repository, which is pinned to the
    reference's compiled CUDA kernels (tests/golden/ref_gpu_golden.npz),
  * ``Tensor.cuda`` made a no-op for the duration of the run (swin3d_layers.py:511 moves the table
    offsets to the GPU).
Recorded: the module's parameters, its inputs (features and the eight attention arguments exactly as
the module receives them, int64 indices included), every argument the module hands to
``SelfAttnAIOFunction.apply``, the module output and the gradients of features and parameters for an
upstream gradient.  tests/test_gpu_window_attention.py replays the recorded call through this
repository's drop-in Function on a GPU and rebuilds the module output around it.

Usage: python tests/golden/make_golden_window_attention.py <reference_root> [output.npz]
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def oracle_attn_cuda():
    """A stand-in for the pybind module ``attn_cuda`` on top of the C oracle (fp64 arithmetic)."""
    from oracle import oracle as O
    m = types.ModuleType("Swin3D.sparse_dl.attn_cuda")
    f64 = lambda t: t.detach().cpu().numpy().astype(np.float64)

    def _unpack(indices):
        m2w, w_sizes, w2m, w2n, n2n, n_crse = indices
        return (w_sizes.numpy().astype(np.int32), w2n.numpy().astype(np.int32), n2n.numpy().astype(np.int32),
                n_crse.detach().numpy().astype(np.float32))

    def _fwd(qkv, tabs, sizes, indices):
        ws, w2n, n2n, nc = _unpack(indices)
        return O.attn_forward(*(f64(x) for x in qkv), *(f64(x) for x in tabs), [int(x) for x in sizes.tolist()],
                              ws, w2n, n2n, nc, dtype=np.float64)

    def cal_max_coffs(qkv, tabs, sizes, indices, mode, pe):
        assert mode == 2 and pe == 3
        _, _, mx = _fwd(qkv, tabs, sizes, indices)
        return torch.from_numpy(mx.astype(np.float32))[..., None]

    def self_attn_forward(qkv, tabs, coff_rmax, sizes, indices, mode, pe):
        out, s, _ = _fwd(qkv, tabs, sizes, indices)
        dt = qkv[0].dtype
        s_t = torch.from_numpy(s)[..., None]
        return [(torch.from_numpy(out) * s_t).to(dt), s_t.to(dt)]      # raw = norm * sum, sum [N,H,1]

    state = {}

    def cal_exp_sum_grads(grads, raw, sums, v, tv):
        # the oracle's backward computes this term itself; hand the pieces on through the next call
        state["raw"], state["sums"] = raw, sums
        return torch.zeros(raw.shape[:2], dtype=raw.dtype)

    def self_attn_indir_backward(grads, exp_sum_grads, raw, sums, rmax, q, k, v, tq, tk, tv, sizes, indices, mode, pe):
        ws, w2n, n2n, nc = _unpack(indices)
        out = f64(raw) / f64(sums)
        g = O.attn_backward(f64(q), f64(k), f64(v), f64(tq), f64(tk), f64(tv), [int(x) for x in sizes.tolist()],
                            ws, w2n, n2n, nc, out, f64(sums)[..., 0], f64(rmax)[..., 0].astype(np.float32),
                            f64(grads), dtype=np.float64)
        return [torch.from_numpy(x).to(q.dtype) for x in g]

    m.cal_max_coffs, m.self_attn_forward = cal_max_coffs, self_attn_forward
    m.cal_exp_sum_grads, m.self_attn_indir_backward = cal_exp_sum_grads, self_attn_indir_backward
    return m


def import_reference(root):
    def stub(name, **attrs):
        mod = types.ModuleType(name)
        mod.__dict__.update(attrs)
        sys.modules[name] = mod
        return mod

    class _Any:
        def __init__(self, *a, **k):
            pass

    me = stub("MinkowskiEngine", SparseTensor=_Any)
    for n in ("MinkowskiMaxPooling", "MinkowskiAvgPooling", "MinkowskiPoolingTranspose", "MinkowskiConvolution",
              "MinkowskiBatchNorm", "MinkowskiReLU", "MinkowskiLinear", "MinkowskiNetwork"):
        setattr(me, n, _Any)
    stub("timm")
    stub("timm.models")
    stub("timm.models.layers", DropPath=torch.nn.Identity, trunc_normal_=torch.nn.init.trunc_normal_)
    sys.path.insert(0, root)
    sys.modules["Swin3D.sparse_dl.attn_cuda"] = oracle_attn_cuda()
    stub("Swin3D.sparse_dl.knn_cuda")
    import Swin3D.modules.swin3d_layers as layers
    import Swin3D.sparse_dl.attn.attn_coff as coff
    import Swin3D.sparse_dl as sdl
    sdl.attn_cuda = sys.modules["Swin3D.sparse_dl.attn_cuda"]
    return layers, coff


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    root = sys.argv[1]
    out_path = sys.argv[2] if len(sys.argv) > 2 else os.path.join(HERE, "window_attention_reference.npz")
    layers, coff = import_reference(root)
    from oracle import oracle as O
    from swin3d_b200 import synthetic as S

    captured = {}
    real_apply = coff.SelfAttnAIOFunction.apply

    def spy(*args):
        captured["args"] = args
        return real_apply(*args)

    layers.SelfAttnAIOFunction = types.SimpleNamespace(apply=spy)
    out = {}
    torch.manual_seed(0)
    ws, quant, heads, dim = 5, 4, 6, 48
    # without autocast (CPU) the three fp16 modes of the module run the same fp32 arithmetic and differ
    # only in the PrecisionMode they pass on, so two recorded cases cover them
    for tag, crse, fp16_mode in (("rgb_m0", "XYZ_RGB", 0), ("norm_m2", "XYZ_RGB_NORM", 2)):
        scene = S.make_planes_and_boxes(3, 320, 20)
        feats_sig = S.signal_feats(scene, crse)
        n2n, n_coords, w_sizes, w2n = O.window_grouping(scene.coords, feats_sig, ws, 0)
        x_off, y_off, m2w, w, w2n64, w2m = O.window_offsets(w_sizes)
        attn_args = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in
                          (x_off, y_off, m2w, w, w2n64, n2n.astype(np.int64), w2m, n_coords))
        mod = layers.WindowAttention(dim, ws, quant, heads, cRSE=crse, fp16_mode=fp16_mode)
        feats = torch.randn(scene.coords.shape[0], dim, dtype=torch.float32, requires_grad=True)
        upstream = torch.randn(scene.coords.shape[0], dim, dtype=torch.float32)
        saved_cuda = torch.Tensor.cuda
        torch.Tensor.cuda = lambda self, *a, **k: self
        try:
            y = mod(feats, attn_args)
            y.backward(upstream)
        finally:
            torch.Tensor.cuda = saved_cuda
        a = captured["args"]
        out[f"{tag}.crse"] = np.array(crse)
        out[f"{tag}.fp16_mode"] = np.array(fp16_mode)
        out[f"{tag}.feats"] = feats.detach().numpy()
        out[f"{tag}.upstream"] = upstream.numpy()
        # x_offset, y_offset and m2w (one int64 per attention pair) are rebuilt by the test from w_sizes
        # with the restatement of sparse_self_attention that tests/golden/offsets_reference.npz pins
        for name, t in zip(("x_offset", "y_offset", "m2w", "w_sizes", "w2n", "n2n", "w2m", "n_coords"), attn_args):
            if name not in ("x_offset", "y_offset", "m2w"):
                out[f"{tag}.arg.{name}"] = t.numpy()
        for name, prm in mod.named_parameters():
            out[f"{tag}.param.{name}"] = prm.detach().numpy()
            out[f"{tag}.grad.{name}"] = prm.grad.numpy()
        out[f"{tag}.grad.feats"] = feats.grad.numpy()
        out[f"{tag}.out"] = y.detach().numpy()
        for name, t in zip(("q", "k", "v", "tq", "tk", "tv", "table_offsets"), a[:7]):
            out[f"{tag}.call.{name}"] = t.detach().numpy()
        for name, t in zip(("m2w", "w_sizes", "w2m", "w2n", "n2n", "n_crse"), a[7]):
            if name != "m2w":
                out[f"{tag}.call.idx.{name}"] = t.detach().numpy()
        out[f"{tag}.call.enums"] = np.array([a[8].value, a[9].value, a[10].value, a[11].value])
        out[f"{tag}.call.result"] = real_apply(*a).detach().numpy()
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays")


if __name__ == "__main__":
    main()
