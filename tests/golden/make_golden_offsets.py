"""Generates tests/golden/offsets_reference.npz by running the reference's own Python code.

Needs a checkout of microsoft/Swin3D (path as first argument); MinkowskiEngine, timm and the two
CUDA extensions are replaced by empty stub modules, which is enough to import
Swin3D.modules.swin3d_layers and to run, on CPU tensors,
  * sparse_self_attention(protocol="v2")      (swin3d_layers.py:76-150)
  * WindowAttention.__init__ table shapes     (swin3d_layers.py:404-478)
  * the enum values of attn_coff.py:20-40.
Usage: python tests/golden/make_golden_offsets.py <reference_root>   (or set SWIN3D_REFERENCE)
"""
import os
import sys
import types

import numpy as np
import torch


def import_reference(root):
    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    class _Any:
        def __init__(self, *a, **k):
            pass

    me = stub("MinkowskiEngine", SparseTensor=_Any)
    for n in ("MinkowskiMaxPooling", "MinkowskiAvgPooling", "MinkowskiPoolingTranspose",
              "MinkowskiConvolution", "MinkowskiBatchNorm", "MinkowskiReLU", "MinkowskiLinear",
              "MinkowskiNetwork"):
        setattr(me, n, _Any)
    stub("timm")
    stub("timm.models")
    stub("timm.models.layers", DropPath=torch.nn.Identity, trunc_normal_=torch.nn.init.trunc_normal_)
    sys.path.insert(0, root)
    stub("Swin3D.sparse_dl.attn_cuda")
    stub("Swin3D.sparse_dl.knn_cuda")
    import Swin3D.modules.swin3d_layers as layers
    import Swin3D.sparse_dl.attn.attn_coff as coff
    return layers, coff


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SWIN3D_REFERENCE")
    if not root:
        raise SystemExit("usage: python " + sys.argv[0] + " <reference_root>   (or set SWIN3D_REFERENCE)")
    layers, coff = import_reference(root)
    out = {}
    rng = np.random.default_rng(0)
    cases = {
        "tiny": np.array([2, 3, 1]),
        "single": np.array([7]),
        "ones": np.ones(9, dtype=np.int64),
        "ragged": rng.integers(1, 126, size=40),
        "full": np.array([125, 343, 1, 64]),
    }
    for name, w in cases.items():
        res = layers.sparse_self_attention(None, torch.tensor(w, dtype=torch.int64), protocol="v2")
        for key, t in zip(("x_offset", "y_offset", "m2w", "w_sizes", "w2n", "w2m"), res):
            out[f"{name}.{key}"] = t.numpy()
    for crse, ws, q, H, dim in (("XYZ", 5, 4, 6, 48), ("XYZ_RGB", 5, 4, 6, 48),
                                ("XYZ_RGB_NORM", 5, 4, 10, 80), ("XYZ_RGB_NORM", 7, 4, 10, 160)):
        wa = layers.WindowAttention(dim, ws, q, H, cRSE=crse)
        out[f"table_offsets.{crse}.{ws}.{q}.{H}.{dim}"] = np.array(wa.table_offsets, dtype=np.int64)
        out[f"xyz_table_shape.{crse}.{ws}.{q}.{H}.{dim}"] = np.array(wa.query_xyz_table.shape)
    for enum_name in ("PosEmb", "TableDims", "IndexMode", "PrecisionMode"):
        e = getattr(coff, enum_name)
        out[f"enum.{enum_name}"] = np.array([[m.name, str(m.value)] for m in e])
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "offsets_reference.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
