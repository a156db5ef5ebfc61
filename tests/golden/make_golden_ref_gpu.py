"""Runs the reference's own compiled CUDA kernels (oracle/_ref/ref_swin3d_cuda.so, built by
oracle/build_ref.py from the sources of microsoft/Swin3D) on seeded inputs on a GPU and writes
their outputs to the .npz file given as the first argument (default: ref_gpu_golden.npz beside this
script).  That file is committed as tests/golden/ref_gpu_golden.npz and pins the CPU oracle
(tests/test_golden_ref_gpu.py).

Only shapes for which the reference forward kernel stays inside its 32-entry shared staging
array are used: head_dim/pack >= 16, i.e. fp32/fp64 with head_dim 16 or 32 and fp16 with
head_dim 32 (see oracle/build_ref.py).

Usage (on a machine with a GPU):  python tests/golden/make_golden_ref_gpu.py [output.npz]
"""
import importlib.machinery
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402
from tests.helpers import make_problem  # noqa: E402

REF_SO = os.path.join(ROOT, "oracle", "_ref", "ref_swin3d_cuda.so")

# name -> make_problem kwargs + dtype
ATTN_CASES = {
    "f32_hd16_xyz": dict(kw=dict(seed=101, n_voxels=350, grid=18, H=2, hd=16, crse="XYZ"), dtype="float32"),
    "f32_hd16_rgb_shift": dict(kw=dict(seed=102, n_voxels=350, grid=18, H=2, hd=16, crse="XYZ_RGB", shift=2), dtype="float32"),
    "f32_hd32_norm": dict(kw=dict(seed=103, n_voxels=300, grid=18, H=2, hd=32, crse="XYZ_RGB_NORM"), dtype="float32"),
    "f64_hd16_rgb": dict(kw=dict(seed=104, n_voxels=200, grid=18, H=2, hd=16, crse="XYZ_RGB"), dtype="float64"),
    "f16_hd32_rgb": dict(kw=dict(seed=105, n_voxels=300, grid=18, H=2, hd=32, crse="XYZ_RGB", round_fp16=True), dtype="float16"),
}
# the cases whose reference outputs are committed as a fixture (the others only run on the GPU)
GOLDEN = ("f32_hd16_rgb_shift", "f64_hd16_rgb", "f16_hd32_rgb", "knn_k3", "knn_k16")
KNN_CASES = {"knn_k3": dict(seed=201, K=3), "knn_k16": dict(seed=202, K=16), "knn_k64": dict(seed=203, K=64)}


def load_ref():
    if not os.path.exists(REF_SO):
        return None
    loader = importlib.machinery.ExtensionFileLoader("ref_swin3d_cuda", REF_SO)
    spec = importlib.util.spec_from_loader("ref_swin3d_cuda", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def knn_inputs(seed):
    from swin3d_b200 import synthetic as S
    srcs, qrys = zip(*[S.make_knn_scene(seed + s, 400, 300 + 50 * s) for s in range(2)])
    src, qry = np.concatenate(srcs), np.concatenate(qrys)
    return src, qry, np.cumsum([len(s) for s in srcs]).astype(np.int32), \
        np.cumsum([len(q) for q in qrys]).astype(np.int32)


def run_ref_attention(ref, p, dtype):
    """The call sequence of SelfAttnAIOFunction.forward/backward (attn_coff.py:180-184,219-224)."""
    tdt = getattr(torch, dtype)
    d = lambda a, dt=tdt: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt)
    qkv = [d(p.q), d(p.k), d(p.v)]
    tabs = [d(p.tq), d(p.tk), d(p.tv)]
    x, y, m2w, ws, w2n, w2m = O.window_offsets(p.w_sizes)
    idx = [d(m2w, torch.int64), d(ws, torch.int64), d(w2m, torch.int64), d(w2n, torch.int64),
           d(p.n2n, torch.int64), d(p.n_crse, torch.float32)]
    offs = torch.IntTensor(list(p.sizes)).cuda()
    mx = ref.cal_max_coffs(qkv, tabs, offs, idx, 2, 3)
    raw, sm = ref.self_attn_forward(qkv, tabs, mx, offs, idx, 2, 3)
    norm = raw / sm
    g = d(p.g)
    raw2 = norm * sm
    dS = ref.cal_exp_sum_grads(g, raw2, sm, qkv[-1], tabs[-1])
    grads = ref.self_attn_indir_backward(g, dS, raw2, sm, mx, *qkv, *tabs, offs, idx, 2, 3)
    torch.cuda.synchronize()
    f = lambda t: t.detach().cpu().numpy()
    return dict(norm=f(norm), sum=f(sm), max=f(mx), dq=f(grads[0]), dk=f(grads[1]), dv=f(grads[2]),
                dtq=f(grads[3]), dtk=f(grads[4]), dtv=f(grads[5]))


def run_ref_knn(ref, K, src, qry, so, qo):
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    idx = torch.zeros((len(qry), K), dtype=torch.int32, device="cuda")
    dist = torch.zeros((len(qry), K), dtype=torch.float32, device="cuda") + 1e10
    ref.knn_cuda(K, d(src), d(qry), d(so), d(qo), idx, dist)
    torch.cuda.synchronize()
    return idx.cpu().numpy(), dist.cpu().numpy()


def main():
    ref = load_ref()
    if ref is None:
        print("oracle/_ref/ref_swin3d_cuda.so not built; nothing to do")
        return 0
    out = {}
    for name, c in ATTN_CASES.items():
        if name not in GOLDEN:
            continue
        p = make_problem(**c["kw"])
        res = run_ref_attention(ref, p, c["dtype"])
        for k, v in res.items():
            out[f"{name}.{k}"] = v
    for name, c in KNN_CASES.items():
        if name not in GOLDEN:
            continue
        src, qry, so, qo = knn_inputs(c["seed"])
        idx, d2 = run_ref_knn(ref, c["K"], src, qry, so, qo)
        out[f"{name}.idx"], out[f"{name}.d2"] = idx, d2
    dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_gpu_golden.npz")
    os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
