"""GPU: the drop-in Function under the reference's ``WindowAttention`` module.

tests/golden/window_attention_reference.npz was recorded by running the reference's own
``WindowAttention.forward`` and ``SelfAttnAIOFunction`` (microsoft/Swin3D,
Swin3D/modules/swin3d_layers.py:480-575, Swin3D/sparse_dl/attn/attn_coff.py:155-232) unchanged on
CPU tensors over the oracle (tests/golden/make_golden_window_attention.py); the reference's Python
cannot be imported on a GPU box.  Two things are checked here:
  * the recorded call -- every argument exactly as the module hands it to
    ``SelfAttnAIOFunction.apply`` (fp32 parameters, int32 table offsets, int64 index tensors, enums) --
    replayed through this repository's Function gives the recorded result;
  * the module's computation around that call (qkv projection, scaling, table concatenation, output
    projection; swin3d_layers.py:502-572), rebuilt from the recorded parameters, reproduces the
    recorded module output and the recorded gradients of the features and of every parameter, for
    fp16_mode 0, 1 and 2 (1 and 2 under autocast, as the reference's examples run them).
"""
import os

import numpy as np
import pytest

from tests.helpers import rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "window_attention_reference.npz")
FP32_TOL, FP16_TOL = 1e-4, 2e-2


def _case(tag):
    d = np.load(FIX)
    return {k[len(tag) + 1:]: d[k] for k in d.files if k.startswith(tag + ".")}


def _indices(c, prefix):
    """The six-tensor list of IndexMode.INDIRECT with the dtypes the module passes (int64 indices);
    m2w is rebuilt from the window sizes (one entry per attention pair, never read by the library)."""
    from oracle import oracle as O
    w = c[prefix + "w_sizes"]
    m2w = O.window_offsets(w)[2]
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return m2w, cu, w


@pytest.mark.parametrize("tag", ["rgb_m0", "norm_m2"])
def test_recorded_function_call_replays_on_the_gpu(tag):
    from swin3d_b200.sparse_dl.attn.attn_coff import (IndexMode, PosEmb, PrecisionMode, SelfAttnAIOFunction,
                                                     TableDims)
    c = _case(tag)
    m2w, cu, _ = _indices(c, "call.idx.")
    idx = [cu(m2w), cu(c["call.idx.w_sizes"]), cu(c["call.idx.w2m"]), cu(c["call.idx.w2n"]), cu(c["call.idx.n2n"]),
           cu(c["call.idx.n_crse"])]
    assert all(t.dtype == torch.int64 for t in idx[:5])
    pe, td, im, pm = (int(x) for x in c["call.enums"])
    assert (pe, td, im) == (PosEmb.SEPARATE.value, TableDims.D0.value, IndexMode.INDIRECT.value)
    out = SelfAttnAIOFunction.apply(cu(c["call.q"]), cu(c["call.k"]), cu(c["call.v"]), cu(c["call.tq"]),
                                    cu(c["call.tk"]), cu(c["call.tv"]), cu(c["call.table_offsets"]), idx,
                                    PosEmb(pe), TableDims(td), IndexMode(im), PrecisionMode(pm))
    assert out.dtype == torch.float32
    assert rel_err(out.cpu().numpy(), c["call.result"]) < FP32_TOL


def _module_forward(c, crse, fp16_mode, feats, params, attn_args):
    """swin3d_layers.py:486-575 around the Function: same operations, same order."""
    from swin3d_b200.sparse_dl.attn.attn_coff import (IndexMode, PosEmb, PrecisionMode, SelfAttnAIOFunction,
                                                     TableDims)
    x_offset, y_offset, m2w, w_sizes, w2n, n2n, w2m, n_coords = attn_args
    dim = feats.shape[1]
    heads = params["query_xyz_table"].shape[2]
    num_sc = dim // heads
    quant = params["query_xyz_table"].shape[1] // (2 * 5)             # table rows = 2 * window * quant
    qkv = torch.nn.functional.linear(feats, params["qkv.weight"], params["qkv.bias"])
    qkv = qkv.reshape(feats.shape[0], 3, heads, num_sc).permute(1, 0, 2, 3).contiguous()
    query, key, value = qkv[0], qkv[1], qkv[2]
    query = query * num_sc ** -0.5
    table_offsets, n_crse, tq, tk, tv = [], [], [], [], []
    for name, cols, scale in (("xyz", slice(0, 3), quant), ("rgb", slice(3, 6), 2 * quant), ("norm", slice(6, 9), 2 * quant)):
        if name.upper() in crse:
            n_crse.append(n_coords[:, cols] * scale)
            for lst, which in ((tq, "query"), (tk, "key"), (tv, "value")):
                lst.append(params[f"{which}_{name}_table"].view(-1))
            table_offsets += [params[f"query_{name}_table"][0].numel()] * 3
    table_offsets = torch.IntTensor(table_offsets).cuda()
    indices = [m2w, w_sizes, w2m, w2n, n2n, torch.cat(n_crse, dim=1)]
    mode = {0: PrecisionMode.HALF_NONE, 1: PrecisionMode.HALF_FORWARD, 2: PrecisionMode.HALF_ALL}[fp16_mode]
    upd = SelfAttnAIOFunction.apply(query, key, value, torch.cat(tq), torch.cat(tk), torch.cat(tv), table_offsets,
                                    indices, PosEmb.SEPARATE, TableDims.D0, IndexMode.INDIRECT, mode)
    upd = upd.flatten(1).view(feats.shape[0], dim)
    return torch.nn.functional.linear(upd, params["proj.weight"], params["proj.bias"])


@pytest.mark.parametrize("tag", ["rgb_m0", "norm_m2"])
@pytest.mark.parametrize("fp16_mode", [0, 1, 2])
def test_module_computation_around_the_function_matches_the_recorded_module(tag, fp16_mode):
    c = _case(tag)
    crse = str(c["crse"])
    m2w, cu, w = _indices(c, "arg.")
    from oracle import oracle as O
    x_off, y_off = O.window_offsets(w)[:2]
    attn_args = (cu(x_off), cu(y_off), cu(m2w), cu(c["arg.w_sizes"]), cu(c["arg.w2n"]), cu(c["arg.n2n"]),
                 cu(c["arg.w2m"]), cu(c["arg.n_coords"]))
    params = {k[len("param."):]: cu(v).requires_grad_() for k, v in c.items() if k.startswith("param.")}
    feats = cu(c["feats"]).requires_grad_()
    half = fp16_mode != 0
    with torch.autocast("cuda", dtype=torch.float16, enabled=half):
        y = _module_forward(c, crse, fp16_mode, feats, params, attn_args)
    y.float().backward(cu(c["upstream"]))
    tol = FP16_TOL if half else FP32_TOL
    assert rel_err(y.float().detach().cpu().numpy(), c["out"]) < tol
    assert rel_err(feats.grad.cpu().numpy(), c["grad.feats"]) < tol
    for name, p in params.items():
        assert p.grad is not None, name
        assert rel_err(p.grad.float().cpu().numpy(), c["grad." + name]) < tol, name
