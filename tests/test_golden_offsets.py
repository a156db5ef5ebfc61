"""CPU: oracle restatements against fixtures produced by the reference's own Python code
(tests/golden/make_golden_offsets.py ran sparse_self_attention, WindowAttention.__init__ and the
enums of microsoft/Swin3D in-process)."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from swin3d_b200 import synthetic as S

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "offsets_reference.npz"))


@pytest.mark.parametrize("case", ["tiny", "single", "ones", "ragged", "full"])
def test_window_offsets_match_reference(case):
    w = G[f"{case}.w_sizes"]
    x, y, m2w, ws, w2n, w2m = O.window_offsets(w)
    for name, got in (("x_offset", x), ("y_offset", y), ("m2w", m2w), ("w_sizes", ws),
                      ("w2n", w2n), ("w2m", w2m)):
        exp = G[f"{case}.{name}"]
        assert got.dtype == exp.dtype == np.int64
        assert np.array_equal(got, exp), name


def test_known_answer_three_windows():
    x, y, m2w, ws, w2n, w2m = O.window_offsets([2, 3, 1])
    assert w2n.tolist() == [0, 2, 5]
    assert w2m.tolist() == [0, 4, 13]
    assert m2w.tolist() == [0] * 4 + [1] * 9 + [2]


@pytest.mark.parametrize("key", [k for k in G.files if k.startswith("table_offsets.")])
def test_table_sizes_match_reference(key):
    _, crse, ws, q, H, dim = key.split(".")
    ws, q, H, dim = int(ws), int(q), int(H), int(dim)
    assert S.table_sizes(ws, q, H, dim // H, crse) == G[key].tolist()
    assert G[key.replace("table_offsets", "xyz_table_shape")].tolist() == [3, 2 * ws * q, H, dim // H]


def test_enum_values_match_reference():
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    for name in ("PosEmb", "TableDims", "IndexMode", "PrecisionMode"):
        ref = {n: int(v) for n, v in G[f"enum.{name}"]}
        mine = {m.name: m.value for m in getattr(C, name)}
        assert mine == ref
