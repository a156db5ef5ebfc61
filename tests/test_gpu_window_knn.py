"""GPU parity: window builder and KNN (through the C-ABI) against the CPU oracles, bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from swin3d_b200 import synthetic as S

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check_window(coords, feats, ws, shift, stride=1):
    from swin3d_b200.window import build_windows
    ref = O.window_grouping(coords, feats, ws, shift, stride)
    wi = build_windows(_dev(coords), _dev(feats), ws, shift, stride)
    assert np.array_equal(wi.n2n.cpu().numpy(), ref[0])
    assert np.array_equal(wi.n_coords.cpu().numpy(), ref[1])
    assert np.array_equal(wi.w_sizes.cpu().numpy(), ref[2])
    assert np.array_equal(wi.w2n.cpu().numpy(), ref[3])
    assert wi.num_pairs == int((ref[2].astype(np.int64) ** 2).sum())
    assert wi.max_window == int(ref[2].max())
    return wi


@pytest.mark.parametrize("ws,shift", [(5, 0), (5, 2), (7, 0), (7, 3)])
def test_window_build_matches_oracle(ws, shift):
    sc = S.concat_scenes([S.make_planes_and_boxes(s, 3000, 48) for s in (1, 2, 3)])
    _check_window(sc.coords, S.signal_feats(sc, "XYZ_RGB_NORM"), ws, shift)


def test_window_build_room_scale_and_tensor_stride():
    sc = S.make_room(3, target_voxels=60_000)
    feats = S.signal_feats(sc, "XYZ_RGB")
    _check_window(sc.coords, feats, 5, 2)
    c2 = sc.coords.copy()
    c2[:, 1:] *= 2                       # tensor stride 2 (a down-sampled stage)
    _check_window(c2, feats, 7, 3, stride=2)


def test_window_build_negative_coordinates_and_tiny_inputs():
    rng = np.random.default_rng(0)
    pts = np.unique(rng.integers(-40, 40, size=(2000, 3)), axis=0)
    coords = np.concatenate([rng.integers(0, 3, size=(len(pts), 1)), pts], 1).astype(np.int32)
    feats = rng.random((len(pts), 3), dtype=np.float32)
    _check_window(coords, feats, 5, 2)
    _check_window(coords[:1], feats[:1], 5, 0)
    from swin3d_b200.window import build_windows
    wi = build_windows(_dev(coords[:0]), _dev(feats[:0]), 5, 0)
    assert wi.w_sizes.numel() == 0 and wi.n2n.numel() == 0 and wi.num_pairs == 0


def test_window_build_rejects_out_of_range_keys():
    from swin3d_b200.window import build_windows
    coords = np.array([[0, 5 * 20000, 0, 0]], dtype=np.int32)
    with pytest.raises(ValueError):
        build_windows(_dev(coords), _dev(np.zeros((1, 3), dtype=np.float32)), 5, 0)


def _knn_gpu(K, src, qry, so, qo):
    from swin3d_b200.sparse_dl.knn.knn import knn_raw
    idx, d2 = knn_raw(K, _dev(src), _dev(qry), _dev(np.asarray(so, dtype=np.int32)),
                      _dev(np.asarray(qo, dtype=np.int32)))
    torch.cuda.synchronize()
    return idx.cpu().numpy(), d2.cpu().numpy()


@pytest.mark.parametrize("K", [1, 3, 16, 33, 64])
def test_knn_bit_exact_vs_heap_oracle(K):
    srcs, qrys = zip(*[S.make_knn_scene(s, 1500, 900 + 100 * s) for s in range(3)])
    src, qry = np.concatenate(srcs), np.concatenate(qrys)
    so = np.cumsum([len(s) for s in srcs])
    qo = np.cumsum([len(q) for q in qrys])
    idx, d2 = _knn_gpu(K, src, qry, so, qo)
    ridx, rd2 = O.knn(K, src, qry, so, qo, fma_mode=2)
    assert np.array_equal(d2.view(np.uint32), rd2.view(np.uint32))
    assert np.array_equal(idx, ridx)


def test_knn_ties_follow_the_reference_heap():
    """Integer lattice points: massive distance ties; indices must still equal the literal heap."""
    g = np.stack(np.meshgrid(*[np.arange(8)] * 3, indexing="ij"), -1).reshape(-1, 3).astype(np.float32)
    rng = np.random.default_rng(1)
    src = g[rng.permutation(len(g))]
    qry = g[::3] + 0.5
    for K in (3, 16):
        idx, d2 = _knn_gpu(K, src, qry, [len(src)], [len(qry)])
        ridx, rd2 = O.knn(K, src, qry, [len(src)], [len(qry)], fma_mode=2)
        assert np.array_equal(idx, ridx) and np.array_equal(d2, rd2)


def _two_scenes(seed):
    srcs, qrys = zip(*[S.make_knn_scene(seed + s, 1300, 1100 + 90 * s) for s in range(2)])
    return (np.concatenate(srcs), np.concatenate(qrys), np.cumsum([len(x) for x in srcs]),
            np.cumsum([len(x) for x in qrys]))


@pytest.mark.parametrize("case", ["offset_1e3", "offset_1e5", "scale_1e-18", "scale_1e-22", "scale_1e18",
                                  "scale_3e19", "nonfinite", "duplicates"])
def test_knn_lower_bound_filter_never_changes_the_result(case):
    """The scan rejects candidates with a rounded lower bound |p|^2 - 2 p.q + margin before the exact
    distance is evaluated; the margin scales with the coordinate magnitudes.  Magnitudes that stress
    it -- far from the origin, products in the subnormal range, squares that overflow, NaN and
    infinite coordinates, sources equal to queries -- must give the literal heap's bits."""
    src, qry, so, qo = _two_scenes(40)
    rng = np.random.default_rng(5)
    if case.startswith("offset"):
        off = np.float32(case.split("_")[1])
        src, qry = src + off, qry + off
    elif case.startswith("scale"):
        sc = np.float32(case.split("_")[1])
        src, qry = src * sc, qry * sc
    elif case == "nonfinite":
        src, qry = src.copy(), qry.copy()
        bad = rng.choice(len(src), 60, replace=False)
        src[bad[:20], rng.integers(0, 3, 20)] = np.nan
        src[bad[20:40], rng.integers(0, 3, 20)] = np.inf
        src[bad[40:], rng.integers(0, 3, 20)] = -np.inf
        qry[5, 1], qry[6, 0], qry[7, 2] = np.nan, np.inf, -np.inf
        src[bad[0] + 1] = 3e19                                   # |p|^2 overflows, the point itself is finite
    elif case == "duplicates":
        src = src.copy()
        src[:400] = qry[:400]
        src[400:600] = qry[:200]                                 # the same point twice: distance 0 ties
    for K in (3, 16):
        idx, d2 = _knn_gpu(K, src, qry, so, qo)
        with np.errstate(all="ignore"):
            ridx, rd2 = O.knn(K, src, qry, so, qo, fma_mode=2)
        assert np.array_equal(d2.view(np.uint32), rd2.view(np.uint32)), case
        assert np.array_equal(idx, ridx), case


def test_knn_fewer_candidates_than_k_and_empty_scene():
    src = np.array([[0, 0, 0], [1, 0, 0]], dtype=np.float32)
    qry = np.array([[0.1, 0, 0], [5, 5, 5]], dtype=np.float32)
    idx, d2 = _knn_gpu(4, src, qry, [2, 2], [1, 2])     # second scene has no source point
    ridx, rd2 = O.knn(4, src, qry, [2, 2], [1, 2])
    assert np.array_equal(idx, ridx) and np.array_equal(d2, rd2)
    assert d2[1].tolist() == [2.0 ** 31] * 4 and idx[1].tolist() == [0] * 4


def test_knn_function_returns_sqrt_distance():
    from swin3d_b200.sparse_dl.knn import KNN
    src, qry = S.make_knn_scene(9, 500, 400)
    idx, dist = KNN.apply(3, _dev(src), _dev(qry), _dev(np.array([400], dtype=np.int32)),
                          _dev(np.array([500], dtype=np.int32)))
    ridx, rd2 = O.knn(3, src, qry, [400], [500])
    assert idx.dtype == torch.int32 and dist.dtype == torch.float32
    assert np.array_equal(idx.cpu().numpy(), ridx)
    assert np.array_equal(dist.cpu().numpy(), np.sqrt(rd2))


def test_knn_config5_scale_properties():
    """One scene at benchmark size (200k queries x 50k sources): ascending distances, indices
    inside the scene, and a sample of rows equal to the heap oracle."""
    src, qry = S.make_knn_scene(0, 200_000, 50_000)
    idx, d2 = _knn_gpu(16, src, qry, [50_000], [200_000])
    assert (np.diff(d2, axis=1) >= 0).all()
    assert idx.min() >= 0 and idx.max() < 50_000
    sel = np.arange(0, 200_000, 997)
    ridx, rd2 = O.knn(16, src, qry[sel], [50_000], [len(sel)])
    assert np.array_equal(idx[sel], ridx) and np.array_equal(d2[sel], rd2)


@pytest.mark.parametrize("K", [3, 16])
def test_knn_block_configurations_agree(K):
    """Long query lists run blocks of 256 queries (two per thread for K <= 4), short ones blocks of 128
    with one query per thread; the same queries through both must give the same bits (the short
    configuration is the one the oracle tests above pin)."""
    src, qry = S.make_knn_scene(11, 700_000, 20_000)
    long_idx, long_d2 = _knn_gpu(K, src, qry, [20_000], [700_000])
    for a, b in ((0, 250_000), (250_000, 500_000), (500_000, 700_000)):
        idx, d2 = _knn_gpu(K, src, qry[a:b], [20_000], [b - a])
        assert np.array_equal(idx, long_idx[a:b])
        assert np.array_equal(d2.view(np.uint32), long_d2[a:b].view(np.uint32))


class _FakeMapKey:
    def __init__(self, stride):
        self._s = [stride] * 3

    def get_tensor_stride(self):
        return self._s


class _FakeSparseTensor:
    """What get_index01 reads of a MinkowskiEngine SparseTensor: .C and the tensor stride."""
    def __init__(self, coords, stride=1):
        self.C = coords
        self.coordinate_map_key = _FakeMapKey(stride)


@pytest.mark.parametrize("shift", [0, 2])
def test_get_index01_drop_in_returns_the_tuple_window_attention_unpacks(shift):
    """BasicLayer.get_index01 without MinkowskiEngine: the 8-tuple matches the numpy restatement of
    the reference's grouping + offsets, whether the shift is passed or the sparse tensor is
    already shifted (get_shifted_sp), and feeds SelfAttnAIOFunction like WindowAttention does."""
    from swin3d_b200.window import get_index01
    from swin3d_b200.sparse_dl.attn.attn_coff import (SelfAttnAIOFunction, PosEmb, TableDims,
                                                      IndexMode, PrecisionMode)
    from tests.helpers import make_problem, oracle_fwd_bwd, rel_err
    sc = S.make_planes_and_boxes(5, 1500, 30)
    p = make_problem(seed=41, scene=sc, ws=5, shift=shift, H=2, hd=16, crse="XYZ_RGB")
    feats = S.signal_feats(sc, "XYZ_RGB")
    local_xyz, colors = _dev(feats[:, :3]), _dev(feats[:, 3:])
    shifted = sc.coords.copy()
    shifted[:, 1:] += shift
    tuples = [get_index01(_FakeSparseTensor(_dev(sc.coords)), local_xyz, colors, 5, shift_size=shift),
              get_index01(_FakeSparseTensor(_dev(shifted)), local_xyz, colors, 5)]
    ref = O.window_grouping(sc.coords, feats, 5, shift)
    _, _, _, ws64, w2n64, w2m = O.window_offsets(ref[2])
    for x_off, y_off, m2w, w_sizes, w2n, n2n, w2m_t, n_coords in tuples:
        assert x_off is None and y_off is None and m2w.numel() == 0
        assert np.array_equal(w_sizes.cpu().numpy(), ws64)
        assert np.array_equal(w2n.cpu().numpy(), w2n64)
        assert np.array_equal(w2m_t.cpu().numpy(), w2m)
        assert np.array_equal(n2n.cpu().numpy(), ref[0])
        assert np.array_equal(n_coords.cpu().numpy(), ref[1])
    # the call WindowAttention.forward makes with that tuple
    _, _, m2w, w_sizes, w2n, n2n, w2m_t, n_coords = tuples[1]
    n_crse = torch.cat([n_coords[:, :3] * p.quant, n_coords[:, 3:6] * (2 * p.quant)], dim=1)
    indices = [m2w, w_sizes, w2m_t, w2n, n2n, n_crse]
    q, k, v = (_dev(a).requires_grad_() for a in (p.q, p.k, p.v))
    tq, tk, tv = (_dev(a).requires_grad_() for a in (p.tq, p.tk, p.tv))
    out = SelfAttnAIOFunction.apply(q, k, v, tq, tk, tv, torch.IntTensor(p.sizes).cuda(), indices,
                                    PosEmb.SEPARATE, TableDims.D0, IndexMode.INDIRECT, PrecisionMode.HALF_NONE)
    out.backward(_dev(p.g))
    o_ref, _, g_ref = oracle_fwd_bwd(p, np.float64)
    assert rel_err(out.detach().cpu().numpy(), o_ref) < 1e-4
    for t, b in zip((q, k, v, tq, tk, tv), g_ref):
        assert rel_err(t.grad.cpu().numpy(), b) < 1e-4
