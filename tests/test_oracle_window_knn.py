"""CPU: window-grouping and KNN oracles against hand-checked known answers and brute force."""
import numpy as np

from oracle import oracle as O
from swin3d_b200 import synthetic as S


def test_window_grouping_invariants():
    sc = S.make_planes_and_boxes(1, 1500, 32)
    feats = S.signal_feats(sc, "XYZ_RGB")
    for shift in (0, 2):
        n2n, nc, ws, w2n = O.window_grouping(sc.coords, feats, 5, shift)
        assert sorted(n2n.tolist()) == list(range(1500))          # a permutation
        assert ws.sum() == 1500 and np.array_equal(w2n, np.cumsum(ws) - ws)
        c = sc.coords[n2n, 1:] + shift
        win = c // 5
        for w in range(len(ws)):
            sl = slice(w2n[w], w2n[w] + ws[w])
            assert (win[sl] == win[sl][0]).all()                  # one window per group
            cell = c[sl] - win[sl] * 5
            cid = (cell[:, 0] * 5 + cell[:, 1]) * 5 + cell[:, 2]
            assert (np.diff(cid) > 0).all()                       # ascending cell id
            assert np.array_equal(np.floor(nc[sl, :3]).astype(int), cell)
        assert np.array_equal(nc[:, 3:], feats[n2n, 3:])
        # windows are in lexicographic order
        firsts = win[w2n]
        key = (firsts[:, 0] * 1000 + firsts[:, 1]) * 1000 + firsts[:, 2]
        assert (np.diff(key) > 0).all()


def test_window_grouping_negative_coordinates_floor():
    coords = np.array([[0, -1, 0, 0], [0, -5, 0, 0], [0, -6, 0, 0], [0, 4, 0, 0]], dtype=np.int32)
    feats = np.zeros((4, 3), dtype=np.float32)
    n2n, nc, ws, w2n = O.window_grouping(coords, feats, 5, 0)
    # windows along x: -6 -> -2 ; -5,-1 -> -1 ; 4 -> 0
    assert ws.tolist() == [1, 2, 1]
    assert n2n.tolist() == [2, 1, 0, 3]
    assert nc[:, 0].tolist() == [4.0, 0.0, 4.0, 4.0]


def test_knn_heap_tie_behaviour_known_answers():
    """The reference's heap keeps later equal-distance candidates out (strict <) but its sift-down
    swaps on equality, so ties do not resolve to the lowest index."""
    src = np.zeros((4, 3), dtype=np.float32)
    src[:, 0] = [np.sqrt(5), -np.sqrt(5), 0, 1]
    src[2, 1] = np.sqrt(5)
    src[:3] = np.array([[2, 1, 0], [1, 2, 0], [0, 1, 2]], dtype=np.float32)   # all at d2 = 5
    src[3] = [1, 0, 0]                                                        # d2 = 1
    q = np.zeros((1, 3), dtype=np.float32)
    idx, d2 = O.knn(2, src, q, [4], [1])
    assert idx[0].tolist() == [3, 1] and d2[0].tolist() == [1.0, 5.0]
    idx, d2 = O.knn(3, src, q, [4], [1])
    assert idx[0].tolist() == [3, 1, 2]
    idx, d2 = O.knn(4, src[[3, 0]], q, [2], [1])
    assert idx[0, :2].tolist() == [0, 1] and d2[0].tolist() == [1.0, 5.0, 2.0 ** 31, 2.0 ** 31]


def test_knn_matches_brute_force_without_ties():
    rng = np.random.default_rng(0)
    src = rng.random((700, 3), dtype=np.float32)
    qry = rng.random((300, 3), dtype=np.float32)
    so, qo = [300, 700], [100, 300]
    for K in (1, 3, 16):
        idx, d2 = O.knn(K, src, qry, so, qo, fma_mode=0)
        for g in range(300):
            s0, s1 = (0, 300) if g < 100 else (300, 700)
            d = ((src[s0:s1].astype(np.float64) - qry[g]) ** 2).sum(1)
            best = np.argsort(d, kind="stable")[:K] + s0
            assert np.array_equal(np.sort(idx[g]), np.sort(best))
            assert (np.diff(d2[g]) >= 0).all()
