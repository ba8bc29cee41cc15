"""CPU checks of the oracle: hand-computed answers, the committed fixtures, the independent
numpy mirror, and the properties the reference's own device tests assert (self-hit at rank 1:
FR/test/ascend/TestAscendIndexFlat.cpp:117-123, TestAscendIndexIVFPQ.cpp:151-166)."""
import os

import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_flat_known_answers():
    xb = np.zeros((5, 16), np.float32)
    xb[:, 0] = [0, 1, 2, 3, 4]
    xq = np.zeros((1, 16), np.float32)
    xq[0, 0] = 1.4
    D, I = oracle.flat_search(oracle.METRIC_L2, xb, xq, 3)
    assert I.tolist() == [[1, 2, 0]]
    np.testing.assert_allclose(D[0], [0.16, 0.36, 1.96], rtol=1e-6)
    D, I = oracle.flat_search(oracle.METRIC_IP, xb, xq, 2)
    assert I.tolist() == [[4, 3]]
    np.testing.assert_allclose(D[0], [5.6, 4.2], rtol=1e-6)


def test_flat_ties_and_padding():
    xb = np.ones((4, 16), np.float32)
    xq = np.ones((2, 16), np.float32)
    D, I = oracle.flat_search(oracle.METRIC_L2, xb, xq, 6)
    assert I[0].tolist() == [0, 1, 2, 3, -1, -1]
    assert np.all(D[:, :4] == 0) and np.all(D[:, 4:] == np.finfo(np.float32).max)
    D, I = oracle.flat_search(oracle.METRIC_L2, xb, xq, 2, labels=np.array([40, 30, 20, 10]))
    assert I[0].tolist() == [40, 30]  # ties break by position, labels are mapped afterwards


def test_int8_known_answers():
    xb = np.zeros((3, 16), np.int8)
    xb[0, :2] = [127, 127]
    xb[1, :2] = [-128, -128]
    xb[2, :2] = [1, 0]
    xq = np.zeros((1, 16), np.int8)
    xq[0, :2] = [-128, -128]
    D, I = oracle.int8_search(oracle.METRIC_IP, xb, xq, 3)
    assert I.tolist() == [[1, 2, 0]]
    assert D[0].tolist() == [32768.0, -128.0, -32512.0]
    D, I = oracle.int8_search(oracle.METRIC_L2, xb, xq, 3)
    assert I.tolist() == [[1, 2, 0]]
    assert D[0].tolist() == [0.0, 129.0 ** 2 + 128.0 ** 2, 2 * 255.0 ** 2]


@pytest.mark.parametrize("metric", [oracle.METRIC_L2, oracle.METRIC_IP])
def test_flat_matches_numpy_mirror(metric):
    xb = datasets.gaussian(1500, 48, seed=11)
    xq = datasets.gaussian(13, 48, seed=12)
    D, I = oracle.flat_search(metric, xb, xq, 20)
    Dp, Ip = oracle.flat_search(metric, xb, xq, 20, precise=True)
    Dn, In = oracle.np_flat_search(metric, xb, xq, 20)
    np.testing.assert_array_equal(Ip, In)
    np.testing.assert_array_equal(Dp, Dn)          # fp64 accumulate, one rounding: identical
    np.testing.assert_allclose(D, Dn, rtol=1e-5)   # canonical fp32 within the fp32 tolerance
    assert (I == In).mean() > 0.995


@pytest.mark.parametrize("metric", [oracle.METRIC_L2, oracle.METRIC_IP])
def test_int8_matches_numpy_mirror(metric):
    xb = datasets.uniform_int8(2000, 32, seed=21)
    xq = datasets.uniform_int8(9, 32, seed=22)
    D, I = oracle.int8_search(metric, xb, xq, 50)
    Dn, In = oracle.np_int8_search(metric, xb, xq, 50)
    np.testing.assert_array_equal(I, In)
    np.testing.assert_array_equal(D, Dn)


def _int8_rows_with_varied_norms(n, d, seed):
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, (n, d)).astype(np.float32) * rng.uniform(0.02, 1.0, (n, 1)).astype(np.float32)
    return np.rint(x).astype(np.int8)


def test_fp16_conversions_match_numpy():
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1, 100, 7e4)]
                        + [np.array([0, -0.0, 65504, 65519.99, 65520, 6e-8, 2.9802322e-8, 2.9802326e-8, np.inf,
                                     -np.inf, 6.1e-5, 6.097e-5], np.float32)])
    with np.errstate(over="ignore"):
        ref = xs.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f2h(float(v)) for v in xs], np.uint16)
    np.testing.assert_array_equal(got, ref)
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    ref = hs.view(np.float16).astype(np.float32)
    got = np.array([oracle.h2f(int(h)) for h in hs], np.float32)
    assert np.all((ref == got) | (np.isnan(ref) & np.isnan(got)))


def test_int8_cosine_known_answers():
    """The reference's fp16 chain by hand: |x|^2 = |q|^2 = 64 * 100^2 = 640000 -> fp16(6400) = 6400,
    rnorm = fp16(1 / 80) = 0.0125 (fp16: 0.012496948); x = q gives fp16(6400 * fp16(rnorm^2))."""
    rn = np.float16(1.0 / 80.0)
    w = np.float16(np.float32(rn) * np.float32(rn))
    expect = float(np.float16(np.float32(6400.0) * np.float32(w)))
    assert oracle.cos16(640000, 640000, 640000) == expect
    assert abs(expect - 1.0) < 2e-3
    assert oracle.cos16(-640000, 640000, 640000) == -expect
    assert oracle.cos16(0, 640000, 640000) == 0.0
    assert oracle.cos16(0, 0, 640000) == -np.inf            # zero vector: 0 x inf = NaN, ranked last
    # |x|^2 * 0.01 beyond the fp16 range: rnorm = 0, and a saturated product times 0 is NaN as well
    assert oracle.cos16(100, 8258048, 640000) == 0.0
    assert oracle.cos16(8258048, 8258048, 8258048) == -np.inf


@pytest.mark.parametrize("d", [32, 512])
def test_int8_cosine_matches_numpy_float16(d):
    xb = _int8_rows_with_varied_norms(3000, d, seed=31)
    xq = _int8_rows_with_varied_norms(11, d, seed=32)
    xb[5] = 0
    xb[7] = 127
    xq[3] = 127
    xb[9] = xq[4]
    D, I = oracle.int8_search(oracle.METRIC_INT8_COS, xb, xq, 40)
    Dn, In = oracle.np_int8_search(oracle.METRIC_INT8_COS, xb, xq, 40)
    np.testing.assert_array_equal(I, In)
    np.testing.assert_array_equal(D, Dn)
    assert I[4, 0] == 9 or D[4, 0] == D[4, list(I[4]).index(9)]


def test_fixtures_reproduce():
    g = np.load(os.path.join(GOLD, "flat_small.npz"))
    for name, metric in (("l2", oracle.METRIC_L2), ("ip", oracle.METRIC_IP)):
        D, I = oracle.flat_search(metric, g["xb"], g["xq"], 10)
        np.testing.assert_array_equal(I, g[f"I_{name}"])
        np.testing.assert_array_equal(D, g[f"D_{name}"])
    g = np.load(os.path.join(GOLD, "int8_small.npz"))
    for name, metric in (("l2", oracle.METRIC_L2), ("ip", oracle.METRIC_IP)):
        D, I = oracle.int8_search(metric, g["xb"], g["xq"], 12)
        np.testing.assert_array_equal(I, g[f"I_{name}"])
        np.testing.assert_array_equal(D, g[f"D_{name}"])
    g = np.load(os.path.join(GOLD, "ivfpq_small.npz"))
    for tag, resid in (("raw", False), ("res", True)):
        ln = oracle.ivf_assign(g[f"cent_{tag}"], g["xb"])
        np.testing.assert_array_equal(ln, g[f"list_no_{tag}"])
        codes = oracle.pq_encode(g[f"cb_{tag}"], g["xb"], resid, g[f"cent_{tag}"], ln)
        np.testing.assert_array_equal(codes, g[f"codes_{tag}"])
        off, cs, ids = oracle.build_lists(ln, codes, np.arange(len(ln)), 16)
        D, I = oracle.ivfpq_search(g[f"cent_{tag}"], g[f"cb_{tag}"], resid, off, cs, ids, g["xq"], 4, 10)
        np.testing.assert_array_equal(I, g[f"I_{tag}"])
        np.testing.assert_array_equal(D, g[f"D_{tag}"])


def test_self_hit_flat_and_ivfpq():
    xb, _ = datasets.mixture(3000, 32, 32, seed=31)
    D, I = oracle.flat_search(oracle.METRIC_L2, xb, xb[:50], 1)
    assert I[:, 0].tolist() == list(range(50)) and np.all(D == 0)
    cent, cb = datasets.train_ivfpq(xb, 16, 8, False, niter=6)
    ln = oracle.ivf_assign(cent, xb)
    codes = oracle.pq_encode(cb, xb, False, cent, ln)
    off, cs, ids = oracle.build_lists(ln, codes, np.arange(len(ln)), 16)
    D, I = oracle.ivfpq_search(cent, cb, False, off, cs, ids, xb[:200], 16, 10)
    assert (I == np.arange(200)[:, None]).any(1).mean() > 0.95  # own id within the top 10 (PQ is lossy)


def test_ivfpq_matches_numpy_mirror_and_empty_lists():
    d, nlist, M = 32, 24, 8
    xb, _ = datasets.mixture(2500, d, 8, seed=41)
    xq, _ = datasets.mixture(11, d, 8, seed=42, centers_seed=41)
    for resid in (False, True):
        cent, cb = datasets.train_ivfpq(xb, nlist, M, resid, niter=5)
        cent[5] = 1e3  # a centroid nobody is assigned to -> empty list that is still probed
        ln = oracle.ivf_assign(cent, xb)
        codes = oracle.pq_encode(cb, xb, resid, cent, ln)
        off, cs, ids = oracle.build_lists(ln, codes, np.arange(len(ln)) * 3 + 7, nlist)
        assert off[6] == off[5]
        D, I, coarse = oracle.ivfpq_search(cent, cb, resid, off, cs, ids, xq, nlist, 15, return_coarse=True)
        Dn, In = oracle.np_ivfpq_search(cent, cb, resid, off, cs, ids, xq, nlist, 15)
        np.testing.assert_allclose(D, Dn, rtol=3e-5)
        assert (I == In).mean() > 0.98
        assert sorted(coarse[0].tolist()) == list(range(nlist))


def test_merge_topk():
    r = np.random.default_rng(5)
    D = np.sort(r.random((3, 4, 6)).astype(np.float32), axis=2)
    I = r.permutation(3 * 4 * 6).reshape(3, 4, 6).astype(np.int64)
    I[2, :, 4:] = -1
    Dm, Im = oracle.merge_topk(D, I)
    for q in range(4):
        pairs = sorted((D[s, q, j], I[s, q, j]) for s in range(3) for j in range(6) if I[s, q, j] >= 0)[:6]
        assert [p[1] for p in pairs] == Im[q].tolist()
        assert [p[0] for p in pairs] == Dm[q].tolist()


def test_rounding_helpers():
    x = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8], np.float32)
    np.testing.assert_array_equal(oracle.round_fp16(x), x.astype(np.float16).astype(np.float32))
    y = np.array([1.0, 1.0 + 2 ** -8, 1.0 + 2 ** -9, 3.0e38], np.float32)
    b = oracle.round_bf16(y)
    assert b[0] == 1.0 and b[1] == 1.0 + 2 ** -7 or b[1] == 1.0  # ties to even
    assert np.all((b.view(np.uint32) & 0xFFFF) == 0)


def test_kmeans_restatement_properties():
    """orc_kmeans: deterministic, start points as documented, every iteration lowers the objective."""
    x, _ = datasets.mixture(3000, 16, 8, seed=3)
    c0 = oracle.kmeans(x, 10, 0, seed=5)
    n = x.shape[0]
    np.testing.assert_array_equal(c0, x[[(c * n // 10 + 5) % n for c in range(10)]])
    prev = None
    for it in (1, 2, 4, 8):
        c = oracle.kmeans(x, 10, it, seed=5)
        a = oracle.ivf_assign(c, x)
        obj = float(((x - c[a]) ** 2).sum())
        assert prev is None or obj <= prev * (1 + 1e-6)
        prev = obj
    np.testing.assert_array_equal(oracle.kmeans(x, 10, 4, seed=5), oracle.kmeans(x, 10, 4, seed=5))
