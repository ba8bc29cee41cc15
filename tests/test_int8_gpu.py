"""GPU parity of Int8Flat search: distances and ids bit-exact against the int32 oracle, ties
broken by the lower id."""
import os

import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets
from helpers import assert_exact

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
L2, IP, COS = 1, 0, 2


@pytest.mark.parametrize("metric", [L2, IP])
def test_golden_fixture(b200, metric):
    g = np.load(os.path.join(GOLD, "int8_small.npz"))
    ix = b200.IndexInt8Flat(64, metric)
    ix.add(g["xb"])
    D, I = ix.search(g["xq"], 12)
    name = "l2" if metric == L2 else "ip"
    assert_exact(D, I, g[f"D_{name}"], g[f"I_{name}"])


@pytest.mark.parametrize("n,nq,k,d", [(1000, 1, 1, 64), (70000, 130, 100, 256), (262144 + 5, 3, 100, 128),
                                      (20000, 9, 10, 1024), (3000, 2, 1000, 64), (7, 2, 10, 64)])
@pytest.mark.parametrize("metric", [L2, IP])
def test_bit_exact_vs_oracle(b200, n, nq, k, d, metric):
    xb = datasets.uniform_int8(n, d, seed=2)
    xq = datasets.uniform_int8(nq, d, seed=3)
    ix = b200.IndexInt8Flat(d, metric)
    ix.add(xb)
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.int8_search(metric, xb, xq, k)
    assert_exact(D, I, Dr, Ir)


def test_extreme_values_and_ties(b200):
    d = 64
    xb = np.full((3000, d), -128, np.int8)
    xb[::2] = 127
    xq = np.full((2, d), -128, np.int8)
    xq[1] = 127
    for metric in (L2, IP):
        ix = b200.IndexInt8Flat(d, metric)
        ix.add(xb)
        D, I = ix.search(xq, 20)
        Dr, Ir = oracle.int8_search(metric, xb, xq, 20)
        assert_exact(D, I, Dr, Ir)
    assert Ir[1].tolist() == [2 * j for j in range(20)]  # ties -> lower id


def test_ids_remove_reset(b200):
    d = 128
    xb = datasets.uniform_int8(4000, d, seed=12)
    xq = datasets.uniform_int8(5, d, seed=13)
    ids = np.arange(4000, dtype=np.int64)[::-1].copy() + 100
    ix = b200.IndexInt8Flat(d, IP)
    ix.add_with_ids(xb, ids)
    D, I = ix.search(xq, 10)
    Dr, Ir = oracle.int8_search(IP, xb, xq, 10, labels=ids)
    assert_exact(D, I, Dr, Ir)
    assert ix.remove_ids(ids[:10]) == 10
    D, I = ix.search(xq, 10)
    Dr, Ir = oracle.int8_search(IP, ix.get_base(), xq, 10, labels=ix.get_ids())
    assert_exact(D, I, Dr, Ir)
    ix.reset()
    assert ix.ntotal == 0


def _rows_with_varied_norms(n, d, seed):
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, (n, d)).astype(np.float32) * rng.uniform(0.02, 1.0, (n, 1)).astype(np.float32)
    return np.rint(x).astype(np.int8)


@pytest.mark.parametrize("n,nq,k,d", [(1000, 1, 1, 64), (70000, 130, 100, 256), (262144 + 5, 3, 100, 128),
                                      (20000, 9, 10, 512), (3000, 2, 1000, 64), (7, 2, 10, 64)])
def test_cosine_bit_exact_vs_oracle(b200, n, nq, k, d):
    """The reference's meaning of METRIC_INNER_PRODUCT on this index: fp16 cosine.  fp16 scores tie
    all the time, so the ids only agree if the order among equal scores (lower position) does."""
    xb = _rows_with_varied_norms(n, d, seed=2)
    xq = _rows_with_varied_norms(nq, d, seed=3)
    ix = b200.IndexInt8Flat(d, COS)
    ix.add(xb)
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.int8_search(COS, xb, xq, k)
    assert_exact(D, I, Dr, Ir)
    assert np.abs(D[np.isfinite(D) & (I >= 0)]).max() <= 1.01


def test_cosine_zero_and_saturated_vectors(b200):
    """Rows whose fp16 arithmetic leaves the number line: a zero vector (0 x inf), norms beyond the
    fp16 range (reciprocal norm 0), a saturated product."""
    d = 512
    xb = _rows_with_varied_norms(3000, d, seed=5)
    xb[10] = 0
    xb[11] = 127
    xb[12] = -128
    xq = _rows_with_varied_norms(6, d, seed=6)
    xq[1] = 127
    xq[2] = 0
    ix = b200.IndexInt8Flat(d, COS)
    ix.add(xb)
    for k in (10, 3000):
        D, I = ix.search(xq, k)
        Dr, Ir = oracle.int8_search(COS, xb, xq, k)
        assert_exact(D, I, Dr, Ir)
    assert D[0, -1] == -np.inf and I[0, -1] == 10          # the zero row ranks last


def test_cosine_ids_masks_and_paging(b200):
    d, n, nq, k = 128, 30000, 70, 20
    xb = _rows_with_varied_norms(n, d, seed=7)
    xq = _rows_with_varied_norms(nq, d, seed=8)
    ids = np.arange(n, dtype=np.int64)[::-1].copy() * 3
    ix = b200.IndexInt8Flat(d, COS)
    ix.add_with_ids(xb[:20000], ids[:20000])
    ix.add_with_ids(xb[20000:], ids[20000:])
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.int8_search(COS, xb, xq, k, labels=ids)
    assert_exact(D, I, Dr, Ir)
    rng = np.random.default_rng(9)
    keep = rng.random((nq, n)) < 0.3
    mask = np.packbits(keep, axis=1, bitorder="little")
    D, I = ix.search_with_masks(xq, k, mask)
    for q in range(0, nq, 9):
        sel = np.nonzero(keep[q])[0]
        Dq, Iq = oracle.int8_search(COS, xb[sel], xq[q:q + 1], k, labels=ids[sel])
        assert_exact(D[q:q + 1], I[q:q + 1], Dq, Iq)
