"""GPU parity of the filtered search (search_with_masks): every query carries a bit per base position;
the result must be the exact top-k of the positions whose bit is set.  The oracle is the plain CPU
search run on the kept rows of each query."""
import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets
from helpers import assert_exact

pytestmark = pytest.mark.gpu
L2, IP = 1, 0


def _expected(search, xb, ids, xq, keep, k):
    D = np.full((xq.shape[0], k), np.finfo(np.float32).max, np.float32)
    I = np.full((xq.shape[0], k), -1, np.int64)
    for q in range(xq.shape[0]):
        rows = np.flatnonzero(keep[q])
        if rows.size == 0:
            continue
        Dq, Iq = search(np.ascontiguousarray(xb[rows]), xq[q:q + 1], k, ids[rows])
        D[q], I[q] = Dq[0], Iq[0]
    return D, I


@pytest.mark.parametrize("metric", [L2, IP])
@pytest.mark.parametrize("n,nq,k,d,density", [
    (3000, 5, 10, 64, 0.5),          # no threshold pass
    (140000, 6, 20, 32, 0.3),        # sampled threshold, two stretches
    (140000, 4, 50, 32, 0.002),      # fewer kept rows than k in some bursts; heavy filtering
    (70000, 130, 10, 128, 0.9),      # two query blocks
])
def test_flat_fp32_masked(b200, metric, n, nq, k, d, density):
    xb = datasets.gaussian(n, d, seed=11)
    xq = datasets.gaussian(nq, d, seed=12)
    ids = np.arange(n, dtype=np.int64) * 2 + 5
    rng = np.random.default_rng(13)
    keep = rng.random((nq, n)) < density
    keep[0, :] = False                      # a query with everything filtered out
    if nq > 1:
        keep[1, :] = True                   # and one with nothing filtered
    ix = b200.IndexFlat(d, metric)
    ix.add_with_ids(xb, ids)
    D, I = ix.search_with_masks(xq, k, np.packbits(keep, axis=1, bitorder="little"))
    De, Ie = _expected(lambda b, q, kk, lab: oracle.flat_search(metric, b, q, kk, labels=lab), xb, ids, xq, keep, k)
    assert_exact(D, I, De, Ie)


def test_int8_masked(b200):
    n, nq, k, d = 90000, 7, 30, 64
    xb = datasets.uniform_int8(n, d, seed=21)
    xq = datasets.uniform_int8(nq, d, seed=22)
    ids = np.arange(n, dtype=np.int64)
    keep = np.random.default_rng(23).random((nq, n)) < 0.25
    ix = b200.IndexInt8Flat(d, IP)
    ix.add_with_ids(xb, ids)
    D, I = ix.search_with_masks(xq, k, np.packbits(keep, axis=1, bitorder="little"))
    De, Ie = _expected(lambda b, q, kk, lab: oracle.int8_search(IP, b, q, kk, labels=lab), xb, ids, xq, keep, k)
    assert_exact(D, I, De, Ie)


def test_masked_rejects_ivfpq_and_null(b200):
    ix = b200.IndexFlat(32, L2)
    ix.add(datasets.gaussian(100, 32, seed=1))
    with pytest.raises(ValueError):
        ix.search_with_masks(datasets.gaussian(2, 32, seed=2), 5, np.zeros((2, 3), np.uint8))
