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
L2, IP = 1, 0


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
