"""GPU parity of exact Flat search (fp32 and fp16 modes) against the CPU oracle, through the
C ABI.  fp32 mode: bit-exact distances and identical ids (the GPU re-computes candidates with
the oracle's canonical fp32 arithmetic).  fp16 mode: 1e-3 relative, gap-aware ids."""
import os

import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets
from helpers import assert_close_gap_aware, assert_exact

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
L2, IP = 1, 0


@pytest.mark.parametrize("metric", [L2, IP])
def test_golden_fixture_fp32(b200, metric):
    g = np.load(os.path.join(GOLD, "flat_small.npz"))
    ix = b200.IndexFlat(64, metric)
    ix.add(g["xb"])
    D, I = ix.search(g["xq"], 10)
    name = "l2" if metric == L2 else "ip"
    assert_exact(D, I, g[f"D_{name}"], g[f"I_{name}"])


@pytest.mark.parametrize("n,nq,k,d", [(1000, 1, 1, 128), (1000, 7, 10, 128), (262144 + 17, 7, 100, 128),
                                      (50000, 130, 100, 128), (40000, 33, 37, 16), (30000, 5, 10, 768),
                                      (100, 3, 100, 32), (5, 2, 8, 16)])
@pytest.mark.parametrize("metric", [L2, IP])
def test_fp32_bit_exact_vs_oracle(b200, n, nq, k, d, metric):
    xb = datasets.gaussian(n, d, seed=100 + d)
    xq = datasets.gaussian(nq, d, seed=200 + d)
    ix = b200.IndexFlat(d, metric)
    ix.add(xb)
    assert ix.ntotal == n
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.flat_search(metric, xb, xq, k)
    assert_exact(D, I, Dr, Ir)
    # and within 1e-5 relative of the fp64-accumulated value
    Dp, _ = oracle.flat_search(metric, xb, xq, k, precise=True)
    real = Ir >= 0
    np.testing.assert_allclose(D[real], Dp[real], rtol=1e-5, atol=1e-5 if metric == IP else 0)


def test_fp32_duplicates_ties_and_overflow_fallback(b200):
    """Heavy ties: many copies of the same vectors overflow the candidate buffers; the
    no-threshold re-run must still return the lowest positions first."""
    base = datasets.gaussian(16, 32, seed=5)
    xb = np.tile(base, (32768, 1))         # 524288 rows, each distinct vector 32768 times
    xq = base[:3] + 0.0
    ix = b200.IndexFlat(32, L2)
    ix.add(xb)
    D, I = ix.search(xq, 50)
    Dr, Ir = oracle.flat_search(L2, xb, xq, 50)
    assert_exact(D, I, Dr, Ir)
    assert np.all(D == 0) and I[0].tolist() == [16 * j for j in range(50)]
    assert ix.stats()["fallback_queries"] == 3


def test_fp32_add_with_ids_incremental_reset_remove(b200):
    d = 64
    xb = datasets.gaussian(5000, d, seed=7)
    xq = datasets.gaussian(9, d, seed=8)
    ids = (np.arange(5000) * 7 + 3).astype(np.int64)
    ix = b200.IndexFlat(d, L2)
    ix.add_with_ids(xb[:2000], ids[:2000])
    ix.add_with_ids(xb[2000:], ids[2000:])
    D, I = ix.search(xq, 10)
    Dr, Ir = oracle.flat_search(L2, xb, xq, 10, labels=ids)
    assert_exact(D, I, Dr, Ir)
    np.testing.assert_array_equal(ix.get_base(100, 5), xb[100:105])
    np.testing.assert_array_equal(ix.get_ids(4990, 10), ids[4990:])
    # remove: swap-with-last compaction keeps the remaining set searchable
    removed = ix.remove_ids(ids[[0, 17, 4999]])
    assert removed == 3 and ix.ntotal == 4997
    keep = np.ones(5000, bool)
    keep[[0, 17, 4999]] = False
    D, I = ix.search(xq, 10)
    base_now, ids_now = ix.get_base(), ix.get_ids()
    assert sorted(ids_now.tolist()) == sorted(ids[keep].tolist())
    Dr, Ir = oracle.flat_search(L2, base_now, xq, 10, labels=ids_now)
    assert_exact(D, I, Dr, Ir)
    ix.reset()
    assert ix.ntotal == 0
    D, I = ix.search(xq, 4)
    assert np.all(I == -1) and np.all(D == np.finfo(np.float32).max)
    ix.add(xb[:300])
    D, I = ix.search(xq, 4)
    Dr, Ir = oracle.flat_search(L2, xb[:300], xq, 4)
    assert_exact(D, I, Dr, Ir)


@pytest.mark.parametrize("metric", [L2, IP])
@pytest.mark.parametrize("n,nq,k,d", [(20000, 9, 10, 128), (70000, 140, 100, 256), (3000, 4, 1000, 64)])
def test_fp16_mode_vs_oracle(b200, metric, n, nq, k, d):
    xb = datasets.gaussian(n, d, seed=300 + d)
    xq = datasets.gaussian(nq, d, seed=400 + d)
    ix = b200.IndexFlat(d, metric, dtype=b200.F16)
    ix.add(xb)
    D, I = ix.search(xq, k)
    xb16, xq16 = oracle.round_fp16(xb), oracle.round_fp16(xq)
    Dr, Ir = oracle.flat_search(metric, xb16, xq16, k, precise=True)
    assert_close_gap_aware(D, I, Dr, Ir, rtol=1e-3, what="fp16 flat")
    # fp16 bit inputs take the same path
    D2, I2 = ix.search_f16(xq.astype(np.float16).view(np.uint16), k)
    np.testing.assert_array_equal(I2, I)
    np.testing.assert_array_equal(D2, D)
    np.testing.assert_array_equal(ix.get_base(0, 3), xb[:3].astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("d", [144, 160])
def test_fp32_operand_layouts_grow_and_remove(b200, d):
    """d = 144 is the widest index whose operand copy is kept in the packed (tile image) layout,
    d = 160 the first that keeps rows: both must survive growth of the buffers over several adds
    that end inside a tile, and the removal of rows (which moves the last row into the gap)."""
    n_parts = [300, 70000, 5, 1111]
    n = sum(n_parts)
    xb = datasets.gaussian(n, d, seed=31)
    xq = datasets.gaussian(21, d, seed=32)
    ids = (np.arange(n) * 3 + 1).astype(np.int64)
    ix = b200.IndexFlat(d, L2)
    o = 0
    for m in n_parts:
        ix.add_with_ids(xb[o:o + m], ids[o:o + m])
        o += m
        D, I = ix.search(xq, 10)
        Dr, Ir = oracle.flat_search(L2, xb[:o], xq, 10, labels=ids[:o])
        assert_exact(D, I, Dr, Ir)
    gone = ids[[0, 255, 256, 300, 70299, n - 1]]
    assert ix.remove_ids(gone) == 6
    base_now, ids_now = ix.get_base(), ix.get_ids()
    D, I = ix.search(xq, 50)
    Dr, Ir = oracle.flat_search(L2, base_now, xq, 50, labels=ids_now)
    assert_exact(D, I, Dr, Ir)
    assert not set(gone.tolist()) & set(I.ravel().tolist())


def test_self_hit_rank_one(b200):
    """The property the reference's device test asserts (TestAscendIndexFlat.cpp:117-123)."""
    xb = datasets.gaussian(20000, 128, seed=9)
    for dtype in (b200.F32, b200.F16):
        ix = b200.IndexFlat(128, L2, dtype=dtype)
        ix.add(xb)
        D, I = ix.search(xb[:200], 5)
        assert I[:, 0].tolist() == list(range(200))


def test_simt_cross_check_matches_tensor_path(b200, monkeypatch):
    """The CUDA-core variant of the distance kernel and the tcgen05 variant feed the same
    selection; in fp32 mode both must give the oracle's bits."""
    xb = datasets.gaussian(9000, 64, seed=1)
    xq = datasets.gaussian(5, 64, seed=2)
    Dr, Ir = oracle.flat_search(L2, xb, xq, 20)
    monkeypatch.setenv("B200IDX_GEMM", "simt")
    ix = b200.IndexFlat(64, L2)
    ix.add(xb)
    D, I = ix.search(xq, 20)
    assert_exact(D, I, Dr, Ir)


def test_argument_errors(b200):
    ix = b200.IndexFlat(64, L2)
    ix.add(datasets.gaussian(10, 64, seed=1))
    with pytest.raises(b200.B200IdxError) as e:
        ix.search(datasets.gaussian(2, 64, seed=2), 5000)
    assert e.value.code == 2001 and "k must be > 0 and <= 4096" in e.value.msg
    with pytest.raises(b200.B200IdxError) as e:
        b200.IndexFlat(100, L2)
    assert "Unsupported dims" in e.value.msg
