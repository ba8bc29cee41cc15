"""GPU parity of IVFPQ (assignment, PQ encoding, three-stage search) against the CPU oracle.

Both encodings -- raw vectors (the reference's mode) and residuals (Faiss default, one table per
(query, list) in the oracle) -- must give codes, list contents, distances and ids that are
bit-identical to the oracle: the GPU's scan is a filter whose survivors are re-computed in the
oracle's canonical arithmetic and verified, with an exact re-scan for queries that fail the check."""
import os

import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets
from helpers import assert_exact

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _build(b200, xb, ids, cent, cb, resid, chunks=1):
    nlist, M = cent.shape[0], cb.shape[0]
    ix = b200.IndexIVFPQ(xb.shape[1], nlist, M, 8, by_residual=resid)
    ix.set_centroids(cent)
    ix.set_codebooks(cb)
    for part, idp in zip(np.array_split(xb, chunks), np.array_split(ids, chunks)):
        ix.add_with_ids(part, idp)
    return ix


def _oracle_lists(xb, ids, cent, cb, resid):
    ln = oracle.ivf_assign(cent, xb)
    codes = oracle.pq_encode(cb, xb, resid, cent, ln)
    return ln, codes, oracle.build_lists(ln, codes, ids, cent.shape[0])


@pytest.mark.parametrize("tag,resid", [("raw", False), ("res", True)])
def test_golden_fixture(b200, tag, resid):
    g = np.load(os.path.join(GOLD, "ivfpq_small.npz"))
    xb = g["xb"]
    ids = np.arange(xb.shape[0], dtype=np.int64)
    ix = _build(b200, xb, ids, g[f"cent_{tag}"], g[f"cb_{tag}"], resid)
    off, cs, idl = oracle.build_lists(g[f"list_no_{tag}"], g[f"codes_{tag}"], ids, 16)
    for l in range(16):
        codes, lid = ix.get_list(l)
        np.testing.assert_array_equal(codes, cs[off[l]:off[l + 1]])
        np.testing.assert_array_equal(lid, idl[off[l]:off[l + 1]])
    ix.nprobe = 4
    D, I = ix.search(g["xq"], 10)
    assert_exact(D, I, g[f"D_{tag}"], g[f"I_{tag}"])


@pytest.mark.parametrize("resid", [False, True])
@pytest.mark.parametrize("d,nlist,M,n,nq,nprobe,k,chunks", [
    (128, 256, 16, 60000, 50, 16, 10, 3),
    (128, 64, 16, 20000, 300, 64, 100, 1),
    (128, 64, 16, 20000, 1500, 24, 10, 1),     # large batch of 16-byte codes: the persistent scan kernel
    (64, 48, 16, 9000, 1300, 48, 40, 1),       # the same with k' = 64
    (96, 128, 48, 30000, 20, 32, 100, 2),
    (64, 32, 8, 5000, 9, 8, 320, 1),
    (128, 100, 32, 8000, 4, 100, 1, 1),
    (64, 16, 4, 3000, 1, 1, 5, 1),
])
def test_search_vs_oracle(b200, resid, d, nlist, M, n, nq, nprobe, k, chunks):
    xb, _ = datasets.mixture(n, d, max(nlist // 2, 4), seed=4)
    xq, _ = datasets.mixture(nq, d, max(nlist // 2, 4), seed=5, centers_seed=4)
    ids = (np.arange(n, dtype=np.int64) * 5 + 11)
    cent, cb = datasets.train_ivfpq(xb[: min(n, 8000)], nlist, M, resid, niter=4)
    ix = _build(b200, xb, ids, cent, cb, resid, chunks)
    assert ix.ntotal == n
    ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, resid)
    assert [ix.list_length(l) for l in range(nlist)] == np.diff(off).tolist()
    for l in (0, nlist // 2, nlist - 1):
        c, i = ix.get_list(l)
        np.testing.assert_array_equal(c, cs[off[l]:off[l + 1]])
        np.testing.assert_array_equal(i, idl[off[l]:off[l + 1]])
    ix.nprobe = nprobe
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, idl, xq, nprobe, k)
    assert_exact(D, I, Dr, Ir)


def test_empty_lists_duplicates_and_short_results(b200):
    d, nlist, M = 64, 32, 16
    xb, _ = datasets.mixture(600, d, 4, seed=9)
    xb = np.concatenate([xb, xb[:100]])          # duplicates -> identical codes -> distance ties
    ids = np.arange(700, dtype=np.int64)[::-1].copy()
    cent, cb = datasets.train_ivfpq(xb, nlist, M, False, niter=3)
    cent[3] = 50.0                                # an empty, far list
    ix = _build(b200, xb, ids, cent, cb, False)
    ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, False)
    xq = xb[:40]
    padded = False
    for nprobe, k in ((nlist, 64), (1, 300), (2, 10)):
        ix.nprobe = nprobe
        D, I = ix.search(xq, k)
        Dr, Ir = oracle.ivfpq_search(cent, cb, False, off, cs, idl, xq, nprobe, k)
        assert_exact(D, I, Dr, Ir)
        padded |= bool((Ir[:, -1] == -1).any())
    assert padded                                 # nprobe=1, k=300 leaves padded tails


@pytest.mark.parametrize("resid", [False, True])
@pytest.mark.parametrize("copies,second_pass", [(200, True), (1500, False)])
def test_more_duplicates_than_the_filter_keeps(b200, resid, copies, second_pass):
    """Many copies of each vector: the filter keeps k' = 32 candidates per query, the top ties are
    wider than that and the verification must fail.  With 200 copies the second filter pass (fixed
    threshold, every tied vector collected, exact order by label) settles the query; with 1500
    copies more vectors lie under its threshold than it can hold and the exact re-scan takes over.
    Either way the lowest labels among the tied vectors must come back."""
    d, nlist, M = 64, 8, 16
    base, _ = datasets.mixture(40, d, 4, seed=3)
    xb = np.repeat(base, copies, axis=0)
    ids = np.random.default_rng(0).permutation(xb.shape[0]).astype(np.int64)
    cent, cb = datasets.train_ivfpq(base, nlist, M, resid, niter=3)
    ix = _build(b200, xb, ids, cent, cb, resid, chunks=2)
    ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, resid)
    ix.nprobe = nlist
    xq = base[:12]
    D, I = ix.search(xq, 10)
    Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, idl, xq, nlist, 10)
    assert_exact(D, I, Dr, Ir)
    st = ix.stats()
    assert st["second_pass_queries"] == 12
    assert st["fallback_queries"] == (0 if second_pass else 12)


def test_exact_scan_kernels_alone(b200, monkeypatch):
    """B200IDX_IVFPQ_EXACT=1 routes every query through the canonical-arithmetic scan kernels
    (per-(query, list) tables in shared memory for residual encoding)."""
    monkeypatch.setenv("B200IDX_IVFPQ_EXACT", "1")
    d, nlist, M = 64, 32, 16
    xb, _ = datasets.mixture(6000, d, 16, seed=4)
    xq, _ = datasets.mixture(9, d, 16, seed=5, centers_seed=4)
    ids = np.arange(6000, dtype=np.int64)
    for resid in (False, True):
        cent, cb = datasets.train_ivfpq(xb, nlist, M, resid, niter=3)
        ix = _build(b200, xb, ids, cent, cb, resid)
        ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, resid)
        ix.nprobe = 8
        D, I = ix.search(xq, 20)
        Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, idl, xq, 8, 20)
        assert_exact(D, I, Dr, Ir)


def test_add_codes_reset_remove(b200):
    d, nlist, M = 64, 16, 8
    xb, _ = datasets.mixture(3000, d, 8, seed=21)
    xq, _ = datasets.mixture(7, d, 8, seed=22, centers_seed=21)
    ids = np.arange(3000, dtype=np.int64)
    cent, cb = datasets.train_ivfpq(xb, nlist, M, True, niter=3)
    ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, True)
    ix = b200.IndexIVFPQ(d, nlist, M, 8, by_residual=True)
    ix.set_centroids(cent)
    ix.set_codebooks(cb)
    ix.add_codes(ln, codes, ids)                  # the copyFrom path: pre-encoded lists
    ix.nprobe = 8
    D, I = ix.search(xq, 10)
    ix2 = _build(b200, xb, ids, cent, cb, True)
    ix2.nprobe = 8
    D2, I2 = ix2.search(xq, 10)
    assert_exact(D, I, D2, I2)
    # reset + re-add gives byte-identical lists (TestAscendIndexIVFPQ.cpp:118-146)
    before = [ix2.get_list(l) for l in range(nlist)]
    ix2.reset()
    assert ix2.ntotal == 0
    ix2.add_with_ids(xb, ids)
    for l in range(nlist):
        c, i = ix2.get_list(l)
        np.testing.assert_array_equal(c, before[l][0])
        np.testing.assert_array_equal(i, before[l][1])
    assert ix.remove_ids(np.array([5, 6, 7, 99999])) == 3
    keep = ~np.isin(ids, [5, 6, 7])
    off2, cs2, idl2 = oracle.build_lists(ln[keep], codes[keep], ids[keep], nlist)
    D, I = ix.search(xq, 10)
    Dr, Ir = oracle.ivfpq_search(cent, cb, True, off2, cs2, idl2, xq, 8, 10)
    assert_exact(D, I, Dr, Ir)


def test_untrained_index_is_rejected(b200):
    ix = b200.IndexIVFPQ(64, 16, 8)
    with pytest.raises(b200.B200IdxError) as e:
        ix.add(datasets.gaussian(10, 64, seed=1))
    assert e.value.code == 2001 and "not trained" in e.value.msg


@pytest.mark.parametrize("bad", [np.nan, np.inf])
def test_vectors_without_a_nearest_centroid_are_refused(b200, bad):
    """A NaN or infinite component leaves a vector without a nearest centroid; its assignment would be -1 and must never index a list.  The
    batch is refused with INVALID_PARAM and the index is left as it was -- from host and from
    device memory, for add and for training."""
    import torch
    d, nlist, M = 32, 16, 4
    xb, _ = datasets.mixture(3000, d, nlist, seed=4)
    cent, cb = datasets.train_ivfpq(xb[:2000], nlist, M, False, niter=3)
    ix = _build(b200, xb[:1000], np.arange(1000, dtype=np.int64), cent, cb, False)
    before = [ix.get_list(l) for l in range(nlist)]
    poisoned = xb[1000:1500].copy()
    poisoned[123, 7] = bad
    with pytest.raises(b200.B200IdxError) as e:
        ix.add_with_ids(poisoned, np.arange(1000, 1500, dtype=np.int64))
    assert e.value.code == 2001
    xd = torch.from_numpy(poisoned).cuda()
    with pytest.raises(b200.B200IdxError) as e:
        ix.add_device(xd.data_ptr(), xd.shape[0], np.arange(1000, 1500, dtype=np.int64))
    assert e.value.code == 2001
    assert ix.ntotal == 1000
    for l in range(nlist):
        c, i = ix.get_list(l)
        assert np.array_equal(c, before[l][0]) and np.array_equal(i, before[l][1])
    # the index still works
    ix.add_with_ids(xb[1000:1500], np.arange(1000, 1500, dtype=np.int64))
    assert ix.ntotal == 1500
    fresh = b200.IndexIVFPQ(d, nlist, M, 8)
    with pytest.raises(b200.B200IdxError) as e:
        fresh.train(np.concatenate([xb[:2000], poisoned]), niter=2, seed=1)
    assert e.value.code == 2001
    with pytest.raises(b200.B200IdxError) as e:
        b200.kmeans(poisoned, 8, niter=2)
    assert e.value.code == 2001


@pytest.mark.parametrize("resid", [False, True])
def test_coarse_plus_preassigned_equals_search(b200, resid):
    """The two halves of a search run apart -- probes selected for slices of the queries, as the
    ranks of a sharded index do, then the scan with those probes -- give the plain search's result."""
    import torch
    d, nlist, M, n, nq, nprobe, k = 64, 64, 16, 20000, 257, 12, 10
    xb, _ = datasets.mixture(n, d, 32, seed=14)
    xq, _ = datasets.mixture(nq, d, 32, seed=15, centers_seed=14)
    ids = np.arange(n, dtype=np.int64) * 3 + 1
    cent, cb = datasets.train_ivfpq(xb[:8000], nlist, M, resid, niter=4)
    ix = _build(b200, xb, ids, cent, cb, resid)
    ix.nprobe = nprobe
    D0, I0 = ix.search(xq, k)
    dev = torch.device("cuda", ix.device)
    xq_d = torch.from_numpy(xq).to(dev)
    cD = torch.empty((nq, nprobe), dtype=torch.float32, device=dev)
    cI = torch.empty((nq, nprobe), dtype=torch.int64, device=dev)
    torch.cuda.synchronize(dev)
    for lo, hi in ((0, 100), (100, 101), (101, nq)):            # three "ranks"
        ix.coarse_device(xq_d[lo:hi].data_ptr(), hi - lo, cD[lo:hi].data_ptr(), cI[lo:hi].data_ptr())
    D = torch.empty((nq, k), dtype=torch.float32, device=dev)
    I = torch.empty((nq, k), dtype=torch.int64, device=dev)
    ix.search_preassigned_device(xq_d.data_ptr(), nq, k, cD.data_ptr(), cI.data_ptr(), D.data_ptr(), I.data_ptr())
    torch.cuda.synchronize(dev)
    assert_exact(D.cpu().numpy(), I.cpu().numpy(), D0, I0)
    # the probes themselves: the oracle's coarse quantizer (same lists in the same order)
    off, cs, idl = _oracle_lists(xb, ids, cent, cb, resid)[2]
    _, _, coarse = oracle.ivfpq_search(cent, cb, resid, off, cs, idl, xq, nprobe, k, return_coarse=True)
    np.testing.assert_array_equal(cI.cpu().numpy(), coarse.astype(np.int64))


@pytest.mark.parametrize("nlist,n,nq,nprobe,k", [
    (64, 20000, 1500, 24, 10),       # ~560 queries per list: several query chunks per list
    (256, 60000, 1300, 16, 16),      # shorter lists, tails of the 128-code tiles
    (1024, 50000, 2000, 64, 1),      # few queries per list, lists shorter than one tile
])
def test_tensor_core_scan_vs_oracle(b200, monkeypatch, nlist, n, nq, nprobe, k):
    """B200IDX_IVFPQ_TC=1: large batches on a residual-encoded d = 128, M = 16 index take the
    list-major tensor-core filter (decode once per list, fp16 two-term product, threshold from a
    table scan of the nearest lists).  Results must stay bit-identical to the oracle, and only a
    small part of the queries may need the exact re-scan."""
    monkeypatch.setenv("B200IDX_IVFPQ_TC", "1")
    d, M = 128, 16
    xb, _ = datasets.mixture(n, d, max(nlist // 2, 4), seed=14)
    xq, _ = datasets.mixture(nq, d, max(nlist // 2, 4), seed=15, centers_seed=14)
    ids = (np.arange(n, dtype=np.int64) * 3 + 7)
    cent, cb = datasets.train_ivfpq(xb[:8000], nlist, M, True, niter=4)
    ix = _build(b200, xb, ids, cent, cb, True, 2)
    ln, codes, (off, cs, idl) = _oracle_lists(xb, ids, cent, cb, True)
    ix.nprobe = nprobe
    D, I = ix.search(xq, k)
    Dr, Ir = oracle.ivfpq_search(cent, cb, True, off, cs, idl, xq, nprobe, k)
    assert_exact(D, I, Dr, Ir)
    st = ix.stats()
    assert st["fallback_queries"] <= nq // 10
    assert st["scan_codes"] > 0
