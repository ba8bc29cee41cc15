"""Seeded sweeps over random shapes: every result is compared with the CPU oracle (bit-exact for
fp32 / int8 indexes and for IVFPQ, within 1e-3 for fp16 storage).  The unit tests pin chosen
shapes; these walk the combinations in between -- dimensions on both sides of the packed-operand
limit, bases that end inside a tile and are added in pieces, every metric, every code width."""
import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets

pytestmark = pytest.mark.gpu


def test_flat_and_int8_random_shapes(b200):
    rng = np.random.default_rng(12345)
    for it in range(40):
        d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 256]))
        n = int(rng.integers(1, 120000))
        nq = int(rng.integers(1, 300))
        k = int(rng.choice([1, 5, 10, 37, 100, 200]))
        kind = str(rng.choice(["f32", "f32", "f32", "f16", "i8"]))
        metric = int(rng.integers(0, 3 if kind == "i8" else 2))      # int8: also the fp16 cosine
        cuts = sorted(set([0, n] + [int(x) for x in rng.integers(0, n + 1, size=int(rng.integers(0, 3)))]))
        if kind == "i8":
            xb = datasets.uniform_int8(n, d, seed=it)
            xq = datasets.uniform_int8(nq, d, seed=1000 + it)
            ix = b200.IndexInt8Flat(d, metric)
        else:
            xb = datasets.gaussian(n, d, seed=it)
            xq = datasets.gaussian(nq, d, seed=1000 + it)
            if kind == "f16":
                xb, xq = oracle.round_fp16(xb), oracle.round_fp16(xq)
            ix = b200.IndexFlat(d, metric, dtype=b200.F16 if kind == "f16" else b200.F32)
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            ix.add(xb[lo:hi])
        D, I = ix.search(xq, k)
        Dr, Ir = (oracle.int8_search if kind == "i8" else oracle.flat_search)(metric, xb, xq, k)
        what = f"case {it}: {kind} metric {metric} d {d} n {n} nq {nq} k {k} adds {cuts}"
        if kind == "f16":
            assert (I == Ir).mean() > 0.995, what
            np.testing.assert_allclose(D[Ir >= 0], Dr[Ir >= 0], rtol=1e-3, atol=1e-3, err_msg=what)
        else:
            assert np.array_equal(I, Ir) and np.array_equal(D, Dr), what


def test_ivfpq_random_configurations(b200):
    rng = np.random.default_rng(777)
    shapes = [(128, 16), (96, 48), (64, 16), (128, 32), (64, 8), (128, 64), (96, 16), (48, 48), (64, 32)]
    for it in range(18):
        d, M = shapes[it % len(shapes)]
        nlist = int(rng.choice([16, 40, 64, 128]))
        n = int(rng.integers(2000, 40000))
        nq = int(rng.choice([3, 40, 300, 1100]))
        nprobe = int(min(nlist, rng.choice([1, 4, 16, 64, 128])))
        k = int(rng.choice([1, 10, 32, 100]))
        resid = bool(rng.integers(0, 2))
        sigma = float(rng.choice([0.1, 0.5, 1.0]))
        xb, _ = datasets.mixture(n, d, nlist, seed=100 + it, sigma=sigma)
        xq, _ = datasets.mixture(nq, d, nlist, seed=500 + it, sigma=sigma, centers_seed=100 + it)
        cent, cb = datasets.train_ivfpq(xb[:min(n, 6000)], nlist, M, resid, niter=3)
        ids = np.arange(n, dtype=np.int64) * 2 + 1
        ix = b200.IndexIVFPQ(d, nlist, M, 8, by_residual=resid)
        ix.set_centroids(cent)
        ix.set_codebooks(cb)
        ix.add_with_ids(xb[:n // 2], ids[:n // 2])
        ix.add_with_ids(xb[n // 2:], ids[n // 2:])
        ix.nprobe = nprobe
        D, I = ix.search(xq, k)
        ln = oracle.ivf_assign(cent, xb)
        codes = oracle.pq_encode(cb, xb, resid, cent, ln)
        off, cs, li = oracle.build_lists(ln, codes, ids, nlist)
        Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, li, xq, nprobe, k)
        what = f"case {it}: d {d} M {M} nlist {nlist} n {n} nq {nq} nprobe {nprobe} k {k} residual {resid} sigma {sigma}"
        assert np.array_equal(I, Ir) and np.array_equal(D, Dr), what
