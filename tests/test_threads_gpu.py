"""Host threads sharing one index handle.

The reference lets several threads search one index when MX_INDEX_MULTITHREAD=1
(feature_retrieval/src/ascendfaiss/ascend/impl/AscendIndexImpl.h:62,230: shared lock for search).
An index here owns one stream and one set of scratch buffers, so the C ABI serialises the calls on
a handle; the test runs searches of different sizes from several threads at once (ctypes releases
the GIL during the call) and compares every result with the single-threaded one.
"""
import threading

import numpy as np
import pytest

from indexsdk_b200 import datasets

pytestmark = pytest.mark.gpu


def _hammer(index, queries, k, expect, errors, rounds):
    try:
        for _ in range(rounds):
            for xq, (Dr, Ir) in zip(queries, expect):
                D, I = index.search(xq, k)
                if not (np.array_equal(I, Ir) and np.array_equal(D.view(np.uint32), Dr.view(np.uint32))):
                    errors.append("result differs from the single-threaded search")
                    return
    except Exception as e:  # noqa: BLE001 - reported to the main thread
        errors.append(repr(e))


def test_concurrent_searches_on_one_flat_index(b200):
    d, k = 64, 10
    ix = b200.IndexFlat(d, b200.METRIC_L2)
    ix.add(datasets.gaussian(30000, d, seed=0))
    # different batch sizes: scratch buffers would be re-sized under a concurrent reader
    queries = [datasets.gaussian(n, d, seed=10 + n) for n in (3, 200, 17, 900)]
    expect = [ix.search(xq, k) for xq in queries]
    errors = []
    threads = [threading.Thread(target=_hammer, args=(ix, queries[i:] + queries[:i], k, expect[i:] + expect[:i], errors, 6))
               for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]


def test_concurrent_searches_on_one_ivfpq_index(b200):
    d, nlist, M, k = 64, 64, 16, 10
    xb, _ = datasets.mixture(20000, d, nlist, seed=4)
    cent, cb = datasets.train_ivfpq(xb[:4000], nlist, M, True, niter=3)
    ix = b200.IndexIVFPQ(d, nlist, M, 8, by_residual=True)
    ix.set_centroids(cent)
    ix.set_codebooks(cb)
    ix.add(xb)
    ix.nprobe = 8
    queries = [datasets.mixture(n, d, nlist, seed=20 + n, centers_seed=4)[0] for n in (5, 1300, 64)]
    expect = [ix.search(xq, k) for xq in queries]
    errors = []
    threads = [threading.Thread(target=_hammer, args=(ix, queries[i:] + queries[:i], k, expect[i:] + expect[:i], errors, 4))
               for i in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
