"""Device k-means training against its CPU restatement: same start, same assignment arithmetic,
same summation order -- the centroids must agree bit for bit."""
import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,d,k,niter,seed", [
    (5000, 64, 32, 6, 0),        # assignment through the Flat fp32 search (tensor-core filter + exact refinement)
    (20000, 128, 300, 4, 7),
    (8000, 8, 256, 5, 3),        # a PQ sub-space: direct assignment kernel
    (3000, 2, 256, 3, 11),
    (600, 16, 600, 2, 1),        # k = n: every start distinct, most clusters single
])
def test_kmeans_matches_oracle(b200, n, d, k, niter, seed):
    x, _ = datasets.mixture(n, d, max(4, min(k, 64)), seed=20 + d)
    got = b200.kmeans(x, k, niter, seed)
    want = oracle.kmeans(x, k, niter, seed)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("resid", [False, True])
def test_ivfpq_train_matches_composed_oracle(b200, resid):
    d, nlist, M, n, niter, seed = 64, 24, 16, 9000, 4, 5
    x, _ = datasets.mixture(n, d, 16, seed=31)
    ix = b200.IndexIVFPQ(d, nlist, M, 8, by_residual=resid)
    ix.train(x, niter, seed)
    cent = oracle.kmeans(x, nlist, niter, seed)
    np.testing.assert_array_equal(ix.get_centroids(), cent)
    res = x - cent[oracle.ivf_assign(cent, x)] if resid else x
    dsub = d // M
    cb = np.stack([oracle.kmeans(np.ascontiguousarray(res[:, m * dsub:(m + 1) * dsub]), 256, niter, seed + 1 + m)
                   for m in range(M)])
    np.testing.assert_array_equal(ix.get_codebooks(), cb)
    # and the trained index searches like the oracle
    ids = np.arange(n, dtype=np.int64)
    ix.add_with_ids(x, ids)
    ix.nprobe = 6
    xq, _ = datasets.mixture(11, d, 16, seed=32, centers_seed=31)
    D, I = ix.search(xq, 10)
    ln = oracle.ivf_assign(cent, x)
    codes = oracle.pq_encode(cb, x, resid, cent, ln)
    off, cs, idl = oracle.build_lists(ln, codes, ids, nlist)
    Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, idl, xq, 6, 10)
    np.testing.assert_array_equal(I, Ir)
    np.testing.assert_array_equal(D, Dr)
