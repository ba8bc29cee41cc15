"""Regenerates tests/golden/*.npz.

The reference ships no golden vectors for the search path (its unit tests run on a mock
runtime whose operators write zeros), so these fixtures are produced by this repository's CPU
oracle (oracle/oracle.c) on small seeded inputs and cross-checked against the independent
float64 numpy mirror before being written.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from indexsdk_b200 import datasets  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def flat_case():
    xb = datasets.gaussian(3000, 64, seed=0)
    xq = datasets.gaussian(37, 64, seed=1)
    out = {"xb": xb, "xq": xq}
    for name, metric in (("l2", oracle.METRIC_L2), ("ip", oracle.METRIC_IP)):
        D, I = oracle.flat_search(metric, xb, xq, 10)
        Dn, In = oracle.np_flat_search(metric, xb, xq, 10)
        assert np.array_equal(I, In) and np.allclose(D, Dn, rtol=1e-5)
        out[f"D_{name}"], out[f"I_{name}"] = D, I
    np.savez_compressed(os.path.join(OUT, "flat_small.npz"), **out)


def int8_case():
    xb = datasets.uniform_int8(2500, 64, seed=2)
    xq = datasets.uniform_int8(19, 64, seed=3)
    out = {"xb": xb, "xq": xq}
    for name, metric in (("l2", oracle.METRIC_L2), ("ip", oracle.METRIC_IP)):
        D, I = oracle.int8_search(metric, xb, xq, 12)
        Dn, In = oracle.np_int8_search(metric, xb, xq, 12)
        assert np.array_equal(I, In) and np.array_equal(D, Dn)
        out[f"D_{name}"], out[f"I_{name}"] = D, I
    np.savez_compressed(os.path.join(OUT, "int8_small.npz"), **out)


def ivfpq_case():
    d, nlist, M = 32, 16, 4
    xb, _ = datasets.mixture(4000, d, 16, seed=4)
    xq, _ = datasets.mixture(23, d, 16, seed=5, centers_seed=4)
    out = {"xb": xb, "xq": xq}
    for tag, resid in (("raw", False), ("res", True)):
        cent, cb = datasets.train_ivfpq(xb[:2000], nlist, M, resid, niter=8)
        ln = oracle.ivf_assign(cent, xb)
        codes = oracle.pq_encode(cb, xb, resid, cent, ln)
        off, cs, ids = oracle.build_lists(ln, codes, np.arange(xb.shape[0]), nlist)
        D, I = oracle.ivfpq_search(cent, cb, resid, off, cs, ids, xq, 4, 10)
        Dn, In = oracle.np_ivfpq_search(cent, cb, resid, off, cs, ids, xq, 4, 10)
        assert np.allclose(D, Dn, rtol=2e-5), np.abs(D - Dn).max()
        assert (I == In).mean() > 0.99
        out.update({f"cent_{tag}": cent, f"cb_{tag}": cb, f"list_no_{tag}": ln, f"codes_{tag}": codes,
                    f"D_{tag}": D, f"I_{tag}": I})
    np.savez_compressed(os.path.join(OUT, "ivfpq_small.npz"), **out)


if __name__ == "__main__":
    flat_case()
    int8_case()
    ivfpq_case()
    print("golden fixtures written to", OUT)
