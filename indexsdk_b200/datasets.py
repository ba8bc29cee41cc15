"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (they stand in for SIFT1M-style files, which are not redistributed here).

All generators are numpy Philox streams keyed by the seed, so any process regenerates the same
bytes.  ``scale`` < 1 shrinks row counts for tests; shapes otherwise follow the configurations.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=seed))


def gaussian(n: int, d: int, seed: int) -> np.ndarray:
    """i.i.d. N(0,1) float32 rows (Flat L2 configuration: base seed 0, queries seed 1)."""
    return _rng(seed).standard_normal((n, d), dtype=np.float32)


def uniform_int8(n: int, d: int, seed: int) -> np.ndarray:
    """int8 uniform in [-128, 127] (Int8Flat configuration: base seed 2, queries seed 3)."""
    return _rng(seed).integers(-128, 128, size=(n, d), dtype=np.int8)


def mixture(n: int, d: int, n_centers: int, seed: int, sigma: float = 0.1, centers_seed: int | None = None):
    """Gaussian mixture: centers ~ N(0,1), points = center + N(0, sigma^2).  Returns (points, centers).
    Base and queries of one configuration share centers_seed so they come from the same mixture."""
    cs = seed if centers_seed is None else centers_seed
    centers = _rng(1_000_003 * (cs + 1)).standard_normal((n_centers, d), dtype=np.float32)
    r = _rng(seed)
    which = r.integers(0, n_centers, size=n)
    pts = centers[which] + sigma * r.standard_normal((n, d), dtype=np.float32)
    return pts.astype(np.float32), centers


def unit_rows(n: int, d: int, seed: int) -> np.ndarray:
    """N(0,1) rows scaled to unit L2 norm (large-k inner-product configuration)."""
    x = gaussian(n, d, seed)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return x


def kmeans(x: np.ndarray, k: int, niter: int = 25, seed: int = 123) -> np.ndarray:
    """Seeded Lloyd k-means (float32, numpy); empty clusters are re-seeded from random points."""
    r = _rng(seed)
    n = x.shape[0]
    cent = x[r.choice(n, size=k, replace=n < k)].copy()
    xn = (x * x).sum(1)
    for _ in range(niter):
        assign = np.empty(n, np.int64)
        for s in range(0, n, 65536):
            xs = x[s:s + 65536]
            dist = xn[s:s + 65536, None] - 2.0 * xs @ cent.T + (cent * cent).sum(1)[None, :]
            assign[s:s + 65536] = dist.argmin(1)
        counts = np.bincount(assign, minlength=k)
        sums = np.zeros_like(cent)
        np.add.at(sums, assign, x)
        nz = counts > 0
        cent[nz] = sums[nz] / counts[nz, None]
        empty = np.flatnonzero(~nz)
        if empty.size:
            cent[empty] = x[r.choice(n, size=empty.size)]
    return cent.astype(np.float32)


def train_ivfpq(sample: np.ndarray, nlist: int, M: int, by_residual: bool, niter: int = 25, seed: int = 7):
    """Coarse centroids [nlist, d] and PQ codebooks [M, 256, d/M] from a training sample."""
    d = sample.shape[1]
    dsub = d // M
    cent = kmeans(sample, nlist, niter, seed)
    train = sample
    if by_residual:
        xn = (sample * sample).sum(1)
        assign = np.concatenate([
            (xn[s:s + 65536, None] - 2.0 * sample[s:s + 65536] @ cent.T + (cent * cent).sum(1)[None, :]).argmin(1)
            for s in range(0, sample.shape[0], 65536)])
        train = sample - cent[assign]
    cb = np.stack([kmeans(np.ascontiguousarray(train[:, m * dsub:(m + 1) * dsub]), 256, niter, seed + 1 + m)
                   for m in range(M)])
    return cent, cb.astype(np.float32)
