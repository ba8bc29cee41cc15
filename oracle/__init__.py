"""ctypes binding of the CPU oracle (``oracle/oracle.c``) plus an independent numpy mirror.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; tests,
``__graft_entry__.smoke()`` and the benchmark's CPU-baseline leg use it as the checker.

PARITY UNPINNED: the reference ships no golden vectors for this path and its CPU ground
truth (Faiss) is not vendored; see the header of ``oracle.c`` for the call sites the
restatement is anchored on.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

METRIC_IP = 0
METRIC_L2 = 1
METRIC_INT8_COS = 2      # int8 only: the reference's fp16 cosine (oracle.c, cos16_*)


def build(force: bool = False) -> str:
    """Compile oracle.c with the committed Makefile; returns the library path."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def flat_search(metric, xb, xq, k, labels=None, precise=False):
    xb, xq = _f32(xb), _f32(xq)
    nb, d = xb.shape
    nq = xq.shape[0]
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    lab = None if labels is None else np.ascontiguousarray(labels, dtype=np.int64)
    rc = lib().orc_flat_search(C.c_int(metric), C.c_int(d), C.c_int64(nb), _p(xb, C.c_float),
                               _p(lab, C.c_int64), C.c_int64(nq), _p(xq, C.c_float), C.c_int(k),
                               C.c_int(int(precise)), _p(D, C.c_float), _p(I, C.c_int64))
    if rc:
        raise RuntimeError(f"orc_flat_search rc={rc}")
    return D, I


def round_fp16(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_round_fp16(C.c_int64(x.size), _p(x, C.c_float), _p(out, C.c_float))
    return out


def round_bf16(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_round_bf16(C.c_int64(x.size), _p(x, C.c_float), _p(out, C.c_float))
    return out


def int8_search(metric, xb, xq, k, labels=None):
    xb = np.ascontiguousarray(xb, dtype=np.int8)
    xq = np.ascontiguousarray(xq, dtype=np.int8)
    nb, d = xb.shape
    nq = xq.shape[0]
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    lab = None if labels is None else np.ascontiguousarray(labels, dtype=np.int64)
    rc = lib().orc_int8_search(C.c_int(metric), C.c_int(d), C.c_int64(nb), _p(xb, C.c_int8),
                               _p(lab, C.c_int64), C.c_int64(nq), _p(xq, C.c_int8), C.c_int(k),
                               _p(D, C.c_float), _p(I, C.c_int64))
    if rc:
        raise RuntimeError(f"orc_int8_search rc={rc}")
    return D, I


def cos16(dot, sq_x, sq_q):
    """One fp16 cosine score from the exact dot product and squared norms (oracle.c: cos16_score)."""
    f = lib().orc_cos16
    f.restype = C.c_float
    return float(f(C.c_int32(int(dot)), C.c_int32(int(sq_x)), C.c_int32(int(sq_q))))


def f2h(x):
    f = lib().orc_f2h
    f.restype = C.c_uint16
    return int(f(C.c_float(x)))


def h2f(h):
    f = lib().orc_h2f
    f.restype = C.c_float
    return float(f(C.c_uint16(h)))


def ivf_assign(centroids, x):
    centroids, x = _f32(centroids), _f32(x)
    nlist, d = centroids.shape
    out = np.empty(x.shape[0], np.int32)
    lib().orc_ivf_assign(C.c_int(d), C.c_int(nlist), _p(centroids, C.c_float), C.c_int64(x.shape[0]),
                         _p(x, C.c_float), _p(out, C.c_int32))
    return out


def pq_encode(codebooks, x, by_residual=False, centroids=None, list_no=None):
    """codebooks: [M, ksub, dsub] float32 -> codes [n, M] uint8."""
    codebooks, x = _f32(codebooks), _f32(x)
    M, ksub, dsub = codebooks.shape
    n, d = x.shape
    assert d == M * dsub
    codes = np.empty((n, M), np.uint8)
    cen = None if centroids is None else _f32(centroids)
    ln = None if list_no is None else np.ascontiguousarray(list_no, dtype=np.int32)
    rc = lib().orc_pq_encode(C.c_int(d), C.c_int(M), C.c_int(ksub), _p(codebooks, C.c_float),
                             C.c_int(int(by_residual)), _p(cen, C.c_float), _p(ln, C.c_int32),
                             C.c_int64(n), _p(x, C.c_float), _p(codes, C.c_uint8))
    if rc:
        raise RuntimeError(f"orc_pq_encode rc={rc}")
    return codes


def build_lists(list_no, codes, ids, nlist):
    """Stable bucket by list -> (list_offsets[nlist+1], codes_sorted, ids_sorted)."""
    order = np.argsort(list_no, kind="stable")
    counts = np.bincount(list_no, minlength=nlist)
    offsets = np.zeros(nlist + 1, np.int64)
    np.cumsum(counts, out=offsets[1:])
    return offsets, np.ascontiguousarray(codes[order]), np.ascontiguousarray(ids[order].astype(np.int64))


def ivfpq_search(centroids, codebooks, by_residual, list_offsets, codes, ids, xq, nprobe, k,
                 return_coarse=False):
    """by_residual: False raw vectors (one table per query), True residual encoding (one table
    per (query, list) on q - centroid)."""
    centroids, codebooks, xq = _f32(centroids), _f32(codebooks), _f32(xq)
    nlist, d = centroids.shape
    M, ksub, _ = codebooks.shape
    nq = xq.shape[0]
    list_offsets = np.ascontiguousarray(list_offsets, dtype=np.int64)
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    npb = min(nprobe, nlist)
    coarse = np.empty((nq, npb), np.int32) if return_coarse else None
    rc = lib().orc_ivfpq_search(C.c_int(d), C.c_int(nlist), C.c_int(M), C.c_int(ksub),
                                _p(centroids, C.c_float), _p(codebooks, C.c_float),
                                C.c_int(int(by_residual)), _p(list_offsets, C.c_int64),
                                _p(codes, C.c_uint8), _p(ids, C.c_int64), C.c_int64(nq),
                                _p(xq, C.c_float), C.c_int(nprobe), C.c_int(k), _p(D, C.c_float),
                                _p(I, C.c_int64), _p(coarse, C.c_int32))
    if rc:
        raise RuntimeError(f"orc_ivfpq_search rc={rc}")
    return (D, I, coarse) if return_coarse else (D, I)


def kmeans(x, k, niter, seed=0):
    """Lloyd k-means in the trainer's canonical arithmetic (see orc_kmeans)."""
    x = _f32(x)
    n, d = x.shape
    out = np.empty((k, d), np.float32)
    rc = lib().orc_kmeans(C.c_int(d), C.c_int64(n), _p(x, C.c_float), C.c_int(k), C.c_int(niter),
                          C.c_uint64(seed), _p(out, C.c_float))
    if rc:
        raise RuntimeError(f"orc_kmeans rc={rc}")
    return out


def merge_topk(Din, Iin, descending=False):
    """Din/Iin: [nsrc, nq, k] -> merged [nq, k]."""
    Din = np.ascontiguousarray(Din, dtype=np.float32)
    Iin = np.ascontiguousarray(Iin, dtype=np.int64)
    nsrc, nq, k = Din.shape
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    lib().orc_merge_topk(C.c_int(nsrc), C.c_int64(nq), C.c_int(k), C.c_int(int(descending)),
                         _p(Din, C.c_float), _p(Iin, C.c_int64), _p(D, C.c_float), _p(I, C.c_int64))
    return D, I


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """OpenMP threads used by the following calls; returns the count in effect."""
    return int(lib().orc_set_num_threads(C.c_int(int(n))))


def use_all_host_threads() -> int:
    """All hardware threads this process may run on, whatever OMP_NUM_THREADS said at start-up
    (torchrun exports OMP_NUM_THREADS=1 to its workers)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return set_num_threads(n)


# ---------------------------------------------------------------------------
# Independent numpy mirror (float64, argsort) used to cross-check oracle.c.
# ---------------------------------------------------------------------------

def np_flat_search(metric, xb, xq, k):
    xb64, xq64 = np.asarray(xb, np.float64), np.asarray(xq, np.float64)
    if metric == METRIC_L2:
        dist = ((xq64[:, None, :] - xb64[None, :, :]) ** 2).sum(-1)
        key = dist.astype(np.float32)
    else:
        dist = xq64 @ xb64.T
        key = -(dist.astype(np.float32))
    order = np.lexsort((np.broadcast_to(np.arange(xb64.shape[0]), key.shape), key), axis=1)[:, :k]
    D = np.take_along_axis(key, order, 1)
    if metric != METRIC_L2:
        D = -D
    return _pad(D.astype(np.float32), order.astype(np.int64), k)


def np_int8_cos_scores(xb, xq):
    """The fp16 cosine with numpy's own float16 (an implementation independent of oracle.c's bit
    routines): [nq, nb] float16, NaN where the reference's arithmetic gives NaN."""
    b, q = np.asarray(xb, np.int64), np.asarray(xq, np.int64)

    def rnorm(v):
        sq = (v * v).sum(1).astype(np.float32)
        s = (sq * np.float32(0.01)).astype(np.float16).astype(np.float32)
        with np.errstate(divide="ignore"):
            return (np.float32(1.0) / np.sqrt(s)).astype(np.float16)
    with np.errstate(over="ignore", invalid="ignore"):
        ip = ((q @ b.T).astype(np.float32) * np.float32(0.01)).astype(np.float16)
        w = (rnorm(q)[:, None].astype(np.float32) * rnorm(b)[None, :].astype(np.float32)).astype(np.float16)
        return (ip.astype(np.float32) * w.astype(np.float32)).astype(np.float16)


def np_int8_search(metric, xb, xq, k):
    b, q = np.asarray(xb, np.int64), np.asarray(xq, np.int64)
    if metric == METRIC_INT8_COS:
        sc = np_int8_cos_scores(xb, xq).astype(np.float32)
        sc = np.where(np.isnan(sc), -np.inf, sc)
        key = -sc
        # -0.0 ranks directly below +0.0 in the restatement
        key = np.where((sc == 0) & np.signbit(sc), np.float32(1e-30), key)
        order = np.lexsort((np.broadcast_to(np.arange(b.shape[0]), key.shape), key), axis=1)[:, :k]
        return _pad(np.take_along_axis(sc, order, 1).astype(np.float32), order.astype(np.int64), k)
    if metric == METRIC_L2:
        key = ((q[:, None, :] - b[None, :, :]) ** 2).sum(-1)
    else:
        key = -(q @ b.T)
    order = np.lexsort((np.broadcast_to(np.arange(b.shape[0]), key.shape), key), axis=1)[:, :k]
    D = np.take_along_axis(key, order, 1).astype(np.float32)
    if metric != METRIC_L2:
        D = -D
    return _pad(D, order.astype(np.int64), k)


def _pad(D, I, k):
    if D.shape[1] < k:
        padD = np.full((D.shape[0], k - D.shape[1]), np.finfo(np.float32).max, np.float32)
        padI = np.full((I.shape[0], k - I.shape[1]), -1, np.int64)
        D, I = np.concatenate([D, padD], 1), np.concatenate([I, padI], 1)
    return D, I


def np_ivfpq_search(centroids, codebooks, by_residual, list_offsets, codes, ids, xq, nprobe, k):
    """float64 mirror of the IVFPQ semantics; distances agree with oracle.c to fp32 rounding."""
    cen, cb, xq = (np.asarray(a, np.float64) for a in (centroids, codebooks, xq))
    nlist, d = cen.shape
    M, ksub, dsub = cb.shape
    nq = xq.shape[0]
    D = np.full((nq, k), np.finfo(np.float32).max, np.float32)
    I = np.full((nq, k), -1, np.int64)
    for q in range(nq):
        cd = ((cen - xq[q]) ** 2).sum(1).astype(np.float32)
        probes = np.lexsort((np.arange(nlist), cd))[:nprobe]
        ds, ls = [], []
        for l in probes:
            b, e = list_offsets[l], list_offsets[l + 1]
            if b == e:
                continue
            v = xq[q] - cen[l] if by_residual else xq[q]
            lut = ((v.reshape(M, 1, dsub) - cb) ** 2).sum(-1)
            ds.append(lut[np.arange(M)[None, :], codes[b:e]].sum(1))
            ls.append(ids[b:e])
        if not ds:
            continue
        ds = np.concatenate(ds).astype(np.float32)
        ls = np.concatenate(ls)
        o = np.lexsort((ls, ds))[:k]
        D[q, :len(o)] = ds[o]
        I[q, :len(o)] = ls[o]
    return D, I
