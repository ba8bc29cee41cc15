"""B200-native search hot path of Ascend/IndexSDK: Python binding of the C ABI.

The compute lives in ``libb200idx.so`` (hand-written sm_100a CUDA behind ``include/b200idx.h``);
this module is a thin ctypes mirror of the reference's index API (Faiss-style ``add`` /
``add_with_ids`` / ``search`` / ``reset`` / ``remove_ids`` and the multi-index ``search_multi``)
used by the tests and the benchmark.  There is no CPU fallback: if the library is missing the
import of any index class fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

METRIC_INNER_PRODUCT = 0
METRIC_L2 = 1
METRIC_INT8_COSINE = 2     # Int8Flat only: the reference's fp16 cosine (see include/b200idx.h)
F32 = 0
F16 = 1

_lib = None


class B200IdxError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


STAGES = ("sample", "full_gemm", "refine", "select", "coarse", "lut", "scan", "merge")


class Stats(C.Structure):
    _fields_ = [("stage_ms", C.c_double * 8), ("stage_launches", C.c_uint64 * 8)] + [
        (n, C.c_uint64) for n in
        ("searches", "queries", "fallback_queries", "gemm_launches", "kernel_launches", "scan_codes",
         "second_pass_queries")]


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python -m indexsdk_b200.build` (needs nvcc); "
                          "this package has no CPU or PyTorch fallback")
    lib = C.CDLL(path)
    vp, i64, i32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t
    pp = C.POINTER(C.c_void_p)
    sigs = {
        "b200idx_create_flat": (i32, [i32, i32, i32, i32, pp]),
        "b200idx_create_int8flat": (i32, [i32, i32, i32, pp]),
        "b200idx_create_ivfpq": (i32, [i32, i32, i32, i32, i32, i32, i32, pp]),
        "b200idx_destroy": (i32, [vp]),
        "b200idx_add": (i32, [vp, i64, vp, vp]),
        "b200idx_add_f16": (i32, [vp, i64, vp, vp]),
        "b200idx_add_device": (i32, [vp, i64, vp, vp]),
        "b200idx_search": (i32, [vp, i64, vp, i32, vp, vp]),
        "b200idx_search_f16": (i32, [vp, i64, vp, i32, vp, vp]),
        "b200idx_search_device": (i32, [vp, i64, vp, i32, vp, vp]),
        "b200idx_search_device_noalloc": (i32, [vp, i64, vp, i32, vp, vp]),
        "b200idx_search_multi": (i32, [pp, i32, i64, vp, i32, vp, vp, i32]),
        "b200idx_search_multi_stats": (i32, [i32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
        "b200idx_merge_topk_device": (i32, [i32, i64, i32, i32, vp, vp, vp, vp, vp]),
        "b200idx_merge_topk_device_strided": (i32, [i32, i64, i32, i32, vp, vp, i64, vp, vp, vp]),
        "b200idx_reset": (i32, [vp]),
        "b200idx_remove_ids": (i32, [vp, i64, vp, C.POINTER(i64)]),
        "b200idx_ntotal": (i64, [vp]),
        "b200idx_dim": (i32, [vp]),
        "b200idx_device": (i32, [vp]),
        "b200idx_get_base": (i32, [vp, i64, i64, vp]),
        "b200idx_get_ids": (i32, [vp, i64, i64, vp]),
        "b200idx_ivfpq_set_centroids": (i32, [vp, vp]),
        "b200idx_ivfpq_set_codebooks": (i32, [vp, vp]),
        "b200idx_ivfpq_get_centroids": (i32, [vp, vp]),
        "b200idx_ivfpq_get_codebooks": (i32, [vp, vp]),
        "b200idx_ivfpq_add_codes": (i32, [vp, i64, vp, vp, vp]),
        "b200idx_search_with_masks": (i32, [vp, i64, vp, i32, vp, vp, vp]),
        "b200idx_kmeans": (i32, [i32, i32, i64, vp, i32, i32, C.c_uint64, vp]),
        "b200idx_ivfpq_train": (i32, [vp, i64, vp, i32, C.c_uint64]),
        "b200idx_save": (i32, [vp, C.c_char_p]),
        "b200idx_load": (i32, [C.c_char_p, i32, C.POINTER(vp)]),
        "b200idx_ivfpq_set_nprobe": (i32, [vp, i32]),
        "b200idx_ivfpq_coarse_device": (i32, [vp, i64, vp, vp, vp]),
        "b200idx_ivfpq_search_preassigned_device": (i32, [vp, i64, vp, i32, vp, vp, vp, vp]),
        "b200idx_ivfpq_get_nprobe": (i32, [vp]),
        "b200idx_ivfpq_list_length": (i64, [vp, i32]),
        "b200idx_ivfpq_get_list": (i32, [vp, i32, vp, vp]),
        "b200idx_stats": (i32, [vp, C.POINTER(Stats), i32]),
        "b200idx_set_timing": (i32, [vp, i32]),
        "b200idx_stream": (vp, [vp]),
        "b200idx_last_error": (C.c_char_p, [vp]),
        "b200idx_status_of_message": (i32, [C.c_char_p]),
        "b200idx_version": (C.c_char_p, []),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


EXPORTED_SYMBOLS = [
    "b200idx_create_flat", "b200idx_create_int8flat", "b200idx_create_ivfpq", "b200idx_destroy", "b200idx_add",
    "b200idx_add_f16", "b200idx_add_device", "b200idx_search", "b200idx_search_f16", "b200idx_search_device",
    "b200idx_search_device_noalloc",
    "b200idx_search_multi", "b200idx_search_multi_stats", "b200idx_merge_topk_device", "b200idx_merge_topk_device_strided", "b200idx_reset", "b200idx_remove_ids", "b200idx_ntotal",
    "b200idx_dim", "b200idx_device", "b200idx_get_base", "b200idx_get_ids", "b200idx_ivfpq_set_centroids",
    "b200idx_ivfpq_set_codebooks", "b200idx_ivfpq_get_centroids", "b200idx_ivfpq_get_codebooks",
    "b200idx_search_with_masks", "b200idx_save", "b200idx_load", "b200idx_kmeans", "b200idx_ivfpq_train", "b200idx_ivfpq_add_codes", "b200idx_ivfpq_set_nprobe", "b200idx_ivfpq_coarse_device",
    "b200idx_ivfpq_search_preassigned_device", "b200idx_ivfpq_get_nprobe", "b200idx_ivfpq_list_length",
    "b200idx_ivfpq_get_list", "b200idx_stats", "b200idx_set_timing", "b200idx_stream", "b200idx_last_error",
    "b200idx_status_of_message",
    "b200idx_version",
]


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _check(rc: int, handle=None):
    if rc != 0:
        msg = load().b200idx_last_error(handle)
        raise B200IdxError(rc, msg.decode() if msg else "")


class _Index:
    """Common part: owns a ``b200idx_t*``."""
    _query_dtype = np.float32

    def __init__(self):
        self._h = C.c_void_p()
        self._lib = load()

    def __del__(self):
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            self._lib.b200idx_destroy(h)
            self._h = None      # (module globals may already be gone when the interpreter shuts down)

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def ntotal(self) -> int:
        return int(self._lib.b200idx_ntotal(self._h))

    @property
    def d(self) -> int:
        return int(self._lib.b200idx_dim(self._h))

    @property
    def device(self) -> int:
        return int(self._lib.b200idx_device(self._h))

    def _prep(self, x):
        x = np.ascontiguousarray(x, dtype=self._query_dtype)
        if x.ndim != 2 or x.shape[1] != self.d:
            raise ValueError(f"expected an [n, {self.d}] array, got {x.shape}")
        return x

    def add(self, x):
        self.add_with_ids(x, None)

    def add_with_ids(self, x, ids):
        x = self._prep(x)
        idp = None if ids is None else np.ascontiguousarray(ids, dtype=np.int64)
        _check(self._lib.b200idx_add(self._h, x.shape[0], _ptr(x), _ptr(idp)), self._h)

    def add_device(self, x_ptr: int, n: int, ids=None):
        """x_ptr: device address of n rows in the index's input dtype (e.g. ``tensor.data_ptr()``)."""
        idp = None if ids is None else np.ascontiguousarray(ids, dtype=np.int64)
        _check(self._lib.b200idx_add_device(self._h, n, C.c_void_p(x_ptr), _ptr(idp)), self._h)

    def search(self, x, k: int):
        x = self._prep(x)
        n = x.shape[0]
        D = np.empty((n, k), np.float32)
        I = np.empty((n, k), np.int64)
        _check(self._lib.b200idx_search(self._h, n, _ptr(x), k, _ptr(D), _ptr(I)), self._h)
        return D, I

    def save(self, path: str):
        """Writes the index in the library's own file format (see b200idx_save)."""
        _check(self._lib.b200idx_save(self._h, str(path).encode()), self._h)

    def search_with_masks(self, x, k: int, mask):
        """mask: uint8 [n][ceil(ntotal / 8)], bit (i % 8) of byte i / 8 = 1 keeps base position i
        (np.packbits(keep, axis=1, bitorder="little"))."""
        x = self._prep(x)
        n = x.shape[0]
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        if mask.shape != (n, (self.ntotal + 7) // 8):
            raise ValueError("mask must have shape [n][ceil(ntotal / 8)]")
        D = np.empty((n, k), np.float32)
        I = np.empty((n, k), np.int64)
        _check(self._lib.b200idx_search_with_masks(self._h, n, _ptr(x), k, _ptr(mask), _ptr(D), _ptr(I)), self._h)
        return D, I

    def search_into(self, x, k: int, D, I):
        """Search with caller-owned output arrays (no allocation in the timed path)."""
        _check(self._lib.b200idx_search(self._h, x.shape[0], _ptr(x), k, _ptr(D), _ptr(I)), self._h)

    def search_device(self, x_ptr: int, n: int, k: int, D_ptr: int, I_ptr: int):
        _check(self._lib.b200idx_search_device(self._h, n, C.c_void_p(x_ptr), k, C.c_void_p(D_ptr),
                                               C.c_void_p(I_ptr)), self._h)

    def search_device_noalloc(self, x_ptr: int, n: int, k: int, D_ptr: int, I_ptr: int):
        """Exact search with all scratch in the library's static device array (Flat / Int8Flat,
        small requests only); for callers that may not allocate device memory while searching."""
        _check(self._lib.b200idx_search_device_noalloc(self._h, n, C.c_void_p(x_ptr), k, C.c_void_p(D_ptr),
                                                       C.c_void_p(I_ptr)), self._h)

    def reset(self):
        _check(self._lib.b200idx_reset(self._h), self._h)

    def remove_ids(self, ids) -> int:
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        out = C.c_int64(0)
        _check(self._lib.b200idx_remove_ids(self._h, ids.size, _ptr(ids), C.byref(out)), self._h)
        return int(out.value)

    def stats(self, reset: bool = False) -> dict:
        s = Stats()
        _check(self._lib.b200idx_stats(self._h, C.byref(s), int(reset)), self._h)
        out = {n: int(getattr(s, n)) for n, _ in Stats._fields_[2:]}
        out["stage_ms"] = {n: float(s.stage_ms[i]) for i, n in enumerate(STAGES)}
        out["stage_launches"] = {n: int(s.stage_launches[i]) for i, n in enumerate(STAGES)}
        return out

    def set_timing(self, enabled: bool):
        _check(self._lib.b200idx_set_timing(self._h, int(enabled)), self._h)

    @property
    def stream_ptr(self) -> int:
        """Address of the cudaStream_t this index launches on."""
        return int(self._lib.b200idx_stream(self._h) or 0)


class IndexFlat(_Index):
    """Exact search, fp32 (default) or fp16 rows -- mirror of ``faiss::ascend::AscendIndexFlat``
    (feature_retrieval/src/ascendfaiss/ascend/AscendIndexFlat.h:48-90) on one device."""

    def __init__(self, d: int, metric: int = METRIC_L2, dtype: int = F32, device: int = 0):
        super().__init__()
        self.metric, self.dtype = metric, dtype
        _check(self._lib.b200idx_create_flat(d, metric, dtype, device, C.byref(self._h)))

    def add_f16(self, x_bits, ids=None):
        x = np.ascontiguousarray(x_bits, dtype=np.uint16)
        idp = None if ids is None else np.ascontiguousarray(ids, dtype=np.int64)
        _check(self._lib.b200idx_add_f16(self._h, x.shape[0], _ptr(x), _ptr(idp)), self._h)

    def search_f16(self, x_bits, k: int):
        x = np.ascontiguousarray(x_bits, dtype=np.uint16)
        n = x.shape[0]
        D = np.empty((n, k), np.float32)
        I = np.empty((n, k), np.int64)
        _check(self._lib.b200idx_search_f16(self._h, n, _ptr(x), k, _ptr(D), _ptr(I)), self._h)
        return D, I

    def get_base(self, offset: int = 0, n: int | None = None):
        n = self.ntotal - offset if n is None else n
        out = np.empty((n, self.d), np.float32 if self.dtype == F32 else np.uint16)
        _check(self._lib.b200idx_get_base(self._h, offset, n, _ptr(out)), self._h)
        return out

    def get_ids(self, offset: int = 0, n: int | None = None):
        n = self.ntotal - offset if n is None else n
        out = np.empty(n, np.int64)
        _check(self._lib.b200idx_get_ids(self._h, offset, n, _ptr(out)), self._h)
        return out


class IndexInt8Flat(_Index):
    """Exact int8 search with int32 accumulation -- mirror of ``faiss::ascend::AscendIndexInt8Flat``
    (feature_retrieval/src/ascendfaiss/ascend/AscendIndexInt8Flat.h:60-109) on one device."""
    _query_dtype = np.int8

    def __init__(self, d: int, metric: int = METRIC_L2, device: int = 0):
        super().__init__()
        self.metric = metric
        _check(self._lib.b200idx_create_int8flat(d, metric, device, C.byref(self._h)))

    def get_base(self, offset: int = 0, n: int | None = None):
        n = self.ntotal - offset if n is None else n
        out = np.empty((n, self.d), np.int8)
        _check(self._lib.b200idx_get_base(self._h, offset, n, _ptr(out)), self._h)
        return out

    def get_ids(self, offset: int = 0, n: int | None = None):
        n = self.ntotal - offset if n is None else n
        out = np.empty(n, np.int64)
        _check(self._lib.b200idx_get_ids(self._h, offset, n, _ptr(out)), self._h)
        return out


class IndexIVFPQ(_Index):
    """IVFPQ, L2, 8-bit codes -- mirror of ``faiss::ascend::AscendIndexIVFPQ``
    (feature_retrieval/src/ascendfaiss/ascend/AscendIndexIVFPQ.h:71-96) on one device.
    Trained state (centroids, codebooks) is set from outside, as ``copyFrom`` does."""

    def __init__(self, d: int, nlist: int, M: int, nbits: int = 8, by_residual: bool = False, device: int = 0):
        super().__init__()
        self.nlist, self.M, self.by_residual = nlist, M, by_residual
        _check(self._lib.b200idx_create_ivfpq(d, METRIC_L2, nlist, M, nbits, int(by_residual), device,
                                              C.byref(self._h)))

    def set_centroids(self, centroids):
        c = np.ascontiguousarray(centroids, dtype=np.float32)
        assert c.shape == (self.nlist, self.d)
        _check(self._lib.b200idx_ivfpq_set_centroids(self._h, _ptr(c)), self._h)

    def set_codebooks(self, codebooks):
        cb = np.ascontiguousarray(codebooks, dtype=np.float32)
        assert cb.shape == (self.M, 256, self.d // self.M)
        _check(self._lib.b200idx_ivfpq_set_codebooks(self._h, _ptr(cb)), self._h)

    def add_codes(self, list_no, codes, ids=None):
        ln = np.ascontiguousarray(list_no, dtype=np.int32)
        cd = np.ascontiguousarray(codes, dtype=np.uint8)
        idp = None if ids is None else np.ascontiguousarray(ids, dtype=np.int64)
        _check(self._lib.b200idx_ivfpq_add_codes(self._h, ln.size, _ptr(ln), _ptr(cd), _ptr(idp)), self._h)

    @property
    def nprobe(self) -> int:
        return int(self._lib.b200idx_ivfpq_get_nprobe(self._h))

    @nprobe.setter
    def nprobe(self, v: int):
        _check(self._lib.b200idx_ivfpq_set_nprobe(self._h, int(v)), self._h)

    def get_centroids(self):
        out = np.empty((self.nlist, self.d), np.float32)
        _check(self._lib.b200idx_ivfpq_get_centroids(self._h, _ptr(out)), self._h)
        return out

    def get_codebooks(self):
        out = np.empty((self.M, 256, self.d // self.M), np.float32)
        _check(self._lib.b200idx_ivfpq_get_codebooks(self._h, _ptr(out)), self._h)
        return out

    def train(self, x, niter: int = 10, seed: int = 0):
        """Coarse centroids and PQ codebooks by k-means on the device (b200idx_ivfpq_train)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        _check(self._lib.b200idx_ivfpq_train(self._h, x.shape[0], _ptr(x), int(niter), C.c_uint64(seed)), self._h)

    def coarse_device(self, x_ptr: int, n: int, cD_ptr: int, cI_ptr: int):
        """Probe selection only: [n][nprobe] distances and list ids (device pointers)."""
        _check(self._lib.b200idx_ivfpq_coarse_device(self._h, n, C.c_void_p(x_ptr), C.c_void_p(cD_ptr),
                                                     C.c_void_p(cI_ptr)), self._h)

    def search_preassigned_device(self, x_ptr: int, n: int, k: int, cD_ptr: int, cI_ptr: int, D_ptr: int, I_ptr: int):
        """Code scan + refinement for given probes (device pointers)."""
        _check(self._lib.b200idx_ivfpq_search_preassigned_device(
            self._h, n, C.c_void_p(x_ptr), k, C.c_void_p(cD_ptr), C.c_void_p(cI_ptr), C.c_void_p(D_ptr),
            C.c_void_p(I_ptr)), self._h)

    def list_length(self, l: int) -> int:
        return int(self._lib.b200idx_ivfpq_list_length(self._h, l))

    def get_list(self, l: int):
        n = self.list_length(l)
        codes = np.empty((n, self.M), np.uint8)
        ids = np.empty(n, np.int64)
        if n:
            _check(self._lib.b200idx_ivfpq_get_list(self._h, l, _ptr(codes), _ptr(ids)), self._h)
        return codes, ids


def kmeans(x, k: int, niter: int = 10, seed: int = 0, device: int = 0):
    """Lloyd k-means on the device (b200idx_kmeans); returns the [k][d] centroids."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty((k, x.shape[1]), np.float32)
    _check(load().b200idx_kmeans(device, x.shape[1], x.shape[0], _ptr(x), k, int(niter), C.c_uint64(seed), _ptr(out)))
    return out


def load_index(path: str, device: int = 0):
    """Reads an index written by ``save`` onto ``device`` (b200idx_load) and returns the matching
    Python object."""
    import struct
    with open(path, "rb") as f:
        head = f.read(4 + 4 + 4 + 12 + 8 + 16)
    if len(head) < 32 or head[:4] != b"B2IX":
        raise B200IdxError(2001, "not an index file of this library")
    _, kind, d, metric, dtype, _ = struct.unpack_from("<IIiiiq", head, 4)
    if kind == 0:
        ix = IndexFlat.__new__(IndexFlat)
        _Index.__init__(ix)
        ix.metric, ix.dtype = metric, (F16 if dtype == 1 else F32)
    elif kind == 1:
        ix = IndexInt8Flat.__new__(IndexInt8Flat)
        _Index.__init__(ix)
        ix.metric = metric
    else:
        nlist, M, _, by_res = struct.unpack_from("<iiii", head, 32)
        ix = IndexIVFPQ.__new__(IndexIVFPQ)
        _Index.__init__(ix)
        ix.nlist, ix.M, ix.by_residual = nlist, M, bool(by_res)
    _check(ix._lib.b200idx_load(str(path).encode(), device, C.byref(ix._h)))
    return ix


def search_multi(indexes, x, k: int, merged: bool = True):
    """Multi-index batch search -- mirror of ``faiss::ascend::Search(indexes, n, x, k, D, I, merged)``
    (feature_retrieval/src/ascendfaiss/ascend/AscendMultiIndexSearch.h:34-44)."""
    lib = load()
    x = indexes[0]._prep(x)
    n, nh = x.shape[0], len(indexes)
    shape = (n, k) if merged else (nh, n, k)
    D = np.empty(shape, np.float32)
    I = np.empty(shape, np.int64)
    arr = (C.c_void_p * nh)(*[ix.handle for ix in indexes])
    rc = lib.b200idx_search_multi(arr, nh, n, _ptr(x), k, _ptr(D), _ptr(I), int(merged))
    _check(rc, indexes[0].handle)
    return D, I


def search_multi_stats(device: int = 0) -> dict:
    """Counters of the segmented (one pass over all small indexes) path of search_multi."""
    a, b_ = C.c_uint64(0), C.c_uint64(0)
    load().b200idx_search_multi_stats(device, C.byref(a), C.byref(b_))
    return dict(group_launches=int(a.value), group_rebuilds=int(b_.value))


def merge_topk_device(nsrc: int, n: int, k: int, descending: bool, Din_ptr: int, Iin_ptr: int, D_ptr: int,
                      I_ptr: int, stream_ptr: int = 0, src_stride_bytes: int = 0):
    """Merge of nsrc sorted per-source results on the device.  src_stride_bytes = 0: dense
    [nsrc][n][k] arrays; otherwise the byte distance between the blocks of consecutive sources
    (packed per-rank blocks after one all-gather)."""
    lib = load()
    if src_stride_bytes:
        rc = lib.b200idx_merge_topk_device_strided(nsrc, n, k, int(descending), C.c_void_p(Din_ptr),
                                                   C.c_void_p(Iin_ptr), src_stride_bytes, C.c_void_p(D_ptr),
                                                   C.c_void_p(I_ptr), C.c_void_p(stream_ptr))
    else:
        rc = lib.b200idx_merge_topk_device(nsrc, n, k, int(descending), C.c_void_p(Din_ptr), C.c_void_p(Iin_ptr),
                                           C.c_void_p(D_ptr), C.c_void_p(I_ptr), C.c_void_p(stream_ptr))
    if rc:
        raise B200IdxError(rc, "merge_topk_device failed")
