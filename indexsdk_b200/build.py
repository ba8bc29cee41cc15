"""Builds the CUDA library in-tree: ``indexsdk_b200/_build/libb200idx.so`` (sm_100a only).

Usage: ``python -m indexsdk_b200.build [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
BUILD_DIR = os.path.join(_HERE, "_build")
LIB_PATH = os.path.join(BUILD_DIR, "libb200idx.so")
SHIM_LIB_PATH = os.path.join(BUILD_DIR, "libb200idx_ascend.so")

SOURCES = ["dist_gemm.cu", "select.cu", "flat_index.cu", "multi_flat.cu", "ivfpq_index.cu", "ivfpq_tc_scan.cu", "kmeans.cu", "c_api.cu", "noalloc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "--expt-relaxed-constexpr",
    "-ccbin", "/usr/bin/g++",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _digest() -> str:
    h = hashlib.sha256()
    inc = os.path.join(_HERE, "..", "include")
    for root in (CSRC, os.path.join(CSRC, "shim"), inc, os.path.join(inc, "b200")):
        for name in sorted(os.listdir(root)):
            p = os.path.join(root, name)
            if os.path.isfile(p):
                h.update(name.encode())
                with open(p, "rb") as f:
                    h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("B200IDX_NVCC_EXTRA", "").encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    stamp = os.path.join(BUILD_DIR, "stamp.txt")
    digest = _digest()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB_PATH
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    # extra nvcc arguments for development builds (e.g. -DB200IDX_DEV_PROF: phase cycle counters)
    extra += os.environ.get("B200IDX_NVCC_EXTRA", "").split()

    def compile_one(src: str) -> str:
        obj = os.path.join(BUILD_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-ccbin", "/usr/bin/g++", "-o", LIB_PATH, *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    # header-compatible faiss::ascend classes over the C ABI (host C++ only)
    shim = os.path.join(CSRC, "shim", "ascend_api.cpp")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I", os.path.join(_HERE, "..", "include"),
           shim, "-o", SHIM_LIB_PATH, "-L", BUILD_DIR, "-lb200idx", "-Wl,-rpath,$ORIGIN", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the faiss::ascend shim failed")
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
