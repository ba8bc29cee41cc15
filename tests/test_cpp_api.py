"""Builds and runs tests/cpp/test_ascend_api.cpp: the faiss::ascend classes (header-compatible
with the reference) driven the way the reference's own unit tests drive them."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "indexsdk_b200", "_build")
EXE = os.path.join(BUILD, "test_ascend_api")


def _build(b200):
    src = os.path.join(ROOT, "tests", "cpp", "test_ascend_api.cpp")
    deps = [src, os.path.join(BUILD, "libb200idx_ascend.so")]
    if not os.path.exists(EXE) or any(os.path.getmtime(p) > os.path.getmtime(EXE) for p in deps):
        subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), src, "-o", EXE,
                        "-L", BUILD, "-lb200idx_ascend", "-lb200idx", "-Wl,-rpath," + BUILD, "-lpthread"], check=True)
    return EXE


def _run(mode, *extra):
    r = subprocess.run([EXE, mode, *extra], capture_output=True, text=True, timeout=1200)
    print(r.stdout[-4000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "0 failed" in r.stdout


def test_cpp_api_parameter_contract(b200):
    """No GPU needed: message substrings, config defaults, loud failure without a device."""
    import torch
    _build(b200)
    if torch.cuda.is_available():
        pytest.skip("the no-device failure path is checked on CPU boxes; the gpu test covers the rest")
    _run("cpu")


@pytest.mark.gpu
def test_cpp_api_on_gpu(b200):
    import torch
    _build(b200)
    _run("gpu", str(torch.cuda.device_count()))
