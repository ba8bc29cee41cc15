"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol that
include/b200idx.h declares, and fails loudly (no CPU fallback) when no GPU is present."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200idx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200idx_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(b200):
    lib = ctypes.CDLL(b200.lib_path())
    names = _declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b200idx.h but not exported"
    assert sorted(b200.EXPORTED_SYMBOLS) == names


def test_version_and_null_handle_behaviour(b200):
    lib = b200.load()
    assert b"sm_100a" in lib.b200idx_version()
    assert lib.b200idx_ntotal(None) == -1
    assert lib.b200idx_reset(None) == 2001
    assert lib.b200idx_search(None, 1, None, 1, None, None) == 2001


def test_parameter_errors_before_any_device_work(b200):
    lib = b200.load()
    h = ctypes.c_void_p()
    assert lib.b200idx_create_flat(100, 1, 0, 0, ctypes.byref(h)) == 2001
    assert b"Unsupported dims" in lib.b200idx_last_error(None)
    assert lib.b200idx_create_flat(128, 7, 0, 0, ctypes.byref(h)) == 2001
    assert b"Unsupported metric type" in lib.b200idx_last_error(None)
    assert lib.b200idx_create_ivfpq(128, 1, 1024, 7, 8, 0, 0, ctypes.byref(h)) in (2001, 2010)


def test_no_cpu_fallback_without_gpu(b200):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-GPU failure path is checked on CPU boxes")
    lib = b200.load()
    h = ctypes.c_void_p()
    rc = lib.b200idx_create_flat(128, 1, 0, 0, ctypes.byref(h))
    assert rc == 2010 and not h.value
    assert b"no CUDA device" in lib.b200idx_last_error(None)
    with pytest.raises(b200.B200IdxError):
        b200.IndexFlat(128)


def test_timeout_status_translation(b200):
    """A kernel whose bounded wait runs out sets a device error word; the host turns that into an
    exception whose text names the bounded wait, and the C ABI maps such a failure to the
    reference's APP_ERR_TIMEOUT (2011) -- any other internal failure is APP_ERR_INNER_ERROR (2010).
    The mapping is host code, so it is checked here with the messages the index classes produce
    and without making a device wait run out."""
    lib = b200.load()
    for msg in (b"device pipeline reported error word 1 (bounded wait ran out)",
                b"IVFPQ tensor-core scan reported error word 1 (bounded wait ran out)"):
        assert lib.b200idx_status_of_message(msg) == 2011
    assert lib.b200idx_status_of_message(b"cudaMalloc failed: out of memory") == 2010
    assert lib.b200idx_status_of_message(None) == 2001
