"""Save / load in the library's own file format: a loaded index answers exactly like the saved one."""
import numpy as np
import pytest

from indexsdk_b200 import datasets

pytestmark = pytest.mark.gpu
L2, IP = 1, 0


def _same(a, b):
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])


@pytest.mark.parametrize("kind", ["f32", "f16", "int8"])
def test_flat_round_trip(b200, tmp_path, kind):
    d, n = 64, 5000
    ids = np.arange(n, dtype=np.int64) * 3 + 7
    if kind == "int8":
        ix = b200.IndexInt8Flat(d, IP)
        xb, xq = datasets.uniform_int8(n, d, seed=1), datasets.uniform_int8(9, d, seed=2)
    else:
        ix = b200.IndexFlat(d, L2, dtype=b200.F32 if kind == "f32" else b200.F16)
        xb, xq = datasets.gaussian(n, d, seed=1), datasets.gaussian(9, d, seed=2)
    ix.add_with_ids(xb, ids)
    path = tmp_path / "flat.b2ix"
    ix.save(path)
    ld = b200.load_index(str(path))
    assert type(ld) is type(ix) and ld.ntotal == n and ld.d == d
    _same(ld.search(xq, 10), ix.search(xq, 10))
    np.testing.assert_array_equal(ld.get_base(10, 4), ix.get_base(10, 4))
    np.testing.assert_array_equal(ld.get_ids(), ids)


@pytest.mark.parametrize("resid", [False, True])
def test_ivfpq_round_trip(b200, tmp_path, resid):
    d, nlist, M, n = 64, 32, 16, 12000
    xb, _ = datasets.mixture(n, d, 16, seed=3)
    xq, _ = datasets.mixture(20, d, 16, seed=4, centers_seed=3)
    cent, cb = datasets.train_ivfpq(xb[:6000], nlist, M, resid, niter=4)
    ix = b200.IndexIVFPQ(d, nlist, M, 8, by_residual=resid)
    ix.set_centroids(cent)
    ix.set_codebooks(cb)
    ix.add_with_ids(xb, np.arange(n, dtype=np.int64) + 100)
    ix.nprobe = 6
    path = tmp_path / "ivfpq.b2ix"
    ix.save(path)
    ld = b200.load_index(str(path))
    assert ld.ntotal == n and ld.nprobe == 6 and ld.by_residual == resid
    for l in (0, 5, nlist - 1):
        ca, ia = ix.get_list(l)
        cb2, ib = ld.get_list(l)
        np.testing.assert_array_equal(ca, cb2)
        np.testing.assert_array_equal(ia, ib)
    _same(ld.search(xq, 10), ix.search(xq, 10))


def test_load_rejects_other_files(b200, tmp_path):
    p = tmp_path / "junk.bin"
    p.write_bytes(b"not an index at all, just some bytes to read" * 4)
    with pytest.raises(b200.B200IdxError):
        b200.load_index(str(p))
