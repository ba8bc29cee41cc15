"""The search entry point that allocates nothing (b200idx_search_device_noalloc).

It exists for callers that may not allocate device memory while they search: a serving process
whose HBM belongs to its own pool, or a loop that cannot take the device-wide synchronisation of
cudaMalloc / cudaFree.  All of its scratch sits in one static device array inside the library, so
consecutive calls reuse (and must re-initialise) the same memory: the test calls it twice in a
row with different queries and checks both results bit for bit against the regular
b200idx_search_device entry point.  This file sorts last so that a run that stops at the first
failure has already run every other test."""
import numpy as np
import pytest

from indexsdk_b200 import datasets

pytestmark = pytest.mark.gpu


def _run(ix, fn, xq_t, k):
    import torch
    n = xq_t.shape[0]
    D = torch.full((n, k), -7.0, dtype=torch.float32, device="cuda")
    I = torch.full((n, k), -7, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    fn(xq_t.data_ptr(), n, k, D.data_ptr(), I.data_ptr())
    torch.cuda.synchronize()
    return D.cpu().numpy(), I.cpu().numpy()


@pytest.mark.parametrize("kind", ["f32_l2", "f32_ip", "f16_l2", "i8_ip", "i8_l2", "i8_cos"])
def test_noalloc_matches_regular_entry_point_twice(b200, kind):
    import torch
    d, n_base, k = 64, 5000, 10
    if kind.startswith("i8"):
        metric = (b200.METRIC_INT8_COSINE if kind.endswith("cos") else
                  b200.METRIC_INNER_PRODUCT if kind.endswith("ip") else b200.METRIC_L2)
        ix = b200.IndexInt8Flat(d, metric)
        ix.add(datasets.uniform_int8(n_base, d, seed=2))
        queries = [torch.from_numpy(datasets.uniform_int8(nq, d, seed=s)).cuda() for nq, s in ((9, 3), (16, 4))]
    else:
        metric = b200.METRIC_INNER_PRODUCT if kind.endswith("ip") else b200.METRIC_L2
        ix = b200.IndexFlat(d, metric, dtype=b200.F16 if kind.startswith("f16") else b200.F32)
        ix.add_with_ids(datasets.gaussian(n_base, d, seed=0), np.arange(n_base, dtype=np.int64) * 3 + 1)
        queries = [torch.from_numpy(datasets.gaussian(nq, d, seed=s)).cuda() for nq, s in ((9, 1), (16, 5))]
    for xq in queries:                                   # two calls in a row on the shared scratch
        Dn, In = _run(ix, ix.search_device_noalloc, xq, k)
        Dr, Ir = _run(ix, ix.search_device, xq, k)
        np.testing.assert_array_equal(In, Ir)
        np.testing.assert_array_equal(Dn.view(np.uint32), Dr.view(np.uint32))
    # k larger than the previous call: nothing stale from earlier calls may leak into the result
    Dn, In = _run(ix, ix.search_device_noalloc, queries[0], 100)
    Dr, Ir = _run(ix, ix.search_device, queries[0], 100)
    np.testing.assert_array_equal(In, Ir)
    np.testing.assert_array_equal(Dn.view(np.uint32), Dr.view(np.uint32))


def test_noalloc_rejects_requests_beyond_the_static_scratch(b200):
    import torch
    ix = b200.IndexInt8Flat(64, b200.METRIC_L2)
    ix.add(datasets.uniform_int8(70000, 64, seed=1))      # padded to 70144 rows
    xq = torch.from_numpy(datasets.uniform_int8(16, 64, seed=2)).cuda()   # 16 * 70144 > 2^20
    D = torch.empty((16, 10), dtype=torch.float32, device="cuda")
    I = torch.empty((16, 10), dtype=torch.int64, device="cuda")
    with pytest.raises(b200.B200IdxError) as e:
        ix.search_device_noalloc(xq.data_ptr(), 16, 10, D.data_ptr(), I.data_ptr())
    assert e.value.code == 2001 and "static scratch" in e.value.msg
    with pytest.raises(b200.B200IdxError) as e:
        ix.search_device_noalloc(xq.data_ptr(), 4, 2000, D.data_ptr(), I.data_ptr())
    assert e.value.code == 2001 and "k must be in [1, 1024]" in e.value.msg
    # a request that fits still works after the rejections
    Dn, In = _run(ix, ix.search_device_noalloc, xq[:8], 10)
    Dr, Ir = _run(ix, ix.search_device, xq[:8], 10)
    np.testing.assert_array_equal(In, Ir)
    np.testing.assert_array_equal(Dn, Dr)


def test_noalloc_query_operand_limit_is_enforced_as_documented(b200, oracle_lib):
    """n * d <= 524288 is the documented limit for the query operand copy.  An fp32 index writes
    rows of d + 16 bf16 values there, so the largest admitted request (n = 1024, d = 512) must
    still fit -- checked against the CPU oracle, which shares no scratch with anything -- and the
    first shape beyond the limit (d = 528) must be refused instead of overrunning the region."""
    import torch
    n, k, n_base = 1024, 10, 1000
    for d, ok in ((512, True), (528, False)):
        ix = b200.IndexFlat(d, b200.METRIC_L2)
        xb = datasets.gaussian(n_base, d, seed=11)
        ix.add(xb)
        xq_np = datasets.gaussian(n, d, seed=12)
        xq = torch.from_numpy(xq_np).cuda()
        if ok:
            for _ in range(2):
                Dn, In = _run(ix, ix.search_device_noalloc, xq, k)
                Dr, Ir = oracle_lib.flat_search(oracle_lib.METRIC_L2, xb, xq_np, k)
                np.testing.assert_array_equal(In, Ir)
                np.testing.assert_array_equal(Dn.view(np.uint32), Dr.view(np.uint32))
        else:
            D = torch.empty((n, k), dtype=torch.float32, device="cuda")
            I = torch.empty((n, k), dtype=torch.int64, device="cuda")
            with pytest.raises(b200.B200IdxError) as e:
                ix.search_device_noalloc(xq.data_ptr(), n, k, D.data_ptr(), I.data_ptr())
            assert e.value.code == 2001 and "n * d <= 524288" in e.value.msg
