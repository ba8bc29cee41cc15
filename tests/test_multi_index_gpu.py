"""GPU parity of multi-index batch search and of the device merge kernel."""
import numpy as np
import pytest

import oracle
from indexsdk_b200 import datasets
from helpers import assert_exact

pytestmark = pytest.mark.gpu
L2, IP = 1, 0


@pytest.mark.parametrize("metric", [L2, IP])
def test_multi_index_flat(b200, metric):
    d, k, nq = 64, 20, 33
    xq = datasets.gaussian(nq, d, seed=1)
    parts, indexes, Ds, Is = [], [], [], []
    base_id = 0
    for s, n in enumerate((3000, 500, 12000, 40)):
        xb = datasets.gaussian(n, d, seed=10 + s)
        ids = np.arange(base_id, base_id + n, dtype=np.int64)
        base_id += n
        ix = b200.IndexFlat(d, metric)
        ix.add_with_ids(xb, ids)
        indexes.append(ix)
        Dr, Ir = oracle.flat_search(metric, xb, xq, k, labels=ids)
        Ds.append(Dr)
        Is.append(Ir)
    D, I = b200.search_multi(indexes, xq, k, merged=False)       # layout [index][query][k]
    assert_exact(D, I, np.stack(Ds), np.stack(Is))
    Dm, Im = b200.search_multi(indexes, xq, k, merged=True)
    Dr, Ir = oracle.merge_topk(np.stack(Ds), np.stack(Is), descending=(metric == IP))
    assert_exact(Dm, Im, Dr, Ir)


def test_multi_index_int8(b200):
    d, k, nq = 64, 10, 5
    xq = datasets.uniform_int8(nq, d, seed=3)
    indexes, Ds, Is = [], [], []
    for s, n in enumerate((2000, 3000)):
        xb = datasets.uniform_int8(n, d, seed=20 + s)
        ids = np.arange(n, dtype=np.int64) + 10000 * s
        ix = b200.IndexInt8Flat(d, IP)
        ix.add_with_ids(xb, ids)
        indexes.append(ix)
        Dr, Ir = oracle.int8_search(IP, xb, xq, k, labels=ids)
        Ds.append(Dr)
        Is.append(Ir)
    Dm, Im = b200.search_multi(indexes, xq, k, merged=True)
    Dr, Ir = oracle.merge_topk(np.stack(Ds), np.stack(Is), descending=True)
    assert_exact(Dm, Im, Dr, Ir)


def test_sharded_base_equals_single_index(b200):
    """A base split over several handles and merged equals one index over the whole base."""
    d, k = 128, 50
    xb = datasets.gaussian(30000, d, seed=5)
    xq = datasets.gaussian(17, d, seed=6)
    ids = np.arange(30000, dtype=np.int64)
    shards = []
    for r in range(3):
        ix = b200.IndexFlat(d, L2)
        ix.add_with_ids(xb[r::3], ids[r::3])
        shards.append(ix)
    Dm, Im = b200.search_multi(shards, xq, k, merged=True)
    Dr, Ir = oracle.flat_search(L2, xb, xq, k)
    assert_exact(Dm, Im, Dr, Ir)


def test_merge_kernel_with_torch_buffers(b200):
    import torch
    r = np.random.default_rng(0)
    nsrc, nq, k = 5, 40, 33
    D = np.sort(r.random((nsrc, nq, k)).astype(np.float32), axis=2)
    I = r.permutation(nsrc * nq * k).reshape(nsrc, nq, k).astype(np.int64)
    I[3, :, 20:] = -1
    Dr, Ir = oracle.merge_topk(D, I)
    dD, dI = torch.from_numpy(D).cuda(), torch.from_numpy(I).cuda()
    oD = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    oI = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    b200.merge_topk_device(nsrc, nq, k, False, dD.data_ptr(), dI.data_ptr(), oD.data_ptr(), oI.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_exact(oD.cpu().numpy(), oI.cpu().numpy(), Dr, Ir)
