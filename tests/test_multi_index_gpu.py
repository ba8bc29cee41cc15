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
    Dr, Ir = oracle.merge_topk(np.stack(Ds), np.stack(Is), descending=(metric != L2))
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


@pytest.mark.parametrize("kind", ["f32_l2", "f32_ip", "i8_ip", "i8_l2", "f16_ip", "i8_cos"])
def test_many_small_indexes_one_pass(b200, kind):
    """64 small indexes of one device: the segmented path searches them in one pass over their
    concatenated bases.  Results per index and merged are those of the oracle; the number of
    kernels launched per call does not depend on the number of indexes; the second call allocates
    nothing; a change of one member is noticed."""
    import torch
    from helpers import assert_close_gap_aware
    d, k, nq, nidx = 64, 10, 33, 64
    rng = np.random.default_rng(5)
    sizes = [int(v) for v in rng.integers(40, 3000, size=nidx)]
    sizes[3], sizes[17] = 256, 257                          # exactly one tile / one row more
    is_int = kind.startswith("i8")
    metric = 2 if kind.endswith("cos") else (IP if kind.endswith("ip") else L2)
    xq = datasets.uniform_int8(nq, d, seed=3) if is_int else datasets.gaussian(nq, d, seed=1)
    if kind.startswith("f16"):
        xq = oracle.round_fp16(xq)
    indexes, Ds, Is, bases = [], [], [], []
    base_id = 0
    for s_, n in enumerate(sizes):
        ids = np.arange(base_id, base_id + n, dtype=np.int64) * 2 + 1
        base_id += n
        if is_int:
            xb = datasets.uniform_int8(n, d, seed=100 + s_)
            ix = b200.IndexInt8Flat(d, metric)
            Dr, Ir = oracle.int8_search(metric, xb, xq, k, labels=ids)
        else:
            xb = datasets.gaussian(n, d, seed=100 + s_)
            if kind.startswith("f16"):
                xb = oracle.round_fp16(xb)
            ix = b200.IndexFlat(d, metric, dtype=b200.F16 if kind.startswith("f16") else b200.F32)
            Dr, Ir = oracle.flat_search(metric, xb, xq, k, labels=ids)
        ix.add_with_ids(xb, ids)
        indexes.append(ix)
        bases.append((xb, ids))
        Ds.append(Dr)
        Is.append(Ir)
    exact = not kind.startswith("f16")

    def check(D, I, Dref, Iref, what):
        if exact:
            assert_exact(D, I, Dref, Iref)
        else:
            assert_close_gap_aware(D.reshape(-1, k), I.reshape(-1, k), Dref.reshape(-1, k), Iref.reshape(-1, k), 1e-3, what)

    s0 = b200.search_multi_stats()
    D, I = b200.search_multi(indexes, xq, k, merged=False)
    s1 = b200.search_multi_stats()
    check(D, I, np.stack(Ds), np.stack(Is), "per index")
    assert s1["group_rebuilds"] == s0["group_rebuilds"] + 1
    per_call_64 = s1["group_launches"] - s0["group_launches"]
    assert 0 < per_call_64 <= 8
    # second call: same copy, same number of launches, no device allocation
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    Dm, Im = b200.search_multi(indexes, xq, k, merged=True)
    free1 = torch.cuda.mem_get_info()[0]
    s2 = b200.search_multi_stats()
    Dr, Ir = oracle.merge_topk(np.stack(Ds), np.stack(Is), descending=(metric != L2))
    check(Dm, Im, Dr, Ir, "merged")
    assert s2["group_rebuilds"] == s1["group_rebuilds"] and s2["group_launches"] - s1["group_launches"] == per_call_64
    D2, I2 = b200.search_multi(indexes, xq, k, merged=False)
    free2 = torch.cuda.mem_get_info()[0]
    assert free2 == free1, "a steady-state multi-index search allocated device memory"
    # eight of them: the same number of launches
    s3 = b200.search_multi_stats()
    D8, I8 = b200.search_multi(indexes[:8], xq, k, merged=False)
    s4 = b200.search_multi_stats()
    check(D8, I8, np.stack(Ds[:8]), np.stack(Is[:8]), "eight indexes")
    assert s4["group_launches"] - s3["group_launches"] == per_call_64
    # a member changes: the copy is rebuilt and the new row is found
    xb5, ids5 = bases[5]
    extra = xq[:1].copy()
    indexes[5].add_with_ids(extra, np.array([10**9], dtype=np.int64))
    Dn, In = b200.search_multi(indexes, xq, k, merged=False)
    assert b200.search_multi_stats()["group_rebuilds"] == s4["group_rebuilds"] + 1   # the copy follows its members
    assert In[5, 0, 0] == 10**9 or metric != L2
    if is_int:
        Dr5, Ir5 = oracle.int8_search(metric, np.concatenate([xb5, extra]), xq, k, labels=np.concatenate([ids5, [10**9]]))
    else:
        Dr5, Ir5 = oracle.flat_search(metric, np.concatenate([xb5, extra]), xq, k, labels=np.concatenate([ids5, [10**9]]))
    check(Dn[5], In[5], Dr5, Ir5, "changed member")


def test_group_copy_does_not_outlive_its_members(b200):
    """The concatenated copy of a group is cached against its members' identity.  New indexes that
    the allocator places where destroyed ones lived (same addresses, same number of adds) must not
    be mistaken for them: several rounds of create / search / destroy with different data and
    alternating metrics, each checked against the oracle."""
    import gc
    d, k, nq = 64, 10, 17
    xq = datasets.gaussian(nq, d, seed=1)
    for rnd in range(6):
        metric = L2 if rnd % 2 == 0 else IP
        indexes, Ds, Is = [], [], []
        for s_, n in enumerate((900, 300, 2000)):
            xb = datasets.gaussian(n, d, seed=1000 + 10 * rnd + s_)
            ids = np.arange(n, dtype=np.int64) + 5000 * s_
            ix = b200.IndexFlat(d, metric)
            ix.add_with_ids(xb, ids)
            indexes.append(ix)
            Dr, Ir = oracle.flat_search(metric, xb, xq, k, labels=ids)
            Ds.append(Dr)
            Is.append(Ir)
        D, I = b200.search_multi(indexes, xq, k, merged=False)
        assert_exact(D, I, np.stack(Ds), np.stack(Is))
        del indexes, ix
        gc.collect()
