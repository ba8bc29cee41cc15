"""World-size-2 checks (gloo, CPU) of the multi-rank search protocol.

`ShardedSearcher` (indexsdk_b200/sharded.py) itself runs here: its slicing, padding, packing,
all-gather and merge logic is driven over the gloo backend with CPU tensors, the rank-local index
being played by a stand-in that answers through the CPU oracle (the product index needs a GPU).
Covered: base sharded by id (Flat, and IVFPQ with the probe exchange, query counts that do and do
not divide by the world size) and the replicated / query-parallel layout; every rank's merged
result is compared bit for bit with the oracle's search over the whole base.
"""
import contextlib
import ctypes
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from indexsdk_b200 import datasets
from indexsdk_b200.sharded import ShardedSearcher, merge_on_host


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _arr(ptr, shape, ctype, dtype):
    n = int(np.prod(shape))
    return np.ctypeslib.as_array((ctype * n).from_address(ptr)).view(dtype).reshape(shape)


class CpuOps:
    """Host-side plumbing with the interface ShardedSearcher expects from its device plumbing."""
    device = torch.device("cpu")

    def empty(self, nbytes):
        return torch.empty(nbytes, dtype=torch.uint8)

    def on_stream(self):
        return contextlib.nullcontext()

    def wait_for_caller(self):
        pass

    def synchronize(self):
        pass

    def caller_waits(self):
        pass

    def synchronize_caller(self):
        pass

    def merge(self, nsrc, n, k, descending, packed, stride_bytes, d_off, i_off, outD, outI):
        blocks = packed.view(nsrc, stride_bytes)
        Ds = [blocks[s, d_off:d_off + n * k * 4].view(torch.float32).view(n, k).numpy() for s in range(nsrc)]
        Is = [blocks[s, i_off:i_off + n * k * 8].view(torch.int64).view(n, k).numpy() for s in range(nsrc)]
        Dm, Im = merge_on_host(Ds, Is, descending)
        outD.copy_(torch.from_numpy(np.ascontiguousarray(Dm)))
        outI.copy_(torch.from_numpy(np.ascontiguousarray(Im)))


class FakeFlat:
    """Rank-local exact index answered by the oracle; pointer-based like the product's binding."""

    def __init__(self, metric, xb, ids):
        self.metric, self.xb, self.ids, self.d = metric, xb, ids, xb.shape[1]

    def search_device(self, x_ptr, n, k, D_ptr, I_ptr):
        xq = _arr(x_ptr, (n, self.d), ctypes.c_float, np.float32)
        D, I = oracle.flat_search(self.metric, self.xb, xq, k, labels=self.ids)
        _arr(D_ptr, (n, k), ctypes.c_float, np.float32)[...] = D
        _arr(I_ptr, (n, k), ctypes.c_int64, np.int64)[...] = I


class FakeIvfpq:
    """Rank-local IVFPQ shard answered by the oracle.  search_preassigned_device insists that the
    probes it is handed are exactly the ones a local selection would produce."""

    def __init__(self, cent, cb, resid, ln, codes, ids, nprobe):
        self.cent, self.cb, self.resid, self.nprobe = cent, cb, resid, nprobe
        self.nlist, self.d = cent.shape[0], cent.shape[1]
        self.off, self.codes, self.ids = oracle.build_lists(ln, codes, ids, self.nlist)
        self.calls = dict(coarse=0, pre=0, plain=0)

    def coarse_device(self, x_ptr, n, cD_ptr, cI_ptr):
        self.calls["coarse"] += 1
        xq = _arr(x_ptr, (n, self.d), ctypes.c_float, np.float32)
        D, I = oracle.flat_search(oracle.METRIC_L2, self.cent, xq, self.nprobe)
        _arr(cD_ptr, (n, self.nprobe), ctypes.c_float, np.float32)[...] = D
        _arr(cI_ptr, (n, self.nprobe), ctypes.c_int64, np.int64)[...] = I

    def search_preassigned_device(self, x_ptr, n, k, cD_ptr, cI_ptr, D_ptr, I_ptr):
        self.calls["pre"] += 1
        xq = _arr(x_ptr, (n, self.d), ctypes.c_float, np.float32)
        cD = _arr(cD_ptr, (n, self.nprobe), ctypes.c_float, np.float32)
        cI = _arr(cI_ptr, (n, self.nprobe), ctypes.c_int64, np.int64)
        Dc, Ic = oracle.flat_search(oracle.METRIC_L2, self.cent, xq, self.nprobe)
        assert np.array_equal(cI, Ic) and np.array_equal(cD, Dc), "exchanged probes differ from a local selection"
        self._search(xq, n, k, D_ptr, I_ptr)

    def search_device(self, x_ptr, n, k, D_ptr, I_ptr):
        self.calls["plain"] += 1
        self._search(_arr(x_ptr, (n, self.d), ctypes.c_float, np.float32), n, k, D_ptr, I_ptr)

    def _search(self, xq, n, k, D_ptr, I_ptr):
        D, I = oracle.ivfpq_search(self.cent, self.cb, self.resid, self.off, self.codes, self.ids, xq, self.nprobe, k)
        _arr(D_ptr, (n, k), ctypes.c_float, np.float32)[...] = D
        _arr(I_ptr, (n, k), ctypes.c_int64, np.int64)[...] = I


def _ivfpq_problem(resid):
    d, nlist, M, n = 32, 16, 4, 4000
    xb, _ = datasets.mixture(n, d, nlist, seed=4)
    cent, cb = datasets.train_ivfpq(xb[:2000], nlist, M, resid, niter=4)
    ln = oracle.ivf_assign(cent, xb)
    codes = oracle.pq_encode(cb, xb, resid, cent, ln)
    return d, nlist, cent, cb, ln, codes, np.arange(n, dtype=np.int64)


def _worker(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = False
    try:
        kind, mode, nq = case
        if kind == "flat":
            metric = oracle.METRIC_IP if mode.endswith("ip") else oracle.METRIC_L2
            d, n, k = 32, 3000, 20
            xb = datasets.gaussian(n, d, seed=1)
            xq = datasets.gaussian(nq, d, seed=2)
            ids = np.arange(n, dtype=np.int64)
            replica = mode.startswith("replica")
            local = FakeFlat(metric, xb, ids) if replica else FakeFlat(metric, xb[rank::world], ids[rank::world])
            s = ShardedSearcher(local, descending=(metric == oracle.METRIC_IP), mode="replica" if replica else "shard",
                                ops=CpuOps())
            D, I = s.search_device(torch.from_numpy(xq), k)
            Dr, Ir = oracle.flat_search(metric, xb, xq, k)
            ok = np.array_equal(I.numpy(), Ir) and np.array_equal(D.numpy(), Dr)
            # host in / host out: rank 0 gets the result, the others None
            res = s.search(torch.from_numpy(xq), k)
            ok = ok and ((res is None) if rank else np.array_equal(res[1].numpy(), Ir))
        else:
            resid = mode.endswith("resid")
            d, nlist, cent, cb, ln, codes, ids = _ivfpq_problem(resid)
            xq, _ = datasets.mixture(nq, d, nlist, seed=5, centers_seed=4)
            k, nprobe = 10, 5
            replica = mode.startswith("replica")
            sel = slice(None) if replica else slice(rank, None, world)     # id mod world
            local = FakeIvfpq(cent, cb, resid, ln[sel], codes[sel], ids[sel], nprobe)
            s = ShardedSearcher(local, mode="replica" if replica else "shard", ops=CpuOps())
            D, I = s.search_device(torch.from_numpy(xq), k)
            off, cs, li = oracle.build_lists(ln, codes, ids, nlist)
            Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, li, xq, nprobe, k)
            ok = np.array_equal(I.numpy(), Ir) and np.array_equal(D.numpy(), Dr)
            if not replica:      # the probe exchange is the path taken once a rank has >= 4 queries
                ok = ok and (local.calls["pre"] == 1 if nq >= 4 * world else local.calls["plain"] == 1)
    finally:
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
        dist.destroy_process_group()


CASES = [
    ("flat", "shard_l2", 11), ("flat", "shard_ip", 11), ("flat", "replica_l2", 11), ("flat", "replica_l2", 1),
    ("ivfpq", "shard_raw", 16), ("ivfpq", "shard_resid", 13), ("ivfpq", "shard_raw", 9), ("ivfpq", "shard_raw", 3),
    ("ivfpq", "replica_resid", 7),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_sharded_searcher_two_ranks(tmp_path, case):
    oracle.build()
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_merge_rule_padding_and_ties():
    D0 = np.array([[0.5, 0.5, 3.0]], np.float32)
    I0 = np.array([[7, 9, -1]], np.int64)
    D1 = np.array([[0.5, 2.0, 3.4e38]], np.float32)
    I1 = np.array([[8, 1, -1]], np.int64)
    D, I = merge_on_host([D0, D1], [I0, I1])
    assert I.tolist() == [[7, 8, 9]] and D.tolist() == [[0.5, 0.5, 0.5]]
    # the C oracle's merge states the same rule
    Dc, Ic = oracle.merge_topk(np.stack([D0, D1]), np.stack([I0, I1]))
    assert Ic.tolist() == [[7, 8, 9]]
