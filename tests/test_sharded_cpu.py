"""World-size-2 check (gloo, CPU) of the sharded search protocol: every rank searches its shard,
per-rank top-k are all-gathered, and the merge rule (key, then label) reproduces the search over
the whole base.  The local search is played by the CPU oracle here; the GPU path uses the same
protocol with NCCL and the device merge kernel (indexsdk_b200/sharded.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from indexsdk_b200 import datasets
from indexsdk_b200.sharded import merge_on_host


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, metric, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, n, nq, k = 32, 3000, 11, 20
        xb = datasets.gaussian(n, d, seed=1)
        xq = datasets.gaussian(nq, d, seed=2)
        ids = np.arange(n, dtype=np.int64)
        # id-round-robin shard, as the IVFPQ configuration shards its base
        D, I = oracle.flat_search(metric, xb[rank::world], xq, k, labels=ids[rank::world])
        allD = [torch.empty(nq, k) for _ in range(world)]
        allI = [torch.empty(nq, k, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(allD, torch.from_numpy(D))
        dist.all_gather(allI, torch.from_numpy(I))
        Dm, Im = merge_on_host([t.numpy() for t in allD], [t.numpy() for t in allI],
                               descending=(metric == oracle.METRIC_IP))
        Dr, Ir = oracle.flat_search(metric, xb, xq, k)
        ok = np.array_equal(Im, Ir) and np.array_equal(Dm, Dr)
        # the C oracle's merge states the same rule
        Dc, Ic = oracle.merge_topk(np.stack([t.numpy() for t in allD]), np.stack([t.numpy() for t in allI]),
                                   descending=(metric == oracle.METRIC_IP))
        ok = ok and np.array_equal(Ic, Ir) and np.array_equal(Dc, Dr)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("metric", [oracle.METRIC_L2, oracle.METRIC_IP])
def test_two_rank_gather_and_merge(tmp_path, metric):
    oracle.build()
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), metric, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_merge_rule_padding_and_ties():
    D0 = np.array([[0.5, 0.5, 3.0]], np.float32)
    I0 = np.array([[7, 9, -1]], np.int64)
    D1 = np.array([[0.5, 2.0, 3.4e38]], np.float32)
    I1 = np.array([[8, 1, -1]], np.int64)
    D, I = merge_on_host([D0, D1], [I0, I1])
    assert I.tolist() == [[7, 8, 9]] and D.tolist() == [[0.5, 0.5, 0.5]]
