"""ShardedSearcher over NCCL on two GPUs (skipped on a box with one): the base sharded by id
(IVFPQ with the probe exchange, Flat) and the replicated / query-parallel layout, every rank's
merged result bit for bit against the CPU oracle's search over the whole base."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import oracle
    import indexsdk_b200 as b
    from indexsdk_b200 import datasets
    from indexsdk_b200.sharded import ShardedSearcher
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    notes = []
    try:
        b.load()
        # ---- IVFPQ, residual and raw encoding, id mod world shards + probe exchange; replica layout
        d, nlist, M, n, k, nprobe = 64, 64, 16, 40000, 10, 8
        xb, _ = datasets.mixture(n, d, nlist, seed=4)
        ids = np.arange(n, dtype=np.int64)
        for resid in (True, False):
            cent, cb = datasets.train_ivfpq(xb[:4000], nlist, M, resid, niter=3)
            ln = oracle.ivf_assign(cent, xb)
            codes = oracle.pq_encode(cb, xb, resid, cent, ln)
            off, cs, li = oracle.build_lists(ln, codes, ids, nlist)

            def make(rows):
                ix = b.IndexIVFPQ(d, nlist, M, 8, by_residual=resid, device=rank)
                ix.set_centroids(cent)
                ix.set_codebooks(cb)
                ix.add_with_ids(xb[rows], ids[rows])
                ix.nprobe = nprobe
                return ix
            shard, full = make(slice(rank, None, world)), make(slice(None))
            for nq in (1501, 7):            # with and without the probe exchange, slices that do not divide
                xq, _ = datasets.mixture(nq, d, nlist, seed=5, centers_seed=4)
                Dr, Ir = oracle.ivfpq_search(cent, cb, resid, off, cs, li, xq, nprobe, k)
                xq_t = torch.from_numpy(xq).to(dev)
                for mode, ix in (("shard", shard), ("replica", full)):
                    D, I = ShardedSearcher(ix, mode=mode).search_device(xq_t, k)
                    if not (np.array_equal(I.cpu().numpy(), Ir) and np.array_equal(D.cpu().numpy(), Dr)):
                        notes.append(f"ivfpq resid={resid} nq={nq} mode={mode}")
        # ---- Flat fp32 (contiguous slices) and Int8Flat
        xf = datasets.gaussian(30000, 64, seed=0)
        xq = datasets.gaussian(300, 64, seed=1)
        lo, hi = 30000 * rank // world, 30000 * (rank + 1) // world
        fx = b.IndexFlat(64, b.METRIC_L2, device=rank)
        fx.add_with_ids(xf[lo:hi], np.arange(lo, hi, dtype=np.int64))
        s = ShardedSearcher(fx)
        D, I = s.search_device(torch.from_numpy(xq).to(dev), 20)
        Dr, Ir = oracle.flat_search(oracle.METRIC_L2, xf, xq, 20)
        if not (np.array_equal(I.cpu().numpy(), Ir) and np.array_equal(D.cpu().numpy(), Dr)):
            notes.append("flat")
        res = s.search(torch.from_numpy(xq).pin_memory(), 20)          # host in, host out
        if rank == 0 and not np.array_equal(res[1].numpy(), Ir):
            notes.append("flat host path")
        xi = datasets.uniform_int8(20000, 64, seed=2)
        qi = datasets.uniform_int8(33, 64, seed=3)
        lo, hi = 20000 * rank // world, 20000 * (rank + 1) // world
        ii = b.IndexInt8Flat(64, b.METRIC_INNER_PRODUCT, device=rank)
        ii.add_with_ids(xi[lo:hi], np.arange(lo, hi, dtype=np.int64))
        D, I = ShardedSearcher(ii, descending=True).search_device(torch.from_numpy(qi).to(dev), 10)
        Dr, Ir = oracle.int8_search(oracle.METRIC_IP, xi, qi, 10)
        if not (np.array_equal(I.cpu().numpy(), Ir) and np.array_equal(D.cpu().numpy(), Dr)):
            notes.append("int8")
    except Exception as e:  # noqa: BLE001
        notes.append(repr(e))
    finally:
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if not notes else "; ".join(notes))
        dist.barrier()
        dist.destroy_process_group()


def test_sharded_searcher_over_nccl(tmp_path, b200, oracle_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"
