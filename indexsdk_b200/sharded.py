"""Search over the ranks of one node: one process per GPU, local top-k on every rank, ONE
all-gather of the per-rank results over NVLink, merge kernel on local memory.

This is the multi-device fan-out / fan-in of the reference
(feature_retrieval/src/ascendfaiss/ascend/impl/AscendIndexImpl.cpp:375-403 fan-out,
:587-642 host merge; IVFPQ device split AscendIndexIVFPQImpl.cpp:304-353) re-cut for one
process per GPU.  Two ways to use the ranks:

* ``mode="shard"`` -- every rank holds a slice of the base (labels = global ids) and searches ALL
  queries on it; the exchange step is the all-gather of n*k (distance, label) pairs and the merge
  orders them by (distance, label).  IVFPQ shards all hold the full coarse quantizer, so each
  rank selects the probes of an even slice of the queries and one more all-gather makes them
  known everywhere.
* ``mode="replica"`` -- every rank holds the WHOLE index and searches an even slice of the queries;
  the exchange step is the all-gather of the result slices.  This is the reference's
  query-parallel search (AscendIndexIVFPQConfig::enableQueryParallelSearch,
  feature_retrieval/src/ascendfaiss/ascend/impl/AscendIndexIVFPQImpl.cpp:1305-1328: the index is
  replicated on every device and the query batch is split across them).

No peer-memory loads: remote results land in local HBM through the collective before a kernel
reads them.  Per-rank blocks are packed -- distances and labels side by side in one byte
buffer -- so that an exchange is one collective, and everything (searches, collectives, merge)
is queued on the index's own stream: the host does not wait between the stages of a step.

The tensor plumbing is injected (``ops``) so that the slicing / padding / packing logic runs
unchanged over the ``gloo`` backend with a CPU stand-in for the index (tests).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def _round8(v: int) -> int:
    return (v + 7) // 8 * 8


class _CudaOps:
    """Device-side plumbing of ShardedSearcher: buffers in HBM, work queued on the index's stream."""

    def __init__(self, index):
        from . import merge_topk_device
        self._merge = merge_topk_device
        self.device = torch.device("cuda", index.device)
        self.stream = torch.cuda.ExternalStream(index.stream_ptr, device=self.device)

    def empty(self, nbytes: int) -> torch.Tensor:
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device)

    def on_stream(self):
        return torch.cuda.stream(self.stream)

    def wait_for_caller(self):
        """The queries were produced on the caller's current stream."""
        self.stream.wait_stream(torch.cuda.current_stream(self.device))

    def synchronize(self):
        self.stream.synchronize()

    def caller_waits(self):
        """Work queued on the caller's stream from here on starts after the index's stream is done."""
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def synchronize_caller(self):
        torch.cuda.current_stream(self.device).synchronize()

    def merge(self, nsrc, n, k, descending, packed, stride_bytes, d_off, i_off, outD, outI):
        base = packed.data_ptr()
        self._merge(nsrc, n, k, descending, base + d_off, base + i_off, outD.data_ptr(), outI.data_ptr(),
                    self.stream.cuda_stream, src_stride_bytes=stride_bytes)


class ShardedSearcher:
    """Wraps a rank-local index (IndexFlat / IndexInt8Flat / IndexIVFPQ) and produces global
    results on every rank.  mode="shard": the index holds this rank's slice of the base;
    mode="replica": the index holds the whole base and the queries are split."""

    def __init__(self, index, descending: bool = False, group=None, mode: str = "shard", ops=None):
        if mode not in ("shard", "replica"):
            raise ValueError("mode must be 'shard' or 'replica'")
        self.index = index
        self.descending = descending
        self.group = group
        self.mode = mode
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops if ops is not None else _CudaOps(index)
        self.device = self.ops.device
        self._buf = {}

    # ---- packed blocks: [rows*cols float32 | pad to 8 | rows*cols int64] -------------------------
    @staticmethod
    def _block_bytes(rows: int, cols: int) -> tuple[int, int]:
        i_off = _round8(rows * cols * 4)
        return i_off + rows * cols * 8, i_off

    def _views(self, buf: torch.Tensor, rows: int, cols: int, i_off: int):
        D = buf[:rows * cols * 4].view(torch.float32).view(rows, cols)
        I = buf[i_off:i_off + rows * cols * 8].view(torch.int64).view(rows, cols)
        return D, I

    def _get(self, key, make):
        if key not in self._buf:
            self._buf[key] = make()
        return self._buf[key]

    # ---- public entry points ----------------------------------------------------------------------
    def search_device(self, xq: torch.Tensor, k: int):
        """xq: [n, d] tensor on the index's device in the index's query dtype.  Returns tensors
        (D, I) holding the global top-k (valid on every rank once the index's stream is idle;
        this call returns after synchronising it)."""
        D, I = self._search_async(xq, k)
        self.ops.synchronize()
        return D, I

    def _search_async(self, xq: torch.Tensor, k: int):
        n = xq.shape[0]
        # Buffers are allocated here, on the caller's stream, and only USED on the index's stream:
        # memory that the caching allocator ties to a stream must not outlive that stream, and the
        # index (which owns it) may be destroyed before these tensors are.
        if self.world == 1:
            b = self._get(("one", n, k), lambda: dict(
                D=self.ops.empty(n * k * 4).view(torch.float32).view(n, k),
                I=self.ops.empty(n * k * 8).view(torch.int64).view(n, k)))
        elif self.mode == "replica":
            b = self._replica_buffers(n, k)
        else:
            b = self._shard_buffers(n, k)
        self.ops.wait_for_caller()
        with self.ops.on_stream():
            if self.world == 1:
                self.index.search_device(xq.data_ptr(), n, k, b["D"].data_ptr(), b["I"].data_ptr())
                return b["D"], b["I"]
            if self.mode == "replica":
                return self._search_replica(xq, n, k, b)
            return self._search_shard(xq, n, k, b)

    # ---- mode "shard" ---------------------------------------------------------------------------
    def _use_probe_exchange(self, n):
        return hasattr(self.index, "coarse_device") and n >= 4 * self.world

    def _shard_buffers(self, n, k):
        blk, i_off = self._block_bytes(n, k)
        b = self._get(("shard", n, k), lambda: dict(
            blk=blk, i_off=i_off, all=self.ops.empty(self.world * blk),
            outD=self.ops.empty(n * k * 4).view(torch.float32).view(n, k),
            outI=self.ops.empty(n * k * 8).view(torch.int64).view(n, k)))
        if self._use_probe_exchange(n):
            nprobe = min(self.index.nprobe, self.index.nlist)      # may change between calls
            per = (n + self.world - 1) // self.world
            pblk, pi_off = self._block_bytes(per, nprobe)
            b["probe"] = self._get(("probe", n, nprobe), lambda: dict(
                nprobe=nprobe, per=per, blk=pblk, i_off=pi_off, all=self.ops.empty(self.world * pblk),
                cD=self.ops.empty(self.world * per * nprobe * 4).view(torch.float32).view(self.world * per, nprobe),
                cI=self.ops.empty(self.world * per * nprobe * 8).view(torch.int64).view(self.world * per, nprobe)))
        return b

    def _search_shard(self, xq, n, k, b):
        blk, i_off = b["blk"], b["i_off"]
        mine = b["all"][self.rank * blk:(self.rank + 1) * blk]      # this rank's block, filled in place
        locD, locI = self._views(mine, n, k, i_off)
        if self._use_probe_exchange(n):
            cD, cI = self._exchange_probes(xq, n, b["probe"])
            self.index.search_preassigned_device(xq.data_ptr(), n, k, cD.data_ptr(), cI.data_ptr(),
                                                 locD.data_ptr(), locI.data_ptr())
        else:
            self.index.search_device(xq.data_ptr(), n, k, locD.data_ptr(), locI.data_ptr())
        dist.all_gather_into_tensor(b["all"], mine, group=self.group)
        self.ops.merge(self.world, n, k, self.descending, b["all"], blk, 0, i_off, b["outD"], b["outI"])
        return b["outD"], b["outI"]

    def _exchange_probes(self, xq, n, p):
        """Each rank selects the probes of an even slice of the queries (every shard holds the full
        coarse quantizer, so the selection would otherwise be repeated on every rank); one
        all-gather of packed (distance, list) blocks makes them known everywhere.  Returns
        [n][nprobe] tensors, identical on every rank and identical to a local probe selection."""
        nprobe, per, blk, i_off = p["nprobe"], p["per"], p["blk"], p["i_off"]
        mine = p["all"][self.rank * blk:(self.rank + 1) * blk]
        myD, myI = self._views(mine, per, nprobe, i_off)
        lo = min(self.rank * per, n)
        cnt = max(0, min(per, n - lo))
        if cnt < per:                       # a short (or empty) last slice: defined padding, same stream
            myD[cnt:].zero_()
            myI[cnt:].fill_(-1)
        if cnt:
            self.index.coarse_device(xq[lo:lo + cnt].data_ptr(), cnt, myD.data_ptr(), myI.data_ptr())
        dist.all_gather_into_tensor(p["all"], mine, group=self.group)
        packed = p["all"].view(self.world, blk)
        p["cD"].view(self.world, per * nprobe).copy_(packed[:, :per * nprobe * 4].view(torch.float32))
        p["cI"].view(self.world, per * nprobe).copy_(packed[:, i_off:i_off + per * nprobe * 8].view(torch.int64))
        return p["cD"], p["cI"]

    # ---- mode "replica" -------------------------------------------------------------------------
    def _replica_buffers(self, n, k):
        per = (n + self.world - 1) // self.world
        blk, i_off = self._block_bytes(per, k)
        return self._get(("replica", n, k), lambda: dict(
            per=per, blk=blk, i_off=i_off, all=self.ops.empty(self.world * blk),
            outD=self.ops.empty(self.world * per * k * 4).view(torch.float32).view(self.world * per, k),
            outI=self.ops.empty(self.world * per * k * 8).view(torch.int64).view(self.world * per, k)))

    def _search_replica(self, xq, n, k, b):
        per, blk, i_off = b["per"], b["blk"], b["i_off"]
        mine = b["all"][self.rank * blk:(self.rank + 1) * blk]
        myD, myI = self._views(mine, per, k, i_off)
        lo = min(self.rank * per, n)
        cnt = max(0, min(per, n - lo))
        if cnt < per:
            myD[cnt:].fill_(3.4028234663852886e38)
            myI[cnt:].fill_(-1)
        if cnt:
            self.index.search_device(xq[lo:lo + cnt].data_ptr(), cnt, k, myD.data_ptr(), myI.data_ptr())
        dist.all_gather_into_tensor(b["all"], mine, group=self.group)
        packed = b["all"].view(self.world, blk)
        b["outD"].view(self.world, per * k).copy_(packed[:, :per * k * 4].view(torch.float32))
        b["outI"].view(self.world, per * k).copy_(packed[:, i_off:i_off + per * k * 8].view(torch.int64))
        return b["outD"][:n], b["outI"][:n]

    # ---- host in, host out ------------------------------------------------------------------------
    def search(self, xq_host: torch.Tensor, k: int, out_D: torch.Tensor | None = None,
               out_I: torch.Tensor | None = None):
        """xq_host is a (preferably pinned) CPU tensor; results are copied back on rank 0 (other
        ranks return None)."""
        shape, dt = tuple(xq_host.shape), xq_host.dtype
        xq = self._get(("xq", shape, dt), lambda: self.ops.empty(xq_host.numel() * xq_host.element_size())
                       .view(dt).view(shape))
        # Copies from and to the caller's host tensors run on the CALLER's stream: the allocator of
        # pinned memory remembers the streams a block was used on until the block is freed, which
        # may be after the index -- and with it the index's stream -- is gone.
        xq.copy_(xq_host, non_blocking=True)
        D, I = self._search_async(xq, k)
        self.ops.caller_waits()
        if self.rank != 0:
            self.ops.synchronize_caller()
            return None
        if out_D is None:
            out_D = torch.empty(D.shape, dtype=D.dtype, pin_memory=D.is_cuda)
            out_I = torch.empty(I.shape, dtype=I.dtype, pin_memory=I.is_cuda)
        out_D.copy_(D, non_blocking=True)
        out_I.copy_(I, non_blocking=True)
        self.ops.synchronize_caller()
        return out_D, out_I


def merge_on_host(Ds, Is, descending: bool = False):
    """CPU statement of the merge rule used by the device kernel (ordering by key then label);
    lets the multi-rank logic be tested with the gloo backend."""
    D = np.concatenate(Ds, axis=1)
    I = np.concatenate(Is, axis=1)
    key = -D if descending else D
    key = np.where(I < 0, np.inf, key)
    k = Ds[0].shape[1]
    order = np.lexsort((I, key), axis=1)[:, :k]
    return np.take_along_axis(D, order, 1), np.take_along_axis(I, order, 1)
