"""Base set sharded over the ranks of one node: one process per GPU, local top-k on every rank,
one NCCL all-gather of the per-rank results over NVLink, merge kernel on local memory.

This is the multi-device fan-out / fan-in of the reference
(feature_retrieval/src/ascendfaiss/ascend/impl/AscendIndexImpl.cpp:375-403 fan-out,
:587-642 host merge; IVFPQ device split AscendIndexIVFPQImpl.cpp:304-353) re-cut for one
process per GPU: the only exchange step is the all-gather of n*k (distance, label) pairs.
No peer-memory loads: remote results land in local HBM through NCCL before the merge kernel
reads them.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import merge_topk_device


class ShardedSearcher:
    """Wraps a rank-local index (IndexFlat / IndexInt8Flat / IndexIVFPQ holding this rank's
    shard, labels = global ids) and produces global results on every rank."""

    def __init__(self, index, descending: bool = False, group=None):
        self.index = index
        self.descending = descending
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device("cuda", index.device)
        self._buf = {}

    def _buffers(self, n: int, k: int):
        key = (n, k)
        if key not in self._buf:
            dev = self.device
            self._buf = {key: dict(
                locD=torch.empty((n, k), dtype=torch.float32, device=dev),
                locI=torch.empty((n, k), dtype=torch.int64, device=dev),
                allD=torch.empty((self.world, n, k), dtype=torch.float32, device=dev),
                allI=torch.empty((self.world, n, k), dtype=torch.int64, device=dev),
                outD=torch.empty((n, k), dtype=torch.float32, device=dev),
                outI=torch.empty((n, k), dtype=torch.int64, device=dev))}
        return self._buf[key]

    def search_device(self, xq: torch.Tensor, k: int):
        """xq: [n, d] device tensor in the index's query dtype.  Returns device tensors (D, I)
        holding the merged global top-k (valid on every rank)."""
        n = xq.shape[0]
        b = self._buffers(n, k)
        torch.cuda.current_stream(self.device).synchronize()   # xq produced on torch's stream
        if self.world > 1 and hasattr(self.index, "coarse_device") and n >= 4 * self.world:
            self._search_ivfpq_split_coarse(xq, n, k, b)
        else:
            self.index.search_device(xq.data_ptr(), n, k, b["locD"].data_ptr(), b["locI"].data_ptr())
        if self.world == 1:
            return b["locD"], b["locI"]
        dist.all_gather_into_tensor(b["allD"], b["locD"], group=self.group)
        dist.all_gather_into_tensor(b["allI"], b["locI"], group=self.group)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        merge_topk_device(self.world, n, k, self.descending, b["allD"].data_ptr(), b["allI"].data_ptr(),
                          b["outD"].data_ptr(), b["outI"].data_ptr(), stream)
        return b["outD"], b["outI"]

    def _search_ivfpq_split_coarse(self, xq, n, k, b):
        """IVFPQ shards hold the full coarse quantizer, so probe selection would be repeated on every
        rank: instead each rank selects the probes of an even slice of the queries, one all-gather
        (n * nprobe * 12 bytes) makes them known everywhere, and every rank scans its shard for all
        queries with the given probes.  Results are those of a plain search."""
        nprobe = min(self.index.nprobe, self.index.nlist)
        per = (n + self.world - 1) // self.world
        key = ("probe", n, nprobe)
        if key not in self._buf:
            dev = self.device
            self._buf[key] = dict(
                myD=torch.empty((per, nprobe), dtype=torch.float32, device=dev),
                myI=torch.empty((per, nprobe), dtype=torch.int64, device=dev),
                allD=torch.empty((self.world * per, nprobe), dtype=torch.float32, device=dev),
                allI=torch.empty((self.world * per, nprobe), dtype=torch.int64, device=dev))
        p = self._buf[key]
        lo = min(self.rank * per, n)
        cnt = max(0, min(per, n - lo))
        if cnt < per:                       # a short (or empty) last slice: defined padding
            p["myD"].zero_()
            p["myI"].fill_(-1)
        if cnt:
            self.index.coarse_device(xq[lo:lo + cnt].data_ptr(), cnt, p["myD"].data_ptr(), p["myI"].data_ptr())
        dist.all_gather_into_tensor(p["allD"], p["myD"], group=self.group)
        dist.all_gather_into_tensor(p["allI"], p["myI"], group=self.group)
        torch.cuda.current_stream(self.device).synchronize()   # the index runs on its own stream
        self.index.search_preassigned_device(xq.data_ptr(), n, k, p["allD"].data_ptr(), p["allI"].data_ptr(),
                                             b["locD"].data_ptr(), b["locI"].data_ptr())

    def search(self, xq_host: torch.Tensor, k: int, out_D: torch.Tensor | None = None,
               out_I: torch.Tensor | None = None):
        """Host in, host out: xq_host is a (preferably pinned) CPU tensor; results are copied
        back on rank 0 (other ranks return None)."""
        xq = xq_host.to(self.device, non_blocking=True)
        D, I = self.search_device(xq, k)
        if self.rank != 0:
            torch.cuda.current_stream(self.device).synchronize()
            return None
        if out_D is None:
            out_D = torch.empty(D.shape, dtype=D.dtype, pin_memory=True)
            out_I = torch.empty(I.shape, dtype=I.dtype, pin_memory=True)
        out_D.copy_(D, non_blocking=True)
        out_I.copy_(I, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
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
