#!/usr/bin/env python
"""Benchmark of the search hot path on seeded synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload ivfpq10m|flat1m|int8flat4m|ivfpq100m|multiflat20m]
                    [--impl ours|reference] [--by-residual 0|1]

One "step" is one pass of the search path over one batch of queries.  The default workload is
the IVFPQ configuration the headline metric is quoted on (10 M vectors, d=128, nlist=16384,
M=16 x 8 bit, nprobe=64, k=10, 10 000 queries per step); `flat1m` and `int8flat4m` are the
exact-search configurations.  Prints ONE JSON line (rank 0).

  value : queries/s with queries and results resident in HBM (device-pointer C ABI call)
  e2e   : queries/s through the host-pointer API, H2D of queries and D2H of results included
  roofline : dominant kernel (IVFPQ: code scan, HBM-bound; Flat: distance GEMM, tensor-bound)
             timed live with CUDA events on the index's own stream
  cpu_baseline : the CPU oracle (a port of the reference's CPU semantics; Faiss itself is not
             installed) on a bounded sample of the same queries, all host threads

With --gpus N > 1 (launched by torchrun) the base is sharded by id modulo N, every rank
searches all queries on its shard, and the per-rank top-k are all-gathered over NCCL and merged
on device (strong scaling: total work is fixed).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

# DRAM bytes (read + write) per launch of the dominant kernel on ONE GPU, from an ncu capture of
# that kernel: full-size launch for the IVFPQ scan; quarter-size captures scaled by four for the
# exact-search GEMMs (their traffic grows with the base).  None until a capture exists.
NCU_TRAFFIC_BYTES = {
    "ivfpq10m": 1.766e9,      # ivfpq_scan_persist_kernel: 1.722 GB read + 43.9 MB written
    "flat1m": 2.98e8,         # append pass, both stretches: 4 x (73.4 MB read + 1.0 MB written)
    "int8flat4m": 1.051e9,    # append pass, both stretches: 4 x (257.3 MB read + 5.4 MB written)
}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            m = json.load(f)
        return dict(hbm=float(m["hbm_gbs"]), tflops=float(m["bf16_tflops"]),
                    tflops_sustained=float(m.get("bf16_tflops_sustained", m["bf16_tflops"])), source="measured")
    return dict(hbm=FALLBACK_HBM_GBS, tflops=FALLBACK_BF16_TFLOPS, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock / throttle-reason sampling while the steps run (reads only, nothing is set).

    A thread polls NVML every 2 ms (the timed regions last tens of milliseconds, too short for an
    external nvidia-smi loop to see) and stamps each sample with time.perf_counter(); `mark()`
    brackets the timed regions, and the summary prefers the samples inside them.  The steps are
    repeated untimed for a short hold phase afterwards so that the driver's own clock counters,
    which refresh more slowly than the poll, are read at least a few times under the same load.
    Without NVML the nvidia-smi loop is the fallback."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str | None = None):
        self.gpu = gpu_index
        self.uuid = uuid
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []          # (t, sm_mhz, power_w, reasons bitmask)
        self.windows = []          # [(t0, t1)] timed regions
        self.smax = None
        self._stop = False
        self.source = None

    def _nvml_loop(self, nv, h):
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                rs = int(get_reasons(h))
                self.samples.append((time.perf_counter(), float(sm), pw, rs))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            h = None
            if self.uuid:
                try:
                    h = nv.nvmlDeviceGetHandleByUUID(self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid)
                except Exception:
                    h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nv = nv
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            self.source = "nvml, 2 ms poll"
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi -lms 100"
        except Exception:
            self.proc = None

    def mark(self, t0, t1):
        self.windows.append((t0, t1))

    def _summarise(self, sm, power, masks, smax, where):
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake_slowdown"}
        reasons = sorted({n for m in masks for bit, n in names.items() if m & bit})
        busy = [c for c, pw in zip(sm, power) if pw >= 0.6 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": smax, "reasons": reasons, "samples": len(sm),
                "power_w_max": max(power), "source": self.source, "window": where}

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            inside = [x for x in self.samples if any(t0 <= x[0] <= t1 for t0, t1 in self.windows)]
            use, where = (inside, "timed regions") if len(inside) >= 3 else \
                (self.samples, "warm-up, timed regions and the untimed hold phase of identical steps")
            if use:
                out = self._summarise([x[1] for x in use], [x[2] for x in use], [x[3] for x in use], self.smax, where)
                out["samples_in_timed_regions"] = len(inside)
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, masks, smax, power = [], [], None, []
        try:
            for line in open(self.path):
                f = [t.strip() for t in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    smax = float(f[2])
                    power.append(float(f[3]))
                except ValueError:
                    continue
                m = 0
                for bit, v in zip((0x8, 0x40, 0x20, 0x4), f[5:9]):
                    if v.lower().startswith("active"):
                        m |= bit
                masks.append(m)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        if sm:
            out = self._summarise(sm, power, masks, smax, "whole run of the sampler")
        return out


# --------------------------------------------------------------------------------------
# workload construction (untimed; torch is plumbing for data generation and training)
# --------------------------------------------------------------------------------------
def farthest_first(x, k, seed):
    """Deterministic k-means++-style seeding (farthest-first traversal): every new centre is the
    point farthest from the centres chosen so far.  The reference exposes the same choice as
    AscendIndexIVFConfig::useKmeansPP; with random seeding Lloyd iterations leave some mixture
    components without a centroid and the inverted lists badly unbalanced."""
    import torch
    g = torch.Generator(device=x.device)
    g.manual_seed(seed)
    n = x.shape[0]
    idx = int(torch.randint(0, n, (1,), generator=g, device=x.device))
    cent = torch.empty((k, x.shape[1]), dtype=x.dtype, device=x.device)
    xn = (x * x).sum(1)
    mind = torch.full((n,), float("inf"), dtype=x.dtype, device=x.device)
    sel = torch.tensor(idx, device=x.device)
    for i in range(k):
        c = x[sel]
        cent[i] = c
        mind = torch.minimum(mind, xn - 2.0 * (x @ c) + (c * c).sum())
        sel = mind.argmax()
    return cent


def torch_kmeans(x, k, niter, seed, plusplus=False):
    import torch
    g = torch.Generator(device=x.device)
    g.manual_seed(seed)
    n = x.shape[0]
    if plusplus:
        cent = farthest_first(x, k, seed)
    else:
        cent = x[torch.randperm(n, generator=g, device=x.device)[:k]].clone()
    step = max(4096, min(131072, (1 << 29) // max(k, 1)))     # rows per distance block (<= 2 GiB of fp32)
    for _ in range(niter):
        cn = (cent * cent).sum(1)
        assign = torch.empty(n, dtype=torch.int64, device=x.device)
        for s in range(0, n, step):
            xs = x[s:s + step]
            assign[s:s + step] = (cn[None, :] - 2.0 * (xs @ cent.T)).argmin(1)
        counts = torch.bincount(assign, minlength=k)
        sums = torch.zeros_like(cent).index_add_(0, assign, x)
        nz = counts > 0
        cent[nz] = sums[nz] / counts[nz, None].to(x.dtype)
        ne = int((~nz).sum())
        if ne:
            cent[~nz] = x[torch.randint(0, n, (ne,), generator=g, device=x.device)]
    return cent


def assign_torch(x, cent):
    import torch
    cn = (cent * cent).sum(1)
    out = torch.empty(x.shape[0], dtype=torch.int64, device=x.device)
    step = max(4096, min(131072, (1 << 29) // max(cent.shape[0], 1)))
    for s in range(0, x.shape[0], step):
        out[s:s + step] = (cn[None, :] - 2.0 * (x[s:s + step] @ cent.T)).argmin(1)
    return out


class Workload:
    name = ""
    k = 10
    nq = 0
    dtype = "f32"
    descending = False
    full_index = None      # unsharded copy of the index (IVFPQ at N > 1 only)


class IvfpqWorkload(Workload):
    """IVFPQ on a Gaussian mixture (centres ~ N(0,1), sigma 0.1), coarse centroids and PQ codebooks
    trained by seeded k-means (25 iterations) on a 500 k sample, 10 000 queries from the same
    mixture.  `ivfpq10m`: d=128, N=10 M, 16384 centres / lists, M=16 x 8 bit, nprobe=64, k=10.
    `ivfpq100m`: d=96, N=100 M, 65536 centres / lists, M=48 x 8 bit, nprobe=128, k=100 (the sharded
    configuration: base vectors round-robin by id over the ranks)."""
    name = "ivfpq10m"
    CONFIGS = {
        "ivfpq10m": dict(d=128, nlist=16384, M=16, nprobe=64, k=10, N=10_000_000, seed=4, qseed=5),
        "ivfpq100m": dict(d=96, nlist=65536, M=48, nprobe=128, k=100, N=100_000_000, seed=6, qseed=7),
    }

    def __init__(self, b, dev, rank, world, by_residual, scale=1.0, name="ivfpq10m", full_copy=False):
        import torch
        self.name = name
        cfg = self.CONFIGS[name]
        self.d, self.nlist, self.M, self.nprobe, self.k = cfg["d"], cfg["nlist"], cfg["M"], cfg["nprobe"], cfg["k"]
        self.N = int(cfg["N"] * scale)
        self.nq = 10_000
        self.by_residual = bool(by_residual)
        self.dtype = "f32"
        nc = self.nlist
        g = torch.Generator(device=dev)
        g.manual_seed(cfg["seed"])
        centers = torch.randn(nc, self.d, generator=g, device=dev)
        chunk = 1_000_000

        def gen(seed, n):
            gg = torch.Generator(device=dev)
            gg.manual_seed(seed)
            which = torch.randint(0, nc, (n,), generator=gg, device=dev)
            return centers[which] + 0.1 * torch.randn(n, self.d, generator=gg, device=dev)

        t0 = time.time()
        base_seed = 1000 * cfg["seed"]
        dsub = self.d // self.M
        if rank == 0 or world == 1:
            sample = gen(base_seed, min(chunk, self.N))[:500_000]
            cent = torch_kmeans(sample, self.nlist, 25, seed=41, plusplus=True)
            train = sample
            if self.by_residual:
                train = sample - cent[assign_torch(sample, cent)]
            cb = torch.stack([torch_kmeans(train[:, m * dsub:(m + 1) * dsub].contiguous(), 256, 25, seed=50 + m)
                              for m in range(self.M)])
            del sample, train
        else:
            cent = torch.empty((self.nlist, self.d), device=dev)
            cb = torch.empty((self.M, 256, dsub), device=dev)
        if world > 1:
            # ONE trained quantizer for all ranks: the k-means above sums with atomics, so two ranks
            # training on their own would end up with centroids that differ in the last bits
            import torch.distributed as dist
            dist.broadcast(cent, 0)
            dist.broadcast(cb, 0)
        self.train_s = time.time() - t0
        self.centroids = cent.cpu().numpy()
        self.codebooks = cb.cpu().numpy()
        def new_index():
            ix = b.IndexIVFPQ(self.d, self.nlist, self.M, 8, by_residual=self.by_residual, device=dev.index)
            ix.set_centroids(self.centroids)
            ix.set_codebooks(self.codebooks)
            ix.nprobe = self.nprobe
            return ix
        ix = new_index()
        # the unsharded index beside the shard: the replicated (query-parallel) layout, and on rank 0
        # the lists the CPU oracle searches when the merged sharded result is checked
        self.full_index = new_index() if (full_copy and world > 1) else None
        t0 = time.time()
        for c in range((self.N + chunk - 1) // chunk):
            n = min(chunk, self.N - c * chunk)
            x = gen(base_seed + c, n)
            ids = np.arange(c * chunk, c * chunk + n, dtype=np.int64)
            torch.cuda.synchronize(dev)
            if self.full_index is not None:
                self.full_index.add_device(x.data_ptr(), n, ids)
            if world > 1:
                x = x[rank::world].contiguous()
                ids = ids[rank::world].copy()
            torch.cuda.synchronize(dev)
            ix.add_device(x.data_ptr(), x.shape[0], ids)
            del x
        self.add_s = time.time() - t0
        self.index = ix
        self._gen, self._base_seed, self._chunk = gen, base_seed, chunk
        self.xq = gen(cfg["qseed"], self.nq).cpu().pin_memory()
        self.units_bytes_per_query = self.nprobe * (self.N / self.nlist) * self.M   # algorithmic scan bytes
        lens = np.array([ix.list_length(l) for l in range(self.nlist)], np.float64)
        self.desc = dict(workload="IVFPQ d=%d N=%d nlist=%d M=%dx8bit nprobe=%d k=%d nq=10000 "
                                  "(Gaussian mixture, seeded k-means++ init + 25 Lloyd it on 500k sample)"
                                  % (self.d, self.N, self.nlist, self.M, self.nprobe, self.k),
                         by_residual=self.by_residual)
        self.run_info = dict(list_len_mean=float(lens.mean()), list_len_max=float(lens.max()),
                             list_len_size_biased_mean=float((lens * lens).sum() / max(lens.sum(), 1)))

    def roofline(self, stats, steps, peaks):
        # the scan stage of ONE search: the filter scan and, where queries were left unverified (raw
        # encoding), the second filter pass -- all of it is charged to the algorithmic bytes of one scan
        ms = stats["stage_ms"]["scan"] / max(1, steps)
        alg = self.units_bytes_per_query * self.nq / max(1, self.world_size)
        ach = alg / (ms * 1e-3) / 1e9 if ms > 0 else None
        visited = stats["scan_codes_delta"] * self.M / max(1, steps)
        kern = "ivfpq_scan_persist_kernel" if self.M == 16 else "ivfpq_fast_scan_kernel"
        return dict(bound="hbm", kernel=kern, achieved=ach, peak=peaks["hbm"], unit="GB/s",
                    frac=(ach / peaks["hbm"]) if ach else None, peak_source=peaks["source"],
                    traffic=NCU_TRAFFIC_BYTES.get(self.name), algorithmic_bytes_per_launch=alg,
                    visited_code_bytes_per_launch=visited, ms_per_launch=ms)

    def first_rows(self, n):
        """The first n base vectors (ids 0 .. n-1), regenerated."""
        return self._gen(self._base_seed, min(self._chunk, self.N))[:n].cpu().numpy()

    def cpu_reference(self, oracle, nsample):
        ix = self.full_index if self.full_index is not None else self.index
        if getattr(self, "_lists", None) is not None:
            offs, codes, ids = self._lists
            return self._cpu_run(oracle, offs, codes, ids)
        offs = np.zeros(self.nlist + 1, np.int64)
        lens = np.array([ix.list_length(l) for l in range(self.nlist)], np.int64)
        np.cumsum(lens, out=offs[1:])
        codes = np.empty((int(offs[-1]), self.M), np.uint8)
        ids = np.empty(int(offs[-1]), np.int64)
        for l in range(self.nlist):
            if lens[l]:
                c, i = ix.get_list(l)
                codes[offs[l]:offs[l + 1]] = c
                ids[offs[l]:offs[l + 1]] = i
        self._lists = (offs, codes, ids)
        return self._cpu_run(oracle, offs, codes, ids)

    def _cpu_run(self, oracle, offs, codes, ids):
        xq = self.xq.numpy()
        variant = 1 if self.by_residual else 0

        def run(n):
            t0 = time.perf_counter()
            D, I = oracle.ivfpq_search(self.centroids, self.codebooks, variant, offs, codes, ids, xq[:n],
                                       self.nprobe, self.k)
            return time.perf_counter() - t0, D, I
        return run


class FlatWorkload(Workload):
    """Flat L2 exact search, fp32: base 1 000 000 x 128 N(0,1), 1024 queries, k=100."""
    name = "flat1m"

    def __init__(self, b, dev, rank, world, scale=1.0):
        import torch
        self.d, self.k, self.nq = 128, 100, 1024
        self.N = int(1_000_000 * scale)
        self.dtype = "bf16 filter + f32 refine"
        g = torch.Generator(device=dev)
        g.manual_seed(0)
        xb = torch.randn(self.N, self.d, generator=g, device=dev)
        g.manual_seed(1)
        xq = torch.randn(self.nq, self.d, generator=g, device=dev)
        ids = np.arange(self.N, dtype=np.int64)
        self.xb_host = None
        if rank == 0:
            self.xb_host = xb.cpu().numpy()
        if world > 1:
            lo, hi = self.N * rank // world, self.N * (rank + 1) // world   # contiguous slices
            xb, ids = xb[lo:hi].contiguous(), ids[lo:hi].copy()
        ix = b.IndexFlat(self.d, b.METRIC_L2, b.F32, device=dev.index)
        torch.cuda.synchronize(dev)
        ix.add_device(xb.data_ptr(), xb.shape[0], ids)
        self.index = ix
        self.xq = xq.cpu().pin_memory()
        self.flops_per_query = 2.0 * self.N * self.d
        self.desc = dict(workload="Flat L2 fp32 N=%d d=128 nq=1024 k=100 (i.i.d. N(0,1))" % self.N)

    def roofline(self, stats, steps, peaks):
        ms = stats["stage_ms"]["full_gemm"] / max(1, stats["stage_launches"]["full_gemm"])
        alg = self.flops_per_query * self.nq / max(1, self.world_size)
        ach = alg / (ms * 1e-3) / 1e12 if ms > 0 else None
        return dict(bound="tensor", kernel="dist_gemm_tc_kernel (append pass)", achieved=ach, peak=peaks["tflops"],
                    unit="TFLOP/s", frac=(ach / peaks["tflops"]) if ach else None, peak_source=peaks["source"],
                    traffic=NCU_TRAFFIC_BYTES.get(self.name), algorithmic_flops_per_launch=alg, ms_per_launch=ms)

    def cpu_reference(self, oracle, nsample):
        xq = self.xq.numpy()

        def run(n):
            t0 = time.perf_counter()
            D, I = oracle.flat_search(oracle.METRIC_L2, self.xb_host, xq[:n], self.k)
            return time.perf_counter() - t0, D, I
        return run


class Int8Workload(Workload):
    """Int8Flat inner product: base 4 000 000 x 256 int8 U[-128,127], 256 queries, k=100."""
    name = "int8flat4m"
    descending = True

    def __init__(self, b, dev, rank, world, scale=1.0):
        import torch
        self.d, self.k, self.nq = 256, 100, 256
        self.N = int(4_000_000 * scale)
        self.dtype = "int8 -> int32"
        g = torch.Generator(device=dev)
        g.manual_seed(2)
        xb = torch.randint(-128, 128, (self.N, self.d), generator=g, device=dev, dtype=torch.int8)
        g.manual_seed(3)
        xq = torch.randint(-128, 128, (self.nq, self.d), generator=g, device=dev, dtype=torch.int8)
        ids = np.arange(self.N, dtype=np.int64)
        self.xb_host = xb.cpu().numpy() if rank == 0 else None
        if world > 1:
            lo, hi = self.N * rank // world, self.N * (rank + 1) // world
            xb, ids = xb[lo:hi].contiguous(), ids[lo:hi].copy()
        ix = b.IndexInt8Flat(self.d, b.METRIC_INNER_PRODUCT, device=dev.index)
        torch.cuda.synchronize(dev)
        ix.add_device(xb.data_ptr(), xb.shape[0], ids)
        self.index = ix
        self.xq = xq.cpu().pin_memory()
        self.desc = dict(workload="Int8Flat IP N=%d d=256 nq=256 k=100 (uniform int8)" % self.N)

    def roofline(self, stats, steps, peaks):
        ms = stats["stage_ms"]["full_gemm"] / max(1, stats["stage_launches"]["full_gemm"])
        alg = float(self.N) * self.d / max(1, self.world_size)          # base bytes streamed once per batch
        ach = alg / (ms * 1e-3) / 1e9 if ms > 0 else None
        return dict(bound="hbm", kernel="dist_gemm_tc_kernel<i8> (append pass)", achieved=ach, peak=peaks["hbm"],
                    unit="GB/s", frac=(ach / peaks["hbm"]) if ach else None, peak_source=peaks["source"],
                    traffic=NCU_TRAFFIC_BYTES.get(self.name), algorithmic_bytes_per_launch=alg, ms_per_launch=ms)

    def cpu_reference(self, oracle, nsample):
        xq = self.xq.numpy()

        def run(n):
            t0 = time.perf_counter()
            D, I = oracle.int8_search(oracle.METRIC_IP, self.xb_host, xq[:n], self.k)
            return time.perf_counter() - t0, D, I
        return run


class MultiIndexAdapter:
    """Several indexes on one device behind the interface the bench drives: every search runs on
    all of them and merges on the device -- what b200idx_search_multi(..., merged) does for host
    pointers, with device pointers for the device-resident figure."""

    def __init__(self, b, indexes, dev, descending):
        import torch
        self.b, self.indexes, self.dev, self.descending = b, indexes, dev, descending
        self.device = indexes[0].device
        self.stream_ptr = indexes[0].stream_ptr
        self._tmp = None
        self._torch = torch

    def set_timing(self, on):
        for ix in self.indexes:
            ix.set_timing(on)

    def stats(self):
        out = None
        for ix in self.indexes:
            s = ix.stats()
            if out is None:
                out = s
                continue
            for key, v in s.items():
                if isinstance(v, dict):
                    for n2 in v:
                        out[key][n2] += v[n2]
                else:
                    out[key] += v
        return out

    def search_device(self, x_ptr, n, k, D_ptr, I_ptr):
        torch = self._torch
        nh = len(self.indexes)
        if self._tmp is None or self._tmp[0].shape != (nh, n, k):
            self._tmp = (torch.empty((nh, n, k), dtype=torch.float32, device=self.dev),
                         torch.empty((nh, n, k), dtype=torch.int64, device=self.dev))
        tD, tI = self._tmp
        for i, ix in enumerate(self.indexes):
            ix.search_device(x_ptr, n, k, tD[i].data_ptr(), tI[i].data_ptr())   # returns when its stream is idle
        self.b.merge_topk_device(nh, n, k, self.descending, tD.data_ptr(), tI.data_ptr(), D_ptr, I_ptr, self.stream_ptr)
        torch.cuda.ExternalStream(self.stream_ptr, device=self.dev).synchronize()

    def search_into(self, x, k, D, I):
        Dm, Im = self.b.search_multi(self.indexes, x, k, merged=True)
        D[...] = Dm
        I[...] = Im


class MultiFlatWorkload(Workload):
    """Eight fp16 Flat inner-product indexes of 2 500 000 x 768 L2-normalised N(0,1) rows each,
    4096 normalised queries, k=1000 merged over all indexes; the indexes are dealt to the ranks
    round-robin (one per GPU at 8 GPUs)."""
    name = "multiflat20m"
    descending = True

    def __init__(self, b, dev, rank, world, scale=1.0):
        import torch
        self.d, self.k, self.nq, self.n_indexes = 768, 1000, 4096, 8
        self.n_each = int(2_500_000 * scale)
        self.N = self.n_each * self.n_indexes
        self.dtype = "fp16 -> f32"
        chunk = 250_000

        def gen(seed, n):
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            x = torch.randn(n, self.d, generator=g, device=dev)
            return x / x.norm(dim=1, keepdim=True)

        mine = [i for i in range(self.n_indexes) if i % world == rank]
        self.indexes, self.first_base = [], None
        for i in mine:
            ix = b.IndexFlat(self.d, b.METRIC_INNER_PRODUCT, dtype=b.F16, device=dev.index)
            for c in range((self.n_each + chunk - 1) // chunk):
                n = min(chunk, self.n_each - c * chunk)
                x = gen(8000 + 100 * i + c, n)
                ids = np.arange(i * self.n_each + c * chunk, i * self.n_each + c * chunk + n, dtype=np.int64)
                torch.cuda.synchronize(dev)
                ix.add_device(x.data_ptr(), n, ids)
                if rank == 0 and i == mine[0]:
                    part = x.half().float().cpu().numpy()     # the values the index holds
                    self.first_base = part if self.first_base is None else np.concatenate([self.first_base, part])
                del x
            self.indexes.append(ix)
        self.index = MultiIndexAdapter(b, self.indexes, dev, True)
        self.xq = gen(9, self.nq).cpu().pin_memory()
        self.flops_per_query = 2.0 * self.N * self.d
        self.desc = dict(workload="8 x Flat IP fp16 N=%d each d=768 nq=4096 k=1000 merged (L2-normalised N(0,1) rows)"
                                  % self.n_each, indexes_on_this_rank=len(mine))

    def roofline(self, stats, steps, peaks):
        launches = max(1, stats["stage_launches"]["full_gemm"])
        ms = stats["stage_ms"]["full_gemm"] / launches
        alg = self.flops_per_query * self.nq / self.n_indexes          # one index's pass
        ach = alg / (ms * 1e-3) / 1e12 if ms > 0 else None
        return dict(bound="tensor", kernel="dist_gemm_tc_kernel<f16> (append pass, one index)", achieved=ach,
                    peak=peaks["tflops"], unit="TFLOP/s", frac=(ach / peaks["tflops"]) if ach else None,
                    peak_source=peaks["source"], traffic=None, algorithmic_flops_per_launch=alg, ms_per_launch=ms)

    def parity_results(self, m):
        """GPU results of the first index alone, to set against the oracle on that index."""
        return self.indexes[0].search(np.ascontiguousarray(self.xq.numpy()[:m]), self.k)

    def cpu_reference(self, oracle, nsample):
        # The CPU arm searches ONE index (7.7 GB of fp32 rows; all eight would not fit the host) and
        # its rate is divided by the number of indexes: exact search is linear in the base size.
        xq = np.ascontiguousarray(self.xq.numpy().astype(np.float16).astype(np.float32))
        self.cpu_note = "; one of the 8 indexes searched, time multiplied by 8"

        def run(n):
            t0 = time.perf_counter()
            D, I = oracle.flat_search(oracle.METRIC_IP, self.first_base, xq[:n], self.k)
            return (time.perf_counter() - t0) * self.n_indexes, D, I
        return run


def make_workload(name, b, dev, rank, world, args, full_copy=False):
    if name in IvfpqWorkload.CONFIGS:
        w = IvfpqWorkload(b, dev, rank, world, args.by_residual, args.scale, name=name,
                          full_copy=full_copy and IvfpqWorkload.CONFIGS[name]["N"] * args.scale <= 20_000_000)
    elif name == "flat1m":
        w = FlatWorkload(b, dev, rank, world, args.scale)
    elif name == "int8flat4m":
        w = Int8Workload(b, dev, rank, world, args.scale)
    elif name == "multiflat20m":
        w = MultiFlatWorkload(b, dev, rank, world, args.scale)
    else:
        raise SystemExit(f"unknown workload {name}")
    w.world_size = world
    return w


def time_cpu(run, nq_total, target_s=12.0, first=16):
    """Bounded CPU sample: a short probe sizes a run of about target_s seconds."""
    n0 = min(first, nq_total)
    t, _, _ = run(n0)
    per = t / n0
    n = int(max(n0, min(nq_total, target_s / max(per, 1e-9))))
    t, D, I = run(n)                      # also warms the caches for the timed passes
    reps = int(max(1, min(200, round(target_s / max(t, 1e-9)))))
    total = 0.0
    for _ in range(reps):
        t, D, I = run(n)
        total += t
    return n * reps / total, n * reps, total


def probe_faiss():
    """Is Faiss (the reference's CPU ground truth) importable on this box?  Recorded in the line;
    when it is, the CPU oracle is cross-checked against it."""
    try:
        import faiss  # noqa: F401
        return dict(importable=True, version=getattr(faiss, "__version__", "?"))
    except Exception as e:  # ImportError on this image
        return dict(importable=False, why=type(e).__name__)


def faiss_cross_check(wl, oracle):
    """Only reached when Faiss is importable: the oracle against Faiss' own Flat search on 64 queries."""
    try:
        import faiss
        if not isinstance(wl, FlatWorkload) or wl.xb_host is None:
            return None
        ix = faiss.IndexFlatL2(wl.d)
        ix.add(wl.xb_host)
        xq = wl.xq.numpy()[:64]
        Df, If = ix.search(xq, wl.k)
        Do, Io = oracle.flat_search(oracle.METRIC_L2, wl.xb_host, xq, wl.k)
        return dict(queries=64, id_agreement=float((If == Io).mean()),
                    max_rel_distance_error=float(np.max(np.abs(Df - Do) / np.maximum(np.abs(Do), 1e-30))))
    except Exception as e:
        return dict(error=str(e)[:200])


def parity_against_oracle(wl, oracle, Dg, Ig, m):
    """The merged GPU results of the first m queries against the CPU oracle on the WHOLE base."""
    run = wl.cpu_reference(oracle, None)
    _, Dr, Ir = run(m)
    if hasattr(wl, "parity_results"):
        Dg, Ig = wl.parity_results(m)
    same = float((Ig[:m] == Ir).mean())
    relerr = float(np.max(np.abs(Dg[:m] - Dr) / np.maximum(np.abs(Dr), 1e-30)))
    return dict(queries=int(m), id_agreement=same, max_rel_distance_error=relerr,
                checked="merged result of all ranks against the CPU oracle on the whole base")


def encode_check(wl, oracle, nsample=4096):
    """IVFPQ: the lists the product built (GPU assignment + PQ encoding) against the oracle's own
    assignment and encoding of the first vectors of the base."""
    if not isinstance(wl, IvfpqWorkload):
        return None
    ix = wl.full_index if wl.full_index is not None else wl.index
    x = wl.first_rows(nsample)
    ln = oracle.ivf_assign(wl.centroids, x)
    codes = oracle.pq_encode(wl.codebooks, x, wl.by_residual, wl.centroids, ln)
    ok_list = ok_code = 0
    cache = {}
    for i in range(x.shape[0]):
        l = int(ln[i])
        if l not in cache:
            cache[l] = ix.get_list(l)
        c, ids = cache[l]
        pos = np.flatnonzero(ids == i)
        if pos.size == 1:
            ok_list += 1
            ok_code += int(np.array_equal(c[pos[0]], codes[i]))
    return dict(vectors=int(x.shape[0]), list_agreement=ok_list / x.shape[0], code_agreement=ok_code / x.shape[0])


def reference_arm(wl, args, oracle):
    """The CPU arm: the oracle port on all host threads, a bounded sample per step."""
    cores = oracle.use_all_host_threads()
    nq = wl.nq
    run = wl.cpu_reference(oracle, None)
    # each step: a bounded sample sized so that warmup + steps stay within a few minutes
    budget = 120.0 / max(1, args.steps + args.warmup)
    t, _, _ = run(min(8, nq))
    n = int(max(8, min(nq, budget / max(t / min(8, nq), 1e-9))))
    for _ in range(args.warmup):
        run(n)
    times = []
    for _ in range(args.steps):
        t, _, _ = run(n)
        times.append(t)
    ms = 1e3 * sum(times) / len(times)
    val = n / (ms * 1e-3)
    sample = "%d of %d queries per step%s" % (n, nq, getattr(wl, "cpu_note", ""))
    return dict(metric="QPS", value=val, unit="queries/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype=wl.dtype, data="synthetic", impl="reference", config=dict(wl.desc),
                cpu_baseline=dict(value=val, unit="queries/s", cores=cores, kind="port",
                                  sample=sample + ", all host threads (OpenMP), CPU oracle port; Faiss is not installed"),
                e2e=dict(value=val, unit="queries/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                encode_check=encode_check(wl, oracle))


def measure(wl, args, b, dev, rank, world, dist, sampler, peaks, mode):
    """Device-resident and end-to-end timing of one workload; returns the JSON line as a dict."""
    import torch
    from indexsdk_b200.sharded import ShardedSearcher
    k, nq = wl.k, wl.nq
    index = wl.full_index if (mode == "replica" and wl.full_index is not None) else wl.index
    searcher = ShardedSearcher(index, descending=wl.descending, mode=mode)
    xq_host = wl.xq                                            # pinned CPU tensor
    xq_dev = xq_host.to(dev)
    outD = torch.empty((nq, k), dtype=torch.float32, pin_memory=True)
    outI = torch.empty((nq, k), dtype=torch.int64, pin_memory=True)
    xq_np, outD_np, outI_np = xq_host.numpy(), outD.numpy(), outI.numpy()
    lib_stream = torch.cuda.ExternalStream(index.stream_ptr, device=dev)

    def step_device():
        searcher.search_device(xq_dev, k)

    def step_e2e():
        if world == 1:
            index.search_into(xq_np, k, outD_np, outI_np)      # host pointers through the C ABI
        else:
            searcher.search(xq_host, k, outD, outI)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        # every stage of a step is queued on the index's own stream: two events on it bracket the steps
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(lib_stream)
        for _ in range(steps):
            fn()
        e1.record(lib_stream)
        e1.synchronize()
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        sampler.mark(t0, t1)
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    for _ in range(args.warmup):
        step_device()
        step_e2e()
    index.set_timing(True)
    s0 = index.stats()
    ms_dev = timed(step_device, args.steps)
    s1 = index.stats()
    index.set_timing(False)
    ms_e2e = timed(step_e2e, args.steps)
    # hold phase: the same steps, untimed, for about half a second, so that the clock counters are
    # read several times under the load that was just timed (same count on every rank)
    for _ in range(min(2000, max(1, int(500.0 / max(ms_dev, 1e-3))))):
        step_device()
    barrier()

    # counters are cumulative: everything below is the difference over the device-resident region
    stats = dict(s1)
    stats["scan_codes_delta"] = s1["scan_codes"] - s0["scan_codes"]
    stats["stage_ms"] = {n: s1["stage_ms"][n] - s0["stage_ms"][n] for n in s1["stage_ms"]}
    stats["stage_launches"] = {n: s1["stage_launches"][n] - s0["stage_launches"][n] for n in s1["stage_launches"]}
    # per step at N > 1: + the merge kernel and the unpack copies of the exchange
    launches = s1["kernel_launches"] - s0["kernel_launches"] + (3 * args.steps if world > 1 else 0)
    roof = wl.roofline(stats, args.steps, peaks)
    if world > 1:
        roof["traffic"] = None           # the ncu capture behind the constant was taken on one GPU
    par = {"shard": ("single GPU" if world == 1 else
                     "base sharded over %d ranks (IVFPQ: id mod N, Flat: contiguous slices), one packed NCCL "
                     "all-gather of per-rank top-k + merge kernel" % world),
           "replica": "index replicated on %d ranks, queries split evenly, one packed NCCL all-gather of the "
                      "result slices (the reference's query-parallel search)" % world}[mode]
    line = dict(metric="QPS", value=nq / (ms_dev * 1e-3), unit="queries/s", n_gpus=world, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms_dev, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype=wl.dtype, data="synthetic", config=dict(wl.desc),
                run=dict(nq_per_step=nq, l2_flush="inputs larger than L2 (codes/base >> 126 MB)", parallelism=par,
                         **getattr(wl, "run_info", {})),
                e2e=dict(value=nq / (ms_e2e * 1e-3), unit="queries/s", ms_per_step=ms_e2e,
                         h2d_bytes_per_step=int(xq_host.numel() * xq_host.element_size()),
                         d2h_bytes_per_step=int(nq * k * 12)),
                gpu_launches=int(launches),
                roofline=roof,
                stage_ms_per_step={n: v / args.steps for n, v in stats["stage_ms"].items() if v > 0},
                fallback_queries_per_step=(s1["fallback_queries"] - s0["fallback_queries"]) / args.steps,
                second_pass_queries_per_step=(s1["second_pass_queries"] - s0["second_pass_queries"]) / args.steps)
    return line, (outD_np, outI_np)


# --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ivfpq10m")
    ap.add_argument("--by-residual", type=int, default=1)
    ap.add_argument("--parallelism", default="shard", choices=["shard", "replica"],
                    help="N > 1: shard the base (default) or replicate it and split the queries")
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the base (development only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-blocks", action="store_true",
                    help="default workload only: skip the Flat-1M block (and the replica block at N > 1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference" and rank != 0:
        return   # the CPU arm runs on rank 0 alone

    import torch
    import torch.distributed as dist
    import indexsdk_b200 as b

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    b.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    ref_arm = args.impl == "reference"
    if world > 1 and not ref_arm:
        dist.init_process_group("nccl", device_id=dev)
    eff_world = 1 if ref_arm else world
    peaks = measured_peaks()
    default_run = args.workload == "ivfpq10m" and not args.no_extra_blocks and args.scale == 1.0

    if ref_arm:
        import oracle
        wl = make_workload(args.workload, b, dev, 0, 1, args)
        line = reference_arm(wl, args, oracle)
        line["faiss"] = probe_faiss()
        if default_run:
            del wl
            wf = make_workload("flat1m", b, dev, 0, 1, args)
            fl = reference_arm(wf, args, oracle)
            line["flat1m"] = {n: fl[n] for n in ("metric", "value", "unit", "ms_per_step", "config", "cpu_baseline")}
        print(json.dumps(line))
        return

    try:
        gpu_uuid = str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local_rank, gpu_uuid)
    if rank == 0:
        sampler.start()

    def one(name, mode, cpu_leg):
        t_setup = time.time()
        want_full = world > 1 and (rank == 0 or mode == "replica" or default_run)
        wl = make_workload(name, b, dev, rank, eff_world, args, full_copy=want_full)
        setup_s = time.time() - t_setup
        line, (oD, oI) = measure(wl, args, b, dev, rank, world, dist, sampler, peaks, mode)
        line["run"]["setup_s"] = round(setup_s, 1)
        if rank == 0 and not args.no_cpu_baseline:
            import oracle
            cores = oracle.use_all_host_threads()
            m = min(64, wl.nq)
            if world > 1 and isinstance(wl, IvfpqWorkload) and wl.full_index is None:
                line["parity_check"] = None      # the whole base is not held by any one rank at this size
            else:
                line["parity_check"] = parity_against_oracle(wl, oracle, oD, oI, m)
            if cpu_leg:
                run = wl.cpu_reference(oracle, None)
                qps, n, t = time_cpu(run, wl.nq)
                line["cpu_baseline"] = dict(value=qps, unit="queries/s", cores=cores, kind="port",
                                            sample="%d queries (the batch of %d, repeated), %.1f s, CPU oracle port "
                                                   "with OpenMP on all host threads (Faiss is not installed)%s"
                                                   % (n, wl.nq, t, getattr(wl, "cpu_note", "")))
                fx = faiss_cross_check(wl, oracle) if probe_faiss()["importable"] else None
                if fx:
                    line["faiss_cross_check"] = fx
        return line, wl

    line, wl = one(args.workload, args.parallelism, cpu_leg=(world == 1))
    if rank == 0:
        line["faiss"] = probe_faiss()
    if default_run:
        # The metric names two workloads; the exact-search one follows as its own block, and at
        # N > 1 the replicated (query-parallel) layout of the IVFPQ index next to the sharded one.
        if world > 1 and args.parallelism == "shard":
            rl, _ = measure(wl, args, b, dev, rank, world, dist, sampler, peaks, "replica")
            if rank == 0:
                line["replica"] = {n: rl[n] for n in ("value", "unit", "ms_per_step", "e2e", "run", "stage_ms_per_step")}
        del wl
        torch.cuda.empty_cache()
        fl, _ = one("flat1m", "shard", cpu_leg=(world == 1))
        if rank == 0:
            keep = ("metric", "value", "unit", "n_gpus", "ms_per_step", "dtype", "config", "run", "e2e", "gpu_launches",
                    "roofline", "stage_ms_per_step", "fallback_queries_per_step", "parity_check", "cpu_baseline")
            line["flat1m"] = {n: fl[n] for n in keep if n in fl}
    if rank == 0:
        line["clocks"] = sampler.stop()
        # the exact-search block goes last so that it survives in a truncated tail of the output
        if "flat1m" in line:
            line["flat1m"] = line.pop("flat1m")
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
