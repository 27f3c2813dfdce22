"""Benchmark of the batch similarity-search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

Metric: queries/sec of exact top-k search (BASELINE.json).  The default workload (c2) is the
configuration the metric is quoted on: flat cosine, 1 000 000 x 768 fp32 rows (N(0,1), L2-normalised),
10 000 queries, k = 100.  A step is one batch search of all queries over the resident database.
With N > 1 (one process per GPU under torchrun) the rows are sharded across ranks and a step is one
vsk_search_sharded call per rank: each rank scans its shard, the shards agree on a per-query bound (one
all-reduce), the per-shard top-k lists travel as packed keys in one all-to-all, and every rank merges and
returns its 1/N of the queries ("scaling": "strong").

Other workloads (not the default line): c1 flat euclidean 100k x 128; c3 IVF (10M x 128, nlist 4096,
20 Lloyd iterations, nprobe 32); c4 int8 dot product 50M x 384; c5 filtered Manhattan 5M x 256; and
reduced copies (suffix s) for profiler captures.

value     queries/s with queries already in HBM (CUDA events on the library's stream, max over ranks)
e2e       queries/s through the host-pointer C-ABI call: pinned host queries in, host results out
roofline  the scan kernels' device time from CUDA events recorded around each launch, in a second timed region
          with the library's profiling on (profiling runs a batch on one stream, so that an event pair brackets
          one kernel alone; the first region runs large batches as two halves on two streams)
cpu_baseline / --impl reference: the CPU restatement of the reference's search on the host cores
other_workloads  (default run on one GPU only) c1, c2 with filters (c2f), c3, one rank's shard of c4, c5 and pq, each run as a child process
          of a few steps: value, ms_per_step, e2e, roofline, clocks (and c3's k-means contraction) of each
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20261125 * 10

# kind, metric, rows, dim, queries, k, name, extra
WORKLOADS = {
    "c1": dict(kind="flat", metric="euclidean", rows=100_000, dim=128, queries=1_000, k=10, cfg=1,
               name="flat-euclidean-100k-d128-q1000-k10"),
    "c2": dict(kind="flat", metric="cosine", rows=1_000_000, dim=768, queries=10_000, k=100, cfg=2,
               name="flat-cosine-1M-d768-q10000-k100"),
    "c2s": dict(kind="flat", metric="cosine", rows=200_000, dim=768, queries=2_048, k=100, cfg=2,
                name="flat-cosine-200k-d768-q2048-k100"),
    # one eighth of c2's rows with all of its queries: what one rank of an 8-GPU run searches
    "c2e": dict(kind="flat", metric="cosine", rows=125_000, dim=768, queries=10_000, k=100, cfg=2,
                name="flat-cosine-125k-d768-q10000-k100"),
    "c3": dict(kind="ivf", metric="euclidean", rows=10_000_000, dim=128, queries=10_000, k=10, cfg=3, nlist=4096,
               nprobe=32, iters=20, name="ivf-euclidean-10M-d128-nlist4096-nprobe32-q10000-k10"),
    "c3s": dict(kind="ivf", metric="euclidean", rows=1_000_000, dim=128, queries=2_048, k=10, cfg=3, nlist=1024,
                nprobe=32, iters=5, name="ivf-euclidean-1M-d128-nlist1024-nprobe32-q2048-k10"),
    "c4": dict(kind="sq8", metric="dotProduct", rows=50_000_000, dim=384, queries=10_000, k=10, cfg=4,
               name="int8-dot-50M-d384-q10000-k10"),
    # one eighth of c4's rows with all of its queries: what one rank of the 8-GPU run searches
    "c4e": dict(kind="sq8", metric="dotProduct", rows=6_250_000, dim=384, queries=10_000, k=10, cfg=4,
                name="int8-dot-6.25M-d384-q10000-k10"),
    "c4s": dict(kind="sq8", metric="dotProduct", rows=2_000_000, dim=384, queries=2_048, k=10, cfg=4,
                name="int8-dot-2M-d384-q2048-k10"),
    # the headline shape with a metadata filter on every query (half of the rows eligible): stays on the tensor path
    "c2f": dict(kind="filtered", metric="cosine", rows=1_000_000, dim=768, queries=10_000, k=100, cfg=2,
                name="filtered-cosine-1M-d768-q10000-k100"),
    "c5": dict(kind="filtered", metric="manhattan", rows=5_000_000, dim=256, queries=10_000, k=50, cfg=5,
               name="filtered-manhattan-5M-d256-q10000-k50"),
    "c5s": dict(kind="filtered", metric="manhattan", rows=500_000, dim=256, queries=1_024, k=50, cfg=5,
                name="filtered-manhattan-500k-d256-q1024-k50"),
    # product-quantised codes searched by asymmetric distance (the storage-scan step after int8)
    "pq": dict(kind="pq", metric="euclidean", rows=10_000_000, dim=128, queries=10_000, k=10, cfg=3, segments=16,
               code_bits=8, train_rows=262_144, iters=10, nlist=4096, name="pq-adc-10M-d128-m16-q10000-k10"),
    "pqs": dict(kind="pq", metric="euclidean", rows=2_000_000, dim=128, queries=2_048, k=10, cfg=3, segments=16,
                code_bits=8, train_rows=131_072, iters=5, nlist=1024, name="pq-adc-2M-d128-m16-q2048-k10"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        super().__init__(daemon=True)
        self.gpu, self.samples, self.stop_flag = gpu, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            time.sleep(0.05)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(self.samples[0][1]) if self.samples[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# synthetic data (seeded, generated on the GPU in slabs; the union over ranks is the same database
# at every world size because every slab has its own seed derived from its first row)
# ---------------------------------------------------------------------------------------------
SLAB = 1 << 18


def _gen_slab(torch, wl, first_row, count, device, centres=None):
    g = torch.Generator(device=device)
    g.manual_seed(SEED + wl["cfg"] * 1_000_003 + first_row)
    dim = wl["dim"]
    if wl["kind"] == "filtered":
        return torch.rand((count, dim), generator=g, dtype=torch.float32, device=device) * 2 - 1
    t = torch.randn((count, dim), generator=g, dtype=torch.float32, device=device)
    if wl["kind"] in ("ivf", "pq"):
        c = torch.randint(0, centres.shape[0], (count,), generator=g, device=device)
        return centres[c] + 0.1 * t
    if wl["metric"] == "cosine":
        t = t / t.norm(dim=1, keepdim=True)
    return t


def gen_rows(torch, wl, lo, hi, device, centres=None, out=None):
    """Rows [lo, hi) of the workload's database; slabs are aligned to SLAB so shards reproduce them."""
    res = out if out is not None else torch.empty((hi - lo, wl["dim"]), dtype=torch.float32, device=device)
    s = (lo // SLAB) * SLAB
    while s < hi:
        e = s + SLAB
        slab = _gen_slab(torch, wl, s, SLAB, device, centres)
        a, b = max(s, lo), min(e, hi)
        res[a - lo:b - lo] = slab[a - s:b - s]
        s = e
    return res


def gen_queries(torch, wl, device, centres=None):
    q = dict(wl)
    q["cfg"] = wl["cfg"] + 50
    return _gen_slab(torch, q, 0, wl["queries"], device, centres)


def gen_masks(torch, wl, lo, hi, device):
    g = torch.Generator(device=device)
    g.manual_seed(SEED + 777 + lo)
    # 64 Bernoulli(0.5) bits per row
    a = torch.randint(0, 2 ** 31, (hi - lo, 2), generator=g, device=device, dtype=torch.int64)
    b = torch.randint(0, 2 ** 2, (hi - lo,), generator=g, device=device, dtype=torch.int64)
    return (a[:, 0] | (a[:, 1] << 31) | (b << 62)).contiguous()


# ---------------------------------------------------------------------------------------------
# CPU baseline: the C++ restatement of the reference's CPU search, OpenMP over queries
# ---------------------------------------------------------------------------------------------
def cpu_rate(fn, nq_total, cores, seconds_target):
    """fn(nq) runs the CPU search on the first nq queries.  Sizes the sample for ~seconds_target."""
    n0 = min(nq_total, max(cores, 4))
    t0 = time.perf_counter()
    fn(n0)
    dt = time.perf_counter() - t0
    nq = int(min(nq_total, max(n0, seconds_target / max(dt / n0, 1e-9))))
    nq = min(nq_total, max(cores, (nq // cores) * cores))
    t0 = time.perf_counter()
    fn(nq)
    dt = time.perf_counter() - t0
    return nq / dt, nq, dt


def get_oracle():
    import oracle
    try:
        oracle.build(native=True)
        return oracle, oracle.CpuOracle(native=True)
    except Exception:
        return oracle, oracle.CpuOracle()


class Bench:
    """One workload on this rank's shard."""

    def __init__(self, torch, vsk, dev, engine, wl, rank, world, device, path):
        self.torch, self.vsk, self.dev, self.engine, self.wl = torch, vsk, dev, engine, wl
        self.rank, self.world, self.device = rank, world, device
        self.lo, self.hi = rank * wl["rows"] // world, (rank + 1) * wl["rows"] // world
        self.k, self.nq = wl["k"], wl["queries"]
        self.path = path
        self.extra = {}
        self.qmasks = None
        getattr(self, "_build_" + wl["kind"])()
        self.q_pinned = self.queries.cpu().pin_memory()
        self.out_d_host = torch.empty((self.nq, self.k), dtype=torch.float32).pin_memory()
        self.out_i_host = torch.empty((self.nq, self.k), dtype=torch.int64).pin_memory()
        self.qm_pinned = self.qmasks.cpu().pin_memory() if self.qmasks is not None else None
        from vectorstorekit_b200.sharded import ShardedSearch, join_communicator
        # every injected function launches on the library's stream; the collectives are ordered on it too
        self.stream = torch.cuda.ExternalStream(dev.stream, device=device)
        # flat fp32 (filtered or not) and int8 indexes: the whole sharded search is one C-ABI call
        # (vsk_search_sharded over the library's own NCCL communicator); IVF and PQ go through the injected form
        self.abi_sharded = world > 1 and wl["kind"] in ("flat", "filtered", "sq8")
        if self.abi_sharded:
            join_communicator(dev)
            first, count = vsk.sharded_slice(self.nq, world, rank)
            self.slice = (first, count)
            self.dev_out = (torch.empty((max(count, 1), self.k), dtype=torch.float32, device=device),
                            torch.empty((max(count, 1), self.k), dtype=torch.int64, device=device))
        self.sharded = ShardedSearch(self.local_search, engine.mergeTopK, stream=self.stream)

    # ---- builders ----
    def _build_flat(self):
        wl, t = self.wl, self.torch
        self.rows = gen_rows(t, wl, self.lo, self.hi, self.device)
        self.queries = gen_queries(t, wl, self.device)
        self.index = self.vsk.FlatIndex(self.dev, wl["dim"], wl["metric"])
        self.index.add(self.rows)
        self.index.set_id_base(self.lo)
        self.flops = 2.0 * self.nq * (self.hi - self.lo) * wl["dim"]
        self.bound = "tensor"

    def _build_filtered(self):
        wl, t = self.wl, self.torch
        self.rows = gen_rows(t, wl, self.lo, self.hi, self.device)
        self.masks = gen_masks(t, wl, self.lo, self.hi, self.device)
        self.queries = gen_queries(t, wl, self.device)
        g = t.Generator(device=self.device)
        g.manual_seed(SEED + 4242)
        self.qmasks = (t.ones(self.nq, dtype=t.int64, device=self.device)
                       << t.randint(0, 63, (self.nq,), generator=g, device=self.device)).contiguous()
        self.index = self.vsk.FlatIndex(self.dev, wl["dim"], wl["metric"])
        self.index.add(self.rows, self.masks)
        self.index.set_id_base(self.lo)
        if wl["metric"] == "manhattan":
            # FP32 lane-instructions of the eligible pairs: 2 per pair-dimension (subtract; add |.|)
            self.flops = 2.0 * self.nq * (self.hi - self.lo) * 0.5 * wl["dim"]
            self.bound = "fp32"
        else:
            # the contraction forms every pair and the filter sits in its epilogue: all pairs are counted, as for the
            # unfiltered workload the step time is compared with
            self.flops = 2.0 * self.nq * (self.hi - self.lo) * wl["dim"]
            self.bound = "tensor"

    def _build_ivf(self):
        wl, t = self.wl, self.torch
        g = t.Generator(device=self.device)
        g.manual_seed(SEED + 31337)
        centres = t.randn((wl["nlist"], wl["dim"]), generator=g, dtype=t.float32, device=self.device)
        self.rows = gen_rows(t, wl, self.lo, self.hi, self.device, centres)
        self.queries = gen_queries(t, wl, self.device, centres)
        ix = self.vsk.IVFIndex(self.dev, wl["dim"], numberOfCentroids=wl["nlist"], numberOfProbes=wl["nprobe"],
                               maxIterations=wl["iters"], tolerance=-1.0)
        t.cuda.synchronize()
        t0 = time.perf_counter()
        if self.world == 1:
            ix.train(self.rows, self.rows[:wl["nlist"]].contiguous())
        else:
            # rows are sharded: every Lloyd iteration all-reduces the per-centroid sums and counts, so that all
            # ranks hold the same centroids and every rank's lists are slices of the same lists
            import torch.distributed as dist
            from vectorstorekit_b200.sharded import ShardedKMeans
            init = gen_rows(t, wl, 0, wl["nlist"], self.device, centres)        # the first rows of the whole database
            # the first collective of a process sets up NCCL's channels (hundreds of ms): not part of an iteration
            warm = t.zeros(1, device=self.device)
            dist.all_reduce(warm)
            t.cuda.synchronize()
            t0 = time.perf_counter()
            trainer = self.vsk.KMeansTrainer(self.dev, self.rows, wl["nlist"])
            cent, _, _ = ShardedKMeans(trainer.step, trainer.finish).cluster(init, wl["iters"], -1.0)
            trainer.close()
            ix.centroids, ix.trained = cent, True
        t.cuda.synchronize()
        t1 = time.perf_counter()
        ix.insert(self.rows)
        if self.world > 1:
            ix.set_id_base(self.lo)
        t.cuda.synchronize()
        t2 = time.perf_counter()
        self.index = ix
        n = self.hi - self.lo
        self.extra = {"train_s": t1 - t0, "train_s_per_iteration": (t1 - t0) / wl["iters"], "build_s": t2 - t1,
                      "train_flops_per_iteration": 2.0 * n * wl["nlist"] * wl["dim"]}
        if self.world == 1:
            # The assignment contraction of a Lloyd iteration, timed by the library's own event log (CUDA events on its
            # stream) over a few more iterations on the same rows, outside every timed region: the launches marked
            # "assign_scan" are the threshold-mode contractions (the first iteration's arg-min launch has another name).
            self.dev.timeline(True)
            km = self.vsk.KMeansClustering(self.dev, maxIterations=6, tolerance=-1.0)
            km.cluster(self.rows, wl["nlist"], self.rows[:wl["nlist"]].contiguous())
            t.cuda.synchronize()
            marks = self.dev.timeline_read()
            self.dev.timeline(False)
            scans = [ms - marks[i - 1][2] for i, (_, what, ms) in enumerate(marks) if what == "assign_scan" and i > 0]
            if len(scans) > 2:
                scan_ms = float(np.median(scans[1:]))      # the first follows the arg-min launch's looser thresholds
                tf = self.extra["train_flops_per_iteration"] / (scan_ms * 1e-3) / 1e12
                pk = peaks()
                self.extra["train_contraction"] = {"kernel": "assign_scan_kernel", "ms_per_launch": scan_ms, "achieved": tf,
                                                   "unit": "TFLOP/s", "peak": pk["bf16_tflops"],
                                                   "frac": tf / pk["bf16_tflops"], "peak_source": pk["source"]}
        asg = ix.assignments()
        sizes = np.bincount(asg, minlength=wl["nlist"])
        self.extra["list_len_mean"] = float(sizes.mean())
        self.extra["list_len_max"] = int(sizes.max())
        # rows each query has to scan: the sizes of its nprobe nearest lists (computed with torch, outside the
        # timed region); lists differ in length, and a long list is also probed by more queries
        cent = ix.centroids if hasattr(ix.centroids, "is_cuda") else t.as_tensor(ix.centroids, device=self.device)
        probe = t.cdist(self.queries, cent).topk(wl["nprobe"], largest=False).indices
        scanned = t.as_tensor(sizes, device=self.device)[probe].sum(dim=1).double()
        self.extra["scanned_rows_per_query_mean"] = float(scanned.mean())
        self.extra["scanned_rows_per_query_max"] = float(scanned.max())
        # query-major algorithmic bytes: every query reads the rows of its nprobe lists once
        self.bytes_per_query = float(scanned.mean()) * wl["dim"] * 4
        self.flops = 2.0 * self.nq * float(scanned.mean()) * wl["dim"]
        # tensor path: the probed lists are scanned by the tcgen05 contraction; fp32 path: list-major FP32 tile
        self.bound = "tensor" if self.path == "tensor" else "hbm"
        self.centroids_host = ix.centroids.cpu().numpy() if hasattr(ix.centroids, "cpu") else ix.centroids
        self.assign_host = asg

    def _build_sq8(self):
        wl, t = self.wl, self.torch
        import torch.distributed as dist
        sq = self.vsk.ScalarQuantizer(self.dev, per_dim=True)
        n = self.hi - self.lo
        step = 1 << 20
        mn = mx = None
        for b in range(self.lo, self.hi, step):
            e = min(self.hi, b + step)
            x = gen_rows(t, wl, b, e, self.device)
            a, c = sq.minmax(x)
            mn = a if mn is None else t.minimum(mn, a)
            mx = c if mx is None else t.maximum(mx, c)
        if self.world > 1:
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        scale, offset = sq.set_range(mn, mx)
        self.index = self.vsk.QuantizedFlatIndex(self.dev, wl["dim"], wl["metric"], scale, offset)
        for b in range(self.lo, self.hi, step):
            e = min(self.hi, b + step)
            x = gen_rows(t, wl, b, e, self.device)
            self.index.add(sq.quantizeBatch(x))      # the fp32 source is dropped after encoding
        self.index.set_id_base(self.lo)
        self.queries = gen_queries(t, wl, self.device)
        self.sq = sq
        self.rows = None
        self.flops = 2.0 * self.nq * n * wl["dim"]
        self.bound = "tensor"

    def _build_pq(self):
        wl, t = self.wl, self.torch
        g = t.Generator(device=self.device)
        g.manual_seed(SEED + 31337)
        centres = t.randn((wl["nlist"], wl["dim"]), generator=g, dtype=t.float32, device=self.device)
        pq = self.vsk.ProductQuantizer(self.dev, wl["dim"], segments=wl["segments"], codeSize=wl["code_bits"],
                                       trainingIterations=wl["iters"])
        sample = gen_rows(t, wl, 0, wl["train_rows"], self.device, centres)     # every rank trains on the same rows
        t.cuda.synchronize()
        t0 = time.perf_counter()
        pq.train(sample)
        t.cuda.synchronize()
        t1 = time.perf_counter()
        self.index = pq.index()
        step = 1 << 20
        for b in range(self.lo, self.hi, step):
            e = min(self.hi, b + step)
            self.index.add(pq.encodeBatch(gen_rows(t, wl, b, e, self.device, centres)))
        t.cuda.synchronize()
        t2 = time.perf_counter()
        self.index.set_id_base(self.lo)
        self.queries = gen_queries(t, wl, self.device, centres)
        self.pq, self.rows, self.centres = pq, None, centres
        n = self.hi - self.lo
        self.extra = {"segments": wl["segments"], "codebook_size": 1 << wl["code_bits"], "train_s": t1 - t0,
                      "encode_rows_per_s": n / (t2 - t1), "code_bytes": n * wl["segments"]}
        # one table look-up (a 4-byte word of shared memory) and one add per (query, row, segment)
        self.flops = 1.0 * self.nq * n * wl["segments"]
        self.bytes_per_query = float(n * wl["segments"])
        self.bound = "smem"

    # ---- steps ----
    def local_search(self, queries, k):
        if self.wl["kind"] == "ivf":
            return self.index.batchSearch(queries, k)
        if self.wl["kind"] == "filtered":
            return self.index.batchSearch(queries, k, self.qmasks)
        return self.index.batchSearch(queries, k)

    def step_device(self):
        if self.abi_sharded:
            # every rank ends the step holding the merged top-k of its 1/N of the queries
            return self.index.shardedSearch(self.queries, self.k, filter_masks=self.qmasks, out=self.dev_out)
        return self.sharded.batchSearch(self.queries, self.k)

    def step_host(self):
        lib, t = self.dev._lib, self.torch
        if self.abi_sharded:
            # pinned host queries in (every rank holds them; each sends its 1/N over PCIe, NVLink does the rest),
            # this rank's slice of the merged result out to pinned host memory: one vsk_search_sharded call
            first, count = self.slice
            self.index.shardedSearch(self.q_pinned, self.k, filter_masks=self.qm_pinned, split_queries=True,
                                     out=(self.out_d_host[first:first + max(count, 1)],
                                          self.out_i_host[first:first + max(count, 1)]))
            return
        if self.world > 1 and self.qm_pinned is None:
            if not hasattr(self, "q_staging"):
                per = -(-self.nq // self.world)
                self.q_staging = t.empty((per * self.world, self.queries.shape[1]), dtype=self.queries.dtype,
                                         device=self.device)
            self.sharded.batchSearchHost(self.q_pinned, self.k, self.out_d_host, self.out_i_host, self.q_staging,
                                         gather_queries=True)
            return
        qp, od, oi = (C.c_void_p(x.data_ptr()) for x in (self.q_pinned, self.out_d_host, self.out_i_host))
        if self.wl["kind"] == "ivf":
            self.dev.check(lib.vsk_ivf_search(self.index._h, qp, self.nq, self.k, self.wl["nprobe"], od, oi))
        else:
            qm = C.c_void_p(self.qm_pinned.data_ptr()) if self.qm_pinned is not None else None
            self.dev.check(lib.vsk_search(self.index._h, qp, self.nq, self.k, qm, od, oi))
        if self.world > 1:
            from vectorstorekit_b200.sharded import ShardedSearch
            d = self.out_d_host.to(self.device, non_blocking=True)
            i = self.out_i_host.to(self.device, non_blocking=True)
            d, i = ShardedSearch(lambda qq, kk: (d, i), self.engine.mergeTopK).batchSearch(None, self.k)
            self.out_d_host.copy_(d)
            self.out_i_host.copy_(i)
            t.cuda.synchronize()

    # ---- CPU baseline on this rank's data ----
    def cpu_baseline(self, seconds_target=15.0):
        oracle, o = get_oracle()
        wl = self.wl
        cores = o.num_threads()
        q = self.queries.cpu().numpy()
        mid = oracle.METRIC_IDS[wl["metric"]]
        if wl["kind"] in ("flat", "filtered"):
            x = self.rows.cpu().numpy()
            rm = self.masks.cpu().numpy().view(np.uint64) if wl["kind"] == "filtered" else None
            qm = self.qmasks.cpu().numpy().view(np.uint64) if wl["kind"] == "filtered" else None
            fn = lambda n: o.flat_search(mid, q[:n], x, self.k, rm, qm[:n] if qm is not None else None, fast=True)
        elif wl["kind"] == "ivf":
            x = self.rows.cpu().numpy()
            fn = lambda n: o.ivf_search(q[:n], x, self.centroids_host, self.assign_host, wl["nprobe"], self.k)
        elif wl["kind"] == "pq":
            n_all = self.hi - self.lo
            n_cpu = min(n_all, 2_000_000)
            xs = gen_rows(self.torch, wl, self.lo, self.lo + n_cpu, self.device, self.centres)
            codes = self.pq.encodeBatch(xs).cpu().numpy()
            del xs
            cb = self.pq.codebooks.cpu().numpy() if hasattr(self.pq.codebooks, "cpu") else self.pq.codebooks
            fn = lambda n: o.pq_search(q[:n], codes, cb, self.k)
            v, nq, dt = cpu_rate(fn, self.nq, cores, seconds_target)
            v *= n_cpu / n_all
            return {"value": v, "unit": "queries/s", "cores": cores, "kind": "port",
                    "sample": f"{nq} of {self.nq} queries over {n_cpu} of {n_all} rows, {dt:.1f} s"
                              + (" (rate scaled by the row ratio: extrapolated)" if n_cpu < n_all else "")}
        else:
            # codes of a bounded prefix of the shard (regenerated and re-encoded on the GPU); the rate is scaled
            # by the row ratio and labelled as extrapolated
            n_all = self.hi - self.lo
            n_cpu = min(n_all, 4_000_000)
            xs = gen_rows(self.torch, wl, self.lo, self.lo + n_cpu, self.device)
            codes = self.sq.quantizeBatch(xs).cpu().numpy()
            del xs
            sc, of = self.sq.scale.cpu().numpy(), self.sq.offset.cpu().numpy()
            fn = lambda n: o.sq8_search(mid, q[:n], codes, sc, of, self.k)
            v, nq, dt = cpu_rate(fn, self.nq, cores, seconds_target)
            v *= n_cpu / n_all
            return {"value": v, "unit": "queries/s", "cores": cores, "kind": "port",
                    "sample": f"{nq} of {self.nq} queries over {n_cpu} of {n_all} rows, {dt:.1f} s"
                              + (" (rate scaled by the row ratio: extrapolated)" if n_cpu < n_all else "")}
        v, nq, dt = cpu_rate(fn, self.nq, cores, seconds_target)
        return {"value": v, "unit": "queries/s", "cores": cores, "kind": "port",
                "sample": f"{nq} of {self.nq} queries over all {self.hi - self.lo} rows, {dt:.1f} s"}


def config_of(wl, world, path):
    """The `config` object of a line: the same for this arm and for the reference arm."""
    shard_rows = wl["rows"] // max(world, 1)
    return {"workload": wl["name"], "rows": wl["rows"], "dim": wl["dim"], "queries": wl["queries"], "k": wl["k"],
            "metric": wl["metric"], "sharding": f"rows/{world}", "search_path": path,
            "l2": "the database read by every pass is larger than L2 (126 MB)"
            if shard_rows * wl["dim"] * 2 > 126e6 else "L2 flushed by the candidate-list traffic only"}


def run_reference(args, wl):
    """--impl reference: the reference's CPU search path (C++ restatement of AccelerateOptimizer /
    UnifiedDistanceComputation; its Swift sources cannot be built on Linux) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run sets OMP_NUM_THREADS=1 for its workers unless it is set: this arm is the one process that
    # works, and it is meant to use every host thread (the OpenMP runtime reads the variable when it is first loaded)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    oracle, o = get_oracle()
    n, dim, nq, k = wl["rows"], wl["dim"], wl["queries"], wl["k"]
    rng = np.random.default_rng(SEED)
    cores = o.num_threads()
    mid = oracle.METRIC_IDS[wl["metric"]]
    scale_rows = 1.0        # rate multiplier when only a prefix of the rows is searched on the CPU (extrapolation)
    note = ""
    if wl["kind"] == "flat":
        x = rng.standard_normal((n, dim), dtype=np.float32)
        q = rng.standard_normal((nq, dim), dtype=np.float32)
        if wl["metric"] == "cosine":
            x /= np.linalg.norm(x, axis=1, keepdims=True)
            q /= np.linalg.norm(q, axis=1, keepdims=True)
        fn = lambda c: o.flat_search(mid, q[:c], x, k, fast=True)
    elif wl["kind"] == "filtered":
        x = rng.random((n, dim), dtype=np.float32) * 2 - 1
        q = rng.random((nq, dim), dtype=np.float32) * 2 - 1
        rm = rng.integers(0, 2 ** 64, n, dtype=np.uint64)
        qm = np.uint64(1) << rng.integers(0, 64, nq).astype(np.uint64)
        fn = lambda c: o.flat_search(mid, q[:c], x, k, rm, qm[:c], fast=True)
    elif wl["kind"] == "ivf":
        # IVFIndex.search on the host.  Training 10 M rows on the CPU would take hours, so the index the CPU arm
        # searches has the mixture's own centres as centroids and every row filed under the centre it was drawn
        # from: lists of the same number and mean length as a trained index.  Only the search is timed.
        nlist = wl["nlist"]
        centres = rng.standard_normal((nlist, dim), dtype=np.float32)
        comp = rng.integers(0, nlist, n).astype(np.int32)
        x = np.empty((n, dim), np.float32)
        for lo in range(0, n, 1 << 20):
            hi = min(n, lo + (1 << 20))
            x[lo:hi] = centres[comp[lo:hi]] + np.float32(0.1) * rng.standard_normal((hi - lo, dim), dtype=np.float32)
        qc = rng.integers(0, nlist, nq)
        q = centres[qc] + np.float32(0.1) * rng.standard_normal((nq, dim), dtype=np.float32)
        fn = lambda c: o.ivf_search(q[:c], x, centres, comp, wl["nprobe"], k)
        note = "; lists = mixture components (training is not part of the timed search)"
    elif wl["kind"] == "sq8":
        # a bounded prefix of the rows (generating and encoding 50 M x 384 on the host alone takes minutes);
        # the rate is scaled by the row ratio and labelled as extrapolated
        n_cpu = min(n, 2_000_000)
        x = rng.standard_normal((n_cpu, dim), dtype=np.float32)
        q = rng.standard_normal((nq, dim), dtype=np.float32)
        sc, of = o.sq8_train(x, True)
        codes = o.sq8_encode(x, sc, of)
        del x
        fn = lambda c: o.sq8_search(mid, q[:c], codes, sc, of, k)
        scale_rows = n_cpu / n
        note = f"; {n_cpu} of {n} rows, rate scaled by the row ratio: extrapolated"
    else:
        print(json.dumps({"impl": "reference", "unavailable": f"no CPU arm for workload kind {wl['kind']}"}))
        return
    per_step = max(5.0, min(30.0, 120.0 / max(1, args.steps + args.warmup)))
    rates, desc = [], ""
    for s_ in range(args.warmup + args.steps):
        r, m, dt = cpu_rate(fn, nq, cores, per_step)
        desc = f"{m} of {nq} queries, {dt:.1f} s, per-query time x {nq} = the batch time (extrapolated)" + note
        if s_ >= args.warmup:
            rates.append(r * scale_rows)
    v = float(np.mean(rates))
    print(json.dumps({
        "impl": "reference", "metric": "queries/sec (k-NN, exact top-k match)", "value": v, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * nq / v,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(wl, max(1, args.gpus), args.path),
        "cpu_baseline": {"value": v, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# The default run (flat cosine, one GPU) also runs the other configurations, each as a child process of a few steps,
# and carries their figures in the same JSON line, so that one run records every configuration on the same box.
OTHER_WORKLOADS = (("c1", 50), ("c2f", 5), ("c3", 5), ("c4e", 3), ("c5", 3), ("pq", 3))   # (workload, timed steps)
OTHERS_BUDGET_S = 150.0


def run_other_workloads(args):
    import subprocess
    out, t_start = {}, time.perf_counter()
    env = {k_: v for k_, v in os.environ.items() if k_ not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")}
    for w, steps in OTHER_WORKLOADS:
        left = OTHERS_BUDGET_S - (time.perf_counter() - t_start)
        if left < 20.0:
            out[w] = {"skipped": "the time set aside for the other configurations was used up"}
            continue
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", w, "--steps", str(steps), "--warmup", "3",
               "--no-cpu-baseline", "--no-others", "--path", args.path]
        try:
            p_ = subprocess.run(cmd, capture_output=True, text=True, timeout=left, cwd=ROOT, env=env)
            d = json.loads([ln for ln in p_.stdout.splitlines() if ln.startswith("{")][-1])
            r = d.get("roofline") or {}
            o = {"workload": d["config"]["workload"], "value": d["value"], "unit": d["unit"], "ms_per_step": d["ms_per_step"],
                 "steps": d["steps"], "warmup": d["warmup"], "e2e": (d.get("e2e") or {}).get("value"),
                 "gpu_launches": d.get("gpu_launches"), "fallback_queries": (d.get("stats") or {}).get("fallback_queries"),
                 "roofline": {k_: r.get(k_) for k_ in ("bound", "achieved", "peak", "unit", "frac", "kernel_ms_per_step", "peak_source")},
                 "clocks": d.get("clocks")}
            for k_ in ("train_contraction", "train_s_per_iteration"):
                if k_ in (d.get("workload_detail") or {}):
                    o[k_] = d["workload_detail"][k_]
            out[w] = o
        except Exception as e:   # a child that fails or runs out of time never costs the main line
            out[w] = {"failed": repr(e)[:300]}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--path", default="tensor", choices=["tensor", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-others", action="store_true",
                    help="the default run (c2, one GPU) does not also run the other configurations as child processes")
    ap.add_argument("--tuning", action="append", default=[], metavar="FIELD=VALUE",
                    help="a field of the library's vsk_tuning (e.g. overlap_min_queries=0, chunk_growth=4)")
    ap.add_argument("--queries", type=int, default=0,
                    help="override the workload's batch size (a few queries show the HBM-bound regime of a scan)")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.queries > 0:
        wl["queries"] = args.queries
        wl["name"] = wl["name"] + f"-batch{args.queries}"
    if args.impl == "reference":
        return run_reference(args, wl)

    import torch
    import torch.distributed as dist
    import vectorstorekit_b200 as vsk

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    dev = vsk.CUDAComputeDevice(local)
    dev.set_search_path(vsk.PATH_TENSOR_RERANK if args.path == "tensor" else vsk.PATH_FP32_SCAN)
    if args.tuning:
        dev.set_tuning(**{kv.split("=")[0]: int(kv.split("=")[1]) for kv in args.tuning})
    engine = vsk.CUDAAccelerationEngine(dev)
    b = Bench(torch, vsk, dev, engine, wl, rank, world, device, args.path)
    nq, k = b.nq, b.k
    ext = b.stream

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        b.step_device()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    st_a = dev.stats()
    barrier()
    t0 = time.perf_counter()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    for _ in range(args.steps):
        b.step_device()
    e1.record(ext)
    barrier()
    wall = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    st_b = dev.stats()
    # second region, profiling on: an event pair around every scan launch (and, at N > 1, around every phase of the
    # sharded call).  Not part of `value`.
    prof_steps = max(1, min(args.steps, 5))
    dev.profile(True)
    b.step_device()
    st0 = dev.stats()
    phases = None
    for _ in range(prof_steps):
        b.step_device()
        if b.abi_sharded:
            ph = dev.sharded_phase_ms()
            phases = ph if phases is None else {k_: phases[k_] + v for k_, v in ph.items()}
    st1 = dev.stats()
    dev.profile(False)
    if phases is not None:
        names = list(phases)
        pt = torch.tensor([phases[n_] / prof_steps for n_ in names], dtype=torch.float64, device=device)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        phases = {n_: round(float(v), 4) for n_, v in zip(names, pt.tolist())}
    # CUDA events on the library's stream, on which the collectives of a sharded step are ordered as well;
    # the wall clock between the two barriers is reported beside it
    elapsed_ms = dev_ms
    wall_t = torch.tensor([wall * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(wall_t, op=dist.ReduceOp.MAX)
    tt = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    elapsed_ms = float(tt.item())

    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            b.step_host()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            b.step_host()
        barrier()
        e2e_s = time.perf_counter() - t0
        tt = torch.tensor([e2e_s], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e = nq * args.steps / float(tt.item())
    if rank == 0:
        sampler.stop_flag = True
        sampler.join(timeout=2)

    launches = st_b["kernel_launches"] - st_a["kernel_launches"]
    scan_ms = st1["scan_kernel_ms"] - st0["scan_kernel_ms"]
    scan_n = max(1, st1["scan_kernel_launches"] - st0["scan_kernel_launches"])
    pk = peaks()
    roof = {"bound": b.bound, "kernel": "scan kernels (distance computation + fused candidate filter)",
            "kernel_ms_per_step": scan_ms / prof_steps, "kernel_launches_per_step": scan_n / prof_steps, "traffic": None,
            "timed_steps": prof_steps}
    secs = scan_ms * 1e-3 * args.steps / prof_steps     # the formulas below are written per `args.steps` steps
    if b.bound == "tensor":
        roof.update(unit="TFLOP/s", achieved=b.flops * args.steps / secs / 1e12 if secs > 0 else None,
                    peak=pk["bf16_tflops"], peak_source=pk["source"] + " (cuBLAS bf16, sustained)")
        if wl["kind"] == "ivf":
            # second view: a contraction this short (two or three K blocks) is paced by reading its accumulators out
            # of tensor memory, 4 bytes per (query, row) pair, against the measured tcgen05.ld rate
            pairs = b.flops / (2.0 * wl["dim"])
            roof.update(tmem_readout={"unit": "TB/s", "achieved": 4.0 * pairs * args.steps / secs / 1e12 if secs > 0 else None,
                                      "peak": dev.measure_peak("tmem_read") / 1e12,
                                      "peak_source": "measured in this run: tcgen05.ld by 16 warps per SM (vsk_measure_peak)"})
            roof.update(algorithmic_query_major_gbs=b.bytes_per_query * nq * args.steps / secs / 1e9 if secs > 0 else None,
                        note="flops count the rows of the probed lists only (2 x queries x scanned rows x dim); with "
                             "d = 128 a tile's MMAs take 0.5 us and the epilogue sets the pace, so the fraction of the "
                             "tensor peak is low by construction; query-major bytes (each query reading its probed "
                             "lists once) are given for the HBM view")
    elif b.bound == "hbm":
        roof.update(unit="GB/s", achieved=b.bytes_per_query * nq * args.steps / secs / 1e9 if secs > 0 else None,
                    peak=pk["hbm_gbs"], peak_source=pk["source"] + " (copy)",
                    note="algorithmic bytes are query-major (each query reads its probed lists once); the list-major "
                         "kernel reuses a list across the queries that probe it, so achieved may exceed peak")
    elif b.bound == "smem":
        sm = dev.info()["sm_count"]
        roof.update(unit="T look-ups/s", achieved=b.flops * args.steps / secs / 1e12 if secs > 0 else None,
                    peak=dev.measure_peak("smem_gather") / 1e12,
                    peak_source="measured in this run: 4-byte shared-memory loads at random addresses (vsk_measure_peak)",
                    nominal_peak=sm * 32 * 1.965e9 / 1e12,
                    algorithmic_codes_gbs=b.bytes_per_query * nq * args.steps / secs / 1e9 if secs > 0 else None,
                    note="one 4-byte table word per (query, row, segment); query-major code bytes are given for "
                         "the HBM view: a query tile re-reads the codes from L2")
    else:
        sm = dev.info()["sm_count"]
        roof.update(unit="T lane-instr/s", achieved=b.flops * args.steps / secs / 1e12 if secs > 0 else None,
                    peak=dev.measure_peak("fp32_issue") / 1e12,
                    peak_source="measured in this run: FADD/FFMA chains on every warp slot (vsk_measure_peak)",
                    nominal_peak=sm * 128 * 1.965e9 / 1e12)
    roof["frac"] = roof["achieved"] / roof["peak"] if roof.get("achieved") else None
    if args.queries > 0 and wl["kind"] in ("flat", "sq8", "filtered") and secs > 0:
        # the HBM view of the same launches: the stored operand the scan reads (fp16 images on the tensor path, else
        # fp32 rows or int8 codes) crossing HBM once per batch; this is what bounds a batch of a few queries
        if args.path == "tensor" and b.bound == "tensor":
            per_row = (wl["dim"] + 63) // 64 * 64 * 2
        else:
            per_row = wl["dim"] * (1 if wl["kind"] == "sq8" else 4)
            if wl["kind"] == "filtered":
                # every row's 8-byte mask, and the rows some query of the batch may see: half of them under one
                # one-hot mask, 1 - 2^-g of them under g distinct ones
                distinct = len(set(b.qmasks.cpu().tolist())) if b.qmasks is not None else 64
                per_row = per_row * (1.0 - 0.5 ** min(distinct, 64)) + 8
        gbs = (b.hi - b.lo) * per_row * args.steps / secs / 1e9
        roof["hbm_view"] = {"bytes_per_row": per_row, "achieved_gbs": gbs, "peak_gbs": pk["hbm_gbs"],
                            "frac": gbs / pk["hbm_gbs"]}
    if wl["kind"] == "flat" and args.path == "tensor" and b.bound == "tensor":
        # DRAM bytes per scan launch, from the ncu capture of the reduced workload c2s:
        # dram__bytes_read equals the fp16 rows of the launch read once plus the query operand, dram__bytes_write is
        # the appended keys (about 6 MB); scaled to this workload by its rows (traffic grows in proportion)
        d16 = (wl["dim"] + 63) // 64 * 64
        per_step = (b.hi - b.lo) * d16 * 2 + (scan_n / prof_steps) * (nq * d16 * 2 + 6.0e6)
        roof["traffic"] = per_step / (scan_n / prof_steps)
        roof["traffic_source"] = "ncu capture of workload c2s, scaled by rows"

    line = {
        "metric": "queries/sec (k-NN, exact top-k match)", "value": nq * args.steps / (elapsed_ms * 1e-3),
        "unit": "queries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "wall_ms_per_step": float(wall_t.item()) / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("f16 operands, f32 accumulate, f32 rerank" if args.path == "tensor" and b.bound == "tensor" else "f32"),
        "data": "synthetic",
        "config": config_of(wl, world, args.path),
        "workload_detail": b.extra,
        "tuning": dev.tuning(),
        "roofline": roof,
        # host -> device bytes of the whole job per step: at N > 1 each rank sends its 1/N of the queries
        "e2e": {"value": e2e, "unit": "queries/s", "h2d_bytes_per_step": nq * wl["dim"] * 4 + (nq * 8 if b.qmasks is not None else 0),
                "d2h_bytes_per_step": nq * k * 12},
        "gpu_launches": int(launches),
        "stats": {"fallback_queries": st_b["fallback_queries"] - st_a["fallback_queries"],
                  "reranked_rows": st_b["reranked_rows"] - st_a["reranked_rows"],
                  "tensor_tiles": st_b["tensor_tiles"] - st_a["tensor_tiles"]},
    }
    if phases is not None:
        line["phases_ms"] = dict(phases, note="one sharded call with profiling on (one stream), max over ranks")
    if world > 1:
        line["result_layout"] = ("every rank holds the merged top-k of its 1/N of the queries"
                                 if b.abi_sharded else "every rank holds all results")
    if rank == 0:
        line["clocks"] = sampler.summary()
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = b.cpu_baseline()
        if (world == 1 and args.workload == "c2" and not args.no_others and not args.no_cpu_baseline and not args.no_e2e
                and not args.tuning and args.queries == 0):
            line["other_workloads"] = run_other_workloads(args)
        print(json.dumps(line), flush=True)
    # release the library's objects in order (the context closes the indices created on it first); left to the
    # interpreter's shutdown, finalisers of the Bench object's reference cycle run in no particular order
    torch.cuda.synchronize()
    dev.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
