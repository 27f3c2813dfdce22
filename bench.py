"""Benchmark of the batch similarity-search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

Metric: queries/sec of exact top-k search (BASELINE.json).  At N = 1 the default workload is the
configuration the metric is quoted on: flat cosine, 1 000 000 x 768 fp32 rows (N(0,1), L2-normalised),
10 000 queries, k = 100.  A step is one batch search of all queries over the resident database.
With N > 1 (one process per GPU under torchrun) the rows are sharded across ranks, each rank
searches its shard, the per-shard top-k lists are all-gathered over NCCL and merged.

value   queries/s with queries already in HBM (CUDA events, max over ranks)
e2e     queries/s through the host-pointer C-ABI call: pinned host queries in, results out
roofline / cpu_baseline: see DESIGN.md
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (metric, rows, dim, queries, k, description)
    "c1": ("euclidean", 100_000, 128, 1_000, 10, "flat-euclidean-100k-d128-q1000-k10"),
    "c2": ("cosine", 1_000_000, 768, 10_000, 100, "flat-cosine-1M-d768-q10000-k100"),
    # reduced copy of c2 for profiler captures: database still larger than L2, under 1 GB on the device
    "c2s": ("cosine", 200_000, 768, 2_048, 100, "flat-cosine-200k-d768-q2048-k100"),
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
            time.sleep(0.1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(self.samples[0][1]) if self.samples[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.samples)}


def gen_rows(torch, n, dim, seed, device, normalise):
    """Seeded N(0,1) rows generated on the GPU, optionally L2-normalised (x_i / |x|, fp32)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.empty((n, dim), dtype=torch.float32, device=device)
    step = 1 << 18
    for b in range(0, n, step):
        e = min(n, b + step)
        t = torch.randn((e - b, dim), generator=g, dtype=torch.float32, device=device)
        if normalise:
            t = t / t.norm(dim=1, keepdim=True)
        out[b:e] = t
    return out


def cpu_search_rate(metric_id, q_host, x_host, k, seconds_target=15.0, nthreads=0):
    """Times the CPU restatement of the reference's search on a bounded query sample of the same
    workload (full database).  Returns (queries/s, cores, description)."""
    import oracle
    try:
        oracle.build(native=True)
        o = oracle.CpuOracle(native=True)
    except Exception:
        o = oracle.CpuOracle()
    cores = o.num_threads() if nthreads == 0 else nthreads
    n0 = min(len(q_host), max(cores, 4))
    t0 = time.perf_counter()
    o.flat_search(metric_id, q_host[:n0], x_host, k, fast=True, nthreads=nthreads)
    dt = time.perf_counter() - t0
    nq = int(min(len(q_host), max(n0, seconds_target / max(dt / n0, 1e-9))))
    nq = max(cores, (nq // cores) * cores)
    t0 = time.perf_counter()
    o.flat_search(metric_id, q_host[:nq], x_host, k, fast=True, nthreads=nthreads)
    dt = time.perf_counter() - t0
    return nq / dt, cores, f"{nq} of {len(q_host)} queries over all {len(x_host)} rows, {dt:.1f} s"


def run_reference(args, wl):
    """--impl reference: the reference's CPU search path (C++ restatement of AccelerateOptimizer /
    UnifiedDistanceComputation; its Swift sources cannot be built on Linux) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    metric, n, dim, nq, k, name = wl
    import oracle
    rng = np.random.default_rng(20261125)
    x = rng.standard_normal((n, dim), dtype=np.float32)
    q = rng.standard_normal((nq, dim), dtype=np.float32)
    if metric == "cosine":
        x /= np.linalg.norm(x, axis=1, keepdims=True)
        q /= np.linalg.norm(q, axis=1, keepdims=True)
    mid = oracle.METRIC_IDS[{"euclidean": "euclidean", "cosine": "cosine"}[metric]]
    per_step = max(5.0, min(30.0, 120.0 / max(1, args.steps + args.warmup)))
    rates = []
    desc = ""
    cores = 1
    for s in range(args.warmup + args.steps):
        r, cores, desc = cpu_search_rate(mid, q, x, k, seconds_target=per_step)
        if s >= args.warmup:
            rates.append(r)
    v = float(np.mean(rates))
    print(json.dumps({
        "impl": "reference", "metric": "queries/sec (k-NN, exact top-k match)", "value": v, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * nq / v,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "rows": n, "dim": dim, "queries": nq, "k": k, "metric": metric},
        "cpu_baseline": {"value": v, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--path", default="tensor", choices=["tensor", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args, wl)

    import torch
    import torch.distributed as dist
    import vectorstorekit_b200 as vsk

    metric, n_total, dim, nq, k, name = wl
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    dev = vsk.CUDAComputeDevice(local)
    dev.set_search_path(vsk.PATH_TENSOR_RERANK if args.path == "tensor" else vsk.PATH_FP32_SCAN)
    engine = vsk.CUDAAccelerationEngine(dev)

    # rows [lo, hi) of the global database live on this rank
    lo, hi = rank * n_total // world, (rank + 1) * n_total // world
    seed = 20261125 * 10 + 2
    # every rank generates the full query set (replicated) and only its rows: the generator is
    # advanced shard by shard so that the union over ranks is the same database at every world size
    shard_rows = []
    for r in range(world):
        rl, rh = r * n_total // world, (r + 1) * n_total // world
        if r == rank:
            shard_rows = gen_rows(torch, rh - rl, dim, seed + 100 + rl, device, metric == "cosine")
    queries = gen_rows(torch, nq, dim, seed + 1000, device, metric == "cosine")
    index = vsk.FlatIndex(dev, dim, metric)
    index.add(shard_rows)
    index.set_id_base(lo)
    q_pinned = queries.cpu().pin_memory()
    out_d_host = torch.empty((nq, k), dtype=torch.float32).pin_memory()
    out_i_host = torch.empty((nq, k), dtype=torch.int64).pin_memory()
    ext = torch.cuda.ExternalStream(dev.stream, device=device)

    from vectorstorekit_b200.sharded import ShardedSearch
    sharded = ShardedSearch(lambda qq, kk: index.batchSearch(qq, kk), engine.mergeTopK)

    def step_device():
        return sharded.batchSearch(queries, k)

    def step_host():
        import ctypes as C
        lib = dev._lib
        dev.check(lib.vsk_search(index._h, C.c_void_p(q_pinned.data_ptr()), nq, k, None,
                                 C.c_void_p(out_d_host.data_ptr()), C.c_void_p(out_i_host.data_ptr())))
        if world > 1:
            d = out_d_host.to(device, non_blocking=True)
            i = out_i_host.to(device, non_blocking=True)
            d, i = ShardedSearch(lambda qq, kk: (d, i), engine.mergeTopK).batchSearch(None, k)
            out_d_host.copy_(d)
            out_i_host.copy_(i)
            torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_device()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dev.profile(True)
    st0 = dev.stats()
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(ext):
        e0 = torch.cuda.Event(enable_timing=True)
        e0.record(ext)
    for _ in range(args.steps):
        d_last, i_last = step_device()
    with torch.cuda.stream(ext):
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record(ext)
    barrier()
    wall = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    st1 = dev.stats()
    dev.profile(False)
    # multi-GPU: the all-gather runs on torch's stream, so the step time is the wall clock between the
    # two barriers (both sides synchronised); single GPU: CUDA events on the library's stream
    elapsed_ms = dev_ms if world == 1 else wall * 1e3
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())

    # end to end through the host-pointer call
    for _ in range(2):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    barrier()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    if rank == 0:
        sampler.stop_flag = True
        sampler.join(timeout=2)

    launches = st1["kernel_launches"] - st0["kernel_launches"]
    scan_ms = st1["scan_kernel_ms"] - st0["scan_kernel_ms"]
    scan_n = max(1, st1["scan_kernel_launches"] - st0["scan_kernel_launches"])
    pk = peaks()
    n_local = hi - lo
    flops_step = 2.0 * nq * n_local * dim      # algorithmic flops of one batch on this rank
    roof = {
        "bound": "tensor", "unit": "TFLOP/s",
        "achieved": flops_step * args.steps / (scan_ms * 1e-3) / 1e12 if scan_ms > 0 else None,
        "peak": pk["bf16_tflops"], "peak_source": pk["source"] + " (cuBLAS bf16, sustained)",
        "kernel": "scan kernels (contraction + fused candidate filter)",
        "kernel_ms_per_step": scan_ms / args.steps, "kernel_launches_per_step": scan_n / args.steps,
        "traffic": None,
    }
    roof["frac"] = roof["achieved"] / roof["peak"] if roof["achieved"] else None

    line = {
        "metric": "queries/sec (k-NN, exact top-k match)", "value": nq * args.steps / (elapsed_ms * 1e-3),
        "unit": "queries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 operands, f32 accumulate, f32 rerank" if args.path == "tensor" else "f32", "data": "synthetic",
        "config": {"workload": name, "rows": n_total, "dim": dim, "queries": nq, "k": k, "metric": metric,
                   "sharding": f"rows/{world}", "search_path": args.path,
                   "l2": "database (>= 1.5 GB per pass) is larger than L2"},
        "roofline": roof,
        "e2e": {"value": nq * args.steps / e2e_s, "unit": "queries/s", "h2d_bytes_per_step": nq * dim * 4,
                "d2h_bytes_per_step": nq * k * 12},
        "gpu_launches": int(launches),
        "stats": {"fallback_queries": st1["fallback_queries"] - st0["fallback_queries"],
                  "reranked_rows": st1["reranked_rows"] - st0["reranked_rows"],
                  "tensor_tiles": st1["tensor_tiles"] - st0["tensor_tiles"]},
    }
    if rank == 0:
        line["clocks"] = sampler.summary()
        if world == 1 and not args.no_cpu_baseline:
            import oracle
            v, cores, desc = cpu_search_rate(oracle.METRIC_IDS[metric], queries.cpu().numpy(), shard_rows.cpu().numpy(), k)
            line["cpu_baseline"] = {"value": v, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line))
    index.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
