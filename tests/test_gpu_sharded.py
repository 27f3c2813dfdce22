"""The row-sharded search behind the C ABI (vsk_comm_init / vsk_search_sharded).

One GPU: a communicator of one rank must return exactly what the plain search returns, in every layout and through
both the host-pointer and the device-pointer form.  Two or more GPUs (skipped on a one-GPU box): one child process per
GPU, each holding a row shard, joined through vsk_comm_unique_id / vsk_comm_init; the merged result must equal the CPU
oracle's search over the whole database (ties by global row), for fp32 cosine / euclidean, a filtered batch, an int8
index and an IVF index (vsk_ivf_search_sharded: every shard holds a slice of every list), with slice and gathered
layouts, uneven query slices and a batch large enough for the two-lane schedule.
"""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


def test_one_rank_communicator_equals_plain_search(vsk, cpu_oracle):
    import torch
    dev = vsk.CUDAComputeDevice(0)
    try:
        dev.comm_init(1, 0, None)
        assert dev.comm_info() == (1, 0)
        rng = np.random.default_rng(3)
        x = rng.standard_normal((30_000, 96)).astype(np.float32)
        q = rng.standard_normal((333, 96)).astype(np.float32)
        ix = vsk.FlatIndex(dev, 96, "cosine")
        ix.add(x)
        pd, pi = ix.batchSearch(q, 12)
        for gather in (False, True):
            sd, si = ix.shardedSearch(q, 12, gather=gather)
            assert np.array_equal(si, pi) and np.array_equal(sd, pd)
            dd, di = ix.shardedSearch(torch.as_tensor(q, device="cuda"), 12, gather=gather)
            assert np.array_equal(di.cpu().numpy(), pi) and np.array_equal(dd.cpu().numpy(), pd)
        rd, ri = cpu_oracle.flat_search(oracle.COSINE, q, x, 12)
        assert_topk_parity(pd, pi, rd, ri)
        ix.close()
        # an IVF index through vsk_ivf_search_sharded
        iv = vsk.IVFIndex(dev, 96, numberOfCentroids=64, numberOfProbes=8, maxIterations=2, tolerance=-1.0)
        iv.train(x, x[:64].copy())
        iv.insert(x)
        pd, pi = iv.batchSearch(q, 12)
        for gather in (False, True):
            sd, si = iv.shardedSearch(q, 12, gather=gather)
            assert np.array_equal(si, pi) and np.array_equal(sd, pd)
            dd, di = iv.shardedSearch(torch.as_tensor(q, device="cuda"), 12, gather=gather)
            assert np.array_equal(di.cpu().numpy(), pi) and np.array_equal(dd.cpu().numpy(), pd)
        iv.close()
        # ... and with row masks and per-query filter masks
        rng = np.random.default_rng(11)
        rm = (np.uint64(1) << rng.integers(0, 4, x.shape[0]).astype(np.uint64))
        qm = (np.uint64(1) << rng.integers(0, 4, q.shape[0]).astype(np.uint64)) | np.uint64(8)
        iv = vsk.IVFIndex(dev, 96, numberOfCentroids=64, numberOfProbes=8, maxIterations=2, tolerance=-1.0)
        iv.train(x, x[:64].copy())
        iv.insert(x, rm)
        pd, pi = iv.batchSearch(q, 12, filter_masks=qm)
        sd, si = iv.shardedSearch(q, 12, filter_masks=qm, gather=True)
        assert np.array_equal(si, pi) and np.array_equal(sd, pd)
        ok = pi >= 0
        assert ok.any() and np.all((rm[pi[ok]] & np.broadcast_to(qm[:, None], pi.shape)[ok]) != 0)
        iv.close()
        dev.comm_destroy()
        assert dev.comm_info() == (1, 0)
    finally:
        dev.close()


CHILD = textwrap.dedent("""
    import os, sys, json, time
    import numpy as np
    sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
    rank, world, idfile, outdir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    import torch
    torch.cuda.set_device(rank)
    import vectorstorekit_b200 as vsk
    from vectorstorekit_b200.engine import sharded_slice
    dev = vsk.CUDAComputeDevice(rank)
    if rank == 0:
        uid = dev.comm_unique_id()
        with open(idfile + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(idfile + ".tmp", idfile)
    else:
        t0 = time.time()
        while not os.path.exists(idfile):
            if time.time() - t0 > 120:
                raise SystemExit("no communicator id")
            time.sleep(0.05)
        uid = open(idfile, "rb").read()
    dev.comm_init(world, rank, uid)
    assert dev.comm_info() == (world, rank)
    results = {}

    def shard(n):
        return rank * n // world, (rank + 1) * n // world

    cases = json.loads(%(cases)r)
    for name, c in cases.items():
        rng = np.random.default_rng(c["seed"])
        n, d, nq, k = c["n"], c["d"], c["nq"], c["k"]
        x = rng.standard_normal((n, d)).astype(np.float32)
        if c.get("dups"):
            x[n // 2:n // 2 + 500] = x[:500]          # equal rows in different shards: ties broken by global row
        q = rng.standard_normal((nq, d)).astype(np.float32)
        lo, hi = shard(n)
        masks = qm = None
        if c.get("masked"):
            masks = rng.integers(0, 2 ** 63, n, dtype=np.uint64)
            qm = (np.uint64(1) << rng.integers(0, 63, nq).astype(np.uint64))
        if c["kind"] == "ivf":
            # every rank trains on the same rows from the same start (the update is deterministic: same centroids
            # everywhere), then files only its own shard: a slice of every list
            ix = vsk.IVFIndex(dev, d, numberOfCentroids=c["nlist"], numberOfProbes=c["nprobe"], maxIterations=3, tolerance=-1.0)
            ix.train(x, x[:c["nlist"]].copy())
            ix.insert(x[lo:hi])
            np.savez(os.path.join(outdir, name + f"_rank{rank}.npz"), assign=ix.assignments(), centroids=ix.centroids)
        elif c["kind"] == "sq8":
            mn, mx = x.min(0), x.max(0)
            sq = vsk.ScalarQuantizer(dev, per_dim=True)
            scale, offset = sq.set_range(torch.as_tensor(mn, device="cuda"), torch.as_tensor(mx, device="cuda"))
            ix = vsk.QuantizedFlatIndex(dev, d, c["metric"], scale, offset)
            ix.add(sq.quantizeBatch(torch.as_tensor(x[lo:hi], device="cuda")))
        else:
            ix = vsk.FlatIndex(dev, d, c["metric"])
            ix.add(x[lo:hi], masks[lo:hi] if masks is not None else None)
        ix.set_id_base(lo)
        first, count = sharded_slice(nq, world, rank)
        # device form, slice layout
        qd = torch.as_tensor(q, device="cuda")
        qmd = torch.as_tensor(qm.view(np.int64), device="cuda") if qm is not None else None
        sd, si = ix.shardedSearch(qd, k, filter_masks=qmd)
        assert sd.shape[0] == count
        # host form, gathered layout, queries split over the ranks' PCIe links
        gd, gi = ix.shardedSearch(q, k, filter_masks=qm, gather=True, split_queries=True)
        assert np.array_equal(gi[first:first + count], si.cpu().numpy())
        assert np.array_equal(gd[first:first + count], sd.cpu().numpy())
        if rank == 0:
            np.savez(os.path.join(outdir, name + ".npz"), d=gd, i=gi)
        ix.close()
    st = dev.stats()
    assert st["tensor_tiles"] > 0
    dev.comm_destroy()
    dev.close()
    print("rank", rank, "ok")
""")

CASES = {
    "cosine": dict(kind="flat", metric="cosine", n=60_001, d=128, nq=1003, k=20, seed=1),
    "euclid_two_lanes": dict(kind="flat", metric="euclidean", n=40_000, d=96, nq=4100, k=10, seed=2, dups=True),
    "masked_dot": dict(kind="flat", metric="dotProduct", n=50_000, d=200, nq=600, k=16, seed=3, masked=True),
    "manhattan": dict(kind="flat", metric="manhattan", n=20_000, d=64, nq=130, k=8, seed=4),
    "int8_dot": dict(kind="sq8", metric="dotProduct", n=80_000, d=96, nq=700, k=10, seed=5),
    "ivf_euclid": dict(kind="ivf", metric="euclidean", n=60_000, d=64, nq=900, k=10, seed=6, nlist=96, nprobe=12),
}


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_search_over_ranks_equals_unsharded_oracle(cpu_oracle, tmp_path, world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import json
    idfile = str(tmp_path / "comm_id")
    code = CHILD % dict(root=ROOT, cases=json.dumps(CASES))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", code, str(r), str(world), idfile, str(tmp_path)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(world)]
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=600))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r}: {se[-3000:]}"
    for name, c in CASES.items():
        rng = np.random.default_rng(c["seed"])
        n, d, nq, k = c["n"], c["d"], c["nq"], c["k"]
        x = rng.standard_normal((n, d)).astype(np.float32)
        if c.get("dups"):
            x[n // 2:n // 2 + 500] = x[:500]
        q = rng.standard_normal((nq, d)).astype(np.float32)
        masks = qm = None
        if c.get("masked"):
            masks = rng.integers(0, 2 ** 63, n, dtype=np.uint64)
            qm = (np.uint64(1) << rng.integers(0, 63, nq).astype(np.uint64))
        got = np.load(tmp_path / (name + ".npz"))
        mid = oracle.METRIC_IDS[c["metric"]]
        if c["kind"] == "ivf":
            # shared state, as in the single-GPU IVF tests: the GPU-trained centroids and the shards' list membership
            parts = [np.load(tmp_path / f"{name}_rank{r}.npz") for r in range(world)]
            for part in parts[1:]:
                assert np.array_equal(part["centroids"], parts[0]["centroids"])     # same centroids on every rank
            asg = np.concatenate([part["assign"] for part in parts])
            rd, ri = cpu_oracle.ivf_search(q, x, parts[0]["centroids"], asg, c["nprobe"], k)
        elif c["kind"] == "sq8":
            scale = (np.float32(255.0) / (x.max(0) - x.min(0))).astype(np.float32)
            offset = (-x.min(0) * scale - np.float32(128.0)).astype(np.float32)
            codes = cpu_oracle.sq8_encode(x, scale, offset)
            rd, ri = cpu_oracle.sq8_search(mid, q, codes, scale, offset, k)
        else:
            rd, ri = cpu_oracle.flat_search(mid, q, x, k, masks, qm)
        assert_topk_parity(got["d"], got["i"], rd, ri)
        if c.get("dups"):
            # queries that hit a duplicated pair see both copies at equal distance: the lower global row comes first
            eq = got["d"][:, :-1] == got["d"][:, 1:]
            assert np.all(got["i"][:, :-1][eq] < got["i"][:, 1:][eq])
