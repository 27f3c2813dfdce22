"""The N > 1 path on CPU: two gloo ranks, each searching its row shard (with the CPU oracle standing in
for the GPU search), all-gather, merge — must equal the unsharded search exactly."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from vectorstorekit_b200.sharded import ShardedSearch, shard_range
    o = oracle.CpuOracle()
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1001, 24)).astype(np.float32)       # odd size: uneven shards
    q = rng.standard_normal((17, 24)).astype(np.float32)
    x[700] = x[3]                                                 # a cross-shard exact tie
    lo, hi = shard_range(len(x), rank, world)

    def local(queries, k):
        d, i = o.flat_search(oracle.EUCLIDEAN, queries.numpy(), x[lo:hi], k)
        return torch.from_numpy(d), torch.from_numpy(np.where(i >= 0, i + lo, -1))

    def merge(gd, gi):
        d, i = o.merge_topk(gd.numpy(), gi.numpy())
        return torch.from_numpy(d), torch.from_numpy(i)

    s = ShardedSearch(local, merge)
    d, i = s.batchSearch(torch.from_numpy(q), 9)
    rd, ri = o.flat_search(oracle.EUCLIDEAN, q, x, 9)
    ok = np.array_equal(i.numpy(), ri) and np.array_equal(d.numpy(), rd)
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_search_equals_unsharded():
    from vectorstorekit_b200.sharded import shard_range
    assert [shard_range(10, r, 3) for r in range(3)] == [(0, 3), (3, 6), (6, 10)]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert ret.get(0) is True and ret.get(1) is True
