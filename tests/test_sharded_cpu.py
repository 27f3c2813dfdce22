"""The N > 1 path on CPU: gloo ranks, each searching its row shard (with the CPU oracle standing in for the GPU
search), the bound all-reduce, the all-to-all of the per-shard lists, the sliced merge and the all-gather — must
equal the unsharded search exactly."""
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

    # the two halves of the local search: `begin` reports the ceil(k / shards)-th best local distance, `finish`
    # drops what lies above the maximum of those over the ranks (and counts what it kept)
    state = {}

    def begin(queries, k, shards):
        d, i = local(queries, k)
        state["res"] = (d, i)
        j = -(-k // shards)
        return d[:, j - 1].clone()

    def finish(bound):
        d, i = state.pop("res")
        keep = d <= bound[:, None]
        state["kept"] = int(keep.sum())
        return torch.where(keep, d, torch.full_like(d, float("inf"))), torch.where(keep, i, torch.full_like(i, -1))

    rd, ri = o.flat_search(oracle.EUCLIDEAN, q, x, 9)
    ok = True
    for s in (ShardedSearch(local, merge), ShardedSearch(local, merge, local_begin=begin, local_finish=finish),
              ShardedSearch(local, merge, local_begin=begin, local_finish=finish, max_queries=5)):
        d, i = s.batchSearch(torch.from_numpy(q), 9)
        ok = ok and np.array_equal(i.numpy(), ri) and np.array_equal(d.numpy(), rd)
    ok = ok and state["kept"] < 2 * 9          # the bound dropped rows (last batch: 2 queries of 9)
    # host buffers in, host buffers out
    hd, hi_ = torch.empty((17, 9), dtype=torch.float32), torch.empty((17, 9), dtype=torch.int64)
    ShardedSearch(local, merge).batchSearchHost(torch.from_numpy(q), 9, hd, hi_)
    ok = ok and np.array_equal(hi_.numpy(), ri) and np.array_equal(hd.numpy(), rd)
    # ... with every rank sending only its share of the queries to the "device" (17 queries: uneven shares)
    per = -(-17 // world)
    stage = torch.full((per * world, 24), float("nan"))
    hd.fill_(0), hi_.fill_(0)
    ShardedSearch(local, merge).batchSearchHost(torch.from_numpy(q), 9, hd, hi_, staging=stage, gather_queries=True)
    ok = ok and np.array_equal(hi_.numpy(), ri) and np.array_equal(hd.numpy(), rd)
    ok = ok and np.array_equal(stage[:17].numpy(), q)
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_search_equals_unsharded(world):
    from vectorstorekit_b200.sharded import shard_range
    assert [shard_range(10, r, 3) for r in range(3)] == [(0, 3), (3, 6), (6, 10)]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29600 + os.getpid() % 300 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert all(ret.get(r) is True for r in range(world))


def _kmeans_worker(rank, world, port, ret):
    """Sharded Lloyd iterations on CPU ranks: numpy stands in for the device step; the result must equal the CPU
    oracle's k-means on the unsharded rows (up to the order of the fp32 sums)."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from vectorstorekit_b200.sharded import ShardedKMeans, shard_range
    o = oracle.CpuOracle()
    rng = np.random.default_rng(11)
    k, d = 7, 6
    centres = rng.standard_normal((k, d)).astype(np.float32) * 3
    x = (centres[rng.integers(0, k - 1, 901)] + 0.3 * rng.standard_normal((901, d))).astype(np.float32)
    init = np.concatenate([x[:k - 1], np.full((1, d), 50.0, np.float32)])     # the last centroid attracts no row
    lo, hi = shard_range(len(x), rank, world)
    mine = x[lo:hi]

    def step(cent):
        c = cent.numpy()
        asg, dist_ = o.assign(mine, c)
        sums = np.zeros((k, d), np.float32)
        np.add.at(sums, asg, mine)
        counts = np.bincount(asg, minlength=k).astype(np.float32)
        return torch.from_numpy(sums), torch.from_numpy(counts), torch.tensor([dist_.sum()], dtype=torch.float32)

    def finish(sums, counts, cent):
        s, c, old = sums.numpy(), counts.numpy(), cent.numpy()
        out = np.where(c[:, None] > 0, s / np.maximum(c, 1)[:, None], old).astype(np.float32)
        return torch.from_numpy(out)

    cent, iters, inertia = ShardedKMeans(step, finish).cluster(torch.from_numpy(init), 5, -1.0)
    rc, ra, rin, rit = o.kmeans(x, init, 5)
    ok = iters == rit == 5 and np.allclose(cent.numpy(), rc, rtol=1e-4, atol=1e-5) and abs(inertia - rin) <= 1e-3 * abs(rin)
    ok = ok and np.array_equal(cent.numpy()[k - 1], init[k - 1])             # the empty cluster kept its centroid
    gathered = [torch.zeros_like(cent) for _ in range(world)]
    dist.all_gather(gathered, cent)
    ok = ok and all(torch.equal(g, cent) for g in gathered)                   # every rank holds the same centroids
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_kmeans_equals_unsharded():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_kmeans_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert ret.get(0) is True and ret.get(1) is True


def _leaving_worker(rank, world, port, ret):
    """Three ranks run sharded searches; after the first step rank 2 leaves (between steps: none of its collectives is
    in flight).  The others must get an error from their next exchange within the group's timeout instead of waiting
    for ever, and the failed call must leave them able to report it."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    import oracle
    from vectorstorekit_b200.sharded import ShardedSearch, shard_range
    o = oracle.CpuOracle()
    rng = np.random.default_rng(8)
    x = rng.standard_normal((600, 8)).astype(np.float32)
    q = rng.standard_normal((9, 8)).astype(np.float32)
    lo, hi = shard_range(len(x), rank, world)

    def local(queries, k):
        d, i = o.flat_search(oracle.EUCLIDEAN, queries.numpy(), x[lo:hi], k)
        return torch.from_numpy(d), torch.from_numpy(np.where(i >= 0, i + lo, -1))

    def merge(gd, gi):
        d, i = o.merge_topk(gd.numpy(), gi.numpy())
        return torch.from_numpy(d), torch.from_numpy(i)

    s = ShardedSearch(local, merge)
    d, i = s.batchSearch(torch.from_numpy(q), 4)          # step 1: everybody is here
    rd, ri = o.flat_search(oracle.EUCLIDEAN, q, x, 4)
    first_ok = np.array_equal(i.numpy(), ri)
    if rank == world - 1:
        ret[rank] = ("left", first_ok)
        os._exit(0)                                       # leaves without a word; the host-side failure of the test
    t0 = time.time()
    try:
        s.batchSearch(torch.from_numpy(q), 4)             # step 2: one rank is gone
        ret[rank] = ("no error", first_ok, time.time() - t0)
    except Exception as e:                                # gloo: connection closed by peer / timed out
        ret[rank] = ("error", first_ok, time.time() - t0, type(e).__name__)
    os._exit(0)                                           # the group is broken: no barrier, no clean shutdown


def test_a_rank_that_leaves_between_steps_fails_the_others_quickly():
    world = 3
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank was still blocked after 90 s")
    assert ret.get(world - 1) == ("left", True)
    for r in range(world - 1):
        state = ret.get(r)
        assert state is not None and state[0] == "error" and state[1] is True, state
        assert state[2] < 60, state
