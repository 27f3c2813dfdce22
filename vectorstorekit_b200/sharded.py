"""Row-sharded search over the ranks of a ``torch.distributed`` group (one process per GPU).

Rank g holds rows ``[g*N/G, (g+1)*N/G)`` of the database and answers every query on its shard.  Two exchanges
make the shards' answers into the result an unsharded search would return (ties by global id):

* half-way through the local search every rank knows a value that its ``ceil(k/G)`` best rows do not exceed; the
  element-wise maximum over the ranks (one small all-reduce) is a value that at least k rows of the whole database
  do not exceed, and the second half of the local search keeps only rows at or below it — about ``k/G`` per rank
  instead of k, which is what makes the per-query work after the scan shrink with the shard;
* the per-rank ``[Q, k]`` (distance, global id) lists are exchanged with an all-to-all so that rank g receives every
  rank's lists for ITS slice of the queries, merges that slice, and an all-gather hands every rank the whole result.

The reference has no sharded search; this is the multi-GPU form of ``batchSearch``.

The local search, its two halves and the merge are injected, so that the exchange logic can be exercised on CPU
ranks (``gloo``) in tests; on GPUs they are ``FlatIndex.batchSearch``, ``FlatIndex.shardSearchBegin`` /
``shardSearchFinish`` and ``CUDAAccelerationEngine.mergeTopK``.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Optional, Tuple


def join_communicator(dev, group=None):
    """Joins `dev` (a ``CUDAComputeDevice``) to a communicator over the ranks of a ``torch.distributed`` group: rank 0
    makes the id (``vsk_comm_unique_id``), the group broadcasts the 128 bytes, every rank calls ``vsk_comm_init``.
    After this, ``FlatIndex.shardedSearch`` / ``QuantizedFlatIndex.shardedSearch`` (``vsk_search_sharded``) do the
    whole sharded search inside the library - scan, bound all-reduce, one all-to-all of packed keys, merge - and
    this module's ``ShardedSearch`` is needed only for index kinds without that entry point and for CPU tests."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    box = [dev.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    dev.comm_init(world, rank, box[0])
    return world, rank


def shard_range(n_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank `rank`; the union over ranks is [0, n_total) with no overlap."""
    return rank * n_total // world, (rank + 1) * n_total // world


class ShardedSearch:
    def __init__(self, local_search: Callable, merge: Callable, group=None, local_begin: Optional[Callable] = None,
                 local_finish: Optional[Callable] = None, stream=None, max_queries: int = 16384):
        """local_search(queries, k) -> (dist [Q,k], ids [Q,k]) with GLOBAL ids (set the index's id base to
        the shard's first row); merge(dist [G,Q,k], ids [G,Q,k]) -> (dist [Q,k], ids [Q,k]).
        local_begin(queries, k, shards) -> bound [Q] and local_finish(bound) -> (dist, ids) are the two halves of
        local_search (optional).  `stream`: a ``torch.cuda.Stream`` on which the collectives are ordered (the
        stream the injected functions launch on), so that nothing has to wait on the host in between."""
        import torch.distributed as dist
        self._dist = dist
        self.local_search = local_search
        self.local_begin, self.local_finish = local_begin, local_finish
        self.merge = merge
        self.group = group
        self.stream = stream
        self.max_queries = max_queries
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def _host_order(self, t):
        # without a common stream the injected functions and the collectives run on different streams:
        # order them through the host
        if self.stream is None and t.is_cuda:
            import torch
            torch.cuda.current_stream().synchronize()

    def _local(self, queries, k):
        if self.world == 1 or self.local_begin is None or self.local_finish is None or queries is None:
            return self.local_search(queries, k)
        import torch
        nq = queries.shape[0]
        if nq > self.max_queries:      # the two-half search takes a bounded batch
            parts = [self._local(queries[b:b + self.max_queries], k) for b in range(0, nq, self.max_queries)]
            return torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
        bound = self.local_begin(queries, k, self.world)
        self._dist.all_reduce(bound, op=self._dist.ReduceOp.MAX, group=self.group)
        self._host_order(bound)
        return self.local_finish(bound)

    def batchSearch(self, queries, k: int):
        import torch
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else contextlib.nullcontext()
        with ctx:
            d, i = self._local(queries, k)
            if self.world == 1:
                return d, i
            world, nq = self.world, d.shape[0]
            per = -(-nq // world)              # queries merged by each rank
            if per * world != nq:              # pad to whole slices (padding rows merge to nothing)
                dp = torch.full((per * world, k), float("inf"), dtype=d.dtype, device=d.device)
                ip = torch.full((per * world, k), -1, dtype=i.dtype, device=i.device)
                dp[:nq], ip[:nq] = d, i
                d, i = dp, ip
            d, i = d.contiguous(), i.contiguous()
            rd, ri = torch.empty_like(d), torch.empty_like(i)     # [world][per][k]: slice of rank r's lists
            self._dist.all_to_all_single(rd, d, group=self.group)
            self._dist.all_to_all_single(ri, i, group=self.group)
            self._host_order(rd)
            md, mi = self.merge(rd.view(world, per, k), ri.view(world, per, k))
            od, oi = torch.empty_like(d), torch.empty_like(i)
            self._dist.all_gather_into_tensor(od, md.contiguous(), group=self.group)
            self._dist.all_gather_into_tensor(oi, mi.contiguous(), group=self.group)
            if d.is_cuda:
                (self.stream or torch.cuda.current_stream()).synchronize()
            return od[:nq], oi[:nq]

    def batchSearchHost(self, queries_host, k: int, out_dist_host, out_ids_host, staging=None,
                        gather_queries: bool = False):
        """Host buffers in, host buffers out: the queries go to `staging` (a device tensor of their shape; CPU ranks
        pass none and search the host tensor itself), the sharded search runs on them, and the merged result is
        copied into the two host tensors.  Everything is ordered on the search's stream; the call returns when the
        results are in host memory.  With `gather_queries` (all ranks were handed the same host queries) a rank copies
        only its share of them to the device and an all-gather hands every rank the rest.  The copies are torch's
        blocking kind on purpose: a non-blocking copy makes
        torch's pinned-memory allocator keep an event of the stream, and the search's stream belongs to the library
        and may be gone when the host buffers are freed."""
        import torch
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else contextlib.nullcontext()
        with ctx:
            q = queries_host
            nq = queries_host.shape[0]
            if staging is not None and gather_queries and self.world > 1:
                # every rank holds the same host queries: each sends only its 1/G of them over PCIe and the ranks
                # exchange the parts over NVLink (`staging` has ceil(Q / G) * G rows; the padding is never read)
                per = -(-nq // self.world)
                r = self._dist.get_rank(self.group)
                lo = min(r * per, nq)
                hi = min(lo + per, nq)
                part = torch.empty((per,) + tuple(staging.shape[1:]), dtype=staging.dtype, device=staging.device)
                if hi > lo:
                    part[:hi - lo].copy_(queries_host[lo:hi])
                self._dist.all_gather_into_tensor(staging, part, group=self.group)
                q = staging[:nq]
            elif staging is not None:
                staging.copy_(queries_host)
                q = staging
            d, i = self.batchSearch(q, k)
            out_dist_host.copy_(d)
            out_ids_host.copy_(i)
        return out_dist_host, out_ids_host


class ShardedKMeans:
    """Lloyd iterations over rows spread across the ranks of a group: every rank assigns its own rows to the
    current centroids and sums them per centroid (``step``), the per-centroid sums, counts and the inertia are added
    up over the ranks with one all-reduce each, and every rank forms the same new centroids (``finish``).  This is
    ``KMeansClustering.cluster`` (``Clustering/KMeansClustering.swift:48-113``) with its update step split at the
    point where shards have to talk; an empty cluster keeps its centroid.

    ``step(centroids) -> (sums [k, d], counts [k], inertia [1])`` and ``finish(sums, counts, centroids) -> centroids``
    are injected (on GPUs: ``KMeansTrainer.step`` / ``KMeansTrainer.finish``), so that the exchange can be exercised
    on CPU ranks in tests."""

    def __init__(self, step: Callable, finish: Callable, group=None):
        import torch.distributed as dist
        self._dist = dist
        self.step, self.finish, self.group = step, finish, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def cluster(self, initial_centroids, max_iterations: int, tolerance: float = 1e-4):
        """-> (centroids, iterations, inertia).  tolerance < 0 runs exactly max_iterations."""
        cent = initial_centroids
        prev, inertia, it = float("inf"), float("inf"), 0
        while it < max_iterations:
            sums, counts, inert = self.step(cent)
            if self.world > 1:
                for t in (sums, counts, inert):
                    self._dist.all_reduce(t, group=self.group)
            cent = self.finish(sums, counts, cent)
            it += 1
            if tolerance < 0:          # a fixed number of iterations: nothing to decide, nothing to read back
                continue
            inertia = float(inert.sum())
            if abs(inertia - prev) < tolerance:     # KMeansClustering.swift:98
                break
            prev = inertia
        if tolerance < 0 and it > 0:
            inertia = float(inert.sum())
        return cent, it, inertia
