"""Row-sharded search over the ranks of a ``torch.distributed`` group (one process per GPU).

Rank g holds rows ``[g*N/G, (g+1)*N/G)`` of the database and answers every query on its shard; the
per-rank ``[Q, k]`` (distance, global id) lists are exchanged with one all-gather and merged into the
result an unsharded search would return (ties by global id).  The reference has no sharded search;
this is the multi-GPU form of ``batchSearch``.

The local search and the merge are injected, so that the exchange logic can be exercised on CPU ranks
(``gloo``) in tests; on GPUs they are ``FlatIndex.batchSearch`` and ``CUDAAccelerationEngine.mergeTopK``.
"""
from __future__ import annotations

from typing import Callable, Tuple


def shard_range(n_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank `rank`; the union over ranks is [0, n_total) with no overlap."""
    return rank * n_total // world, (rank + 1) * n_total // world


class ShardedSearch:
    def __init__(self, local_search: Callable, merge: Callable, group=None):
        """local_search(queries, k) -> (dist [Q,k], ids [Q,k]) with GLOBAL ids (set the index's id base to
        the shard's first row); merge(dist [G,Q,k], ids [G,Q,k]) -> (dist [Q,k], ids [Q,k])."""
        import torch.distributed as dist
        self._dist = dist
        self.local_search = local_search
        self.merge = merge
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def batchSearch(self, queries, k: int):
        import torch
        d, i = self.local_search(queries, k)
        if self.world == 1:
            return d, i
        gd = torch.empty((self.world,) + tuple(d.shape), dtype=d.dtype, device=d.device)
        gi = torch.empty((self.world,) + tuple(i.shape), dtype=i.dtype, device=i.device)
        if d.is_cuda:   # NCCL: one collective straight into the stacked buffer
            self._dist.all_gather_into_tensor(gd, d.contiguous(), group=self.group)
            self._dist.all_gather_into_tensor(gi, i.contiguous(), group=self.group)
        else:           # gloo (CPU tests)
            self._dist.all_gather(list(gd.unbind(0)), d.contiguous(), group=self.group)
            self._dist.all_gather(list(gi.unbind(0)), i.contiguous(), group=self.group)
        if d.is_cuda:
            torch.cuda.current_stream().synchronize()
        return self.merge(gd, gi)


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
            inertia = float(inert.sum())
            it += 1
            if tolerance >= 0 and abs(inertia - prev) < tolerance:     # KMeansClustering.swift:98
                break
            prev = inertia
        return cent, it, inertia
