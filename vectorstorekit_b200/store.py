"""The caller's side of the search path: entries with string ids and metadata in, ``SearchResult`` objects out.

The GPU library works on dense insertion indices and 64-bit row masks.  The reference's callers work on
``VectorEntry(id:vector:metadata:)`` and get ``[SearchResult]`` with ``id: VectorID`` (a String) and the entry's
metadata back (``Core/VectorTypes.swift:23-45``, ``Core/SearchTypes.swift:11-55``); ``IVFIndex`` keeps ids and metadata
host-side next to the vectors (``Indexes/IVFIndex.swift:104-111``) and evaluates a ``SearchFilter`` on the probed
candidates before ranking them (``:162-165``).  This module is that layer over the C ABI:

* an id table (insertion index -> VectorID) and the metadata of every row, kept on the host as the reference does;
* a ``FilterBitmaskCompiler`` that turns the filters searches use into row masks.  A filter is registered the first
  time a search uses it (or up front, ``filters=``), the row masks are recomputed on the host and pushed to the index,
  and from then on the filter costs one AND per candidate on the GPU instead of a JSON evaluation per stored vector
  and search (``Core/FilterEvaluator.swift:375-437``);
* ``search`` / ``batchSearch`` with the reference's signature and result type.

``VectorStore`` wraps a flat exact index (``VectorStore.search``, ``API/VectorStore.swift:271-318`` over a flat primary
index; one query is the streaming scan); ``IVFVectorIndex`` wraps ``IVFIndex`` with ``train(on:)``, one-entry
``insert`` and ``search(query:k:strategy:filter:)``.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from . import engine as _e
from .filters import FilterBitmaskCompiler, SearchFilter


@dataclasses.dataclass(frozen=True)
class VectorEntry:
    """``VectorEntry`` (``Core/VectorTypes.swift:23-45``): id, vector, metadata (a JSON-like dict or None)."""
    id: str
    vector: Any
    metadata: Optional[Dict[str, Any]] = None


@dataclasses.dataclass(frozen=True)
class SearchResult:
    """``SearchResult`` (``Core/SearchTypes.swift:11-55``): the fields the search path fills."""
    id: str
    distance: float
    metadata: Optional[Dict[str, Any]]
    tier: str = "hot"
    confidence: float = 1.0


@dataclasses.dataclass(frozen=True)
class InsertResult:
    """``InsertResult`` (``Core/Protocols.swift:411-423``)."""
    success: bool
    insertTime: float
    memoryImpact: int
    indexReorganization: bool


class _IdTable:
    """Insertion index -> (VectorID, metadata, vector); the masks of the registered filters."""

    def __init__(self, dimensions: int, filters: Sequence[SearchFilter] = ()):
        self.dimensions = dimensions
        self.ids: List[str] = []
        self.metadata: List[Optional[dict]] = []
        self.vectors: List[np.ndarray] = []
        self.by_id: Dict[str, int] = {}
        self.compiler = FilterBitmaskCompiler()
        for f in filters:
            self.compiler.register(f)

    def append(self, entry: VectorEntry) -> np.ndarray:
        v = np.ascontiguousarray(np.asarray(entry.vector, np.float32).reshape(-1))
        if v.size != self.dimensions:
            raise _e.DimensionMismatch(f"expected {self.dimensions}, got {v.size}")
        self.by_id[entry.id] = len(self.ids)
        self.ids.append(entry.id)
        self.metadata.append(entry.metadata)
        self.vectors.append(v)
        return v

    def masks(self, lo: int = 0, hi: Optional[int] = None) -> np.ndarray:
        hi = len(self.ids) if hi is None else hi
        if hi <= lo:
            return np.zeros(0, np.uint64)
        if not self.compiler.registered:
            return np.zeros(hi - lo, np.uint64)
        return self.compiler.row_masks(self.metadata[lo:hi], np.stack(self.vectors[lo:hi]))

    def results(self, dist_row, id_row) -> List[SearchResult]:
        out = []
        for d, i in zip(dist_row, id_row):
            i = int(i)
            if i < 0:
                break                                   # fewer than k eligible rows: the list just ends
            out.append(SearchResult(self.ids[i], float(d), self.metadata[i]))
        return out


class VectorStore:
    """A flat exact store: ``add`` entries, ``search(query:k:strategy:filter:)`` -> ``[SearchResult]``."""

    def __init__(self, dev: _e.CUDAComputeDevice, dimensions: int, metric=_e.DistanceMetric.euclidean,
                 filters: Sequence[SearchFilter] = ()):
        self.dev, self.dimensions, self.metric = dev, int(dimensions), metric
        self.table = _IdTable(self.dimensions, filters)
        self._index: Optional[_e.FlatIndex] = None
        self._indexed = 0           # rows the GPU index holds
        self._masks_stale = False   # a filter was registered after rows were indexed

    @property
    def count(self) -> int:
        return len(self.table.ids)

    def add(self, entries: Sequence[VectorEntry]) -> InsertResult:
        t0 = time.perf_counter()
        for e in entries:
            self.table.append(e)
        return InsertResult(True, time.perf_counter() - t0, 4 * self.dimensions * len(entries), False)

    def _sync(self):
        # The flat index takes either masks on every block or on none, and a filter registered later changes the masks
        # of rows already stored: in both cases the GPU index is rebuilt from the host copy the table keeps.
        n = self.count
        if self._index is not None and (self._masks_stale or self._indexed > n):
            self._index.close()
            self._index, self._indexed = None, 0
        if self._index is None:
            self._index = _e.FlatIndex(self.dev, self.dimensions, self.metric)
        if self._indexed < n:
            rows = np.stack(self.table.vectors[self._indexed:n])
            self._index.add(rows, self.table.masks(self._indexed, n))
            self._indexed = n
        self._masks_stale = False

    def _query_masks(self, filters: Sequence[Optional[SearchFilter]]):
        if all(f is None for f in filters):
            return None
        for f in filters:
            if f is not None and f not in self.table.compiler.registered:
                try:
                    self.table.compiler.query_mask(f)          # an `or` of registered filters needs no bit of its own
                except KeyError:
                    self.table.compiler.register(f)
                    self._masks_stale = True
        return filters

    def batchSearch(self, queries, k: int, filters: Optional[Sequence[Optional[SearchFilter]]] = None) -> List[List[SearchResult]]:
        if self.count == 0:
            raise _e.EmptyInput("the store is empty")
        q = np.ascontiguousarray(np.asarray(queries, np.float32).reshape(-1, self.dimensions))
        flt = self._query_masks(filters) if filters is not None else None
        self._sync()
        if flt is None:
            d, i = self._index.batchSearch(q, int(k))
        else:
            # a query without a filter sees every row: its rows are searched unfiltered
            qm = self.table.compiler.query_masks([f for f in flt])
            d, i = self._index.batchSearch(q, int(k), qm)
            free = [a for a, f in enumerate(flt) if f is None]
            if free:
                d2, i2 = self._index.batchSearch(q[free], int(k))
                d[free], i[free] = d2, i2
        return [self.table.results(d[a], i[a]) for a in range(q.shape[0])]

    def search(self, query, k: int, strategy: _e.SearchStrategy = _e.SearchStrategy.adaptive,
               filter: Optional[SearchFilter] = None) -> List[SearchResult]:
        return self.batchSearch(np.asarray(query, np.float32).reshape(1, -1), k, None if filter is None else [filter])[0]

    def close(self):
        if self._index is not None:
            self._index.close()
            self._index = None


class IVFVectorIndex:
    """``IVFIndex<Vector, Metadata>`` as its callers see it: ``train(on:)``, ``insert(_ entry:)``,
    ``search(query:k:strategy:filter:) -> [SearchResult]`` (``Indexes/IVFIndex.swift:80-202,397-446``)."""

    def __init__(self, dev: _e.CUDAComputeDevice, dimensions: int, numberOfCentroids: int = 1024, numberOfProbes: int = 10,
                 maxIterations: int = 100, tolerance: float = 1e-4, seed: Optional[int] = None,
                 filters: Sequence[SearchFilter] = ()):
        self.index = _e.IVFIndex(dev, dimensions, numberOfCentroids, min(numberOfProbes, numberOfCentroids), maxIterations,
                                 tolerance, trainingSampleSize=max(100_000, numberOfCentroids), seed=seed)
        self.dimensions = int(dimensions)
        self.table = _IdTable(self.dimensions, filters)
        self._indexed = 0
        self._masks_stale = False

    @property
    def count(self) -> int:
        return len(self.table.ids)

    @property
    def trained(self) -> bool:
        return self.index.trained

    def train(self, samples, initialCentroids=None):
        """Training clears the lists (``IVFIndex.swift:441-445``)."""
        self.index.train(np.ascontiguousarray(np.asarray(samples, np.float32)), initialCentroids)
        self.table = _IdTable(self.dimensions, self.table.compiler.registered)
        self._indexed = 0

    def insert(self, entry: VectorEntry) -> InsertResult:
        t0 = time.perf_counter()
        if not self.index.trained:
            raise _e.NotTrained("Index must be trained before use")
        self.table.append(entry)
        return InsertResult(True, time.perf_counter() - t0, 4 * self.dimensions, False)

    def _sync(self):
        n = self.count
        if self._indexed < n:
            # new rows go behind the rows their lists already hold; they carry masks iff the index does
            rows = np.stack(self.table.vectors[self._indexed:n])
            self.index.insert(rows, self.table.masks(self._indexed, n) if self.index._has_masks else None)
            self._indexed = n
        if self.table.compiler.registered and (self._masks_stale or not self.index._has_masks):
            m = self.table.masks(0, n)           # every row against every registered filter, in insertion order
            self.index.dev.check(self.index._lib.vsk_ivf_set_masks(self.index._h, _e._ptr(m)))
            self.index._has_masks = True
        self._masks_stale = False

    def search(self, query, k: int, strategy: _e.SearchStrategy = _e.SearchStrategy.adaptive,
               filter: Optional[SearchFilter] = None) -> List[SearchResult]:
        if not self.index.trained:
            raise _e.NotTrained("Index must be trained before use")
        if self.count == 0:
            return []
        qm = None
        if filter is not None:
            try:
                bit = self.table.compiler.query_mask(filter)
            except KeyError:
                self.table.compiler.register(filter)
                self._masks_stale = True
                bit = self.table.compiler.query_mask(filter)
            qm = np.array([bit], np.uint64)
        self._sync()
        q = np.ascontiguousarray(np.asarray(query, np.float32).reshape(1, -1))
        d, i = self.index.batchSearch(q, int(k), strategy, qm)
        return self.table.results(d[0], i[0])

    def close(self):
        self.index.close()
