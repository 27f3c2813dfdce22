"""Host-side mirror of VectorStoreKit's acceleration interface over the CUDA C ABI.

Names, argument meaning and error behaviour follow the reference's Swift types for this path
(paths relative to ``Sources/VectorStoreKit``):

* ``DistanceMetric``              — ``Core/SearchTypes.swift:105-118``
* ``CUDAAcceleratorStrategy``     — a ``ComputeAccelerator`` (``Core/Protocols.swift:11-20``), the
  plug-in point the Metal strategies implement (``API/Strategies/AcceleratorStrategies.swift``)
* ``CUDAAccelerationEngine``      — ``MetalAccelerationEngine.computeDistances`` /
  ``batchComputeDistances(queries:candidates:metric:topK:)``
  (``Acceleration/MetalAccelerationEngine.swift:76-204``)
* ``FlatIndex``                   — the resident flat exact search behind ``VectorStore.search`` /
  batch search (``API/VectorStore.swift:271-318``, ``LLM/LLMVectorStore.swift:83-114``)
* ``IVFIndex``                    — ``Indexes/IVFIndex.swift`` train / insert / search
* ``ScalarQuantizer``             — ``Quantization/ScalarQuantizer.swift`` (int8)

Arrays may be numpy arrays (host memory: copied in and out by the library) or torch CUDA tensors
(device memory of the engine's GPU: used in place, results returned as CUDA tensors).
"""
from __future__ import annotations

import ctypes as C
import os
import enum
import weakref
from typing import Optional, Sequence

import numpy as np

from . import _lib

try:  # torch is plumbing for device memory only
    import torch
except Exception:  # pragma: no cover
    torch = None


class DistanceMetric(enum.Enum):
    """``DistanceMetric`` of the reference; only the first four run on the accelerated path
    (``MetalDistanceCompute.swift:342-344`` throws ``unsupportedOperation`` for the rest)."""
    euclidean = "euclidean"
    cosine = "cosine"
    dotProduct = "dotProduct"
    manhattan = "manhattan"
    chebyshev = "chebyshev"
    minkowski = "minkowski"
    hamming = "hamming"
    jaccard = "jaccard"
    mahalanobis = "mahalanobis"
    earth_mover = "earth_mover"
    learned = "learned"
    adaptive = "adaptive"


_METRIC_ID = {DistanceMetric.euclidean: 0, DistanceMetric.cosine: 1, DistanceMetric.dotProduct: 2,
              DistanceMetric.manhattan: 3}
_METRIC_OF_ID = {v: k for k, v in _METRIC_ID.items()}


class SearchStrategy(enum.Enum):
    """``SearchStrategy`` cases that matter to IVF probing (``IVFIndex.swift:551-560``)."""
    exact = "exact"
    approximate = "approximate"
    adaptive = "adaptive"


# ---- errors: MetalComputeError (Metal/MetalErrors.swift:10-39), IVFError (IVFIndex.swift:619-637)
class VSKError(RuntimeError):
    status = -1


class DeviceNotAvailable(VSKError):
    status = 1


class DeviceOutOfMemory(VSKError):
    status = 2


class UnsupportedOperation(VSKError):
    status = 3


class InvalidBufferSize(VSKError):
    status = 4


class ExecutionFailed(VSKError):
    status = 5


class Timeout(VSKError):
    status = 6


class InvalidInput(VSKError):
    status = 7


class DimensionMismatch(VSKError):
    status = 8


class EmptyInput(VSKError):
    status = 9


class NotTrained(VSKError):
    status = 10


class InsufficientTrainingData(VSKError):
    status = 11


class ImportFailed(VSKError):
    """``ImportError.decodingFailed`` (``Indexes/IVFIndex.swift:640-643``): not an index image, truncated, or a
    section's checksum does not match."""
    status = 12


class ExportFailed(VSKError):
    """``VectorStoreError.exportError`` (``Core/Errors.swift:661-680``)."""
    status = 13


_ERRORS = {c.status: c for c in (DeviceNotAvailable, DeviceOutOfMemory, UnsupportedOperation, InvalidBufferSize,
                                 ExecutionFailed, Timeout, InvalidInput, DimensionMismatch, EmptyInput, NotTrained,
                                 InsufficientTrainingData, ImportFailed, ExportFailed)}


def _metric_id(metric) -> int:
    if isinstance(metric, str):
        metric = DistanceMetric(metric)
    if metric not in _METRIC_ID:
        raise UnsupportedOperation(f"Distance metric {metric.value} not supported on GPU")
    return _METRIC_ID[metric]


def _is_dev(a) -> bool:
    return torch is not None and isinstance(a, torch.Tensor) and a.is_cuda


def _host(a, dtype):
    if torch is not None and isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=dtype)


def _ptr(a):
    """Address of an array for the C ABI.  The library works on its own CUDA stream, which does not wait for
    torch's: a CUDA tensor is handed over only after the torch stream that produced it has drained."""
    if a is None:
        return None
    if _is_dev(a):
        torch.cuda.current_stream(a.device).synchronize()
        if _lib.CHECKED and a.numel():
            # the checked build tests every kernel access against the buffers it knows: announce this one
            _lib.load().vsk_checked_register(C.c_void_p(a.data_ptr()), a.numel() * a.element_size())
        return C.c_void_p(a.data_ptr())
    return C.c_void_p(a.ctypes.data)


class CUDAComputeDevice:
    """What ``CUDAAcceleratorStrategy.initialize()`` returns: an opened context on one GPU."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        st = self._lib.vsk_open(device, C.byref(h))
        if st != 0:
            raise _ERRORS.get(st, VSKError)(
                f"cannot open CUDA device {device}: {self._lib.vsk_status_string(st).decode()}")
        self._h = h
        self.device = device
        self._children = weakref.WeakSet()   # indices and trainers created on this context: closed before it
        self._inflight = set()          # asynchronous calls whose callback has not run
        self._inflight_keep = {}        # their buffers and callback objects

    # The checked build variant (``VSK_CHECKED=1``; ``vsk_checked_*``): refused accesses since the last call as
    # (count, first address, size | write << 8 | misaligned << 9); always (0, 0, 0) in the normal library.
    def checked_faults(self):
        out = (C.c_uint64 * 3)()
        self.check(self._lib.vsk_checked_faults(self._h, out))
        return int(out[0]), int(out[1]), int(out[2])

    def checked_selftest(self):
        self.check(self._lib.vsk_checked_selftest(self._h))

    def wait(self):
        """``vsk_wait``: blocks until every asynchronous call has completed; raises the first failure."""
        st = self._lib.vsk_wait(self._h)
        self._inflight_keep = {k: v for k, v in self._inflight_keep.items() if k in self._inflight}
        self.check(st)

    def close(self):
        if getattr(self, "_h", None):
            for child in list(self._children):
                try:
                    child.close()
                except Exception:
                    pass
            self._lib.vsk_close(self._h)
            self._h = None
            self._inflight_keep = {}

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def check(self, st: int):
        if st != 0:
            msg = self._lib.vsk_last_error(self._h).decode()
            raise _ERRORS.get(st, VSKError)(msg or self._lib.vsk_status_string(st).decode())

    def info(self) -> dict:
        d = _lib.DeviceInfo()
        self.check(self._lib.vsk_device_info_get(self._h, C.byref(d)))
        return {"device": d.device, "name": d.name.decode(), "sm_count": d.sm_count,
                "compute_capability": (d.cc_major, d.cc_minor), "hbm_bytes": d.hbm_bytes, "l2_bytes": d.l2_bytes,
                "max_smem_per_block": d.max_smem_per_block}

    def stats(self) -> dict:
        s = _lib.Stats()
        self.check(self._lib.vsk_stats_get(self._h, C.byref(s)))
        return {f: getattr(s, f) for f, _ in s._fields_}

    def profile(self, enable: bool):
        self.check(self._lib.vsk_profile(self._h, 1 if enable else 0))

    def set_search_path(self, path: int):
        self.check(self._lib.vsk_set_search_path(self._h, path))

    @property
    def stream(self) -> int:
        return int(self._lib.vsk_stream(self._h) or 0)

    def timeline(self, enable: bool):
        self.check(self._lib.vsk_timeline(self._h, 1 if enable else 0))

    def timeline_read(self):
        """-> [(lane, what, ms)] of the calls since the log was switched on or last read."""
        buf = C.create_string_buffer(1 << 20)
        n = self._lib.vsk_timeline_read(self._h, buf, len(buf))
        out = []
        for line in buf.raw[:max(n, 0)].decode().splitlines():
            lane, what, ms = line.split()
            out.append((int(lane), what, float(ms)))
        return out

    def measure_peak(self, what: str) -> float:
        """``vsk_measure_peak``: "fp32_issue" (FP32 instructions/s per thread), "smem_gather" (4-byte words/s) or
        "tmem_read" (bytes/s read out of tensor memory)."""
        v = C.c_double()
        self.check(self._lib.vsk_measure_peak(self._h, {"fp32_issue": 0, "smem_gather": 1, "tmem_read": 2}[what], C.byref(v)))
        return float(v.value)

    # ---- tuning of the search schedule (``vsk_tuning``) ----
    def tuning(self) -> dict:
        t = _lib.Tuning()
        self.check(self._lib.vsk_tuning_get(self._h, C.byref(t)))
        return {f: getattr(t, f) for f, _ in t._fields_ if f != "reserved"}

    def set_tuning(self, **fields):
        t = _lib.Tuning()
        self.check(self._lib.vsk_tuning_get(self._h, C.byref(t)))
        for name, value in fields.items():
            if name == "reserved" or not hasattr(t, name):
                raise InvalidInput(f"unknown tuning field {name}")
            setattr(t, name, int(value))
        self.check(self._lib.vsk_tuning_set(self._h, C.byref(t)))

    # ---- communicator of a row-sharded search: one process and one device object per GPU ----
    def comm_unique_id(self) -> bytes:
        """128 bytes made on ONE rank; hand the same bytes to ``comm_init`` on every rank."""
        buf = (C.c_ubyte * _lib.COMM_ID_BYTES)()
        st = self._lib.vsk_comm_unique_id(buf)
        if st != 0:
            raise ExecutionFailed("NCCL is not available (libnccl.so.2 could not be loaded)")
        return bytes(buf)

    def comm_init(self, nranks: int, rank: int, unique_id: Optional[bytes]):
        buf = (C.c_ubyte * _lib.COMM_ID_BYTES).from_buffer_copy(unique_id) if unique_id is not None else None
        self.check(self._lib.vsk_comm_init(self._h, int(nranks), int(rank), buf))

    def comm_destroy(self):
        self.check(self._lib.vsk_comm_destroy(self._h))

    def comm_info(self):
        n, r = C.c_int32(), C.c_int32()
        self.check(self._lib.vsk_comm_info(self._h, C.byref(n), C.byref(r)))
        return n.value, r.value

    def sharded_phase_ms(self):
        ms = (C.c_float * _lib.SHARDED_PHASES)()
        self.check(self._lib.vsk_sharded_phase_ms(self._h, ms))
        names = ("queries", "scan", "bound_allreduce", "finish", "all_to_all", "merge", "gather")
        return dict(zip(names, (float(x) for x in ms)))


class CUDAAcceleratorStrategy:
    """``ComputeAccelerator`` conformance for a B200 (``Core/Protocols.swift:11-20``)."""

    identifier = "cuda-sm100a"
    requirements = {"minimumMemory": 1 << 30, "requiredFeatures": ["cuda", "sm_100a"], "optionalFeatures": ["nvlink"]}

    def __init__(self, device: int = 0):
        self.device_index = device
        self._dev: Optional[CUDAComputeDevice] = None

    def initialize(self) -> CUDAComputeDevice:
        """Raises ``DeviceNotAvailable`` (the reference's ``AcceleratorError.noDevice``) without a B200."""
        if self._dev is None:
            self._dev = CUDAComputeDevice(self.device_index)
        return self._dev

    def capabilities(self) -> dict:
        return self.initialize().info()


PATH_TENSOR_RERANK, PATH_FP32_SCAN = 0, 1


class CUDAAccelerationEngine:
    """Signature mirror of ``MetalAccelerationEngine`` for distances and batch top-k."""

    def __init__(self, device: Optional[CUDAComputeDevice] = None):
        self.dev = device or CUDAComputeDevice(0)
        self._lib = self.dev._lib

    # MetalAccelerationEngine.computeDistances(query:candidates:metric:) -> [Float]
    def computeDistances(self, query, candidates, metric):
        q = query.reshape(1, -1) if hasattr(query, "reshape") else np.asarray(query, np.float32).reshape(1, -1)
        return self.batchComputeDistances(q, candidates, metric)[0]

    # MetalAccelerationEngine.batchComputeDistances(queries:candidates:metric:topK:) -> [[Float]]
    def batchComputeDistances(self, queries, candidates, metric, topK: Optional[int] = None):
        """Q x N distances, or per query the ``topK`` smallest ascending (distances only, as the
        reference returns)."""
        mid = _metric_id(metric)
        if len(candidates) == 0 or len(queries) == 0:
            raise EmptyInput("Empty input provided for distance computation")
        if topK is not None:
            index = FlatIndex(self.dev, queries.shape[1], metric)
            try:
                index.add(candidates)
                d, _ = index.batchSearch(queries, min(topK, len(candidates)))
            finally:
                index.close()
            return d
        if _is_dev(queries) != _is_dev(candidates):
            raise InvalidInput("queries and candidates must both be host arrays or both CUDA tensors")
        if queries.shape[1] != candidates.shape[1]:
            raise DimensionMismatch(f"expected {queries.shape[1]}, got {candidates.shape[1]}")
        nq, d = queries.shape
        nx = candidates.shape[0]
        if _is_dev(queries):
            q = queries.contiguous().float()
            x = candidates.contiguous().float()
            out = torch.empty((nq, nx), dtype=torch.float32, device=q.device)
            self.dev.check(self._lib.vsk_batch_distances_dev(self.dev._h, mid, _ptr(q), nq, _ptr(x), nx, d, _ptr(out)))
            return out
        q, x = _host(queries, np.float32), _host(candidates, np.float32)
        out = np.empty((nq, nx), np.float32)
        self.dev.check(self._lib.vsk_batch_distances(self.dev._h, mid, _ptr(q), nq, _ptr(x), nx, d, _ptr(out)))
        return out

    # MetalDistanceMatrix.computeDistanceMatrix(vectorsA:vectorsB:metric:) -> [[Float]]
    # (Acceleration/Metal/MetalDistanceMatrix.swift:49-119).  With vectorsB omitted the matrix of vectorsA against
    # itself is returned and, as the reference does (:352-381), the upper triangle (with the diagonal) is what is
    # computed: the lower triangle is its mirror image.
    def computeDistanceMatrix(self, vectorsA, vectorsB=None, metric=DistanceMetric.euclidean):
        out = self.batchComputeDistances(vectorsA, vectorsA if vectorsB is None else vectorsB, metric)
        if vectorsB is None:
            if _is_dev(out):
                out = torch.triu(out) + torch.triu(out, 1).T
            else:
                out = np.triu(out) + np.triu(out, 1).T
        return out

    def mergeTopK(self, dist, ids):
        """[G, Q, k] per-shard results with global ids (CUDA tensors) -> merged [Q, k]."""
        g, nq, k = dist.shape
        dist = dist.contiguous()
        ids = ids.contiguous()
        od = torch.empty((nq, k), dtype=torch.float32, device=dist.device)
        oi = torch.empty((nq, k), dtype=torch.int64, device=dist.device)
        self.dev.check(self._lib.vsk_merge_topk_dev(self.dev._h, _ptr(dist), _ptr(ids), g, nq, k, _ptr(od), _ptr(oi)))
        return od, oi


class _IndexBase:
    def __init__(self, dev: CUDAComputeDevice):
        self.dev = dev
        self._lib = dev._lib
        self._h = None
        dev._children.add(self)

    def close(self):
        # An index lives inside its context: once the device object is closed (it closes its indices first) the
        # handle is gone too.  At interpreter shutdown finalisers run in no particular order, hence the check.
        if self._h and getattr(self.dev, "_h", None):
            self._lib.vsk_index_destroy(self._h)
        self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    @property
    def count(self) -> int:
        return int(self._lib.vsk_index_size(self._h)) if self._h else 0

    def set_id_base(self, base: int):
        self.dev.check(self._lib.vsk_index_set_id_base(self._h, base))

    def info(self) -> dict:
        d = _lib.IndexInfo()
        self.dev.check(self._lib.vsk_index_info_get(self._h, C.byref(d)))
        return {"kind": ("flat_f32", "flat_i8", "ivf", "pq")[d.kind], "metric": _METRIC_OF_ID[d.metric],
                "dimensions": d.dimensions, "count": d.count, "id_base": d.id_base, "nlist": d.nlist,
                "has_masks": bool(d.has_masks), "pq_segments": d.pq_segments, "pq_codebook_size": d.pq_codebook_size}

    # ``VectorIndex.export(format:) -> Data`` / ``import(data:format:)`` (``Core/Protocols.swift:157-160``); only the
    # binary format exists here, any other raises as ``IVFIndex.export`` does (``Indexes/IVFIndex.swift:304-311``).
    def export(self, format: str = "binary") -> bytes:
        if format != "binary":
            raise ExportFailed(f"unsupported export format {format}")
        size = C.c_int64()
        self.dev.check(self._lib.vsk_index_image_size(self._h, C.byref(size)))
        buf = np.empty(size.value, np.uint8)
        written = C.c_int64()
        self.dev.check(self._lib.vsk_index_export(self._h, _ptr(buf), size.value, C.byref(written)))
        return buf[: written.value].tobytes()

    def save(self, path: str):
        self.dev.check(self._lib.vsk_index_save(self._h, str(path).encode()))

    def _search(self, queries, k, qmasks=None):
        nq = queries.shape[0]
        if _is_dev(queries):
            q = queries.contiguous().float()
            od = torch.empty((nq, k), dtype=torch.float32, device=q.device)
            oi = torch.empty((nq, k), dtype=torch.int64, device=q.device)
            qm = qmasks.contiguous() if qmasks is not None else None
            self.dev.check(self._lib.vsk_search_dev(self._h, _ptr(q), nq, k, _ptr(qm), _ptr(od), _ptr(oi)))
            return od, oi
        q = _host(queries, np.float32)
        od = np.empty((nq, k), np.float32)
        oi = np.empty((nq, k), np.int64)
        qm = _host(qmasks, np.uint64) if qmasks is not None else None
        self.dev.check(self._lib.vsk_search(self._h, _ptr(q), nq, k, _ptr(qm), _ptr(od), _ptr(oi)))
        return od, oi

    def _searchAsync(self, queries, k, qmasks=None):
        """``vsk_search_async`` / ``vsk_search_dev_async``: returns a ``concurrent.futures.Future`` that the library's
        worker thread resolves to (dist, ids), or fails with the error class of the status.  Until the future is
        done the device object takes only further ``*Async`` calls and ``wait()``."""
        import concurrent.futures
        fut = concurrent.futures.Future()
        nq = queries.shape[0]
        dev_side = _is_dev(queries)
        if dev_side:
            q = queries.contiguous().float()
            od = torch.empty((nq, k), dtype=torch.float32, device=q.device)
            oi = torch.empty((nq, k), dtype=torch.int64, device=q.device)
            qm = qmasks.contiguous() if qmasks is not None else None
            call = self._lib.vsk_search_dev_async
        else:
            q = _host(queries, np.float32)
            od = np.empty((nq, k), np.float32)
            oi = np.empty((nq, k), np.int64)
            qm = _host(qmasks, np.uint64) if qmasks is not None else None
            call = self._lib.vsk_search_async
        keep = []                                   # buffers and the callback object live until the callback ran

        def done(_user, st):
            try:
                if st == 0:
                    fut.set_result((od, oi))
                else:
                    msg = self._lib.vsk_last_error(self.dev._h).decode()
                    fut.set_exception(_ERRORS.get(st, VSKError)(msg or self._lib.vsk_status_string(st).decode()))
            finally:
                self.dev._inflight.discard(id(keep))

        cb = _lib.DONE_FN(done)
        keep.extend((q, qm, od, oi, cb, keep))
        self.dev._inflight_keep[id(keep)] = keep
        self.dev._inflight.add(id(keep))
        st = call(self._h, _ptr(q), nq, k, _ptr(qm), _ptr(od), _ptr(oi), cb, None)
        if st != 0:
            self.dev._inflight.discard(id(keep))
            self.dev._inflight_keep.pop(id(keep), None)
            self.dev.check(st)
        return fut


def sharded_slice(nq: int, nranks: int, rank: int):
    """Queries [first, first + count) whose merged results rank `rank` returns under the SLICE layout."""
    per = -(-nq // max(nranks, 1))
    lo = min(rank * per, nq)
    return lo, min(per, nq - lo)


class _ShardedSearchMixin:
    """``vsk_search_sharded`` (``vsk_ivf_search_sharded`` for an IVF index): the row-sharded form of ``batchSearch``
    for an index whose device object has joined a communicator (``CUDAComputeDevice.comm_init``).  Every rank passes
    the same queries."""
    _sharded_names = ("vsk_search_sharded_dev", "vsk_search_sharded")

    def _sharded_extra(self):
        """Arguments between k and the query masks (the IVF form's nprobe)."""
        return ()

    def shardedSearch(self, queries, k: int, filter_masks=None, gather: bool = False, split_queries: bool = False,
                      out=None):
        """-> (dist, ids).  gather=False: this rank's slice of the queries (``sharded_slice``), merged over all
        shards; gather=True: all queries on every rank.  Device tensors in -> device tensors out; host arrays (numpy,
        or pinned torch CPU tensors) in -> host out, copies inside the call.  `out` = (dist, ids) buffers to fill."""
        nq, k = int(queries.shape[0]), int(k)
        if nq == 0:
            raise EmptyInput("no queries")
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        nranks, rank = self.dev.comm_info()
        rows = nq if (gather or nranks == 1) else sharded_slice(nq, nranks, rank)[1]
        layout = (_lib.SHARDED_ALL if gather else _lib.SHARDED_SLICE) | (_lib.SHARDED_QUERIES_SPLIT if split_queries else 0)
        if _is_dev(queries):
            q = queries.contiguous().float()
            od, oi = out if out is not None else (torch.empty((max(rows, 1), k), dtype=torch.float32, device=q.device),
                                                  torch.empty((max(rows, 1), k), dtype=torch.int64, device=q.device))
            qm = filter_masks.contiguous() if filter_masks is not None else None
            fn = getattr(self._lib, self._sharded_names[0])
            self.dev.check(fn(self._h, _ptr(q), nq, k, *self._sharded_extra(), _ptr(qm), layout, _ptr(od), _ptr(oi)))
            return od[:rows], oi[:rows]
        if torch is not None and isinstance(queries, torch.Tensor):      # a (pinned) CPU tensor
            q = queries.contiguous()
            od, oi = out if out is not None else (torch.empty((max(rows, 1), k), dtype=torch.float32),
                                                  torch.empty((max(rows, 1), k), dtype=torch.int64))
            qm = filter_masks.contiguous() if filter_masks is not None else None
            ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
            fn = getattr(self._lib, self._sharded_names[1])
            self.dev.check(fn(self._h, ptr(q), nq, k, *self._sharded_extra(), ptr(qm), layout, ptr(od), ptr(oi)))
            return od[:rows], oi[:rows]
        q = _host(queries, np.float32)
        od, oi = out if out is not None else (np.empty((max(rows, 1), k), np.float32), np.empty((max(rows, 1), k), np.int64))
        qm = _host(filter_masks, np.uint64) if filter_masks is not None else None
        fn = getattr(self._lib, self._sharded_names[1])
        self.dev.check(fn(self._h, _ptr(q), nq, k, *self._sharded_extra(), _ptr(qm), layout, _ptr(od), _ptr(oi)))
        return od[:rows], oi[:rows]


def _adopt(dev: "CUDAComputeDevice", h):
    """Wrap a handle that came out of an index image in the class of its kind."""
    probe = _IndexBase(dev)
    probe._h = h
    info = probe.info()
    cls = {"flat_f32": FlatIndex, "flat_i8": QuantizedFlatIndex, "ivf": IVFIndex, "pq": PQIndex}[info["kind"]]
    ix = cls.__new__(cls)
    _IndexBase.__init__(ix, dev)
    ix._h, probe._h = h, None
    ix.dimensions = info["dimensions"]
    if cls is PQIndex:
        ix.segments, ix.codebookSize = info["pq_segments"], info["pq_codebook_size"]
    if cls is IVFIndex:
        ix._has_masks = info["has_masks"]
        ix._pending_rows, ix._pending_masks = [], []
        ix.trainingSampleSize, ix.seed = 100_000, None
        ix.numberOfCentroids = info["nlist"]
        ix.numberOfProbes = min(10, info["nlist"])      # IVFConfiguration default (IVFConfiguration.swift:32)
        ix.clustering = KMeansClustering(dev)
        cent = np.empty((info["nlist"], info["dimensions"]), np.float32)
        dev.check(dev._lib.vsk_ivf_centroids(h, _ptr(cent)))
        ix.centroids = cent
        ix.trained = True
    return ix


def import_index(dev: "CUDAComputeDevice", data, format: str = "binary"):
    """``import(data:format:)``: rebuild an index from the bytes ``export`` produced."""
    if format != "binary":
        raise ImportFailed(f"unsupported import format {format}")
    buf = np.frombuffer(data, np.uint8)
    h = C.c_void_p()
    dev.check(dev._lib.vsk_index_import(dev._h, _ptr(buf), buf.size, C.byref(h)))
    return _adopt(dev, h)


def load_index(dev: "CUDAComputeDevice", path: str):
    """Rebuild an index from the file ``save`` wrote."""
    h = C.c_void_p()
    dev.check(dev._lib.vsk_index_load(dev._h, str(path).encode(), C.byref(h)))
    return _adopt(dev, h)


class FlatIndex(_IndexBase, _ShardedSearchMixin):
    """Resident database + exact k-NN.  ``masks`` are per-row uint64 metadata bitmasks; a search
    with ``filter_masks`` keeps row r for query q iff ``masks[r] & filter_masks[q] != 0`` — the
    bitmask form of the reference's pre-filter (``Indexes/IVFIndex.swift:163-172``)."""

    def __init__(self, dev: CUDAComputeDevice, dimensions: int, metric=DistanceMetric.euclidean):
        super().__init__(dev)
        h = C.c_void_p()
        dev.check(self._lib.vsk_flat_create(dev._h, _metric_id(metric), int(dimensions), C.byref(h)))
        self._h = h
        self.dimensions = int(dimensions)

    def add(self, rows, masks=None):
        if len(rows) == 0:
            raise EmptyInput("no rows to add")
        if rows.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {rows.shape[1]}")
        if _is_dev(rows):
            r = rows.contiguous().float()
            m = masks.contiguous() if masks is not None else None
            self.dev.check(self._lib.vsk_flat_add_f32_dev(self._h, _ptr(r), r.shape[0], _ptr(m)))
        else:
            r = _host(rows, np.float32)
            m = _host(masks, np.uint64) if masks is not None else None
            self.dev.check(self._lib.vsk_flat_add_f32(self._h, _ptr(r), r.shape[0], _ptr(m)))

    # VectorStore.search(query:k:strategy:filter:) for one query
    def search(self, query, k: int, filter_mask: Optional[int] = None):
        q = query.reshape(1, -1)
        fm = None
        if filter_mask is not None:
            fm = (torch.tensor([filter_mask], dtype=torch.int64, device=q.device).view(torch.int64) if _is_dev(q)
                  else np.array([filter_mask], np.uint64))
        d, i = self.batchSearch(q, k, fm)
        return d[0], i[0]

    # batchSearch(queries:k:filter:) — one ascending row of k hits per query, in query order
    def batchSearch(self, queries, k: int, filter_masks=None):
        if len(queries) == 0:
            raise EmptyInput("no queries")
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        return self._search(queries, int(k), filter_masks)

    # The awaited form (``MetalAccelerationEngine.batchComputeDistances`` is ``async``, :139-204): a future of
    # batchSearch's result.
    def batchSearchAsync(self, queries, k: int, filter_masks=None):
        if len(queries) == 0:
            raise EmptyInput("no queries")
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        return self._searchAsync(queries, int(k), filter_masks)

    def coarseValues(self, queries, rows: int):
        """``vsk_coarse_values_dev``: the tensor path's coarse values of the first `rows` rows and the per-query
        bound the certificate assumes on |coarse - exact| (device tensors), for auditing that bound."""
        q = queries.contiguous().float()
        coarse = torch.empty((q.shape[0], int(rows)), dtype=torch.float32, device=q.device)
        eps = torch.empty(q.shape[0], dtype=torch.float32, device=q.device)
        self.dev.check(self._lib.vsk_coarse_values_dev(self._h, _ptr(q), q.shape[0], int(rows), _ptr(coarse), _ptr(eps)))
        return coarse, eps

    # The search in two halves, for one shard of a row-sharded database (``sharded.ShardedSearch``): `begin` scans
    # and returns, per query, a value that this shard's ceil(k / shards) best rows do not exceed; the caller takes the
    # maximum over the shards and `finish` returns this shard's rows that can still be among the overall k best
    # (others padded with +inf / -1).  Device tensors; no other call on the device object in between.  `begin`
    # returns while its kernels still run on the library's stream (``dev.stream``): reduce the bound on that stream
    # (``torch.cuda.ExternalStream``) or synchronise first.
    def shardSearchBegin(self, queries, k: int, shards: int):
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        if not _is_dev(queries):
            raise InvalidInput("the two-half search takes device tensors")
        q = queries.contiguous().float()
        bound = torch.empty(q.shape[0], dtype=torch.float32, device=q.device)
        self.dev.check(self._lib.vsk_search_shard_begin_dev(self._h, _ptr(q), q.shape[0], int(k), int(shards), _ptr(bound)))
        self._pending = (q, int(k))
        return bound

    def shardSearchFinish(self, bound):
        q, k = self._pending
        od = torch.empty((q.shape[0], k), dtype=torch.float32, device=q.device)
        oi = torch.empty((q.shape[0], k), dtype=torch.int64, device=q.device)
        self.dev.check(self._lib.vsk_search_shard_finish_dev(self._h, _ptr(bound.contiguous()), _ptr(od), _ptr(oi)))
        self._pending = None
        return od, oi


class KMeansClustering:
    """``KMeansClustering.cluster`` (``Clustering/KMeansClustering.swift:48-113``) with ``.custom``
    initial centroids (:189-193).  Returns (centroids, assignments, iterations, inertia)."""

    def __init__(self, dev: CUDAComputeDevice, maxIterations: int = 100, tolerance: float = 1e-4,
                 seed: Optional[int] = None):
        self.dev = dev
        self._lib = dev._lib
        self.maxIterations = maxIterations
        self.tolerance = tolerance
        self.seed = seed          # KMeansClusteringConfiguration.seed; None = drawn from the system, as SystemRNG is

    def initializeKMeansPlusPlus(self, vectors, k: int, seed: Optional[int] = None):
        """``initializeKMeansPlusPlus`` (``KMeansClustering.swift:209-260``) -> (centroids, picked row indices)."""
        n, d = vectors.shape
        if seed is None:
            seed = self.seed
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        picked = np.empty(k, np.int64)
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            cent = torch.empty((k, d), dtype=torch.float32, device=x.device)
            self.dev.check(self._lib.vsk_kmeans_init_plusplus_dev(self.dev._h, _ptr(x), n, d, k, C.c_uint64(seed), _ptr(cent),
                                                                  _ptr(picked)))
        else:
            x = _host(vectors, np.float32)
            cent = np.empty((k, d), np.float32)
            self.dev.check(self._lib.vsk_kmeans_init_plusplus(self.dev._h, _ptr(x), n, d, k, C.c_uint64(seed), _ptr(cent),
                                                              _ptr(picked)))
        return cent, picked

    def cluster(self, vectors, k: int, initialCentroids=None):
        """initialCentroids=None: k-means++ (the reference's default ``initMethod``); else ``.custom``."""
        if len(vectors) == 0:
            raise EmptyInput("emptyDataset")
        n, d = vectors.shape
        if initialCentroids is None:
            initialCentroids, _ = self.initializeKMeansPlusPlus(vectors, k)
        inertia = C.c_float()
        iters = C.c_int32()
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            init = initialCentroids.contiguous().float()
            cent = torch.empty((k, d), dtype=torch.float32, device=x.device)
            asg = torch.empty(n, dtype=torch.int32, device=x.device)
            self.dev.check(self._lib.vsk_kmeans_dev(self.dev._h, _ptr(x), n, d, k, self.maxIterations, self.tolerance,
                                                    _ptr(init), _ptr(cent), _ptr(asg), C.byref(inertia),
                                                    C.byref(iters)))
        else:
            x = _host(vectors, np.float32)
            init = _host(initialCentroids, np.float32)
            cent = np.empty((k, d), np.float32)
            asg = np.empty(n, np.int32)
            self.dev.check(self._lib.vsk_kmeans(self.dev._h, _ptr(x), n, d, k, self.maxIterations, self.tolerance,
                                                _ptr(init), _ptr(cent), _ptr(asg), C.byref(inertia), C.byref(iters)))
        return cent, asg, int(iters.value), float(inertia.value)

    def assign(self, vectors, centroids):
        """Nearest centroid and rooted distance per row (CUDA tensors)."""
        x = vectors.contiguous().float()
        c = centroids.contiguous().float()
        asg = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
        dist = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        self.dev.check(self._lib.vsk_assign_dev(self.dev._h, _ptr(x), x.shape[0], x.shape[1], _ptr(c), c.shape[0],
                                                _ptr(asg), _ptr(dist)))
        return asg, dist


class KMeansTrainer:
    """One shard's side of a multi-GPU k-means run (``vectorstorekit_b200.sharded.ShardedKMeans`` drives it): the
    shard's rows stay on the device, ``step`` assigns them to the given centroids and returns this shard's
    per-centroid sums, counts and inertia as CUDA tensors, ``finish`` forms the means from summed contributions."""

    def __init__(self, dev: CUDAComputeDevice, rows, k: int):
        if not _is_dev(rows):
            raise InvalidInput("KMeansTrainer takes a CUDA tensor of rows")
        self.dev, self._lib = dev, dev._lib
        self.rows = rows.contiguous().float()          # kept alive: the library reads it on every step
        self.k = int(k)
        self.n, self.dim = self.rows.shape
        h = C.c_void_p()
        dev.check(self._lib.vsk_kmeans_trainer_create_dev(dev._h, _ptr(self.rows), self.n, self.dim, self.k, C.byref(h)))
        self._h = h
        dev._children.add(self)

    def step(self, centroids):
        c = centroids.contiguous().float()
        sums = torch.empty((self.k, self.dim), dtype=torch.float32, device=c.device)
        counts = torch.empty((self.k,), dtype=torch.float32, device=c.device)
        inertia = torch.empty((1,), dtype=torch.float32, device=c.device)
        self.dev.check(self._lib.vsk_kmeans_trainer_step_dev(self._h, _ptr(c), _ptr(sums), _ptr(counts), _ptr(inertia)))
        return sums, counts, inertia

    def finish(self, sums, counts, centroids):
        out = torch.empty_like(sums)
        self.dev.check(self._lib.vsk_kmeans_finish_dev(self.dev._h, _ptr(sums.contiguous()), _ptr(counts.contiguous()),
                                                       _ptr(centroids.contiguous().float()), self.k, self.dim, _ptr(out)))
        return out

    def assignments(self):
        a = torch.empty((self.n,), dtype=torch.int32, device=self.rows.device)
        self.dev.check(self._lib.vsk_kmeans_trainer_assignments_dev(self._h, _ptr(a)))
        return a

    def close(self):
        if self._h and getattr(self.dev, "_h", None):
            self._lib.vsk_kmeans_trainer_destroy(self._h)
        self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


class IVFIndex(_IndexBase, _ShardedSearchMixin):
    """``IVFIndex`` (``Indexes/IVFIndex.swift``): ``train(on:)`` runs k-means for the centroids, ``insert`` files rows
    under their nearest centroid's list, ``search`` probes ``numberOfProbes`` lists (all of them for
    ``SearchStrategy.exact``) with rooted L2, after the metadata filter when one is given.  Ids are insertion
    indices.  The first ``insert`` builds the lists; later ones append to them (``vsk_ivf_add``) without touching the
    assignment of the rows already stored.  ``insertEntry`` is the reference's one-entry ``insert``: entries are
    collected on the host and appended as one block before the next search."""

    def __init__(self, dev: CUDAComputeDevice, dimensions: int, numberOfCentroids: int = 1024,
                 numberOfProbes: int = 10, maxIterations: int = 100, tolerance: float = 1e-4,
                 trainingSampleSize: int = 100_000, seed: Optional[int] = None):
        super().__init__(dev)
        if dimensions <= 0 or numberOfCentroids <= 0 or not (0 < numberOfProbes <= numberOfCentroids) \
                or trainingSampleSize < numberOfCentroids:
            raise InvalidInput("IVFConfiguration.validate failed")  # IVFConfiguration.swift:49-59
        self.dimensions = dimensions
        self.numberOfCentroids = numberOfCentroids
        self.numberOfProbes = numberOfProbes
        self.trainingSampleSize = trainingSampleSize            # IVFConfiguration.swift:12,33
        self.seed = seed
        self.clustering = KMeansClustering(dev, maxIterations, tolerance, seed=seed)
        self.centroids = None
        self.trained = False
        self._has_masks = False
        self._pending_rows, self._pending_masks = [], []

    def train(self, samples, initialCentroids=None):
        """``train(on:)`` (``IVFIndex.swift:397-446``).  initialCentroids=None is the reference's default
        initialisation, k-means++ (``KMeansClustering.swift:209-260``), seeded by ``seed``."""
        if len(samples) < self.numberOfCentroids:
            raise InsufficientTrainingData(f"provided {len(samples)}, required {self.numberOfCentroids}")
        self.centroids, _, iters, inertia = self.clustering.cluster(samples, self.numberOfCentroids, initialCentroids)
        self.trained = True
        self.close()
        self._has_masks = False
        self._pending_rows, self._pending_masks = [], []
        return iters, inertia

    def trainOnSample(self, allVectors, initialCentroids=None):
        """What ``optimize`` / re-training do with a large store (``IVFIndex.swift:462-468``): train on
        ``trainingSampleSize`` rows drawn without replacement (seeded permutation) when there are more."""
        n = len(allVectors)
        if n > self.trainingSampleSize:
            rng = np.random.default_rng(self.seed)
            pick = np.sort(rng.permutation(n)[: self.trainingSampleSize])
            if _is_dev(allVectors):
                allVectors = allVectors[torch.as_tensor(pick, device=allVectors.device)]
            else:
                allVectors = np.asarray(allVectors)[pick]
        return self.train(allVectors, initialCentroids)

    def insert(self, rows, masks=None):
        """A block of rows (and their filter masks); ids continue from ``count``."""
        if not self.trained:
            raise NotTrained("Index must be trained before use")
        n, d = rows.shape
        if d != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {d}")
        self._flush()
        on_dev = _is_dev(rows)
        if on_dev:
            r = rows.contiguous().float()
            m = masks.contiguous() if masks is not None else None
        else:
            r = _host(rows, np.float32)
            m = _host(masks, np.uint64) if masks is not None else None
        if self._h:   # append to the lists
            fn = self._lib.vsk_ivf_add_dev if on_dev else self._lib.vsk_ivf_add
            self.dev.check(fn(self._h, _ptr(r), n, _ptr(m)))
            return
        h = C.c_void_p()
        if on_dev:
            c = self.centroids if _is_dev(self.centroids) else torch.as_tensor(self.centroids, device=r.device)
            self.dev.check(self._lib.vsk_ivf_build_dev(self.dev._h, _ptr(c.contiguous()), self.numberOfCentroids,
                                                       _ptr(r), n, d, C.byref(h)))
        else:
            c = _host(self.centroids, np.float32)
            self.dev.check(self._lib.vsk_ivf_build(self.dev._h, _ptr(c), self.numberOfCentroids, _ptr(r), n, d,
                                                   C.byref(h)))
        self._h = h
        if m is not None:
            fn = self._lib.vsk_ivf_set_masks_dev if on_dev else self._lib.vsk_ivf_set_masks
            self.dev.check(fn(self._h, _ptr(m)))
            self._has_masks = True

    def insertEntry(self, vector, mask: Optional[int] = None) -> int:
        """``insert(_ entry:)`` (``IVFIndex.swift:80-122``): one vector; returns its id."""
        if not self.trained:
            raise NotTrained("Index must be trained before use")
        v = _host(vector, np.float32).reshape(-1)
        if v.size != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {v.size}")
        self._pending_rows.append(v)
        self._pending_masks.append(mask)
        return self.count - 1

    def _flush(self):
        if not self._pending_rows:
            return
        rows = np.stack(self._pending_rows)
        masks = None
        if any(m is not None for m in self._pending_masks):
            masks = np.array([0 if m is None else m for m in self._pending_masks], np.uint64)
        self._pending_rows, self._pending_masks = [], []
        self.insert(rows, masks)

    @property
    def count(self) -> int:
        return (int(self._lib.vsk_index_size(self._h)) if self._h else 0) + len(self._pending_rows)

    def assignments(self):
        self._flush()
        out = np.empty(self.count, np.int32)
        self.dev.check(self._lib.vsk_ivf_assignments(self._h, _ptr(out)))
        return out

    def batchSearch(self, queries, k: int, strategy: SearchStrategy = SearchStrategy.adaptive, filter_masks=None):
        if not self.trained:
            raise NotTrained("Index must be trained before use")
        self._flush()
        if not self._h:
            raise NotTrained("Index must be trained before use")
        nprobe = self.numberOfCentroids if strategy == SearchStrategy.exact else self.numberOfProbes
        nq = queries.shape[0]
        if _is_dev(queries):
            q = queries.contiguous().float()
            od = torch.empty((nq, k), dtype=torch.float32, device=q.device)
            oi = torch.empty((nq, k), dtype=torch.int64, device=q.device)
            qm = filter_masks.contiguous() if filter_masks is not None else None
            self.dev.check(self._lib.vsk_ivf_search_filtered_dev(self._h, _ptr(q), nq, k, nprobe, _ptr(qm), _ptr(od), _ptr(oi)))
            return od, oi
        q = _host(queries, np.float32)
        od = np.empty((nq, k), np.float32)
        oi = np.empty((nq, k), np.int64)
        qm = _host(filter_masks, np.uint64) if filter_masks is not None else None
        self.dev.check(self._lib.vsk_ivf_search_filtered(self._h, _ptr(q), nq, k, nprobe, _ptr(qm), _ptr(od), _ptr(oi)))
        return od, oi

    # the row-sharded form (``vsk_ivf_search_sharded``): every rank holds a slice of every list and probes
    # ``numberOfProbes`` of them; see ``_ShardedSearchMixin.shardedSearch``
    _sharded_names = ("vsk_ivf_search_sharded_dev", "vsk_ivf_search_sharded")

    def _sharded_extra(self):
        return (int(self.numberOfProbes),)

    def shardedSearch(self, queries, k: int, filter_masks=None, gather: bool = False, split_queries: bool = False, out=None):
        if not self.trained:
            raise NotTrained("Index must be trained before use")
        self._flush()
        return _ShardedSearchMixin.shardedSearch(self, queries, k, filter_masks, gather, split_queries, out)

    def search(self, query, k: int, strategy: SearchStrategy = SearchStrategy.adaptive, filter_mask: Optional[int] = None):
        fm = None if filter_mask is None else np.array([filter_mask], np.uint64)
        if fm is not None and _is_dev(query):
            fm = torch.as_tensor(fm.view(np.int64), device=query.device)
        d, i = self.batchSearch(query.reshape(1, -1), k, strategy, fm)
        return d[0], i[0]


class ScalarQuantizer:
    """``ScalarQuantizer`` for ``.int8`` (``Quantization/ScalarQuantizer.swift``).  ``per_dim=False``
    is the reference's behaviour (one scale/offset for the whole batch)."""

    def __init__(self, dev: CUDAComputeDevice, per_dim: bool = False):
        self.dev = dev
        self._lib = dev._lib
        self.per_dim = per_dim
        self.scale = None
        self.offset = None

    def train(self, vectors):
        n, d = vectors.shape
        mode = 1 if self.per_dim else 0
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            mn = torch.empty(d, dtype=torch.float32, device=x.device)
            mx = torch.empty_like(mn)
            self.dev.check(self._lib.vsk_sq8_minmax_dev(self.dev._h, _ptr(x), n, d, _ptr(mn), _ptr(mx)))
            return self.set_range(mn, mx)
        x = _host(vectors, np.float32)
        self.scale = np.empty(d, np.float32)
        self.offset = np.empty(d, np.float32)
        self.dev.check(self._lib.vsk_sq8_train(self.dev._h, _ptr(x), n, d, mode, _ptr(self.scale), _ptr(self.offset)))
        return self.scale, self.offset

    def minmax(self, vectors):
        """Per-dimension min/max of CUDA rows (to be reduced across shards by the caller)."""
        x = vectors.contiguous().float()
        mn = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
        mx = torch.empty_like(mn)
        self.dev.check(self._lib.vsk_sq8_minmax_dev(self.dev._h, _ptr(x), x.shape[0], x.shape[1], _ptr(mn), _ptr(mx)))
        return mn, mx

    def set_range(self, mn, mx):
        d = mn.shape[0]
        self.scale = torch.empty(d, dtype=torch.float32, device=mn.device)
        self.offset = torch.empty_like(self.scale)
        self.dev.check(self._lib.vsk_sq8_params_dev(self.dev._h, _ptr(mn.contiguous()), _ptr(mx.contiguous()), d,
                                                    1 if self.per_dim else 0, _ptr(self.scale), _ptr(self.offset)))
        return self.scale, self.offset

    def quantizeBatch(self, vectors):
        n, d = vectors.shape
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            codes = torch.empty((n, d), dtype=torch.int8, device=x.device)
            s = self.scale if _is_dev(self.scale) else torch.as_tensor(self.scale, device=x.device)
            o = self.offset if _is_dev(self.offset) else torch.as_tensor(self.offset, device=x.device)
            self.dev.check(self._lib.vsk_sq8_encode_dev(self.dev._h, _ptr(x), n, d, _ptr(s), _ptr(o), _ptr(codes)))
            return codes
        x = _host(vectors, np.float32)
        codes = np.empty((n, d), np.int8)
        self.dev.check(self._lib.vsk_sq8_encode(self.dev._h, _ptr(x), n, d, _ptr(_host(self.scale, np.float32)),
                                                _ptr(_host(self.offset, np.float32)), _ptr(codes)))
        return codes

    def dequantizeBatch(self, codes):
        codes = _host(codes, np.int8)
        out = np.empty(codes.shape, np.float32)
        self.dev.check(self._lib.vsk_sq8_decode(self.dev._h, _ptr(codes), codes.shape[0], codes.shape[1],
                                                _ptr(_host(self.scale, np.float32)),
                                                _ptr(_host(self.offset, np.float32)), _ptr(out)))
        return out


class QuantizedFlatIndex(_IndexBase, _ShardedSearchMixin):
    """Flat index over int8 codes; distances are taken against the dequantised rows."""

    def __init__(self, dev: CUDAComputeDevice, dimensions: int, metric, scale, offset):
        super().__init__(dev)
        h = C.c_void_p()
        s = scale.contiguous() if _is_dev(scale) else _host(scale, np.float32)
        o = offset.contiguous() if _is_dev(offset) else _host(offset, np.float32)
        dev.check(self._lib.vsk_sq8_index_create(dev._h, _metric_id(metric), int(dimensions), _ptr(s), _ptr(o),
                                                 C.byref(h)))
        self._h = h
        self.dimensions = int(dimensions)

    def add(self, codes):
        if _is_dev(codes):
            c = codes.contiguous()
            self.dev.check(self._lib.vsk_sq8_index_add_dev(self._h, _ptr(c), c.shape[0]))
        else:
            c = _host(codes, np.int8)
            self.dev.check(self._lib.vsk_sq8_index_add(self._h, _ptr(c), c.shape[0]))

    def batchSearch(self, queries, k: int):
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        return self._search(queries, int(k))


class ProductQuantizer:
    """``ProductQuantizer`` (``Quantization/ProductQuantizer.swift``) with ``ProductQuantizationConfig``'s fields
    (``Config/Quantization/ProductQuantizationConfig.swift:8-50``): ``segments`` sub-spaces, ``codeSize`` bits per
    code (at most 8: a code is one byte), ``codebookSize = 1 << codeSize`` codewords each.  ``codebooks`` is
    ``[segments][codebookSize][dimensions / segments]``.  Training starts from caller-supplied codewords (default:
    the segments of the first ``codebookSize`` vectors); the reference's k-means++ / mini-batch draws cannot be
    reproduced."""

    def __init__(self, dev: CUDAComputeDevice, dimensions: int, segments: int = 8, codeSize: int = 8,
                 trainingIterations: int = 25):
        if dimensions <= 0 or segments <= 0 or dimensions % segments != 0:
            raise InvalidInput(f"invalid segmentation: {dimensions} dimensions into {segments} segments")
        if not (4 <= codeSize <= 16):                       # ProductQuantizationConfig.validate :46-48
            raise InvalidInput(f"invalid code size {codeSize}")
        if codeSize > 8:
            raise UnsupportedOperation("codes are stored as one byte per segment: codeSize must be at most 8")
        self.dev, self._lib = dev, dev._lib
        self.dimensions, self.segments, self.codeSize = int(dimensions), int(segments), int(codeSize)
        self.codebookSize = 1 << codeSize
        self.segmentDimensions = dimensions // segments
        self.trainingIterations = int(trainingIterations)
        self.codebooks = None
        self.trained = False

    def _shape(self):
        return self.dimensions, self.segments, self.codebookSize

    def _cb(self, like=None):
        if not self.trained:
            raise NotTrained("Quantizer must be trained before use")
        if like is not None and _is_dev(like):
            return self.codebooks if _is_dev(self.codebooks) else torch.as_tensor(self.codebooks, device=like.device)
        return _host(self.codebooks, np.float32)

    def set_codebooks(self, codebooks):
        if tuple(codebooks.shape) != (self.segments, self.codebookSize, self.segmentDimensions):
            raise DimensionMismatch("codebooks must be [segments][codebookSize][dimensions / segments]")
        self.codebooks = codebooks.contiguous().float() if _is_dev(codebooks) else _host(codebooks, np.float32)
        self.trained = True

    def train(self, vectors, initialCodebooks=None):
        n, d = vectors.shape
        if d != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {d}")
        dim, m, ks = self._shape()
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            init = None if initialCodebooks is None else torch.as_tensor(initialCodebooks, device=x.device).contiguous().float()
            cb = torch.empty((m, ks, dim // m), dtype=torch.float32, device=x.device)
            self.dev.check(self._lib.vsk_pq_train_dev(self.dev._h, _ptr(x), n, dim, m, ks, self.trainingIterations,
                                                      _ptr(init), _ptr(cb)))
        else:
            x = _host(vectors, np.float32)
            init = None if initialCodebooks is None else _host(initialCodebooks, np.float32)
            cb = np.empty((m, ks, dim // m), np.float32)
            self.dev.check(self._lib.vsk_pq_train(self.dev._h, _ptr(x), n, dim, m, ks, self.trainingIterations,
                                                  _ptr(init), _ptr(cb)))
        self.codebooks = cb
        self.trained = True
        return cb

    def encodeBatch(self, vectors):
        n, d = vectors.shape
        if d != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {d}")
        dim, m, ks = self._shape()
        cb = self._cb(vectors)
        if _is_dev(vectors):
            x = vectors.contiguous().float()
            codes = torch.empty((n, m), dtype=torch.uint8, device=x.device)
            self.dev.check(self._lib.vsk_pq_encode_dev(self.dev._h, _ptr(cb), dim, m, ks, _ptr(x), n, _ptr(codes)))
            return codes
        x = _host(vectors, np.float32)
        codes = np.empty((n, m), np.uint8)
        self.dev.check(self._lib.vsk_pq_encode(self.dev._h, _ptr(cb), dim, m, ks, _ptr(x), n, _ptr(codes)))
        return codes

    def decodeBatch(self, codes):
        dim, m, ks = self._shape()
        c = _host(codes, np.uint8)
        out = np.empty((c.shape[0], dim), np.float32)
        self.dev.check(self._lib.vsk_pq_decode(self.dev._h, _ptr(self._cb()), dim, m, ks, _ptr(c), c.shape[0], _ptr(out)))
        return out

    # precomputeDistanceTables(query:) (:205-233), for a batch: [nq][segments][codebookSize]
    def precomputeDistanceTables(self, queries):
        dim, m, ks = self._shape()
        q = _host(queries, np.float32)
        if q.ndim == 1:
            q = q[None]
        if q.shape[1] != dim:
            raise DimensionMismatch(f"expected {dim}, got {q.shape[1]}")
        out = np.empty((q.shape[0], m, ks), np.float32)
        self.dev.check(self._lib.vsk_pq_distance_tables(self.dev._h, _ptr(self._cb()), dim, m, ks, _ptr(q), q.shape[0],
                                                        _ptr(out)))
        return out

    def index(self):
        """A resident index of codes searched by asymmetric distance."""
        return PQIndex(self.dev, self.dimensions, self.segments, self.codebookSize, self._cb())


class PQIndex(_IndexBase):
    """Codes resident on the GPU; ``batchSearch`` returns per query the ``k`` rows with the smallest asymmetric
    distance (``DistanceTables.computeDistance``, ``ProductQuantizerTypes.swift:14-20``), ascending, ties by row."""

    def __init__(self, dev: CUDAComputeDevice, dimensions: int, segments: int, codebookSize: int, codebooks):
        super().__init__(dev)
        h = C.c_void_p()
        cb = codebooks.contiguous().float() if _is_dev(codebooks) else _host(codebooks, np.float32)
        dev.check(self._lib.vsk_pq_index_create(dev._h, int(dimensions), int(segments), int(codebookSize), _ptr(cb),
                                                C.byref(h)))
        self._h = h
        self.dimensions, self.segments, self.codebookSize = int(dimensions), int(segments), int(codebookSize)

    def add(self, codes):
        if codes.shape[1] != self.segments:
            raise DimensionMismatch(f"expected {self.segments} codes per row, got {codes.shape[1]}")
        if _is_dev(codes):
            c = codes.contiguous()
            self.dev.check(self._lib.vsk_pq_index_add_dev(self._h, _ptr(c), c.shape[0]))
        else:
            c = _host(codes, np.uint8)
            self.dev.check(self._lib.vsk_pq_index_add(self._h, _ptr(c), c.shape[0]))

    def batchSearch(self, queries, k: int):
        if queries.shape[1] != self.dimensions:
            raise DimensionMismatch(f"expected {self.dimensions}, got {queries.shape[1]}")
        return self._search(queries, int(k))
