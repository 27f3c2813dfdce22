"""TEST INFRASTRUCTURE — not part of the product.

ctypes front-end to the two CPU checkers built by ``oracle/Makefile``:

* ``cpu``   — ``_build/libvsk_oracle.so``: the C++ restatement of the reference's
  CPU search arithmetic (``cpu_ref.cpp``).
* ``metal`` — ``_ref/libvsk_metalref.so``: the reference's own Metal shader source
  compiled as host C++ (present only where it was built from the reference tree).

Only ``tests/``, the smoke check and the benchmark's cpu-baseline leg may import
this package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

EUCLIDEAN, COSINE, DOT, MANHATTAN = 0, 1, 2, 3
METRIC_IDS = {"euclidean": 0, "cosine": 1, "dotProduct": 2, "manhattan": 3}

_f32p = C.POINTER(C.c_float)
_i64p = C.POINTER(C.c_int64)
_i32p = C.POINTER(C.c_int32)
_u64p = C.POINTER(C.c_uint64)
_i8p = C.POINTER(C.c_int8)
_u8p = C.POINTER(C.c_uint8)
_u32p = C.POINTER(C.c_uint32)


def reference_tree():
    """The reference checkout, if this machine has one: $VSK_REFERENCE_TREE, else a folder named `reference` beside the
    repository.  Only the build of the shader checker reads it."""
    cand = os.environ.get("VSK_REFERENCE_TREE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "Sources", "VectorStoreKit")) else None


def build(native: bool = False) -> None:
    """Run the Makefile (compiles cpu_ref.cpp; compiles the reference shaders when the
    reference checkout is present)."""
    ref = reference_tree()
    subprocess.run(["make", "-C", _HERE, "all"] + (["native"] if native else []) + ([f"REF={ref}"] if ref else []),
                   check=True, stdout=subprocess.DEVNULL)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a, t):
    return a.ctypes.data_as(t) if a is not None else None


class CpuOracle:
    """The C++ restatement."""

    def __init__(self, native: bool = False):
        name = "libvsk_oracle_native.so" if native else "libvsk_oracle.so"
        path = os.path.join(_HERE, "_build", name)
        if not os.path.exists(path):
            build(native)
        self.lib = L = C.CDLL(path)
        L.vskref_distance.restype = C.c_float
        L.vskref_distance.argtypes = [C.c_int, _f32p, _f32p, C.c_int]
        L.vskref_batch_distances.argtypes = [C.c_int, _f32p, C.c_int64, _f32p, C.c_int64, C.c_int, _f32p]
        L.vskref_flat_search.argtypes = [C.c_int, _f32p, C.c_int64, _f32p, C.c_int64, C.c_int, C.c_int,
                                         _u64p, _u64p, _f32p, _i64p, C.c_int, C.c_int]
        L.vskref_normalize_rows.argtypes = [_f32p, C.c_int64, C.c_int]
        L.vskref_kmeans.argtypes = [_f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_float, _f32p, _f32p,
                                    _i32p, _f32p, _i32p]
        L.vskref_assign.argtypes = [_f32p, C.c_int64, C.c_int, _f32p, C.c_int, _i32p, _f32p]
        L.vskref_ivf_search.argtypes = [_f32p, C.c_int64, _f32p, C.c_int64, C.c_int, _f32p, C.c_int, _i32p,
                                        C.c_int, C.c_int, _f32p, _i64p]
        L.vskref_ivf_search_filtered.argtypes = [_f32p, C.c_int64, _f32p, C.c_int64, C.c_int, _f32p, C.c_int, _i32p,
                                                 C.c_int, C.c_int, _u64p, _u64p, _f32p, _i64p]
        L.vskref_kmeans_plusplus.argtypes = [_f32p, C.c_int64, C.c_int, C.c_int, C.c_uint64, _f32p, _i64p]
        L.vskref_sq8_train.argtypes = [_f32p, C.c_int64, C.c_int, C.c_int, _f32p, _f32p]
        L.vskref_sq8_encode.argtypes = [_f32p, C.c_int64, C.c_int, _f32p, _f32p, _i8p]
        L.vskref_sq8_decode.argtypes = [_i8p, C.c_int64, C.c_int, _f32p, _f32p, _f32p]
        L.vskref_sq8_search.argtypes = [C.c_int, _f32p, C.c_int64, _i8p, C.c_int64, C.c_int, _f32p, _f32p,
                                        C.c_int, _f32p, _i64p]
        L.vskref_merge_topk.argtypes = [_f32p, _i64p, C.c_int, C.c_int64, C.c_int, _f32p, _i64p]
        L.vskref_num_threads.restype = C.c_int

    def num_threads(self) -> int:
        return int(self.lib.vskref_num_threads())

    def distance(self, metric, q, x) -> float:
        q, x = _f32(q), _f32(x)
        return float(self.lib.vskref_distance(metric, _ptr(q, _f32p), _ptr(x, _f32p), q.size))

    def batch_distances(self, metric, q, x):
        q, x = _f32(q), _f32(x)
        out = np.empty((q.shape[0], x.shape[0]), np.float32)
        self.lib.vskref_batch_distances(metric, _ptr(q, _f32p), q.shape[0], _ptr(x, _f32p), x.shape[0],
                                        q.shape[1], _ptr(out, _f32p))
        return out

    def flat_search(self, metric, q, x, k, row_masks=None, query_masks=None, fast=False, nthreads=0):
        q, x = _f32(q), _f32(x)
        nq = q.shape[0]
        dist = np.empty((nq, k), np.float32)
        ids = np.empty((nq, k), np.int64)
        rm = np.ascontiguousarray(row_masks, np.uint64) if row_masks is not None else None
        qm = np.ascontiguousarray(query_masks, np.uint64) if query_masks is not None else None
        self.lib.vskref_flat_search(metric, _ptr(q, _f32p), nq, _ptr(x, _f32p), x.shape[0], q.shape[1], k,
                                    _ptr(rm, _u64p), _ptr(qm, _u64p), _ptr(dist, _f32p), _ptr(ids, _i64p),
                                    1 if fast else 0, nthreads)
        return dist, ids

    def normalize_rows(self, x):
        x = _f32(x).copy()
        self.lib.vskref_normalize_rows(_ptr(x, _f32p), x.shape[0], x.shape[1])
        return x

    def kmeans(self, x, init, max_iters, tolerance=-1.0):
        x, init = _f32(x), _f32(init)
        n, d = x.shape
        k = init.shape[0]
        cent = np.empty((k, d), np.float32)
        asg = np.empty(n, np.int32)
        inertia = C.c_float()
        iters = C.c_int32()
        self.lib.vskref_kmeans(_ptr(x, _f32p), n, d, k, max_iters, tolerance, _ptr(init, _f32p),
                               _ptr(cent, _f32p), _ptr(asg, _i32p), C.byref(inertia), C.byref(iters))
        return cent, asg, float(inertia.value), int(iters.value)

    def assign(self, x, centroids):
        x, centroids = _f32(x), _f32(centroids)
        asg = np.empty(x.shape[0], np.int32)
        dist = np.empty(x.shape[0], np.float32)
        self.lib.vskref_assign(_ptr(x, _f32p), x.shape[0], x.shape[1], _ptr(centroids, _f32p),
                               centroids.shape[0], _ptr(asg, _i32p), _ptr(dist, _f32p))
        return asg, dist

    def ivf_search(self, q, x, centroids, assign, nprobe, k):
        q, x, centroids = _f32(q), _f32(x), _f32(centroids)
        assign = np.ascontiguousarray(assign, np.int32)
        dist = np.empty((q.shape[0], k), np.float32)
        ids = np.empty((q.shape[0], k), np.int64)
        self.lib.vskref_ivf_search(_ptr(q, _f32p), q.shape[0], _ptr(x, _f32p), x.shape[0], x.shape[1],
                                   _ptr(centroids, _f32p), centroids.shape[0], _ptr(assign, _i32p), nprobe, k,
                                   _ptr(dist, _f32p), _ptr(ids, _i64p))
        return dist, ids

    def ivf_search_filtered(self, q, x, centroids, assign, nprobe, k, row_masks, query_masks):
        q, x, centroids = _f32(q), _f32(x), _f32(centroids)
        assign = np.ascontiguousarray(assign, np.int32)
        rm = np.ascontiguousarray(row_masks, np.uint64) if row_masks is not None else None
        qm = np.ascontiguousarray(query_masks, np.uint64) if query_masks is not None else None
        dist = np.empty((q.shape[0], k), np.float32)
        ids = np.empty((q.shape[0], k), np.int64)
        self.lib.vskref_ivf_search_filtered(_ptr(q, _f32p), q.shape[0], _ptr(x, _f32p), x.shape[0], x.shape[1],
                                            _ptr(centroids, _f32p), centroids.shape[0], _ptr(assign, _i32p), nprobe, k,
                                            _ptr(rm, _u64p), _ptr(qm, _u64p), _ptr(dist, _f32p), _ptr(ids, _i64p))
        return dist, ids

    def kmeans_plusplus(self, x, k, seed):
        x = _f32(x)
        cent = np.empty((k, x.shape[1]), np.float32)
        picked = np.empty(k, np.int64)
        self.lib.vskref_kmeans_plusplus(_ptr(x, _f32p), x.shape[0], x.shape[1], k, C.c_uint64(seed), _ptr(cent, _f32p),
                                        _ptr(picked, _i64p))
        return cent, picked

    def sq8_train(self, x, per_dim):
        x = _f32(x)
        scale = np.empty(x.shape[1], np.float32)
        offset = np.empty(x.shape[1], np.float32)
        self.lib.vskref_sq8_train(_ptr(x, _f32p), x.shape[0], x.shape[1], int(per_dim), _ptr(scale, _f32p),
                                  _ptr(offset, _f32p))
        return scale, offset

    def sq8_encode(self, x, scale, offset):
        x, scale, offset = _f32(x), _f32(scale), _f32(offset)
        codes = np.empty(x.shape, np.int8)
        self.lib.vskref_sq8_encode(_ptr(x, _f32p), x.shape[0], x.shape[1], _ptr(scale, _f32p),
                                   _ptr(offset, _f32p), _ptr(codes, _i8p))
        return codes

    def sq8_decode(self, codes, scale, offset):
        codes = np.ascontiguousarray(codes, np.int8)
        scale, offset = _f32(scale), _f32(offset)
        x = np.empty(codes.shape, np.float32)
        self.lib.vskref_sq8_decode(_ptr(codes, _i8p), codes.shape[0], codes.shape[1], _ptr(scale, _f32p),
                                   _ptr(offset, _f32p), _ptr(x, _f32p))
        return x

    def sq8_search(self, metric, q, codes, scale, offset, k):
        q = _f32(q)
        codes = np.ascontiguousarray(codes, np.int8)
        scale, offset = _f32(scale), _f32(offset)
        dist = np.empty((q.shape[0], k), np.float32)
        ids = np.empty((q.shape[0], k), np.int64)
        self.lib.vskref_sq8_search(metric, _ptr(q, _f32p), q.shape[0], _ptr(codes, _i8p), codes.shape[0],
                                   codes.shape[1], _ptr(scale, _f32p), _ptr(offset, _f32p), k,
                                   _ptr(dist, _f32p), _ptr(ids, _i64p))
        return dist, ids

    # ---- product quantisation (codebooks: [m][ksub][d/m]) ----
    def pq_encode(self, x, codebooks):
        x, cb = _f32(x), _f32(codebooks)
        m, ksub, _ = cb.shape
        codes = np.empty((x.shape[0], m), np.uint8)
        self.lib.vskref_pq_encode(_ptr(x, _f32p), C.c_int64(x.shape[0]), x.shape[1], m, ksub, _ptr(cb, _f32p),
                                  _ptr(codes, _u8p))
        return codes

    def pq_decode(self, codes, codebooks):
        cb = _f32(codebooks)
        codes = np.ascontiguousarray(codes, np.uint8)
        m, ksub, ds = cb.shape
        x = np.empty((codes.shape[0], m * ds), np.float32)
        self.lib.vskref_pq_decode(_ptr(codes, _u8p), C.c_int64(codes.shape[0]), m * ds, m, ksub, _ptr(cb, _f32p),
                                  _ptr(x, _f32p))
        return x

    def pq_tables(self, q, codebooks):
        q, cb = _f32(q), _f32(codebooks)
        m, ksub, _ = cb.shape
        t = np.empty((q.shape[0], m, ksub), np.float32)
        self.lib.vskref_pq_tables(_ptr(q, _f32p), C.c_int64(q.shape[0]), q.shape[1], m, ksub, _ptr(cb, _f32p),
                                  _ptr(t, _f32p))
        return t

    def pq_search(self, q, codes, codebooks, k):
        q, cb = _f32(q), _f32(codebooks)
        codes = np.ascontiguousarray(codes, np.uint8)
        m, ksub, _ = cb.shape
        dist = np.empty((q.shape[0], k), np.float32)
        ids = np.empty((q.shape[0], k), np.int64)
        self.lib.vskref_pq_search(_ptr(q, _f32p), C.c_int64(q.shape[0]), _ptr(codes, _u8p), C.c_int64(codes.shape[0]),
                                  q.shape[1], m, ksub, _ptr(cb, _f32p), k, _ptr(dist, _f32p), _ptr(ids, _i64p))
        return dist, ids

    def pq_train(self, x, init_codebooks, iters):
        x, init = _f32(x), _f32(init_codebooks)
        m, ksub, _ = init.shape
        out = np.empty_like(init)
        self.lib.vskref_pq_train(_ptr(x, _f32p), C.c_int64(x.shape[0]), x.shape[1], m, ksub, iters, _ptr(init, _f32p),
                                 _ptr(out, _f32p))
        return out

    def merge_topk(self, dist, ids):
        """dist/ids: [G, Q, k] per-shard lists with global ids -> merged [Q, k]."""
        dist = _f32(dist)
        ids = np.ascontiguousarray(ids, np.int64)
        g, nq, k = dist.shape
        od = np.empty((nq, k), np.float32)
        oi = np.empty((nq, k), np.int64)
        self.lib.vskref_merge_topk(_ptr(dist, _f32p), _ptr(ids, _i64p), g, nq, k, _ptr(od, _f32p),
                                   _ptr(oi, _i64p))
        return od, oi


class MetalRef:
    """The reference's shader source compiled as C++ (distances, k-means step, uint8 quantiser)."""

    PATH = os.path.join(_HERE, "_ref", "libvsk_metalref.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        self.lib = L = C.CDLL(self.PATH)
        L.metalref_distances.argtypes = [C.c_int, _f32p, _f32p, C.c_uint, C.c_uint, _f32p]
        L.metalref_batch_distances.argtypes = [C.c_int, _f32p, C.c_uint, _f32p, C.c_uint, C.c_uint, _f32p]
        L.metalref_kmeans_step.argtypes = [_f32p, C.c_uint, C.c_uint, _f32p, C.c_uint, _u32p, _f32p, _f32p, _u32p]
        L.metalref_min_distances.argtypes = [_f32p, C.c_uint, C.c_uint, _f32p, C.c_uint, _f32p]
        L.metalref_scalar_quantize.argtypes = [_f32p, _u8p, C.c_float, C.c_float, C.c_uint]
        L.metalref_scalar_dequantize.argtypes = [_u8p, _f32p, C.c_float, C.c_float, C.c_uint]
        if hasattr(L, "metalref_product_quantize"):
            L.metalref_product_quantize.argtypes = [_f32p, _f32p, _u8p, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint]
            L.metalref_product_dequantize.argtypes = [_u8p, _f32p, _f32p, C.c_uint, C.c_uint, C.c_uint, C.c_uint]

    def product_quantize(self, x, codebooks):
        """Shader productQuantize (QuantizationShaders.metal:113-156); codebooks [m][ksub][d/m]."""
        x, cb = _f32(x), _f32(codebooks)
        m, ksub, ds = cb.shape
        codes = np.empty((x.shape[0], m), np.uint8)
        self.lib.metalref_product_quantize(_ptr(x, _f32p), _ptr(cb, _f32p), _ptr(codes, _u8p), x.shape[0], x.shape[1],
                                           m, ds, ksub)
        return codes

    def product_dequantize(self, codes, codebooks):
        """Shader productDequantize (:177-204); assumes 256 codes per subspace."""
        cb = _f32(codebooks)
        codes = np.ascontiguousarray(codes, np.uint8)
        m, ksub, ds = cb.shape
        assert ksub == 256
        x = np.empty((codes.shape[0], m * ds), np.float32)
        self.lib.metalref_product_dequantize(_ptr(codes, _u8p), _ptr(cb, _f32p), _ptr(x, _f32p), codes.shape[0],
                                             m * ds, m, ds)
        return x

    def distances(self, metric, q, x):
        q, x = _f32(q), _f32(x)
        out = np.empty(x.shape[0], np.float32)
        self.lib.metalref_distances(metric, _ptr(q, _f32p), _ptr(x, _f32p), x.shape[0], x.shape[1],
                                    _ptr(out, _f32p))
        return out

    def batch_distances(self, metric, q, x):
        q, x = _f32(q), _f32(x)
        out = np.empty((q.shape[0], x.shape[0]), np.float32)
        self.lib.metalref_batch_distances(metric, _ptr(q, _f32p), q.shape[0], _ptr(x, _f32p), x.shape[0],
                                          x.shape[1], _ptr(out, _f32p))
        return out

    def kmeans_step(self, x, centroids):
        x = _f32(x)
        cent = _f32(centroids).copy()
        n, d = x.shape
        k = cent.shape[0]
        asg = np.empty(n, np.uint32)
        dist = np.empty(n, np.float32)
        sums = np.empty((k, d), np.float32)
        counts = np.empty(k, np.uint32)
        self.lib.metalref_kmeans_step(_ptr(x, _f32p), n, d, _ptr(cent, _f32p), k, _ptr(asg, _u32p),
                                      _ptr(dist, _f32p), _ptr(sums, _f32p), _ptr(counts, _u32p))
        return cent, asg.astype(np.int32), dist

    def min_distances(self, x, centroids):
        x, centroids = _f32(x), _f32(centroids)
        out = np.empty(x.shape[0], np.float32)
        self.lib.metalref_min_distances(_ptr(x, _f32p), x.shape[0], x.shape[1], _ptr(centroids, _f32p),
                                        centroids.shape[0], _ptr(out, _f32p))
        return out

    def scalar_quantize(self, x, scale, offset):
        x = _f32(x).ravel()
        out = np.empty(x.size, np.uint8)
        self.lib.metalref_scalar_quantize(_ptr(x, _f32p), _ptr(out, _u8p), scale, offset, x.size)
        return out

    def scalar_dequantize(self, codes, scale, offset):
        codes = np.ascontiguousarray(codes, np.uint8).ravel()
        out = np.empty(codes.size, np.float32)
        self.lib.metalref_scalar_dequantize(_ptr(codes, _u8p), _ptr(out, _f32p), scale, offset, codes.size)
        return out
