"""ctypes binding of ``libvsk_cuda.so`` (``include/vsk_cuda.h``).

There is no CPU implementation behind this package: if the library is missing it must be
built (``python -m vectorstorekit_b200.build``), and opening a context without a B200 raises
``DeviceNotAvailable``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# VSK_CHECKED=1 selects the checked build variant (every global access of every kernel range-tested; see
# ``build.py --checked``).  It is a testing aid: same entry points, several times slower.
CHECKED = os.environ.get("VSK_CHECKED", "0") not in ("", "0")
LIB_PATH = os.path.join(HERE, "libvsk_cuda_checked.so" if CHECKED else "libvsk_cuda.so")

c_f32p = C.POINTER(C.c_float)
c_i64p = C.POINTER(C.c_int64)
c_i32p = C.POINTER(C.c_int32)
c_u64p = C.POINTER(C.c_uint64)
c_i8p = C.POINTER(C.c_int8)
vp = C.c_void_p
DONE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int32)   # vsk_done_fn


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int32), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("hbm_bytes", C.c_int64), ("l2_bytes", C.c_int64), ("max_smem_per_block", C.c_int32),
                ("name", C.c_char * 128)]


class Stats(C.Structure):
    _fields_ = [("searches", C.c_int64), ("queries", C.c_int64), ("kernel_launches", C.c_int64),
                ("tensor_tiles", C.c_int64), ("reranked_rows", C.c_int64), ("fallback_queries", C.c_int64),
                ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64), ("scan_kernel_launches", C.c_int64),
                ("scan_kernel_ms", C.c_double)]


class IndexInfo(C.Structure):
    _fields_ = [("kind", C.c_int32), ("metric", C.c_int32), ("dimensions", C.c_int32), ("nlist", C.c_int32),
                ("count", C.c_int64), ("id_base", C.c_int64), ("has_masks", C.c_int32), ("pq_segments", C.c_int32),
                ("pq_codebook_size", C.c_int32), ("reserved", C.c_int32)]


class Tuning(C.Structure):
    _fields_ = [("fold_row_term", C.c_int32), ("chunk_growth", C.c_int32), ("dense_rows", C.c_int32),
                ("ivf_pilot_tiles", C.c_int32), ("stream_scan", C.c_int32), ("overlap_min_queries", C.c_int32),
                ("wait_limit_log2", C.c_int32), ("test_stall_scan", C.c_int32), ("assign_stages", C.c_int32),
                ("stage_kblocks", C.c_int32), ("reserved", C.c_int32 * 6)]


COMM_ID_BYTES = 128
SHARDED_SLICE, SHARDED_ALL, SHARDED_QUERIES_SPLIT = 0, 1, 16
SHARDED_PHASES = 7

# name -> (restype, argtypes).  Pointers that may be host or device memory are void*.
SIGNATURES = {
    "vsk_open": (C.c_int32, [C.c_int32, C.POINTER(vp)]),
    "vsk_close": (C.c_int32, [vp]),
    "vsk_device_info_get": (C.c_int32, [vp, C.POINTER(DeviceInfo)]),
    "vsk_stats_get": (C.c_int32, [vp, C.POINTER(Stats)]),
    "vsk_last_error": (C.c_char_p, [vp]),
    "vsk_status_string": (C.c_char_p, [C.c_int32]),
    "vsk_set_search_path": (C.c_int32, [vp, C.c_int32]),
    "vsk_stream": (vp, [vp]),
    "vsk_profile": (C.c_int32, [vp, C.c_int32]),
    "vsk_schedule_chunk": (C.c_int64, [C.c_int64, C.c_int32, C.c_int32]),
    "vsk_measure_peak": (C.c_int32, [vp, C.c_int32, C.POINTER(C.c_double)]),
    "vsk_timeline": (C.c_int32, [vp, C.c_int32]),
    "vsk_timeline_read": (C.c_int64, [vp, C.c_char_p, C.c_int64]),
    "vsk_tuning_get": (C.c_int32, [vp, C.POINTER(Tuning)]),
    "vsk_tuning_set": (C.c_int32, [vp, C.POINTER(Tuning)]),
    "vsk_comm_unique_id": (C.c_int32, [vp]),
    "vsk_comm_init": (C.c_int32, [vp, C.c_int32, C.c_int32, vp]),
    "vsk_comm_destroy": (C.c_int32, [vp]),
    "vsk_comm_info": (C.c_int32, [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "vsk_sharded_slice": (None, [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "vsk_search_sharded_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_search_sharded": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_ivf_search_sharded_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_ivf_search_sharded": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_sharded_phase_ms": (C.c_int32, [vp, C.POINTER(C.c_float)]),
    "vsk_coarse_values_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int64, vp, vp]),
    "vsk_batch_distances": (C.c_int32, [vp, C.c_int32, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "vsk_batch_distances_dev": (C.c_int32, [vp, C.c_int32, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "vsk_flat_create": (C.c_int32, [vp, C.c_int32, C.c_int32, C.POINTER(vp)]),
    "vsk_flat_add_f32": (C.c_int32, [vp, vp, C.c_int64, vp]),
    "vsk_flat_add_f32_dev": (C.c_int32, [vp, vp, C.c_int64, vp]),
    "vsk_index_destroy": (C.c_int32, [vp]),
    "vsk_index_size": (C.c_int64, [vp]),
    "vsk_index_set_id_base": (C.c_int32, [vp, C.c_int64]),
    "vsk_index_info_get": (C.c_int32, [vp, C.POINTER(IndexInfo)]),
    "vsk_ivf_centroids": (C.c_int32, [vp, vp]),
    "vsk_kmeans_trainer_create_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.POINTER(vp)]),
    "vsk_kmeans_trainer_step_dev": (C.c_int32, [vp, vp, vp, vp, vp]),
    "vsk_kmeans_trainer_assignments_dev": (C.c_int32, [vp, vp]),
    "vsk_kmeans_trainer_destroy": (C.c_int32, [vp]),
    "vsk_kmeans_finish_dev": (C.c_int32, [vp, vp, vp, vp, C.c_int32, C.c_int32, vp]),
    "vsk_pq_train": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp, vp]),
    "vsk_pq_train_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp, vp]),
    "vsk_pq_encode": (C.c_int32, [vp, vp, C.c_int32, C.c_int32, C.c_int32, vp, C.c_int64, vp]),
    "vsk_pq_encode_dev": (C.c_int32, [vp, vp, C.c_int32, C.c_int32, C.c_int32, vp, C.c_int64, vp]),
    "vsk_pq_decode": (C.c_int32, [vp, vp, C.c_int32, C.c_int32, C.c_int32, vp, C.c_int64, vp]),
    "vsk_pq_distance_tables": (C.c_int32, [vp, vp, C.c_int32, C.c_int32, C.c_int32, vp, C.c_int64, vp]),
    "vsk_pq_index_create": (C.c_int32, [vp, C.c_int32, C.c_int32, C.c_int32, vp, C.POINTER(vp)]),
    "vsk_pq_index_add": (C.c_int32, [vp, vp, C.c_int64]),
    "vsk_pq_index_add_dev": (C.c_int32, [vp, vp, C.c_int64]),
    "vsk_index_image_size": (C.c_int32, [vp, C.POINTER(C.c_int64)]),
    "vsk_index_export": (C.c_int32, [vp, vp, C.c_int64, C.POINTER(C.c_int64)]),
    "vsk_index_import": (C.c_int32, [vp, vp, C.c_int64, C.POINTER(vp)]),
    "vsk_index_save": (C.c_int32, [vp, C.c_char_p]),
    "vsk_index_load": (C.c_int32, [vp, C.c_char_p, C.POINTER(vp)]),
    "vsk_search": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "vsk_search_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "vsk_search_async": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp, DONE_FN, vp]),
    "vsk_search_dev_async": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp, DONE_FN, vp]),
    "vsk_wait": (C.c_int32, [vp]),
    "vsk_checked_build": (C.c_int32, []),
    "vsk_checked_register": (C.c_int32, [vp, C.c_int64]),
    "vsk_checked_unregister": (C.c_int32, [vp]),
    "vsk_checked_faults": (C.c_int32, [vp, vp]),
    "vsk_checked_selftest": (C.c_int32, [vp]),
    "vsk_search_shard_begin_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp]),
    "vsk_search_shard_finish_dev": (C.c_int32, [vp, vp, vp, vp]),
    "vsk_merge_topk_dev": (C.c_int32, [vp, vp, vp, C.c_int32, C.c_int64, C.c_int32, vp, vp]),
    "vsk_kmeans": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_float, vp, vp, vp,
                               C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "vsk_kmeans_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_float, vp, vp, vp,
                                   C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "vsk_kmeans_init_plusplus": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_uint64, vp, vp]),
    "vsk_kmeans_init_plusplus_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_uint64, vp, vp]),
    "vsk_assign_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_assign_static_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int32, vp, vp]),
    "vsk_ivf_build": (C.c_int32, [vp, vp, C.c_int32, vp, C.c_int64, C.c_int32, C.POINTER(vp)]),
    "vsk_ivf_build_dev": (C.c_int32, [vp, vp, C.c_int32, vp, C.c_int64, C.c_int32, C.POINTER(vp)]),
    "vsk_ivf_assignments": (C.c_int32, [vp, vp]),
    "vsk_ivf_search": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp]),
    "vsk_ivf_search_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp]),
    "vsk_ivf_set_masks": (C.c_int32, [vp, vp]),
    "vsk_ivf_set_masks_dev": (C.c_int32, [vp, vp]),
    "vsk_ivf_search_filtered": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp, vp]),
    "vsk_ivf_search_filtered_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp, vp]),
    "vsk_ivf_add": (C.c_int32, [vp, vp, C.c_int64, vp]),
    "vsk_ivf_add_dev": (C.c_int32, [vp, vp, C.c_int64, vp]),
    "vsk_sq8_train": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp]),
    "vsk_sq8_minmax_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp]),
    "vsk_sq8_params_dev": (C.c_int32, [vp, vp, vp, C.c_int32, C.c_int32, vp, vp]),
    "vsk_sq8_encode": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "vsk_sq8_encode_dev": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "vsk_sq8_decode": (C.c_int32, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "vsk_sq8_index_create": (C.c_int32, [vp, C.c_int32, C.c_int32, vp, vp, C.POINTER(vp)]),
    "vsk_sq8_index_add": (C.c_int32, [vp, vp, C.c_int64]),
    "vsk_sq8_index_add_dev": (C.c_int32, [vp, vp, C.c_int64]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library and binds every declared symbol; raises if one is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m vectorstorekit_b200.build{' --checked' if CHECKED else ''}` "
            "(there is no CPU implementation to fall back on)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
