"""Loads ``librsfk.so`` (the sm_100a build) and declares its C ABI.

The library is a required part of the package: there is no Python or CPU
fallback, and a missing library is an ImportError-like hard failure.
"""
import ctypes
import os

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_DIR, "librsfk.so")

STATUS_NAMES = {0: "ok", 1: "cuda error", 2: "invalid argument", 3: "unsupported",
                4: "internal table overflow", 5: "out of memory"}

_c_int_p = ctypes.POINTER(ctypes.c_int)
_lib = None


class RSFKLibraryError(RuntimeError):
    """The native library reported a failure (see ``rsfk_last_status``)."""


def load():
    """Returns the ctypes handle of librsfk.so with every prototype declared."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RSFKLibraryError(
            "librsfk.so is missing from %s; build it with `python gpu-rsfk_b200/build.py` "
            "(there is no CPU fallback)" % _DIR)
    L = np.ctypeslib.load_library("librsfk", _DIR)
    i, f, vp, ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

    L.pymodule_rsfk_knn.restype = None
    L.pymodule_rsfk_knn.argtypes = [i] * 10 + [
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
        np.ctypeslib.ndpointer(np.int32, ndim=2, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.float32, ndim=1, flags="ALIGNED, CONTIGUOUS, WRITEABLE")]
    L.pymodule_cluster_by_sample_tree.restype = None
    L.pymodule_cluster_by_sample_tree.argtypes = [i] * 7 + [
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
        ctypes.POINTER(_c_int_p), ctypes.POINTER(_c_int_p), _c_int_p, _c_int_p]
    L.pymodule_rsfk_knn_ann.restype = None
    L.pymodule_rsfk_knn_ann.argtypes = [i] * 11 + [
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
        np.ctypeslib.ndpointer(np.int32, ndim=2, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.float32, ndim=1, flags="ALIGNED, CONTIGUOUS, WRITEABLE")]

    L.rsfk_kmeans.restype = None
    L.rsfk_kmeans.argtypes = [i] * 5 + [
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
        np.ctypeslib.ndpointer(np.float32, ndim=2, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.int32, ndim=1, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        np.ctypeslib.ndpointer(np.float32, ndim=1, flags="ALIGNED, CONTIGUOUS, WRITEABLE"),
        _c_int_p]

    L.rsfk_last_status.restype = i
    L.rsfk_last_status.argtypes = []
    L.rsfk_last_message.restype = ctypes.c_char_p
    L.rsfk_last_message.argtypes = []
    L.rsfk_free.restype = None
    L.rsfk_free.argtypes = [vp]
    L.rsfk_kernel_launches.restype = ll
    L.rsfk_kernel_launches.argtypes = []
    L.rsfk_release_memory.restype = None
    L.rsfk_release_memory.argtypes = []
    L.rsfk_max_neighbors.restype = i
    L.rsfk_max_neighbors.argtypes = []
    L.rsfk_set_devices.restype = i
    L.rsfk_set_devices.argtypes = [i, _c_int_p]

    L.rsfk_ctx_create.restype = vp
    L.rsfk_ctx_create.argtypes = [i, vp]
    L.rsfk_ctx_destroy.restype = None
    L.rsfk_ctx_destroy.argtypes = [vp]
    L.rsfk_ctx_status.restype = i
    L.rsfk_ctx_status.argtypes = [vp]
    L.rsfk_ctx_synchronize.restype = i
    L.rsfk_ctx_synchronize.argtypes = [vp]
    L.rsfk_ctx_stats.restype = i
    L.rsfk_ctx_stats.argtypes = [vp, ctypes.POINTER(ctypes.c_double), i]
    L.rsfk_dev_sort_rows.restype = i
    L.rsfk_dev_sort_rows.argtypes = [vp, vp, vp, ll, i]
    L.rsfk_dev_tree_build.restype = i
    L.rsfk_dev_tree_build.argtypes = [vp, vp, i, i, i, i, i, i, vp, i, _c_int_p, _c_int_p, _c_int_p, _c_int_p]
    L.rsfk_dev_tree_export.restype = i
    L.rsfk_dev_tree_export.argtypes = [vp, i, vp, vp, vp]
    L.rsfk_dev_bucket_knn.restype = i
    L.rsfk_dev_bucket_knn.argtypes = [vp, vp, i, i, i, vp, vp]
    L.rsfk_dev_bucket_knn_table.restype = i
    L.rsfk_dev_bucket_knn_table.argtypes = [vp, vp, i, i, i, vp, vp, vp, i, i, vp, vp]
    L.rsfk_dev_forest.restype = i
    L.rsfk_dev_forest.argtypes = [vp, vp, i, i, i, i, i, i, i, i, i, i, vp, vp, vp]
    L.rsfk_dev_explore.restype = i
    L.rsfk_dev_explore.argtypes = [vp, vp, i, i, i, vp, vp, vp, i, i, i]
    L.rsfk_dev_merge_lists.restype = i
    L.rsfk_dev_merge_lists.argtypes = [vp, ll, i, i, vp, vp, vp, vp]
    L.rsfk_ctx_set_lanes.restype = i
    L.rsfk_ctx_set_lanes.argtypes = [vp, i]
    L.rsfk_ctx_set_tc.restype = i
    L.rsfk_ctx_set_tc.argtypes = [vp, i]
    L.rsfk_ctx_set_wait_limits.restype = i
    L.rsfk_ctx_set_wait_limits.argtypes = [vp, i, i]
    L.rsfk_ctx_keep_index.restype = i
    L.rsfk_ctx_keep_index.argtypes = [vp, i]
    L.rsfk_dev_route_queries.restype = i
    L.rsfk_dev_route_queries.argtypes = [vp, vp, i, i, vp, i, vp, vp]
    L.rsfk_dev_ann_bucket_knn.restype = i
    L.rsfk_dev_ann_bucket_knn.argtypes = [vp, vp, i, vp, i, i, i, vp, vp]
    L.rsfk_dev_forest_ann.restype = i
    L.rsfk_dev_forest_ann.argtypes = [vp, vp, i, vp, i, i, i, i, i, i, i, i, i, i, vp, vp]
    L.rsfk_dev_symmetrize_count.restype = i
    L.rsfk_dev_symmetrize_count.argtypes = [vp, i, i, vp, vp, ctypes.POINTER(ll)]
    L.rsfk_dev_symmetrize_fill.restype = i
    L.rsfk_dev_symmetrize_fill.argtypes = [vp, i, i, vp, vp, vp, vp, vp]
    L.rsfk_dev_kmeans.restype = i
    L.rsfk_dev_kmeans.argtypes = [vp, vp, i, i, i, i, i, vp, vp, vp, _c_int_p]
    L.rsfk_explore_sweep_static.restype = i
    L.rsfk_explore_sweep_static.argtypes = [vp, i, i, i, vp, vp, vp]
    _lib = L
    return L


def raise_on_status(code, what):
    if code != 0:
        raise RSFKLibraryError("%s failed: %s (status %d)" % (what, STATUS_NAMES.get(code, "?"), code))


def check_last(what):
    L = load()
    code = L.rsfk_last_status()
    if code != 0:
        msg = L.rsfk_last_message().decode("utf-8", "replace")
        raise RSFKLibraryError("%s failed: %s (status %d)" % (what, msg, code))
