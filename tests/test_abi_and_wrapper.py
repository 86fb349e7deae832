"""Host-side checks that need no GPU: the C-ABI library loads and exports every
symbol the header declares; the drop-in Python class validates arguments and
parses the forest log like the reference wrapper."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rsfk_b200.h")).read()
    return re.findall(r"RSFK_EXPORT\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    from gpu_rsfk import _lib
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 20
    for required in ("pymodule_rsfk_knn", "pymodule_cluster_by_sample_tree", "pymodule_rsfk_knn_ann"):
        assert required in names
    for name in names:
        assert hasattr(L, name), name


def test_library_is_named_and_placed_like_the_reference():
    from gpu_rsfk import _lib
    assert os.path.basename(_lib.LIB_PATH) == "librsfk.so"
    assert os.path.dirname(_lib.LIB_PATH) == os.path.dirname(os.path.abspath(_lib.__file__))


def test_status_entry_points_without_a_gpu():
    from gpu_rsfk import _lib
    L = _lib.load()
    assert L.rsfk_max_neighbors() == 256
    assert L.rsfk_kernel_launches() >= 0
    assert isinstance(L.rsfk_last_message(), bytes)
    L.rsfk_free(None)


def test_device_list_arguments_without_a_gpu():
    """rsfk_set_devices: an empty list (back to one GPU) needs no device; impossible lists are refused."""
    import gpu_rsfk
    from gpu_rsfk import _lib
    L = _lib.load()
    assert L.rsfk_set_devices(0, None) == 0
    gpu_rsfk.set_devices(None)
    gpu_rsfk.set_devices([])
    three = (ctypes.c_int * 3)(0, 1, 2)
    assert L.rsfk_set_devices(-1, three) == 2           # invalid argument
    assert L.rsfk_set_devices(9, three) == 2
    assert L.rsfk_set_devices(3, None) == 2
    many = (ctypes.c_int * 2)(0, 1000)
    assert L.rsfk_set_devices(2, many) == 2             # no such device (or no device at all)
    with pytest.raises(ValueError):
        gpu_rsfk.set_devices([0, 1000])
    assert L.rsfk_set_devices(0, None) == 0


def test_ann_entry_point_refuses_null_buffers():
    from gpu_rsfk import _lib
    _lib.load()
    raw = ctypes.CDLL(_lib.LIB_PATH)  # no prototypes: NULL buffers reach the library
    raw.pymodule_rsfk_knn_ann(*([ctypes.c_int(0)] * 11 + [None] * 5))
    # 2 = invalid argument; 1 = no CUDA device, which a box without a GPU reports first
    assert raw.rsfk_last_status() in (1, 2)


def test_ann_wrapper_argument_validation():
    from gpu_rsfk import RSFK
    r = RSFK()
    X, Q = np.zeros((10, 3), np.float32), np.zeros((4, 3), np.float32)
    with pytest.raises(Exception, match="max_tree_children must be at least 2\\*min_tree_children"):
        r.find_nearest_neighbors_ann(X, Q, 4, min_tree_children=8, max_tree_children=9)
    with pytest.raises(Exception, match="same number of dimensions"):
        r.find_nearest_neighbors_ann(X, np.zeros((4, 5), np.float32), 4)


def test_wrapper_argument_validation_matches_reference():
    from gpu_rsfk import RSFK
    r = RSFK(random_state=3)
    assert r.random_state == 3
    X = np.zeros((10, 3), np.float32)
    with pytest.raises(Exception, match="max_tree_children must be at least 2\\*min_tree_children"):
        r.find_nearest_neighbors(X, 4, min_tree_children=8, max_tree_children=9)
    with pytest.raises(Exception, match="min_tree_children must be at least 1"):
        r.find_nearest_neighbors(X, 4, min_tree_children=-5, max_tree_children=10)
    with pytest.raises(Exception, match="max_tree_children must be at least"):
        r.cluster_by_sample_tree(X, min_tree_children=32, max_tree_children=40)


def test_forest_log_layout():
    from gpu_rsfk import ForestLog
    T = 3
    data = np.arange(16 * T + 2, dtype=np.float32)
    log = ForestLog(data)
    assert log.data["Tree Depth"] == [0, 1, 2]
    assert log.data["Total Leaves"] == [9, 10, 11]
    assert list(log.data["KNN Sets Updates"]) == [45.0, 46.0, 47.0]
    assert len(log.data) == 16
    assert log.total_forest_time == 48.0 and log.exploration_time == 49.0


def test_random_motion_moves_points_slightly():
    from gpu_rsfk import random_motion
    np.random.seed(0)
    X = np.random.rand(100, 4)
    Y = X.copy()
    random_motion(Y, 1.0)
    assert (Y != X).any() and np.abs(Y - X).max() <= 1.0 / 100 + 1e-12


def test_no_gpu_means_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from gpu_rsfk import RSFK, RSFKLibraryError
    with pytest.raises(RSFKLibraryError):
        RSFK().find_nearest_neighbors(np.random.rand(50, 4).astype(np.float32), 3, n_trees=1)
    with pytest.raises(RSFKLibraryError):
        RSFK().find_nearest_neighbors_ann(np.random.rand(50, 4).astype(np.float32),
                                          np.random.rand(5, 4).astype(np.float32), 3, n_trees=1)
    from gpu_rsfk.device import DeviceForest
    with pytest.raises(RSFKLibraryError):
        DeviceForest()


def test_bench_names_the_larger_kernel_when_two_phases_tie():
    """bench.py's roofline names the phase with the most kernel time; phases within 2 % count as tied
    and the one with the fewest launches wins, so the line does not flip between runs."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("rsfk_bench_for_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    phases = {"bucket_knn": {"total_ms": 59.0, "launches": 50.0}, "tree_project": {"total_ms": 66.2, "launches": 753.0},
              "tree_level_rest": {"total_ms": 99.0, "launches": 753.0}, "explore": {"total_ms": 66.0, "launches": 1}}
    assert bench.dominant_phase(phases) == "explore"
    phases["explore"]["total_ms"] = 60.0
    assert bench.dominant_phase(phases) == "tree_project"
