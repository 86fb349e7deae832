"""The reference project's own ctypes wrapper, unmodified, driving this repository's
librsfk.so (python/gpu_rsfk/RSFK.py:100-644 of the reference is the caller of record
of the drop-in boundary).

The file is loaded from the reference tree or from the scratch copy the build leaves
under oracle/_ref.  Two things it needs no longer exist in this environment and are
stood in for inside the test only: ``pkg_resources`` (the wrapper asks it for the
package directory, python/gpu_rsfk/RSFK.py:112) and ``np.int`` (:637-638)."""
import importlib.util
import os
import sys
import types

import numpy as np
import pytest


def _load_reference_wrapper():
    from oracle import rsfk_oracle
    from gpu_rsfk import _lib
    path = rsfk_oracle.reference_wrapper_path()
    if path is None:
        pytest.skip("the reference wrapper is not on this machine (make -C oracle ref_wrapper)")
    shim = types.ModuleType("pkg_resources")
    shim.resource_filename = lambda package, name: os.path.dirname(_lib.LIB_PATH)
    sys.modules["pkg_resources"] = shim
    if not hasattr(np, "int"):
        np.int = int
    spec = importlib.util.spec_from_file_location("reference_rsfk_wrapper", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_wrapper_binds_every_entry_point():
    """Constructing the reference's RSFK class loads ``librsfk`` from the package directory
    and declares the argument types of the three entry points: that must succeed against
    this library (no GPU call is made)."""
    mod = _load_reference_wrapper()
    r = mod.RSFK(random_state=3)
    for name in ("pymodule_rsfk_knn", "pymodule_rsfk_knn_ann", "pymodule_cluster_by_sample_tree"):
        assert getattr(r._lib, name) is not None
    assert len(r._lib.pymodule_rsfk_knn.argtypes) == 14
    assert len(r._lib.pymodule_rsfk_knn_ann.argtypes) == 16
    assert len(r._lib.pymodule_cluster_by_sample_tree.argtypes) == 12


@pytest.mark.gpu
def test_reference_wrapper_smoke_tests_and_small_configuration(oracle):
    """The reference's own ``test1`` (no slot keeps index -1) and ``test2`` (a clustering
    call), then the small plumbing configuration (N=20000, D=32, K=16, 4 trees, 32/128, one
    sweep) through the reference's ``find_nearest_neighbors``: the graph must be the
    oracle pipeline's, bit for bit, and the forest log must parse."""
    mod = _load_reference_wrapper()
    np.random.seed(0)
    mod.test1()
    mod.test2()
    np.random.seed(0)
    X = np.random.uniform(0, 1, (20000, 32)).astype(np.float32)
    r = mod.RSFK(random_state=0)
    idx, dist = r.find_nearest_neighbors(X, 16, n_trees=4, min_tree_children=32, max_tree_children=128,
                                         nn_exploring_factor=1)
    oi, od = oracle.init_lists(20000, 16)
    for t in range(4):
        tr = oracle.build_tree(X, 32, 128, seed=t)
        oi, od = oracle.bucket_knn(X, 16, tr["perm"], tr["leaf_start"], tr["leaf_count"], oi, od)
    oi, od = oracle.explore(X, oi, oi, od)
    np.testing.assert_array_equal(idx, oi)
    np.testing.assert_array_equal(dist.view(np.int32), od.view(np.int32))
    log = r.log_forest.data
    assert len(log["Total Leaves"]) == 4 and min(log["Total Leaves"]) > 0
    assert min(log["Check Points Side Time"]) > 0 and min(log["Bucket Creation Time"]) > 0
    # clustering through the reference wrapper, numpy result format (uses np.int)
    n_leaves, width, buckets, sizes = r.cluster_by_sample_tree(X, min_tree_children=64, max_tree_children=256,
                                                               verbose=0)
    ref = oracle.build_tree(X, 64, 256, seed=0)
    assert n_leaves == len(ref["leaf_count"]) and width == ref["leaf_count"].max()
    np.testing.assert_array_equal(np.asarray(sizes), ref["leaf_count"])
