"""Bounded waits that run out, on purpose, without faulting or hanging anything:
a query descent limited to zero steps and a tree level whose host wait is cut to
zero both end with an error status and leave the context usable.  Also: per-tree
calls after a forest that ran on several lanes, and the per-tree rows of the
forest log."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _uniform(N, D, seed=0):
    return np.random.RandomState(seed).uniform(0, 1, (N, D)).astype(np.float32)


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_query_descent_that_runs_out_of_steps_reports_an_error(oracle):
    import torch
    from gpu_rsfk import _lib
    from gpu_rsfk.device import DeviceForest
    f = DeviceForest(torch.device("cuda", 0))
    try:
        N, D = 4000, 24
        X = _uniform(N, D, 1)
        Q = _uniform(500, D, 2)
        f.keep_index(True)
        f.tree_build(_dev(X), 16, 32, seed=3)
        f.set_wait_limits(route_max_steps=0)              # no query can reach a leaf
        with pytest.raises(_lib.RSFKLibraryError):
            f.route_queries(_dev(X), _dev(Q))
        f.set_wait_limits()                               # built-in limits again: the same context works
        qs, qc = f.route_queries(_dev(X), _dev(Q))
        ref = oracle.build_tree_route(X, Q, 16, 32, seed=3) if hasattr(oracle, "build_tree_route") else None
        assert (qc > 0).all() and (qs >= 0).all()
        if ref is not None and "q_start" in ref:
            np.testing.assert_array_equal(qs, ref["q_start"])
    finally:
        f.close()


def test_tree_level_wait_that_runs_out_reports_an_error(oracle):
    import torch
    from gpu_rsfk import _lib
    from gpu_rsfk.device import DeviceForest
    f = DeviceForest(torch.device("cuda", 0))
    try:
        N, D = 20000, 32
        X = _uniform(N, D, 4)
        d_X = _dev(X)
        f.set_wait_limits(level_wait_ms=0)                # the host does not wait for the level mailbox at all
        with pytest.raises(_lib.RSFKLibraryError):
            f.tree_build(d_X, 32, 128, seed=0)
        f.set_wait_limits()
        info = f.tree_build(d_X, 32, 128, seed=0)         # nothing was left in flight: same buckets as the oracle
        perm, ls, lc = f.tree_export()
        ref = oracle.build_tree(X, 32, 128, seed=0)
        np.testing.assert_array_equal(perm, ref["perm"])
        np.testing.assert_array_equal(lc, ref["leaf_count"])
        assert info["n_leaves"] == len(ref["leaf_count"])
    finally:
        f.close()


def test_per_tree_calls_after_a_forest_on_lanes(oracle):
    """A forest on three lanes leaves the first lane's last tree in the context; a
    query update that follows must descend that tree with that tree's hyperplanes,
    not with those of a tree the context routed through before."""
    import torch
    from gpu_rsfk.device import DeviceForest
    f = DeviceForest(torch.device("cuda", 0))
    try:
        N, NQ, D, K, T = 5000, 1200, 20, 8, 6
        X, Q = _uniform(N, D, 5), _uniform(NQ, D, 6)
        d_X, d_Q = _dev(X), _dev(Q)
        f.keep_index(True)
        f.tree_build(d_X, 16, 32, seed=99)
        f.route_queries(d_X, d_Q)                          # hyperplanes of tree 99 are now materialised
        f.set_lanes(3)
        idx, dist = f.init_lists(NQ, K, d_X.device, self_in_row=False)
        f.forest_ann(d_X, d_Q, idx, dist, T, 16, 32, seed=10)
        f.set_lanes(0)
        # lane 0 built trees 10, 13: the context now holds tree 13
        f.ann_bucket_knn(d_X, d_Q, idx, dist)              # once more into the same lists: no change
        f.synchronize()
        ri, rd = oracle.ann_forest(X, Q, K, T, 16, 32, seed=10)
        np.testing.assert_array_equal(idx.cpu().numpy(), ri)
        np.testing.assert_array_equal(dist.cpu().numpy().view(np.int32), rd.view(np.int32))
        # and a forest on lanes keeps the index when the caller asked for it
        f.set_lanes(2)
        gi, gd = f.init_lists(N, K, d_X.device)
        f.forest(d_X, gi, gd, 4, 16, 32, seed=30)
        f.set_lanes(0)
        qs, qc = f.route_queries(d_X, d_Q)
        assert (qc >= 16).all()
    finally:
        f.close()


@pytest.mark.parametrize("lanes", [1, 3])
def test_forest_log_rows_are_filled(forest, lanes):
    """Every per-tree attribute that has a counterpart in this implementation is written
    (seconds; the attribute order is the reference wrapper's, python/gpu_rsfk/RSFK.py:71-88)."""
    N, D, K, T = 30000, 32, 16, 6
    X = _uniform(N, D, 7)
    d_X = _dev(X)
    idx, dist = forest.init_lists(N, K, d_X.device)
    forest.set_lanes(lanes)
    try:
        log = forest.forest(d_X, idx, dist, T, 17, 34, seed=1, want_log=True)
    finally:
        forest.set_lanes(0)
    row = lambda a: log[a * T:(a + 1) * T]
    for a in (0, 1, 2, 3):
        assert (row(a) > 0).all()
    assert (row(2) >= 17).all() and (row(1) <= 34).all()
    for a in (4, 5, 7, 8, 12, 13, 14, 15):                 # init, build, check side, count, update, buckets, end, KNN
        assert (row(a) > 0).all(), a
    assert (row(7) < row(5)).all()                          # a part is smaller than the whole
    assert log[16 * T] > 0
