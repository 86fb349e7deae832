"""The allocation-free sweep entry point, through the C ABI.

Some hosts may not allocate device memory where the sweep runs (all of it was
handed to their own arena at start-up, or cudaMalloc's device-wide
synchronisation is not allowed there).  ``rsfk_explore_sweep_static`` serves
them from a fixed buffer inside the library.  It must give exactly what the
regular entry point gives from a caller-made snapshot -- also on a second call,
when the built-in buffer still holds the first call's data -- and must refuse
problems larger than that buffer.

This file sorts last so that a run stopping at the first failure has already
executed every other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _lists_after_trees(oracle, X, K, trees):
    idx, dist = oracle.init_lists(len(X), K)
    for t in range(trees):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    return idx, dist


def test_static_sweep_matches_regular_entry_point_twice(forest, oracle):
    import torch
    from gpu_rsfk import _lib
    L = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (N, D, K) in enumerate([(9000, 40, 24), (5000, 100, 32)]):
        X = np.random.RandomState(30 + call).uniform(0, 1, (N, D)).astype(np.float32)
        idx, dist = _lists_after_trees(oracle, X, K, 2)
        d_X = torch.from_numpy(X).cuda()
        # regular entry point: caller-provided snapshot
        ref_i, ref_d = torch.from_numpy(idx).cuda(), torch.from_numpy(dist).cuda()
        forest.explore(d_X, ref_i.clone(), ref_i, ref_d)
        # allocation-free entry point: in place
        new_i, new_d = torch.from_numpy(idx).cuda(), torch.from_numpy(dist).cuda()
        code = L.rsfk_explore_sweep_static(ctypes.c_void_p(d_X.data_ptr()), N, D, K,
                                           ctypes.c_void_p(new_i.data_ptr()),
                                           ctypes.c_void_p(new_d.data_ptr()), stream)
        assert code == 0
        torch.cuda.synchronize()
        # integer and distance results are bit-exact (tolerance 0, as in the other parity tests)
        np.testing.assert_array_equal(new_i.cpu().numpy(), ref_i.cpu().numpy())
        np.testing.assert_array_equal(new_d.cpu().numpy(), ref_d.cpu().numpy())
        assert not np.array_equal(new_i.cpu().numpy(), idx)          # the sweep did change rows


def test_static_sweep_rejects_oversized_problems():
    import torch
    from gpu_rsfk import _lib
    L = _lib.load()
    K = 64
    N = (4 * 1024 * 1024) // K + 1                                   # one row beyond the built-in capacity
    dummy = torch.zeros(16, device="cuda")
    p = ctypes.c_void_p(dummy.data_ptr())
    assert L.rsfk_explore_sweep_static(p, N, 4, K, p, p, None) == 2  # refused before touching memory
    assert L.rsfk_explore_sweep_static(p, 100, 4, 300, p, p, None) == 3
