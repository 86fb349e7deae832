"""Many small random shapes, GPU against the oracle bit for bit: trees (with
coincident points and a low depth limit), bucket KNN, one sweep, and the query
path.  The shapes come from a fixed seed, so a failure names its case."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for c in range(n):
        N = int(rng.choice([1, 2, 3, 17, 33, 64, 100, 257, 700, 1500, 4000]))
        D = int(rng.choice([1, 2, 3, 4, 7, 8, 15, 16, 17, 31, 32, 33, 63, 64, 100, 129]))
        K = int(rng.choice([1, 2, 5, 16, 31, 32, 33, 64, 65, 100]))
        MIN = int(rng.choice([1, 2, 5, 9, 17, 33, 60]))
        MAX = 2 * MIN + int(rng.integers(0, 2 * MIN + 3))
        out.append((c, N, D, K, MIN, MAX, bool(rng.integers(0, 2)), int(rng.choice([6, 12, 5000]))))
    return out


def _data(c, N, D, repeats):
    rng = np.random.default_rng(1000 + c)
    X = rng.uniform(0, 1, (N, D)).astype(np.float32)
    if repeats and N > 3:
        X[rng.integers(0, N, N // 3)] = X[0]
    return X


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("c,N,D,K,MIN,MAX,repeats,depth", _cases(48, 7))
def test_random_shape_matches_oracle(forest, oracle, c, N, D, K, MIN, MAX, repeats, depth):
    import torch
    X = _data(c, N, D, repeats)
    NQ = max(1, N // 3)
    Q = np.random.default_rng(2000 + c).uniform(0, 1, (NQ, D)).astype(np.float32)
    dX, dQ = _dev(X), _dev(Q)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist = _dev(idx), _dev(dist)
    qi, qd = oracle.init_lists(NQ, K, self_in_row=False)
    d_qi, d_qd = _dev(qi), _dev(qd)
    forest.keep_index(True)
    try:
        for t in range(2):
            ref = oracle.build_tree_route(X, Q, MIN, MAX, max_depth=depth, seed=c + t)
            info = forest.tree_build(dX, MIN, MAX, max_depth=depth, seed=c + t)
            perm, ls, lc = forest.tree_export()
            np.testing.assert_array_equal(perm, ref["perm"])
            np.testing.assert_array_equal(ls, ref["leaf_start"])
            np.testing.assert_array_equal(lc, ref["leaf_count"])
            qs, qc = forest.route_queries(dX, dQ)
            np.testing.assert_array_equal(qs, ref["q_start"])
            np.testing.assert_array_equal(qc, ref["q_count"])
            idx, dist = oracle.bucket_knn(X, K, ref["perm"], ref["leaf_start"], ref["leaf_count"], idx, dist)
            forest.bucket_knn(dX, d_idx, d_dist)
            qi, qd = oracle.ann_bucket_knn(X, Q, K, ref["perm"], ref["q_start"], ref["q_count"], qi, qd)
            forest.ann_bucket_knn(dX, dQ, d_qi, d_qd)
            assert info["n_leaves"] == len(ls)
    finally:
        forest.keep_index(False)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
    np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
    np.testing.assert_array_equal(d_qi.cpu().numpy(), qi)
    np.testing.assert_array_equal(d_qd.cpu().numpy().view(np.int32), qd.view(np.int32))
    idx, dist = oracle.explore(X, idx, idx, dist)
    forest.explore(dX, d_idx.clone(), d_idx, d_dist)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
    np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
