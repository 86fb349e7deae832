"""Full-size runs (the headline shape: 1 000 000 x 100, K=32) checked through
size-independent properties, since the CPU oracle cannot finish them in
seconds: permutation and leaf-size invariants of a tree, sorted canonical rows,
distances that equal an exact recomputation, idempotence of the bucket update,
monotone improvement by a sweep, and recall against exact KNN on a seeded
subsample of queries."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, D, K, MIN, MAX = 1_000_000, 100, 32, 33, 66


@pytest.fixture(scope="module")
def points():
    import torch
    np.random.seed(0)
    X = np.random.uniform(0, 1, (N, D)).astype(np.float32)
    return X, torch.from_numpy(X).cuda()


def test_full_size_tree_invariants(forest, points):
    X, d_X = points
    info = forest.tree_build(d_X, MIN, MAX, seed=5)
    perm, ls, lc = forest.tree_export()
    assert lc.sum() == N and info["n_leaves"] == len(ls)
    np.testing.assert_array_equal(ls, np.cumsum(lc) - lc)             # leaves tile [0, N)
    assert lc.min() >= MIN and lc.max() <= MAX
    assert np.array_equal(np.sort(perm), np.arange(N, dtype=np.int32))  # every point exactly once
    # same seed, same tree; another seed, another tree
    forest.tree_build(d_X, MIN, MAX, seed=5)
    perm2, _, _ = forest.tree_export()
    np.testing.assert_array_equal(perm, perm2)
    forest.tree_build(d_X, MIN, MAX, seed=6)
    perm3, _, _ = forest.tree_export()
    assert not np.array_equal(perm, perm3)


def test_full_size_graph_properties(forest, points, oracle):
    import torch
    X, d_X = points
    idx, dist = forest.init_lists(N, K, d_X.device)
    forest.forest(d_X, idx, dist, 6, MIN, MAX, seed=0)
    h_idx, h_dist = idx.cpu().numpy(), dist.cpu().numpy()
    assert (h_idx[:, 0] == np.arange(N)).all() and (h_dist[:, 0] == 0).all()      # self first
    assert (h_idx >= 0).all() and (h_idx < N).all()                               # min >= K+1: no empty slot
    assert (np.diff(h_dist, axis=1) >= 0).all()                                   # rows ordered by distance
    srt = np.sort(h_idx, axis=1)
    assert (np.diff(srt, axis=1) > 0).all()                                       # distinct indices per row
    rng = np.random.default_rng(1)
    for p in rng.integers(0, N, 300):                                             # stored distances are exact
        for k in (1, K // 2, K - 1):
            assert np.float32(oracle.dist_sqr(X[p], X[h_idx[p, k]])) == h_dist[p, k]

    # idempotence: the same tree's buckets applied twice change nothing
    forest.tree_build(d_X, MIN, MAX, seed=3)
    forest.bucket_knn(d_X, idx, dist)
    once_i, once_d = idx.clone(), dist.clone()
    forest.bucket_knn(d_X, idx, dist)
    assert torch.equal(idx, once_i) and torch.equal(dist, once_d)

    # a sweep never worsens any slot, and a second sweep from the same snapshot is a no-op
    before = dist.clone()
    snap = idx.clone()
    forest.explore(d_X, snap, idx, dist)
    assert bool((dist <= before).all())
    again_i, again_d = idx.clone(), dist.clone()
    forest.explore(d_X, snap, idx, dist)
    assert torch.equal(idx, again_i) and torch.equal(dist, again_d)

    # recall on a seeded query subsample against exact brute force (CPU oracle, 200 rows)
    q = np.sort(np.random.default_rng(1000).choice(N, 200, replace=False)).astype(np.int32)
    ti, td, _ = oracle.bruteforce_knn(X, K, q)
    rec = oracle.recall(ti, idx.cpu().numpy()[q])
    assert 0.01 < rec <= 1.0
    # every reported neighbour is at least as far as the exact k-th neighbour
    assert (idx.cpu().numpy()[q][:, 0] == q).all()
    assert (dist.cpu().numpy()[q] >= td - 1e-5 * td).all()                        # 1e-5 relative
