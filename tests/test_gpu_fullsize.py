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


def test_full_size_query_search_properties(forest, oracle):
    """The query search at the size of its bench line (1.5 M base points x 32, as many
    queries, K = 32, buckets of 32..256), through properties that need no oracle run:
    a query that is a base point finds itself first at distance 0 and ends in its own
    bucket; rows are ordered, distinct, in range, with exact distances; a second forest
    only improves the rows; recall against exact search on a seeded subsample."""
    import torch
    NB, DQ, KQ = 1_500_000, 32, 32
    rng = np.random.default_rng(4)
    c = rng.normal(0, 1, (200, DQ)) / np.sqrt(1.0 + np.arange(DQ))
    X = (c[rng.integers(0, 200, NB)] + rng.normal(0, 0.5, (NB, DQ)) / np.sqrt(1.0 + np.arange(DQ))).astype(np.float32)
    d_X = torch.from_numpy(X).cuda()
    forest.keep_index(True)
    try:
        forest.tree_build(d_X, 32, 256, seed=9)
        perm, ls, lc = forest.tree_export()
        qs, qc = forest.route_queries(d_X, d_X)
    finally:
        forest.keep_index(False)
    own = np.empty(NB, np.int32)
    own[perm] = np.repeat(ls, lc)
    np.testing.assert_array_equal(qs, own)                                        # own bucket
    assert qc.min() >= 32 and qc.max() <= 256

    idx, dist = forest.init_lists(NB, KQ, d_X.device, self_in_row=False)
    forest.forest_ann(d_X, d_X, idx, dist, 5, 32, 256, seed=0)
    h_idx, h_dist = idx.cpu().numpy(), dist.cpu().numpy()
    assert (h_dist[:, 0] == 0).all()                                              # itself (or a twin) first
    assert (h_idx >= 0).all() and (h_idx < NB).all()                              # buckets >= 32 = K: rows full
    assert (np.diff(h_dist, axis=1) >= 0).all()
    assert (np.diff(np.sort(h_idx, axis=1), axis=1) > 0).all()
    for p in rng.integers(0, NB, 200):
        for k in (1, KQ // 2, KQ - 1):
            assert np.float32(oracle.dist_sqr(X[p], X[h_idx[p, k]])) == h_dist[p, k]
    before = dist.clone()
    forest.forest_ann(d_X, d_X, idx, dist, 3, 32, 256, seed=100)
    assert bool((dist <= before).all())                                           # more trees never worsen a row
    rows = np.sort(rng.choice(NB, 500, replace=False))
    q = d_X[torch.as_tensor(rows, device=d_X.device)]
    d2 = (d_X * d_X).sum(1)[None, :] - 2.0 * (q @ d_X.T)
    truth = d2.topk(KQ, dim=1, largest=False).indices.cpu().numpy()
    rec = oracle.recall(truth.astype(np.int32), idx[torch.as_tensor(rows, device=d_X.device)].cpu().numpy())
    assert rec > 0.6, rec
