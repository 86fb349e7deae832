"""GPU k-means against the CPU statement of its rules (oracle/rsfk_oracle.c,
orc_kmeans_*).  Parity is unpinned by nature: the reference has no k-means function,
so the oracle states this repository's own rules; labels, distances and centroids
must agree bit for bit all the same, because both sides fix the order of every
floating-point sum."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _blobs(N, D, C, seed, sigma=1.0):
    rng = np.random.default_rng(seed)
    c = rng.normal(0, 6, (C, D))
    return (c[rng.integers(0, C, N)] + rng.normal(0, sigma, (N, D))).astype(np.float32)


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("N,D,C", [(20000, 16, 8), (6000, 100, 37), (3000, 2, 5), (5000, 33, 300), (2000, 960, 12)])
def test_one_assignment_and_one_update_bit_exact(forest, oracle, N, D, C):
    X = _blobs(N, D, max(2, C // 3), 1)
    rng = np.random.default_rng(2)
    cent = X[np.sort(rng.choice(N, C, replace=False))].copy()
    d_cent = _dev(cent)
    labels, dist, done = forest.kmeans(_dev(X), d_cent, max_iter=0)        # assignment only
    rl, rd = oracle.kmeans_assign(X, cent)
    np.testing.assert_array_equal(labels.cpu().numpy(), rl)
    np.testing.assert_array_equal(dist.cpu().numpy().view(np.int32), rd.view(np.int32))
    assert done == 0
    np.testing.assert_array_equal(d_cent.cpu().numpy(), cent)               # untouched without an iteration
    # one iteration = update from those labels + assignment
    labels, dist, done = forest.kmeans(_dev(X), d_cent, max_iter=1)
    rc, counts = oracle.kmeans_update(X, rl, cent)
    np.testing.assert_array_equal(d_cent.cpu().numpy().view(np.int32), rc.view(np.int32))
    rl2, rd2 = oracle.kmeans_assign(X, rc)
    np.testing.assert_array_equal(labels.cpu().numpy(), rl2)
    np.testing.assert_array_equal(dist.cpu().numpy().view(np.int32), rd2.view(np.int32))


def test_lloyd_iterations_converge_like_the_oracle(forest, oracle):
    N, D, C = 12000, 24, 10
    X = _blobs(N, D, C, 5)
    cent0 = X[:C].copy()
    rc, rl, rd, rit = oracle.kmeans(X, cent0, 40)
    d_cent = _dev(cent0)
    labels, dist, done = forest.kmeans(_dev(X), d_cent, max_iter=40)
    assert done == rit and done < 40                                         # converged, in as many iterations
    np.testing.assert_array_equal(labels.cpu().numpy(), rl)
    np.testing.assert_array_equal(d_cent.cpu().numpy().view(np.int32), rc.view(np.int32))
    np.testing.assert_array_equal(dist.cpu().numpy().view(np.int32), rd.view(np.int32))
    # Lloyd never increases the within-cluster sum of squares
    inertia = []
    c = cent0.copy()
    for it in range(5):
        l, d = oracle.kmeans_assign(X, c)
        inertia.append(float(d.astype(np.float64).sum()))
        c, _ = oracle.kmeans_update(X, l, c)
    assert all(b <= a * (1 + 1e-6) for a, b in zip(inertia, inertia[1:]))


def test_empty_cluster_keeps_its_centroid_and_ties_go_to_the_lower_index(forest, oracle):
    N, D = 4000, 8
    X = _blobs(N, D, 3, 7)
    cent = np.vstack([X[:3], X[0:1], np.full((1, D), 1e6, np.float32)]).astype(np.float32)   # a duplicate and a far one
    d_cent = _dev(cent)
    labels, dist, done = forest.kmeans(_dev(X), d_cent, max_iter=0)        # the assignment alone
    got = labels.cpu().numpy()
    assert (got != 3).all() and (got != 4).all()          # the duplicate (index 3) loses every tie; nobody is near 1e6
    labels, dist, done = forest.kmeans(_dev(X), d_cent, max_iter=3)
    rc, rl, rd, rit = oracle.kmeans(X, cent, 3)
    np.testing.assert_array_equal(labels.cpu().numpy(), rl)
    assert (labels.cpu().numpy() != 4).all()
    np.testing.assert_array_equal(d_cent.cpu().numpy()[4], cent[4])        # never had a member: untouched
    np.testing.assert_array_equal(d_cent.cpu().numpy().view(np.int32), rc.view(np.int32))


def test_kmeans_on_top_of_a_sample_tree_through_the_wrapper(oracle):
    """The drop-in class: the buckets of one sample tree as starting groups, refined by
    Lloyd iterations; and cluster_by_sample_tree itself gives what it gave before."""
    from gpu_rsfk import RSFK
    N, D = 30000, 2
    X = _blobs(N, D, 12, 9, sigma=0.7)
    r = RSFK(random_state=4)
    before = r.cluster_by_sample_tree(X.copy(), min_tree_children=1000, max_tree_children=4000, verbose=0)
    centroids, labels, sq = r.cluster_by_kmeans(X.copy(), init="sample_tree", min_tree_children=1000,
                                                max_tree_children=4000, max_iter=30)
    after = r.cluster_by_sample_tree(X.copy(), min_tree_children=1000, max_tree_children=4000, verbose=0)
    assert before[0] == after[0] and np.array_equal(before[2], after[2]) and np.array_equal(before[3], after[3])
    C = before[0]
    assert centroids.shape == (C, D) and labels.min() >= 0 and labels.max() < C
    # the same run in the oracle: tree buckets -> labels -> Lloyd
    tr = oracle.build_tree(X, 1000, 4000, seed=4)
    lab0 = np.empty(N, np.int32)
    for b, (s, c) in enumerate(zip(tr["leaf_start"], tr["leaf_count"])):
        lab0[tr["perm"][s:s + c]] = b
    rc, rl, rd, rit = oracle.kmeans(X, np.zeros((C, D), np.float32), 30, labels=lab0)
    np.testing.assert_array_equal(labels, rl)
    np.testing.assert_array_equal(centroids.view(np.int32), rc.view(np.int32))
    assert r.n_iter_ == rit
    # refinement can only lower the within-cluster sum of squares of the tree's partition
    c0, _ = oracle.kmeans_update(X, lab0, np.zeros((C, D), np.float32))
    tree_ss = float(((X - c0[lab0]) ** 2).sum())
    assert float(sq.astype(np.float64).sum()) <= tree_ss
    cents2, labels2, _ = r.cluster_by_kmeans(X.copy(), n_clusters=12, init="points", max_iter=50)
    assert cents2.shape == (12, D) and len(np.unique(labels2)) <= 12
