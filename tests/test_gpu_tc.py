"""The tensor-core (tcgen05) bucket kernel against the CPU oracle, through the C ABI.

The Gram value only filters; stored indices and distances must be the oracle's,
bit for bit.  Every test forces the tensor-core kernel with ``set_tc(1)`` and
asserts through the context's counters that it was the kernel launched."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _uniform(N, D, seed=0):
    return np.random.RandomState(seed).uniform(0, 1, (N, D)).astype(np.float32)


def _clustered(N, D, seed, centers=12, sigma=0.4):
    rng = np.random.default_rng(seed)
    c = rng.normal(0, 1, (centers, D))
    return (c[rng.integers(0, centers, N)] + rng.normal(0, sigma, (N, D))).astype(np.float32)


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture()
def tc_forest(forest):
    forest.set_tc(1)
    yield forest
    forest.set_tc(-1)


def _run_trees(forest, oracle, X, K, MIN, MAX, trees, seed0=50, max_leaf_limit=None):
    N = len(X)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist, d_X = _dev(idx), _dev(dist), _dev(X)
    before = forest.stats()
    for t in range(trees):
        tr = oracle.build_tree(X, MIN, MAX, seed=seed0 + t)
        if max_leaf_limit is not None:
            assert tr["leaf_count"].max() <= max_leaf_limit
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
        forest.bucket_knn_table(d_X, _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                                int(tr["leaf_count"].max()), d_idx, d_dist)
        forest.synchronize()
        np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
        np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
    after = forest.stats()
    assert after["tc_launches"] - before["tc_launches"] == trees      # the tensor-core kernel ran
    return after["tc_pairs_passed"] - before["tc_pairs_passed"], after["tc_pairs_seen"] - before["tc_pairs_seen"]


TC_CASES = [
    # N, D, K, MIN, MAX  -- D >= 64, leaves of at most 128 points: one tile, one column group
    (6000, 100, 32, 33, 66),
    (5000, 128, 16, 40, 128),
    (4000, 64, 8, 9, 18),
    (3000, 200, 30, 31, 128),
    (2500, 99, 20, 21, 42),        # D not a multiple of 4
    (2000, 960, 32, 33, 100),
    (3000, 72, 64, 60, 128),       # lists longer than some buckets: empty slots survive
]


@pytest.mark.parametrize("N,D,K,MIN,MAX", TC_CASES)
def test_small_leaves_on_tensor_cores_bit_exact(tc_forest, oracle, N, D, K, MIN, MAX):
    X = _clustered(N, D, 17) if D != 100 else _uniform(N, D, 17)
    _run_trees(tc_forest, oracle, X, K, MIN, MAX, trees=4, max_leaf_limit=128)


@pytest.mark.parametrize("N,D,K,MIN,MAX", [(6000, 300, 32, 500, 1500), (5000, 96, 16, 300, 700)])
def test_multi_tile_leaves_bit_exact(tc_forest, oracle, N, D, K, MIN, MAX):
    """Leaves of several 128-row tiles and several 256-column groups."""
    X = _uniform(N, D, 9)
    _run_trees(tc_forest, oracle, X, K, MIN, MAX, trees=3, seed0=4)


@pytest.mark.parametrize("D", [64, 960])
def test_one_leaf_of_2048_points(tc_forest, oracle, D):
    """The largest leaf the kernel takes: 16 tiles, 8 column groups, every pass word in use."""
    N, K = 2048, 32
    X = _clustered(N, D, 23, centers=3, sigma=0.3)
    rng = np.random.default_rng(5)
    perm = rng.permutation(N).astype(np.int32)
    ls, lc = np.array([0], np.int32), np.array([N], np.int32)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist = _dev(idx), _dev(dist)
    before = tc_forest.stats()
    for _ in range(2):        # second pass: lists are full, the filter has a threshold everywhere
        idx, dist = oracle.bucket_knn(X, K, perm, ls, lc, idx, dist)
        tc_forest.bucket_knn_table(_dev(X), _dev(perm), _dev(ls), _dev(lc), N, d_idx, d_dist)
        tc_forest.synchronize()
        np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
        np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
    assert tc_forest.stats()["tc_launches"] - before["tc_launches"] == 2


def test_integer_valued_points_with_ties(tc_forest, oracle):
    """Integer coordinates in [0, 255] around cluster centres (the shape of the 20 M-point
    configuration): squared distances are exact integers and tie often; ties go to the
    lower index on both sides."""
    rng = np.random.default_rng(3)
    N, D, K = 6000, 128, 64
    c = rng.integers(0, 256, (20, D)).astype(np.float32)
    X = np.clip(np.rint(c[rng.integers(0, 20, N)] + rng.normal(0, 12, (N, D))), 0, 255).astype(np.float32)
    X[1::2] = X[::2]                                         # coincident pairs: distance 0 ties
    X += (rng.integers(0, 2, (N, 1)) * 1.0).astype(np.float32)   # keep some pairs apart by exactly 1 per dimension
    _run_trees(tc_forest, oracle, X, K, 65, 130, trees=3, seed0=7)


@pytest.mark.parametrize("kind", ["offset", "mixed", "scaled"])
def test_filter_margin_on_hard_magnitudes(tc_forest, oracle, kind):
    """Data on which an uncentred Gram distance cancels badly: a large common offset,
    coordinates of very different magnitudes, tiny overall scale."""
    N, D, K = 5000, 160, 24
    X = _clustered(N, D, 31, centers=8, sigma=0.2)
    if kind == "offset":
        X = (X + np.float32(1000.0)).astype(np.float32)
    elif kind == "mixed":
        scale = np.where(np.arange(D) % 5 == 0, 300.0, 0.01).astype(np.float32)
        X = (X * scale).astype(np.float32)
    else:
        X = (X * np.float32(1e-12)).astype(np.float32)
    passed, seen = _run_trees(tc_forest, oracle, X, K, 200, 600, trees=4, seed0=11)
    assert seen > 0


def test_filter_passes_a_small_share_once_lists_are_full(tc_forest, oracle):
    """The point of the Gram filter: with full lists only a small share of the pairs goes
    on to the exact evaluation (a margin that lets everything through would still give the
    right lists, as a slow SIMT kernel)."""
    N, D, K = 8000, 128, 16
    X = _clustered(N, D, 41, centers=6, sigma=0.5)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist, d_X = _dev(idx), _dev(dist), _dev(X)
    shares = []
    for t in range(6):
        tr = oracle.build_tree(X, 300, 900, seed=21 + t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
        before = tc_forest.stats()
        tc_forest.bucket_knn_table(d_X, _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                                   int(tr["leaf_count"].max()), d_idx, d_dist)
        tc_forest.synchronize()
        after = tc_forest.stats()
        shares.append((after["tc_pairs_passed"] - before["tc_pairs_passed"]) /
                      max(1.0, after["tc_pairs_seen"] - before["tc_pairs_seen"]))
    np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
    np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
    print("share of pairs passed, tree by tree:", ["%.4f" % v for v in shares])
    # empty lists get their thresholds from a first pass over the leaf (K of 300-900 candidates
    # plus the margin's share go on, not the whole first column group); full lists let fewer through
    assert shares[0] < 0.1 and shares[-1] < 0.05 and shares[-1] < 0.6 * shares[0]


def test_sampled_leaves_of_a_large_high_dimensional_tree(tc_forest, oracle):
    """The shape of the 1 M x 960 configuration at a size the oracle can follow on a
    sample: one tree with leaves of up to 2048 points over 150 000 x 960 points, built
    and processed on the GPU; the rows of 12 sampled leaves are compared with the
    oracle's bucket KNN of exactly those leaves."""
    import torch
    N, D, K = 150_000, 960, 32
    rng = np.random.default_rng(2)
    c = rng.normal(0, 1, (100, D))
    X = np.empty((N, D), np.float32)
    for s in range(0, N, 25_000):
        X[s:s + 25_000] = c[rng.integers(0, 100, 25_000)] + rng.normal(0, 0.3, (25_000, D))
    d_X = _dev(X)
    info = tc_forest.tree_build(d_X, 33, 2048, seed=5)
    perm, ls, lc = tc_forest.tree_export()
    assert info["max_leaf"] > 1024
    d_idx, d_dist = tc_forest.init_lists(N, K, d_X.device)
    before = tc_forest.stats()
    tc_forest.bucket_knn(d_X, d_idx, d_dist)
    tc_forest.synchronize()
    assert tc_forest.stats()["tc_launches"] - before["tc_launches"] == 1
    pick = np.sort(rng.choice(len(ls), 12, replace=False))
    pick[0] = int(np.argmax(lc))                           # the largest leaf is always checked
    idx, dist = oracle.init_lists(N, K)
    sub_ls, sub_lc = ls[pick].astype(np.int32), lc[pick].astype(np.int32)
    ridx, rdist = oracle.bucket_knn(X, K, perm, sub_ls, sub_lc, idx, dist)
    rows = np.concatenate([perm[s:s + n] for s, n in zip(sub_ls, sub_lc)])
    rows_t = torch.as_tensor(rows.astype(np.int64), device=d_X.device)
    np.testing.assert_array_equal(d_idx[rows_t].cpu().numpy(), ridx[rows])
    np.testing.assert_array_equal(d_dist[rows_t].cpu().numpy().view(np.int32), rdist[rows].view(np.int32))


def test_understated_max_leaf_is_clamped(tc_forest, oracle):
    """A caller's table whose max_leaf is smaller than a real leaf: the kernel works on the
    first max_leaf members of such a leaf and the context stays usable."""
    N, D, K = 3000, 64, 8
    X = _uniform(N, D, 3)
    tr = oracle.build_tree(X, 100, 300, seed=1)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist = _dev(idx), _dev(dist)
    tc_forest.bucket_knn_table(_dev(X), _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                               int(tr["leaf_count"].max()) // 2, d_idx, d_dist)
    tc_forest.synchronize()
    got = d_idx.cpu().numpy()
    assert (got[:, 0] == np.arange(N)).all()
    ridx, rdist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    tc_forest.bucket_knn_table(_dev(X), _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                               int(tr["leaf_count"].max()), d_idx, d_dist)
    tc_forest.synchronize()
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)


EXACT_CASES = [
    # N, D, K, MIN, MAX -- D >= 64 and leaves that fit one CTA: the library's own choice is the exact kernel
    (6000, 100, 32, 33, 66),
    (4000, 128, 64, 65, 130),
    (3000, 64, 100, 101, 202),
]


@pytest.mark.parametrize("mode", [-1, 0, 1])
@pytest.mark.parametrize("N,D,K,MIN,MAX", EXACT_CASES)
def test_every_kernel_choice_gives_the_same_lists(forest, oracle, N, D, K, MIN, MAX, mode):
    """set_tc(-1) (the library's choice), 0 (exact SIMT kernel only) and 1 (tcgen05 filter)
    on the same trees: the oracle's lists bit for bit each time; coincident points included
    (a tie at the K-th distance with a lower index must get through the filter)."""
    X = _uniform(N, D, 19)
    X[np.random.default_rng(1).integers(0, N, N // 4)] = X[0]
    forest.set_tc(mode)
    try:
        idx, dist = oracle.init_lists(N, K)
        d_idx, d_dist, d_X = _dev(idx), _dev(dist), _dev(X)
        before = forest.stats()
        for t in range(4):
            tr = oracle.build_tree(X, MIN, MAX, seed=70 + t, max_depth=40)
            idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
            forest.bucket_knn_table(d_X, _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                                    int(tr["leaf_count"].max()), d_idx, d_dist)
            forest.synchronize()
            np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
            np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
        ran_tc = forest.stats()["tc_launches"] - before["tc_launches"]
        # the library's own choice depends on the largest leaf of each tree
        assert ran_tc == 4 if mode == 1 else (ran_tc == 0 if mode == 0 else 0 <= ran_tc <= 4)
    finally:
        forest.set_tc(-1)


@pytest.mark.parametrize("N,D,K,MIN,MAX", [(6000, 128, 16, 400, 1200), (4000, 96, 32, 300, 700)])
def test_rows_with_and_without_a_full_list_in_the_same_tiles(tc_forest, oracle, N, D, K, MIN, MAX):
    """Lists of two trees, then every third row emptied again (and a few rows left half full): the
    first pass gives the emptied rows a threshold from their whole leaf while their neighbours in
    the same 128-row tile keep the threshold of their own full list."""
    X = _clustered(N, D, 23, centers=5, sigma=0.6)
    idx, dist = oracle.init_lists(N, K)
    for t in range(2):
        tr = oracle.build_tree(X, MIN, MAX, seed=70 + t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    empty_i, empty_d = oracle.init_lists(N, K)
    idx[::3], dist[::3] = empty_i[::3], empty_d[::3]
    idx[1::7, K // 2:], dist[1::7, K // 2:] = -1, np.inf          # rows that are half full
    d_idx, d_dist, d_X = _dev(idx), _dev(dist), _dev(X)
    before = tc_forest.stats()
    for t in range(2):
        tr = oracle.build_tree(X, MIN, MAX, seed=80 + t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
        tc_forest.bucket_knn_table(d_X, _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                                   int(tr["leaf_count"].max()), d_idx, d_dist)
        tc_forest.synchronize()
        np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
        np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), dist.view(np.int32))
    assert tc_forest.stats()["tc_launches"] - before["tc_launches"] == 2
