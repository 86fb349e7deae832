"""Parity of the sm_100a kernels against the CPU oracle, through the C ABI.

Integer results (bucket membership, neighbour indices) must be bit-exact.
Squared distances are computed in the reference's summation order on both
sides, so they are compared bit-exactly as well (tolerance 0; the specification
allows 1e-5 relative)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _uniform(N, D, seed=0):
    rng = np.random.RandomState(seed)
    return rng.uniform(0, 1, (N, D)).astype(np.float32)


def _clustered(N, D, seed, centers=16, sigma=0.3):
    rng = np.random.default_rng(seed)
    c = rng.normal(0, 1, (centers, D))
    return (c[rng.integers(0, centers, N)] + rng.normal(0, sigma, (N, D))).astype(np.float32)


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


TREE_CASES = [
    # N, D, MIN, MAX, seed, data
    (20000, 32, 32, 128, 0, "uniform"),
    (5000, 100, 33, 66, 1, "uniform"),
    (30000, 2, 256, 1024, 2, "clustered"),
    (3000, 200, 31, 128, 3, "uniform"),
    (4096, 99, 136, 408, 4, "uniform"),
    (2000, 7, 5, 10, 5, "uniform"),
    (1500, 960, 33, 700, 6, "clustered"),
    (100, 16, 33, 66, 7, "uniform"),      # root children below MIN
    (1, 8, 4, 8, 8, "uniform"),
    (2, 8, 4, 8, 9, "uniform"),
    (50000, 3, 17, 34, 10, "uniform"),
]


@pytest.mark.parametrize("N,D,MIN,MAX,seed,kind", TREE_CASES)
def test_tree_buckets_match_oracle(forest, oracle, N, D, MIN, MAX, seed, kind):
    X = _uniform(N, D, seed) if kind == "uniform" else _clustered(N, D, seed)
    ref = oracle.build_tree(X, MIN, MAX, seed=seed, record=True)
    info = forest.tree_build(_dev(X), MIN, MAX, seed=seed)
    perm, ls, lc = forest.tree_export()
    assert info["n_leaves"] == len(ref["leaf_start"])
    np.testing.assert_array_equal(ls, ref["leaf_start"])
    np.testing.assert_array_equal(lc, ref["leaf_count"])
    np.testing.assert_array_equal(perm, ref["perm"])
    assert info["levels"] == ref["depth"]
    assert info["max_leaf"] == ref["leaf_count"].max()
    assert info["min_leaf"] == ref["leaf_count"].min()


@pytest.mark.parametrize("N,D,MIN,MAX", [(20000, 32, 32, 128), (6000, 100, 33, 66), (20000, 2, 64, 256)])
def test_tree_replays_explicit_split_pairs(forest, oracle, N, D, MIN, MAX):
    """Split pairs fed as explicit input (drawn here by an unrelated seed) give
    bit-identical buckets on both sides."""
    X = _uniform(N, D, 11)
    src = oracle.build_tree(X, MIN, MAX, seed=777, record=True)
    ref = oracle.build_tree(X, MIN, MAX, seed=1, table=src["table"])
    np.testing.assert_array_equal(ref["perm"], src["perm"])
    forest.tree_build(_dev(X), MIN, MAX, seed=2, table=_dev(src["table"]))
    perm, ls, lc = forest.tree_export()
    np.testing.assert_array_equal(perm, ref["perm"])
    np.testing.assert_array_equal(ls, ref["leaf_start"])
    np.testing.assert_array_equal(lc, ref["leaf_count"])


def test_tree_depth_limit_forces_leaves(forest, oracle):
    X = np.zeros((500, 8), np.float32)          # coincident points never split
    X[:10] = _uniform(10, 8, 3)
    ref = oracle.build_tree(X, 8, 16, max_depth=12, seed=0)
    info = forest.tree_build(_dev(X), 8, 16, max_depth=12, seed=0)
    perm, ls, lc = forest.tree_export()
    np.testing.assert_array_equal(perm, ref["perm"])
    np.testing.assert_array_equal(ls, ref["leaf_start"])
    np.testing.assert_array_equal(lc, ref["leaf_count"])
    assert lc.max() <= 16 and lc.sum() == 500 and info["n_leaves"] == len(ls)


KNN_CASES = [
    # N, D, K, MIN, MAX
    (20000, 32, 16, 32, 128),
    (6000, 100, 32, 33, 66),
    (20000, 2, 32, 256, 1024),
    (3000, 200, 30, 31, 128),
    (4000, 128, 64, 65, 130),
    (3000, 17, 5, 6, 12),
    (1200, 960, 32, 33, 600),
    (3000, 64, 100, 101, 202),
    (2500, 33, 200, 201, 402),
]


@pytest.mark.parametrize("N,D,K,MIN,MAX", KNN_CASES)
def test_bucket_knn_bit_exact(forest, oracle, N, D, K, MIN, MAX):
    X = _uniform(N, D, 5)
    idx, dist = oracle.init_lists(N, K)
    d_idx, d_dist, d_X = _dev(idx), _dev(dist), _dev(X)
    for t in range(3):       # lists accumulate over trees
        tr = oracle.build_tree(X, MIN, MAX, seed=t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
        forest.bucket_knn_table(d_X, _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                                int(tr["leaf_count"].max()), d_idx, d_dist)
        np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
        np.testing.assert_array_equal(d_dist.cpu().numpy(), dist)


def test_bucket_knn_integer_data_ties(forest, oracle):
    """Integer-valued coordinates make many distances tie exactly; ties go to
    the lower index on both sides."""
    rng = np.random.default_rng(3)
    X = rng.integers(0, 4, (4000, 12)).astype(np.float32)
    X += rng.integers(0, 2, X.shape).astype(np.float32) * 0.5
    K = 16
    tr = oracle.build_tree(X, 17, 64, seed=0, max_depth=200)
    idx, dist = oracle.init_lists(len(X), K)
    ridx, rdist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    d_idx, d_dist = _dev(idx), _dev(dist)
    forest.bucket_knn_table(_dev(X), _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                            int(tr["leaf_count"].max()), d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)


def test_bucket_knn_large_leaves_tiled(forest, oracle):
    """Leaves larger than one shared-memory block take the block-pair path."""
    X = _uniform(6000, 300, 9)
    K = 32
    tr = oracle.build_tree(X, 500, 1500, seed=4)
    assert tr["leaf_count"].max() > 160
    idx, dist = oracle.init_lists(len(X), K)
    ridx, rdist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    d_idx, d_dist = _dev(idx), _dev(dist)
    forest.bucket_knn_table(_dev(X), _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                            int(tr["leaf_count"].max()), d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)


def test_sort_rows_canonicalises(forest, oracle):
    rng = np.random.default_rng(0)
    N, K = 3000, 48
    idx = rng.integers(-1, 200, (N, K)).astype(np.int32)      # repeats and empties
    dist = rng.random((N, K)).astype(np.float32)
    dist[idx < 0] = np.float32(3.4028235e38)                   # FLT_MAX marks empty in the C driver
    ridx, rdist = oracle.sort_rows(idx, dist)
    d_idx, d_dist = _dev(idx), _dev(dist)
    forest.sort_rows(d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)


@pytest.mark.parametrize("N,D,K", [(20000, 32, 16), (5000, 100, 32), (3000, 128, 64), (4000, 2, 32), (2000, 50, 7),
                                   # long lists of medium rows: the sweep that stages rows in shared memory
                                   (2500, 100, 64), (2000, 64, 40), (1500, 96, 33), (1800, 128, 50),
                                   # wide rows: one row per shared-memory buffer, five, three or two buffers per warp
                                   (1500, 960, 32), (1200, 512, 16), (900, 1024, 20), (700, 1500, 8), (600, 1900, 5)])
def test_explore_bit_exact(forest, oracle, N, D, K):
    X = _uniform(N, D, 6)
    idx, dist = oracle.init_lists(N, K)
    for t in range(3):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    d_X, d_idx, d_dist = _dev(X), _dev(idx), _dev(dist)
    for sweep in range(2):
        ridx, rdist = oracle.explore(X, idx, idx, dist)
        snap = d_idx.clone()
        forest.explore(d_X, snap, d_idx, d_dist)
        np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
        np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)
        idx, dist = ridx, rdist


@pytest.mark.parametrize("N,D,K", [(3000, 24, 20), (3000, 72, 40), (2500, 640, 20)])
def test_explore_skips_empty_slots_and_row_range(forest, oracle, N, D, K):
    X = _uniform(N, D, 8)
    idx, dist = oracle.init_lists(N, K)
    tr = oracle.build_tree(X, 8, 16, seed=0)     # buckets smaller than K leave -1 slots
    idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    assert (idx < 0).any()
    ridx, rdist = oracle.explore(X, idx, idx, dist, 1000, 2200)
    d_idx, d_dist = _dev(idx), _dev(dist)
    forest.explore(_dev(X), d_idx.clone(), d_idx, d_dist, 1000, 2200)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)


def test_merge_lists_bit_exact(forest, oracle):
    N, D, K, G = 4000, 40, 32, 4
    X = _uniform(N, D, 12)
    lists = []
    for g in range(G):
        idx, dist = oracle.init_lists(N, K)
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=100 + g)
        lists.append(oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist))
    ridx, rdist = oracle.merge_lists([l[0] for l in lists], [l[1] for l in lists])
    import torch
    out_i = torch.empty((N, K), dtype=torch.int32, device="cuda")
    out_d = torch.empty((N, K), dtype=torch.float32, device="cuda")
    forest.merge_lists([_dev(l[0]) for l in lists], [_dev(l[1]) for l in lists], out_i, out_d)
    np.testing.assert_array_equal(out_i.cpu().numpy(), ridx)
    np.testing.assert_array_equal(out_d.cpu().numpy(), rdist)


def test_forest_equals_oracle_pipeline(forest, oracle):
    """Whole device pipeline (trees + buckets + sweep) equals the oracle's."""
    N, D, K, T = 8000, 48, 16, 4
    X = _uniform(N, D, 21)
    idx, dist = oracle.init_lists(N, K)
    for t in range(T):
        tr = oracle.build_tree(X, 17, 34, seed=5 + t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    idx, dist = oracle.explore(X, idx, idx, dist)
    d_X = _dev(X)
    d_idx, d_dist = forest.init_lists(N, K, d_X.device)
    log = forest.forest(d_X, d_idx, d_dist, T, 17, 34, seed=5, want_log=True)
    forest.explore(d_X, d_idx.clone(), d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), idx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), dist)
    assert log[3 * T:4 * T].min() > 0          # total leaves per tree


@pytest.mark.parametrize("lanes", [1, 2, 3, 4])
def test_forest_lanes_do_not_change_the_graph(forest, oracle, lanes):
    """A forest split over several tree sequences on one GPU (each with lists of
    its own, combined at the end) returns the rows of the oracle's sequential
    pipeline, whatever the number of lanes; caller-supplied rows take part once."""
    N, D, K, T = 6000, 40, 12, 9
    X = _uniform(N, D, 23)
    idx, dist = oracle.init_lists(N, K)
    idx[:, 1] = (np.arange(N) + 1) % N                    # a valid neighbour the caller already knows
    dist[:, 1] = [oracle.dist_sqr(X[p], X[(p + 1) % N]) for p in range(N)]
    d_idx, d_dist = _dev(idx), _dev(dist)
    ridx, rdist = oracle.sort_rows(idx, dist)
    for t in range(T):
        tr = oracle.build_tree(X, 13, 26, seed=50 + t)
        ridx, rdist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], ridx, rdist)
    forest.set_lanes(lanes)
    try:
        forest.sort_rows(d_idx, d_dist)
        log = forest.forest(_dev(X), d_idx, d_dist, T, 13, 26, seed=50, want_log=True)
    finally:
        forest.set_lanes(0)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy().view(np.int32), rdist.view(np.int32))
    assert (log[3 * T:4 * T] > 0).all() and (log[15 * T:16 * T] > 0).all()   # every tree logged
    st = forest.stats()
    assert st["trees"] >= T


def test_config1_recall_through_wrapper(oracle):
    """Small plumbing configuration: N=20000, D=32, K=16, 4 trees, 32/128, one
    sweep, through the drop-in Python class; recall against exact brute force."""
    from gpu_rsfk import RSFK
    np.random.seed(0)
    X = np.random.uniform(0, 1, (20000, 32)).astype(np.float32)
    r = RSFK(random_state=0)
    idx, dist = r.find_nearest_neighbors(X, 16, n_trees=4, min_tree_children=32, max_tree_children=128,
                                         nn_exploring_factor=1)
    assert idx.dtype == np.int32 and dist.dtype == np.float32 and idx.shape == (20000, 16)
    assert (idx[:, 0] == np.arange(20000)).all() and (dist[:, 0] == 0).all()
    assert (idx >= 0).all()
    assert (np.diff(dist, axis=1) >= 0).all()
    q = np.arange(0, 20000, 10, dtype=np.int32)
    ti, td, _ = oracle.bruteforce_knn(X, 16, q)
    rec = oracle.recall(ti, idx[q])
    # oracle pipeline with the same seeds gives the same graph, hence the same recall
    oi, od = oracle.init_lists(20000, 16)
    for t in range(4):
        tr = oracle.build_tree(X, 32, 128, seed=t)
        oi, od = oracle.bucket_knn(X, 16, tr["perm"], tr["leaf_start"], tr["leaf_count"], oi, od)
    oi, od = oracle.explore(X, oi, oi, od)
    np.testing.assert_array_equal(idx, oi)
    np.testing.assert_array_equal(dist, od)
    assert rec > 0.25
    assert len(r.log_forest.data["Total Leaves"]) == 4


def test_cluster_by_sample_tree_matches_oracle(oracle):
    from gpu_rsfk import RSFK
    X = _clustered(40000, 2, 1, centers=64, sigma=1.0)
    n_leaves, width, buckets, sizes = RSFK(random_state=3).cluster_by_sample_tree(
        X, min_tree_children=256, max_tree_children=1024, verbose=0)
    ref = oracle.build_tree(X, 256, 1024, seed=3)
    assert n_leaves == len(ref["leaf_start"]) and width == ref["leaf_count"].max()
    np.testing.assert_array_equal(sizes, ref["leaf_count"])
    table = buckets.reshape(n_leaves, width)
    for b in range(n_leaves):
        s, c = ref["leaf_start"][b], ref["leaf_count"][b]
        np.testing.assert_array_equal(table[b, :c], ref["perm"][s:s + c])
        assert (table[b, c:] == -1).all()
    assert sizes.min() >= 256 and sizes.max() <= 1024


def test_reference_smoke_suite():
    """The two live smoke tests of the reference package (no -1 index; a
    clustering call runs) pass on this library."""
    import gpu_rsfk
    gpu_rsfk.test()


def test_maximum_list_length_and_refusal_beyond_it(forest, oracle):
    """K = 256 is the largest list the kernels hold; 257 is refused with a status,
    not computed wrongly."""
    import torch
    from gpu_rsfk import _lib
    N, D, K = 1500, 24, 256
    X = _uniform(N, D, 31)
    idx, dist = oracle.init_lists(N, K)
    tr = oracle.build_tree(X, 300, 700, seed=1)
    ridx, rdist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    d_idx, d_dist = _dev(idx), _dev(dist)
    forest.bucket_knn_table(_dev(X), _dev(tr["perm"]), _dev(tr["leaf_start"]), _dev(tr["leaf_count"]),
                            int(tr["leaf_count"].max()), d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), ridx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), rdist)
    eidx, edist = oracle.explore(X, ridx, ridx, rdist)
    forest.explore(_dev(X), d_idx.clone(), d_idx, d_dist)
    np.testing.assert_array_equal(d_idx.cpu().numpy(), eidx)
    np.testing.assert_array_equal(d_dist.cpu().numpy(), edist)
    big_i = torch.full((N, 257), -1, dtype=torch.int32, device="cuda")
    big_d = torch.full((N, 257), float("inf"), dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.RSFKLibraryError):
        forest.sort_rows(big_i, big_d)


def test_one_dimension_and_no_trees_through_the_host_entry_point(oracle):
    """D = 1 and n_trees = 0 (sweeps only, on caller-provided lists) through the
    drop-in C ABI with host buffers."""
    from gpu_rsfk import _lib
    L = _lib.load()
    N, D, K = 4000, 1, 6
    X = _uniform(N, D, 33)
    idx, dist = oracle.init_lists(N, K)
    for t in range(2):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    shuffled_i, shuffled_d = idx[:, ::-1].copy(), dist[:, ::-1].copy()      # caller's rows are unordered
    ei, ed = oracle.explore(X, idx, idx, dist)
    ei, ed = oracle.explore(X, ei, ei, ed)
    log = np.zeros(2, np.float32)
    L.pymodule_rsfk_knn(0, K, N, D, K + 1, 2 * K + 2, 5000, 0, 0, 2, X, shuffled_i, shuffled_d, log)
    _lib.check_last("pymodule_rsfk_knn")
    np.testing.assert_array_equal(shuffled_i, ei)
    np.testing.assert_array_equal(shuffled_d, ed)
    # invalid arguments leave the outputs untouched and set a status
    before = shuffled_i.copy()
    L.pymodule_rsfk_knn(1, 0, N, D, 7, 14, 5000, 0, 0, 0, X, shuffled_i, shuffled_d, log)
    assert L.rsfk_last_status() == 2
    np.testing.assert_array_equal(shuffled_i, before)
    L.rsfk_release_memory()


@pytest.mark.parametrize("N,D,K", [(5000, 8, 10), (3000, 40, 33), (1, 3, 4), (20000, 3, 64), (9000, 16, 1)])
def test_symmetric_closure_matches_oracle(forest, oracle, N, D, K):
    """CSR of the graph united with its transpose: offsets, indices (ordered by
    index) and the edges' squared distances equal the oracle's."""
    import torch
    X = _uniform(N, D, 61)
    idx, dist = oracle.init_lists(N, K)
    tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=5)
    idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    if N > 100:
        idx[::7, K - 1] = -1                          # some empty slots
        dist[::7, K - 1] = np.inf
    off, ind, val = oracle.symmetrize(idx, dist)
    d_off, d_ind, d_val = forest.symmetrize(_dev(idx), _dev(dist))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(d_off.cpu().numpy(), off)
    np.testing.assert_array_equal(d_ind.cpu().numpy(), ind)
    np.testing.assert_array_equal(d_val.cpu().numpy().view(np.int32), val.view(np.int32))
    o2, i2, none = forest.symmetrize(_dev(idx))
    torch.cuda.synchronize()
    assert none is None
    np.testing.assert_array_equal(i2.cpu().numpy(), ind)
    # a hub: one point listed by everybody gets a long row
    hub = np.full((N, 2), -1, np.int32)
    hub[:, 0] = 0
    ho, hi, _ = oracle.symmetrize(hub)
    go, gi, _ = forest.symmetrize(_dev(hub))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(go.cpu().numpy(), ho)
    np.testing.assert_array_equal(gi.cpu().numpy(), hi)
