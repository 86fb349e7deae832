"""Parity of the query (base/query) path against the CPU oracle, through the C ABI:
the leaf bucket every query is routed to, and the query lists after the bucket
update, bit for bit (indices and squared distances)."""
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


@pytest.fixture()
def indexed(forest):
    forest.keep_index(True)
    yield forest
    forest.keep_index(False)


ROUTE_CASES = [
    # N, NQ, D, MIN, MAX, seed, data
    (20000, 5000, 32, 32, 128, 0, "uniform"),
    (6000, 6000, 100, 33, 66, 1, "uniform"),
    (30000, 4000, 2, 256, 1024, 2, "clustered"),
    (3000, 1000, 200, 31, 128, 3, "uniform"),
    (4096, 777, 99, 136, 408, 4, "uniform"),
    (2000, 3000, 7, 5, 10, 5, "uniform"),      # many dissolved sides
    (1500, 100, 960, 33, 700, 6, "clustered"),
    (100, 50, 16, 33, 66, 7, "uniform"),       # root children below MIN
    (1, 5, 8, 4, 8, 8, "uniform"),             # single point: one leaf
    (2, 5, 8, 4, 8, 9, "uniform"),
    (50000, 20000, 3, 17, 34, 10, "uniform"),
    (300000, 1000, 24, 20, 60, 11, "uniform"),  # level kernels and in-CTA subtrees both file rows
]


@pytest.mark.parametrize("N,NQ,D,MIN,MAX,seed,kind", ROUTE_CASES)
def test_query_routing_matches_oracle(indexed, oracle, N, NQ, D, MIN, MAX, seed, kind):
    X = _uniform(N, D, seed) if kind == "uniform" else _clustered(N, D, seed)
    Q = _uniform(NQ, D, seed + 100) if kind == "uniform" else _clustered(NQ, D, seed)
    ref = oracle.build_tree_route(X, Q, MIN, MAX, seed=seed)
    dX, dQ = _dev(X), _dev(Q)
    indexed.tree_build(dX, MIN, MAX, seed=seed)
    perm, ls, lc = indexed.tree_export()
    np.testing.assert_array_equal(perm, ref["perm"])
    qs, qc = indexed.route_queries(dX, dQ)
    np.testing.assert_array_equal(qs, ref["q_start"])
    np.testing.assert_array_equal(qc, ref["q_count"])


def test_base_points_route_to_their_own_bucket(indexed, oracle):
    X = _uniform(40000, 48, 21)
    dX = _dev(X)
    indexed.tree_build(dX, 25, 50, seed=4)
    perm, ls, lc = indexed.tree_export()
    own_start = np.empty(len(X), np.int32)
    own_count = np.empty(len(X), np.int32)
    for s, c in zip(ls, lc):
        own_start[perm[s:s + c]] = s
        own_count[perm[s:s + c]] = c
    qs, qc = indexed.route_queries(dX, dX)
    np.testing.assert_array_equal(qs, own_start)
    np.testing.assert_array_equal(qc, own_count)


def test_routing_with_replayed_split_pairs(indexed, oracle):
    X, Q = _uniform(8000, 40, 31), _uniform(2000, 40, 32)
    src = oracle.build_tree(X, 20, 40, seed=555, record=True)
    ref = oracle.build_tree_route(X, Q, 20, 40, seed=1, table=src["table"])
    dX = _dev(X)
    indexed.tree_build(dX, 20, 40, seed=2, table=_dev(src["table"]))
    qs, qc = indexed.route_queries(dX, _dev(Q))
    np.testing.assert_array_equal(qs, ref["q_start"])
    np.testing.assert_array_equal(qc, ref["q_count"])


def test_routing_at_the_depth_limit(indexed, oracle):
    X = np.zeros((500, 8), np.float32)          # coincident points never split
    X[:10] = _uniform(10, 8, 3)
    Q = np.concatenate([_uniform(20, 8, 4), np.zeros((5, 8), np.float32)])
    ref = oracle.build_tree_route(X, Q, 8, 16, max_depth=12, seed=0)
    dX = _dev(X)
    indexed.tree_build(dX, 8, 16, max_depth=12, seed=0)
    qs, qc = indexed.route_queries(dX, _dev(Q))
    np.testing.assert_array_equal(qs, ref["q_start"])
    np.testing.assert_array_equal(qc, ref["q_count"])


def test_routing_needs_the_index(forest):
    from gpu_rsfk import RSFKLibraryError
    X = _dev(_uniform(2000, 8, 1))
    forest.keep_index(False)
    forest.tree_build(X, 8, 16, seed=0)
    with pytest.raises(RSFKLibraryError):
        forest.route_queries(X, X)


ANN_CASES = [
    # N, NQ, D, K, MIN, MAX
    (20000, 5000, 32, 16, 32, 128),
    (6000, 6000, 100, 32, 33, 66),
    (30000, 3000, 2, 32, 256, 1024),
    (5000, 900, 100, 64, 65, 130),
    (3000, 500, 17, 5, 3, 9),          # buckets smaller than K leave empty slots
    (4000, 1000, 64, 100, 101, 202),
    (3000, 300, 33, 256, 257, 514),
    (1500, 100, 960, 32, 33, 700),
]


@pytest.mark.parametrize("N,NQ,D,K,MIN,MAX", ANN_CASES)
def test_query_bucket_update_matches_oracle(indexed, oracle, N, NQ, D, K, MIN, MAX):
    import torch
    X, Q = _uniform(N, D, 41), _uniform(NQ, D, 42)
    dX, dQ = _dev(X), _dev(Q)
    i0, d0 = oracle.init_lists(NQ, K, self_in_row=False)
    didx, ddist = _dev(i0), _dev(d0)
    ri, rd = i0, d0
    for t in range(3):                   # later trees merge into the earlier result
        ref = oracle.build_tree_route(X, Q, MIN, MAX, seed=7 + t)
        ri, rd = oracle.ann_bucket_knn(X, Q, K, ref["perm"], ref["q_start"], ref["q_count"], ri, rd)
        indexed.tree_build(dX, MIN, MAX, seed=7 + t)
        indexed.ann_bucket_knn(dX, dQ, didx, ddist)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(didx.cpu().numpy(), ri)
        np.testing.assert_array_equal(ddist.cpu().numpy().view(np.int32), rd.view(np.int32))


def test_query_update_on_integer_data_with_ties(indexed, oracle):
    import torch
    rng = np.random.default_rng(9)
    X = rng.integers(0, 6, (5000, 12)).astype(np.float32)
    Q = rng.integers(0, 6, (1500, 12)).astype(np.float32)
    K = 10
    ref = oracle.build_tree_route(X, Q, 11, 40, seed=3)
    i0, d0 = oracle.init_lists(len(Q), K, self_in_row=False)
    ri, rd = oracle.ann_bucket_knn(X, Q, K, ref["perm"], ref["q_start"], ref["q_count"], i0, d0)
    dX, dQ, didx, ddist = _dev(X), _dev(Q), _dev(i0), _dev(d0)
    indexed.tree_build(dX, 11, 40, seed=3)
    indexed.ann_bucket_knn(dX, dQ, didx, ddist)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(didx.cpu().numpy(), ri)
    np.testing.assert_array_equal(ddist.cpu().numpy().view(np.int32), rd.view(np.int32))


def test_query_forest_on_the_device_matches_oracle(indexed, oracle):
    import torch
    X, Q = _clustered(12000, 24, 5), _clustered(3000, 24, 6)
    K, T = 12, 6
    ri, rd = oracle.ann_forest(X, Q, K, T, 13, 26, seed=100)
    i0, d0 = oracle.init_lists(len(Q), K, self_in_row=False)
    didx, ddist = _dev(i0), _dev(d0)
    indexed.forest_ann(_dev(X), _dev(Q), didx, ddist, T, 13, 26, seed=100)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(didx.cpu().numpy(), ri)
    np.testing.assert_array_equal(ddist.cpu().numpy().view(np.int32), rd.view(np.int32))
    # the same forest as three tree sequences side by side
    li, ld = _dev(i0), _dev(d0)
    indexed.set_lanes(3)
    try:
        indexed.forest_ann(_dev(X), _dev(Q), li, ld, T, 13, 26, seed=100)
    finally:
        indexed.set_lanes(0)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(li.cpu().numpy(), ri)
    np.testing.assert_array_equal(ld.cpu().numpy().view(np.int32), rd.view(np.int32))
    # sharded over two "ranks" (trees 0,2,4 and 1,3,5) then merged = the same lists
    parts = []
    for g in range(2):
        pi, pd = _dev(i0), _dev(d0)
        indexed.forest_ann(_dev(X), _dev(Q), pi, pd, T // 2, 13, 26, seed=100, first_tree=g, tree_stride=2)
        parts.append((pi, pd))
    oi, od = torch.empty_like(didx), torch.empty_like(ddist)
    indexed.merge_lists([p[0] for p in parts], [p[1] for p in parts], oi, od)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(oi.cpu().numpy(), ri)
    np.testing.assert_array_equal(od.cpu().numpy().view(np.int32), rd.view(np.int32))


def test_wrapper_query_search_matches_oracle_and_finds_neighbours(oracle):
    from gpu_rsfk import RSFK
    X, Q = _clustered(20000, 32, 7), _clustered(2500, 32, 8)
    K, T = 16, 8
    idx, dist = RSFK(random_state=5).find_nearest_neighbors_ann(X, Q, K, n_trees=T)
    assert idx.shape == (len(Q), K) and idx.dtype == np.int32 and dist.dtype == np.float32
    ri, rd = oracle.ann_forest(X, Q, K, T, K + 1, 2 * (K + 1), seed=5)
    np.testing.assert_array_equal(idx, ri)
    np.testing.assert_array_equal(dist.view(np.int32), rd.view(np.int32))
    assert (idx >= 0).all() and (idx < len(X)).all()     # min_tree_children = K+1 fills every slot
    assert (np.diff(dist, axis=1) >= 0).all()
    bi, bd = oracle.bruteforce_ann(X, Q, K)
    assert oracle.recall(bi, idx) > 0.1     # 8 trees on 32-D data: far above chance (K/N), far from exact
    # ensure_valid_indices: small buckets, then one tree of K+1 .. 3(K+1) points fills the rows
    idx2, _ = RSFK(random_state=5).find_nearest_neighbors_ann(X, Q, K, n_trees=2, min_tree_children=4,
                                                              max_tree_children=9)
    assert (idx2 >= 0).all()
    idx3, _ = RSFK(random_state=5).find_nearest_neighbors_ann(X, Q, K, n_trees=2, min_tree_children=4,
                                                              max_tree_children=9, ensure_valid_indices=False)
    assert (idx3 == -1).any()


def test_query_lists_given_by_the_caller_are_merged(oracle):
    """The C entry point merges into the lists it is handed (FLT_MAX or +inf = empty)."""
    from gpu_rsfk import _lib
    L = _lib.load()
    X, Q = _uniform(5000, 20, 51), _uniform(700, 20, 52)
    K = 8
    bi, bd = oracle.bruteforce_ann(X, Q, K)
    idx = np.full((len(Q), K), -1, np.int32)
    dist = np.full((len(Q), K), np.finfo(np.float32).max, np.float32)
    idx[:, 3] = bi[:, 0]                 # the true nearest neighbour, in an arbitrary slot
    dist[:, 3] = bd[:, 0]
    log = np.zeros(16 * 2 + 2, np.float32)
    L.pymodule_rsfk_knn_ann(2, K, len(X), len(Q), 20, 9, 18, 5000, 0, 3, 0, X, Q, idx, dist, log)
    _lib.check_last("pymodule_rsfk_knn_ann")
    np.testing.assert_array_equal(idx[:, 0], bi[:, 0])
    i0 = np.full((len(Q), K), -1, np.int32); d0 = np.full((len(Q), K), np.inf, np.float32)
    i0[:, 0] = bi[:, 0]; d0[:, 0] = bd[:, 0]
    ri, rd = oracle.ann_forest(X, Q, K, 2, 9, 18, seed=3, idx=i0, dist=d0)
    np.testing.assert_array_equal(idx, ri)
    np.testing.assert_array_equal(dist.view(np.int32), rd.view(np.int32))


def test_query_search_edge_cases(indexed, oracle):
    import torch
    from gpu_rsfk import RSFK, RSFKLibraryError
    # one base point: every query row holds it, with its distance, and nothing else
    X = _uniform(1, 5, 1)
    Q = _uniform(7, 5, 2)
    idx, dist = RSFK(random_state=0).find_nearest_neighbors_ann(X, Q, 3, n_trees=2, ensure_valid_indices=False)
    assert (idx[:, 0] == 0).all() and (idx[:, 1:] == -1).all()
    want = np.array([oracle.dist_sqr(q, X[0]) for q in Q], np.float32)
    np.testing.assert_array_equal(dist[:, 0].view(np.int32), want.view(np.int32))
    assert np.isinf(dist[:, 1:]).all()
    # one query, one dimension, fewer base points than K
    X1, Q1 = _uniform(40, 1, 3), _uniform(1, 1, 4)
    i1, d1 = RSFK(random_state=0).find_nearest_neighbors_ann(X1, Q1, 64, n_trees=3)
    ri, rd = oracle.ann_forest(X1, Q1, 64, 3, 65, 130, seed=0)
    np.testing.assert_array_equal(i1, ri)
    assert (i1[0, :40] >= 0).all() and (i1[0, 40:] == -1).all()
    # no tree at all: lists come back as given (canonical order)
    didx, ddist = _dev(np.full((5, 4), -1, np.int32)), _dev(np.full((5, 4), np.inf, np.float32))
    indexed.forest_ann(_dev(_uniform(100, 3, 5)), _dev(_uniform(5, 3, 6)), didx, ddist, 0, 4, 8)
    torch.cuda.synchronize()
    assert (didx.cpu().numpy() == -1).all()
    # the largest supported K, and one beyond
    Xk, Qk = _uniform(3000, 6, 7), _uniform(50, 6, 8)
    ik, dk = RSFK(random_state=1).find_nearest_neighbors_ann(Xk, Qk, 256, n_trees=2)
    rk, _ = oracle.ann_forest(Xk, Qk, 256, 2, 257, 514, seed=1)
    np.testing.assert_array_equal(ik, rk)
    with pytest.raises(RSFKLibraryError):
        RSFK().find_nearest_neighbors_ann(Xk, Qk, 257, n_trees=1)
    # shapes that do not agree are refused before the library is called
    with pytest.raises(Exception):
        RSFK().find_nearest_neighbors_ann(Xk, _uniform(5, 7, 9), 4, n_trees=1)
    with pytest.raises(ValueError):
        indexed.forest_ann(_dev(Xk), _dev(_uniform(5, 7, 9)), didx, ddist, 1, 4, 8)
