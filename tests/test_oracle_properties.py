"""Properties of the CPU oracle itself (no GPU): its restated arithmetic
against plain float64 numpy, tree invariants, replay, and agreement between
its reference-order and canonical statements."""
import numpy as np
import pytest


def _uniform(N, D, seed=0):
    return np.random.RandomState(seed).uniform(0, 1, (N, D)).astype(np.float32)


@pytest.mark.parametrize("D", [1, 2, 3, 31, 32, 33, 100, 960])
def test_distance_and_projection_close_to_float64(oracle, D):
    rng = np.random.default_rng(D)
    a, b = rng.normal(size=D).astype(np.float32), rng.normal(size=D).astype(np.float32)
    exact = float(((a.astype(np.float64) - b.astype(np.float64)) ** 2).sum())
    assert abs(oracle.dist_sqr(a, b) - exact) <= 1e-5 * max(exact, 1e-30)      # 1e-5 relative
    assert oracle.dist_sqr(a, b) == oracle.dist_sqr(b, a)
    assert oracle.dist_sqr(a, a) == 0.0
    for is_root in (True, False):
        n, c = oracle.hyperplane(a, b, is_root)
        np.testing.assert_array_equal(n, a - b)
        mid = float((n.astype(np.float64) * (a.astype(np.float64) + b) / 2).sum())
        assert abs(float(c) - mid) <= 1e-4 * max(1.0, abs(mid))
        # p1 lies on the left of its own hyperplane, p2 on the right
        assert not (oracle.project(n, a) < c)
        assert oracle.project(n, b) < c


def test_sample_positions_are_distinct_and_in_range(oracle):
    seen = set()
    for start in range(0, 2000, 37):
        for count in (1, 2, 3, 66, 1000):
            r1, r2 = oracle.sample_positions(5, 3, start, count)
            assert 0 <= r1 < count and 0 <= r2 < count
            assert count == 1 or r1 != r2
            seen.add((r1, r2))
    assert len(seen) > 50


@pytest.mark.parametrize("N,D,MIN,MAX", [(20000, 32, 32, 128), (5000, 100, 33, 66), (30000, 2, 256, 1024),
                                         (3000, 8, 1, 2), (777, 5, 10, 20)])
def test_tree_invariants(oracle, N, D, MIN, MAX):
    X = _uniform(N, D, 1)
    tr = oracle.build_tree(X, MIN, MAX, seed=4)
    assert sorted(tr["perm"].tolist()) == list(range(N))          # every point in exactly one bucket
    assert tr["leaf_count"].sum() == N
    np.testing.assert_array_equal(tr["leaf_start"], np.cumsum(tr["leaf_count"]) - tr["leaf_count"])
    assert tr["leaf_count"].min() >= MIN and tr["leaf_count"].max() <= MAX


def test_tree_is_deterministic_and_seed_dependent(oracle):
    X = _uniform(6000, 16, 2)
    a = oracle.build_tree(X, 20, 40, seed=1)
    b = oracle.build_tree(X, 20, 40, seed=1)
    c = oracle.build_tree(X, 20, 40, seed=2)
    np.testing.assert_array_equal(a["perm"], b["perm"])
    assert not np.array_equal(a["perm"], c["perm"])


def test_tree_replay_of_recorded_pairs(oracle):
    X = _uniform(8000, 24, 3)
    a = oracle.build_tree(X, 16, 32, seed=9, record=True)
    b = oracle.build_tree(X, 16, 32, seed=12345, table=a["table"])
    np.testing.assert_array_equal(a["perm"], b["perm"])
    np.testing.assert_array_equal(a["leaf_count"], b["leaf_count"])
    assert oracle.leaf_sets(a["perm"], a["leaf_start"], a["leaf_count"]) == \
        oracle.leaf_sets(b["perm"], b["leaf_start"], b["leaf_count"])


def test_tree_edge_cases(oracle):
    one = oracle.build_tree(_uniform(1, 4), 2, 4)
    assert one["leaf_count"].tolist() == [1]
    two = oracle.build_tree(_uniform(2, 4), 1, 4)
    assert two["leaf_count"].sum() == 2
    small = oracle.build_tree(_uniform(40, 6), 33, 66)           # both root children below MIN: one bucket
    assert small["leaf_count"].tolist() == [40]
    same = np.zeros((300, 5), np.float32)                        # coincident points: depth limit, forced leaves
    forced = oracle.build_tree(same, 8, 16, max_depth=10)
    assert forced["leaf_count"].sum() == 300 and forced["leaf_count"].max() <= 16


@pytest.mark.parametrize("N,D,K", [(4000, 32, 16), (2000, 100, 32), (3000, 3, 40)])
def test_bucket_update_reference_order_equals_canonical(oracle, N, D, K):
    X = _uniform(N, D, 5)
    i_ref, d_ref = oracle.init_lists(N, K)
    i_can, d_can = i_ref.copy(), d_ref.copy()
    for t in range(3):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=t)
        i_ref, d_ref = oracle.bucket_knn_ref(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], i_ref, d_ref)
        i_can, d_can = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], i_can, d_can)
        si, sd = oracle.sort_rows(i_ref, d_ref)
        np.testing.assert_array_equal(si, i_can)
        np.testing.assert_array_equal(sd, d_can)
    assert (i_can >= 0).all()                                   # min >= K+1: no empty slot survives


def test_bucket_update_with_ties_matches_up_to_tie_groups(oracle):
    """Integer data: the reference-order rule keeps the earlier arrival among
    equal distances, the canonical rule the lower index; distances agree and
    indices agree outside the tie group at the K-th distance."""
    rng = np.random.default_rng(7)
    X = rng.integers(0, 3, (1500, 6)).astype(np.float32)
    K = 8
    tr = oracle.build_tree(X, 9, 40, seed=0, max_depth=300)
    i0, d0 = oracle.init_lists(len(X), K)
    ri, rd = oracle.sort_rows(*oracle.bucket_knn_ref(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], i0, d0))
    ci, cd = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], i0, d0)
    np.testing.assert_array_equal(rd, cd)
    for p in range(len(X)):
        inner = cd[p] < cd[p, -1]
        assert set(ri[p][inner]) == set(ci[p][inner])


def test_exploration_reference_order_equals_canonical(oracle):
    N, D, K = 3000, 20, 12
    X = _uniform(N, D, 6)
    idx, dist = oracle.init_lists(N, K)
    for t in range(2):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=t)
        idx, dist = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
    a = oracle.sort_rows(*oracle.explore_ref(X, idx, idx, dist))
    b = oracle.explore(X, idx, idx, dist)
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])
    part = oracle.explore(X, idx, idx, dist, 100, 900)
    np.testing.assert_array_equal(part[0][100:900], b[0][100:900])
    np.testing.assert_array_equal(part[0][:100], idx[:100])


def test_merge_lists_is_the_union_top_k(oracle):
    N, D, K = 2000, 16, 10
    X = _uniform(N, D, 8)
    parts = []
    for g in range(3):
        i0, d0 = oracle.init_lists(N, K)
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=40 + g)
        parts.append(oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], i0, d0))
    mi, md = oracle.merge_lists([p[0] for p in parts], [p[1] for p in parts])
    # sequential accumulation over the same trees gives the same lists
    si, sd = oracle.init_lists(N, K)
    for g in range(3):
        tr = oracle.build_tree(X, K + 1, 2 * K + 2, seed=40 + g)
        si, sd = oracle.bucket_knn(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], si, sd)
    np.testing.assert_array_equal(mi, si)
    np.testing.assert_array_equal(md, sd)


def test_bruteforce_and_recall(oracle):
    N, D, K = 1500, 12, 9
    X = _uniform(N, D, 9)
    bi, bd, threads = oracle.bruteforce_knn(X, K)
    assert threads >= 1
    d2 = ((X[:, None, :].astype(np.float64) - X[None, :, :]) ** 2).sum(-1)
    order = np.argsort(d2, axis=1, kind="stable")[:, :K]
    assert (bi[:, 0] == np.arange(N)).all()
    np.testing.assert_allclose(bd, np.take_along_axis(d2, order, 1), rtol=1e-5, atol=1e-7)   # 1e-5 relative
    assert oracle.recall(order.astype(np.int32), bi) > 0.999
    assert oracle.recall(bi, bi) == 1.0
    shuffled = bi[:, ::-1].copy()
    assert oracle.recall(bi, shuffled) == 1.0
    wrong = np.full_like(bi, -1)
    assert oracle.recall(bi, wrong) == 0.0


# ---------------------------------------------------------------- query path
@pytest.mark.parametrize("N,D,MIN,MAX", [(3000, 17, 8, 24), (5000, 32, 33, 66), (2000, 3, 4, 12),
                                         (4000, 100, 10, 40), (100, 16, 33, 66), (1, 4, 2, 4)])
def test_routing_sends_a_base_point_to_its_own_bucket(oracle, N, D, MIN, MAX):
    """A query equal to base point p takes p's side at every split, and follows p
    when p's side dissolves: it must end in p's bucket.  The tree itself is the
    one build_tree gives."""
    X = _uniform(N, D, 3)
    t0 = oracle.build_tree(X, MIN, MAX, seed=3)
    t = oracle.build_tree_route(X, X, MIN, MAX, seed=3)
    np.testing.assert_array_equal(t["perm"], t0["perm"])
    np.testing.assert_array_equal(t["leaf_start"], t0["leaf_start"])
    np.testing.assert_array_equal(t["leaf_count"], t0["leaf_count"])
    start_of, count_of = np.empty(N, np.int32), np.empty(N, np.int32)
    for s, c in zip(t["leaf_start"], t["leaf_count"]):
        start_of[t["perm"][s:s + c]] = s
        count_of[t["perm"][s:s + c]] = c
    np.testing.assert_array_equal(t["q_start"], start_of)
    np.testing.assert_array_equal(t["q_count"], count_of)


def test_routing_follows_the_split_rule_of_the_recorded_tree(oracle):
    """Walk the recorded tree by hand: at row r the query goes right iff n.q < c;
    a side without a row of its own leads to a leaf or to the sibling's row."""
    N, NQ, D, MIN, MAX = 3000, 400, 9, 6, 14
    X, Q = _uniform(N, D, 5), _uniform(NQ, D, 6)
    rec = oracle.build_tree(X, MIN, MAX, seed=8, record=True)
    t = oracle.build_tree_route(X, Q, MIN, MAX, seed=8)
    table = rec["table"]
    starts = set(int(s) for s in t["leaf_start"])
    assert set(int(s) for s in t["q_start"]) <= starts
    # every query's bucket must be on the query's side of the ROOT hyperplane
    n, c = oracle.hyperplane(X[table[0, 0]], X[table[0, 1]], True)
    root_right = np.array([oracle.project(n, q) < c for q in Q])
    base_right = np.array([oracle.project(n, x) < c for x in X])
    n_left = int((~base_right).sum())
    if n_left >= MIN and N - n_left >= MIN:       # neither side dissolved
        assert ((t["q_start"] >= n_left) == root_right).all()


def test_query_update_reference_order_equals_canonical(oracle):
    N, NQ, D, K = 4000, 1200, 20, 10
    X, Q = _uniform(N, D, 11), _uniform(NQ, D, 12)
    i0, d0 = oracle.init_lists(NQ, K, self_in_row=False)
    ia, da, ir, dr = i0, d0, i0, d0
    for seed in (1, 2, 3):
        t = oracle.build_tree_route(X, Q, 8, 24, seed=seed)
        ia, da = oracle.ann_bucket_knn(X, Q, K, t["perm"], t["q_start"], t["q_count"], ia, da)
        ir, dr = oracle.ann_bucket_knn_ref(X, Q, K, t["perm"], t["q_start"], t["q_count"], ir, dr)
        si, sd = oracle.sort_rows(ir, dr)
        np.testing.assert_array_equal(ia, si)
        np.testing.assert_array_equal(da.view(np.int32), sd.view(np.int32))
    # each row holds the K nearest of the union of the three buckets it met
    assert (np.diff(da, axis=1) >= 0).all()


def test_query_forest_recall_grows_with_trees(oracle):
    X, Q = _uniform(4000, 8, 13), _uniform(500, 8, 14)
    K = 8
    bi, bd = oracle.bruteforce_ann(X, Q, K)
    d2 = ((Q[:, None, :].astype(np.float64) - X[None, :, :]) ** 2).sum(-1)
    np.testing.assert_allclose(bd, np.sort(d2, axis=1)[:, :K], rtol=1e-5, atol=1e-7)   # 1e-5 relative
    r = [oracle.recall(bi, oracle.ann_forest(X, Q, K, T, 9, 18, seed=2)[0]) for T in (1, 4, 16)]
    assert r[0] < r[1] < r[2] and r[2] > 0.9


# ---------------------------------------------------------------- symmetric closure
def test_symmetric_closure_is_the_union_with_the_transpose(oracle):
    N, D, K = 400, 5, 6
    X = _uniform(N, D, 21)
    bi, bd, _ = oracle.bruteforce_knn(X, K)
    bi[::13, 2] = -1                                   # empty slots are skipped
    off, ind, val = oracle.symmetrize(bi, bd)
    A = np.zeros((N, N), bool)
    W = np.zeros((N, N), np.float32)
    for p in range(N):
        for k in range(K):
            q = bi[p, k]
            if q >= 0:
                A[p, q] = True
                W[p, q] = bd[p, k]
    S = A | A.T
    assert off[0] == 0 and off[-1] == S.sum() == len(ind)
    for p in range(N):
        row = ind[off[p]:off[p + 1]]
        np.testing.assert_array_equal(row, np.nonzero(S[p])[0])             # ordered by index, distinct
        for q, v in zip(row, val[off[p]:off[p + 1]]):
            assert v == (W[p, q] if A[p, q] else W[q, p])                     # the edge's own distance
    off2, ind2, none = oracle.symmetrize(bi)
    np.testing.assert_array_equal(off2, off)
    np.testing.assert_array_equal(ind2, ind)
    assert none is None
