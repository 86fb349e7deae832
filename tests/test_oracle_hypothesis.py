"""Property tests of the CPU oracle on tiny random problems (hypothesis): the
invariants every tree, bucket update and query descent must keep whatever the
sizes, including degenerate ones (N below the leaf size, one dimension, repeated
points)."""
import numpy as np
from hypothesis import given, settings, strategies as st, HealthCheck

SETTINGS = dict(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])


def _points(seed, N, D, repeats):
    rng = np.random.default_rng(seed)
    X = rng.uniform(0, 1, (N, D)).astype(np.float32)
    if repeats and N > 3:                       # a few coincident points
        X[rng.integers(0, N, N // 3)] = X[0]
    return X


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), N=st.integers(1, 300), D=st.integers(1, 40), MIN=st.integers(1, 20),
       extra=st.integers(0, 30), repeats=st.booleans())
def test_tree_is_a_partition_with_bounded_leaves(oracle, seed, N, D, MIN, extra, repeats):
    MAX = 2 * MIN + extra
    X = _points(seed, N, D, repeats)
    t = oracle.build_tree(X, MIN, MAX, max_depth=40, seed=seed)
    perm, ls, lc = t["perm"], t["leaf_start"], t["leaf_count"]
    assert np.array_equal(np.sort(perm), np.arange(N))
    assert lc.sum() == N and (lc > 0).all()
    assert np.array_equal(ls, np.cumsum(lc) - lc)
    if N > MAX:
        assert lc.max() <= MAX                  # also at the depth limit: open nodes are cut to <= MAX
    # same seed, same tree
    t2 = oracle.build_tree(X, MIN, MAX, max_depth=40, seed=seed)
    assert np.array_equal(t2["perm"], perm)


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), N=st.integers(2, 250), D=st.integers(1, 24), K=st.integers(1, 40),
       MIN=st.integers(1, 12))
def test_bucket_update_gives_the_k_nearest_of_each_bucket(oracle, seed, N, D, K, MIN):
    MAX = 3 * MIN + 2
    X = _points(seed, N, D, False)
    t = oracle.build_tree(X, MIN, MAX, max_depth=60, seed=seed)
    i0, d0 = oracle.init_lists(N, K)
    idx, dist = oracle.bucket_knn(X, K, t["perm"], t["leaf_start"], t["leaf_count"], i0, d0)
    assert (idx[:, 0] == np.arange(N)).all() and (dist[:, 0] == 0).all()
    for s, c in zip(t["leaf_start"], t["leaf_count"]):
        members = t["perm"][s:s + c]
        for p in members[:3]:
            want = sorted((np.float32(oracle.dist_sqr(X[p], X[q])), int(q)) for q in members)
            got = [(np.float32(dist[p, k]), int(idx[p, k])) for k in range(K) if idx[p, k] >= 0]
            assert got == want[:K][:len(got)] and len(got) == min(K, len(members))
    # slot-level restatement agrees where no two distances tie
    ri, rd = oracle.bucket_knn_ref(X, K, t["perm"], t["leaf_start"], t["leaf_count"], i0, d0)
    si, sd = oracle.sort_rows(ri, rd)
    assert np.array_equal(sd, dist)


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), N=st.integers(1, 250), NQ=st.integers(1, 60), D=st.integers(1, 24),
       MIN=st.integers(1, 12), extra=st.integers(0, 12))
def test_query_descent_ends_in_a_leaf_and_twins_agree(oracle, seed, N, NQ, D, MIN, extra):
    MAX = 2 * MIN + extra
    X = _points(seed, N, D, False)
    rng = np.random.default_rng(seed + 1)
    Q = rng.uniform(0, 1, (NQ, D)).astype(np.float32)
    Q[: min(NQ, N)] = X[: min(NQ, N)]           # some queries are base points
    t = oracle.build_tree_route(X, Q, MIN, MAX, max_depth=40, seed=seed)
    starts = dict(zip(t["leaf_start"].tolist(), t["leaf_count"].tolist()))
    for q in range(NQ):
        assert int(t["q_start"][q]) in starts and starts[int(t["q_start"][q])] == int(t["q_count"][q])
    own = np.empty(N, np.int64)
    for s, c in starts.items():
        own[t["perm"][s:s + c]] = s
    for q in range(min(NQ, N)):                 # a base point used as a query finds its own leaf
        assert t["q_start"][q] == own[q]
    K = 5
    i0, d0 = oracle.init_lists(NQ, K, self_in_row=False)
    idx, dist = oracle.ann_bucket_knn(X, Q, K, t["perm"], t["q_start"], t["q_count"], i0, d0)
    for q in range(min(NQ, 5)):
        members = t["perm"][t["q_start"][q]: t["q_start"][q] + t["q_count"][q]]
        want = sorted((np.float32(oracle.dist_sqr(Q[q], X[b])), int(b)) for b in members)[:K]
        got = [(np.float32(dist[q, k]), int(idx[q, k])) for k in range(K) if idx[q, k] >= 0]
        assert got == want
