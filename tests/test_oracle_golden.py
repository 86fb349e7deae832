"""The CPU oracle against outputs of the reference project's own CUDA library.

The fixtures under tests/golden/ were produced on a B200 by
tests/golden/make_ref_golden.py from the reference's unmodified sources.  They
pin the oracle's distance bits, bucket update rule and exploration sweep; the
tree's split rule is pinned by recovering, for a reference tree, split pairs
that reproduce its buckets exactly."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(pattern):
    files = sorted(glob.glob(os.path.join(GOLDEN, pattern)))
    assert files, "fixtures missing: " + pattern
    return files


@pytest.mark.parametrize("path", _load("ref_buckets_*.npz"))
def test_reference_distance_bits_and_bucket_partition(oracle, path):
    z = np.load(path)
    X, idx, dist = z["X"], z["idx"], z["dist"]
    N, D, MIN, MAX, K = [int(v) for v in z["params"]]
    # every row lists its whole bucket (K > MAX): buckets are the row sets
    buckets = {}
    for p in range(N):
        members = frozenset(idx[p][idx[p] >= 0].tolist())
        assert p in members
        buckets.setdefault(members, 0)
        buckets[members] += 1
    sizes = []
    for members, rows in buckets.items():
        assert rows == len(members)            # all members agree on the bucket
        sizes.append(len(members))
    assert sum(sizes) == N
    assert min(sizes) >= MIN and max(sizes) <= MAX
    # the oracle's squared distance carries the reference's bits for every pair
    checked = 0
    for p in range(N):
        for k in range(K):
            q = idx[p, k]
            if q < 0 or q == p:
                continue
            assert np.float32(oracle.dist_sqr(X[p], X[q])) == dist[p, k], (p, q)
            checked += 1
    assert checked > N
    # and the canonical bucket update over those buckets returns the same rows
    perm = np.concatenate([np.array(sorted(b), np.int32) for b in buckets])
    counts = np.array([len(b) for b in buckets], np.int32)
    starts = (np.cumsum(counts) - counts).astype(np.int32)
    i0, d0 = oracle.init_lists(N, K)
    oi, od = oracle.bucket_knn(X, K, perm, starts, counts, i0, d0)
    si, sd = oracle.sort_rows(idx, dist)
    np.testing.assert_array_equal(oi, si)
    np.testing.assert_array_equal(od, sd)


@pytest.mark.parametrize("path", _load("ref_explore_*.npz"))
def test_reference_exploration_sweep(oracle, path):
    z = np.load(path)
    X = z["X"]
    N, D, K, sweeps = [int(v) for v in z["params"]]
    idx, dist = z["idx_in"], z["dist_in"]
    ci, cd = oracle.sort_rows(idx, dist)
    for _ in range(sweeps):
        idx, dist = oracle.explore_ref(X, idx, idx, dist)      # slot-for-slot restatement
        ci, cd = oracle.explore(X, ci, ci, cd)                 # canonical statement
    np.testing.assert_array_equal(idx, z["idx_out"])
    np.testing.assert_array_equal(dist, z["dist_out"])
    si, sd = oracle.sort_rows(z["idx_out"], z["dist_out"])
    np.testing.assert_array_equal(ci, si)
    np.testing.assert_array_equal(cd, sd)


@pytest.mark.parametrize("path", _load("ref_update_*.npz"))
def test_reference_bucket_update_rule(oracle, path):
    z = np.load(path)
    X = z["X"]
    N, D, K, MAX = [int(v) for v in z["params"]]
    big = z["big_idx"]
    buckets = sorted({frozenset(r[r >= 0].tolist()) for r in big}, key=min)
    assert len(buckets) == 2 and sum(len(b) for b in buckets) == N
    perm = np.concatenate([np.array(sorted(b), np.int32) for b in buckets])
    counts = np.array([len(b) for b in buckets], np.int32)
    starts = (np.cumsum(counts) - counts).astype(np.int32)
    i0, d0 = oracle.init_lists(N, K)
    oi, od = oracle.bucket_knn(X, K, perm, starts, counts, i0, d0)
    ri, rd = oracle.bucket_knn_ref(X, K, perm, starts, counts, i0, d0)
    si, sd = oracle.sort_rows(z["idx"], z["dist"])
    np.testing.assert_array_equal(oi, si)
    np.testing.assert_array_equal(od, sd)
    ri, rd = oracle.sort_rows(ri, rd)
    np.testing.assert_array_equal(ri, si)
    np.testing.assert_array_equal(rd, sd)


@pytest.mark.parametrize("path", _load("ref_update_*.npz"))
def test_reference_root_split_is_reproduced_by_some_pair(oracle, path):
    """The two leaves of a reference tree over N <= MAX-2 points are the two
    sides of the root hyperplane of SOME pair of points; the oracle's split rule
    (n.x < c goes right, serial-sum offset at the root) must reproduce that
    partition exactly for at least one pair."""
    z = np.load(path)
    X = z["X"]
    N = X.shape[0]
    buckets = sorted({frozenset(r[r >= 0].tolist()) for r in z["big_idx"]}, key=min)
    target = np.zeros(N, bool)
    target[list(buckets[1])] = True
    found = None
    for p1 in range(N):
        for p2 in range(N):
            if p1 == p2 or target[p1] == target[p2]:
                continue
            n, c = oracle.hyperplane(X[p1], X[p2], True)
            # cheap float64 screen before the bit-exact check
            right = (X.astype(np.float64) @ n.astype(np.float64)) < float(c)
            if (right != target).sum() > 2 and (right == target).sum() > 2:
                continue
            exact = np.array([oracle.project(n, X[q]) < c for q in range(N)])
            if (exact == target).all() or (exact == ~target).all():
                found = (p1, p2)
                break
        if found:
            break
    assert found is not None


def _reconstruct(oracle, X, ids, label, MIN, MAX, is_root, depth=0):
    """True when the leaves below this node (label per point) can be produced by
    the restated rules from SOME split pair at every internal node."""
    n = len(ids)
    labels = np.unique(label)
    if len(labels) == 1:
        return (not is_root) and n <= MAX           # a leaf: at most MAX-2 points, or MAX-1..MAX after a merge
    if not is_root and n <= MAX - 2:
        return False                                # such a node would have been a leaf
    local = np.searchsorted(labels, label).astype(np.int32)
    if len(labels) > 64:
        return False
    for mask, _pair in oracle.find_leaf_separations(X, ids, local, is_root, MIN):
        right = np.array([(mask >> int(l)) & 1 for l in local], bool)
        if _reconstruct(oracle, X, ids[~right], label[~right], MIN, MAX, False, depth + 1) and \
           _reconstruct(oracle, X, ids[right], label[right], MIN, MAX, False, depth + 1):
            return True
    return False


@pytest.mark.parametrize("path", _load("ref_buckets_*.npz"))
def test_reference_tree_is_reproduced_by_the_restated_rules(oracle, path):
    """Whole reference trees (20-60 leaves, several levels): at every internal
    node some pair of the node's own points separates its leaves under the
    restated split rule (lane-strided offset below the root), both sides keep at
    least MIN points, and every group of at most MAX-2 points is a single leaf.
    This pins the non-root hyperplane arithmetic and the leaf/merge rule to the
    reference binary without knowing which pairs it sampled."""
    z = np.load(path)
    X, idx = z["X"], z["idx"]
    N, D, MIN, MAX, K = [int(v) for v in z["params"]]
    buckets = sorted({frozenset(r[r >= 0].tolist()) for r in idx}, key=min)
    label = np.empty(N, np.int32)
    for b, members in enumerate(buckets):
        label[list(members)] = b
    assert _reconstruct(oracle, X, np.arange(N, dtype=np.int32), label, MIN, MAX, True)


def _fill_order(K):
    """Slots in the order the reference's replace-the-worst rule fills an empty
    (all +inf) K-list.  Lane l of the warp scans slots l, l+32, ... and keeps its
    first strictly larger value; a shfl_down tree (16, 8, 4, 2, 1) then keeps the
    receiving lane's value on ties
    (src/kernels/build_tree_update_parents_ann.cu:300-345).  While an empty slot
    is left the winner does not depend on the finite values."""
    filled = np.zeros(K, bool)
    order = []
    for _ in range(K):
        val = np.full(32, -1.0)
        pos = np.full(32, -1)
        for lane in range(32):
            for k in range(lane, K, 32):
                v = 0.0 if filled[k] else np.inf
                if v > val[lane]:
                    val[lane], pos[lane] = v, k
        for off in (16, 8, 4, 2, 1):
            nv, npos = val.copy(), pos.copy()
            for lane in range(32 - off):
                if val[lane + off] > val[lane]:
                    nv[lane], npos[lane] = val[lane + off], pos[lane + off]
            val, pos = nv, npos
        order.append(int(pos[0]))
        filled[pos[0]] = True
    return order


@pytest.mark.parametrize("path", _load("ref_ann_*.npz"))
def test_reference_query_path_on_its_own_base_points(oracle, path):
    """pymodule_rsfk_knn_ann of the reference binary with the query set equal to
    the base set (tests/golden/make_ref_ann_golden.py), one tree, K > MAX."""
    z = np.load(path)
    X, idx, dist = z["X"], z["idx"], z["dist"]
    N, D, MIN, MAX, K = [int(v) for v in z["params"]]
    fill = _fill_order(K)
    # routing: a query equal to base point p ends in p's bucket, so the rows of the
    # members of a bucket all list that bucket, p itself at distance 0
    orders = {}
    for p in range(N):
        m = int((idx[p] >= 0).sum())
        seq = idx[p][fill[:m]]                  # bucket order as this row saw it
        assert (seq >= 0).all()                 # filled slots are exactly the first m of the fill order
        assert p in seq.tolist()
        assert dist[p][idx[p] == p][0] == 0.0
        key = frozenset(seq.tolist())
        orders.setdefault(key, []).append(tuple(seq.tolist()))
    sizes = []
    for members, seqs in orders.items():
        assert len(seqs) == len(members)        # every member routed here, nobody else
        assert len(set(seqs)) == 1              # all rows met the bucket in the same order
        sizes.append(len(members))
    assert sum(sizes) == N and min(sizes) >= MIN and max(sizes) <= MAX
    # update rule and distance bits: the oracle over the same buckets (same order)
    perm = np.concatenate([np.array(seqs[0], np.int32) for seqs in orders.values()])
    counts = np.array([len(seqs[0]) for seqs in orders.values()], np.int32)
    starts = (np.cumsum(counts) - counts).astype(np.int32)
    q_start, q_count = np.empty(N, np.int32), np.empty(N, np.int32)
    for s, c in zip(starts, counts):
        q_start[perm[s:s + c]] = s
        q_count[perm[s:s + c]] = c
    i0, d0 = oracle.init_lists(N, K, self_in_row=False)
    ri, rd = oracle.ann_bucket_knn_ref(X, X, K, perm, q_start, q_count, i0, d0)
    np.testing.assert_array_equal(ri, idx)                                   # slot for slot
    np.testing.assert_array_equal(rd.view(np.int32), dist.view(np.int32))    # bit for bit
    ci, cd = oracle.ann_bucket_knn(X, X, K, perm, q_start, q_count, i0, d0)
    si, sd = oracle.sort_rows(idx, dist)
    np.testing.assert_array_equal(ci, si)
    np.testing.assert_array_equal(cd.view(np.int32), sd.view(np.int32))
    # and the routing rule reproduces it: a tree whose buckets are these buckets sends
    # every base point, used as a query, to the bucket that holds it (property of
    # orc_build_tree_route, checked on the oracle's own trees in test_oracle_properties)
