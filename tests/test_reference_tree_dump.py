"""Whole trees as the reference built them, node by node (tests/golden/ref_tree_*.npz: dumps of
the reference's own index tree, written by the scratch build of oracle/patch_ref_dump.py and
tests/golden/make_ref_tree_golden.py on a B200).

The dump has every node's hyperplane, so nothing about the reference's sampling has to be
guessed: the pair (p1, p2) a node sampled is read back from its normal x[p1] - x[p2], the offset
must have the restated rule's bits, the restated side rule must send the node's points to its
children exactly as the reference did, and a tree that REPLAYS those pairs (the explicit split
table) must come out with the reference's buckets -- on the CPU oracle and on the GPU.
"""
import glob
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
PATHS = sorted(glob.glob(os.path.join(HERE, "golden", "ref_tree_*.npz")))


class RefTree(object):
    """The dump as a tree: node g of level d is row off[d] + g."""

    def __init__(self, path):
        z = np.load(path)
        self.X = z["X"]
        self.N, self.D, self.MIN, self.MAX = [int(v) for v in z["params"]]
        self.n_level = z["n_level"]
        self.off = np.concatenate([[0], np.cumsum(self.n_level)]).astype(int)
        self.planes, self.children = z["planes"], z["children"]
        self.is_leaf, self.count = z["is_leaf"], z["count"]
        sizes = z["bucket_sizes"]
        self.buckets = {frozenset(int(v) for v in row[:n]) for row, n in zip(z["buckets"], sizes)}
        assert sum(len(b) for b in self.buckets) == self.N

    def child(self, d, g, side):
        k = int(self.children[self.off[d] + g][side])
        return None if k < 0 else (d + 1, k)

    def row(self, d, g):
        return self.off[d] + g

    def dead(self, d, g):
        # a child that was too small and dissolved into its sibling stays behind as an empty node
        r = self.row(d, g)
        return self.count[r] == 0 and not self.is_leaf[r]


def _pair_of_normal(X, ids, normal):
    """(p1, p2) among ids with x[p1] - x[p2] == normal in every coordinate (fp32), or None."""
    k = int(np.argmax(np.abs(normal)))
    col = X[ids, k]
    order = np.argsort(col, kind="stable")
    sorted_col = col[order]
    for a_pos, a in enumerate(ids):
        want = np.float32(X[a, k] - normal[k])
        lo = np.searchsorted(sorted_col, want - np.float32(4e-7) * max(1.0, abs(float(want))), "left")
        hi = np.searchsorted(sorted_col, want + np.float32(4e-7) * max(1.0, abs(float(want))), "right")
        for j in range(lo, hi):
            b = ids[order[j]]
            if b != a and np.array_equal((X[a] - X[b]).astype(np.float32), normal):
                return int(a), int(b)
    return None


def _walk(oracle, t):
    """Top-down over the dump.  Returns (replay table, leaf sets reached by the restated side rule)."""
    X = t.X
    table = []          # rows {p1, p2, left row, right row}
    leaves = []

    def visit(d, g, ids, is_root):
        r = t.row(d, g)
        assert t.count[r] == len(ids), "node (%d,%d): %d points in the dump, %d by the restated rules" % (
            d, g, t.count[r], len(ids))
        if t.is_leaf[r]:
            leaves.append(frozenset(int(v) for v in ids))
            return -1
        normal, c_ref = t.planes[r][:t.D].copy(), t.planes[r][t.D]
        pair = _pair_of_normal(X, ids, normal)
        assert pair is not None, "node (%d,%d): no pair of its own points has the dumped normal" % (d, g)
        n, c = oracle.hyperplane(X[pair[0]], X[pair[1]], is_root)
        assert np.array_equal(n, normal)
        assert np.float32(c).view(np.int32) == np.float32(c_ref).view(np.int32), \
            "node (%d,%d): offset %r, restated %r" % (d, g, c_ref, c)
        right = np.array([oracle.project(n, X[p]) < c for p in ids], bool)
        me = len(table)
        table.append([pair[0], pair[1], -1, -1])
        kids = [t.child(d, g, 0), t.child(d, g, 1)]
        live = [k for k in kids if k is not None and not t.dead(*k)]
        if len(live) == 1:      # the other side was empty or dissolved: everything goes on together
            side = kids.index(live[0])
            sub = visit(live[0][0], live[0][1], ids, False)
            table[me][2 + side] = sub
        else:
            assert len(live) == 2
            for side, part in ((0, ids[~right]), (1, ids[right])):
                table[me][2 + side] = visit(kids[side][0], kids[side][1], part, False)
        return me

    visit(0, 0, np.arange(t.N, dtype=np.int32), True)
    return np.array(table, np.int32).reshape(-1, 4), leaves


@pytest.mark.parametrize("path", PATHS)
def test_restated_rules_reproduce_the_reference_tree_node_by_node(oracle, path):
    t = RefTree(path)
    table, leaves = _walk(oracle, t)
    assert set(leaves) == t.buckets
    assert min(len(b) for b in leaves) >= t.MIN and max(len(b) for b in leaves) <= t.MAX


@pytest.mark.parametrize("path", PATHS)
def test_oracle_tree_replaying_the_reference_pairs_has_the_reference_buckets(oracle, path):
    t = RefTree(path)
    table, _ = _walk(oracle, t)
    tr = oracle.build_tree(t.X, t.MIN, t.MAX, seed=12345, table=table)
    got = {frozenset(int(v) for v in tr["perm"][s:s + c]) for s, c in zip(tr["leaf_start"], tr["leaf_count"])}
    assert got == t.buckets


@pytest.mark.gpu
@pytest.mark.parametrize("path", PATHS)
def test_gpu_tree_replaying_the_reference_pairs_has_the_reference_buckets(oracle, path):
    import torch
    from gpu_rsfk.device import DeviceForest
    t = RefTree(path)
    table, _ = _walk(oracle, t)
    dev = torch.device("cuda", 0)
    f = DeviceForest(dev)
    f.tree_build(torch.from_numpy(t.X).to(dev), t.MIN, t.MAX, seed=999, table=torch.from_numpy(table).to(dev))
    perm, ls, lc = f.tree_export()
    got = {frozenset(int(v) for v in perm[s:s + c]) for s, c in zip(ls, lc)}
    assert got == t.buckets


def test_dump_patch_applies_to_the_reference_driver(oracle, tmp_path):
    """The script that adds the tree dump to a scratch copy of the reference's driver finds its two
    anchors exactly once (skipped where the reference's sources are not on this machine)."""
    import subprocess
    import sys
    ref = oracle.reference_root()
    if ref is None:
        pytest.skip("reference sources not on this machine")
    out = tmp_path / "rsfk.cu"
    script = os.path.join(os.path.dirname(HERE), "oracle", "patch_ref_dump.py")
    subprocess.run([sys.executable, script, ref, str(out)], check=True)
    patched = out.read_text()
    original = open(os.path.join(ref, "src", "rsfk.cu")).read()
    assert patched.count("rsfk_b200_dump_tree(") == 2          # the definition and the one call
    assert patched.count('getenv("RSFK_DUMP_TREE")') == 1
    # nothing of the reference is removed: taking the two additions out gives the original back
    added = len(patched) - len(original)
    assert added > 0 and patched.replace("\r", "").count("\n") > original.count("\n")
