"""Generates tests/golden/ref_*.npz from the REFERENCE project's own CUDA
library (unmodified sources compiled by ``make -C oracle ref`` into
oracle/_ref/librsfk_ref.so).  Needs a GPU; run once on a GPU box:

    python tests/golden/make_ref_golden.py <output directory>

and commit the small .npz files it writes.  They pin the CPU oracle (and
through it the sm_100a kernels) to what the reference binary really computes:

* ref_buckets_*: one tree with K >= max_tree_children and empty start lists, so
  every row returns its whole leaf bucket: bucket membership of a real
  reference tree plus the reference's squared distance for every in-bucket pair.
* ref_explore_*: n_trees = 0 and valid start lists: the exploration sweep is
  then a deterministic function of its inputs.
* ref_update_*: one tree over N <= max_tree_children-2 points (root + two leaves)
  with K smaller than the buckets, and the same tree with K >= the bucket size,
  which reveals the two buckets: the bucket update rule on known buckets.
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_ref():
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "librsfk_ref.so"))
    L.pymodule_rsfk_knn.restype = None
    L.pymodule_rsfk_knn.argtypes = [ctypes.c_int] * 10 + [ctypes.c_void_p] * 4
    return L


def ref_knn(L, X, K, n_trees, MIN, MAX, seed, sweeps, idx=None, dist=None):
    N, D = X.shape
    if idx is None:
        idx = np.full((N, K), -1, np.int32)
        dist = np.full((N, K), np.inf, np.float32)
        idx[:, 0] = np.arange(N)
        dist[:, 0] = 0
    idx, dist = idx.copy(), dist.copy()
    log = np.zeros(16 * max(n_trees, 1) + 2, np.float32)
    L.pymodule_rsfk_knn(n_trees, K, N, D, MIN, MAX, 5000, 0, seed, sweeps,
                        X.ctypes.data, idx.ctypes.data, dist.ctypes.data, log.ctypes.data)
    return idx, dist


def main(out):
    from oracle import rsfk_oracle as orc
    os.makedirs(out, exist_ok=True)
    L = load_ref()
    rng = np.random.default_rng(2024)

    # -- whole buckets and their distances ----------------------------------
    for tag, (N, D, MIN, MAX) in {"a": (600, 37, 20, 40), "b": (900, 100, 12, 30), "c": (500, 2, 10, 24),
                                  "d": (400, 200, 16, 48), "e": (700, 33, 8, 16)}.items():
        X = rng.uniform(0, 1, (N, D)).astype(np.float32)
        K = MAX + 1
        idx, dist = ref_knn(L, X, K, 1, MIN, MAX, 11, 0)
        np.savez_compressed(os.path.join(out, "ref_buckets_%s.npz" % tag), X=X, idx=idx, dist=dist,
                            params=np.array([N, D, MIN, MAX, K], np.int32))

    # -- exploration sweeps ----------------------------------------------------
    for tag, (N, D, K, sweeps) in {"a": (1500, 24, 8, 1), "b": (1200, 100, 16, 2), "c": (800, 3, 32, 1),
                                   "d": (1000, 64, 40, 1)}.items():
        X = rng.uniform(0, 1, (N, D)).astype(np.float32)
        idx, dist = orc.init_lists(N, K)
        for t in range(2):
            tr = orc.build_tree(X, K + 1, 2 * K + 2, seed=t)
            idx, dist = orc.bucket_knn_ref(X, K, tr["perm"], tr["leaf_start"], tr["leaf_count"], idx, dist)
        assert (idx >= 0).all()
        oi, od = ref_knn(L, X, K, 0, K + 1, 2 * K + 2, 0, sweeps, idx, dist)
        np.savez_compressed(os.path.join(out, "ref_explore_%s.npz" % tag), X=X, idx_in=idx, dist_in=dist,
                            idx_out=oi, dist_out=od, params=np.array([N, D, K, sweeps], np.int32))

    # -- bucket update rule on a two-leaf tree -------------------------------
    for tag, (N, D, K, MAX) in {"a": (120, 20, 10, 128), "b": (200, 64, 32, 256), "c": (90, 5, 4, 100)}.items():
        X = rng.uniform(0, 1, (N, D)).astype(np.float32)
        big_i, big_d = ref_knn(L, X, N, 1, 1, MAX, 5, 0)          # reveals the two buckets
        small_i, small_d = ref_knn(L, X, K, 1, 1, MAX, 5, 0)      # same seed: same root pair
        np.savez_compressed(os.path.join(out, "ref_update_%s.npz" % tag), X=X, big_idx=big_i, big_dist=big_d,
                            idx=small_i, dist=small_d, params=np.array([N, D, K, MAX], np.int32))
    print("wrote fixtures to", out)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
