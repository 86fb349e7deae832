"""Generates tests/golden/ref_ann_*.npz from the REFERENCE project's own CUDA
library (unmodified sources compiled by ``make -C oracle ref`` into
oracle/_ref/librsfk_ref.so).  Needs a GPU; run once on a GPU box:

    python tests/golden/make_ref_ann_golden.py <output directory>

and commit the small .npz files it writes.

The reference's query entry point, ``pymodule_rsfk_knn_ann``, is driven the way
the reference's own experiment drives it (``test_ann.py:80-81``): the query set
IS the base set (NQ = N).  That is also the only shape for which reading the
reference shows every access in bounds: its query driver sizes the per-query
arrays by NQ but runs ``build_tree_bucket_points`` over N entries of them and
into a bucket table sized for the base buckets (``src/rsfk.cu:396-403``).

One tree, empty start lists and K > max_tree_children: every query row then
returns its whole leaf bucket, in the slots the reference's replace-the-worst
rule fills, with the reference's squared distances.
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
    L.pymodule_rsfk_knn_ann.restype = None
    L.pymodule_rsfk_knn_ann.argtypes = [ctypes.c_int] * 11 + [ctypes.c_void_p] * 5
    return L


def ref_ann_self(L, X, K, MIN, MAX, seed):
    N, D = X.shape
    Q = X.copy()
    idx = np.full((N, K), -1, np.int32)
    dist = np.full((N, K), np.inf, np.float32)
    log = np.zeros(16 + 2, np.float32)
    L.pymodule_rsfk_knn_ann(1, K, N, N, D, MIN, MAX, 5000, 0, seed, 0,
                            X.ctypes.data, Q.ctypes.data, idx.ctypes.data, dist.ctypes.data,
                            log.ctypes.data)
    return idx, dist


def main(out):
    os.makedirs(out, exist_ok=True)
    L = load_ref()
    rng = np.random.default_rng(4048)
    for tag, (N, D, MIN, MAX) in {"a": (600, 37, 20, 40), "b": (800, 100, 12, 30), "c": (500, 2, 10, 24),
                                  "d": (700, 33, 8, 16)}.items():
        X = rng.uniform(0, 1, (N, D)).astype(np.float32)
        K = MAX + 1
        idx, dist = ref_ann_self(L, X, K, MIN, MAX, 11)
        np.savez_compressed(os.path.join(out, "ref_ann_%s.npz" % tag), X=X, idx=idx, dist=dist,
                            params=np.array([N, D, MIN, MAX, K], np.int32))
        print(tag, "rows with self:", int((idx == np.arange(N)[:, None]).any(1).sum()), "of", N, flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE))
