"""Generates tests/golden/ref_tree_*.npz: whole trees as the REFERENCE built them, with the
hyperplane of every node, from the reference's sources plus the dump that
``oracle/patch_ref_dump.py`` adds to a scratch copy (``make -C oracle ref_dump`` ->
oracle/_ref/librsfk_ref_dump.so).  Needs a GPU; run once on a GPU box:

    python tests/golden/make_ref_tree_golden.py <output directory>

and commit the small .npz files it writes.

The reference keeps a tree only on its query path (RSFKIndexTree, src/include/rsfk.h:89-127), so
``pymodule_rsfk_knn_ann`` is driven the way its own experiment drives it (test_ann.py:80-81: the
query set is the base set, NQ = N; the only shape whose accesses are all in bounds, src/rsfk.cu:396-403)
with one tree.  The dump holds, level by level, each node's hyperplane (normal, offset:
src/kernels/create_node.cu:42-134), parent, children, leaf flag and point count, and the bucket table.
A fixture keeps the points, those arrays and the buckets.
"""
import ctypes
import os
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_ref():
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "librsfk_ref_dump.so"))
    L.pymodule_rsfk_knn_ann.restype = None
    L.pymodule_rsfk_knn_ann.argtypes = [ctypes.c_int] * 11 + [ctypes.c_void_p] * 5
    return L


def read_dump(path):
    raw = open(path, "rb").read()
    magic, D, depths, total_leaves, max_child = struct.unpack_from("<5i", raw, 0)
    assert magic == 0x52534654
    off = 20
    out = dict(D=D, depths=depths, total_leaves=total_leaves, max_child=max_child)
    planes, parents, children, is_leaf, count, n_level = [], [], [], [], [], []
    for d in range(depths):
        (n,) = struct.unpack_from("<i", raw, off); off += 4
        n_level.append(n)
        planes.append(np.frombuffer(raw, np.float32, n * (D + 1), off).reshape(n, D + 1)); off += 4 * n * (D + 1)
        parents.append(np.frombuffer(raw, np.int32, n, off)); off += 4 * n
        children.append(np.frombuffer(raw, np.int32, 2 * n, off).reshape(n, 2)); off += 8 * n
        is_leaf.append(np.frombuffer(raw, np.uint8, n, off)); off += n
        count.append(np.frombuffer(raw, np.int32, n, off)); off += 4 * n
    level_count = np.frombuffer(raw, np.int32, depths, off); off += 4 * depths
    buckets = np.frombuffer(raw, np.int32, total_leaves * max_child, off).reshape(total_leaves, max_child)
    off += 4 * total_leaves * max_child
    sizes = np.frombuffer(raw, np.int32, total_leaves, off); off += 4 * total_leaves
    assert off == len(raw)
    # one flat table of nodes: level, plane, parent (index inside the level above), children
    # (indices inside the level below), leaf flag, count
    out.update(n_level=np.array(n_level, np.int32), level_count=level_count.copy(),
               planes=np.concatenate(planes, 0) if planes else np.zeros((0, D + 1), np.float32),
               parents=np.concatenate(parents), children=np.concatenate(children, 0),
               is_leaf=np.concatenate(is_leaf), count=np.concatenate(count),
               buckets=buckets.copy(), bucket_sizes=sizes.copy())
    return out


def main(out):
    os.makedirs(out, exist_ok=True)
    L = load_ref()
    rng = np.random.default_rng(7071)
    cases = {"a": (3000, 8, 20, 60), "b": (2500, 32, 33, 66), "c": (2000, 100, 16, 40), "d": (4000, 2, 64, 256)}
    for tag, (N, D, MIN, MAX) in cases.items():
        X = rng.uniform(0, 1, (N, D)).astype(np.float32)
        K = 4
        idx = np.full((N, K), -1, np.int32)
        dist = np.full((N, K), np.inf, np.float32)
        log = np.zeros(16 + 2, np.float32)
        Q = X.copy()
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "tree.bin")
            os.environ["RSFK_DUMP_TREE"] = path
            L.pymodule_rsfk_knn_ann(1, K, N, N, D, MIN, MAX, 5000, 0, 11, 0,
                                    X.ctypes.data, Q.ctypes.data, idx.ctypes.data, dist.ctypes.data,
                                    log.ctypes.data)
            del os.environ["RSFK_DUMP_TREE"]
            t = read_dump(path)
        sizes = t["bucket_sizes"]
        print(tag, "levels", t["depths"], "leaves", t["total_leaves"], "bucket sizes", int(sizes.min()), "..",
              int(sizes.max()), "points in buckets", int(sizes.sum()), "of", N, flush=True)
        np.savez_compressed(os.path.join(out, "ref_tree_%s.npz" % tag), X=X,
                            params=np.array([N, D, MIN, MAX], np.int32), **{k: v for k, v in t.items()
                                                                           if isinstance(v, np.ndarray)},
                            dims=np.array([t["D"], t["depths"], t["total_leaves"], t["max_child"]], np.int32))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
