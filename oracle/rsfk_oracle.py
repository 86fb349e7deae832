"""ctypes bindings of the CPU oracle (``rsfk_oracle.c``).  TEST INFRASTRUCTURE.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import
this module; the product never does.  The shared object is built by
``make -C oracle`` (``build()`` below runs it when the library is missing).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librsfk_oracle.so")
_lib = None

_f32 = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32 = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_c_int_p = ctypes.POINTER(ctypes.c_int)


def build(force=False):
    """Compile the C oracle next to its source (system gcc, OpenMP)."""
    src = os.path.join(_HERE, "rsfk_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def build_reference():
    """Compile the reference's own CUDA library into ``oracle/_ref`` when its
    sources are present on this machine; returns the path or None."""
    out = os.path.join(_HERE, "_ref", "librsfk_ref.so")
    tiles = os.path.join(_HERE, "_ref", "librsfk_ref_tiles.so")
    dump = os.path.join(_HERE, "_ref", "librsfk_ref_dump.so")
    wrapper = os.path.join(_HERE, "_ref", "ref_wrapper", "RSFK.py")
    if os.path.exists(out) and os.path.exists(tiles) and os.path.exists(dump) and os.path.exists(wrapper):
        return out
    ref = reference_root()
    if ref is None:
        return out if os.path.exists(out) else None
    subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "ref_tiles", "ref_dump", "ref_wrapper", "REF=" + ref])
    return out


def reference_wrapper_path():
    """The reference's own ctypes wrapper (python/gpu_rsfk/RSFK.py of the reference project):
    from its tree when that is on this machine, else the scratch copy the build left under
    oracle/_ref; None when there is neither."""
    ref = reference_root()
    if ref is not None:
        return os.path.join(ref, "python", "gpu_rsfk", "RSFK.py")
    copy = os.path.join(_HERE, "_ref", "ref_wrapper", "RSFK.py")
    return copy if os.path.exists(copy) else None


def reference_root():
    """Root of the reference project on this machine, or None: the environment variable
    RSFK_REFERENCE_ROOT, else a directory ``reference`` beside this repository."""
    ref = os.environ.get("RSFK_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if not os.path.exists(os.path.join(ref, "src", "python", "pymodule_ext.cu")):
        return None
    return os.path.abspath(ref)


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        L.orc_dist_sqr.restype = ctypes.c_float
        L.orc_dist_sqr.argtypes = [_f32, _f32, ctypes.c_int]
        L.orc_hyperplane.restype = ctypes.c_float
        L.orc_hyperplane.argtypes = [_f32, _f32, ctypes.c_int, ctypes.c_int, _f32]
        L.orc_project.restype = ctypes.c_float
        L.orc_project.argtypes = [_f32, _f32, ctypes.c_int]
        L.orc_sample_positions.restype = None
        L.orc_sample_positions.argtypes = [ctypes.c_int] * 4 + [_c_int_p, _c_int_p]
        L.orc_build_tree.restype = ctypes.c_int
        L.orc_build_tree.argtypes = [
            _f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_int, ctypes.c_void_p, ctypes.c_int, _i32,
            ctypes.POINTER(_c_int_p), ctypes.POINTER(_c_int_p), _c_int_p,
            ctypes.c_void_p, ctypes.c_int, _c_int_p]
        L.orc_free.restype = None
        L.orc_free.argtypes = [ctypes.c_void_p]
        for name in ("orc_bucket_knn_ref", "orc_bucket_knn"):
            fn = getattr(L, name)
            fn.restype = None
            fn.argtypes = [_f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i32, _i32, _i32,
                           ctypes.c_int, _i32, _f32]
        L.orc_sort_rows.restype = None
        L.orc_sort_rows.argtypes = [ctypes.c_int, ctypes.c_int, _i32, _f32]
        L.orc_explore_ref.restype = None
        L.orc_explore_ref.argtypes = [_f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i32, _i32, _f32]
        L.orc_explore.restype = None
        L.orc_explore.argtypes = [_f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i32, _i32, _f32,
                                  ctypes.c_int, ctypes.c_int]
        L.orc_merge_lists.restype = None
        L.orc_merge_lists.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                      ctypes.c_void_p, _i32, _f32]
        L.orc_bruteforce_knn.restype = ctypes.c_int
        L.orc_bruteforce_knn.argtypes = [_f32, ctypes.c_int, ctypes.c_int, _i32, ctypes.c_int,
                                         ctypes.c_int, _i32, _f32]
        L.orc_recall.restype = ctypes.c_double
        L.orc_recall.argtypes = [_i32, _i32, ctypes.c_int, ctypes.c_int]
        L.orc_build_tree_route.restype = ctypes.c_int
        L.orc_build_tree_route.argtypes = [
            _f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_int, _i32,
            ctypes.POINTER(_c_int_p), ctypes.POINTER(_c_int_p), _c_int_p,
            _f32, ctypes.c_int, _i32, _i32]
        for fn in (L.orc_ann_bucket_knn_ref, L.orc_ann_bucket_knn):
            fn.restype = None
            fn.argtypes = [_f32, _f32, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i32, _i32, _i32,
                           _i32, _f32]
        L.orc_symmetrize.restype = ctypes.c_longlong
        L.orc_symmetrize.argtypes = [ctypes.c_int, ctypes.c_int, _i32, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p]
        L.orc_bruteforce_ann.restype = None
        L.orc_bruteforce_ann.argtypes = [_f32, ctypes.c_int, _f32, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, _i32, _f32]
        L.orc_kmeans_assign.restype = None
        L.orc_kmeans_assign.argtypes = [_f32, ctypes.c_int, ctypes.c_int, _f32, ctypes.c_int, _i32, _f32]
        L.orc_kmeans_update.restype = None
        L.orc_kmeans_update.argtypes = [_f32, ctypes.c_int, ctypes.c_int, _i32, ctypes.c_int, _f32, _i32]
        _lib = L
    return _lib


def _pts(points):
    return np.ascontiguousarray(points, dtype=np.float32)


def dist_sqr(a, b):
    a, b = _pts(a), _pts(b)
    return float(lib().orc_dist_sqr(a, b, a.shape[0]))


def hyperplane(x1, x2, is_root):
    x1, x2 = _pts(x1), _pts(x2)
    n = np.empty_like(x1)
    c = lib().orc_hyperplane(x1, x2, x1.shape[0], int(is_root), n)
    return n, np.float32(c)


def project(n, x):
    n, x = _pts(n), _pts(x)
    return np.float32(lib().orc_project(n, x, n.shape[0]))


def sample_positions(seed, depth, start, count):
    r1, r2 = ctypes.c_int(), ctypes.c_int()
    lib().orc_sample_positions(seed, depth, start, count, ctypes.byref(r1), ctypes.byref(r2))
    return r1.value, r2.value


def build_tree(points, min_children, max_children, max_depth=5000, seed=0, table=None,
               record=False):
    """Returns dict(perm, leaf_start, leaf_count, depth[, table])."""
    points = _pts(points)
    N, D = points.shape
    perm = np.empty(N, np.int32)
    ls, lc, nl = _c_int_p(), _c_int_p(), ctypes.c_int()
    tbl_ptr, n_tbl = None, 0
    if table is not None:
        table = np.ascontiguousarray(table, np.int32).reshape(-1, 4)
        tbl_ptr, n_tbl = table.ctypes.data, table.shape[0]
    rec, rec_ptr, rec_cap, n_rec = None, None, 0, ctypes.c_int()
    if record:
        rec_cap = 2 * N + 16
        rec = np.full((rec_cap, 4), -1, np.int32)
        rec_ptr = rec.ctypes.data
    depth = lib().orc_build_tree(points, N, D, min_children, max_children, max_depth, seed,
                                 tbl_ptr, n_tbl, perm, ctypes.byref(ls), ctypes.byref(lc),
                                 ctypes.byref(nl), rec_ptr, rec_cap, ctypes.byref(n_rec))
    n = nl.value
    out = dict(perm=perm,
               leaf_start=np.ctypeslib.as_array(ls, shape=(max(n, 1),))[:n].copy(),
               leaf_count=np.ctypeslib.as_array(lc, shape=(max(n, 1),))[:n].copy(),
               depth=depth)
    lib().orc_free(ls)
    lib().orc_free(lc)
    if record:
        out["table"] = rec[:n_rec.value].copy()
    return out


def build_tree_route(points, queries, min_children, max_children, max_depth=5000, seed=0,
                     table=None):
    """The tree of build_tree plus, per query row, the leaf bucket it is routed
    to: dict(perm, leaf_start, leaf_count, depth, q_start, q_count)."""
    points, queries = _pts(points), _pts(queries)
    N, D = points.shape
    NQ = queries.shape[0]
    perm = np.empty(N, np.int32)
    ls, lc, nl = _c_int_p(), _c_int_p(), ctypes.c_int()
    tbl_ptr, n_tbl = None, 0
    if table is not None:
        table = np.ascontiguousarray(table, np.int32).reshape(-1, 4)
        tbl_ptr, n_tbl = table.ctypes.data, table.shape[0]
    q_start = np.full(max(NQ, 1), -1, np.int32)
    q_count = np.zeros(max(NQ, 1), np.int32)
    depth = lib().orc_build_tree_route(points, N, D, min_children, max_children, max_depth, seed,
                                       tbl_ptr, n_tbl, perm, ctypes.byref(ls), ctypes.byref(lc),
                                       ctypes.byref(nl), queries, NQ, q_start, q_count)
    n = nl.value
    out = dict(perm=perm,
               leaf_start=np.ctypeslib.as_array(ls, shape=(max(n, 1),))[:n].copy(),
               leaf_count=np.ctypeslib.as_array(lc, shape=(max(n, 1),))[:n].copy(),
               depth=depth, q_start=q_start[:NQ], q_count=q_count[:NQ])
    lib().orc_free(ls)
    lib().orc_free(lc)
    return out


def _ann(fn, points, queries, K, perm, q_start, q_count, idx, dist):
    points, queries = _pts(points), _pts(queries)
    NQ, D = queries.shape
    idx = np.ascontiguousarray(idx, np.int32).copy()
    dist = np.ascontiguousarray(dist, np.float32).copy()
    fn(points, queries, NQ, D, K, np.ascontiguousarray(perm, np.int32),
       np.ascontiguousarray(q_start, np.int32), np.ascontiguousarray(q_count, np.int32), idx, dist)
    return idx, dist


def ann_bucket_knn_ref(points, queries, K, perm, q_start, q_count, idx, dist):
    return _ann(lib().orc_ann_bucket_knn_ref, points, queries, K, perm, q_start, q_count, idx, dist)


def ann_bucket_knn(points, queries, K, perm, q_start, q_count, idx, dist):
    return _ann(lib().orc_ann_bucket_knn, points, queries, K, perm, q_start, q_count, idx, dist)


def ann_forest(points, queries, K, n_trees, min_children, max_children, max_depth=5000, seed=0,
               idx=None, dist=None):
    """The whole query path: tree t (seed+t) over the base points, queries
    routed, their lists merged with the bucket they land in."""
    queries = _pts(queries)
    if idx is None:
        idx, dist = init_lists(queries.shape[0], K, self_in_row=False)
    idx, dist = sort_rows(idx, dist)
    for t in range(n_trees):
        tr = build_tree_route(points, queries, min_children, max_children, max_depth, seed + t)
        idx, dist = ann_bucket_knn(points, queries, K, tr["perm"], tr["q_start"], tr["q_count"],
                                   idx, dist)
    return idx, dist


def kmeans_assign(points, centroids):
    """(labels int32 [N], squared distance float32 [N]) of the nearest centroid, ties to
    the lower centroid index (no reference counterpart: see the C source)."""
    points, centroids = _pts(points), _pts(centroids)
    N, D = points.shape
    labels = np.empty(N, np.int32)
    dist = np.empty(N, np.float32)
    lib().orc_kmeans_assign(points, N, D, centroids, centroids.shape[0], labels, dist)
    return labels, dist


def kmeans_update(points, labels, centroids):
    """(centroids float32 [C, D], counts int32 [C]): means of the members, empty clusters
    keep their centroid."""
    points = _pts(points)
    N, D = points.shape
    out = _pts(centroids).copy()
    counts = np.zeros(out.shape[0], np.int32)
    lib().orc_kmeans_update(points, N, D, np.ascontiguousarray(labels, np.int32), out.shape[0], out, counts)
    return out, counts


def kmeans(points, centroids, max_iter, labels=None):
    """Lloyd iterations from the given centroids (or, with ``labels``, from the means of
    those groups): stops after ``max_iter`` iterations or when no label changes.
    Returns (centroids, labels, squared distances, iterations run)."""
    cent = _pts(centroids).copy()
    if labels is not None:
        cent, _ = kmeans_update(points, labels, cent)
    prev = None
    done = 0
    lab, dist = kmeans_assign(points, cent)
    for it in range(max_iter):
        done = it + 1
        if prev is not None and np.array_equal(prev, lab):
            break
        prev = lab
        cent, _ = kmeans_update(points, lab, cent)
        lab, dist = kmeans_assign(points, cent)
    return cent, lab, dist, done


def symmetrize(idx, dist=None):
    """Symmetric closure of a K-NN graph as CSR: (offsets int64 [N+1], indices, values or None)."""
    idx = np.ascontiguousarray(idx, np.int32)
    N, K = idx.shape
    dist = None if dist is None else np.ascontiguousarray(dist, np.float32)
    offsets = np.empty(N + 1, np.int64)
    nnz = lib().orc_symmetrize(N, K, idx, None if dist is None else dist.ctypes.data, offsets.ctypes.data, None, None)
    indices = np.empty(max(nnz, 1), np.int32)
    values = np.empty(max(nnz, 1), np.float32) if dist is not None else None
    lib().orc_symmetrize(N, K, idx, None if dist is None else dist.ctypes.data, offsets.ctypes.data,
                         indices.ctypes.data, None if values is None else values.ctypes.data)
    return offsets, indices[:nnz], (None if values is None else values[:nnz])


def bruteforce_ann(points, queries, K):
    """Exact K nearest base points of every query row."""
    points, queries = _pts(points), _pts(queries)
    oi = np.empty((queries.shape[0], K), np.int32)
    od = np.empty((queries.shape[0], K), np.float32)
    lib().orc_bruteforce_ann(points, points.shape[0], queries, queries.shape[0], points.shape[1],
                             K, oi, od)
    return oi, od


def _bucket(fn, points, K, perm, leaf_start, leaf_count, idx, dist):
    points = _pts(points)
    N, D = points.shape
    idx = np.ascontiguousarray(idx, np.int32).copy()
    dist = np.ascontiguousarray(dist, np.float32).copy()
    fn(points, N, D, K, np.ascontiguousarray(perm, np.int32),
       np.ascontiguousarray(leaf_start, np.int32), np.ascontiguousarray(leaf_count, np.int32),
       len(leaf_start), idx, dist)
    return idx, dist


def bucket_knn_ref(points, K, perm, leaf_start, leaf_count, idx, dist):
    return _bucket(lib().orc_bucket_knn_ref, points, K, perm, leaf_start, leaf_count, idx, dist)


def bucket_knn(points, K, perm, leaf_start, leaf_count, idx, dist):
    return _bucket(lib().orc_bucket_knn, points, K, perm, leaf_start, leaf_count, idx, dist)


def sort_rows(idx, dist):
    idx = np.ascontiguousarray(idx, np.int32).copy()
    dist = np.ascontiguousarray(dist, np.float32).copy()
    lib().orc_sort_rows(idx.shape[0], idx.shape[1], idx, dist)
    return idx, dist


def explore_ref(points, old_idx, idx, dist):
    points = _pts(points)
    N, D = points.shape
    idx = np.ascontiguousarray(idx, np.int32).copy()
    dist = np.ascontiguousarray(dist, np.float32).copy()
    lib().orc_explore_ref(points, N, D, idx.shape[1], np.ascontiguousarray(old_idx, np.int32), idx, dist)
    return idx, dist


def explore(points, old_idx, idx, dist, row_begin=0, row_end=None):
    points = _pts(points)
    N, D = points.shape
    idx = np.ascontiguousarray(idx, np.int32).copy()
    dist = np.ascontiguousarray(dist, np.float32).copy()
    lib().orc_explore(points, N, D, idx.shape[1], np.ascontiguousarray(old_idx, np.int32), idx, dist,
                      row_begin, N if row_end is None else row_end)
    return idx, dist


def merge_lists(idx_lists, dist_lists):
    G = len(idx_lists)
    idx_lists = [np.ascontiguousarray(a, np.int32) for a in idx_lists]
    dist_lists = [np.ascontiguousarray(a, np.float32) for a in dist_lists]
    rows, K = idx_lists[0].shape
    ip = (ctypes.c_void_p * G)(*[a.ctypes.data for a in idx_lists])
    dp = (ctypes.c_void_p * G)(*[a.ctypes.data for a in dist_lists])
    oi, od = np.empty((rows, K), np.int32), np.empty((rows, K), np.float32)
    lib().orc_merge_lists(rows, K, G, ctypes.cast(ip, ctypes.c_void_p), ctypes.cast(dp, ctypes.c_void_p), oi, od)
    return oi, od


def bruteforce_knn(points, K, queries=None):
    """Exact KNN (self included) of the query rows; returns (idx, dist, threads)."""
    points = _pts(points)
    N, D = points.shape
    q = np.arange(N, dtype=np.int32) if queries is None else np.ascontiguousarray(queries, np.int32)
    oi, od = np.empty((len(q), K), np.int32), np.empty((len(q), K), np.float32)
    threads = lib().orc_bruteforce_knn(points, N, D, q, len(q), K, oi, od)
    return oi, od, threads


def recall(truth_idx, approx_idx):
    t = np.ascontiguousarray(truth_idx, np.int32)
    a = np.ascontiguousarray(approx_idx, np.int32)
    return float(lib().orc_recall(t, a, t.shape[0], t.shape[1]))


def init_lists(N, K, self_in_row=True):
    """The start lists the reference wrapper hands to the library
    (python/gpu_rsfk/RSFK.py:318-327): -1 / +inf, self at column 0."""
    idx = np.full((N, K), -1, np.int32)
    dist = np.full((N, K), np.inf, np.float32)
    if self_in_row:
        idx[:, 0] = np.arange(N)
        dist[:, 0] = 0.0
    return idx, dist


def leaf_sets(perm, leaf_start, leaf_count):
    """Partition as a set of frozensets, independent of leaf and slot order."""
    return {frozenset(perm[s:s + c].tolist()) for s, c in zip(leaf_start, leaf_count)}


def find_leaf_separations(points, ids, leaf, is_root, min_side, cap=64):
    """Distinct leaf separations a pair of the node's points can produce
    (see orc_find_leaf_separations); returns [(right_mask, (p1, p2)), ...]."""
    points = _pts(points)
    L = lib()
    L.orc_find_leaf_separations.restype = ctypes.c_int
    L.orc_find_leaf_separations.argtypes = [_f32, ctypes.c_int, _i32, _i32, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_int]
    ids = np.ascontiguousarray(ids, np.int32)
    leaf = np.ascontiguousarray(leaf, np.int32)
    masks = np.zeros(cap, np.uint64)
    pairs = np.zeros(2 * cap, np.int32)
    n = L.orc_find_leaf_separations(points, points.shape[1], ids, leaf, len(ids), int(leaf.max()) + 1,
                                    int(is_root), int(min_side), masks.ctypes.data, pairs.ctypes.data, cap)
    return [(int(masks[k]), (int(pairs[2 * k]), int(pairs[2 * k + 1]))) for k in range(n)]
