"""Drop-in ``gpu_rsfk.RSFK`` surface over the sm_100a ``librsfk.so``.

Same class, method names, keyword arguments, defaults, return values and
raised exceptions as the reference wrapper (python/gpu_rsfk/RSFK.py:100-644 of
the reference project); the native work happens behind the same three
``extern "C"`` symbols.  Differences, all compatible refinements:

* rows come back ordered by (squared distance, index) instead of unordered;
* a failure inside the library raises ``RSFKLibraryError`` instead of ending
  the process;
* the library directory is found next to this file (no ``pkg_resources``) and
  ``int`` replaces the removed ``np.int``.
"""
import ctypes
import math
import time

import numpy as np

from . import _lib

_FOREST_LOG_FIELDS = (
    # attribute order of the reference's flattened ForestLog
    # (python/gpu_rsfk/RSFK.py:71-88, src/rsfk.cu:2148-2173)
    ("Tree Depth", True),
    ("Max Leaf Size", True),
    ("Min Leaf Size", True),
    ("Total Leaves", True),
    ("Tree Initialization Time", False),
    ("Total Tree Building Time", False),
    ("Check Active Points Time", False),
    ("Check Points Side Time", False),
    ("Count New Nodes Time", False),
    ("Dynamic Memory Allocation Time", False),
    ("Preprocessing Split Points Time", False),
    ("Create Nodes Time", False),
    ("Update Nodes Time", False),
    ("Bucket Creation Time", False),
    ("End Tree Time", False),
    ("KNN Sets Updates", False),
)


def random_motion(points, random_motion_force):
    """Jitters ``points`` in place, one dimension at a time, by a uniform offset
    of at most ``random_motion_force * (max - min) / N`` of that dimension, so
    that coincident points separate (python/gpu_rsfk/RSFK.py:40-66)."""
    n_points = points.shape[0]
    for d in range(points.shape[1]):
        column = points[:, d]
        span = (column.max() - column.min()) / n_points
        points[:, d] = column + random_motion_force * np.random.uniform(-span, span, n_points)


class ForestLog(object):
    """Per-tree statistics of the last ``find_nearest_neighbors`` call:
    ``data[name]`` is a list with one value per tree."""

    def __init__(self, data):
        n_trees = (len(data) - 2) // 16
        self.data = {}
        for row, (name, integral) in enumerate(_FOREST_LOG_FIELDS):
            values = data[row * n_trees:(row + 1) * n_trees]
            self.data[name] = [int(round(v)) for v in values] if integral else values
        self.total_forest_time = float(data[16 * n_trees]) if len(data) >= 2 else 0.0
        self.exploration_time = float(data[16 * n_trees + 1]) if len(data) >= 2 else 0.0


def set_devices(devices=None):
    """GPUs that one ``find_nearest_neighbors`` call is spread over inside the library
    (``rsfk_set_devices``): a list of device numbers, or None / one device for a single GPU.
    The graph is the single-GPU graph bit for bit.  The reference has no counterpart (it runs
    on one GPU); without this call ``RSFK_DEVICES`` or ``RSFK_NUM_GPUS`` in the environment
    are honoured, which also works from the reference's own wrapper."""
    devs = [] if devices is None else [int(d) for d in devices]
    arr = (ctypes.c_int * max(1, len(devs)))(*devs)
    rc = _lib.load().rsfk_set_devices(len(devs), arr)
    if rc != 0:
        raise ValueError("set_devices: unknown device in %r" % (devs,))


def _check_children(min_tree_children, max_tree_children):
    if min_tree_children < 0:
        raise Exception('min_tree_children = {} \t => min_tree_children must be at least 1'
                        .format(min_tree_children))
    if max_tree_children < 2 * min_tree_children:
        raise Exception('min_tree_children = {}, max_tree_children = {} \t => max_tree_children '
                        'must be at least 2*min_tree_children'.format(min_tree_children, max_tree_children))


class RSFK(object):
    def __init__(self, random_state=0):
        """``random_state`` seeds the forest: tree ``t`` of a call uses
        ``random_state + t``."""
        self.random_state = int(random_state)
        self._path = _lib._DIR
        self._lib = _lib.load()
        self.log_forest = None
        self._last_search_time = None
        self._last_cluster_time = None

    # ------------------------------------------------------------------ KNN
    def _knn_call(self, n_trees, K, min_children, max_children, max_depth, verbose, sweeps,
                  points, indices, sq_dist):
        N, D = points.shape
        log = np.zeros(n_trees * 16 + 2, np.float32)
        self._lib.pymodule_rsfk_knn(n_trees, K, N, D, min_children, max_children, max_depth, verbose,
                                    self.random_state, sweeps, points, indices, sq_dist, log)
        _lib.check_last("pymodule_rsfk_knn")
        return log

    def find_nearest_neighbors(self, points, num_nearest_neighbors,
                               n_trees=-1, max_tree_depth=5000,
                               verbose=0, min_tree_children=-1,
                               max_tree_children=-1,
                               ensure_valid_indices=True,
                               add_bit_random_motion=False,
                               random_motion_force=1.0,
                               nn_exploring_factor=-1,
                               point_in_self_neigh=True):
        """Approximate K-NN graph of ``points`` (``[n_points, n_dimensions]``).

        Returns ``(knn_indices int32 [N, K], knn_squared_dist float32 [N, K])``,
        rows ordered by distance; with ``point_in_self_neigh`` each point is its
        own first neighbour at distance 0.  Defaults: ``min_tree_children=K+1``,
        ``max_tree_children=2*min_tree_children``, one exploration sweep when
        ``K <= 32`` else none, ``n_trees`` from the reference's heuristic
        (at least 50).  When ``min_tree_children < K+1`` and
        ``ensure_valid_indices`` a further tree with buckets of ``K+1 .. 3(K+1)``
        points guarantees that no slot keeps index -1.
        """
        points = np.require(points, np.float32, ['CONTIGUOUS', 'ALIGNED'])
        max_tree_depth, verbose = int(max_tree_depth), int(verbose)
        max_tree_children, n_trees = int(max_tree_children), int(n_trees)
        N, D = points.shape
        K = int(num_nearest_neighbors)

        if nn_exploring_factor == -1:
            nn_exploring_factor = 1 if K <= 32 else 0
        if min_tree_children == -1:
            min_tree_children = K + 1
        if max_tree_children == -1 and min_tree_children >= 0:
            max_tree_children = 2 * min_tree_children
        _check_children(min_tree_children, max_tree_children)

        if n_trees == -1:
            mean_bucket = (min_tree_children + max_tree_children) / 2
            n_trees = int(max(math.ceil((N * D) / (mean_bucket * 24913)), 50))
            if verbose > 0:
                print("Automatically setting n_trees to {}".format(n_trees))

        if add_bit_random_motion:
            random_motion(points, random_motion_force)

        knn_indices = np.full((N, K), -1, np.int32)
        knn_squared_dist = np.full((N, K), np.inf, np.float32)
        if point_in_self_neigh:
            knn_indices[:, 0] = np.arange(N, dtype=np.int32)
            knn_squared_dist[:, 0] = 0.0

        t_init = time.time()
        log = self._knn_call(n_trees, K, int(min_tree_children), max_tree_children, max_tree_depth,
                             verbose, int(nn_exploring_factor), points, knn_indices, knn_squared_dist)
        self.log_forest = ForestLog(log)
        if ensure_valid_indices and min_tree_children < K + 1:
            self._knn_call(1, K, K + 1, 3 * (K + 1), max_tree_depth, verbose,
                           int(nn_exploring_factor), points, knn_indices, knn_squared_dist)
        self._last_search_time = time.time() - t_init
        return knn_indices, knn_squared_dist

    def _ann_call(self, n_trees, K, min_children, max_children, max_depth, verbose, sweeps,
                  points, query_points, indices, sq_dist):
        N, D = points.shape
        log = np.zeros(n_trees * 16 + 2, np.float32)
        self._lib.pymodule_rsfk_knn_ann(n_trees, K, N, query_points.shape[0], D, min_children,
                                        max_children, max_depth, verbose, self.random_state, sweeps,
                                        points, query_points, indices, sq_dist, log)
        _lib.check_last("pymodule_rsfk_knn_ann")

    def find_nearest_neighbors_ann(self, points, query_points, num_nearest_neighbors,
                                   n_trees=-1, max_tree_depth=5000,
                                   verbose=0, min_tree_children=-1,
                                   max_tree_children=-1,
                                   ensure_valid_indices=True,
                                   add_bit_random_motion=False,
                                   random_motion_force=1.0,
                                   nn_exploring_factor=-1):
        """Approximate K nearest ``points`` (base set, ``[n_points, n_dimensions]``)
        of every row of ``query_points`` (``[n_queries, n_dimensions]``).

        Every tree is built over the base points; a query descends it to a leaf
        and is compared with the base points of that leaf.  Returns
        ``(knn_indices int32 [NQ, K], knn_squared_dist float32 [NQ, K])``,
        indices into ``points``, rows ordered by distance.  Parameters and
        defaults as ``find_nearest_neighbors``; the exploration sweeps do not
        apply to this search (``nn_exploring_factor`` is accepted and passed on,
        as in the reference, but has no effect).
        """
        points = np.require(points, np.float32, ['CONTIGUOUS', 'ALIGNED'])
        query_points = np.require(query_points, np.float32, ['CONTIGUOUS', 'ALIGNED'])
        if points.ndim != 2 or query_points.ndim != 2 or points.shape[1] != query_points.shape[1]:
            raise Exception('points and query_points must be 2-D arrays with the same number of dimensions')
        max_tree_depth, verbose = int(max_tree_depth), int(verbose)
        max_tree_children, n_trees = int(max_tree_children), int(n_trees)
        N, D = points.shape
        NQ = query_points.shape[0]
        K = int(num_nearest_neighbors)

        if nn_exploring_factor == -1:
            nn_exploring_factor = 1 if K <= 32 else 0
        if min_tree_children == -1:
            min_tree_children = K + 1
        if max_tree_children == -1 and min_tree_children >= 0:
            max_tree_children = 2 * min_tree_children
        _check_children(min_tree_children, max_tree_children)

        if n_trees == -1:
            mean_bucket = (min_tree_children + max_tree_children) / 2
            n_trees = int(max(math.ceil((N * D) / (mean_bucket * 24913)), 50))
            if verbose > 0:
                print("Automatically setting n_trees to {}".format(n_trees))

        if add_bit_random_motion:
            random_motion(points, random_motion_force)
            random_motion(query_points, random_motion_force)

        knn_indices = np.full((NQ, K), -1, np.int32)
        knn_squared_dist = np.full((NQ, K), np.inf, np.float32)

        t_init = time.time()
        self._ann_call(n_trees, K, int(min_tree_children), max_tree_children, max_tree_depth, verbose,
                       int(nn_exploring_factor), points, query_points, knn_indices, knn_squared_dist)
        if ensure_valid_indices and min_tree_children < K + 1:
            self._ann_call(1, K, K + 1, 3 * (K + 1), max_tree_depth, verbose,
                           int(nn_exploring_factor), points, query_points, knn_indices, knn_squared_dist)
        self._last_search_time = time.time() - t_init
        return knn_indices, knn_squared_dist

    # -------------------------------------------------------------- cluster
    def cluster_by_sample_tree(self, points, max_tree_depth=5000,
                               verbose=1, min_tree_children=32,
                               max_tree_children=128,
                               add_bit_random_motion=False,
                               random_motion_force=1.0,
                               numpy_result_format=True):
        """Partitions ``points`` with a single random sample tree.

        Returns ``(total_leaves, max_child, nodes_buckets, bucket_sizes)``:
        ``nodes_buckets`` holds ``total_leaves`` consecutive groups of
        ``max_child`` point indices, padded with -1; ``bucket_sizes[b]`` is the
        number of points of bucket ``b``.  With ``numpy_result_format=False`` the
        raw ctypes values are returned instead of ints and ndarrays.
        """
        points = np.require(points, np.float32, ['CONTIGUOUS', 'ALIGNED'])
        max_tree_depth, verbose = int(max_tree_depth), int(verbose)
        max_tree_children = int(max_tree_children)
        N, D = points.shape
        _check_children(min_tree_children, max_tree_children)
        if add_bit_random_motion:
            random_motion(points, random_motion_force)

        t_init = time.time()
        nodes_buckets = ctypes.POINTER(ctypes.c_int)()
        bucket_sizes = ctypes.POINTER(ctypes.c_int)()
        total_leaves, max_child = ctypes.c_int(0), ctypes.c_int(0)
        self._lib.pymodule_cluster_by_sample_tree(
            N, D, int(min_tree_children), max_tree_children, max_tree_depth, verbose,
            self.random_state, points, ctypes.byref(nodes_buckets), ctypes.byref(bucket_sizes),
            ctypes.byref(total_leaves), ctypes.byref(max_child))
        _lib.check_last("pymodule_cluster_by_sample_tree")
        self._last_cluster_time = time.time() - t_init

        if not numpy_result_format:
            return total_leaves, max_child, nodes_buckets, bucket_sizes
        n_leaves, width = int(total_leaves.value), int(max_child.value)
        buckets = np.ctypeslib.as_array(nodes_buckets, shape=(n_leaves * width,)).copy()
        sizes = np.ctypeslib.as_array(bucket_sizes, shape=(n_leaves,)).copy()
        self._lib.rsfk_free(nodes_buckets)
        self._lib.rsfk_free(bucket_sizes)
        return n_leaves, width, buckets, sizes


    # -------------------------------------------------------------- k-means
    def cluster_by_kmeans(self, points, n_clusters=None, max_iter=25, init="sample_tree",
                          min_tree_children=32, max_tree_children=128, max_tree_depth=5000, verbose=0):
        """k-means clustering on the GPU (Lloyd iterations), by default refining the
        partition of a random sample tree.

        ``init="sample_tree"``: one sample tree is built (``cluster_by_sample_tree`` with the
        given ``min/max_tree_children``), its buckets are the starting groups and their
        number is the number of clusters (``n_clusters`` must be None).
        ``init="points"``: ``n_clusters`` distinct points drawn with ``random_state`` are the
        starting centroids.

        Returns ``(centroids float32 [C, D], labels int32 [N], squared_dist float32 [N])``;
        ``n_iter_`` holds the iterations run.  The reference package has no counterpart
        (its k-means lives inside nvGRAPH's spectral clustering, which its code no longer
        calls); ``cluster_by_sample_tree`` itself is unchanged by this method.
        """
        points = np.require(points, np.float32, ['CONTIGUOUS', 'ALIGNED'])
        N, D = points.shape
        labels = np.zeros(N, np.int32)
        if init == "sample_tree":
            if n_clusters is not None:
                raise Exception('n_clusters is decided by the sample tree when init="sample_tree"')
            n_leaves, width, buckets, sizes = self.cluster_by_sample_tree(
                points, max_tree_depth=max_tree_depth, verbose=verbose, min_tree_children=min_tree_children,
                max_tree_children=max_tree_children)
            table = buckets.reshape(n_leaves, width)
            for b in range(n_leaves):
                labels[table[b, :sizes[b]]] = b
            C = int(n_leaves)
            centroids = np.zeros((C, D), np.float32)
            from_labels = 1
        elif init == "points":
            C = int(n_clusters)
            if C < 1 or C > N:
                raise Exception('n_clusters = {} \t => must be between 1 and the number of points'.format(C))
            pick = np.sort(np.random.RandomState(self.random_state).choice(N, C, replace=False))
            centroids = points[pick].copy()
            from_labels = 0
        else:
            raise Exception('init must be "sample_tree" or "points"')
        sq_dist = np.empty(N, np.float32)
        done = ctypes.c_int(0)
        t_init = time.time()
        self._lib.rsfk_kmeans(N, D, C, int(max_iter), from_labels, points, centroids, labels, sq_dist,
                              ctypes.byref(done))
        _lib.check_last("rsfk_kmeans")
        self._last_cluster_time = time.time() - t_init
        self.n_iter_ = int(done.value)
        return centroids, labels, sq_dist


def test():
    """Smoke checks in the spirit of the reference's ``test1``/``test2``
    (python/gpu_rsfk/RSFK.py:841-903): no slot may keep index -1, and a
    clustering call must cover every point once."""
    rng = np.random.RandomState(0)
    data = rng.random_sample((3000, 200))
    indices, _ = RSFK(random_state=0).find_nearest_neighbors(
        data, 30, max_tree_children=128, n_trees=10, random_motion_force=0.01,
        nn_exploring_factor=2, add_bit_random_motion=True)
    missing = int(np.sum(indices == -1))
    if missing > 0:
        raise Exception('{} Negative indices'.format(missing))
    n_points = 2 ** 12
    pts = rng.random_sample((n_points, 99))
    low = n_points // 30
    n_leaves, width, buckets, sizes = RSFK(random_state=0).cluster_by_sample_tree(
        pts, min_tree_children=low, max_tree_children=3 * low, verbose=0)
    members = buckets[buckets >= 0]
    if len(members) != n_points or len(np.unique(members)) != n_points or sizes.sum() != n_points:
        raise Exception('cluster_by_sample_tree did not partition the points')
