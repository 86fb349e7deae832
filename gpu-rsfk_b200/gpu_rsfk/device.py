"""Device-resident interface: the library's kernels on torch CUDA tensors.

torch supplies device memory and streams only; every computation is a kernel of
``librsfk.so`` reached through its C ABI (``rsfk_dev_*``).
"""
import ctypes

import numpy as np
import torch

from . import _lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _want(t, dtype, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise ValueError("%s must be a contiguous CUDA tensor of dtype %s" % (name, dtype))
    return t


class DeviceForest(object):
    """One context (device + stream + scratch memory) of the native library."""

    def __init__(self, device=None, stream=None):
        self._lib = _lib.load()
        if not torch.cuda.is_available():
            raise _lib.RSFKLibraryError("DeviceForest needs a CUDA device (there is no CPU fallback)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        self._ctx = self._lib.rsfk_ctx_create(self.device.index or 0, ctypes.c_void_p(self.stream.cuda_stream))
        if not self._ctx:
            raise _lib.RSFKLibraryError("rsfk_ctx_create failed")
        self.tree_info = None

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.rsfk_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def synchronize(self):
        _lib.raise_on_status(self._lib.rsfk_ctx_synchronize(self._ctx), "synchronize")

    # ------------------------------------------------------------------
    @staticmethod
    def init_lists(N, K, device, self_in_row=True):
        """Start lists as the reference wrapper builds them: -1 / +inf, self first."""
        idx = torch.full((N, K), -1, dtype=torch.int32, device=device)
        dist = torch.full((N, K), float("inf"), dtype=torch.float32, device=device)
        if self_in_row:
            idx[:, 0] = torch.arange(N, dtype=torch.int32, device=device)
            dist[:, 0] = 0.0
        return idx, dist

    def sort_rows(self, idx, dist):
        _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        rows, K = idx.shape
        _lib.raise_on_status(self._lib.rsfk_dev_sort_rows(self._ctx, _ptr(idx), _ptr(dist), rows, K), "sort_rows")

    def tree_build(self, points, min_children, max_children, max_depth=5000, seed=0, table=None):
        _want(points, torch.float32, "points")
        N, D = points.shape
        n_table = 0
        if table is not None:
            _want(table, torch.int32, "table")
            n_table = table.shape[0]
        out = [ctypes.c_int() for _ in range(4)]
        code = self._lib.rsfk_dev_tree_build(self._ctx, _ptr(points), N, D, min_children, max_children,
                                             max_depth, seed, _ptr(table), n_table,
                                             *[ctypes.byref(o) for o in out])
        _lib.raise_on_status(code, "tree_build")
        self.tree_info = dict(N=N, n_leaves=out[0].value, max_leaf=out[1].value,
                              min_leaf=out[2].value, levels=out[3].value)
        return self.tree_info

    def tree_export(self):
        """(perm, leaf_start, leaf_count) of the last tree as numpy arrays, leaves by start."""
        info = self.tree_info
        perm = np.empty(info["N"], np.int32)
        ls = np.empty(info["n_leaves"], np.int32)
        lc = np.empty(info["n_leaves"], np.int32)
        code = self._lib.rsfk_dev_tree_export(self._ctx, info["N"], perm.ctypes.data, ls.ctypes.data, lc.ctypes.data)
        _lib.raise_on_status(code, "tree_export")
        return perm, ls, lc

    def bucket_knn(self, points, idx, dist):
        _want(points, torch.float32, "points"); _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        _lib.raise_on_status(self._lib.rsfk_dev_bucket_knn(self._ctx, _ptr(points), N, D, idx.shape[1],
                                                          _ptr(idx), _ptr(dist)), "bucket_knn")

    def bucket_knn_table(self, points, perm, leaf_start, leaf_count, max_leaf, idx, dist):
        for t, name in ((perm, "perm"), (leaf_start, "leaf_start"), (leaf_count, "leaf_count"), (idx, "idx")):
            _want(t, torch.int32, name)
        _want(points, torch.float32, "points"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        code = self._lib.rsfk_dev_bucket_knn_table(self._ctx, _ptr(points), N, D, idx.shape[1], _ptr(perm),
                                                   _ptr(leaf_start), _ptr(leaf_count), leaf_start.shape[0],
                                                   int(max_leaf), _ptr(idx), _ptr(dist))
        _lib.raise_on_status(code, "bucket_knn_table")

    def set_lanes(self, lanes):
        """Tree sequences a forest call runs side by side (1..4; 0 = library default).
        The result does not depend on it."""
        _lib.raise_on_status(self._lib.rsfk_ctx_set_lanes(self._ctx, int(lanes)), "set_lanes")

    def set_tc(self, mode):
        """Bucket KNN on the tensor cores where D >= 64: 1 always, 0 never, -1 the
        library's choice.  The lists do not depend on it."""
        _lib.raise_on_status(self._lib.rsfk_ctx_set_tc(self._ctx, int(mode)), "set_tc")

    def set_wait_limits(self, route_max_steps=-1, level_wait_ms=-1):
        """Limits of the bounded waits (negative: built-in): tree levels a query may
        descend, milliseconds the host waits for a batch of tree levels."""
        _lib.raise_on_status(self._lib.rsfk_ctx_set_wait_limits(self._ctx, int(route_max_steps),
                                                                int(level_wait_ms)), "set_wait_limits")

    def forest(self, points, idx, dist, n_trees, min_children, max_children, max_depth=5000, seed=0,
               first_tree=0, tree_stride=1, want_log=False):
        _want(points, torch.float32, "points"); _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        log = np.zeros(16 * n_trees + 2, np.float32) if want_log else None
        code = self._lib.rsfk_dev_forest(self._ctx, _ptr(points), N, D, idx.shape[1], n_trees, first_tree,
                                         tree_stride, min_children, max_children, max_depth, seed,
                                         _ptr(idx), _ptr(dist), log.ctypes.data if want_log else None)
        _lib.raise_on_status(code, "forest")
        return log

    # ------------------------------------------------------------------ query path
    def keep_index(self, on=True):
        """Later tree builds keep the tree index that queries descend."""
        _lib.raise_on_status(self._lib.rsfk_ctx_keep_index(self._ctx, 1 if on else 0), "keep_index")

    def route_queries(self, points, queries):
        """(q_start, q_count) numpy arrays: the segment of ``perm`` (``tree_export``)
        that is the leaf bucket each query row ends in under the last tree."""
        _want(points, torch.float32, "points"); _want(queries, torch.float32, "queries")
        N, D = points.shape
        NQ = queries.shape[0]
        if queries.shape[1] != D:
            raise ValueError("points and queries differ in dimension")
        qs, qc = np.empty(NQ, np.int32), np.empty(NQ, np.int32)
        code = self._lib.rsfk_dev_route_queries(self._ctx, _ptr(points), N, D, _ptr(queries), NQ,
                                                qs.ctypes.data, qc.ctypes.data)
        _lib.raise_on_status(code, "route_queries")
        return qs, qc

    def ann_bucket_knn(self, points, queries, idx, dist):
        """Query lists (rows of ``idx``/``dist``, indices of base points) take in the
        base points of the bucket each query is routed to under the last tree."""
        _want(points, torch.float32, "points"); _want(queries, torch.float32, "queries")
        _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        NQ = queries.shape[0]
        if queries.shape[1] != D or idx.shape[0] != NQ or dist.shape != idx.shape:
            raise ValueError("shapes of queries and lists do not agree")
        code = self._lib.rsfk_dev_ann_bucket_knn(self._ctx, _ptr(points), N, _ptr(queries), NQ, D,
                                                 idx.shape[1], _ptr(idx), _ptr(dist))
        _lib.raise_on_status(code, "ann_bucket_knn")

    def forest_ann(self, points, queries, idx, dist, n_trees, min_children, max_children,
                   max_depth=5000, seed=0, first_tree=0, tree_stride=1):
        """Trees over the base points, each followed by the query update."""
        _want(points, torch.float32, "points"); _want(queries, torch.float32, "queries")
        _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        NQ = queries.shape[0]
        if queries.shape[1] != D or idx.shape[0] != NQ or dist.shape != idx.shape:
            raise ValueError("shapes of queries and lists do not agree")
        code = self._lib.rsfk_dev_forest_ann(self._ctx, _ptr(points), N, _ptr(queries), NQ, D, idx.shape[1],
                                             n_trees, first_tree, tree_stride, min_children, max_children,
                                             max_depth, seed, _ptr(idx), _ptr(dist))
        _lib.raise_on_status(code, "forest_ann")

    def explore(self, points, old_idx, idx, dist, row_begin=0, row_end=None, list_row0=0):
        """One sweep over rows [row_begin,row_end); ``idx``/``dist`` start at row ``list_row0``."""
        _want(points, torch.float32, "points"); _want(old_idx, torch.int32, "old_idx")
        _want(idx, torch.int32, "idx"); _want(dist, torch.float32, "dist")
        N, D = points.shape
        row_end = N if row_end is None else row_end
        if idx.shape[0] < row_end - list_row0:
            raise ValueError("idx/dist do not cover rows up to row_end")
        code = self._lib.rsfk_dev_explore(self._ctx, _ptr(points), N, D, idx.shape[1], _ptr(old_idx),
                                          _ptr(idx), _ptr(dist), row_begin, row_end, list_row0)
        _lib.raise_on_status(code, "explore")

    def merge_lists(self, idx_lists, dist_lists, out_idx, out_dist):
        G = len(idx_lists)
        rows, K = out_idx.shape
        for t in idx_lists:
            _want(t, torch.int32, "idx list")
        for t in dist_lists:
            _want(t, torch.float32, "dist list")
        ip = (ctypes.c_void_p * G)(*[t.data_ptr() for t in idx_lists])
        dp = (ctypes.c_void_p * G)(*[t.data_ptr() for t in dist_lists])
        code = self._lib.rsfk_dev_merge_lists(self._ctx, rows, K, G, ctypes.cast(ip, ctypes.c_void_p),
                                              ctypes.cast(dp, ctypes.c_void_p), _ptr(out_idx), _ptr(out_dist))
        _lib.raise_on_status(code, "merge_lists")

    def kmeans(self, points, centroids, max_iter=25, labels=None):
        """Lloyd iterations on the GPU from ``centroids`` ([C, D], updated in place) or, when
        ``labels`` (int32 [N], values in [0, C)) is given, from the means of those groups.
        Returns ``(labels int32 [N], squared distances float32 [N], iterations run)``."""
        _want(points, torch.float32, "points"); _want(centroids, torch.float32, "centroids")
        N, D = points.shape
        C = centroids.shape[0]
        from_labels = labels is not None
        if from_labels:
            _want(labels, torch.int32, "labels")
        else:
            labels = torch.empty(N, dtype=torch.int32, device=points.device)
        dist = torch.empty(N, dtype=torch.float32, device=points.device)
        done = ctypes.c_int(0)
        code = self._lib.rsfk_dev_kmeans(self._ctx, _ptr(points), N, D, C, int(max_iter), 1 if from_labels else 0,
                                         _ptr(centroids), _ptr(labels), _ptr(dist), ctypes.byref(done))
        _lib.raise_on_status(code, "kmeans")
        return labels, dist, done.value

    def symmetrize(self, idx, dist=None):
        """Symmetric closure of the K-NN graph ``idx`` ([N, K], -1 = empty) as CSR:
        ``(offsets int64 [N+1], indices int32 [nnz], values float32 [nnz] or None)``;
        row p holds p's neighbours and every q that lists p, ordered by index, with
        the squared distance of the edge when ``dist`` is given."""
        _want(idx, torch.int32, "idx")
        if dist is not None:
            _want(dist, torch.float32, "dist")
        N, K = idx.shape
        offsets = torch.empty(N + 1, dtype=torch.int64, device=idx.device)
        nnz = ctypes.c_longlong(0)
        code = self._lib.rsfk_dev_symmetrize_count(self._ctx, N, K, _ptr(idx), _ptr(offsets), ctypes.byref(nnz))
        _lib.raise_on_status(code, "symmetrize_count")
        indices = torch.empty(nnz.value, dtype=torch.int32, device=idx.device)
        values = torch.empty(nnz.value, dtype=torch.float32, device=idx.device) if dist is not None else None
        code = self._lib.rsfk_dev_symmetrize_fill(self._ctx, N, K, _ptr(idx), _ptr(dist), _ptr(offsets),
                                                  _ptr(indices), _ptr(values))
        _lib.raise_on_status(code, "symmetrize_fill")
        return offsets, indices, values

    def stats(self):
        """Work counters of this context (synchronizes the stream)."""
        out = (ctypes.c_double * 17)()
        _lib.raise_on_status(self._lib.rsfk_ctx_stats(self._ctx, out, 17), "stats")
        names = ("trees", "tree_active_points", "tree_nodes", "bucket_knn_us", "explore_candidates",
                 "subtree_us", "sub_active_points", "sub_nodes", "tree_build_us",
                 "project_us", "project_launches", "route_us", "query_update_us",
                 "tc_launches", "tc_gram_flops", "tc_pairs_passed", "tc_pairs_seen")
        return dict(zip(names, [float(v) for v in out]))

    def kernel_launches(self):
        return int(self._lib.rsfk_kernel_launches())
