"""The multi-GPU driver's host logic on CPU: world_size-2 (and 3) `gloo` runs
of gpu_rsfk.distributed.build_knn_graph with the CPU oracle standing in for the
CUDA engine must equal the single-rank result bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleEngine(object):
    """DeviceForest's interface backed by the CPU oracle (tests only)."""

    def __init__(self):
        from oracle import rsfk_oracle
        self.orc = rsfk_oracle

    def init_lists(self, N, K, device, self_in_row=True):
        i, d = self.orc.init_lists(N, K, self_in_row)
        return torch.from_numpy(i), torch.from_numpy(d)

    def forest(self, points, idx, dst, n_trees, min_children, max_children, max_depth=5000, seed=0,
               first_tree=0, tree_stride=1):
        X = points.numpy()
        i, d = idx.numpy(), dst.numpy()
        for k in range(n_trees):
            t = first_tree + k * tree_stride
            tr = self.orc.build_tree(X, min_children, max_children, max_depth, seed + t)
            i, d = self.orc.bucket_knn(X, idx.shape[1], tr["perm"], tr["leaf_start"], tr["leaf_count"], i, d)
        idx.copy_(torch.from_numpy(i))
        dst.copy_(torch.from_numpy(d))

    def forest_ann(self, points, queries, idx, dst, n_trees, min_children, max_children, max_depth=5000,
                   seed=0, first_tree=0, tree_stride=1):
        X, Q = points.numpy(), queries.numpy()
        i, d = idx.numpy(), dst.numpy()
        for k in range(n_trees):
            t = first_tree + k * tree_stride
            tr = self.orc.build_tree_route(X, Q, min_children, max_children, max_depth, seed + t)
            i, d = self.orc.ann_bucket_knn(X, Q, idx.shape[1], tr["perm"], tr["q_start"], tr["q_count"], i, d)
        idx.copy_(torch.from_numpy(i))
        dst.copy_(torch.from_numpy(d))

    def merge_lists(self, idx_lists, dist_lists, out_idx, out_dist):
        i, d = self.orc.merge_lists([t.numpy() for t in idx_lists], [t.numpy() for t in dist_lists])
        out_idx.copy_(torch.from_numpy(i))
        out_dist.copy_(torch.from_numpy(d))

    def explore(self, points, old_idx, idx, dst, row_begin=0, row_end=None, list_row0=0):
        N, K = points.shape[0], idx.shape[1]
        full_i = np.full((N, K), -1, np.int32)
        full_d = np.full((N, K), np.inf, np.float32)
        n_own = row_end - list_row0
        full_i[list_row0:row_end] = idx.numpy()[:n_own]
        full_d[list_row0:row_end] = dst.numpy()[:n_own]
        oi, od = self.orc.explore(points.numpy(), old_idx.numpy()[:N], full_i, full_d, row_begin, row_end)
        idx[:n_own].copy_(torch.from_numpy(oi[list_row0:row_end]))
        dst[:n_own].copy_(torch.from_numpy(od[list_row0:row_end]))


def _params():
    return dict(K=8, n_trees=5, min_children=9, max_children=18, seed=3, sweeps=2)


def _points(N=1501, D=12):
    return torch.from_numpy(np.random.RandomState(1).uniform(0, 1, (N, D)).astype(np.float32))


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "gpu-rsfk_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from gpu_rsfk import distributed as rdist
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        X = _points()
        oi, od, begin, end = rdist.build_knn_graph(OracleEngine(), X, **_params())
        assert (begin, end) == rdist.owned_rows(X.shape[0], rank, world)
        fi, fd = rdist.gather_graph(oi, od, X.shape[0])
        if rank == 0:
            np.savez(os.path.join(out_dir, "w%d.npz" % world), idx=fi.numpy(), dist=fd.numpy())
    finally:
        dist.destroy_process_group()


def _queries(NQ=703, D=12):
    return torch.from_numpy(np.random.RandomState(2).uniform(0, 1, (NQ, D)).astype(np.float32))


def _query_params():
    return dict(K=6, n_trees=5, min_children=7, max_children=14, seed=11)


def _query_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "gpu-rsfk_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from gpu_rsfk import distributed as rdist
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        X, Q = _points(), _queries()
        oi, od, begin, end = rdist.search_queries(OracleEngine(), X, Q, **_query_params())
        assert (begin, end) == rdist.owned_rows(Q.shape[0], rank, world)
        fi, fd = rdist.gather_graph(oi, od, Q.shape[0])
        if rank == 0:
            np.savez(os.path.join(out_dir, "q%d.npz" % world), idx=fi.numpy(), dist=fd.numpy())
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_build_equals_single_rank(tmp_path, world):
    from gpu_rsfk import distributed as rdist
    X = _points()
    si, sd, b, e = rdist.build_knn_graph(OracleEngine(), X, **_params())
    assert (b, e) == (0, X.shape[0])
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    z = np.load(os.path.join(str(tmp_path), "w%d.npz" % world))
    np.testing.assert_array_equal(z["idx"], si.numpy())
    np.testing.assert_array_equal(z["dist"], sd.numpy())


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_query_search_equals_single_rank(tmp_path, world):
    from gpu_rsfk import distributed as rdist
    X, Q = _points(), _queries()
    si, sd, b, e = rdist.search_queries(OracleEngine(), X, Q, **_query_params())
    assert (b, e) == (0, Q.shape[0])
    mp.spawn(_query_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    z = np.load(os.path.join(str(tmp_path), "q%d.npz" % world))
    np.testing.assert_array_equal(z["idx"], si.numpy())
    np.testing.assert_array_equal(z["dist"].view(np.int32), sd.numpy().view(np.int32))


def test_tree_and_row_sharding_helpers():
    from gpu_rsfk import distributed as rdist
    for T in (0, 1, 7, 50, 64):
        for G in (1, 2, 3, 8):
            assert sum(rdist.tree_share(T, g, G) for g in range(G)) == T
    for N in (1, 10, 1501, 20_000_000):
        for G in (1, 2, 4, 8):
            rows = [rdist.owned_rows(N, g, G) for g in range(G)]
            assert rows[0][0] == 0 and rows[-1][1] == N
            assert all(rows[g][1] == rows[g + 1][0] for g in range(G - 1))
            assert all(0 <= e - b <= rdist.row_block(N, G) for b, e in rows)
