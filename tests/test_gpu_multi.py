"""Trees sharded over two or more GPUs (NCCL) give the single-GPU graph bit for
bit.  Skipped on boxes with a single GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(%(root)r, "gpu-rsfk_b200"))
from gpu_rsfk.device import DeviceForest
from gpu_rsfk import distributed as rdist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
X = torch.from_numpy(np.random.RandomState(3).uniform(0, 1, (30011, 48)).astype(np.float32)).to(dev)
eng = DeviceForest(dev)
oi, od, b, e = rdist.build_knn_graph(eng, X, 16, 7, 17, 34, 5000, 11, 2, True)
fi, fd = rdist.gather_graph(oi, od, X.shape[0])
Q = torch.from_numpy(np.random.RandomState(4).uniform(0, 1, (9001, 48)).astype(np.float32)).to(dev)
qi, qd, qb, qe = rdist.search_queries(eng, X, Q, 16, 7, 17, 34, 5000, 11)
gqi, gqd = rdist.gather_graph(qi, qd, Q.shape[0])
if rank == 0:
    np.savez(%(out)r, idx=fi.cpu().numpy(), dist=fd.cpu().numpy(), q_idx=gqi.cpu().numpy(), q_dist=gqd.cpu().numpy())
dist.barrier()
dist.destroy_process_group()
'''


def test_two_gpu_build_equals_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from gpu_rsfk.device import DeviceForest
    from gpu_rsfk import distributed as rdist
    world = min(4, torch.cuda.device_count())
    out = str(tmp_path / "multi.npz")
    script = tmp_path / "worker.py"
    script.write_text(WORKER % dict(root=ROOT, out=out))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                    "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                   check=True, env=env, timeout=600)
    dev = torch.device("cuda", 0)
    X = torch.from_numpy(np.random.RandomState(3).uniform(0, 1, (30011, 48)).astype(np.float32)).to(dev)
    si, sd, _, _ = rdist.build_knn_graph(DeviceForest(dev), X, 16, 7, 17, 34, 5000, 11, 2, True)
    z = np.load(out)
    np.testing.assert_array_equal(z["idx"], si.cpu().numpy())
    np.testing.assert_array_equal(z["dist"], sd.cpu().numpy())
    # the query search, sharded the same way
    Q = torch.from_numpy(np.random.RandomState(4).uniform(0, 1, (9001, 48)).astype(np.float32)).to(dev)
    qi, qd, _, _ = rdist.search_queries(DeviceForest(dev), X, Q, 16, 7, 17, 34, 5000, 11)
    np.testing.assert_array_equal(z["q_idx"], qi.cpu().numpy())
    np.testing.assert_array_equal(z["q_dist"], qd.cpu().numpy())


@pytest.mark.parametrize("shape", [(30011, 48, 16, 7, 17, 34, 2), (5003, 100, 32, 3, 33, 66, 1), (9000, 8, 8, 9, 16, 64, 0)])
def test_host_entry_point_on_several_gpus_equals_one_gpu(shape):
    """pymodule_rsfk_knn spread over the box's GPUs by rsfk_set_devices (one process, a host
    thread per GPU, lists fetched from the peers) returns the single-GPU graph bit for bit;
    lists the caller passes in take part, and the forest log has a row for every tree."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import gpu_rsfk
    N, D, K, trees, mn, mx, sweeps = shape
    X = np.random.RandomState(5).uniform(0, 1, (N, D)).astype(np.float32)
    # lists that already hold something: a first, small forest on one GPU
    first = gpu_rsfk.RSFK(random_state=3)
    i0, d0 = first.find_nearest_neighbors(X, K, max_tree_children=mx, min_tree_children=mn, n_trees=1,
                                          max_tree_depth=5000, verbose=0, nn_exploring_factor=0)
    results = []
    for devices in (None, list(range(min(4, torch.cuda.device_count())))):
        gpu_rsfk.set_devices(devices)
        try:
            r = gpu_rsfk.RSFK(random_state=11)
            idx, dist = i0.copy(), d0.copy()
            log = r._knn_call(trees, K, mn, mx, 5000, 0, sweeps, X, idx, dist)
            results.append((idx, dist, np.array(log)))
        finally:
            gpu_rsfk.set_devices(None)
    np.testing.assert_array_equal(results[0][0], results[1][0])
    np.testing.assert_array_equal(results[0][1], results[1][1])
    # rows 0-3 of the log (depth, largest and smallest bucket, buckets) describe the same trees
    np.testing.assert_array_equal(results[0][2][:4 * trees], results[1][2][:4 * trees])
    assert (results[1][2][:trees] > 0).all()
