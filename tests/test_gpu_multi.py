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
