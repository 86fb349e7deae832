import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "gpu-rsfk_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import rsfk_oracle
    rsfk_oracle.build()
    return rsfk_oracle


@pytest.fixture(scope="session")
def forest():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from gpu_rsfk.device import DeviceForest
    f = DeviceForest(torch.device("cuda", 0))
    yield f
    f.close()
