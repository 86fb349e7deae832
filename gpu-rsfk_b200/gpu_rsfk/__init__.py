"""gpu_rsfk: Random Sample Forest K-NN graphs on NVIDIA B200 (sm_100a).

``RSFK`` is the drop-in class of the reference package; ``DeviceForest`` is the
device-resident interface (torch CUDA tensors in and out, no host copies).
"""
from .RSFK import RSFK, ForestLog, random_motion, set_devices, test  # noqa: F401
from ._lib import RSFKLibraryError  # noqa: F401

__all__ = ["RSFK", "ForestLog", "random_motion", "set_devices", "test", "RSFKLibraryError"]
