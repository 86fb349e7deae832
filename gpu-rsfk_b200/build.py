"""Builds ``gpu_rsfk/librsfk.so`` for sm_100a with nvcc (no GPU needed).

    python gpu-rsfk_b200/build.py [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "gpu_rsfk", "librsfk.so")
SOURCES = ["rsfk_api.cu", "rsfk_tree.cu", "rsfk_knn.cu", "rsfk_graph.cu", "rsfk_kmeans.cu"]
HEADERS = ["rsfk_common.cuh", "rsfk_context.h", "rsfk_bucket_tc.cuh", os.path.join("..", "..", "include", "rsfk_b200.h")]
FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--compiler-options", "-fPIC,-fvisibility=hidden",
    "-Xcompiler", "-Wall",
    "--shared",
]


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += [os.path.join(CSRC, f) for f in SOURCES] + ["-o", OUT]
    env = dict(os.environ)
    # the image's $CC/$CXX wrappers are not what nvcc should pick as host compiler
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.check_call(cmd, env=env)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
