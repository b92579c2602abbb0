"""Builds libvlgpu.so (the sm_100a kernels + C ABI) in-tree with nvcc.

    python vectorlink-gpu_b200/build.py [--force]

nvcc cross-compiles for sm_100a without a GPU.  The library lands beside the Python
package (vectorlink_gpu/libvlgpu.so), where the ctypes loader looks for it.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.abspath(os.path.join(HERE, "..", "include"))
OUT = os.path.join(HERE, "vectorlink_gpu", "libvlgpu.so")
SOURCES = ["vl_api.cu", "vl_distance.cu", "vl_queue.cu", "vl_prune.cu", "vl_symmetrize.cu", "vl_components.cu", "vl_beam.cu", "vl_knn_tile.cu"]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-I", INCLUDE, "-shared", "-Xcompiler", "-fPIC", "-o", OUT] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
