"""Builds ``liblloom_b200.so`` in-tree with nvcc for sm_100a (no other architecture, no JIT cache)."""
from __future__ import annotations

import os
import shutil
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(_PKG, "csrc")
LIB_PATH = os.path.join(_PKG, "liblloom_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-ffp-contract=off",  # host-side quantizers: strict sequential f32, like the reference
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build liblloom_b200.so")
    return nvcc


def sources() -> list[str]:
    out = []
    for root, _, files in os.walk(SRC_DIR):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h", ".hpp", ".cpp"))]
    inc = os.path.join(os.path.dirname(_PKG), "include")
    out += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    return sorted(out)


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in sources())


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source of the package into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    units = [os.path.join(SRC_DIR, "lloom_b200.cu"), os.path.join(SRC_DIR, "host", "qcuda_storage.cpp")]
    units = [u for u in units if os.path.exists(u)]
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *units]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
