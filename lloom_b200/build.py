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


def translation_units() -> list[str]:
    """Every .cu / .cpp under csrc/: the kernels are split over several units so that they compile in parallel."""
    out = []
    for root, _, files in os.walk(SRC_DIR):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cpp"))]
    return sorted(out)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source of the package (one object per translation unit, in parallel) and link them
    into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    obj_dir = os.path.join(_PKG, "build")
    os.makedirs(obj_dir, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f != "--shared"]

    def compile_unit(src: str) -> tuple[str, str]:
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        cmd = [_nvcc(), *compile_flags, "-c", src, "-o", obj]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_unit, translation_units()))
    if verbose:
        for _, log in results:
            print(log)
    cmd = [_nvcc(), "--shared", "-o", LIB_PATH, *[obj for obj, _ in results]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
