"""Compiles the CUDA library in-tree with nvcc for sm_100a.

``python kapy-lang_b200/build.py`` (or ``build()`` from Python) produces
``kapy-lang_b200/libkapyb.so``; nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libkapyb.so")
_SRC = os.path.join(_HERE, "csrc", "kapyb_abi.cu")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]


def _sources():
    out = [os.path.join(_HERE, "..", "include", "kapyb.h")]
    d = os.path.join(_HERE, "csrc")
    out += [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".cu", ".cuh", ".h"))]
    return out


def is_stale() -> bool:
    if not os.path.exists(SO_PATH):
        return True
    t = os.path.getmtime(SO_PATH)
    return any(os.path.getmtime(s) > t for s in _sources() if os.path.exists(s))


def build(force: bool = False, verbose: bool = False) -> str:
    """KAPYB_DEBUG_SWITCHES=1 in the environment compiles the profiling switches
    that make kernels skip work (and the epilogue's per-phase clock probes) in."""
    if not force and not is_stale():
        return SO_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", SO_PATH, _SRC]
    if os.environ.get("KAPYB_DEBUG_SWITCHES", "") not in ("", "0"):
        cmd.insert(1, "-DKAPYB_DEBUG_SWITCHES")
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return SO_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(SO_PATH)
