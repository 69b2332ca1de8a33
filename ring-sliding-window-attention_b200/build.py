"""Builds ring_swa/librswa.so (the C-ABI library of include/rswa.h) with nvcc for sm_100a.

    python ring-sliding-window-attention_b200/build.py [--force] [--verbose]

The library is built in-tree, next to the Python package that loads it with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "ring_swa", "librswa.so")
SOURCES = ["rswa_api.cu", "rswa_fwd.cu", "rswa_bwd.cu", "rswa_dq.cu", "rswa_aux.cu", "rswa_selftest.cu", "rswa_noalloc.cu", "rswa_peer.cu"]
HEADERS = ["tc05.cuh", "rswa_common.cuh", "rswa_tiles.cuh", os.path.join("..", "..", "include", "rswa.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources() + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return OUT
    cmd = [
        _nvcc(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-shared", "-Xcompiler", "-fPIC",
        "-o", OUT,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
