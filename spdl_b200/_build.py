"""Builds ``libb2frames.so`` (sm_100a) in-tree with nvcc.

Usage: ``python -m spdl_b200._build [--verbose]``.  The library lands next to this file in
``spdl_b200/lib/`` and is what :mod:`spdl_b200._lib` loads.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libb2frames.so"
INCLUDE = PKG.parent / "include"

SOURCES = ["b2_api.cu", "b2_dense.cu", "b2_resize.cu", "b2_misc.cu"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; libb2frames.so cannot be built")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > built for p in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    if not force and not is_stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [
        nvcc_path(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
        "-DCUDA_API_PER_THREAD_DEFAULT_STREAM",
        "--threads", "0",
        "-I", str(INCLUDE), "-I", str(CSRC),
        "-o", str(LIB_PATH),
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
