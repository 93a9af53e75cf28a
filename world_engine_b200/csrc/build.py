"""Builds libwe_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: python -m world_engine_b200.csrc.build [--debug] [--verbose] [-DNAME ...]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SOURCES = ["abi.cu", "kv_append.cu", "block_mask.cu", "frame_attn.cu", "qkv_prologue.cu"]
HEADERS = ["common.cuh", "ptx.cuh", os.path.join("..", "..", "include", "we_b200.h")]


def lib_path(debug: bool = False) -> str:
    return os.path.join(PKG, "libwe_b200_debug.so" if debug else "libwe_b200.so")


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: libwe_b200.so cannot be built")
    return cand


def needs_build(debug: bool = False) -> bool:
    out = lib_path(debug)
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(debug: bool = False, verbose: bool = False, force: bool = False) -> str:
    out = lib_path(debug)
    if not force and not needs_build(debug):
        return out
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
        "-Xcompiler", "-Wall",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    if debug:
        cmd += ["-DWE_ATTN_DEBUG"]
    cmd += [a for a in sys.argv[1:] if a.startswith("-D")]
    cmd += [os.path.join(HERE, s) for s in SOURCES]
    cmd += ["-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libwe_b200.so")
    return out


if __name__ == "__main__":
    build(debug="--debug" in sys.argv, verbose="--verbose" in sys.argv, force=True)
    print(lib_path("--debug" in sys.argv))
