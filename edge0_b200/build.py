"""Builds edge0_b200/lib/libedge0_b200.so (the C-ABI library with the sm_100a kernels) with nvcc.

Cross-compiles without a GPU.  Usage: python -m edge0_b200.build [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
SRC = [os.path.join(ROOT, "csrc", "capi.cu"), os.path.join(ROOT, "csrc", "gguf_reader.cpp")]
DEPS = [os.path.join(ROOT, "csrc", f) for f in os.listdir(os.path.join(ROOT, "csrc"))] + [
    os.path.join(os.path.dirname(ROOT), "include", "edge0_b200_moe.h")]
LIB = os.path.join(ROOT, "lib", "libedge0_b200.so")


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def up_to_date() -> bool:
    return os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    cmd = [nvcc(), "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-o", LIB] + SRC
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    cmd[1:1] = os.environ.get("B200MOE_NVCC_FLAGS", "").split()   # development switches, e.g. -DB200MOE_FP4_PROF
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
