"""In-tree build of librzlinear_b200.so (nvcc, sm_100a only).

    python -m rzlinear_b200.build [--force] [--verbose]

The library is plain CUDA C++ behind a C ABI (include/rzlinear_b200.h); it does not link
against PyTorch.  nvcc cross-compiles it on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "librzlinear_b200.so")
SOURCES = ["rz_abi.cu", "rz_simt.cu", "rz_tc.cu", "rz_noalloc.cu", "rz_elementwise.cu"]
HEADERS = ["rz_common.h", "rz_hash.h", "rz_ptx.cuh", os.path.join("..", "..", "include", "rzlinear_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
           "-Xlinker", "-rpath=/usr/local/cuda/lib64", "-o", LIB_PATH]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode:
        raise RuntimeError("nvcc failed building librzlinear_b200.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
