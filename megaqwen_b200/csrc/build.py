"""Ahead-of-time build of libmegaqwen_b200.so for sm_100a with nvcc.

The shared library has a plain C ABI (include/megaqwen_b200.h) and no torch
dependency; it is built in-tree next to the Python package.  nvcc
cross-compiles without a GPU.  Run ``python -m megaqwen_b200.csrc.build``.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SOURCES = ["decode.cu", "decode_stream.cu", "prefill.cu", "ops.cu"]
OUT = os.environ.get("MQ_LIB_OUT") or os.path.join(PKG, "libmegaqwen_b200.so")


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "megaqwen_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-o", OUT]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("MQ_NVCC_FLAGS", "").split()
    cmd += [os.path.join(HERE, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libmegaqwen_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
