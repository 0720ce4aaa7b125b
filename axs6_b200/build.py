"""Builds ``libaxs6_b200.so`` (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m axs6_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The quantiser translation units are built
with ``-fmad=false -ftz=false -prec-div=true`` so that no step is contracted into an FMA and
denormals survive: their results are compared bit for bit with the reference's eager CPU path.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaxs6_b200.so")

EXACT_SOURCES = ["abi.cu", "fq.cu", "codec.cu", "exchange.cu", "linear.cu"]      # bit-exact arithmetic: no fma contraction
FAST_SOURCES: list[str] = ["gemm.cu"]                          # tensor-core kernels

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
EXACT = ["-fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true"]


def _newest_source() -> float:
    t = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cu", ".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    t = max(t, os.path.getmtime(os.path.join(os.path.dirname(HERE), "include", "axs6_b200.h")))
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src, extra in [(s, EXACT) for s in EXACT_SOURCES] + [(s, []) for s in FAST_SOURCES]:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd)))
    for src, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    cmd = [nvcc, *ARCH, "-shared", "-o", LIB, *objs]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
