"""Builds libleapquant_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m leapquant_b200.csrc.build [--verbose]

The library depends on the CUDA runtime only: no torch headers, no Python headers.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libleapquant_b200.so")
SOURCES = ["leapquant_b200.cu"]
DEPS = ["lq_abi.cu", "lq_quant.cu", "lq_flush.cu", "lq_step.cu", "lq_common.cuh", "lq_linalg.cuh", "lq_step_warp.cuh",
        os.path.join("..", "..", "include", "leapquant_b200.h")]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(HERE, f)) > t for f in SOURCES + DEPS)


def build(verbose=False, force=False):
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-shared", "-Xcompiler", "-fPIC"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB] + [os.path.join(HERE, s) for s in SOURCES]
    res = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libleapquant_b200.so")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
