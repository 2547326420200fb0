"""Builds librgb200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

The arch-specific target has to be spelled as a -gencode pair: the tcgen05 instructions exist only
in the "a" feature set and the shorthand -arch=sm_100a would add a plain compute_100 PTX target
that rejects them.  No fast-math, no FTZ, precise division, no FMA contraction: the output bits are
defined by IEEE single operations (the reference states the same discipline at
repro_gemm_cuda/repro_gemm.cuh:23 and repro_torch/setup.py:24).
"""
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "librgb200.so")
SOURCES = ["rgb200_api.cu", "rgb200_cxx.cu"]
HEADERS = ["rgb200_math.cuh", "rgb200_mma.cuh", "rgb200_smallk.cuh", "rgb200_rowfused.cuh", "rgb200_prepass.cuh",
           "rgb200_prepass_cluster.cuh", "rgb200_conv.cuh", "rgb200_conv_direct.cuh",
           os.path.join("..", "..", "include", "rgb200.h"), os.path.join("..", "..", "include", "repro_gemm.cuh"),
           os.path.join("..", "..", "include", "repro_conv.cuh")]

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--fmad=false",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "static"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; librgb200.so cannot be built")


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources; returns its path."""
    if force or stale():
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
        res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
