"""Build libpaired_nvfp4_b200.so in-tree with nvcc for sm_100a (no torch dependency).

    python grouped-sparse-gemm_b200/build.py [--force] [--ptxas-v]

The library lands in grouped-sparse-gemm_b200/paired_nvfp4_kernels/, next to the Python package
that loads it.  PAIRED_NVFP4_PTXAS_V=1 (or --ptxas-v) prints registers / spills / shared memory.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "paired_nvfp4_kernels", "libpaired_nvfp4_b200.so")
SOURCES = ["abi.cu", "quant.cu", "compress.cu", "routing.cu", "group_mm.cu"]


def _inputs():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(os.path.dirname(HERE), "include", "paired_nvfp4_b200.h"))
    return files


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(f) <= t for f in _inputs())


def build(force=False, ptxas_v=False, verbose=True):
    if not force and up_to_date():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-std=c++17", "-O3", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT]
    if ptxas_v or os.environ.get("PAIRED_NVFP4_PTXAS_V") == "1":
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("PAIRED_NVFP4_NVCC_FLAGS", "").split()      # developer builds, e.g. -DPNV_WIDE_PROFILE
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, ptxas_v="--ptxas-v" in sys.argv)
