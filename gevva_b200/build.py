"""Compiles the CUDA sources under csrc/ into libgevva_moe.so (sm_100a only).

The library is built in-tree with nvcc directly; it has no Python or torch
dependency and exports the C ABI of include/gevva_moe.h.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libgevva_moe.so")
SOURCES = ["moe_kernels.cu", "grouped_gemm.cu", "grouped_gemm_pair.cu", "grouped_gemm_w13_pair.cu", "grouped_gemm_decode.cu", "moe_abi.cu", "router_project.cu", "route_sort_noalloc.cu", "ep.cu", "dense_ff.cu", "dense_abi.cu", "sidecar.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v",
]


def needs_build():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    for root, _, files in os.walk(CSRC):
        for name in files:
            if name.endswith((".cu", ".cuh", ".h", ".cpp")) and os.path.getmtime(os.path.join(root, name)) > built:
                return True
    header = os.path.join(HERE, "..", "include", "gevva_moe.h")
    return os.path.getmtime(header) > built


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    cmd = [NVCC] + FLAGS + ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed building libgevva_moe.so")
    return LIB


if __name__ == "__main__":
    build(force=True, verbose=True)
    print(LIB)
