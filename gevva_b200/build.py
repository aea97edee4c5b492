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
    for root, dirs, files in os.walk(CSRC):
        if "probes" in dirs:
            dirs.remove("probes")  # stand-alone programs, not part of the library
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


PROBES = ["tensor_pipe_probe", "tma_intake_probe"]


def build_probes():
    """Stand-alone measurement programs (csrc/probes/*.cu -> gevva_b200/probes/<name>): what the tensor
    pipe and the TMA intake of an SM sustain for the stage shapes of the expert GEMMs."""
    out_dir = os.path.join(HERE, "probes")
    os.makedirs(out_dir, exist_ok=True)
    built = []
    for name in PROBES:
        target = os.path.join(out_dir, name)
        cmd = [NVCC, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-o", target,
               os.path.join(CSRC, "probes", name + ".cu")]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("nvcc failed building " + name)
        built.append(target)
    return built


if __name__ == "__main__":
    if "--probes" in sys.argv:
        print("\n".join(build_probes()))
    else:
        build(force=True, verbose=True)
        print(LIB)
