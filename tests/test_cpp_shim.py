"""The header-only C++ class include/gevva/nvfp4_expert_runner.hpp compiles with g++ against a
stand-in DeviceModel, has the reference's methods, and turns C-ABI error codes into
std::runtime_error (tests/shim_probe.cpp).  The GPU half runs a batch through it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    from gevva_b200 import build
    build.build()
    binary = str(tmp_path_factory.mktemp("shim") / "shim_probe")
    lib_dir = os.path.join(ROOT, "gevva_b200")
    compiler = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.run([compiler, "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(CUDA, "include"), os.path.join(ROOT, "tests", "shim_probe.cpp"),
                    "-o", binary, "-L", lib_dir, "-l:libgevva_moe.so", "-L", os.path.join(CUDA, "lib64"),
                    "-lcudart", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"],
                   check=True, capture_output=True, text=True)
    return binary


def test_shim_compiles_and_rejects_on_the_host(probe):
    result = subprocess.run([probe], capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "host checks ok" in result.stdout


@pytest.mark.gpu
def test_shim_runs_a_batch(probe, cuda_device):
    result = subprocess.run([probe, "gpu"], capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "gpu checks ok" in result.stdout
