"""Failure detection without a GPU fault: the expert-parallel barrier protocol with a withheld
rank (threads on the CPU) and the runner's scratch acquisition with an allocator that fails at
every step in turn.  Both run the very headers the CUDA library compiles (tests/failure_probe.cpp)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_barrier_timeout_and_allocation_failure(tmp_path):
    binary = str(tmp_path / "failure_probe")
    compiler = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.run([compiler, "-std=c++17", "-O1", "-Wall", "-Werror", "-pthread",
                    os.path.join(ROOT, "tests", "failure_probe.cpp"), "-o", binary],
                   check=True, capture_output=True, text=True)
    result = subprocess.run([binary], capture_output=True, text=True, timeout=60)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "barrier checks ok" in result.stdout and "scratch checks ok" in result.stdout
