import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _ensure_oracle():
    lib = os.path.join(ROOT, "oracle", "libgevva_golden.so")
    pin = os.path.join(ROOT, "oracle", "_ref", "libgv_pin_toolkit.so")
    src = os.path.join(ROOT, "oracle", "gevva_golden.cpp")
    stale = os.path.exists(lib) and os.path.getmtime(src) > os.path.getmtime(lib)
    if stale or not os.path.exists(lib) or not os.path.exists(pin):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True,
                       capture_output=True)
    return lib


@pytest.fixture(scope="session")
def oracle():
    _ensure_oracle()
    from tests import oracle_api
    return oracle_api.Oracle()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
