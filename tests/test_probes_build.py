"""The stand-alone measurement programs under gevva_b200/csrc/probes compile for sm_100a."""
import os
import shutil

import pytest


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                    reason="needs nvcc")
def test_probes_compile():
    from gevva_b200 import build
    built = build.build_probes()
    assert len(built) == len(build.PROBES)
    for path in built:
        assert os.path.isfile(path) and os.access(path, os.X_OK)
