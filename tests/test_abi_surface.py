"""The C-ABI library loads without a GPU, exports every function include/gevva_moe.h
declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "gevva_b200", "libgevva_moe.so")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        from gevva_b200 import build
        build.build()
    return ctypes.CDLL(LIB)


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gevva_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gevva_(?:moe|ff|dense|pack|sidecar)_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert "gevva_moe_create" in names and "gevva_moe_launch" in names and len(names) >= 11
    for name in names:
        assert hasattr(lib, name), name


def test_strerror_covers_every_status(lib):
    lib.gevva_moe_strerror.restype = ctypes.c_char_p
    lib.gevva_moe_strerror.argtypes = [ctypes.c_int]
    texts = [lib.gevva_moe_strerror(-i).decode() for i in range(0, 7)]
    assert texts[0] == "ok" and len(set(texts)) == 7
    assert lib.gevva_moe_strerror(-99).decode() == "unknown status"


def test_null_arguments_are_rejected_without_cuda(lib):
    vp = ctypes.c_void_p
    lib.gevva_moe_create.argtypes = [vp, vp, ctypes.c_int, vp, vp]
    assert lib.gevva_moe_create(None, None, 16, None, None) == -3
    lib.gevva_moe_route.argtypes = [vp, ctypes.c_int, vp, vp, vp, ctypes.c_int, vp, vp, vp]
    assert lib.gevva_moe_route(None, 128, None, None, None, 4, None, None, None) == -3
    lib.gevva_moe_launch.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int, vp]
    assert lib.gevva_moe_launch(None, None, None, None, None, 1, None) == -3
    lib.gevva_moe_pack_experts.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp]
    assert lib.gevva_moe_pack_experts(None, 1, 128, 64, None, None, None, None) == -3
    lib.gevva_moe_destroy.argtypes = [vp]
    lib.gevva_moe_destroy(None)  # no-op


def test_expert_parallel_receive_capacity_below_worst_case_is_refused(lib):
    """A receive buffer smaller than world * 8 * max_tokens rows could be overrun by a skewed
    batch (stores into another GPU's memory); creation refuses it before any CUDA call."""
    from gevva_b200.expert_parallel import _EpConfig
    from gevva_b200.runtime import _Weights
    vp = ctypes.c_void_p
    world, max_tokens = 2, 64
    fake = (vp * world)(0x1000, 0x2000)   # never dereferenced: the size check comes first
    cast = lambda a: ctypes.cast(a, ctypes.POINTER(vp))
    weights = _Weights(*([0x1000] * 8))
    scale = vp(0x1000)
    lib.gevva_moe_ep_create.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(_Weights), vp, ctypes.POINTER(_EpConfig)]
    handle = vp()
    for capacity in (0, world * 8 * max_tokens - 1):
        config = _EpConfig(0, world, max_tokens, capacity, cast(fake), cast(fake), cast(fake), cast(fake),
                           cast(fake), None)
        assert lib.gevva_moe_ep_create(ctypes.byref(handle), ctypes.byref(weights), scale,
                                       ctypes.byref(config)) == -3
    # a null peer table is refused too
    config = _EpConfig(0, world, max_tokens, world * 8 * max_tokens, None, cast(fake), cast(fake), cast(fake),
                       cast(fake), None)
    assert lib.gevva_moe_ep_create(ctypes.byref(handle), ctypes.byref(weights), scale, ctypes.byref(config)) == -3


def test_python_mirror_fails_loudly_without_library(monkeypatch, tmp_path):
    from gevva_b200 import runtime
    monkeypatch.setattr(runtime, "_lib", None)
    monkeypatch.setattr(runtime, "_LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        runtime.library()
