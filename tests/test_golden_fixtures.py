"""The CPU oracle must reproduce the committed vectors in tests/golden/moe_golden.npz
bit for bit (they were made by tests/golden/make_golden.py)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "moe_golden.npz"))


@pytest.fixture(scope="module")
def maker():
    import make_golden
    return make_golden


def test_router_and_sort_vectors(oracle, golden, maker):
    import torch
    rows = 64
    rank = (np.arange(128)[None, :] * 37 + np.arange(rows)[:, None] * 19) & 127
    logits = torch.tensor((rank - 64) * 0.0625, dtype=torch.float32).to(torch.bfloat16)
    scale = torch.tensor(0.5 + (np.arange(128) % 17) * 0.07, dtype=torch.float32).to(torch.bfloat16)
    w, ids = oracle.route(maker.bits(logits), maker.bits(scale))
    assert (ids == golden["router_ids"]).all()
    assert (w.view(np.uint32) == golden["router_weights"].view(np.uint32)).all()
    plan = oracle.sort(maker.skewed_ids(300))
    for key in ("sorted_experts", "sorted_routes", "inverse", "offsets", "scale_rows"):
        assert (plan[key] == golden["sort_" + key]).all(), key


def test_quantiser_vectors(oracle, golden, maker):
    from tests import hashgen
    ids = maker.skewed_ids(37)
    plan = oracle.sort(ids)
    x = hashgen.activations(37, 2816, 3)
    q1 = np.full(128, np.float32(1) / maker.S1, np.float32)
    codes, sf = oracle.quantize_sorted(maker.bits(x), q1, plan)
    assert (maker.sha(codes) == golden["quant_codes_sha"]).all()
    assert (maker.sha(sf) == golden["quant_sf_sha"]).all()
    assert (codes[0] == golden["quant_codes_row0"]).all()
    fused = hashgen.activations(37 * 8, 1408, 9, scale=0.9)
    q2 = np.full(128, np.float32(1) / maker.S2, np.float32)
    codes2, sf2 = oracle.geglu_quantize(maker.bits(fused), q2, plan)
    assert (maker.sha(codes2) == golden["geglu_codes_sha"]).all()
    assert (maker.sha(sf2) == golden["geglu_sf_sha"]).all()


def test_layer_vector(oracle, golden, maker):
    """The 16-token configuration end to end (packs all 128 experts: about half a minute)."""
    packed = maker.packed_layer(oracle)
    for key in ("w13", "w13_sf", "w2", "w2_sf"):
        assert (maker.sha(packed[key]) == golden["packed_" + key + "_sha"]).all(), key
    case = maker.layer_case(oracle, packed)
    assert (case["layer_ids"] == golden["layer_ids"]).all()
    assert (case["layer_out"] == golden["layer_out"]).all()
    assert (case["layer_inverse"] == golden["layer_inverse"]).all()
    assert (case["layer_routed_sha"] == golden["layer_routed_sha"]).all()
