"""gevva_moe_pack_checkpoint_layer against a numpy statement of the reference's packing script
(tools/pack_trtllm_experts.py:88-148): stack, [up; gate] concatenation, the 128x4 block-scale
interleave written as the reshape/permute TensorRT-LLM documents for it, and the derived
alpha / input_scale_quant vectors.  CPU only."""
import numpy as np
import pytest

from gevva_b200.sidecar import (LAYER_TENSORS, ExpertSidecar, SidecarError, deinterleave_scales,
                                pack_checkpoint_layer, write_sidecar)


def make_checkpoint(experts, hidden, inter, seed, layer=3):
    rng = np.random.default_rng(seed)
    store = {}
    for e in range(experts):
        shared_input = np.float32(rng.uniform(0.001, 0.01))
        for name, rows, k in (("gate_proj", inter, hidden), ("up_proj", inter, hidden), ("down_proj", hidden, inter)):
            prefix = f"model.language_model.layers.{layer}.experts.{e}.{name}."
            store[prefix + "weight"] = rng.integers(0, 256, (rows, k // 2), dtype=np.uint8)
            store[prefix + "weight_scale"] = rng.integers(0, 127, (rows, k // 16), dtype=np.uint8)
            store[prefix + "weight_scale_2"] = np.float32(rng.uniform(1e-5, 1e-4))
            store[prefix + "input_scale"] = shared_input if name != "down_proj" else np.float32(rng.uniform(0.001, 0.01))
    return store


def interleave_as_documented(scales):
    """[rows, groups] row-major -> swizzled, rows % 128 == 0 and groups % 4 == 0: view as
    [rows/128, 4, 32, groups/4, 4] and move the axes to (0, 3, 2, 1, 4)."""
    rows, groups = scales.shape
    return np.ascontiguousarray(
        scales.reshape(rows // 128, 4, 32, groups // 4, 4).transpose(0, 3, 2, 1, 4)).reshape(rows, groups)


def script_statement(store, layer, experts):
    stack = lambda proj, suffix: np.stack(
        [store[f"model.language_model.layers.{layer}.experts.{e}.{proj}.{suffix}"] for e in range(experts)])
    gate_w, up_w, down_w = (stack(p, "weight") for p in ("gate_proj", "up_proj", "down_proj"))
    gate_s, up_s, down_s = (stack(p, "weight_scale") for p in ("gate_proj", "up_proj", "down_proj"))
    s13 = np.concatenate((up_s, gate_s), axis=1)
    gate_in, up_in, down_in = (stack(p, "input_scale").astype(np.float32) for p in ("gate_proj", "up_proj", "down_proj"))
    gate_g, up_g, down_g = (stack(p, "weight_scale_2").astype(np.float32) for p in ("gate_proj", "up_proj", "down_proj"))
    return {
        "w13.weight": np.concatenate((up_w, gate_w), axis=1),
        "w13.weight_scale": np.stack([interleave_as_documented(s) for s in s13]),
        "w2.weight": down_w,
        "w2.weight_scale": np.stack([interleave_as_documented(s) for s in down_s]),
        "w13.input_scale": gate_in, "w2.input_scale": down_in,
        "w13.weight_scale_2": np.stack((gate_g, up_g), axis=1), "w2.weight_scale_2": down_g,
        "g1.alpha": gate_in * gate_g, "g1.alpha_up": up_in * up_g, "g2.alpha": down_in * down_g,
        "g1.input_scale_quant": np.float32(1.0) / gate_in, "g2.input_scale_quant": np.float32(1.0) / down_in,
    }


@pytest.mark.parametrize("experts,hidden,inter", [(3, 256, 128), (2, 384, 192)])
def test_packer_equals_the_script_statement(experts, hidden, inter):
    store = make_checkpoint(experts, hidden, inter, seed=experts)
    got = pack_checkpoint_layer(store.__getitem__, 3, experts=experts, hidden=hidden, intermediate=inter)
    want = script_statement(store, 3, experts)
    assert set(got) == {t[0] for t in LAYER_TENSORS}
    for name, value in want.items():
        assert got[name].dtype == value.dtype and got[name].shape == value.shape, name
        assert (got[name].view(np.uint8) == value.view(np.uint8)).all(), name
    # the interleave is a permutation: undoing it returns the checkpoint's rows
    e = experts - 1
    back = deinterleave_scales(got["w2.weight_scale"][e])
    assert (back == store[f"model.language_model.layers.3.experts.{e}.down_proj.weight_scale"]).all()


def test_gate_up_scale_mismatch_is_an_error():
    store = make_checkpoint(2, 256, 128, seed=9)
    store["model.language_model.layers.3.experts.1.up_proj.input_scale"] = np.float32(0.5)
    with pytest.raises(SidecarError, match="gate/up activation scales differ"):
        pack_checkpoint_layer(store.__getitem__, 3, experts=2, hidden=256, intermediate=128)
    with pytest.raises(ValueError):   # a tensor of the wrong shape
        store["model.language_model.layers.3.experts.0.down_proj.weight"] = np.zeros((4, 4), np.uint8)
        pack_checkpoint_layer(store.__getitem__, 3, experts=2, hidden=256, intermediate=128)


def test_full_size_layer_passes_the_schema_check(tmp_path):
    """128 experts at Gemma-4 26B-A4B sizes -> sidecar file -> the reader's 13-tensor schema."""
    experts, hidden, inter = 128, 2816, 704
    rng = np.random.default_rng(0)
    w_in = rng.integers(0, 256, (inter, hidden // 2), dtype=np.uint8)
    s_in = rng.integers(0, 127, (inter, hidden // 16), dtype=np.uint8)
    w_out = rng.integers(0, 256, (hidden, inter // 2), dtype=np.uint8)
    s_out = rng.integers(0, 127, (hidden, inter // 16), dtype=np.uint8)

    def get(name):
        parts = name.split(".")
        expert, projection, suffix = int(parts[5]), parts[6], parts[7]
        if suffix == "weight":
            return (w_out if projection == "down_proj" else w_in) ^ np.uint8(expert)
        if suffix == "weight_scale":
            return s_out if projection == "down_proj" else s_in
        return np.float32(0.001 * (1 + expert)) if suffix == "input_scale" else np.float32(2e-5)

    tensors = pack_checkpoint_layer(get, 0)
    path = tmp_path / "experts-00.safetensors"
    write_sidecar(path, [tensors])
    with ExpertSidecar(path) as sidecar:
        sidecar.check_layers(1)
        assert (sidecar.tensor("layers.0.w13.weight")[5, 704:] == (w_in ^ np.uint8(5))).all()   # gate rows second
        assert np.allclose(sidecar.tensor("layers.0.g1.input_scale_quant")[9], 1.0 / 0.01)
