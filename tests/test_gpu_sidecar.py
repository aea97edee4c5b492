"""A synthetic layer stored as a packed expert sidecar and loaded back through the reader
drives the runner to the same output bits as the in-memory weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sidecar_round_trip_runs_the_layer(tmp_path):
    import gevva_b200
    from gevva_b200.runtime import Nvfp4ExpertRunner
    from gevva_b200.sidecar import ExpertSidecar, synthetic_layer_tensors, write_sidecar
    from gevva_b200.synthetic import SyntheticLayer

    tokens = 96
    layer = SyntheticLayer(seed=3, max_tokens=tokens)
    layer.set_scales(0.002, 0.006)
    x = layer.inputs(tokens, seed=11)
    expected = layer.forward(x)
    torch.cuda.synchronize()

    path = tmp_path / "experts-00.safetensors"
    write_sidecar(path, [synthetic_layer_tensors(layer.packed, layer.weights, layer.s1, layer.s2)])
    with ExpertSidecar(path) as sidecar:
        sidecar.check_layers(1)
        weights = sidecar.layer_weights(0, device=x.device)
    for name in ("w13", "w13_sf", "w2", "w2_sf", "alpha1", "alpha2", "in_scale_q1", "in_scale_q2"):
        assert torch.equal(getattr(weights, name), getattr(layer.weights, name)), name

    runner = Nvfp4ExpertRunner(weights, tokens)
    route_weights, ids = gevva_b200.route_128_top8(layer.logits(x), layer.expert_scale)
    out = torch.empty_like(x)
    runner.launch_batch(x, ids, route_weights, out, tokens)
    runner.check()
    assert torch.equal(out, expected)
