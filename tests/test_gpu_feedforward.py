"""Dense FP8 GeGLU MLP and the feed-forward pre/post steps against the CPU oracle.
Bit-exact where both sides see the same bytes (norm outputs, FP8 codes, row scales,
finalize); 2e-2 relative L2 for the FP8 GEMM outputs."""
import numpy as np
import pytest
import torch

from tests import hashgen
from tests.oracle_api import EXPERTS, HIDDEN, TOP_K, DenseOracle, bf16_to_f32

pytestmark = pytest.mark.gpu
DENSE = 2112


def bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_l2(got, want):
    got, want = got.astype(np.float64), want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def norm_weight(seed, device):
    return (1.0 + 0.25 * hashgen.hash_uniform(HIDDEN, seed, device)).to(torch.bfloat16)


@pytest.fixture(scope="module")
def dense_oracle(oracle):
    return DenseOracle(oracle)


@pytest.mark.parametrize("rows", [1, 5, 300])
def test_ff_prepare_bit_exact(dense_oracle, cuda_device, rows):
    from gevva_b200 import feedforward as ff
    x = hashgen.activations(rows, HIDDEN, 71, cuda_device)
    dw, ew, rs = norm_weight(1, cuda_device), norm_weight(2, cuda_device), norm_weight(3, cuda_device)
    got = ff.ff_prepare(x, dw, ew, rs)
    want = dense_oracle.ff_prepare(bits(x), bits(dw), bits(ew), bits(rs))
    for g, w, name in zip(got, want, ("dense", "expert", "router")):
        assert (bits(g) == w).all(), name


def test_pack_fp8_matches_oracle(dense_oracle, cuda_device):
    from gevva_b200 import feedforward as ff
    w = hashgen.expert_weights_chunk(0, 1, 256, HIDDEN, 33, cuda_device)[0]
    q, scale = ff.pack_fp8(w)
    oq, oscale = dense_oracle.pack_fp8(w.cpu().numpy())
    assert scale == oscale and (q.cpu().numpy() == oq).all()


@pytest.fixture(scope="module")
def dense_weights(cuda_device):
    from gevva_b200 import feedforward as ff
    gate = hashgen.expert_weights_chunk(0, 1, DENSE, HIDDEN, 51, cuda_device)[0]
    up = hashgen.expert_weights_chunk(0, 1, DENSE, HIDDEN, 52, cuda_device)[0]
    down = hashgen.expert_weights_chunk(0, 1, HIDDEN, DENSE, 53, cuda_device)[0]
    gq, gs = ff.pack_fp8(gate)
    uq, us = ff.pack_fp8(up)
    dq, ds = ff.pack_fp8(down)
    return torch.cat([gq, uq]).contiguous(), dq, gs, us, ds


@pytest.mark.parametrize("tokens", [1, 37, 300])
def test_dense_mlp_stages(dense_oracle, dense_weights, cuda_device, tokens):
    from gevva_b200 import feedforward as ff
    gate_up, down, gs, us, ds = dense_weights
    mlp = ff.DenseMlp(gate_up, down, gs, us, ds, 512)
    x = hashgen.activations(tokens, HIDDEN, 81, cuda_device)
    out, out_scales = mlp.launch(x)
    torch.cuda.synchronize()
    # stage 1: row quantisation, bit-exact
    q, s = dense_oracle.quantize_rows(bits(x))
    assert (mlp.buffer(0, torch.uint8)[: tokens * HIDDEN].cpu().numpy().reshape(tokens, HIDDEN) == q).all()
    assert (mlp.buffer(1, torch.float32)[:tokens].cpu().numpy() == s).all()
    # stage 2: gate|up GEMM on the same FP8 bytes
    want_gu = dense_oracle.gemm(q, gate_up.cpu().numpy())
    got_gu = bits(mlp.buffer(2, torch.bfloat16)[: tokens * 2 * DENSE]).reshape(tokens, 2 * DENSE)
    assert rel_l2(bf16_to_f32(got_gu), bf16_to_f32(want_gu)) < 5e-3
    # stage 3: GeGLU + requantise, bit-exact given the GPU's own gate|up output
    pq, ps = dense_oracle.gelu_quantize(got_gu, s, gs, us)
    assert (mlp.buffer(3, torch.uint8)[: tokens * DENSE].cpu().numpy().reshape(tokens, DENSE) == pq).all()
    assert (out_scales.cpu().numpy() == ps).all()
    # stage 4: down GEMM
    want_out = dense_oracle.gemm(pq, down.cpu().numpy())
    assert rel_l2(bf16_to_f32(bits(out)), bf16_to_f32(want_out)) < 5e-3


def test_ff_finalize_bit_exact(dense_oracle, cuda_device):
    from gevva_b200 import feedforward as ff
    rows = 41
    dense = hashgen.activations(rows, HIDDEN, 91, cuda_device)
    routes = hashgen.activations(rows * TOP_K, HIDDEN, 92, cuda_device)
    residual = hashgen.activations(rows, HIDDEN, 93, cuda_device)
    gen = torch.Generator().manual_seed(4)
    rw = (torch.rand((rows, TOP_K), generator=gen) * 0.3).to(cuda_device)
    inverse = torch.randperm(rows * TOP_K, generator=gen).to(torch.int32).to(cuda_device)
    act_scales = (0.5 + torch.rand(rows, generator=gen)).to(cuda_device)
    dw, ew, cw = norm_weight(4, cuda_device), norm_weight(5, cuda_device), norm_weight(6, cuda_device)
    scalar = torch.tensor([0.75], dtype=torch.bfloat16, device=cuda_device)
    for scales, proj in ((act_scales, 0.013), (None, 1.0)):
        proj_dev = None if scales is None else torch.tensor([proj], dtype=torch.float32, device=cuda_device)
        got = ff.ff_finalize(dense, dw, routes, rw, inverse, ew, cw, residual, scalar, scales, proj_dev)
        want = dense_oracle.finalize(bits(dense), bits(dw), bits(routes), rw.cpu().numpy(),
                                     inverse.cpu().numpy(), bits(ew), bits(cw), bits(residual),
                                     bits(scalar)[0], None if scales is None else scales.cpu().numpy(), float(np.float32(proj)))
        assert (bits(got) == want).all()


def test_layer_wiring_against_oracle(oracle, dense_oracle, dense_weights, cuda_device):
    """One layer of the FFN stack (pre-norms, router, experts beside the dense MLP, fused
    finalize) against the same chain on the CPU; the router logits are shared so that both
    sides route identically."""
    import gevva_b200 as gm
    from gevva_b200 import feedforward as ff
    from gevva_b200.synthetic import make_packed_experts
    tokens = 24
    p = make_packed_experts(3, cuda_device, chunk=32)
    s1, s2 = 6.0 / 2688.0, 8.0 / 2688.0
    ones = torch.ones(EXPERTS, dtype=torch.float32, device=cuda_device)
    w = gm.ExpertWeights(p["w13"], p["w13_sf"], p["w2"], p["w2_sf"], (p["g13"] * s1).contiguous(),
                         (p["g2"] * s2).contiguous(), (ones / s1).contiguous(), (ones / s2).contiguous())
    gate_up, down, gs, us, ds = dense_weights
    dw, ew, rs = norm_weight(1, cuda_device), norm_weight(2, cuda_device), norm_weight(3, cuda_device)
    dpost, epost, cpost = norm_weight(4, cuda_device), norm_weight(5, cuda_device), norm_weight(6, cuda_device)
    scalar = torch.tensor([0.5], dtype=torch.bfloat16, device=cuda_device)
    router_w = (hashgen.hash_uniform(EXPERTS * HIDDEN, 5, cuda_device) * 0.0346).view(EXPERTS, HIDDEN).to(
        torch.bfloat16)
    layer = ff.FeedForwardLayer(dw, ew, rs, router_w, torch.ones(EXPERTS, dtype=torch.bfloat16, device=cuda_device),
                                dpost, epost, cpost, scalar, gm.Nvfp4ExpertRunner(w, 64),
                                ff.DenseMlp(gate_up, down, gs, us, ds, 64))
    hidden = hashgen.activations(tokens, HIDDEN, 101, cuda_device)
    got = layer.forward(hidden, torch.cuda.Stream(device=cuda_device))
    torch.cuda.synchronize()
    # CPU chain
    dense_in, expert_in, router_in = dense_oracle.ff_prepare(bits(hidden), bits(dw), bits(ew), bits(rs))
    # the library's own logits (fused projection, deterministic), so that both sides route alike
    _, _, logits = gm.route_project(torch.from_numpy(router_in.view(np.int16)).to(cuda_device).view(torch.bfloat16),
                                    router_w, torch.ones(EXPERTS, dtype=torch.bfloat16, device=cuda_device),
                                    want_logits=True)
    rw, ids = oracle.route(bits(logits), bits(torch.ones(EXPERTS, dtype=torch.bfloat16)))
    hw = dict(w13=p["w13"].cpu().numpy(), w13_sf=p["w13_sf"].cpu().numpy(), w2=p["w2"].cpu().numpy(),
              w2_sf=p["w2_sf"].cpu().numpy(), alpha1=w.alpha1.cpu().numpy(), alpha2=w.alpha2.cpu().numpy(),
              in_scale_q1=w.in_scale_q1.cpu().numpy(), in_scale_q2=w.in_scale_q2.cpu().numpy())
    _, routed, inverse = oracle.moe_layer(expert_in, ids, rw, hw, want_routed=True)
    q, s = dense_oracle.quantize_rows(dense_in)
    pq, ps = dense_oracle.gelu_quantize(dense_oracle.gemm(q, gate_up.cpu().numpy()), s, gs, us)
    dense_out = dense_oracle.gemm(pq, down.cpu().numpy())
    want = dense_oracle.finalize(dense_out, bits(dpost), routed, rw, inverse, bits(epost), bits(cpost),
                                 bits(hidden), bits(scalar)[0], ps, ds)
    assert rel_l2(bf16_to_f32(bits(got)), bf16_to_f32(want)) < 2e-2


def test_ffn_stack_runs_at_configured_size(cuda_device):
    """30 layers x 2048 tokens: finite output, identical on a second pass, and the two-stream
    schedule equals the single-stream one."""
    from gevva_b200.synthetic import SyntheticStack
    stack = SyntheticStack(30, 2048, cuda_device, distinct_experts=False)
    hidden = hashgen.activations(2048, HIDDEN, 7, cuda_device)
    a = stack.forward(hidden)
    b = stack.forward(hidden)
    c = stack.forward(hidden, concurrent=False)
    torch.cuda.synchronize()
    assert torch.isfinite(a.float()).all() and a.float().abs().max() > 0
    assert torch.equal(a, b) and torch.equal(a, c)


def test_thirty_layers_captured_into_one_graph_at_verifier_size(cuda_device):
    """The decode-side caller of the path: rows = sessions x (drafts + 1) <= 40, the whole
    30-layer enqueue (prepare -> router -> route -> experts unreduced beside the dense MLP on a
    second stream -> finalize) captured once and replayed (src/cuda/runtime/verifier.cuh:960-1042,
    capture :1058-1078).  Replays must reproduce the eager pass bit for bit, also after the input
    buffer has been refilled."""
    from gevva_b200.synthetic import SyntheticStack
    rows = 40
    stack = SyntheticStack(30, rows, cuda_device, distinct_experts=False)
    first = hashgen.activations(rows, HIDDEN, 11, cuda_device)
    second = hashgen.activations(rows, HIDDEN, 12, cuda_device)
    want_first = stack.forward(first, concurrent=False).clone()
    want_second = stack.forward(second, concurrent=False).clone()
    torch.cuda.synchronize()
    assert not torch.equal(want_first, want_second)
    static_in = first.clone()
    stack.forward(static_in)            # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = stack.forward(static_in)
    for _ in range(2):
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_out, want_first)
    static_in.copy_(second)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, want_second)
    for layer in stack.layers:
        layer.experts.check()
