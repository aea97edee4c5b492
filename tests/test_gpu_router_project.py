"""Router projection fused with top-8 routing (gevva_moe_route_project) against the CPU oracle.

The projection is a floating-point GEMM: the kernel accumulates in fp32 on the tensor cores, the
oracle takes the dot product in double.  Protocol: every logit within one bf16 ulp of the oracle's (plus 5e-7 of sum |x||w| for logits
that nearly cancel to zero);
ids and weights bit-exact against the oracle's router applied to the kernel's own logits (the same
bytes on both sides); and, against the oracle's own logits, ids equal on every row whose 8th and
9th largest logits differ by more than one bf16 ulp (a smaller gap can legitimately go either
way); such rows are counted and printed.  Sizes: 1, 16 (CPU-runnable configuration), 40 (the
verifier's rows), 64 (decode), 129 (two tiles, one nearly empty), 4096 (prefill) with and without
the benchmark's router bias; the same at the FP8 sidecar's operand type."""
import numpy as np
import pytest
import torch

from tests.parity_util import EXPERTS, HIDDEN, TOP_K, bf16_to_f32, bits

pytestmark = pytest.mark.gpu


def off_by(got_bits, want_bits, magnitude):
    """|got - want| in units of the bf16 step at `want`, after an allowance for fp32 accumulation
    error of 5e-7 of sum_k |x||w| (`magnitude`, per logit): a logit that nearly cancels to zero has
    a bf16 step far below the accumulation error of any fp32 GEMM over 2816 terms."""
    got, want = bf16_to_f32(got_bits).astype(np.float64), bf16_to_f32(want_bits).astype(np.float64)
    step = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    return np.maximum(np.abs(got - want) - 5e-7 * magnitude, 0.0) / step


def check_against_oracle(oracle, logits_bits, want_bits, magnitude, ids, weights, scale_bits, act=None, ws=None):
    distance = off_by(logits_bits, want_bits, magnitude)
    assert distance.max() <= 1.0, f"a logit is {distance.max()} bf16 steps from the oracle's"
    # the router on identical bytes: exact
    ow, oids = oracle.route(logits_bits, scale_bits, act, ws)
    assert (ids == oids).all()
    assert (weights.view(np.uint32) == ow.view(np.uint32)).all()
    # the oracle end to end: exact wherever the 8th/9th gap is decisive
    _, ids_end_to_end = oracle.route(want_bits, scale_bits, act, ws)
    values = bf16_to_f32(want_bits)
    if act is not None:
        values = values * (act * ws[0])[:, None]
    ordered = np.sort(values, axis=1)[:, ::-1]
    one_ulp = np.abs(ordered[:, TOP_K - 1]) * 2.0 ** -7 + 1e-30
    decisive = (ordered[:, TOP_K - 1] - ordered[:, TOP_K]) > 2 * one_ulp
    same_set = np.array([set(a) == set(b) for a, b in zip(ids, ids_end_to_end)])
    assert same_set[decisive].all()
    return int((distance > 0).sum()), int((~decisive).sum()), int((~same_set).sum())


@pytest.mark.parametrize("rows,biased", [(1, False), (16, False), (40, True), (64, False), (129, True),
                                         (4096, True), (4096, False),
                                         (6000, True),     # K split over two CTAs per tile
                                         (11000, True)])   # one CTA per tile
def test_bf16_router_projection(oracle, cuda_device, rows, biased):
    import gevva_b200 as gm
    gen = torch.Generator().manual_seed(1000 + rows)
    x = torch.randn((rows, HIDDEN), generator=gen).to(torch.bfloat16)
    router = (torch.randn((EXPERTS, HIDDEN), generator=gen) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(EXPERTS, generator=gen) * 0.5).float() if biased else None
    scale = (0.5 + torch.rand(EXPERTS, generator=gen)).to(torch.bfloat16)
    w, ids, logits = gm.route_project(x.to(cuda_device), router.to(cuda_device), scale.to(cuda_device),
                                      bias=None if bias is None else bias.to(cuda_device), want_logits=True)
    torch.cuda.synchronize()
    want = oracle.router_logits(bits(x), bits(router), None if bias is None else bias.numpy())
    off, close_rows, moved = check_against_oracle(oracle, bits(logits), want,
                                                  (x.float().abs() @ router.float().abs().t()).numpy(),
                                                  ids.cpu().numpy(), w.cpu().numpy(), bits(scale))
    print(f"router projection {rows} rows: {off} of {rows * EXPERTS} logits one ulp off; {close_rows} rows with "
          f"an 8th/9th gap within two ulp, {moved} of them routed differently from the oracle end to end")
    # repeatable, and the same without the logits output
    w2, ids2 = gm.route_project(x.to(cuda_device), router.to(cuda_device), scale.to(cuda_device),
                                bias=None if bias is None else bias.to(cuda_device))
    assert torch.equal(ids, ids2) and torch.equal(w, w2)


@pytest.mark.parametrize("rows", [1, 40, 300, 4096, 6000, 11000])
def test_fp8_router_projection(oracle, cuda_device, rows):
    import gevva_b200 as gm
    gen = torch.Generator().manual_seed(2000 + rows)
    x = torch.randn((rows, HIDDEN), generator=gen)
    act = (x.abs().amax(dim=1) / 448.0).float()
    xq = (x / act[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    router = torch.randn((EXPERTS, HIDDEN), generator=gen) * 0.02
    ws = (router.abs().max() / 448.0).float().reshape(1)
    rq = (router / ws).to(torch.float8_e4m3fn).view(torch.uint8)
    scale = torch.ones(EXPERTS, dtype=torch.bfloat16)
    w, ids, logits = gm.route_project(xq.to(cuda_device), rq.to(cuda_device), scale.to(cuda_device),
                                      activation_scales=act.to(cuda_device), weight_scale=ws.to(cuda_device),
                                      want_logits=True)
    torch.cuda.synchronize()
    want = oracle.router_logits(xq.numpy(), rq.numpy(), e4m3=True)
    off, close_rows, moved = check_against_oracle(
        oracle, bits(logits), want,
        (xq.view(torch.float8_e4m3fn).float().abs() @ rq.view(torch.float8_e4m3fn).float().abs().t()).numpy(),
        ids.cpu().numpy(), w.cpu().numpy(), bits(scale), act.numpy(), ws.numpy())
    print(f"FP8 router projection {rows} rows: {off} logits one ulp off; {close_rows} close rows, {moved} moved")


def test_router_projection_feeds_the_layer(oracle, cuda_device):
    """The fused router in front of the expert runner: the layer step made of C-ABI calls only."""
    import gevva_b200 as gm
    from gevva_b200.synthetic import SyntheticLayer
    tokens = 48
    layer = SyntheticLayer(seed=2, max_tokens=tokens, device=cuda_device, bias_std=0.5)
    layer.set_scales(0.002, 0.006)
    x = layer.inputs(tokens, seed=5)
    w, ids, logits = gm.route_project(x, layer.router_w, layer.expert_scale, bias=layer.bias, want_logits=True,
                                      status_of=layer.runner)
    out = torch.empty_like(x)
    layer.runner.launch_batch(x, ids, w, out, tokens)
    layer.runner.check()
    ow, oids = oracle.route(bits(logits), bits(layer.expert_scale))
    assert (ids.cpu().numpy() == oids).all()
    hw = {n: getattr(layer.weights, n).cpu().numpy() for n in
          ("w13", "w13_sf", "w2", "w2_sf", "alpha1", "alpha2", "in_scale_q1", "in_scale_q2")}
    want = oracle.moe_layer(bits(x), oids, ow, hw)
    got_f, want_f = bf16_to_f32(bits(out)).astype(np.float64), bf16_to_f32(want).astype(np.float64)
    assert np.linalg.norm(got_f - want_f) / np.linalg.norm(want_f) < 2e-2
