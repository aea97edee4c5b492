"""Parity of the CUDA path (through the C ABI) with the CPU oracle on a B200.

Bit-exact: top-k ids, router weights, permutation arrays, FP4 codes and E4M3 scale
bytes (each stage fed the same bytes on both sides).  Tolerance 2e-2 relative L2
for GEMM outputs and the layer output (accumulation order differs)."""
import numpy as np
import pytest
import torch

from tests import hashgen
from tests.oracle_api import EXPERTS, HIDDEN, INTER, TOP_K, bf16_to_f32, sf_bytes

pytestmark = pytest.mark.gpu

W13_OUT = 2 * INTER
REL_L2 = 2e-2


def bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(a, device):
    return torch.from_numpy(a.view(np.int16).copy()).to(device).view(torch.bfloat16)


def rel_l2(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def random_ids(tokens, seed):
    rng = np.random.default_rng(seed)
    return np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int32)


def skewed_ids(tokens):
    """Route 0 always on expert 0, the rest hashed into experts 1..36: few active experts
    with unequal row counts (the shape of the reference's repeatability test routing,
    src/nvfp4_cutlass.cu:1962-1974)."""
    t = np.arange(tokens, dtype=np.uint64)[:, None]
    k = np.arange(TOP_K, dtype=np.uint64)[None, :]
    mixed = (t * 2654435761 + k * 2246822519) & 0xFFFFFFFF
    ids = 1 + ((mixed >> 24) + k * k) % 36
    ids[:, 0] = 0
    # a token must not name one expert twice for the layer semantics to make sense; keep
    # duplicates out by re-drawing deterministically
    ids = ids.astype(np.int32)
    for row in ids:
        seen = set()
        for j in range(TOP_K):
            while int(row[j]) in seen:
                row[j] = 1 + (row[j] + 7) % 36
            seen.add(int(row[j]))
    return ids


@pytest.fixture(scope="module")
def gm(cuda_device):
    import gevva_b200
    return gevva_b200


@pytest.fixture(scope="module")
def packed(cuda_device, gm):
    """One layer of hash-generated experts packed on the GPU, plus host copies."""
    out = {k: [] for k in ("w13", "w13_sf", "g13", "w2", "w2_sf", "g2")}
    chunk = 16
    for first in range(0, EXPERTS, chunk):
        w13 = hashgen.expert_weights_chunk(first, chunk, W13_OUT, HIDDEN, 11, cuda_device)
        c, s, g = gm.pack_experts(w13)
        out["w13"].append(c), out["w13_sf"].append(s), out["g13"].append(g)
        del w13
        w2 = hashgen.expert_weights_chunk(first, chunk, HIDDEN, INTER, 12, cuda_device)
        c, s, g = gm.pack_experts(w2)
        out["w2"].append(c), out["w2_sf"].append(s), out["g2"].append(g)
        del w2
    dev = {k: torch.cat(v) for k, v in out.items()}
    host = {k: v.cpu().numpy() for k, v in dev.items()}
    return dev, host


def make_weights(gm, packed, s1, s2, device, varied=False):
    """`varied`: every expert gets its own static activation scales (s * a factor of 1 to
    1.125 that depends on the expert), so a scale taken from the wrong expert changes bits."""
    dev, host = packed
    ones = torch.ones(EXPERTS, dtype=torch.float32, device=device)
    index = torch.arange(EXPERTS, dtype=torch.float32, device=device)
    f1 = ones + (index % 5) * 0.03125 if varied else ones
    f2 = ones + (index % 3) * 0.0625 if varied else ones
    w = gm.ExpertWeights(dev["w13"], dev["w13_sf"], dev["w2"], dev["w2_sf"],
                         (dev["g13"] * s1 * f1).contiguous(), (dev["g2"] * s2 * f2).contiguous(),
                         (ones / (s1 * f1)).contiguous(), (ones / (s2 * f2)).contiguous())
    hw = dict(w13=host["w13"], w13_sf=host["w13_sf"], w2=host["w2"], w2_sf=host["w2_sf"],
              alpha1=w.alpha1.cpu().numpy(), alpha2=w.alpha2.cpu().numpy(),
              in_scale_q1=w.in_scale_q1.cpu().numpy(), in_scale_q2=w.in_scale_q2.cpu().numpy())
    return w, hw


# Static activation scales amax/(6*448): the hashed activations are bounded by 3.4, and
# gelu(gate)*up of the w13 output stays below 16 for these weights.
S1 = np.float32(4.0 / (6.0 * 448.0))
S2 = np.float32(16.0 / (6.0 * 448.0))


@pytest.fixture(scope="module")
def weights(gm, packed, cuda_device):
    return make_weights(gm, packed, float(S1), float(S2), cuda_device)


@pytest.fixture(scope="module")
def varied_weights(gm, packed, cuda_device):
    return make_weights(gm, packed, float(S1), float(S2), cuda_device, varied=True)


# ---------------------------------------------------------------------------------------
def test_packer_matches_oracle(gm, packed, oracle, cuda_device):
    dev, host = packed
    for expert in (0, 77, 127):
        w13 = hashgen.expert_weights_chunk(expert, 1, W13_OUT, HIDDEN, 11, "cpu")[0].numpy()
        c, s, g = oracle.pack_weight(w13)
        assert (host["w13"][expert] == c).all()
        assert (host["w13_sf"][expert] == s).all()
        assert host["g13"][expert] == g
        w2 = hashgen.expert_weights_chunk(expert, 1, HIDDEN, INTER, 12, "cpu")[0].numpy()
        c, s, g = oracle.pack_weight(w2)
        assert (host["w2"][expert] == c).all()
        assert (host["w2_sf"][expert] == s).all()
        assert host["g2"][expert] == g


def test_router_permutation_logits(gm, oracle, cuda_device):
    rows = 64
    rank = (np.arange(EXPERTS)[None, :] * 37 + np.arange(rows)[:, None] * 19) & 127
    logits = torch.tensor((rank - 64) * 0.0625, dtype=torch.float32).to(torch.bfloat16).to(cuda_device)
    scale = torch.tensor(0.5 + (np.arange(EXPERTS) % 17) * 0.07, dtype=torch.float32).to(
        torch.bfloat16).to(cuda_device)
    w, ids = gm.route_128_top8(logits, scale)
    ow, oids = oracle.route(bits(logits), bits(scale))
    assert (ids.cpu().numpy() == oids).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


@pytest.mark.parametrize("rows", [1, 3, 4, 5, 257, 4096])
def test_router_random_with_ties(gm, oracle, cuda_device, rows):
    gen = torch.Generator(device="cpu").manual_seed(rows)
    logits = (torch.randn((rows, EXPERTS), generator=gen) * 0.5).to(torch.bfloat16)
    logits[0, :16] = 0.0
    logits[0, 1:16:2] = -0.0
    if rows > 2:
        logits[2] = logits[2, 0]          # a whole row of ties
    scale = (0.5 + torch.rand(EXPERTS, generator=gen)).to(torch.bfloat16)
    w, ids = gm.route_128_top8(logits.to(cuda_device), scale.to(cuda_device))
    ow, oids = oracle.route(bits(logits), bits(scale))
    assert (ids.cpu().numpy() == oids).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


def test_router_padded_rows_and_fp8_rescale(gm, oracle, cuda_device):
    gen = torch.Generator(device="cpu").manual_seed(5)
    rows = 37
    padded = torch.randn((48, 160), generator=gen).to(torch.bfloat16)
    view = padded[:rows, :EXPERTS]
    act = (0.5 + torch.rand(rows, generator=gen)).float()
    ws = torch.tensor([0.37], dtype=torch.float32)
    scale = torch.ones(EXPERTS, dtype=torch.bfloat16)
    dview = padded.to(cuda_device)[:rows, :EXPERTS]
    w, ids = gm.route_128_top8(dview, scale.to(cuda_device), act.to(cuda_device), ws.to(cuda_device))
    ow, oids = oracle.route(bits(view.contiguous()), bits(scale), act.numpy(), ws.numpy())
    assert (ids.cpu().numpy() == oids).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


def plan_arrays(gm, runner, routes):
    from gevva_b200 import runtime as rt
    i32 = torch.int32
    return dict(
        sorted_experts=runner.buffer(rt.BUF_SORTED_EXPERTS, i32)[:routes].cpu().numpy(),
        sorted_routes=runner.buffer(rt.BUF_SORTED_ROUTES, i32)[:routes].cpu().numpy(),
        inverse=runner.buffer(rt.BUF_INVERSE_ROUTES, i32)[:routes].cpu().numpy(),
        offsets=runner.buffer(rt.BUF_EXPERT_OFFSETS, i32)[:EXPERTS].cpu().numpy(),
        scale_rows=runner.buffer(rt.BUF_SCALE_ROW_OFFSETS, i32)[:EXPERTS].cpu().numpy(),
        num_tiles=int(runner.buffer(rt.BUF_NUM_TILES, i32)[0]),
        tile_expert=runner.buffer(rt.BUF_TILE_EXPERT, i32).cpu().numpy())


@pytest.fixture(scope="module")
def big_runner(gm, weights):
    return gm.Nvfp4ExpertRunner(weights[0], 4096)


@pytest.mark.parametrize("tokens,kind", [(1, "random"), (2, "random"), (7, "random"), (16, "random"),
                                         (128, "random"), (129, "random"), (1000, "skewed"),
                                         (4096, "random"), (4096, "skewed")])
def test_route_sort_matches_oracle(gm, oracle, big_runner, cuda_device, tokens, kind):
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, tokens) if kind == "random" else skewed_ids(tokens)
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=dev_ids)
    assert big_runner.last_status() == 0
    got = plan_arrays(gm, big_runner, tokens * TOP_K)
    want = oracle.sort(ids)
    for key in ("sorted_experts", "sorted_routes", "inverse", "offsets", "scale_rows"):
        assert (got[key] == want[key]).all(), key
    counts = np.bincount(ids.reshape(-1), minlength=EXPERTS)
    tiles = (counts + 127) // 128
    assert got["num_tiles"] == tiles.sum()
    assert (got["tile_expert"][:tiles.sum()] == np.repeat(np.arange(EXPERTS), tiles)).all()


def test_bad_expert_id_is_reported(gm, big_runner, cuda_device):
    from gevva_b200 import runtime as rt
    for tokens in (4, 300):
        ids = random_ids(tokens, 1)
        ids[tokens // 2, 3] = 128
        big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=torch.from_numpy(ids).to(cuda_device))
        assert big_runner.last_status() == -1
        assert big_runner.last_status() == 0  # cleared by the read


def test_capacity_and_argument_errors(gm, weights, cuda_device):
    runner = gm.Nvfp4ExpertRunner(weights[0], 16)
    x = torch.zeros((17, HIDDEN), dtype=torch.bfloat16, device=cuda_device)
    ids = torch.zeros((17, TOP_K), dtype=torch.int32, device=cuda_device)
    with pytest.raises(gm.GevvaMoeError):
        runner.launch_batch_unreduced(x, ids, 17)
    with pytest.raises(gm.GevvaMoeError):
        gm.Nvfp4ExpertRunner(weights[0], 32, shared_scratch=runner)  # capacity mismatch
    with pytest.raises(gm.GevvaMoeError):
        gm.Nvfp4ExpertRunner(weights[0], 0)


@pytest.mark.parametrize("tokens,kind", [(1, "random"), (16, "random"), (128, "skewed"), (129, "skewed"),
                                         (300, "random")])
def test_input_quantiser_bit_exact(gm, oracle, weights, big_runner, cuda_device, tokens, kind):
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 7 + tokens) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, 3, "cpu")
    if tokens > 1:
        x[1, 32:48] = 0          # an all-zero block: scale byte 0, codes 0
        x[1, 48] = -0.0
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    big_runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, tokens, input=x.to(cuda_device),
                             expert_ids=dev_ids)
    assert big_runner.last_status() == 0
    routes = tokens * TOP_K
    plan = oracle.sort(ids)
    want_codes, want_sf = oracle.quantize_sorted(bits(x), weights[1]["in_scale_q1"], plan)
    got_codes = big_runner.buffer(rt.BUF_INPUT_CODES)[: routes * HIDDEN // 2].cpu().numpy()
    assert (got_codes.reshape(routes, -1) == want_codes).all()
    got_sf = big_runner.buffer(rt.BUF_INPUT_SF)[: sf_bytes(routes, HIDDEN)].cpu().numpy()
    # compare only the bytes this launch owns (padding rows keep earlier contents)
    groups = HIDDEN // 16
    for expert in np.unique(ids):
        rows = int((plan["sorted_experts"] == expert).sum())
        base = plan["scale_rows"][expert] * groups
        r = np.arange(rows)[:, None]
        g = np.arange(groups)[None, :]
        off = base + (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
        assert (got_sf[off] == want_sf[off]).all(), int(expert)


def stage_inputs(oracle, weights, tokens, kind, seed):
    ids = random_ids(tokens, seed) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, seed, "cpu")
    plan = oracle.sort(ids)
    codes, sf = oracle.quantize_sorted(bits(x), weights[1]["in_scale_q1"], plan)
    return ids, x, plan, codes, sf


def upload(runner, buffer_id, array):
    flat = torch.from_numpy(np.ascontiguousarray(array).reshape(-1).view(np.uint8))
    runner.buffer(buffer_id)[: flat.numel()].copy_(flat)


@pytest.mark.parametrize("tokens,kind", [(16, "random"), (40, "skewed")])
def test_w13_gemm_stage(gm, oracle, weights, big_runner, cuda_device, tokens, kind):
    from gevva_b200 import runtime as rt
    ids, x, plan, codes, sf = stage_inputs(oracle, weights, tokens, kind, 21)
    routes = tokens * TOP_K
    big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=torch.from_numpy(ids).to(cuda_device))
    upload(big_runner, rt.BUF_INPUT_CODES, codes)
    upload(big_runner, rt.BUF_INPUT_SF, sf)
    big_runner.launch_stages(rt.STAGE_W13, tokens)
    assert big_runner.last_status() == 0
    got = big_runner.buffer(rt.BUF_W13_OUT, torch.bfloat16)[: routes * W13_OUT].view(routes, W13_OUT)
    hw = weights[1]
    want = oracle.grouped_gemm(codes, sf, plan, hw["w13"], hw["w13_sf"], hw["alpha1"], W13_OUT, HIDDEN)
    err = rel_l2(bf16_to_f32(bits(got)), bf16_to_f32(want))
    assert err < 5e-3, err


@pytest.mark.parametrize("tokens,kind", [(16, "random"), (129, "skewed")])
def test_geglu_quantiser_bit_exact(gm, oracle, weights, big_runner, cuda_device, tokens, kind):
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 31) if kind == "random" else skewed_ids(tokens)
    routes = tokens * TOP_K
    plan = oracle.sort(ids)
    fused = hashgen.activations(routes, W13_OUT, 9, "cpu", scale=0.9)
    fused[0, :16] = 0
    big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=torch.from_numpy(ids).to(cuda_device))
    upload(big_runner, rt.BUF_W13_OUT, bits(fused))
    big_runner.launch_stages(rt.STAGE_GEGLU, tokens)
    assert big_runner.last_status() == 0
    want_codes, want_sf = oracle.geglu_quantize(bits(fused), weights[1]["in_scale_q2"], plan)
    got_codes = big_runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2].cpu().numpy()
    assert (got_codes.reshape(routes, -1) == want_codes).all()
    got_sf = big_runner.buffer(rt.BUF_INTER_SF)[: sf_bytes(routes, INTER)].cpu().numpy()
    groups = INTER // 16
    for expert in np.unique(ids):
        rows = int((plan["sorted_experts"] == expert).sum())
        base = plan["scale_rows"][expert] * groups
        r = np.arange(rows)[:, None]
        g = np.arange(groups)[None, :]
        off = base + (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
        assert (got_sf[off] == want_sf[off]).all(), int(expert)


@pytest.mark.parametrize("tokens,kind", [(16, "random"), (300, "skewed"), (4096, "random")])
def test_fused_w13_epilogue_equals_separate_kernels(gm, weights, big_runner, cuda_device, tokens, kind):
    """GeGLU + requantise inside the w13 epilogue must give the very bytes that the bf16
    GEMM followed by the stand-alone GeGLU quantiser gives (same accumulators, same
    bf16 rounding point, same block quantiser)."""
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 77) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, 61, cuda_device)
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    routes = tokens * TOP_K
    codes = big_runner.buffer(rt.BUF_INTER_CODES)
    sf = big_runner.buffer(rt.BUF_INTER_SF)
    big_runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, tokens, input=x, expert_ids=dev_ids)
    results = []
    for extra in (rt.STAGE_UNFUSED, 0):
        codes.zero_()
        sf.zero_()
        big_runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU | extra, tokens)
        assert big_runner.last_status() == 0
        results.append((codes[: routes * INTER // 2].clone(), sf.clone()))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])
    assert results[0][0].any() and results[0][1].any()


def test_w2_gemm_stage(gm, oracle, weights, big_runner, cuda_device):
    from gevva_b200 import runtime as rt
    tokens = 24
    ids = skewed_ids(tokens)
    routes = tokens * TOP_K
    plan = oracle.sort(ids)
    fused = hashgen.activations(routes, W13_OUT, 19, "cpu", scale=0.9)
    codes, sf = oracle.geglu_quantize(bits(fused), weights[1]["in_scale_q2"], plan)
    big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=torch.from_numpy(ids).to(cuda_device))
    upload(big_runner, rt.BUF_INTER_CODES, codes)
    upload(big_runner, rt.BUF_INTER_SF, sf)
    big_runner.launch_stages(rt.STAGE_W2, tokens)
    assert big_runner.last_status() == 0
    got = big_runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN].view(routes, HIDDEN)
    hw = weights[1]
    want = oracle.grouped_gemm(codes, sf, plan, hw["w2"], hw["w2_sf"], hw["alpha2"], HIDDEN, INTER)
    err = rel_l2(bf16_to_f32(bits(got)), bf16_to_f32(want))
    assert err < 5e-3, err


def test_reduce_bit_exact(gm, oracle, big_runner, cuda_device):
    from gevva_b200 import runtime as rt
    tokens = 33
    ids = random_ids(tokens, 2)
    routes = tokens * TOP_K
    routed = hashgen.activations(routes, HIDDEN, 29, "cpu")
    w = torch.rand((tokens, TOP_K), generator=torch.Generator().manual_seed(1)) * 0.3
    big_runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=torch.from_numpy(ids).to(cuda_device))
    upload(big_runner, rt.BUF_W2_OUT, bits(routed))
    out = torch.empty((tokens, HIDDEN), dtype=torch.bfloat16, device=cuda_device)
    big_runner.launch_stages(rt.STAGE_REDUCE, tokens, route_weights=w.to(cuda_device), output=out)
    want = oracle.reduce(bits(routed), w.numpy(), oracle.sort(ids)["inverse"], tokens)
    assert (bits(out) == want).all()


@pytest.mark.parametrize("tokens,kind", [(1, "router"), (16, "router"), (40, "skewed")])
def test_layer_against_oracle(gm, oracle, weights, cuda_device, tokens, kind):
    """Config-0 shape (16 tokens) and neighbours: ids exact, output within 2e-2 rel-L2."""
    w, hw = weights
    x = hashgen.activations(tokens, HIDDEN, 41, "cpu")
    dx = x.to(cuda_device)
    if kind == "router":
        router_w = (hashgen.hash_uniform(EXPERTS * HIDDEN, 5, "cpu") * 0.0346).view(EXPERTS, HIDDEN)
        logits = (x.float() @ router_w.t()).to(torch.bfloat16)
        scale = torch.ones(EXPERTS, dtype=torch.bfloat16)
        rw, ids = gm.route_128_top8(logits.to(cuda_device), scale.to(cuda_device))
        orw, oids = oracle.route(bits(logits), bits(scale))
        assert (ids.cpu().numpy() == oids).all()
        assert (rw.cpu().numpy().view(np.uint32) == orw.view(np.uint32)).all()
    else:
        ids = torch.from_numpy(skewed_ids(tokens)).to(cuda_device)
        rw = torch.tensor([0.24, 0.19, 0.15, 0.12, 0.10, 0.08, 0.07, 0.05], device=cuda_device).repeat(tokens, 1)
    runner = gm.Nvfp4ExpertRunner(w, max(tokens, 2))
    out = torch.empty_like(dx)
    if tokens == 1:
        runner.launch(dx, ids, rw, out)
    else:
        runner.launch_batch(dx, ids, rw, out, tokens)
    runner.check()
    want, want_routed, want_inverse = oracle.moe_layer(bits(x), ids.cpu().numpy(), rw.cpu().numpy(), hw,
                                                       want_routed=True)
    err = rel_l2(bf16_to_f32(bits(out)), bf16_to_f32(want))
    assert err < REL_L2, err
    assert np.abs(bf16_to_f32(want)).max() > 0
    # unreduced form on a runner sharing the first one's scratch
    second = gm.Nvfp4ExpertRunner(w, max(tokens, 2), shared_scratch=runner)
    second.launch_batch_unreduced(dx, ids, tokens)
    second.check()
    assert (second.inverse_routes().cpu().numpy() == want_inverse).all()
    routed = second.routed_output()
    assert rel_l2(bf16_to_f32(bits(routed)), bf16_to_f32(want_routed)) < REL_L2
    # reducing the exposed buffer by hand reproduces launch_batch bit for bit
    manual = oracle.reduce(bits(routed), rw.cpu().numpy(), want_inverse, tokens)
    assert (manual == bits(out)).all()


@pytest.mark.parametrize("tokens", [5, 130, 300])
def test_distinct_expert_scales_stage_by_stage(gm, oracle, varied_weights, cuda_device, tokens):
    """Per-expert static scales that all differ: input codes and scale bytes, and the fused
    w13 epilogue's codes and scale bytes (same GEMM output, separate kernels as the checker),
    are those of the oracle with every expert's own scale."""
    from gevva_b200 import runtime as rt
    w, hw = varied_weights
    runner = gm.Nvfp4ExpertRunner(w, tokens)
    ids = random_ids(tokens, 900 + tokens)
    x = hashgen.activations(tokens, HIDDEN, 77, "cpu")
    routes = tokens * TOP_K
    runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, tokens, input=x.to(cuda_device),
                         expert_ids=torch.from_numpy(ids).to(cuda_device))
    assert runner.last_status() == 0
    plan = oracle.sort(ids)
    want_codes, want_sf = oracle.quantize_sorted(bits(x), hw["in_scale_q1"], plan)
    got_codes = runner.buffer(rt.BUF_INPUT_CODES)[: routes * HIDDEN // 2].cpu().numpy()
    assert (got_codes.reshape(routes, -1) == want_codes).all()
    got_sf = runner.buffer(rt.BUF_INPUT_SF)[: sf_bytes(routes, HIDDEN)].cpu().numpy()
    groups = HIDDEN // 16
    for expert in np.unique(ids):
        rows = int((plan["sorted_experts"] == expert).sum())
        base = plan["scale_rows"][expert] * groups
        r = np.arange(rows)[:, None]
        g = np.arange(groups)[None, :]
        off = base + (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
        assert (got_sf[off] == want_sf[off]).all(), int(expert)
    # fused epilogue against unfused GEMM + GeGLU kernel on the same operands
    runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU, tokens)
    fused_codes = runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2].clone()
    fused_sf = runner.buffer(rt.BUF_INTER_SF)[: sf_bytes(routes, INTER)].clone()
    runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU | rt.STAGE_UNFUSED, tokens)
    runner.check()
    assert torch.equal(fused_codes, runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2])
    w13_out = runner.buffer(rt.BUF_W13_OUT, torch.bfloat16)[: routes * W13_OUT]
    want_inter, want_inter_sf = oracle.geglu_quantize(bits(w13_out).reshape(routes, W13_OUT), hw["in_scale_q2"], plan)
    assert (fused_codes.cpu().numpy().reshape(routes, -1) == want_inter).all()
    groups = INTER // 16
    got = fused_sf.cpu().numpy()
    for expert in np.unique(ids):
        rows = int((plan["sorted_experts"] == expert).sum())
        base = plan["scale_rows"][expert] * groups
        r = np.arange(rows)[:, None]
        g = np.arange(groups)[None, :]
        off = base + (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
        assert (got[off] == want_inter_sf[off]).all(), int(expert)


def test_distinct_expert_scales_whole_layer(gm, oracle, varied_weights, cuda_device):
    w, hw = varied_weights
    tokens = 24
    x = hashgen.activations(tokens, HIDDEN, 43, "cpu")
    ids = torch.from_numpy(random_ids(tokens, 31)).to(cuda_device)
    rw = torch.tensor([0.24, 0.19, 0.15, 0.12, 0.10, 0.08, 0.07, 0.05], device=cuda_device).repeat(tokens, 1)
    runner = gm.Nvfp4ExpertRunner(w, tokens)
    out = torch.empty((tokens, HIDDEN), dtype=torch.bfloat16, device=cuda_device)
    runner.launch_batch(x.to(cuda_device), ids, rw, out, tokens)
    runner.check()
    want = oracle.moe_layer(bits(x), ids.cpu().numpy(), rw.cpu().numpy(), hw)
    assert rel_l2(bf16_to_f32(bits(out)), bf16_to_f32(want)) < REL_L2


def test_against_committed_golden_vectors(gm, packed, weights, cuda_device):
    """tests/golden/moe_golden.npz: packed weights of all 128 experts (checksums), router,
    and the 16-token layer output."""
    import hashlib
    import os
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "moe_golden.npz"))

    def sha(a):
        return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)

    dev, host = packed
    for key in ("w13", "w13_sf", "w2", "w2_sf"):
        assert (sha(host[key]) == golden["packed_" + key + "_sha"]).all(), key
    assert (host["g13"] == golden["packed_g13"]).all() and (host["g2"] == golden["packed_g2"]).all()
    tokens = 16
    x = hashgen.activations(tokens, HIDDEN, 41, cuda_device)
    logits = from_bits(golden["layer_logits"], cuda_device).view(tokens, EXPERTS)
    rw, ids = gm.route_128_top8(logits, torch.ones(EXPERTS, dtype=torch.bfloat16, device=cuda_device))
    assert (ids.cpu().numpy() == golden["layer_ids"]).all()
    assert (rw.cpu().numpy().view(np.uint32) == golden["layer_route_weights"].view(np.uint32)).all()
    runner = gm.Nvfp4ExpertRunner(weights[0], tokens)
    out = torch.empty_like(x)
    runner.launch_batch(x, ids, rw, out, tokens)
    runner.check()
    assert (runner.inverse_routes().cpu().numpy() == golden["layer_inverse"]).all()
    assert rel_l2(bf16_to_f32(bits(out)), bf16_to_f32(golden["layer_out"])) < REL_L2


@pytest.mark.parametrize("tokens,kind", [(130, "random"), (300, "skewed"), (4096, "random")])
def test_cta_pair_gemms_equal_the_single_cta_gemms(gm, weights, cuda_device, tokens, kind):
    """The two expert GEMMs run by CTA pairs (tcgen05 cta_group::2: two row tiles of an expert
    against shared weight rows, odd last tiles alone in their pair) give the bits of the
    one-CTA-per-tile kernels: w2 operand codes and scales, routed rows, layer output."""
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 5) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, 71, cuda_device)
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
    routes = tokens * TOP_K
    results = []
    for pairs in (False, True):
        runner = gm.Nvfp4ExpertRunner(weights[0], tokens, pairs=pairs)
        out = torch.empty_like(x)
        runner.launch_batch(x, dev_ids, rw, out, tokens)
        runner.check()
        results.append((out, runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2].clone(),
                        runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN].clone()))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert results[0][0].float().abs().max() > 0


@pytest.mark.parametrize("tokens,kind", [(129, "random"), (130, "skewed"), (300, "skewed"), (777, "random"),
                                         (4096, "random")])
def test_weight_major_pair_w13_equals_the_single_cta_w13(gm, weights, cuda_device, tokens, kind):
    """The fused w13 stage run by CTA pairs with the weights on the MMA's M side and up to 256 rows of
    an expert on its N side (any multiple of 16) writes the same w2 operand codes and scale bytes as
    the one-CTA-per-tile kernel, and the layer output follows."""
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 23) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, 79, cuda_device)
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
    routes = tokens * TOP_K
    results = []
    for form in (False, True):
        runner = gm.Nvfp4ExpertRunner(weights[0], tokens, w13_pairs=form)
        out = torch.empty_like(x)
        runner.buffer(rt.BUF_INTER_CODES).zero_()
        runner.buffer(rt.BUF_INTER_SF).zero_()
        for _ in range(2):
            runner.launch_batch(x, dev_ids, rw, out, tokens)
        runner.check()
        results.append((out, runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2].clone(),
                        runner.buffer(rt.BUF_INTER_SF).clone()))
    sf_a, sf_b = results[0][2], results[1][2]
    codes_a, codes_b = results[0][1], results[1][1]
    assert torch.equal(codes_a, codes_b), f"{(codes_a != codes_b).sum().item()} code bytes differ"
    assert torch.equal(sf_a, sf_b), f"{(sf_a != sf_b).sum().item()} scale bytes differ"
    assert torch.equal(results[0][0], results[1][0])
    assert results[0][0].float().abs().max() > 0


@pytest.mark.parametrize("tokens,kind", [(1, "random"), (8, "random"), (40, "skewed"), (64, "random"),
                                         (128, "skewed")])
def test_merged_decode_launch_equals_two_launches(gm, weights, cuda_device, tokens, kind, monkeypatch):
    """Batches of at most 128 tokens run both expert GEMMs in one persistent launch (w2 items wait
    on per-tile readiness counters); the bits must be those of the two separate launches, also when
    the launch is repeated on the same scratch (the counters are reset by the sort)."""
    from gevva_b200 import runtime as rt
    ids = random_ids(tokens, 17) if kind == "random" else skewed_ids(tokens)
    x = hashgen.activations(tokens, HIDDEN, 73, cuda_device)
    dev_ids = torch.from_numpy(ids).to(cuda_device)
    rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
    routes = tokens * TOP_K
    results = []
    for merged in ("0", "1"):
        monkeypatch.setenv("GEVVA_MOE_DECODE_MERGED", merged)
        runner = gm.Nvfp4ExpertRunner(weights[0], max(tokens, 2))
        out = torch.empty_like(x)
        for _ in range(3):
            out.zero_()
            runner.launch_batch(x, dev_ids, rw, out, tokens)
        runner.check()
        results.append((out, runner.buffer(rt.BUF_INTER_CODES)[: routes * INTER // 2].clone(),
                        runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN].clone()))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert results[0][0].float().abs().max() > 0


def test_decode_kernel_that_sorts_and_quantises_itself(gm, weights, cuda_device, monkeypatch):
    """Batches of at most 128 tokens sort their routes and quantise their input inside the merged
    expert launch.  Against a runner that keeps the sort + quantise launch of its own
    (GEVVA_MOE_DECODE_FRONT=0): the same route plan, operand bytes, routed rows and output, over a
    sequence of batch sizes on one runner (the launch puts its counters back itself), and an expert
    id outside [0,128) is reported and its route left out as before."""
    from gevva_b200 import runtime as rt
    sequence = [(64, "random"), (8, "random"), (128, "skewed"), (1, "random"), (40, "skewed"), (64, "random")]
    runners = {}
    for front in ("0", "1"):
        monkeypatch.setenv("GEVVA_MOE_DECODE_FRONT", front)
        runners[front] = gm.Nvfp4ExpertRunner(weights[0], 128)
    plan_buffers = (rt.BUF_SORTED_EXPERTS, rt.BUF_SORTED_ROUTES, rt.BUF_INVERSE_ROUTES, rt.BUF_EXPERT_OFFSETS,
                    rt.BUF_SCALE_ROW_OFFSETS, rt.BUF_NUM_TILES)
    for step, (tokens, kind) in enumerate(sequence):
        ids = random_ids(tokens, 31 + step) if kind == "random" else skewed_ids(tokens)
        x = hashgen.activations(tokens, HIDDEN, 90 + step, cuda_device)
        dev_ids = torch.from_numpy(ids).to(cuda_device)
        rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
        routes = tokens * TOP_K
        seen = []
        for front in ("0", "1"):
            runner = runners[front]
            out = torch.zeros_like(x)
            runner.launch_batch(x, dev_ids, rw, out, tokens)
            runner.check()
            record = [out, runner.buffer(rt.BUF_INPUT_CODES)[: routes * HIDDEN // 2].clone(),
                      runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN].clone()]
            for buffer_id in plan_buffers:
                view = runner.buffer(buffer_id, torch.int32)
                record.append((view[:routes] if buffer_id <= rt.BUF_INVERSE_ROUTES else view).clone())
            tiles = int(runner.buffer(rt.BUF_NUM_TILES, torch.int32)[0])
            record.append(runner.buffer(rt.BUF_TILE_EXPERT, torch.int32)[:tiles].clone())
            seen.append(record)
        for a, b in zip(*seen):
            assert torch.equal(a, b), f"step {step} ({tokens} tokens)"
        assert seen[0][0].float().abs().max() > 0
    # a rejected expert id
    tokens = 16
    ids = random_ids(tokens, 5)
    ids[7, 2] = 128
    x = hashgen.activations(tokens, HIDDEN, 12, cuda_device)
    rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
    outs = []
    for front in ("0", "1"):
        out = torch.zeros_like(x)
        runners[front].launch_stages(rt.STAGE_ALL & ~rt.STAGE_REDUCE, tokens, input=x,
                                     expert_ids=torch.from_numpy(ids).to(cuda_device))
        assert runners[front].last_status() == -1
        assert runners[front].last_status() == 0
        inverse = runners[front].buffer(rt.BUF_INVERSE_ROUTES, torch.int32)[: tokens * TOP_K].clone()
        rows = runners[front].buffer(rt.BUF_W2_OUT, torch.bfloat16)[: tokens * TOP_K * HIDDEN].view(-1, HIDDEN)
        keep = torch.ones(tokens * TOP_K, dtype=torch.bool, device=cuda_device)
        keep[7 * TOP_K + 2] = False
        outs.append(rows[inverse[keep].long()].clone())
    assert torch.equal(outs[0], outs[1])


def test_nvtx_ranges_do_not_change_results(gm, weights, cuda_device):
    """A runner created with the NVTX option marks its stages and computes the same bits; unknown
    option flags are refused."""
    import ctypes
    from gevva_b200 import runtime as rt
    tokens = 200
    x = hashgen.activations(tokens, HIDDEN, 44, cuda_device)
    ids = torch.from_numpy(random_ids(tokens, 9)).to(cuda_device)
    rw = torch.full((tokens, TOP_K), 0.125, device=cuda_device)
    outs = []
    for nvtx in (False, True):
        runner = gm.Nvfp4ExpertRunner(weights[0], tokens, nvtx=nvtx)
        out = torch.empty_like(x)
        runner.launch_batch(x, ids, rw, out, tokens)
        runner.check()
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    w = weights[0]
    packed = rt._Weights(*[t.data_ptr() for t in (w.w13, w.w13_sf, w.w2, w.w2_sf, w.alpha1, w.alpha2,
                                                  w.in_scale_q1, w.in_scale_q2)])
    handle = ctypes.c_void_p()
    bad = rt._Options(0x80)   # an option bit that does not exist
    assert rt.library().gevva_moe_create(ctypes.byref(handle), ctypes.byref(packed), 16, None,
                                         ctypes.byref(bad)) == -3


def test_bounded_wait_times_out_and_context_survives(gm, weights, cuda_device):
    """A wait that nothing satisfies must end by itself with WAIT_TIMEOUT in the status word
    (about a millisecond here) and leave the device usable: the next layer launch is correct."""
    import ctypes
    from gevva_b200 import runtime as rt
    runner = gm.Nvfp4ExpertRunner(weights[0], 16)
    lib = rt.library()
    lib.gevva_moe_probe_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    status = lib.gevva_moe_probe_bounded_wait(runner._handle, 2000000,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == 0
    assert runner.last_status() == -2
    assert runner.last_status() == 0
    x = hashgen.activations(16, HIDDEN, 41, cuda_device)
    ids = torch.from_numpy(random_ids(16, 3)).to(cuda_device)
    rw = torch.full((16, TOP_K), 0.125, device=cuda_device)
    out = torch.empty_like(x)
    runner.launch_batch(x, ids, rw, out, 16)
    runner.check()
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("tokens", [4096, 16384, 20000])
def test_full_size_properties(gm, weights, cuda_device, tokens):
    """4096 and 16384 tokens (the prefill configurations' sizes) and 20000 (more route chunks
    than SMs, so the route sort takes its three-launch form): properties that need no oracle."""
    from gevva_b200 import runtime as rt
    w, _ = weights
    x = hashgen.activations(tokens, HIDDEN, 51, cuda_device)
    router_w = (hashgen.hash_uniform(EXPERTS * HIDDEN, 5, cuda_device) * 0.0346).view(EXPERTS, HIDDEN)
    bias = hashgen.hash_uniform(EXPERTS, 6, cuda_device) * 0.9
    logits = (x.float() @ router_w.t() + bias).to(torch.bfloat16)
    rw, ids = gm.route_128_top8(logits, torch.ones(EXPERTS, dtype=torch.bfloat16, device=cuda_device))
    # top-8 really are the eight largest, in order
    top = torch.gather(logits.float(), 1, ids.long())
    assert (top[:, :-1] >= top[:, 1:]).all()
    kth = torch.topk(logits.float(), TOP_K, dim=1).values[:, -1]
    assert (top[:, -1] == kth).all()
    assert torch.allclose(rw.sum(1), torch.ones(tokens, device=cuda_device), atol=1e-5)
    runner = gm.Nvfp4ExpertRunner(w, tokens)
    out = torch.empty_like(x)
    runner.launch_batch(x, ids, rw, out, tokens)
    runner.check()
    routes = tokens * TOP_K
    se = runner.buffer(rt.BUF_SORTED_EXPERTS, torch.int32)[:routes]
    sr = runner.buffer(rt.BUF_SORTED_ROUTES, torch.int32)[:routes].long()
    inv = runner.inverse_routes().long()
    assert (se[1:] >= se[:-1]).all()                                   # sortedness
    assert (inv[sr] == torch.arange(routes, device=cuda_device)).all()  # inverse permutation
    assert (ids.reshape(-1)[sr] == se).all()
    same = se[1:] == se[:-1]
    assert (sr[1:][same] > sr[:-1][same]).all()                        # stability
    assert torch.isfinite(out.float()).all() and out.float().abs().max() > 0
    # run-to-run repeatability (the reference's own hot-path test, src/nvfp4_cutlass.cu:1940-2052)
    out2 = torch.empty_like(x)
    runner.launch_batch(x, ids, rw, out2, tokens)
    assert torch.equal(out, out2)
    # batch invariance: a token's result does not depend on what else is in the batch
    # The sort is stable, so the first tokens of a batch are the first rows of every expert (row
    # tile 0): the last tokens and a random draw are the ones that land in the higher tiles.
    picks = torch.cat([torch.arange(tokens - 16, tokens),
                       torch.randperm(tokens, generator=torch.Generator().manual_seed(tokens))[:64]])
    picks = picks.to(cuda_device)
    small = gm.Nvfp4ExpertRunner(w, picks.numel())
    out3 = torch.empty((picks.numel(), HIDDEN), dtype=torch.bfloat16, device=cuda_device)
    small.launch_batch(x[picks].contiguous(), ids[picks].contiguous(), rw[picks].contiguous(), out3,
                       picks.numel())
    small.check()
    assert torch.equal(out3, out[picks])
