"""Parity with the CPU oracle at the benchmark's own sizes and routing distributions.

Two batches, built exactly as bench.py builds them (gevva_b200.synthetic.SyntheticLayer):
  * the prefill configuration: 4096 tokens, per-expert router bias ~N(0, 0.5); every stage of
    the whole batch goes through the oracle;
  * the expert-parallel configuration's batch: 16384 tokens, Zipf(1.1) router bias, 128
    distinct static scales; ids and the route sort of the whole batch go through the oracle,
    the arithmetic stages go through it for the last 2048 tokens, whose routes are the last
    rows of every expert (the stable sort keeps token order), i.e. the highest row tiles.
Bit-exact: ids, router weights, permutation arrays, FP4 codes, E4M3 scale bytes, weighted
reduce.  GEMM outputs and the layer output: relative L2 <= 2e-2, checked per expert and per
128-row tile so that one wrong tile cannot hide in the norm of the batch (the reference's own
full-size test uses skewed routing for the same reason, src/nvfp4_cutlass.cu:1940-2052)."""
import numpy as np
import pytest
import torch

from tests.parity_util import (EXPERTS, HIDDEN, INTER, TOP_K, bf16_to_f32, bits, gather_sf, rel_l2,
                               scatter_sf, worst_tile)

pytestmark = pytest.mark.gpu

W13_OUT = 2 * INTER
REL_L2 = 2e-2


def host_weights(w):
    return {name: getattr(w, name).cpu().numpy() for name in
            ("w13", "w13_sf", "w2", "w2_sf", "alpha1", "alpha2", "in_scale_q1", "in_scale_q2")}


@pytest.fixture(scope="module")
def prefill_layer(cuda_device):
    """bench.py's layer: seed 0, bias ~N(0, 0.5), scales calibrated on the seed-1000 batch."""
    from gevva_b200.synthetic import SyntheticLayer
    layer = SyntheticLayer(seed=0, max_tokens=4096, device=cuda_device, bias_std=0.5)
    layer.calibrate(layer.inputs(4096, seed=1000))
    return layer


def row_geometry(plan, routes):
    expert_of_row = plan["sorted_experts"][:routes]
    row_in_expert = np.arange(routes) - plan["offsets"][expert_of_row]
    return expert_of_row, row_in_expert


def test_prefill_batch_every_stage(prefill_layer, oracle, cuda_device):
    import gevva_b200 as gm
    from gevva_b200 import runtime as rt
    layer = prefill_layer
    tokens, routes = 4096, 4096 * TOP_K
    hw = host_weights(layer.weights)
    x = layer.inputs(tokens, seed=1000)
    logits = layer.logits(x)
    rw, ids = gm.route_128_top8(logits, layer.expert_scale)
    ow, oids = oracle.route(bits(logits), bits(layer.expert_scale))
    assert (ids.cpu().numpy() == oids).all()
    assert (rw.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()

    runner = layer.runner
    runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, tokens, input=x, expert_ids=ids)
    assert runner.last_status() == 0
    plan = oracle.sort(oids)
    i32 = torch.int32
    for key, buffer_id, count in (("sorted_experts", rt.BUF_SORTED_EXPERTS, routes),
                                  ("sorted_routes", rt.BUF_SORTED_ROUTES, routes),
                                  ("inverse", rt.BUF_INVERSE_ROUTES, routes),
                                  ("offsets", rt.BUF_EXPERT_OFFSETS, EXPERTS),
                                  ("scale_rows", rt.BUF_SCALE_ROW_OFFSETS, EXPERTS)):
        assert (runner.buffer(buffer_id, i32)[:count].cpu().numpy() == plan[key]).all(), key
    counts = np.bincount(oids.reshape(-1), minlength=EXPERTS)
    assert counts.max() > 3 * 128, "the biased router must give some expert several row tiles"
    expert_of_row, row_in_expert = row_geometry(plan, routes)
    tile_of_row = row_in_expert // 128

    want_codes, want_sf = oracle.quantize_sorted(bits(x), hw["in_scale_q1"], plan)
    got_codes = runner.buffer(rt.BUF_INPUT_CODES)[: routes * HIDDEN // 2].cpu().numpy().reshape(routes, -1)
    assert (got_codes == want_codes).all()
    got_sf = runner.buffer(rt.BUF_INPUT_SF).cpu().numpy()
    assert (gather_sf(got_sf, expert_of_row, row_in_expert, plan["scale_rows"], HIDDEN // 16) ==
            gather_sf(want_sf, expert_of_row, row_in_expert, plan["scale_rows"], HIDDEN // 16)).all()

    # w13 as a bf16 GEMM, the same operand bytes on both sides
    runner.launch_stages(rt.STAGE_W13, tokens)
    assert runner.last_status() == 0
    got13 = bits(runner.buffer(rt.BUF_W13_OUT, torch.bfloat16)[: routes * W13_OUT]).reshape(routes, W13_OUT)
    want13 = oracle.grouped_gemm(want_codes, want_sf, plan, hw["w13"], hw["w13_sf"], hw["alpha1"], W13_OUT, HIDDEN)
    err, expert, tile, groups, top = worst_tile(bf16_to_f32(got13), bf16_to_f32(want13), expert_of_row, tile_of_row)
    print(f"w13: worst (expert {expert}, tile {tile}) rel-L2 {err:.2e} over {groups} tiles, highest tile {top}")
    assert err < REL_L2 and top >= 3

    # production form: GeGLU + requantise in the w13 epilogue; the oracle's GeGLU quantiser fed the
    # GPU's own bf16 GEMM output must give the same bytes
    inter_codes = runner.buffer(rt.BUF_INTER_CODES)
    inter_sf = runner.buffer(rt.BUF_INTER_SF)
    inter_codes.zero_()
    inter_sf.zero_()
    runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU, tokens)
    assert runner.last_status() == 0
    want_inter, want_inter_sf = oracle.geglu_quantize(got13, hw["in_scale_q2"], plan)
    got_inter = inter_codes[: routes * INTER // 2].cpu().numpy().reshape(routes, -1)
    assert (got_inter == want_inter).all()
    got_inter_sf = inter_sf.cpu().numpy()
    assert (gather_sf(got_inter_sf, expert_of_row, row_in_expert, plan["scale_rows"], INTER // 16) ==
            gather_sf(want_inter_sf, expert_of_row, row_in_expert, plan["scale_rows"], INTER // 16)).all()

    runner.launch_stages(rt.STAGE_W2, tokens)
    assert runner.last_status() == 0
    got2 = bits(runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN]).reshape(routes, HIDDEN)
    want2 = oracle.grouped_gemm(want_inter, want_inter_sf, plan, hw["w2"], hw["w2_sf"], hw["alpha2"], HIDDEN, INTER)
    err, expert, tile, groups, top = worst_tile(bf16_to_f32(got2), bf16_to_f32(want2), expert_of_row, tile_of_row)
    print(f"w2: worst (expert {expert}, tile {tile}) rel-L2 {err:.2e} over {groups} tiles")
    assert err < REL_L2

    out = torch.empty_like(x)
    runner.launch_stages(rt.STAGE_REDUCE, tokens, route_weights=rw, output=out)
    assert runner.last_status() == 0
    assert (bits(out) == oracle.reduce(got2, ow, plan["inverse"], tokens)).all()

    # the whole layer in one call against the oracle's whole layer
    out.zero_()
    runner.launch_batch(x, ids, rw, out, tokens)
    runner.check()
    want = oracle.moe_layer(bits(x), oids, ow, hw)
    got_f, want_f = bf16_to_f32(bits(out)), bf16_to_f32(want)
    assert rel_l2(got_f, want_f) < REL_L2
    blocks = [rel_l2(got_f[i:i + 128], want_f[i:i + 128]) for i in range(0, tokens, 128)]
    print(f"layer: rel-L2 {rel_l2(got_f, want_f):.2e}, worst 128-token block {max(blocks):.2e}")
    assert max(blocks) < REL_L2


def test_zipf_batch_last_rows_of_every_expert(prefill_layer, oracle, cuda_device):
    import gevva_b200 as gm
    from gevva_b200 import runtime as rt
    from gevva_b200.synthetic import SyntheticLayer
    tokens, routes = 16384, 16384 * TOP_K
    first, count = tokens - 2048, 2048
    layer = SyntheticLayer(seed=0, max_tokens=16, device=cuda_device, zipf=True, packed=prefill_layer.packed)
    # 128 distinct static scales around the calibrated ones
    p = layer.packed
    index = torch.arange(EXPERTS, dtype=torch.float32, device=cuda_device)
    f1 = 1.0 + (index % 7) * 0.03125
    f2 = 1.0 + (index % 5) * 0.0625
    s1, s2 = prefill_layer.s1, prefill_layer.s2
    w = gm.ExpertWeights(p["w13"], p["w13_sf"], p["w2"], p["w2_sf"],
                         (p["g13"] * s1 * f1).contiguous(), (p["g2"] * s2 * f2).contiguous(),
                         (1.0 / (s1 * f1)).contiguous(), (1.0 / (s2 * f2)).contiguous())
    hw = host_weights(w)
    x = layer.inputs(tokens, seed=3000)
    logits = layer.logits(x)
    rw, ids = gm.route_128_top8(logits, layer.expert_scale)
    ow, oids = oracle.route(bits(logits), bits(layer.expert_scale))
    assert (ids.cpu().numpy() == oids).all()
    assert (rw.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()
    loads = np.bincount(oids.reshape(-1), minlength=EXPERTS)
    print(f"zipf loads: max {loads.max()}, min {loads.min()}, experts with <= 32 rows {(loads <= 32).sum()}")

    runner = gm.Nvfp4ExpertRunner(w, tokens)
    runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE | rt.STAGE_W13, tokens, input=x, expert_ids=ids)
    assert runner.last_status() == 0
    plan = oracle.sort(oids)
    i32 = torch.int32
    for key, buffer_id, n in (("sorted_experts", rt.BUF_SORTED_EXPERTS, routes),
                              ("sorted_routes", rt.BUF_SORTED_ROUTES, routes),
                              ("inverse", rt.BUF_INVERSE_ROUTES, routes),
                              ("offsets", rt.BUF_EXPERT_OFFSETS, EXPERTS),
                              ("scale_rows", rt.BUF_SCALE_ROW_OFFSETS, EXPERTS)):
        assert (runner.buffer(buffer_id, i32)[:n].cpu().numpy() == plan[key]).all(), key

    # ---- the slice: its own (small) oracle plan, and where its rows sit in the full batch
    sids = oids[first:]
    splan = oracle.sort(sids)
    sroutes = count * TOP_K
    s_expert, s_row = row_geometry(splan, sroutes)
    full_row = plan["inverse"][first * TOP_K + splan["sorted_routes"]]   # full sorted row of slice row j
    assert (plan["sorted_experts"][full_row] == s_expert).all()
    f_row_in_expert = full_row - plan["offsets"][s_expert]
    tile_of_row = f_row_in_expert // 128
    assert tile_of_row.max() >= 8, "the slice must reach high row tiles"
    gather = torch.from_numpy(full_row.astype(np.int64)).to(cuda_device)

    xs = bits(x[first:])
    want_codes, want_sf = oracle.quantize_sorted(xs, hw["in_scale_q1"], splan)
    got_codes = runner.buffer(rt.BUF_INPUT_CODES)[: routes * HIDDEN // 2].view(routes, -1)[gather].cpu().numpy()
    assert (got_codes == want_codes).all()
    got_sf = runner.buffer(rt.BUF_INPUT_SF).cpu().numpy()
    assert (gather_sf(got_sf, s_expert, f_row_in_expert, plan["scale_rows"], HIDDEN // 16) ==
            gather_sf(want_sf, s_expert, s_row, splan["scale_rows"], HIDDEN // 16)).all()

    got13 = bits(runner.buffer(rt.BUF_W13_OUT, torch.bfloat16)[: routes * W13_OUT].view(routes, W13_OUT)[gather])
    want13 = oracle.grouped_gemm(want_codes, want_sf, splan, hw["w13"], hw["w13_sf"], hw["alpha1"], W13_OUT, HIDDEN)
    err, expert, tile, groups, top = worst_tile(bf16_to_f32(got13), bf16_to_f32(want13), s_expert, tile_of_row)
    print(f"w13: worst (expert {expert}, tile {tile}) rel-L2 {err:.2e} over {groups} tiles, highest tile {top}")
    assert err < REL_L2

    inter_codes = runner.buffer(rt.BUF_INTER_CODES)
    inter_sf = runner.buffer(rt.BUF_INTER_SF)
    inter_codes.zero_()
    inter_sf.zero_()
    runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU | rt.STAGE_W2, tokens)   # fused epilogue, then w2
    assert runner.last_status() == 0
    want_inter, want_inter_sf = oracle.geglu_quantize(got13, hw["in_scale_q2"], splan)
    got_inter = inter_codes[: routes * INTER // 2].view(routes, -1)[gather].cpu().numpy()
    assert (got_inter == want_inter).all()
    got_inter_sf = gather_sf(inter_sf.cpu().numpy(), s_expert, f_row_in_expert, plan["scale_rows"], INTER // 16)
    assert (got_inter_sf == gather_sf(want_inter_sf, s_expert, s_row, splan["scale_rows"], INTER // 16)).all()

    got2 = bits(runner.buffer(rt.BUF_W2_OUT, torch.bfloat16)[: routes * HIDDEN].view(routes, HIDDEN)[gather])
    want2 = oracle.grouped_gemm(want_inter, want_inter_sf, splan, hw["w2"], hw["w2_sf"], hw["alpha2"], HIDDEN, INTER)
    err, expert, tile, groups, top = worst_tile(bf16_to_f32(got2), bf16_to_f32(want2), s_expert, tile_of_row)
    print(f"w2: worst (expert {expert}, tile {tile}) rel-L2 {err:.2e} over {groups} tiles")
    assert err < REL_L2

    out = torch.empty_like(x)
    runner.launch_batch(x, ids, rw, out, tokens)
    runner.check()
    want = oracle.moe_layer(xs, sids, ow[first:], hw)
    got_f, want_f = bf16_to_f32(bits(out[first:])), bf16_to_f32(want)
    blocks = [rel_l2(got_f[i:i + 128], want_f[i:i + 128]) for i in range(0, count, 128)]
    print(f"layer (last {count} tokens): rel-L2 {rel_l2(got_f, want_f):.2e}, worst 128-token block {max(blocks):.2e}")
    assert rel_l2(got_f, want_f) < REL_L2 and max(blocks) < REL_L2
