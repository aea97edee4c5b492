"""Properties of the CPU oracle's stages, including the edge cases the path has:
a single token, every route on one expert (129 rows: two 128-row scale blocks),
ties and signed zeros in the router, out-of-range expert ids."""
import numpy as np
import pytest

from tests.oracle_api import EXPERTS, HIDDEN, INTER, TOP_K, bf16_to_f32, sf_bytes

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def f32_to_bf16_bits(x):
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def e4m3_table(oracle):
    return np.array([oracle.lib.gvo_decode_e4m3(c) for c in range(256)], np.float32)


def dequant(oracle, packed, scales_region, rows, width):
    """codes [rows, width/2] + swizzled scale region -> fp32 [rows, width]."""
    groups = width // 16
    lo, hi = packed & 15, packed >> 4
    vals = np.empty((rows, width), np.float32)
    vals[:, 0::2] = E2M1[lo]
    vals[:, 1::2] = E2M1[hi]
    tab = e4m3_table(oracle)
    r = np.arange(rows)[:, None]
    g = np.arange(groups)[None, :]
    off = (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
    sf = tab[scales_region[off]]
    return vals * np.repeat(sf, 16, axis=1)


def test_router_permutation_logits(oracle):
    # 64 rows of a row-dependent permutation of bf16-separated values, every expert id
    # exercised, no ties (the shape of the reference's routing self-test inputs,
    # src/cuda/diagnostics/primitives_layers.cuh:13-22)
    rows = 64
    rank = (np.arange(EXPERTS)[None, :] * 37 + np.arange(rows)[:, None] * 19) & 127
    logits = ((rank - 64) * 0.0625).astype(np.float32)
    scale = (0.5 + (np.arange(EXPERTS) % 17) * 0.07).astype(np.float32)
    w, ids = oracle.route(f32_to_bf16_bits(logits), f32_to_bf16_bits(scale))
    order = np.argsort(-logits, axis=1, kind="stable")[:, :TOP_K]
    assert (ids == order).all()
    top = np.take_along_axis(logits, order, 1).astype(np.float64)
    p = np.exp(top - top[:, :1])
    p /= p.sum(1, keepdims=True)
    want = p * bf16_to_f32(f32_to_bf16_bits(scale))[order]
    assert np.abs(w - want).max() < 1e-6


def test_router_ties_and_signed_zero(oracle):
    logits = np.zeros((3, EXPERTS), np.float32)
    logits[1, ::2] = -0.0              # -0 ties with +0: lower id first
    logits[2, :] = 1.0
    logits[2, 100] = 2.0
    _, ids = oracle.route(f32_to_bf16_bits(logits), f32_to_bf16_bits(np.ones(EXPERTS, np.float32)))
    assert (ids[0] == np.arange(8)).all()
    assert (ids[1] == np.arange(8)).all()
    assert (ids[2] == np.array([100, 0, 1, 2, 3, 4, 5, 6])).all()


def test_router_fp8_rescale_path(oracle):
    rng = np.random.default_rng(1)
    logits = rng.normal(0, 1, (5, EXPERTS)).astype(np.float32)
    act = rng.uniform(0.5, 2, 5).astype(np.float32)
    ws = np.array([0.37], np.float32)
    bits = f32_to_bf16_bits(logits)
    w, ids = oracle.route(bits, f32_to_bf16_bits(np.ones(EXPERTS, np.float32)), act, ws)
    scaled = bf16_to_f32(f32_to_bf16_bits(bf16_to_f32(bits) * (act * ws[0])[:, None]))
    assert (ids == np.argsort(-scaled, axis=1, kind="stable")[:, :TOP_K]).all()
    assert np.allclose(w.sum(1), 1, atol=1e-6)


@pytest.mark.parametrize("tokens", [1, 2, 7, 16, 129, 1000])
def test_sort_is_a_stable_counting_sort(oracle, tokens):
    rng = np.random.default_rng(tokens)
    ids = np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int32)
    plan = oracle.sort(ids)
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    assert plan["status"] == 0
    assert (plan["sorted_routes"] == order).all()
    assert (plan["sorted_experts"] == flat[order]).all()
    assert (plan["inverse"][order] == np.arange(flat.size)).all()
    counts = np.bincount(flat, minlength=EXPERTS)
    assert (plan["offsets"] == np.concatenate([[0], np.cumsum(counts)[:-1]])).all()
    padded = (counts + 127) // 128 * 128
    assert (plan["scale_rows"] == np.concatenate([[0], np.cumsum(padded)[:-1]])).all()


def test_sort_rejects_bad_ids(oracle):
    ids = np.arange(8, dtype=np.int32)[None, :].copy()
    ids[0, 3] = 128
    assert oracle.sort(ids)["status"] == -1
    ids[0, 3] = -1
    assert oracle.sort(ids)["status"] == -1


def test_quantize_roundtrip_error_and_layout(oracle):
    rng = np.random.default_rng(3)
    tokens = 17
    x = f32_to_bf16_bits(rng.normal(0, 1, (tokens, HIDDEN)).astype(np.float32))
    # 129 routes on expert 5 -> second 128-row scale block; the rest spread out
    ids = np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int32)
    ids[:, 0] = 5
    plan = oracle.sort(ids)
    xf = bf16_to_f32(x)
    s1 = np.abs(xf).max() / (6 * 448)
    q = np.full(EXPERTS, 1 / s1, np.float32)
    packed, scales = oracle.quantize_sorted(x, q, plan)
    assert scales.size == sf_bytes(tokens * TOP_K, HIDDEN)
    for expert in (5, int(ids[3, 1])):
        begin = plan["offsets"][expert]
        rows = int((plan["sorted_experts"] == expert).sum())
        region = scales[plan["scale_rows"][expert] * (HIDDEN // 16):]
        deq = dequant(oracle, packed[begin:begin + rows], region, rows, HIDDEN) * s1
        src = xf[plan["sorted_routes"][begin:begin + rows] // TOP_K]
        blocks = np.abs(src).reshape(rows, -1, 16).max(2)
        # E2M1 step is at most 2 (between 4 and 6) of 6, the E4M3 scale adds 1/16 relative
        err = np.abs(deq - src).reshape(rows, -1, 16).max(2)
        assert (err <= blocks * (1.0 / 6 + 1.0 / 8) + 1e-6).all()


def test_zero_block_quantises_to_zero(oracle):
    x = np.zeros((1, HIDDEN), np.uint16)
    ids = np.arange(8, dtype=np.int32)[None, :]
    plan = oracle.sort(ids)
    packed, scales = oracle.quantize_sorted(x, np.ones(EXPERTS, np.float32), plan)
    assert not packed.any() and not scales.any()


def test_grouped_gemm_matches_float64(oracle):
    rng = np.random.default_rng(4)
    tokens = 3
    ids = np.array([[0, 1, 2, 3, 4, 5, 6, 7], [0, 9, 2, 11, 4, 13, 6, 15], [0, 1, 2, 3, 20, 21, 22, 23]],
                   np.int32)
    plan = oracle.sort(ids)
    x = f32_to_bf16_bits(rng.normal(0, 1, (tokens, INTER)).astype(np.float32))
    q = np.full(EXPERTS, 448 * 6 / 4.0, np.float32)
    packed, scales = oracle.quantize_sorted(x, q, plan)  # width 704 works for any multiple of 64
    n_out = 128
    w = np.zeros((EXPERTS, n_out, INTER // 2), np.uint8)
    wsf = np.zeros((EXPERTS, n_out, INTER // 16), np.uint8)
    dense = {}
    for expert in np.unique(ids):
        wf = rng.normal(0, 0.02, (n_out, INTER)).astype(np.float32)
        c, s, g = oracle.pack_weight(wf)
        w[expert], wsf[expert] = c, s
        dense[int(expert)] = dequant(oracle, c, s.reshape(-1), n_out, INTER).astype(np.float64)
    alpha = np.zeros(EXPERTS, np.float32)
    scale_of = {}
    for expert in np.unique(ids):
        scale_of[int(expert)] = rng.uniform(0.5, 2.0)
        alpha[expert] = scale_of[int(expert)]
    out = bf16_to_f32(oracle.grouped_gemm(packed, scales, plan, w, wsf, alpha, n_out, INTER))
    for expert in np.unique(ids):
        begin = plan["offsets"][expert]
        rows = int((plan["sorted_experts"] == expert).sum())
        region = scales[plan["scale_rows"][expert] * (INTER // 16):]
        a = dequant(oracle, packed[begin:begin + rows], region, rows, INTER).astype(np.float64)
        want = np.float64(alpha[expert]) * (a @ dense[int(expert)].T)
        got = out[begin:begin + rows].astype(np.float64)
        assert np.abs(got - want).max() <= 0.006 * np.abs(want).max() + 1e-12  # bf16 rounding


def test_reduce_is_fma_in_route_order(oracle):
    rng = np.random.default_rng(5)
    tokens = 4
    routed = f32_to_bf16_bits(rng.normal(0, 1, (tokens * TOP_K, HIDDEN)).astype(np.float32))
    w = rng.uniform(0, 0.3, (tokens, TOP_K)).astype(np.float32)
    inverse = rng.permutation(tokens * TOP_K).astype(np.int32)
    out = oracle.reduce(routed, w, inverse, tokens)
    rf = bf16_to_f32(routed).astype(np.float64)
    want = np.zeros((tokens, HIDDEN))
    for t in range(tokens):
        for k in range(TOP_K):
            want[t] += rf[inverse[t * TOP_K + k]] * np.float64(w[t, k])
    assert np.abs(bf16_to_f32(out) - want).max() < 0.02
