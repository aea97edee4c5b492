"""Pins the CPU oracle's arithmetic to the conversions the reference kernels call
(toolkit host paths) and to the reference's own decode helpers."""
import math

import numpy as np
import pytest


def _probe_values():
    rng = np.random.default_rng(0)
    hi = np.arange(65536, dtype=np.uint32) << 16
    vals = np.concatenate([hi, hi | 0x8000, hi | 0x7FFF, hi | 0x8001,
                           hi | rng.integers(0, 65536, 65536).astype(np.uint32)]).view(np.float32)
    edge = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5, 6, 6.5, 7, 0.0, 0.1, 448, 449, 464, 480,
                     500, 1e-5, 2 ** -9, 2 ** -10, 1.5 * 2 ** -10, 2 ** -6, 2 ** -7 * 1.0625],
                    dtype=np.float32)
    return np.concatenate([vals, edge, -edge])


def test_e4m3_encoder_matches_toolkit(oracle):
    vals = _probe_values()
    for v in vals[:: 7]:
        assert oracle.lib.gvo_encode_e4m3(float(v)) == oracle.pin.pin_encode_e4m3(float(v)), v


def test_e2m1_encoder_matches_toolkit(oracle):
    vals = _probe_values()
    for v in vals[:: 7]:
        mine = oracle.lib.gvo_encode_e2m1(float(v))
        assert mine == (oracle.pin.pin_encode_e2m1x2(float(v), 0.0) & 15), v
        assert (mine << 4) == (oracle.pin.pin_encode_e2m1x2(0.0, float(v)) & 0xF0), v


def test_known_answer_rounding_and_saturation_points(oracle):
    # round-to-nearest-even and saturation points of E2M1 / E4M3
    table = {0.25: 0x0, 0.75: 0x2, 1.25: 0x2, 1.75: 0x4, 2.5: 0x4, 3.5: 0x6, 5.0: 0x6, 7.0: 0x7,
             -6.5: 0xF}
    for value, code in table.items():
        assert oracle.lib.gvo_encode_e2m1(value) == code
    assert oracle.lib.gvo_encode_e4m3(500.0) == 0x7E
    assert oracle.lib.gvo_encode_e4m3(1e-5) == 0x00


def test_bf16_rounding_matches_toolkit(oracle):
    vals = _probe_values()
    for v in vals[:: 11]:
        if np.isnan(v):
            continue
        assert oracle.lib.gvo_float_to_bf16(float(v)) == oracle.pin.pin_float_to_bf16(float(v)), v


def test_decoders_match_toolkit_and_reference(oracle):
    for code in range(256):
        mine = oracle.lib.gvo_decode_e4m3(code)
        tk = oracle.pin.pin_decode_e4m3(code)
        assert (math.isnan(mine) and math.isnan(tk)) or mine == tk
    if oracle.ref is None:
        pytest.skip("oracle/_ref/libgv_ref_decode.so not built (reference tree absent)")
    for code in range(256):
        mine = oracle.lib.gvo_decode_e4m3(code)
        ref = oracle.ref.ref_decode_e4m3(code)
        assert (math.isnan(mine) and math.isnan(ref)) or mine == ref
    for code in range(16):
        assert oracle.lib.gvo_decode_e2m1(code) == oracle.ref.ref_decode_e2m1(code)


def test_e2m1_roundtrip(oracle):
    for code in range(16):
        value = oracle.lib.gvo_decode_e2m1(code)
        assert oracle.lib.gvo_encode_e2m1(value) == code


def test_sf_offset_is_the_reference_formula_and_a_bijection(oracle):
    for groups in (176, 44):
        rows = 256
        seen = set()
        for row in range(rows):
            for group in range(groups):
                off = oracle.lib.gvo_sf_offset(row, group, groups)
                # src/nvfp4_cutlass.cu:321-323 written out
                want = (row // 128) * (128 * groups) + (group // 4) * 512 + (row % 32) * 16 + \
                    ((row // 32) % 4) * 4 + group % 4
                assert off == want
                seen.add(off)
        assert seen == set(range(rows * groups))


def test_erf_and_exp_accuracy(oracle):
    xs = np.concatenate([np.linspace(-6, 6, 20001), [0.0, -0.0, 1.0, 2.0, 3.0, 4.0, 1e-8, -1e-8]])
    worst = max(abs(oracle.lib.gvo_erff(float(np.float32(x))) - math.erf(float(np.float32(x))))
                for x in xs)
    assert worst < 1.5e-7
    assert oracle.lib.gvo_erff(float("inf")) == 1.0 and oracle.lib.gvo_erff(float("-inf")) == -1.0
    for x in np.linspace(-87, 0, 5001):
        x = float(np.float32(x))
        assert abs(oracle.lib.gvo_expf(x) / math.exp(x) - 1) < 3e-7
    assert oracle.lib.gvo_expf(0.0) == 1.0
    assert oracle.lib.gvo_expf(-100.0) == 0.0


def test_gelu_matches_definition(oracle):
    for x in np.linspace(-8, 8, 4001):
        x = float(np.float32(x))
        want = 0.5 * x * (1 + math.erf(x / math.sqrt(2)))
        assert abs(oracle.lib.gvo_gelu(x) - want) < 2e-6 * max(1.0, abs(x))
