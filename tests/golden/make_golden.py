"""Generates tests/golden/moe_golden.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference ships no golden vectors for the MoE path (its self-tests need an SM120
GPU and the real checkpoint), so these vectors are outputs of the pinned CPU oracle on
device-independent synthetic inputs (tests/hashgen.py).  They serve two purposes: the
CPU suite checks that the oracle still reproduces them (a change of compiler, flags or
code that moves a single bit is caught), and the GPU suite compares the CUDA path with
them without running the oracle for the large case.
"""
import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests import hashgen  # noqa: E402
from tests.oracle_api import EXPERTS, HIDDEN, INTER, TOP_K, Oracle  # noqa: E402

W13_OUT = 2 * INTER
S1 = np.float32(4.0 / (6.0 * 448.0))
S2 = np.float32(16.0 / (6.0 * 448.0))


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(array):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(array).tobytes()).digest(), np.uint8)


def skewed_ids(tokens):
    t = np.arange(tokens, dtype=np.uint64)[:, None]
    k = np.arange(TOP_K, dtype=np.uint64)[None, :]
    mixed = (t * 2654435761 + k * 2246822519) & 0xFFFFFFFF
    ids = (1 + ((mixed >> 24) + k * k) % 36).astype(np.int32)
    ids[:, 0] = 0
    for row in ids:
        seen = set()
        for j in range(TOP_K):
            while int(row[j]) in seen:
                row[j] = 1 + (row[j] + 7) % 36
            seen.add(int(row[j]))
    return ids


def packed_layer(oracle):
    """All 128 hash-generated experts packed by the oracle (the GPU suite's `packed`
    fixture makes the same bytes with the CUDA packer)."""
    out = {k: [] for k in ("w13", "w13_sf", "g13", "w2", "w2_sf", "g2")}
    for expert in range(EXPERTS):
        w13 = hashgen.expert_weights_chunk(expert, 1, W13_OUT, HIDDEN, 11)[0].numpy()
        c, s, g = oracle.pack_weight(w13)
        out["w13"].append(c), out["w13_sf"].append(s), out["g13"].append(g)
        w2 = hashgen.expert_weights_chunk(expert, 1, HIDDEN, INTER, 12)[0].numpy()
        c, s, g = oracle.pack_weight(w2)
        out["w2"].append(c), out["w2_sf"].append(s), out["g2"].append(g)
    return {k: np.stack(v) if v[0].ndim else np.array(v, np.float32) for k, v in out.items()}


def layer_case(oracle, packed, tokens=16):
    x = hashgen.activations(tokens, HIDDEN, 41)
    router_w = (hashgen.hash_uniform(EXPERTS * HIDDEN, 5) * 0.0346).view(EXPERTS, HIDDEN)
    logits = (x.float() @ router_w.t()).to(torch.bfloat16)
    scale = torch.ones(EXPERTS, dtype=torch.bfloat16)
    rw, ids = oracle.route(bits(logits), bits(scale))
    weights = dict(w13=packed["w13"], w13_sf=packed["w13_sf"], w2=packed["w2"], w2_sf=packed["w2_sf"],
                   alpha1=packed["g13"] * S1, alpha2=packed["g2"] * S2,
                   in_scale_q1=np.full(EXPERTS, np.float32(1) / S1, np.float32),
                   in_scale_q2=np.full(EXPERTS, np.float32(1) / S2, np.float32))
    out, routed, inverse = oracle.moe_layer(bits(x), ids, rw, weights, want_routed=True)
    return dict(layer_logits=bits(logits), layer_ids=ids, layer_route_weights=rw, layer_out=out,
                layer_routed_sha=sha(routed), layer_inverse=inverse)


def main():
    oracle = Oracle()
    g = {}
    # router: 64 rows of a row-dependent permutation of bf16-separated logits
    rows = 64
    rank = (np.arange(EXPERTS)[None, :] * 37 + np.arange(rows)[:, None] * 19) & 127
    logits = torch.tensor((rank - 64) * 0.0625, dtype=torch.float32).to(torch.bfloat16)
    scale = torch.tensor(0.5 + (np.arange(EXPERTS) % 17) * 0.07, dtype=torch.float32).to(torch.bfloat16)
    g["router_weights"], g["router_ids"] = oracle.route(bits(logits), bits(scale))
    # route sort: 300 tokens of skewed routing
    plan = oracle.sort(skewed_ids(300))
    for key in ("sorted_experts", "sorted_routes", "inverse", "offsets", "scale_rows"):
        g["sort_" + key] = plan[key]
    # quantisers on a ragged case: 37 tokens, expert 0 takes a row from every token
    ids = skewed_ids(37)
    plan = oracle.sort(ids)
    x = hashgen.activations(37, HIDDEN, 3)
    q1 = np.full(EXPERTS, np.float32(1) / S1, np.float32)
    codes, sf = oracle.quantize_sorted(bits(x), q1, plan)
    g["quant_codes_sha"], g["quant_sf_sha"] = sha(codes), sha(sf)
    g["quant_codes_row0"], g["quant_sf_head"] = codes[0], sf[:512]
    fused = hashgen.activations(37 * TOP_K, W13_OUT, 9, scale=0.9)
    q2 = np.full(EXPERTS, np.float32(1) / S2, np.float32)
    codes2, sf2 = oracle.geglu_quantize(bits(fused), q2, plan)
    g["geglu_codes_sha"], g["geglu_sf_sha"] = sha(codes2), sha(sf2)
    g["geglu_codes_row0"] = codes2[0]
    # whole layer, the 16-token configuration
    packed = packed_layer(oracle)
    for key in ("w13", "w13_sf", "w2", "w2_sf"):
        g["packed_" + key + "_sha"] = sha(packed[key])
    g["packed_g13"], g["packed_g2"] = packed["g13"], packed["g2"]
    g.update(layer_case(oracle, packed))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_golden.npz")
    np.savez_compressed(path, **g)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
