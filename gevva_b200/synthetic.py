"""Seeded synthetic stand-ins for the Gemma-4 26B-A4B expert sidecar and inputs.

The real checkpoint (nvidia/Gemma-4-26B-A4B-NVFP4) is not available offline, so
weights and activations are drawn with the shapes and value distributions the
benchmark configurations name: expert weights ~N(0, 0.02) quantised to NVFP4 with
a per-expert global scale amax/(6*448) and E4M3 block scales, router weights
~N(0, 0.02), activations ~N(0, 1) in bf16.  Tensor shapes and layouts are the
sidecar's (src/runtime.cpp:233-252, tools/pack_trtllm_experts.py:134-148):
w13 rows are [up; gate], block scales are interleaved per expert, and one alpha
per expert per GEMM is input_scale * weight_global.
"""
import math

import torch

from .runtime import (EXPERTS, HIDDEN, INTER, STAGE_QUANTIZE, STAGE_SORT, STAGE_W13, TOP_K,
                      W13_OUT, BUF_W13_OUT, ExpertWeights, Nvfp4ExpertRunner, pack_experts,
                      route_128_top8, route_project)


def _randn(shape, std, generator, device):
    return torch.randn(shape, generator=generator, device=device, dtype=torch.float32) * std


def make_packed_experts(seed, device, chunk=16, keep_fp32=False):
    """Returns dict(w13, w13_sf, g13, w2, w2_sf, g2[, w13_f32, w2_f32]) on `device`.

    fp32 weights are generated and packed `chunk` experts at a time (the fp32 form
    of one layer is 3 GB)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {k: [] for k in ("w13", "w13_sf", "g13", "w2", "w2_sf", "g2", "w13_f32", "w2_f32")}
    for _ in range(0, EXPERTS, chunk):
        w13 = _randn((chunk, W13_OUT, HIDDEN), 0.02, gen, device)  # rows [up; gate]
        w2 = _randn((chunk, HIDDEN, INTER), 0.02, gen, device)
        c13, s13, g13 = pack_experts(w13)
        c2, s2, g2 = pack_experts(w2)
        for key, value in (("w13", c13), ("w13_sf", s13), ("g13", g13), ("w2", c2),
                           ("w2_sf", s2), ("g2", g2)):
            out[key].append(value)
        if keep_fp32:
            out["w13_f32"].append(w13.cpu())
            out["w2_f32"].append(w2.cpu())
    result = {k: torch.cat(v) for k, v in out.items() if v}
    return result


def zipf_bias(seed, s=1.1):
    """log of a Zipf(s) pmf laid over a fixed random permutation of the experts."""
    gen = torch.Generator().manual_seed(seed)
    ranks = torch.arange(1, EXPERTS + 1, dtype=torch.float64)
    pmf = ranks.pow(-s)
    pmf = pmf / pmf.sum()
    perm = torch.randperm(EXPERTS, generator=gen)
    bias = torch.empty(EXPERTS, dtype=torch.float64)
    bias[perm] = pmf.log()
    return bias.float()


class SyntheticLayer:
    """One MoE layer with synthetic weights, router and a calibrated runner."""

    def __init__(self, seed, max_tokens, device="cuda:0", bias_std=0.0, zipf=False,
                 shared_scratch=None, packed=None):
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed * 7919 + 13)
        self.router_w = _randn((EXPERTS, HIDDEN), 0.02, gen, self.device).to(torch.bfloat16)
        self.expert_scale = torch.ones(EXPERTS, dtype=torch.bfloat16, device=self.device)
        self.bias = None
        if zipf:
            self.bias = zipf_bias(seed).to(self.device)
        elif bias_std > 0:
            self.bias = _randn((EXPERTS,), bias_std, gen, self.device)
        self.packed = packed if packed is not None else make_packed_experts(seed, self.device)
        self.max_tokens = max_tokens
        self._shared = shared_scratch
        self.weights = None
        self.runner = None

    def inputs(self, tokens, seed):
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        return torch.randn((tokens, HIDDEN), generator=gen, device=self.device,
                           dtype=torch.float32).to(torch.bfloat16)

    def route(self, x, weights=None, ids=None, want_logits=False, runner=None):
        """Router projection, per-expert bias (the model of uneven expert load), top-8 and
        softmax in one kernel of the library (gevva_moe_route_project)."""
        return route_project(x, self.router_w, self.expert_scale, bias=self.bias, want_logits=want_logits,
                             status_of=runner if runner is not None else self.runner, weights=weights, ids=ids)

    def logits(self, x):
        """Router logits by a plain library GEMM, as the reference computes them
        (src/cuda/runtime/prefill.cuh:414-419), for tests that hand identical logits to the
        library and to the oracle; the optional per-expert bias models uneven expert load."""
        out = torch.matmul(x, self.router_w.t())
        if self.bias is not None:
            out = (out.float() + self.bias).to(torch.bfloat16)
        return out

    def calibrate(self, x):
        """Fixes the static activation scales the way a calibration run would:
        s1 = amax(x)/(6*448); s2 = amax(gelu(gate)*up)/(6*448) from one pass."""
        s1 = float(x.float().abs().max()) / (6.0 * 448.0)
        ones = torch.ones(EXPERTS, dtype=torch.float32, device=self.device)
        p = self.packed
        provisional = ExpertWeights(p["w13"], p["w13_sf"], p["w2"], p["w2_sf"],
                                    (p["g13"] * s1).contiguous(), p["g2"].clone(),
                                    (ones / s1).contiguous(), ones.clone())
        tokens = x.shape[0]
        runner = Nvfp4ExpertRunner(provisional, tokens)
        _, ids = self.route(x, runner=runner)
        runner.launch_stages(STAGE_SORT | STAGE_QUANTIZE | STAGE_W13, tokens, input=x,
                             expert_ids=ids)
        runner.check()
        fused = runner.buffer(BUF_W13_OUT, torch.bfloat16)[: tokens * TOP_K * W13_OUT]
        fused = fused.view(tokens * TOP_K, W13_OUT).float()
        up, gate = fused[:, :INTER], fused[:, INTER:]
        act = 0.5 * gate * (1.0 + torch.erf(gate * (1.0 / math.sqrt(2.0)))) * up
        s2 = float(act.abs().max()) / (6.0 * 448.0)
        del runner
        self.set_scales(s1, s2)
        return s1, s2

    def set_scales(self, s1, s2):
        ones = torch.ones(EXPERTS, dtype=torch.float32, device=self.device)
        p = self.packed
        self.s1, self.s2 = s1, s2
        self.weights = ExpertWeights(p["w13"], p["w13_sf"], p["w2"], p["w2_sf"],
                                     (p["g13"] * s1).contiguous(), (p["g2"] * s2).contiguous(),
                                     (ones / s1).contiguous(), (ones / s2).contiguous())
        self.runner = Nvfp4ExpertRunner(self.weights, self.max_tokens, self._shared)

    def forward(self, x, out=None):
        """Router projection -> route -> experts; returns bf16 [tokens, 2816]."""
        tokens = x.shape[0]
        weights, ids = self.route(x)
        if out is None:
            out = torch.empty_like(x)
        self.runner.launch_batch(x, ids, weights, out, tokens)
        return out


class SyntheticStack:
    """Random-init FFN stack in the shape of Gemma-4 26B-A4B with attention replaced by
    identity: per layer the MoE above plus a dense FP8 GeGLU MLP of width 2112 (weights
    ~N(0, 0.02), per-tensor scale amax/448), norm weights 1, layer scalar 1.  With
    `distinct_experts=False` every layer shares one packed expert set (tests)."""

    def __init__(self, layers, max_tokens, device="cuda:0", seed=0, distinct_experts=True, s1=None, s2=None):
        from .feedforward import DENSE, DenseMlp, FeedForwardLayer, pack_fp8
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed + 4242)
        ones = torch.ones(HIDDEN, dtype=torch.bfloat16, device=self.device)
        self.layers = []
        first_runner = None
        packed = None
        for index in range(layers):
            if packed is None or distinct_experts:
                packed = make_packed_experts(seed + index, self.device)
            base = SyntheticLayer(seed + index, max_tokens, self.device, shared_scratch=first_runner,
                                  packed=packed)
            if s1 is None:
                calib = base.inputs(min(max_tokens, 256), seed + 17)
                s1, s2 = base.calibrate(calib)
            base.set_scales(s1, s2)
            first_runner = first_runner or base.runner
            gate = _randn((DENSE, HIDDEN), 0.02, gen, self.device)
            up = _randn((DENSE, HIDDEN), 0.02, gen, self.device)
            down = _randn((HIDDEN, DENSE), 0.02, gen, self.device)
            gq, gs = pack_fp8(gate)
            uq, us = pack_fp8(up)
            dq, ds = pack_fp8(down)
            dense = DenseMlp(torch.cat([gq, uq]).contiguous(), dq, gs, us, ds, max_tokens)
            self.layers.append(FeedForwardLayer(
                dense_pre=ones, expert_pre=ones, router_scale=ones, router_w=base.router_w,
                expert_scale=base.expert_scale, dense_post=ones, expert_post=ones, combined_post=ones,
                layer_scalar=torch.ones(1, dtype=torch.bfloat16, device=self.device),
                experts=base.runner, dense=dense))
            self._keep = getattr(self, "_keep", []) + [base]
        self.aux = torch.cuda.Stream(device=self.device)

    def forward(self, hidden, concurrent=True):
        for layer in self.layers:
            hidden = layer.forward(hidden, self.aux if concurrent else None)
        return hidden
