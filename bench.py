"""Benchmark of the NVFP4 MoE layer (Gemma-4 26B-A4B shapes) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the layer over one batch, made of calls into the library only: router
projection fused with top-8 routing, route sort, NVFP4 quantise, grouped w13 GEMM with
GeGLU+requantise in its epilogue, grouped w2 GEMM, weighted reduce.  Workload of `value` at
every N: the prefill configuration, 4096 tokens per GPU with a per-expert router bias
~N(0, 0.5); four different input batches are rotated.  Beside it the line carries: the same step
looped for two seconds (`sustained`), the end-to-end figure through host buffers (`e2e`), the
dominant kernel's roofline, the decode sweep, the 30-layer FFN stack (`config3`), the
16384-token Zipf batch on one GPU (`config4_single_gpu`) and, with several GPUs, the
expert-parallel form of that batch (`ep_config4`).  Prints one JSON line (rank 0).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOKENS = 4096
CONFIG4_TOKENS = 16384
HIDDEN, EXPERTS, TOP_K, INTER, DENSE = 2816, 128, 8, 704, 2112
FLOP_PER_TOKEN = TOP_K * (2 * 2 * INTER * HIDDEN + 2 * HIDDEN * INTER)  # 95 158 272
W13_FLOP_PER_TOKEN = TOP_K * 2 * 2 * INTER * HIDDEN                      # 63 438 848
DENSE_FLOP_PER_TOKEN = 2 * 3 * DENSE * HIDDEN                            # 35 684 352
LAYER_WEIGHT_BYTES = 428212224
NOMINAL_FP4_TFLOPS = 9000.0
# fused w13 launch at 4096 tokens: weights + weight scales + operand codes/scales + output codes/scales
W13_ALGORITHMIC_BYTES = 128 * (1982464 + 247808) + 32768 * (1408 + 176) + 32768 * (352 + 44)
# RECORDED figures (ncu captures summarised under profiles/, not measured by this run):
# dram__bytes_read.sum + dram__bytes_write.sum of one fused w13 launch at this workload
W13_DRAM_TRAFFIC_BYTES_RECORDED = 342586368 + 12649216
# DRAM bytes of one layer step at 4096 tokens: the two GEMMs as captured, the quantiser
# (23 MB read + 52 MB written) and the reduce (185 MB read + 23 MB written) by their algorithmic bytes
LAYER_DRAM_BYTES_RECORDED = (342586368 + 12649216) + (156119808 + 134346240) + 75000000 + 207600000
WORKLOAD = "prefill_4096_tokens_router_bias_N(0,0.5)"
INPUT_BATCHES = 4


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons (read-only query) while a timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period_ms=100):
        self.index = index
        self.period_ms = period_ms
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_layer(device, rank):
    """Same experts, router and static scales on every rank (seed 0, calibrated on one fixed
    batch); each rank then gets its own input batches."""
    from gevva_b200.synthetic import SyntheticLayer
    layer = SyntheticLayer(seed=0, max_tokens=TOKENS, device=device, bias_std=0.5)
    layer.calibrate(layer.inputs(TOKENS, seed=1000))
    return layer, [layer.inputs(TOKENS, seed=1000 + rank + 100 * i) for i in range(INPUT_BATCHES)]


def library_nvfp4_gemm_tflops(device, size=8192, launches=20):
    """Comparison figure only: the library's block-scaled NVFP4 GEMM (cuBLASLt through
    torch._scaled_mm) on a dense size^3 problem, timed here with CUDA events.  It is the FP4
    throughput this box reaches with a library kernel; MEASURED_PEAKS.json has no FP4 entry."""
    import torch
    try:
        a = torch.randint(0, 255, (size, size // 2), dtype=torch.uint8, device=device).view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 255, (size, size // 2), dtype=torch.uint8, device=device).view(torch.float4_e2m1fn_x2)
        sa = torch.ones(size * size // 16, device=device).to(torch.float8_e4m3fn)
        sb = torch.ones(size * size // 16, device=device).to(torch.float8_e4m3fn)
        run = lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            run()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(launches):
            run()
        end.record()
        torch.cuda.synchronize()
        return 2.0 * size ** 3 / (start.elapsed_time(end) / launches * 1e-3) / 1e12
    except Exception:  # not every torch build exposes the FP4 path
        return None


def layer_step(layer, x, out, weights, ids):
    """The timed unit; every kernel in it belongs to the library.  With more than one GPU the
    experts are sharded and `layer.ep` exchanges rows over NVLink."""
    layer.route(x, weights=weights, ids=ids)
    runner = layer.ep if getattr(layer, "ep", None) is not None else layer.runner
    runner.launch_batch(x, ids, weights, out, x.shape[0])


def launches_per_step(world, tokens, sm_count=148, ep_chunks=2, ep_parts=1):
    """Kernels of the library that one layer step launches, counted from the launch paths
    (gevva_moe_launch_stages in csrc/moe_abi.cu, the four gevva_moe_ep_* calls in csrc/ep.cu)."""
    sort = 1 if tokens * TOP_K <= 1024 or (tokens * TOP_K + 1023) // 1024 <= sm_count else 3
    if world == 1:
        if tokens <= 128:
            return 1 + 1 + 1          # fused router; sort, quantiser and both expert GEMMs in one launch; reduce
        return 1 + sort + 1 + 3       # fused router; sort; quantise; w13, w2, reduce
    # fused router; sort + count exchange (with the first barrier inside); dispatch, row destinations;
    # scale re-tiling (waits for every rank's rows) + (w13, w2) per compute part; reduce; one flag barrier
    # (the router once; everything else once per micro-batch in flight)
    if ep_parts > 1:
        share = (tokens + ep_parts - 1) // ep_parts
        sort = 1 if share * TOP_K <= 1024 or (share * TOP_K + 1023) // 1024 <= sm_count else 3
    return 1 + ep_parts * ((sort + 1) + 2 + (1 + 2 * ep_chunks) + 1 + 1)


def timed_loop(fn, steps):
    import torch
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        fn(i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop)


def decode_sweep(layer, device, steps):
    """Decode-sized batches (1, 8, 32, 64 tokens, unbiased router): the layer is bound by
    streaming the routed experts' weights from HBM.  32 different batches are cycled so a
    step's experts are not the previous steps' (428 MB of weights against 126 MB of L2)."""
    import torch
    import gevva_b200
    from gevva_b200.runtime import Nvfp4ExpertRunner
    peaks, _ = measured_peaks()
    runner = Nvfp4ExpertRunner(layer.weights, 64)
    rows = []
    for tokens in (1, 8, 32, 64):
        pool = [layer.inputs(tokens, seed=5000 + 97 * tokens + i) for i in range(32)]
        out = torch.empty_like(pool[0])
        weights = torch.empty((tokens, TOP_K), dtype=torch.float32, device=device)
        ids = torch.empty((tokens, TOP_K), dtype=torch.int32, device=device)
        distinct = []

        def step(x):
            gevva_b200.route_project(x, layer.router_w, layer.expert_scale, weights=weights, ids=ids,
                                     status_of=runner)
            runner.launch_batch(x, ids, weights, out, tokens)

        graphs = []
        for x in pool:
            step(x)
            distinct.append(int(torch.unique(ids).numel()))
        torch.cuda.synchronize()
        # CUDA graphs of eight layer steps (eight different batches) each: the layer's launches
        # allocate nothing and never touch the host, so they capture as they stand, and a decode
        # loop is captured as a whole, many layers per graph, in the reference too
        # (src/cuda/runtime/verifier.cuh:1058-1078).
        per_graph = 8
        for first in range(0, len(pool), per_graph):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for x in pool[first:first + per_graph]:
                    step(x)
            graphs.append(graph)
        for graph in graphs:
            graph.replay()
        torch.cuda.synchronize()
        replays = max(1, (steps + per_graph - 1) // per_graph)
        us = timed_loop(lambda i: graphs[i % len(graphs)].replay(), replays) * 1e3 / (replays * per_graph)
        d = sum(distinct) / len(distinct)
        algorithmic = d * 3345408 + 720896 + 2 * tokens * HIDDEN * 2
        gbs = algorithmic / (us * 1e-6) / 1e9
        rows.append({"tokens": tokens, "us_per_layer": us, "distinct_experts": d,
                     "algorithmic_bytes": algorithmic, "hbm_gbs": gbs,
                     "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"]),
                     "frac_of_8000_gbs": gbs / 8000.0, "tokens_per_s": tokens / (us * 1e-6),
                     "launch": f"CUDA graphs of 8 layer steps, {launches_per_step(1, tokens)} kernels per layer"})
    runner.check()
    return rows


def decode_eager(layer, device, tokens, steps):
    """For a profiler: `steps` decode-sized layer steps launched one by one (no CUDA graph),
    each on a different batch so that the routed experts' weights come from HBM."""
    import torch
    import gevva_b200
    from gevva_b200.runtime import Nvfp4ExpertRunner
    runner = Nvfp4ExpertRunner(layer.weights, max(tokens, 1))
    out = torch.empty((tokens, HIDDEN), dtype=torch.bfloat16, device=device)
    weights = torch.empty((tokens, TOP_K), dtype=torch.float32, device=device)
    ids = torch.empty((tokens, TOP_K), dtype=torch.int32, device=device)
    for i in range(steps):
        x = layer.inputs(tokens, seed=7000 + i)
        gevva_b200.route_project(x, layer.router_w, layer.expert_scale, weights=weights, ids=ids, status_of=runner)
        runner.launch_batch(x, ids, weights, out, tokens)
    torch.cuda.synchronize()
    runner.check()


def config3_stack(device, passes=5):
    """The 30-layer configuration: 30 random-init layers (MoE + dense FP8 GeGLU MLP of width 2112 +
    the pre/post norm steps, attention = identity), 2048 tokens, distinct weights per layer."""
    import torch
    from gevva_b200.synthetic import SyntheticStack
    tokens, layers = 2048, 30
    stack = SyntheticStack(layers, tokens, device, seed=0)
    gen = torch.Generator(device=device)
    gen.manual_seed(77)
    hidden = torch.randn((tokens, HIDDEN), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    for _ in range(3):
        stack.forward(hidden)
    torch.cuda.synchronize()
    eager_ms = timed_loop(lambda i: stack.forward(hidden), passes) / passes
    # the whole pass as one CUDA graph (the reference captures its layer loop too,
    # src/cuda/runtime/verifier.cuh:1058-1078): nothing in it allocates or touches the host
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        stack.forward(hidden)
    graph.replay()
    torch.cuda.synchronize()
    ms = timed_loop(lambda i: graph.replay(), passes) / passes
    for layer in stack.layers:
        layer.experts.check()
    del graph
    moe_flop = layers * tokens * FLOP_PER_TOKEN
    dense_flop = layers * tokens * DENSE_FLOP_PER_TOKEN
    del stack
    torch.cuda.empty_cache()
    return {"workload": "30-layer FFN stack, 2048 tokens, distinct weights per layer (13.4 GB)",
            "ms_per_pass": ms, "us_per_layer": ms * 1e3 / layers, "tokens_per_s": tokens / (ms * 1e-3),
            "moe_flop_fraction": moe_flop / (moe_flop + dense_flop),
            "dense_fp8_flop_fraction": dense_flop / (moe_flop + dense_flop),
            "tflops_both_gemm_kinds": (moe_flop + dense_flop) / (ms * 1e-3) / 1e12,
            "passes": passes, "ms_per_pass_eager": eager_ms,
            "schedule": "dense MLP on a second stream beside the experts; the pass replayed as one CUDA graph"}


def config4_layer(base_layer, device):
    """The Zipf(1.1)-biased router of the 16384-token expert-parallel configuration over the same experts."""
    from gevva_b200.synthetic import SyntheticLayer
    layer = SyntheticLayer(seed=0, max_tokens=16, device=device, zipf=True, packed=base_layer.packed)
    layer.weights = base_layer.weights      # same calibrated static scales
    return layer


def config4_single_gpu(base_layer, device, steps):
    import torch
    from gevva_b200.runtime import Nvfp4ExpertRunner
    layer = config4_layer(base_layer, device)
    runner = Nvfp4ExpertRunner(layer.weights, CONFIG4_TOKENS)
    pool = [layer.inputs(CONFIG4_TOKENS, seed=9000 + i) for i in range(2)]
    out = torch.empty_like(pool[0])
    weights = torch.empty((CONFIG4_TOKENS, TOP_K), dtype=torch.float32, device=device)
    ids = torch.empty((CONFIG4_TOKENS, TOP_K), dtype=torch.int32, device=device)

    def step(i):
        layer.route(pool[i % 2], weights=weights, ids=ids, runner=runner)
        runner.launch_batch(pool[i % 2], ids, weights, out, CONFIG4_TOKENS)

    for i in range(3):
        step(i)
    runner.check()
    ms = timed_loop(step, steps) / steps
    loads = torch.bincount(ids.reshape(-1).long(), minlength=EXPERTS)
    runner.check()
    result = {"workload": "16384 tokens, Zipf(1.1) router bias, one GPU", "ms_per_step": ms,
              "tokens_per_s": CONFIG4_TOKENS / (ms * 1e-3),
              "layer_tflops": FLOP_PER_TOKEN * CONFIG4_TOKENS / (ms * 1e-3) / 1e12,
              "rows_of_most_loaded_expert": int(loads.max()), "rows_of_least_loaded_expert": int(loads.min())}
    del runner
    torch.cuda.empty_cache()
    return result


def quantiser_with_distinct_scales(layer, x, ids, device, steps):
    """The input quantiser with 128 different static scales (a real sidecar has a different
    g1.input_scale_quant per expert; the synthetic set-up replicates one)."""
    import torch
    import gevva_b200 as gm
    from gevva_b200 import runtime as rt
    w = layer.weights
    factor = 1.0 + 0.01 * torch.arange(EXPERTS, dtype=torch.float32, device=device)
    varied = gm.ExpertWeights(w.w13, w.w13_sf, w.w2, w.w2_sf, (w.alpha1 * factor).contiguous(), w.alpha2,
                              (w.in_scale_q1 / factor).contiguous(), w.in_scale_q2)
    out = {}
    for name, weights in (("one_scale", w), ("distinct_scales", varied)):
        runner = gm.Nvfp4ExpertRunner(weights, TOKENS)
        runner.launch_stages(rt.STAGE_SORT, TOKENS, expert_ids=ids)
        for _ in range(3):
            runner.launch_stages(rt.STAGE_QUANTIZE, TOKENS, input=x, expert_ids=ids)
        out[name + "_us"] = timed_loop(
            lambda i: runner.launch_stages(rt.STAGE_QUANTIZE, TOKENS, input=x, expert_ids=ids), steps) * 1e3 / steps
        runner.check()
        del runner
    return out


# ------------------------------------------------------------------------------------------
# CPU legs
# ------------------------------------------------------------------------------------------
def oracle_sample(rank_seed, tokens):
    """Synthetic inputs for the CPU legs, generated without a GPU."""
    import numpy as np
    import torch
    from tests.oracle_api import Oracle
    oracle = Oracle()
    oracle.lib.gvo_set_threads(os.cpu_count() or 1)   # torchrun exports OMP_NUM_THREADS=1
    gen = torch.Generator().manual_seed(rank_seed)
    hw = {k: [] for k in ("w13", "w13_sf", "g13", "w2", "w2_sf", "g2")}
    for _ in range(EXPERTS):
        w13 = (torch.randn((2 * INTER, HIDDEN), generator=gen) * 0.02).numpy()
        c, s, g = oracle.pack_weight(w13)
        hw["w13"].append(c), hw["w13_sf"].append(s), hw["g13"].append(g)
        w2 = (torch.randn((HIDDEN, INTER), generator=gen) * 0.02).numpy()
        c, s, g = oracle.pack_weight(w2)
        hw["w2"].append(c), hw["w2_sf"].append(s), hw["g2"].append(g)
    x = torch.randn((tokens, HIDDEN), generator=gen).to(torch.bfloat16)
    router = (torch.randn((EXPERTS, HIDDEN), generator=gen) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(EXPERTS, generator=gen) * 0.5).numpy()

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    s1 = float(x.float().abs().max()) / (6 * 448)
    s2 = 16.0 / (6 * 448)
    weights = dict(
        w13=np.stack(hw["w13"]), w13_sf=np.stack(hw["w13_sf"]), w2=np.stack(hw["w2"]),
        w2_sf=np.stack(hw["w2_sf"]),
        alpha1=(np.array(hw["g13"], np.float32) * np.float32(s1)),
        alpha2=(np.array(hw["g2"], np.float32) * np.float32(s2)),
        in_scale_q1=np.full(EXPERTS, 1 / s1, np.float32),
        in_scale_q2=np.full(EXPERTS, 1 / s2, np.float32))
    scale = bits(torch.ones(EXPERTS, dtype=torch.bfloat16))
    return oracle, bits(x), bits(router), bias, scale, weights


def time_oracle(oracle, x_bits, router_bits, bias, scale_bits, weights, tokens, repeats):
    """Whole layer steps on the CPU: router projection, routing, experts."""
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        logits = oracle.router_logits(x_bits[:tokens], router_bits, bias)
        rw, ids = oracle.route(logits, scale_bits)
        oracle.moe_layer(x_bits[:tokens], ids, rw, weights)
        times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    """The reference has no CPU path and its GPU kernels are SM120-only, so this arm times the CPU
    oracle (a restatement: dequantise to fp32, then matmul) with all host threads, on the bench's
    own configuration: every timed step is the whole 4096-token batch when the run then fits in a
    few minutes, otherwise the largest slice of it that does (stated in `config`)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle, x_bits, router_bits, bias, scale_bits, weights = oracle_sample(0, TOKENS)
    threads = oracle.lib.gvo_threads()
    # a small pass warms caches and the thread pool, then one probe decides the step size
    time_oracle(oracle, x_bits, router_bits, bias, scale_bits, weights, 128, 1)
    probe = time_oracle(oracle, x_bits, router_bits, bias, scale_bits, weights, 512, 1)[0]
    budget_s = 200.0
    per_token = probe / 512
    sample = TOKENS
    while sample > 256 and per_token * sample * args.steps > budget_s:
        sample //= 2
    for _ in range(min(args.warmup, 1)):
        time_oracle(oracle, x_bits, router_bits, bias, scale_bits, weights, sample, 1)
    times = time_oracle(oracle, x_bits, router_bits, bias, scale_bits, weights, sample, args.steps)
    per_step = sum(times) / len(times)
    value = sample / per_step
    what = "the whole 4096-token batch" if sample == TOKENS else f"a {sample}-token slice of the 4096-token batch"
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": sample,
                   "note": f"CPU oracle port; each timed step is {what} (router projection, routing, experts); "
                           "one untimed warm-up step of the same size, earlier warm-ups on 128 and 512 tokens"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "nproc": os.cpu_count(),
                         "sample": f"{sample} of {TOKENS} tokens per step, all 128 experts' weights"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# expert parallel records (N > 1)
# ------------------------------------------------------------------------------------------
def placement_from_calibration(layer, world, rank, tokens):
    import torch
    import torch.distributed as dist
    from gevva_b200.expert_parallel import balanced_placement
    calibration = layer.inputs(tokens, seed=2000 + rank)
    _, ids = layer.route(calibration)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=EXPERTS)
    dist.all_reduce(counts)
    return balanced_placement(counts.tolist(), world)


def nccl_exchange_only(count_matrix, world, rank, device, repeats=10):
    """Comparison figure: the two exchanges of one expert-parallel step as NCCL all-to-alls of the
    same bytes with the same per-destination splits (host-known, as a library all-to-all needs
    them): dispatch 1584 B per route, combine 5632 B per route.  No permutation or GEMM."""
    import torch
    import torch.distributed as dist
    el = EXPERTS // world
    sent = [int(count_matrix[rank, d * el:(d + 1) * el].sum()) for d in range(world)]       # my rows to rank d
    received = [int(count_matrix[s, rank * el:(rank + 1) * el].sum()) for s in range(world)]  # rows from rank s
    out = {}
    for name, row_bytes, send_counts, recv_counts in (("dispatch", 1584, sent, received),
                                                      ("combine", 5632, received, sent)):
        src = torch.empty(sum(send_counts) * row_bytes, dtype=torch.uint8, device=device)
        dst = torch.empty(sum(recv_counts) * row_bytes, dtype=torch.uint8, device=device)
        in_splits = [c * row_bytes for c in send_counts]
        out_splits = [c * row_bytes for c in recv_counts]
        for _ in range(3):
            dist.all_to_all_single(dst, src, out_splits, in_splits)
        torch.cuda.synchronize()
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(repeats):
            dist.all_to_all_single(dst, src, out_splits, in_splits)
        stop.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / repeats * 1e3], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name + "_us"] = float(t[0])
        out[name + "_bytes_sent_rank0"] = sum(send_counts) * row_bytes
    return out


def ep_record(layer, world, rank, device, tokens_per_gpu, placement_kind, steps, seed):
    """One expert-parallel configuration: parity against the single-GPU runner on this rank's own
    batch, timed steps (max over ranks), phase times, load imbalance, and the exposed communication
    (step time minus the same stages with every store kept local)."""
    import torch
    import torch.distributed as dist
    from gevva_b200.expert_parallel import ExpertParallelRunner, local_expert_weights, strided_placement
    from gevva_b200.runtime import Nvfp4ExpertRunner, _ptr, _stream_handle
    placement = strided_placement(world) if placement_kind == "strided" else \
        placement_from_calibration(layer, world, rank, tokens_per_gpu)
    ep = ExpertParallelRunner(local_expert_weights(layer.weights, rank, world, placement),
                              layer.weights.in_scale_q1, tokens_per_gpu, placement=placement)
    single = Nvfp4ExpertRunner(layer.weights, tokens_per_gpu)
    x = layer.inputs(tokens_per_gpu, seed=seed + rank)
    weights, ids = layer.route(x, runner=single)
    want, got = torch.empty_like(x), torch.empty_like(x)
    single.launch_batch(x, ids, weights, want, tokens_per_gpu)
    single.check()
    ep.launch_batch(x, ids, weights, got, tokens_per_gpu)
    status, received = ep.status()
    if status != 0:
        raise RuntimeError(f"expert-parallel device status {status}")
    equal = torch.tensor([1 if torch.equal(got, want) else 0], device=device)
    dist.all_reduce(equal, op=dist.ReduceOp.MIN)

    def step(i):
        layer.route(x, weights=weights, ids=ids, runner=single)
        ep.launch_batch(x, ids, weights, got, tokens_per_gpu)

    for i in range(3):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    ms = timed_loop(step, steps) / steps
    phases = [ep.timed_step(x, ids, weights, got, tokens_per_gpu) for _ in range(4)]
    phases = {k: sum(p[k] for p in phases[1:]) / 3 for k in phases[0]}
    dist.barrier()   # no rank may still be storing into a peer while the local variants run
    # the same stages with every store kept on this GPU (buffers of the last step are reused)
    s = _stream_handle(None)
    local = {}
    for name, call in (("dispatch_local", lambda: ep._call("gevva_moe_ep_dispatch_local", _ptr(x), _ptr(ids),
                                                           tokens_per_gpu, s)),
                       ("compute_local", lambda: ep._call("gevva_moe_ep_compute_local", s))):
        call()
        torch.cuda.synchronize()
        local[name] = timed_loop(lambda i: call(), 5) * 1e3 / 5
    dist.barrier()
    ep.launch_batch(x, ids, weights, got, tokens_per_gpu)    # leave the buffers consistent again
    torch.cuda.synchronize()
    router_us = timed_loop(lambda i: layer.route(x, weights=weights, ids=ids, runner=single), 5) * 1e3 / 5
    no_comm_us = router_us + phases["route_sort"] + local["dispatch_local"] + local["compute_local"] + phases["reduce"]
    stats = torch.tensor([ms, no_comm_us, float(received)], dtype=torch.float64, device=device)
    worst = stats.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    total = stats.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    counts = torch.zeros((world, EXPERTS), dtype=torch.int64, device=device)
    remap = torch.tensor(placement, device=device)
    counts[rank].scatter_add_(0, remap[ids.reshape(-1).long()], torch.ones(ids.numel(), dtype=torch.int64, device=device))
    dist.all_reduce(counts)
    step_us = float(worst[0]) * 1e3
    record = {
        "tokens_total": tokens_per_gpu * world, "tokens_per_gpu": tokens_per_gpu, "placement": placement_kind,
        "ep_parity": "bit-equal to the single-GPU runner on every rank" if int(equal[0]) == 1 else "MISMATCH",
        "ms_per_step": step_us * 1e-3, "tokens_per_s": tokens_per_gpu * world / (step_us * 1e-6),
        "load_imbalance_max_over_mean_rows": float(worst[2]) / (float(total[2]) / world),
        "phases_us_rank0": phases,
        "no_comm_us_max_over_ranks": float(worst[1]),
        "exposed_comm_us": step_us - float(worst[1]),
        "exposed_comm_definition": "step time minus (router + route sort with its count exchange + dispatch with local stores + compute "
                                   "with local result stores + reduce), max over ranks",
        "nccl_all_to_all_exchange_only": nccl_exchange_only(counts.cpu(), world, rank, device),
    }
    del ep, single
    torch.cuda.empty_cache()
    return record


def ep_one_rank(layer, batches, device, steps):
    """For a profiler (which must not wrap a multi-rank command): the expert-parallel step with a
    process group of one rank, i.e. the whole protocol (count exchange, dispatch, compute in two
    halves, barrier, reduce) with every store staying on this GPU.  The result must be the plain
    runner's, bit for bit."""
    import torch
    import torch.distributed as dist
    from gevva_b200.expert_parallel import ExpertParallelRunner, local_expert_weights
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    ep = ExpertParallelRunner(local_expert_weights(layer.weights, 0, 1), layer.weights.in_scale_q1, TOKENS)
    x = batches[0]
    weights, ids = layer.route(x)
    want, got = torch.empty_like(x), torch.empty_like(x)
    layer.runner.launch_batch(x, ids, weights, want, TOKENS)
    for _ in range(steps):
        ep.launch_batch(x, ids, weights, got, TOKENS)
    status, _ = ep.status()
    if status != 0 or not torch.equal(got, want):
        raise RuntimeError(f"one-rank expert-parallel step: status {status}, equal {torch.equal(got, want)}")
    phases = [ep.timed_step(x, ids, weights, got, TOKENS) for _ in range(4)]
    print(json.dumps({"ep_one_rank_phases_us": {k: sum(p[k] for p in phases[1:]) / 3 for k in phases[0]}}), flush=True)
    del ep
    dist.destroy_process_group()


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from gevva_b200 import runtime as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layer, batches = build_layer(device, rank)
    layer.ep = None
    if args.profile_decode:
        decode_eager(layer, device, args.profile_decode, 6)
        if rank == 0:
            print(json.dumps({"profile_decode_tokens": args.profile_decode, "steps": 6}), flush=True)
        return
    if args.profile_ep_one_rank:
        ep_one_rank(layer, batches, device, 8)
        if rank == 0:
            print(json.dumps({"profile_ep_one_rank": True, "steps": 8}), flush=True)
        return
    x = batches[0]
    out = torch.empty_like(x)
    weights = torch.empty((TOKENS, TOP_K), dtype=torch.float32, device=device)
    ids = torch.empty((TOKENS, TOP_K), dtype=torch.int32, device=device)
    ep_parity = None
    ep = None
    if world > 1:
        from gevva_b200.expert_parallel import ExpertParallelRunner, local_expert_weights
        # Experts are placed by load observed on a calibration batch (other tokens than the timed
        # ones, same router): most loaded first, each to the least loaded rank with a free slot.
        placement = placement_from_calibration(layer, world, rank, TOKENS)
        ep = ExpertParallelRunner(local_expert_weights(layer.weights, rank, world, placement),
                                  layer.weights.in_scale_q1, TOKENS, placement=placement)
        # before anything is timed: the expert-parallel result of this rank's batch must be the
        # single-GPU runner's, bit for bit
        want = torch.empty_like(x)
        layer.route(x, weights=weights, ids=ids)
        layer.runner.launch_batch(x, ids, weights, want, TOKENS)
        ep.launch_batch(x, ids, weights, out, TOKENS)
        status, _ = ep.status()
        layer.runner.check()
        equal = torch.tensor([1 if (status == 0 and torch.equal(out, want)) else 0], device=device)
        dist.all_reduce(equal, op=dist.ReduceOp.MIN)
        ep_parity = "bit-equal" if int(equal[0]) == 1 else "MISMATCH"
        layer.ep = ep
        if args.ep_parts > 1:
            # the timed step runs the batch as micro-batches in flight on streams of their own (the
            # plain runner stays for the phase times); same bits required
            from gevva_b200.expert_parallel import MicroBatchedExpertParallel
            micro = MicroBatchedExpertParallel(local_expert_weights(layer.weights, rank, world, placement),
                                               layer.weights.in_scale_q1, TOKENS, placement=placement,
                                               parts=args.ep_parts)
            out.zero_()
            micro.launch_batch(x, ids, weights, out, TOKENS)
            status, _ = micro.status()
            equal = torch.tensor([1 if (status == 0 and torch.equal(out, want)) else 0], device=device)
            dist.all_reduce(equal, op=dist.ReduceOp.MIN)
            if int(equal[0]) != 1:
                ep_parity = "MISMATCH"
            layer.ep = micro

    def check():
        if layer.ep is not None:
            status, _ = layer.ep.status()
            if status != 0:
                raise RuntimeError(f"expert-parallel device status {status}")
        layer.runner.check()

    step = lambda i: layer_step(layer, batches[i % INPUT_BATCHES], out, weights, ids)
    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    check()

    # ---- device-resident throughput ("value") -----------------------------------
    sampler = ClockSampler(local_rank, period_ms=20)
    barrier()
    sampler.start()
    elapsed_ms = timed_loop(step, args.steps)
    barrier()
    clocks = sampler.stop()
    check()

    # ---- the same step for at least two seconds ("sustained") ---------------------
    sampler = ClockSampler(local_rank, period_ms=100)
    barrier()
    sampler.start()
    chunk = 500
    sustained_ms, sustained_steps = 0.0, 0
    wall = time.perf_counter()
    while not args.no_sustained:
        sustained_ms += timed_loop(step, chunk)
        sustained_steps += chunk
        go_on = torch.tensor([1 if time.perf_counter() - wall < 2.0 else 0], device=device)
        if world > 1:   # every rank must leave the loop after the same number of steps
            dist.all_reduce(go_on, op=dist.ReduceOp.MIN)
        if int(go_on[0]) == 0:
            break
    barrier()
    sustained_clocks = sampler.stop()
    check()

    # ---- end to end through host buffers ("e2e") -------------------------------
    # Every step copies its 4096-token batch from pinned host memory and its result back.
    # Three streams, two buffers: the copy-in of step i+1 and the copy-out of step i-1 run
    # beside the layer of step i (PCIe is full duplex); everything is inside the timed region.
    host_in = [b.cpu().pin_memory() for b in batches]
    host_out = [torch.empty_like(host_in[0]).pin_memory() for _ in range(2)]
    dev_in = [torch.empty_like(x) for _ in range(2)]
    dev_out = [torch.empty_like(x) for _ in range(2)]
    s_in, s_run, s_out = (torch.cuda.Stream(device=device) for _ in range(3))

    def e2e_loop(steps):
        ev_in = [None, None]
        ev_run = [None, None]
        ev_out = [None, None]
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if ev_run[b] is not None:
                    s_in.wait_event(ev_run[b])      # the layer of step i-2 has read this buffer
                dev_in[b].copy_(host_in[i % INPUT_BATCHES], non_blocking=True)
                ev_in[b] = s_in.record_event()
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[b])
                if ev_out[b] is not None:
                    s_run.wait_event(ev_out[b])     # the result of step i-2 has left this buffer
                layer_step(layer, dev_in[b], dev_out[b], weights, ids)
                ev_run[b] = s_run.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[b])
                host_out[b].copy_(dev_out[b], non_blocking=True)
                ev_out[b] = s_out.record_event()

    main = torch.cuda.current_stream()
    e2e_loop(4)
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for s_ in (s_in, s_run, s_out):
        s_.wait_stream(main)
    e2e_loop(args.steps)
    for s_ in (s_in, s_run, s_out):
        main.wait_stream(s_)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)

    # ---- the two GEMM kernels timed alone inside full steps of the single-GPU stages ---------
    g0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    g1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    h0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    h1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    runner = layer.runner
    for i in range(args.steps):
        xi = batches[i % INPUT_BATCHES]
        layer.route(xi, weights=weights, ids=ids)
        runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, TOKENS, input=xi, expert_ids=ids)
        g0[i].record()
        runner.launch_stages(rt.STAGE_W13 | rt.STAGE_GEGLU, TOKENS)  # one kernel: GeGLU in the epilogue
        g1[i].record()
        h0[i].record()
        runner.launch_stages(rt.STAGE_W2, TOKENS)
        h1[i].record()
        runner.launch_stages(rt.STAGE_REDUCE, TOKENS, route_weights=weights, output=out)
    torch.cuda.synchronize()
    w13_ms = sum(a.elapsed_time(b) for a, b in zip(g0, g1)) / args.steps
    w2_ms = sum(a.elapsed_time(b) for a, b in zip(h0, h1)) / args.steps

    ep_phases = None
    if ep is not None:
        samples = [ep.timed_step(x, ids, weights, out, TOKENS) for _ in range(5)]
        ep_phases = {k: sum(s[k] for s in samples[1:]) / (len(samples) - 1) for k in samples[0]}

    times = torch.tensor([elapsed_ms, e2e_ms, sustained_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, sustained_ms = (float(t) for t in times)

    ep_config4 = None
    if world > 1 and not args.no_ep_config4:
        layer.ep = None
        del ep
        torch.cuda.empty_cache()
        zipf = config4_layer(layer, device)
        zipf.runner = layer.runner
        ep_config4 = [ep_record(zipf, world, rank, device, CONFIG4_TOKENS // world, kind, max(args.steps, 10), 9000)
                      for kind in ("strided", "balanced")]

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        fp4_peak = 4.0 * float(peaks["bf16_tflops"])
        achieved = W13_FLOP_PER_TOKEN * TOKENS / (w13_ms * 1e-3) / 1e12
        total_tokens = TOKENS * world * args.steps
        value = total_tokens / (elapsed_ms * 1e-3)
        per_step = launches_per_step(world, TOKENS, ep_parts=args.ep_parts if world > 1 else 1)
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "experts": EXPERTS,
                       "top_k": TOP_K, "hidden": HIDDEN, "expert_width": INTER,
                       "input_batches_rotated": INPUT_BATCHES,
                       "parallelism": "single GPU" if world == 1 else
                       f"expert parallel x{world}: 128/{world} experts per GPU placed by the load of a "
                       "calibration batch, tokens data-parallel, "
                       "dispatch/combine by stores into peer memory over NVLink"
                       + (f", {args.ep_parts} micro-batches of a rank's batch in flight on streams of their own"
                          if args.ep_parts > 1 else ""),
                       "l2": "inputs larger than L2: 428 MB of expert weights stream every step"},
            "layer_tflops": FLOP_PER_TOKEN * TOKENS / (elapsed_ms / args.steps * 1e-3) / 1e12,
            "sustained": None if args.no_sustained else {
                "tokens_per_s": TOKENS * world * sustained_steps / (sustained_ms * 1e-3),
                "ms_per_step": sustained_ms / sustained_steps, "steps": sustained_steps,
                "seconds": sustained_ms * 1e-3, "clocks": sustained_clocks,
                "note": "the same step looped back to back for at least two seconds"},
            "roofline": {"bound": "tensor", "kernel": "grouped_nvfp4_gemm_kernel<kGeglu> (w13 + GeGLU + requantise)",
                         "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                         "frac": achieved / fp4_peak,
                         "traffic": W13_DRAM_TRAFFIC_BYTES_RECORDED,
                         "traffic_source": "recorded: dram__bytes_read+write of one launch, ncu capture of this "
                                           "workload summarised in profiles/grouped_nvfp4_gemm_prefill4096.md",
                         "algorithmic_bytes": W13_ALGORITHMIC_BYTES,
                         "peak_source": f"4 x bf16_tflops of MEASURED_PEAKS.json ({peak_kind}); "
                                        "no FP4 entry exists",
                         "frac_of_nominal_9000": achieved / NOMINAL_FP4_TFLOPS,
                         "measured_on": "this GPU's own 4096-token batches through the single-GPU stages",
                         "kernel_ms": w13_ms, "w2_kernel_ms": w2_ms,
                         "w2_tflops": (FLOP_PER_TOKEN - W13_FLOP_PER_TOKEN) * TOKENS / (w2_ms * 1e-3) / 1e12},
            "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": TOKENS * HIDDEN * 2, "d2h_bytes_per_step": TOKENS * HIDDEN * 2},
            "gpu_launches": per_step * args.steps,
            "gpu_launches_per_step": per_step,
            "clocks": clocks,
        }
        if ep_parity is not None:
            line["ep_parity"] = ep_parity
        if world == 1:
            step_seconds = elapsed_ms / args.steps * 1e-3
            line["layer_hbm"] = {
                "bytes_per_step_recorded": LAYER_DRAM_BYTES_RECORDED,
                "achieved_gbs": LAYER_DRAM_BYTES_RECORDED / step_seconds / 1e9,
                "peak_gbs": float(peaks["hbm_gbs"]),
                "frac": LAYER_DRAM_BYTES_RECORDED / step_seconds / 1e9 / float(peaks["hbm_gbs"]),
                "note": "whole layer step against the measured copy bandwidth, bytes as recorded by ncu for the "
                        "GEMMs plus the algorithmic bytes of quantiser and reduce: at 4096 tokens the layer "
                        "moves about 1 GB for 390 GFLOP, below the machine balance of the FP4 tensor pipe"}
            line["quantiser"] = quantiser_with_distinct_scales(layer, x, ids, device, args.steps)
        if world == 1 and not args.no_library_compare:
            library = library_nvfp4_gemm_tflops(device)
            if library:
                line["roofline"]["library_nvfp4_gemm_tflops"] = library
                line["roofline"]["frac_of_library_nvfp4_gemm"] = achieved / library
                line["roofline"]["library_note"] = ("comparison only: cuBLASLt block-scaled NVFP4 GEMM, dense "
                                                    "8192^3, timed in this run")
        if ep_phases is not None:
            line["ep_phases_us_rank0"] = ep_phases
        if ep_config4 is not None:
            line["ep_config4"] = ep_config4
        if world == 1 and not args.no_decode:
            line["decode"] = decode_sweep(layer, device, max(args.steps, 20))
        if world == 1 and not args.no_config4:
            line["config4_single_gpu"] = config4_single_gpu(layer, device, max(args.steps, 10))
        if world == 1 and not args.no_config3:
            layer.runner = None
            torch.cuda.empty_cache()
            line["config3"] = config3_stack(device)
        if world == 1 and not args.no_cpu_baseline:
            oracle, x_bits, router_bits, bias, scale_bits, hw = oracle_sample(0, TOKENS)
            time_oracle(oracle, x_bits, router_bits, bias, scale_bits, hw, 128, 1)
            t = time_oracle(oracle, x_bits, router_bits, bias, scale_bits, hw, TOKENS, 1)[0]
            line["cpu_baseline"] = {
                "value": TOKENS / t, "unit": "tokens/s", "cores": oracle.lib.gvo_threads(),
                "nproc": os.cpu_count(), "kind": "port",
                "sample": f"one pass over the whole {TOKENS}-token batch through the CPU oracle after a "
                          "128-token warm-up"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--no-library-compare", action="store_true",
                        help="skip timing the library NVFP4 GEMM that is reported beside the roofline")
    parser.add_argument("--profile-decode", type=int, default=0, metavar="TOKENS",
                        help="run a few eager decode-sized layer steps of TOKENS tokens and exit (for ncu)")
    parser.add_argument("--profile-ep-one-rank", action="store_true",
                        help="for a profiler: eight expert-parallel steps with a process group of one rank")
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-decode", action="store_true", help="skip the decode-size sweep")
    parser.add_argument("--no-config3", action="store_true", help="skip the 30-layer FFN stack record")
    parser.add_argument("--no-config4", action="store_true", help="skip the 16384-token single-GPU record")
    parser.add_argument("--no-sustained", action="store_true",
                        help="skip the two-second loop (for a profiler, which would replay thousands of launches)")
    parser.add_argument("--ep-parts", type=int, default=1,
                        help="micro-batches of a rank's batch in flight in the expert-parallel step "
                             "(measured slower at 2 than at 1 on two GPUs, so 1)")
    parser.add_argument("--no-ep-config4", action="store_true",
                        help="with several GPUs: skip the 16384-token Zipf expert-parallel records")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
