"""Benchmark of the NVFP4 MoE layer (Gemma-4 26B-A4B shapes) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the layer over one batch: router projection (library GEMM,
as in the reference), route_128_top8, route sort, NVFP4 quantise, grouped w13 GEMM with
GeGLU+requantise in its epilogue, grouped w2 GEMM, weighted reduce.  Workload at every N: the
prefill configuration, 4096 tokens per GPU with a per-expert router bias ~N(0, 0.5).
Prints one JSON line (rank 0).
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
HIDDEN, EXPERTS, TOP_K, INTER = 2816, 128, 8, 704
FLOP_PER_TOKEN = TOP_K * (2 * 2 * INTER * HIDDEN + 2 * HIDDEN * INTER)  # 95 158 272
W13_FLOP_PER_TOKEN = TOP_K * 2 * 2 * INTER * HIDDEN                      # 63 438 848
LAYER_WEIGHT_BYTES = 428212224
NOMINAL_FP4_TFLOPS = 9000.0
# fused w13 launch at 4096 tokens: weights + weight scales + operand codes/scales + output codes/scales
W13_ALGORITHMIC_BYTES = 128 * (1982464 + 247808) + 32768 * (1408 + 176) + 32768 * (352 + 44)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch (ncu capture summarised under profiles/)
W13_DRAM_TRAFFIC_BYTES = 342586368 + 12649216
# DRAM bytes of one layer step at 4096 tokens: the two GEMMs as measured by ncu (profiles/), the
# quantiser (23 MB read + 52 MB written) and the reduce (185 MB read + 23 MB written) by their
# algorithmic bytes, which their kernels move once
LAYER_DRAM_BYTES = (342586368 + 12649216) + (156119808 + 134346240) + 75000000 + 207600000
WORKLOAD = "prefill_4096_tokens_router_bias_N(0,0.5)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
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
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_layer(device, rank):
    """Same experts, router and static scales on every rank (seed 0, calibrated on one fixed
    batch); each rank then gets its own input batch."""
    import torch
    from gevva_b200.synthetic import SyntheticLayer
    layer = SyntheticLayer(seed=0, max_tokens=TOKENS, device=device, bias_std=0.5)
    layer.calibrate(layer.inputs(TOKENS, seed=1000))
    return layer, layer.inputs(TOKENS, seed=1000 + rank)


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
    """The timed unit: router projection with bias (one library GEMM) + our kernels.  With more
    than one GPU the experts are sharded and `layer.ep` exchanges rows over NVLink."""
    import torch
    import gevva_b200
    layer.route(x, weights=weights, ids=ids)
    runner = layer.ep if getattr(layer, "ep", None) is not None else layer.runner
    runner.launch_batch(x, ids, weights, out, x.shape[0])


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
        # One CUDA graph per batch: the layer's launches allocate nothing and never touch the
        # host, so they capture as they stand (the reference captures its decode loop too,
        # src/cuda/runtime/verifier.cuh:1058-1078).
        for x in pool:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step(x)
            graphs.append(graph)
        for graph in graphs[:4]:
            graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            graphs[i % len(graphs)].replay()
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / steps
        d = sum(distinct) / len(distinct)
        algorithmic = d * 3345408 + 720896 + 2 * tokens * HIDDEN * 2
        gbs = algorithmic / (us * 1e-6) / 1e9
        rows.append({"tokens": tokens, "us_per_layer": us, "distinct_experts": d,
                     "algorithmic_bytes": algorithmic, "hbm_gbs": gbs,
                     "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"]),
                     "frac_of_8000_gbs": gbs / 8000.0, "tokens_per_s": tokens / (us * 1e-6),
                     "launch": "CUDA graph replay, 6 kernels per layer"})
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


def oracle_sample(rank_seed, tokens):
    """Synthetic inputs for the CPU legs, generated without a GPU."""
    import numpy as np
    import torch
    from tests.oracle_api import Oracle
    oracle = Oracle()
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
    bias = torch.randn(EXPERTS, generator=gen) * 0.5
    logits = (x.float() @ router.float().t() + bias).to(torch.bfloat16)

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
    return oracle, bits(x), bits(logits), scale, weights


def time_oracle(oracle, x_bits, logit_bits, scale_bits, weights, repeats):
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        rw, ids = oracle.route(logit_bits, scale_bits)
        oracle.moe_layer(x_bits, ids, rw, weights)
        times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    """The reference has no CPU path and its GPU kernels are SM120-only, so this arm
    times the CPU oracle (a restatement: dequantise to fp32, then matmul) with all the
    host threads OpenMP gives it, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 256
    oracle, x_bits, logit_bits, scale_bits, weights = oracle_sample(0, sample)
    threads = oracle.lib.gvo_threads()
    time_oracle(oracle, x_bits, logit_bits, scale_bits, weights, max(1, min(args.warmup, 1)))
    times = time_oracle(oracle, x_bits, logit_bits, scale_bits, weights, args.steps)
    per_step = sum(times) / len(times)
    value = sample / per_step
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": sample,
                   "note": "CPU oracle port; each step is a 256-token sample of the 4096-token batch"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} of {TOKENS} tokens, all 128 experts' weights"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import gevva_b200
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

    layer, x = build_layer(device, rank)
    layer.ep = None
    if args.profile_decode:
        decode_eager(layer, device, args.profile_decode, 6)
        if rank == 0:
            print(json.dumps({"profile_decode_tokens": args.profile_decode, "steps": 6}), flush=True)
        return
    if world > 1:
        from gevva_b200.expert_parallel import (ExpertParallelRunner, balanced_placement,
                                                local_expert_weights)
        # Experts are placed by load observed on a calibration batch (other tokens than the timed
        # ones, same router): most loaded first, each to the least loaded rank with a free slot.
        calibration = layer.inputs(TOKENS, seed=2000 + rank)
        _, calibration_ids = layer.route(calibration)
        counts = torch.bincount(calibration_ids.reshape(-1).long(), minlength=EXPERTS)
        dist.all_reduce(counts)
        placement = balanced_placement(counts.tolist(), world)
        layer.ep = ExpertParallelRunner(local_expert_weights(layer.weights, rank, world, placement),
                                        layer.weights.in_scale_q1, TOKENS, placement=placement)
    out = torch.empty_like(x)
    weights = torch.empty((TOKENS, TOP_K), dtype=torch.float32, device=device)
    ids = torch.empty((TOKENS, TOP_K), dtype=torch.int32, device=device)

    def check():
        if layer.ep is not None:
            status, _ = layer.ep.status()
            if status != 0:
                raise RuntimeError(f"expert-parallel device status {status}")
        layer.runner.check()

    for _ in range(max(args.warmup, 3)):
        layer_step(layer, x, out, weights, ids)
    check()

    # ---- device-resident throughput ("value") -----------------------------------
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        layer_step(layer, x, out, weights, ids)
    stop.record()
    barrier()
    clocks = sampler.stop()
    elapsed_ms = start.elapsed_time(stop)
    check()

    # ---- end to end through host buffers ("e2e") -------------------------------
    # Every step copies its 4096-token batch from pinned host memory and its result back.
    # Three streams, two buffers: the copy-in of step i+1 and the copy-out of step i-1 run
    # beside the layer of step i (PCIe is full duplex); everything is inside the timed region.
    host_in = x.cpu().pin_memory()
    host_out = [torch.empty_like(host_in).pin_memory() for _ in range(2)]
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
                dev_in[b].copy_(host_in, non_blocking=True)
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

    # ---- dominant kernel (grouped w13 GEMM) timed alone inside full steps --------------
    g0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    g1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    h0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    h1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    runner = layer.runner
    for i in range(args.steps):
        layer.route(x, weights=weights, ids=ids)
        runner.launch_stages(rt.STAGE_SORT | rt.STAGE_QUANTIZE, TOKENS, input=x, expert_ids=ids)
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
    if layer.ep is not None:
        samples = [layer.ep.timed_step(x, ids, weights, out, TOKENS) for _ in range(5)]
        ep_phases = {k: sum(s[k] for s in samples[1:]) / (len(samples) - 1) for k in samples[0]}

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        fp4_peak = 4.0 * float(peaks["bf16_tflops"])
        achieved = W13_FLOP_PER_TOKEN * TOKENS / (w13_ms * 1e-3) / 1e12
        total_tokens = TOKENS * world * args.steps
        value = total_tokens / (elapsed_ms * 1e-3)
        # our kernels per step.  Single GPU: route, sort, quantise, w13 (+GeGLU), w2, reduce.
        # Expert parallel: route, sort, publish counts, 3 barriers, send bases, dispatch, receive
        # plan, scale swizzle, row destinations, w13, w2, reduce.
        launches_per_step = 6 if world == 1 else 14
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "experts": EXPERTS,
                       "top_k": TOP_K, "hidden": HIDDEN, "expert_width": INTER,
                       "parallelism": "single GPU" if world == 1 else
                       f"expert parallel x{world}: 128/{world} experts per GPU placed by the load of a "
                       "calibration batch, tokens data-parallel, "
                       "dispatch/combine by stores into peer memory over NVLink",
                       "l2": "inputs larger than L2: 428 MB of expert weights stream every step"},
            "layer_tflops": FLOP_PER_TOKEN * TOKENS / (elapsed_ms / args.steps * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "kernel": "grouped_nvfp4_gemm_kernel<kGeglu> (w13 + GeGLU + requantise)",
                         "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                         "frac": achieved / fp4_peak,
                         # dram__bytes_read + dram__bytes_write of one launch, ncu capture of this workload
                         "traffic": W13_DRAM_TRAFFIC_BYTES, "algorithmic_bytes": W13_ALGORITHMIC_BYTES,
                         "peak_source": f"4 x bf16_tflops of MEASURED_PEAKS.json ({peak_kind}); "
                                        "no FP4 entry exists",
                         "frac_of_nominal_9000": achieved / NOMINAL_FP4_TFLOPS,
                         "measured_on": "this GPU's own 4096-token batch through the single-GPU stages",
                         "kernel_ms": w13_ms, "w2_kernel_ms": w2_ms,
                         "w2_tflops": (FLOP_PER_TOKEN - W13_FLOP_PER_TOKEN) * TOKENS / (w2_ms * 1e-3) / 1e12},
            "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": TOKENS * HIDDEN * 2, "d2h_bytes_per_step": TOKENS * HIDDEN * 2},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if world == 1:
            step_seconds = elapsed_ms / args.steps * 1e-3
            line["layer_hbm"] = {
                "bytes_per_step": LAYER_DRAM_BYTES, "achieved_gbs": LAYER_DRAM_BYTES / step_seconds / 1e9,
                "peak_gbs": float(peaks["hbm_gbs"]),
                "frac": LAYER_DRAM_BYTES / step_seconds / 1e9 / float(peaks["hbm_gbs"]),
                "note": "whole layer step against the measured copy bandwidth: at 4096 tokens the layer "
                        "moves about 1 GB for 390 GFLOP, below the machine balance of the FP4 tensor pipe"}
        if world == 1 and not args.no_library_compare:
            library = library_nvfp4_gemm_tflops(device)
            if library:
                line["roofline"]["library_nvfp4_gemm_tflops"] = library
                line["roofline"]["frac_of_library_nvfp4_gemm"] = achieved / library
                line["roofline"]["library_note"] = ("comparison only: cuBLASLt block-scaled NVFP4 GEMM, dense "
                                                    "8192^3, timed in this run")
        if ep_phases is not None:
            line["ep_phases_us_rank0"] = ep_phases
        if world == 1 and not args.no_decode:
            line["decode"] = decode_sweep(layer, device, max(args.steps, 20))
        if world == 1 and not args.no_cpu_baseline:
            sample = 128
            oracle, x_bits, logit_bits, scale_bits, hw = oracle_sample(0, sample)
            t = time_oracle(oracle, x_bits, logit_bits, scale_bits, hw, 2)[-1]
            line["cpu_baseline"] = {
                "value": sample / t, "unit": "tokens/s", "cores": oracle.lib.gvo_threads(),
                "kind": "port",
                "sample": f"{sample} of {TOKENS} tokens through the CPU oracle, all 128 experts' weights"}
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
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-decode", action="store_true", help="skip the decode-size sweep")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
