"""Expert-parallel layer on 2 (or more) GPUs against the single-GPU runner.

Every rank also holds the full expert set, runs its own tokens through the ordinary runner
and wants the expert-parallel result to be the same bits: rows are quantised with the same
static scales, each row's GEMM result does not depend on its neighbours, and the weighted
reduce runs in the same route order.  Needs >= 2 GPUs; run by hand on a multi-GPU box."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

EXPERTS, TOP_K, HIDDEN, INTER = 128, 8, 2816, 704


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    device = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import gevva_b200 as gm
        from gevva_b200.expert_parallel import ExpertParallelRunner, local_expert_weights
        from tests import hashgen
        out = {k: [] for k in ("w13", "w13_sf", "g13", "w2", "w2_sf", "g2")}
        for first in range(0, EXPERTS, 16):
            w13 = hashgen.expert_weights_chunk(first, 16, 2 * INTER, HIDDEN, 11, device)
            c, s, g = gm.pack_experts(w13)
            out["w13"].append(c), out["w13_sf"].append(s), out["g13"].append(g)
            del w13
            w2 = hashgen.expert_weights_chunk(first, 16, HIDDEN, INTER, 12, device)
            c, s, g = gm.pack_experts(w2)
            out["w2"].append(c), out["w2_sf"].append(s), out["g2"].append(g)
            del w2
        p = {k: torch.cat(v) for k, v in out.items()}
        s1, s2 = 4.0 / 2688.0, 16.0 / 2688.0
        # per-expert scales that differ, so a mix-up of expert indices cannot go unnoticed
        wobble = 1.0 + 0.01 * torch.arange(EXPERTS, device=device, dtype=torch.float32)
        full = gm.ExpertWeights(p["w13"], p["w13_sf"], p["w2"], p["w2_sf"],
                                (p["g13"] * s1 * wobble).contiguous(), (p["g2"] * s2 * wobble).contiguous(),
                                (1.0 / (s1 * wobble)).contiguous(), (1.0 / (s2 * wobble)).contiguous())
        for round_index, base_tokens in enumerate((300, 45)):
            tokens = base_tokens + 37 * rank   # ragged across ranks
            x = hashgen.activations(tokens, HIDDEN, 900 + rank + 10 * round_index, device)
            router_w = (hashgen.hash_uniform(EXPERTS * HIDDEN, 5, device) * 0.0346).view(EXPERTS, HIDDEN)
            logits = (x.float() @ router_w.t()).to(torch.bfloat16)
            rw, ids = gm.route_128_top8(logits, torch.ones(EXPERTS, dtype=torch.bfloat16, device=device))
            single = gm.Nvfp4ExpertRunner(full, 512)
            want = torch.empty_like(x)
            single.launch_batch(x, ids, rw, want, tokens)
            single.check()
            if round_index == 0:
                ep = ExpertParallelRunner(local_expert_weights(full, rank, world), full.in_scale_q1, 512)
            got = torch.empty_like(x)
            ep.launch_batch(x, ids, rw, got, tokens)
            status, rows = ep.status()
            assert status == 0, status
            total = torch.tensor([rows, tokens * TOP_K], device=device)
            dist.all_reduce(total)
            assert int(total[0]) == int(total[1]), "rows received != routes sent"
            assert torch.equal(got, want), f"rank {rank} round {round_index}: " \
                f"{(got != want).sum().item()} of {got.numel()} elements differ"
        # the same batch with experts placed by observed load instead of e % world
        from gevva_b200.expert_parallel import balanced_placement
        counts = torch.bincount(ids.reshape(-1).long(), minlength=EXPERTS)
        dist.all_reduce(counts)
        placement = balanced_placement(counts.tolist(), world)
        assert placement != [(e % world) * (EXPERTS // world) + e // world for e in range(EXPERTS)]
        placed = ExpertParallelRunner(local_expert_weights(full, rank, world, placement), full.in_scale_q1, 512,
                                      placement=placement)
        got = torch.empty_like(x)
        placed.launch_batch(x, ids, rw, got, tokens)
        status, rows = placed.status()
        assert status == 0, status
        assert torch.equal(got, want), f"rank {rank} balanced placement: {(got != want).sum().item()} differ"
        # the same step enqueued on a stream that is not the current one: phases and barriers
        # must all be ordered on that stream
        other = torch.cuda.Stream(device=device)
        got = torch.zeros_like(x)
        other.wait_stream(torch.cuda.current_stream())
        placed.launch_batch(x, ids, rw, got, tokens, stream=other)
        torch.cuda.current_stream().wait_stream(other)
        status, rows = placed.status()
        assert status == 0, status
        assert torch.equal(got, want), f"rank {rank} explicit stream: {(got != want).sum().item()} differ"
        # two micro-batches in flight on two streams, each with peer buffers of its own: the same bits,
        # also when the step is repeated back to back
        from gevva_b200.expert_parallel import MicroBatchedExpertParallel
        halves = MicroBatchedExpertParallel(local_expert_weights(full, rank, world, placement), full.in_scale_q1,
                                            512, placement=placement)
        for repeat in range(3):
            got = torch.zeros_like(x)
            halves.launch_batch(x, ids, rw, got, tokens)
            status, rows = halves.status()
            assert status == 0, status
            assert rows > 0
            assert torch.equal(got, want), f"rank {rank} micro-batches, repeat {repeat}: " \
                f"{(got != want).sum().item()} differ"
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_expert_parallel_equals_single_gpu(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if world == 3:
        world = 2
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, 29731, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
