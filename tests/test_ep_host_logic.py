"""Multi-rank bookkeeping of the expert-parallel path, on CPU ranks (gloo, world sizes 2
and 4): counts are all-gathered, every rank derives its send/receive tables
(gevva_b200/ep_plan.py, the host mirror of csrc/ep.cu), rows are exchanged, and the receive
layout must equal one global stable sort by (owner, local expert, source rank, source order);
the combine step must bring every row back to its source position."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

EXPERTS, TOP_K = 128, 8


def _ids(tokens, seed):
    rng = np.random.default_rng(seed)
    return np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int64)


def _worker(rank, world, port, tokens, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gevva_b200 import ep_plan
    try:
        remap = ep_plan.remap(world)
        el = EXPERTS // world
        ids = _ids(tokens + rank, 100 + rank)            # ragged: ranks hold different token counts
        v = remap[ids.reshape(-1)]
        order = np.argsort(v, kind="stable")             # this rank's sorted routes
        counts_local = np.bincount(v, minlength=EXPERTS)
        gathered = [torch.zeros(EXPERTS, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts_local))
        counts = torch.stack(gathered).numpy()
        row_base, src_prefix, _ = ep_plan.send_tables(counts, rank)
        offsets_v = np.concatenate([[0], np.cumsum(counts_local)])
        # every route as a tagged payload (source rank, source route index)
        sends = []
        for pos, route in enumerate(order):
            vv = int(v[route])
            j = pos - offsets_v[vv]
            sends.append((vv // el, int(row_base[vv] + j), rank, int(route)))
        everything = [None] * world
        dist.all_gather_object(everything, sends)
        total = int(counts[:, rank * el:(rank + 1) * el].sum())
        recv = [None] * total
        for src_sends in everything:
            for owner, row, src, route in src_sends:
                if owner == rank:
                    assert recv[row] is None, "two routes landed on one receive row"
                    recv[row] = (src, route)
        assert all(r is not None for r in recv)
        # expected layout: stable sort by (local expert, source rank, source sorted order)
        all_ids = [None] * world
        dist.all_gather_object(all_ids, ids)
        expected = []
        for le in range(el):
            for src in range(world):
                vsrc = remap[all_ids[src].reshape(-1)]
                expected += [(src, int(r)) for r in np.nonzero(vsrc == rank * el + le)[0]]
        assert recv == expected
        # combine: every receive row returns to the sorted position its source gave it
        for row, (src, route) in enumerate(recv):
            s, dst = ep_plan.combine_destination(counts, rank, row)
            assert s == src
            vsrc = remap[all_ids[src].reshape(-1)]
            src_order = np.argsort(vsrc, kind="stable")
            assert src_order[dst] == route
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens", [(2, 9), (4, 33)])
def test_dispatch_and_combine_bookkeeping(tmp_path, world, tokens):
    port = 29650 + world
    mp.spawn(_worker, args=(world, port, tokens, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_balanced_placement_is_a_permutation_and_balances():
    from gevva_b200 import ep_plan
    from gevva_b200.expert_parallel import balanced_placement, strided_placement
    rng = np.random.default_rng(3)
    counts = (1000 * rng.pareto(1.2, EXPERTS)).astype(np.int64) + 1
    for world in (1, 2, 4, 8):
        el = EXPERTS // world
        placement = balanced_placement(counts.tolist(), world)
        assert sorted(placement) == list(range(EXPERTS))
        load = lambda table: max(sum(int(counts[e]) for e in range(EXPERTS) if table[e] // el == r)
                                 for r in range(world))
        assert load(placement) <= load(strided_placement(world))
        assert (ep_plan.remap(world, placement) == np.asarray(placement)).all()
        assert (ep_plan.remap(world) == np.asarray(strided_placement(world))).all()



@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_compute_parts_cover_the_tiles_and_cut_at_an_expert(world):
    """The two parts of the compute phase: together every tile once, the cut on an expert boundary,
    the first part the smallest run of experts that reaches its share."""
    from gevva_b200 import ep_plan
    rng = np.random.default_rng(40 + world)
    el = ep_plan.EXPERTS // world
    for trial in range(20):
        counts = rng.integers(0, 700, size=(world, ep_plan.EXPERTS))
        if trial % 5 == 0:
            counts[:, rng.integers(0, ep_plan.EXPERTS, size=40)] = 0   # experts without rows
        for rank in range(world):
            rows = counts[:, rank * el:(rank + 1) * el].sum(0)
            tiles = (rows + 127) // 128
            starts = np.concatenate([[0], np.cumsum(tiles)])
            (a0, n0), (a1, n1) = ep_plan.compute_parts(counts, rank)
            assert a0 == 0 and a1 == n0 and n0 + n1 == starts[-1]
            assert n0 in set(starts.tolist())
            share = ep_plan.default_first_share(world)
            if n0 < starts[-1]:
                assert 100 * n0 >= share * starts[-1]
                earlier = [t for t in starts[1:el].tolist() if t < n0]
                assert all(100 * t < share * starts[-1] for t in earlier)
    assert [ep_plan.default_first_share(w) for w in (1, 2, 4, 8)] == [50, 54, 44, 40]
