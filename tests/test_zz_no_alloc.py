"""gevva_moe_route_sort_noalloc against the ordinary sort stage.

The no-allocation entry point exists for hosts that cannot call cudaMalloc while the
layer runs: their own arena already owns all device memory, or their serving loop may
not stall on the device-wide synchronisation an allocation implies.  Its
working memory is one fixed array inside the library that every call shares and that
keeps the previous call's contents, so the check runs two calls back to back, the
second smaller than the first, and wants both to equal the runner's own sort exactly
(integers: no tolerance).  Collected last so that a failure here cannot hide another
test's result."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

EXPERTS, TOP_K, HIDDEN, INTER = 128, 8, 2816, 704


def _ids(tokens, seed):
    rng = np.random.default_rng(seed)
    return np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int32)


def _dummy_weights(gm, device):
    z8 = lambda *shape: torch.zeros(shape, dtype=torch.uint8, device=device)
    ones = torch.ones(EXPERTS, dtype=torch.float32, device=device)
    return gm.ExpertWeights(z8(EXPERTS, 2 * INTER, HIDDEN // 2), z8(EXPERTS, 2 * INTER, HIDDEN // 16),
                            z8(EXPERTS, HIDDEN, INTER // 2), z8(EXPERTS, HIDDEN, INTER // 16),
                            ones, ones.clone(), ones.clone(), ones.clone())


def test_noalloc_sort_equals_runner_sort_twice_in_a_row(cuda_device):
    import gevva_b200 as gm
    from gevva_b200 import runtime as rt
    runner = gm.Nvfp4ExpertRunner(_dummy_weights(gm, cuda_device), 4096)
    for tokens, seed in ((4096, 1), (300, 2)):   # multi-block path, then a smaller call
        ids = torch.from_numpy(_ids(tokens, seed)).to(cuda_device)
        routes = tokens * TOP_K
        got = rt.route_sort_noalloc(ids)
        runner.launch_stages(rt.STAGE_SORT, tokens, expert_ids=ids)
        assert runner.last_status() == 0
        assert int(got["status"][0]) == 0
        i32 = torch.int32
        want = {
            "sorted_experts": runner.buffer(rt.BUF_SORTED_EXPERTS, i32)[:routes],
            "sorted_routes": runner.buffer(rt.BUF_SORTED_ROUTES, i32)[:routes],
            "inverse_routes": runner.buffer(rt.BUF_INVERSE_ROUTES, i32)[:routes],
            "expert_offsets": runner.buffer(rt.BUF_EXPERT_OFFSETS, i32)[:EXPERTS + 1],
            "scale_row_offsets": runner.buffer(rt.BUF_SCALE_ROW_OFFSETS, i32)[:EXPERTS + 1],
        }
        for name, tensor in want.items():
            assert torch.equal(got[name], tensor), (tokens, name)


def test_noalloc_sort_single_block_path_and_bad_id(cuda_device):
    from gevva_b200 import runtime as rt
    ids = _ids(16, 3)
    got = rt.route_sort_noalloc(torch.from_numpy(ids).to(cuda_device))
    order = np.argsort(ids.reshape(-1), kind="stable")
    assert (got["sorted_routes"].cpu().numpy() == order).all()
    ids[5, 2] = 200
    got = rt.route_sort_noalloc(torch.from_numpy(ids).to(cuda_device))
    assert int(got["status"][0]) == 1


def test_noalloc_sort_at_its_maximum_size(cuda_device):
    """16384 tokens = 128 chunks of 1024 routes: every histogram row of the fixed array is in use."""
    from gevva_b200 import runtime as rt
    ids = _ids(16384, 4)
    got = rt.route_sort_noalloc(torch.from_numpy(ids).to(cuda_device))
    assert int(got["status"][0]) == 0
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    assert (got["sorted_routes"].cpu().numpy() == order).all()
    assert (got["sorted_experts"].cpu().numpy() == flat[order]).all()
    inverse = np.empty_like(order)
    inverse[order] = np.arange(order.size)
    assert (got["inverse_routes"].cpu().numpy() == inverse).all()
    counts = np.bincount(flat, minlength=EXPERTS)
    assert (got["expert_offsets"].cpu().numpy() == np.r_[0, np.cumsum(counts)]).all()
    assert (got["scale_row_offsets"].cpu().numpy() == np.r_[0, np.cumsum((counts + 127) // 128 * 128)]).all()


def test_noalloc_sort_rejects_sizes_beyond_its_fixed_array(cuda_device):
    import gevva_b200 as gm
    from gevva_b200 import runtime as rt
    ids = torch.zeros((16385, TOP_K), dtype=torch.int32, device=cuda_device)
    with pytest.raises(gm.GevvaMoeError) as info:
        rt.route_sort_noalloc(ids)
    assert info.value.status == -6
