"""Host mirror of the persistent GEMM kernels' work distribution (work_item in
gevva_b200/csrc/grouped_gemm.cu): every (row tile, weight tile) item is taken by exactly one
CTA, in both item numberings, and the cost-sorted numbering balances a decode-sized launch."""
import pytest


def work_items(cta, grid, m_tiles, n_tiles, fused_wide):
    total = m_tiles * n_tiles
    rounds = (total + grid - 1) // grid
    for r in range(rounds):
        slot = grid - 1 - cta if r & 1 else cta
        index = r * grid + slot
        if index >= total:
            continue
        if fused_wide and total <= 8 * grid:
            full = m_tiles * (n_tiles - 1)
            if index < full:
                yield index // (n_tiles - 1), index % (n_tiles - 1)
            else:
                yield index - full, n_tiles - 1
        else:
            yield index // n_tiles, index % n_tiles


@pytest.mark.parametrize("m_tiles,n_tiles,fused", [(128, 6, True), (1, 6, True), (8, 6, True), (320, 6, True),
                                                   (197, 6, True), (198, 6, True), (320, 11, False),
                                                   (1, 11, False), (0, 6, True), (128, 11, False)])
def test_every_item_once(m_tiles, n_tiles, fused):
    grid = 148
    seen = {}
    for cta in range(grid):
        for item in work_items(cta, grid, m_tiles, n_tiles, fused):
            assert item not in seen, item
            seen[item] = cta
    assert len(seen) == m_tiles * n_tiles
    assert all(0 <= m < m_tiles and 0 <= n < n_tiles for m, n in seen)


def test_decode_sized_launch_is_balanced():
    """128 experts x (5 full + 1 half item): no CTA carries more than 5 units of weight bytes
    (the mean is 4.76); plain round-robin over (tile, item) order reaches 5.5."""
    grid, m_tiles, n_tiles = 148, 128, 6
    cost = lambda n: 0.5 if n == n_tiles - 1 else 1.0
    loads = [sum(cost(n) for _, n in work_items(cta, grid, m_tiles, n_tiles, True)) for cta in range(grid)]
    assert max(loads) <= 5.0 and abs(sum(loads) - 128 * 5.5) < 1e-9
    naive = [0.0] * grid
    for index in range(m_tiles * n_tiles):
        naive[index % grid] += cost(index % n_tiles)
    assert max(naive) > max(loads)
