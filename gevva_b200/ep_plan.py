"""Host mirror (numpy) of the expert-parallel bookkeeping done on the device in csrc/ep.cu.

Given the all-gathered count matrix counts[s, v] (routes of source rank s for virtual expert
v = owner * EL + local_expert), these functions say where every row goes; the CUDA kernels
ep_exchange_kernel (send tables, receive tables, compute parts) and ep_row_destinations_kernel
(combine destinations) compute the same numbers.  Used by the CPU (gloo) tests of the
multi-rank path."""
import numpy as np

EXPERTS = 128
TILE = 128


def remap(world, placement=None):
    """expert id e -> virtual id v = owner * EL + local index: by default owner e % world and
    local index e // world, else the given placement table."""
    if placement is not None:
        return np.asarray(placement, dtype=np.int64)
    e = np.arange(EXPERTS)
    return (e % world) * (EXPERTS // world) + e // world


def send_tables(counts, rank):
    """For source `rank`: per v, first receive row on the owner, rows of lower sources in the
    same expert, and the owner's scale-row offset of that expert."""
    world = counts.shape[0]
    el = EXPERTS // world
    totals = counts.sum(0)
    row_base = np.zeros(EXPERTS, np.int64)
    src_prefix = counts[:rank].sum(0)
    scale_rows = np.zeros(EXPERTS, np.int64)
    for v in range(EXPERTS):
        first = (v // el) * el
        row_base[v] = totals[first:v].sum() + src_prefix[v]
        scale_rows[v] = (((totals[first:v] + TILE - 1) // TILE) * TILE).sum()
    return row_base, src_prefix, scale_rows


def receive_tables(counts, rank):
    """For owner `rank`: expert_offsets[EL+1] of its receive buffer and, per (source, local
    expert), the source's own sorted position of the first row it sent."""
    world = counts.shape[0]
    el = EXPERTS // world
    mine = counts[:, rank * el:(rank + 1) * el]
    offsets = np.concatenate([[0], np.cumsum(mine.sum(0))])
    source_offsets = np.zeros((world, el), np.int64)
    for s in range(world):
        prefix = np.concatenate([[0], np.cumsum(counts[s])])
        source_offsets[s] = prefix[rank * el:(rank + 1) * el]
    return offsets, source_offsets


def combine_destination(counts, rank, row):
    """(source rank, row in the source's sorted order) of receive row `row` on owner `rank`."""
    world = counts.shape[0]
    el = EXPERTS // world
    offsets, source_offsets = receive_tables(counts, rank)
    le = int(np.searchsorted(offsets, row, side="right") - 1)
    within = row - offsets[le]
    v = rank * el + le
    for s in range(world):
        if within < counts[s, v]:
            return s, int(source_offsets[s, le] + within)
        within -= counts[s, v]
    raise ValueError("row beyond the received rows")


def default_first_share(world):
    """Percent of an owner's row tiles in the first of its two compute parts, as gevva_moe_ep_create
    chooses it: the first part's result rows cross NVLink while the second part's w13 runs, and the
    more ranks there are, the larger the share of rows that must cross."""
    return 40 if world >= 8 else 44 if world >= 4 else 54 if world >= 2 else 50


def compute_parts(counts, rank, first_share=None):
    """The two parts of owner `rank`'s compute phase as (first tile, tile count) pairs: the tile
    list is cut at the first local expert, after the first, whose first tile t satisfies
    100 * t >= first_share * tiles; without such an expert the first part takes everything."""
    world = counts.shape[0]
    el = EXPERTS // world
    share = default_first_share(world) if first_share is None else first_share
    rows = counts[:, rank * el:(rank + 1) * el].sum(0)
    tiles = (rows + TILE - 1) // TILE
    first_tile = np.concatenate([[0], np.cumsum(tiles)])
    total = int(first_tile[-1])
    cut = total
    for e in range(1, el):
        if 100 * int(first_tile[e]) >= share * total:
            cut = int(first_tile[e])
            break
    return [(0, cut), (cut, total - cut)]
