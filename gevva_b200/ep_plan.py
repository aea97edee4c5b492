"""Host mirror (numpy) of the expert-parallel bookkeeping done on the device in csrc/ep.cu.

Given the all-gathered count matrix counts[s, v] (routes of source rank s for virtual expert
v = owner * EL + local_expert), these functions say where every row goes; the CUDA kernels
ep_send_bases_kernel / ep_receive_plan_kernel / ep_combine_kernel compute the same numbers.
Used by the CPU (gloo) tests of the multi-rank path."""
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
