"""Helpers shared by the GPU parity tests: bf16 bit views, error norms, and access to the
128-row x 4-scale interleaved scale-factor layout (reference: src/nvfp4_cutlass.cu:321-323)."""
import numpy as np
import torch

EXPERTS, TOP_K, HIDDEN, INTER = 128, 8, 2816, 704


def bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(a, device):
    return torch.from_numpy(a.view(np.int16).copy()).to(device).view(torch.bfloat16)


def bf16_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def rel_l2(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def sf_offsets(expert_of_row, row_in_expert, scale_rows, groups):
    """Byte offsets [rows, groups] of the scales of the given rows inside an operand's
    scale buffer."""
    r = np.asarray(row_in_expert, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    base = np.asarray(scale_rows, dtype=np.int64)[np.asarray(expert_of_row)][:, None] * groups
    return base + (r // 128) * (128 * groups) + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4


def gather_sf(buffer, expert_of_row, row_in_expert, scale_rows, groups):
    """Row-major scale bytes [rows, groups] of the given rows."""
    return buffer[sf_offsets(expert_of_row, row_in_expert, scale_rows, groups)]


def scatter_sf(row_major, expert_of_row, row_in_expert, scale_rows, groups, size):
    out = np.zeros(size, np.uint8)
    out[sf_offsets(expert_of_row, row_in_expert, scale_rows, groups)] = row_major
    return out


def worst_tile(got, want, expert_of_row, tile_of_row):
    """Largest relative L2 error over (expert, 128-row tile) groups of rows; got/want are
    float arrays [rows, n].  Returns (error, expert, tile, groups seen, highest tile index)."""
    key = np.asarray(expert_of_row, dtype=np.int64) * 100000 + np.asarray(tile_of_row, dtype=np.int64)
    order = np.argsort(key, kind="stable")
    key_sorted = key[order]
    starts = np.flatnonzero(np.r_[True, key_sorted[1:] != key_sorted[:-1]])
    ends = np.r_[starts[1:], key_sorted.size]
    diff = ((got.astype(np.float64) - want.astype(np.float64)) ** 2).sum(1)[order]
    norm = (want.astype(np.float64) ** 2).sum(1)[order]
    worst = (0.0, -1, -1)
    for a, b in zip(starts, ends):
        err = float(np.sqrt(diff[a:b].sum() / max(norm[a:b].sum(), 1e-30)))
        if err > worst[0]:
            worst = (err, int(key_sorted[a] // 100000), int(key_sorted[a] % 100000))
    return worst + (int(starts.size), int(np.max(tile_of_row)))


def random_ids(tokens, seed):
    rng = np.random.default_rng(seed)
    return np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(tokens)]).astype(np.int32)


def skewed_ids(tokens):
    """Route 0 always on expert 0, the rest hashed into experts 1..36 without repeats inside a
    token: few active experts with unequal row counts (the shape of the reference's own
    repeatability-test routing, src/nvfp4_cutlass.cu:1962-1974)."""
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


def dummy_weights(gm, device):
    """All-zero expert tensors with unit scales, for tests that exercise only the stages around
    the GEMMs."""
    z8 = lambda *shape: torch.zeros(shape, dtype=torch.uint8, device=device)
    ones = torch.ones(EXPERTS, dtype=torch.float32, device=device)
    return gm.ExpertWeights(z8(EXPERTS, 2 * INTER, HIDDEN // 2), z8(EXPERTS, 2 * INTER, HIDDEN // 16),
                            z8(EXPERTS, HIDDEN, INTER // 2), z8(EXPERTS, HIDDEN, INTER // 16),
                            ones, ones.clone(), ones.clone(), ones.clone())
