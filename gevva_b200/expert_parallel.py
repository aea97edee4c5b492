"""Expert-parallel MoE layer over the GPUs of one node (one process per GPU).

torch.distributed supplies the process group, the symmetric (peer-mapped) buffers and the
barriers; rows move by stores from the kernels in csrc/ep.cu into peer memory.  The
reference is single-GPU and has no counterpart."""
import ctypes

import torch
import torch.distributed as dist

from .runtime import (EXPERTS, HIDDEN, INTER, TOP_K, W13_OUT, ExpertWeights, GevvaMoeError, _Weights,
                      _check, _ptr, _stream_handle, library)


class _EpConfig(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("max_tokens", ctypes.c_int),
                ("recv_capacity_rows", ctypes.c_size_t),
                ("peer_recv_codes", ctypes.POINTER(ctypes.c_void_p)),
                ("peer_recv_sf", ctypes.POINTER(ctypes.c_void_p)),
                ("peer_combine", ctypes.POINTER(ctypes.c_void_p)),
                ("peer_counts", ctypes.POINTER(ctypes.c_void_p)),
                ("peer_flags", ctypes.POINTER(ctypes.c_void_p)),
                ("placement", ctypes.POINTER(ctypes.c_int))]


def strided_placement(world):
    """placement[e] = owner * (128/world) + local index: expert e on rank e % world at e // world."""
    el = EXPERTS // world
    return [(e % world) * el + e // world for e in range(EXPERTS)]


def balanced_placement(counts, world):
    """Placement from observed per-expert route counts (e.g. of a calibration batch): experts in
    order of decreasing count, each to the least loaded rank that still has a free slot
    (longest-processing-time rule).  Deterministic, so every rank computes the same table."""
    el = EXPERTS // world
    counts = [int(c) for c in counts]
    assert len(counts) == EXPERTS
    load = [0] * world
    members = [[] for _ in range(world)]
    for e in sorted(range(EXPERTS), key=lambda i: (-counts[i], i)):
        rank = min((r for r in range(world) if len(members[r]) < el), key=lambda r: (load[r], r))
        members[rank].append(e)
        load[rank] += counts[e]
    placement = [0] * EXPERTS
    for rank in range(world):
        for index, e in enumerate(sorted(members[rank])):
            placement[e] = rank * el + index
    return placement


def local_expert_weights(full: ExpertWeights, rank: int, world: int, placement=None) -> ExpertWeights:
    """This rank's shard in local-index order: by default experts rank, rank+world, ...;
    with a placement table the experts e with placement[e] // (128/world) == rank."""
    el = EXPERTS // world
    placement = placement or strided_placement(world)
    order = sorted((e for e in range(EXPERTS) if placement[e] // el == rank), key=lambda e: placement[e])
    index = torch.tensor(order, dtype=torch.long, device=full.w13.device)
    pick = lambda t: t.index_select(0, index).contiguous()
    return ExpertWeights(pick(full.w13), pick(full.w13_sf), pick(full.w2), pick(full.w2_sf),
                         pick(full.alpha1), pick(full.alpha2), pick(full.in_scale_q1),
                         pick(full.in_scale_q2))


class ExpertParallelRunner:
    def __init__(self, local_weights: ExpertWeights, in_scale_q1_global: torch.Tensor, max_tokens: int,
                 group=None, placement=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.group = group
        self.device = local_weights.w13.device
        self.max_tokens = max_tokens
        el = EXPERTS // self.world
        _check(local_weights.w13, torch.uint8, (el, W13_OUT, HIDDEN // 2), "w13.weight")
        _check(local_weights.w2, torch.uint8, (el, HIDDEN, INTER // 2), "w2.weight")
        _check(in_scale_q1_global, torch.float32, (EXPERTS,), "g1.input_scale_quant (all experts)")
        self._weights, self._scale_q1 = local_weights, in_scale_q1_global
        routes = max_tokens * TOP_K
        cap = self.world * routes
        align = lambda n: (n + 255) // 256 * 256
        sizes = [align(self.world * EXPERTS * 4), align(cap * (HIDDEN // 2)),
                 align(cap * (HIDDEN // 16)), align(routes * HIDDEN * 2), 256]
        offsets = [0]
        for size in sizes:
            offsets.append(offsets[-1] + size)
        self._buffer = symm_mem.empty(offsets[-1], dtype=torch.uint8, device=self.device)
        self._buffer.zero_()
        self._handle_symm = symm_mem.rendezvous(self._buffer, group.group_name)
        bases = [int(p) for p in self._handle_symm.buffer_ptrs]
        arrays = []
        for region in range(5):
            arr = (ctypes.c_void_p * self.world)(*[b + offsets[region] for b in bases])
            arrays.append(arr)
        self._arrays = arrays
        config = _EpConfig(self.rank, self.world, max_tokens, cap,
                           ctypes.cast(arrays[1], ctypes.POINTER(ctypes.c_void_p)),
                           ctypes.cast(arrays[2], ctypes.POINTER(ctypes.c_void_p)),
                           ctypes.cast(arrays[3], ctypes.POINTER(ctypes.c_void_p)),
                           ctypes.cast(arrays[0], ctypes.POINTER(ctypes.c_void_p)),
                           ctypes.cast(arrays[4], ctypes.POINTER(ctypes.c_void_p)),
                           (ctypes.c_int * EXPERTS)(*placement) if placement is not None else None)
        lib = library()
        vp = ctypes.c_void_p
        lib.gevva_moe_ep_create.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(_Weights), vp,
                                            ctypes.POINTER(_EpConfig)]
        lib.gevva_moe_ep_destroy.argtypes = [vp]
        lib.gevva_moe_ep_destroy.restype = None
        lib.gevva_moe_ep_barrier.argtypes = [vp, vp]
        lib.gevva_moe_ep_route_sort.argtypes = [vp, vp, ctypes.c_int, vp]
        lib.gevva_moe_ep_dispatch.argtypes = [vp, vp, vp, ctypes.c_int, vp]
        lib.gevva_moe_ep_compute.argtypes = [vp, vp]
        lib.gevva_moe_ep_reduce.argtypes = [vp, vp, vp, ctypes.c_int, vp]
        lib.gevva_moe_ep_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int)]
        w = local_weights
        packed = _Weights(*[t.data_ptr() for t in (w.w13, w.w13_sf, w.w2, w.w2_sf, w.alpha1, w.alpha2,
                                                   w.in_scale_q1, w.in_scale_q2)])
        handle = vp()
        with torch.cuda.device(self.device):
            status = lib.gevva_moe_ep_create(ctypes.byref(handle), ctypes.byref(packed),
                                             _ptr(in_scale_q1_global), ctypes.byref(config))
        if status != 0:
            raise GevvaMoeError(status, "ExpertParallelRunner")
        self._handle = handle
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        # GEVVA_EP_NCCL_BARRIER=1 swaps the flag barrier of csrc/ep.cu for an NCCL all-reduce
        import os
        self._nccl_barrier = os.environ.get("GEVVA_EP_NCCL_BARRIER", "0") == "1"
        dist.barrier(group)

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle:
            library().gevva_moe_ep_destroy(handle)
            self._handle = None

    def _barrier(self, stream=None):
        # a collective ordered on the same stream as the phases: no rank's next phase starts
        # before every rank's previous phase (and its stores into peer memory) has finished
        if self._nccl_barrier:
            with torch.cuda.stream(stream if stream is not None else torch.cuda.current_stream()):
                dist.all_reduce(self._flag, group=self.group)
        else:
            self._call("gevva_moe_ep_barrier", _stream_handle(stream))

    def _call(self, name, *args):
        with torch.cuda.device(self.device):
            status = getattr(library(), name)(self._handle, *args)
        if status != 0:
            raise GevvaMoeError(status, name)

    def launch_batch(self, input, expert_ids, route_weights, output, tokens, stream=None):
        """Same contract as Nvfp4ExpertRunner.launch_batch, for this rank's tokens."""
        _check(input, torch.bfloat16, (tokens, HIDDEN), "input")
        _check(expert_ids, torch.int32, (tokens, TOP_K), "expert_ids")
        _check(route_weights, torch.float32, (tokens, TOP_K), "route_weights")
        _check(output, torch.bfloat16, (tokens, HIDDEN), "output")
        s = _stream_handle(stream)
        # route sort + count exchange; the exchange carries the step's first cross-rank barrier
        self._call("gevva_moe_ep_route_sort", _ptr(expert_ids), tokens, s)
        # dispatch ends by announcing its rows; compute starts by waiting for every rank's
        self._call("gevva_moe_ep_dispatch", _ptr(input), _ptr(expert_ids), tokens, s)
        self._call("gevva_moe_ep_compute", s)
        self._barrier(stream)
        self._call("gevva_moe_ep_reduce", _ptr(route_weights), _ptr(output), tokens, s)

    def timed_step(self, input, expert_ids, route_weights, output, tokens):
        """One step with CUDA events between the phases; returns microseconds per phase
        (`route_sort` includes the count exchange and the flag barrier inside it, `compute` the
        wait for every rank's dispatched rows; both include waiting for the slowest rank)."""
        names = ["route_sort", "dispatch", "compute", "barrier", "reduce"]
        events = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        s = _stream_handle(None)
        events[0].record()
        self._call("gevva_moe_ep_route_sort", _ptr(expert_ids), tokens, s)
        events[1].record()
        self._call("gevva_moe_ep_dispatch", _ptr(input), _ptr(expert_ids), tokens, s)
        events[2].record()
        self._call("gevva_moe_ep_compute", s)
        events[3].record()
        self._barrier()
        events[4].record()
        self._call("gevva_moe_ep_reduce", _ptr(route_weights), _ptr(output), tokens, s)
        events[5].record()
        torch.cuda.synchronize()
        return {n: events[i].elapsed_time(events[i + 1]) * 1e3 for i, n in enumerate(names)}

    def status(self):
        rows = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            status = library().gevva_moe_ep_status(self._handle, ctypes.byref(rows))
        return status, rows.value


class MicroBatchedExpertParallel:
    """The same layer with a rank's batch cut into `parts` micro-batches (two by default), each
    with an ExpertParallelRunner of its own (own peer buffers and flags) on a stream of its own.

    The phases of a step alternate between the NVLink (dispatch, the w2 epilogue's stores) and the
    SMs (sort, w13); one batch leaves each idle half of the time.  Two micro-batches in flight fill
    the gaps: while one streams its results to the peers the other computes.  Every token's result
    is what the single runner gives, bit for bit: a sorted row's arithmetic does not depend on
    which rows share its tile.  `launch_batch` returns with the caller's stream waiting for all
    micro-batches, so a step is still a step.

    Measured on two B200s at 4096 tokens per GPU: 0.434 ms per step with two micro-batches against
    0.394 ms with one (every fixed cost of a step is paid twice and the persistent GEMM launches
    of the two streams take turns on the SMs rather than sharing them), so the plain runner is
    what the benchmark uses; this class is kept as the tested way to run it."""

    def __init__(self, local_weights: ExpertWeights, in_scale_q1_global: torch.Tensor, max_tokens: int,
                 group=None, placement=None, parts: int = 2):
        if parts < 1:
            raise ValueError("parts: at least one micro-batch")
        self.parts = parts
        self.max_tokens = max_tokens
        self._share = (max_tokens + parts - 1) // parts
        self._runners = [ExpertParallelRunner(local_weights, in_scale_q1_global, self._share, group, placement)
                         for _ in range(parts)]
        self.device = self._runners[0].device
        self.rank, self.world = self._runners[0].rank, self._runners[0].world
        self._streams = [torch.cuda.Stream(device=self.device) for _ in range(parts)]

    def launch_batch(self, input, expert_ids, route_weights, output, tokens, stream=None):
        """Same contract as ExpertParallelRunner.launch_batch."""
        _check(input, torch.bfloat16, (tokens, HIDDEN), "input")
        _check(expert_ids, torch.int32, (tokens, TOP_K), "expert_ids")
        _check(route_weights, torch.float32, (tokens, TOP_K), "route_weights")
        _check(output, torch.bfloat16, (tokens, HIDDEN), "output")
        if tokens > self.max_tokens:
            raise GevvaMoeError(-3, "MicroBatchedExpertParallel.launch_batch")
        caller = stream if stream is not None else torch.cuda.current_stream(self.device)
        # every rank must run the same number of micro-batches (their barriers pair up), so the
        # cut depends on the capacity only, and ranks are expected to bring equal token counts
        share = (tokens + self.parts - 1) // self.parts
        ready = caller.record_event()
        first = 0
        for runner, side in zip(self._runners, self._streams):
            count = min(share, tokens - first)
            if count <= 0:
                break
            side.wait_event(ready)
            rows = slice(first, first + count)
            runner.launch_batch(input[rows], expert_ids[rows], route_weights[rows], output[rows], count, side)
            caller.wait_event(side.record_event())
            first += count

    def status(self):
        worst, rows = 0, 0
        for runner in self._runners:
            status, received = runner.status()
            worst = worst or status
            rows += received
        return worst, rows
