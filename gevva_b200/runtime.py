"""ctypes binding of libgevva_moe.so and the Python mirror of the reference operator.

Names, argument meaning and error behaviour follow the reference class
``gevva::Nvfp4ExpertRunner`` (include/gevva/gpu.hpp:217-247): the constructor
takes the layer's expert tensors and a token capacity, optionally sharing scratch
with another runner; ``launch`` / ``launch_batch`` / ``launch_batch_unreduced``
enqueue on a stream; ``routed_output`` / ``inverse_routes`` expose runner-owned
results; failures raise (``GevvaMoeError`` here, ``std::runtime_error`` there).
"""
import ctypes
import os
from dataclasses import dataclass

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgevva_moe.so")
_lib = None

EXPERTS = 128
TOP_K = 8
HIDDEN = 2816
INTER = 704
W13_OUT = 2 * INTER

STAGE_SORT, STAGE_QUANTIZE, STAGE_W13, STAGE_GEGLU, STAGE_W2, STAGE_REDUCE = 1, 2, 4, 8, 16, 32
STAGE_ALL = 63
STAGE_UNFUSED = 64  # keep W13 and GEGLU as two kernels (bf16 w13 output materialised)

BUF_INPUT_CODES, BUF_INPUT_SF, BUF_W13_OUT, BUF_INTER_CODES, BUF_INTER_SF, BUF_W2_OUT = range(6)
(BUF_SORTED_EXPERTS, BUF_SORTED_ROUTES, BUF_INVERSE_ROUTES, BUF_EXPERT_OFFSETS,
 BUF_SCALE_ROW_OFFSETS, BUF_TILE_EXPERT, BUF_NUM_TILES) = range(6, 13)


class GevvaMoeError(RuntimeError):
    """Raised where the reference throws std::runtime_error."""

    def __init__(self, status, where):
        self.status = status
        text = library().gevva_moe_strerror(status).decode()
        super().__init__(f"{where}: {text} ({status})")


class _Options(ctypes.Structure):
    _fields_ = [("flags", ctypes.c_uint32), ("reserved", ctypes.c_uint32 * 7)]


OPTION_NVTX = 1
OPTION_PAIRS = 2
OPTION_W13_PAIRS = 4


class _Weights(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in
                ("w13", "w13_sf", "w2", "w2_sf", "alpha1", "alpha2", "in_scale_q1", "in_scale_q2")]


def library():
    """Loads libgevva_moe.so; there is no fallback when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m gevva_b200.build` "
            "(needs nvcc; the MoE path has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i32, u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
    lib.gevva_moe_create.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(_Weights), i32, vp, vp]
    lib.gevva_moe_create.restype = i32
    lib.gevva_moe_destroy.argtypes = [vp]
    lib.gevva_moe_destroy.restype = None
    lib.gevva_moe_route.argtypes = [vp, i32, vp, vp, vp, i32, vp, vp, vp]
    lib.gevva_moe_route.restype = i32
    lib.gevva_moe_launch.argtypes = [vp, vp, vp, vp, vp, i32, vp]
    lib.gevva_moe_launch.restype = i32
    lib.gevva_moe_launch_stages.argtypes = [vp, vp, vp, vp, vp, i32, u32, vp]
    lib.gevva_moe_launch_stages.restype = i32
    lib.gevva_moe_routed_output.argtypes = [vp]
    lib.gevva_moe_routed_output.restype = vp
    lib.gevva_moe_inverse_routes.argtypes = [vp]
    lib.gevva_moe_inverse_routes.restype = vp
    lib.gevva_moe_last_status.argtypes = [vp]
    lib.gevva_moe_last_status.restype = i32
    lib.gevva_moe_strerror.argtypes = [i32]
    lib.gevva_moe_strerror.restype = ctypes.c_char_p
    lib.gevva_moe_buffer.argtypes = [vp, i32, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    lib.gevva_moe_buffer.restype = i32
    lib.gevva_moe_pack_experts.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp]
    lib.gevva_moe_pack_experts.restype = i32
    _lib = lib
    return lib


def _stream_handle(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    if isinstance(stream, int):
        return ctypes.c_void_p(stream)
    return ctypes.c_void_p(stream.cuda_stream)


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else ctypes.c_void_p(0)


def _check(tensor, dtype, shape, name):
    if tensor.dtype != dtype or tuple(tensor.shape) != tuple(shape) or not tensor.is_contiguous() \
            or not tensor.is_cuda:
        raise ValueError(f"{name}: expected contiguous CUDA {dtype} {tuple(shape)}, got "
                         f"{tensor.dtype} {tuple(tensor.shape)} on {tensor.device}")


class _DeviceView:
    """Wraps a raw device pointer for torch.as_tensor (no copy, no ownership)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {
            "data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 3,
            "strides": None}


def _view(ptr, shape, dtype, device):
    typestr = {torch.uint8: "|u1", torch.int32: "<i4", torch.int16: "<i2"}[
        torch.int16 if dtype == torch.bfloat16 else dtype]
    tensor = torch.as_tensor(_DeviceView(ptr, shape, typestr), device=device)
    return tensor.view(torch.bfloat16) if dtype == torch.bfloat16 else tensor


@dataclass
class ExpertWeights:
    """The eight per-layer sidecar tensors the reference resolves by name
    (src/nvfp4_cutlass.cu:1792-1802), as CUDA tensors in the sidecar layout."""
    w13: torch.Tensor          # u8 [128,1408,1408]
    w13_sf: torch.Tensor       # u8 [128,1408,176]
    w2: torch.Tensor           # u8 [128,2816,352]
    w2_sf: torch.Tensor        # u8 [128,2816,44]
    alpha1: torch.Tensor       # f32 [128]  g1.alpha
    alpha2: torch.Tensor       # f32 [128]  g2.alpha
    in_scale_q1: torch.Tensor  # f32 [128]  g1.input_scale_quant
    in_scale_q2: torch.Tensor  # f32 [128]  g2.input_scale_quant

    def validate(self):
        _check(self.w13, torch.uint8, (EXPERTS, W13_OUT, HIDDEN // 2), "w13.weight")
        _check(self.w13_sf, torch.uint8, (EXPERTS, W13_OUT, HIDDEN // 16), "w13.weight_scale")
        _check(self.w2, torch.uint8, (EXPERTS, HIDDEN, INTER // 2), "w2.weight")
        _check(self.w2_sf, torch.uint8, (EXPERTS, HIDDEN, INTER // 16), "w2.weight_scale")
        for name in ("alpha1", "alpha2", "in_scale_q1", "in_scale_q2"):
            _check(getattr(self, name), torch.float32, (EXPERTS,), name)


class Nvfp4ExpertRunner:
    """Mirror of gevva::Nvfp4ExpertRunner (include/gevva/gpu.hpp:217-247)."""

    def __init__(self, experts: ExpertWeights, maximum_tokens: int = 1, shared_scratch=None, nvtx=False,
                 pairs=False, w13_pairs=False):
        """nvtx: wrap every stage's launches in a named NVTX range; pairs: run the expert GEMMs of
        batches above 128 tokens as CTA pairs; w13_pairs: run the fused w13 stage of such batches as
        CTA pairs with the weights on the MMA's M side (all additions of this build, same bits)."""
        experts.validate()
        self._weights = experts  # keeps the tensors alive, as the DeviceModel arena does
        self._device = experts.w13.device
        self.maximum_tokens = int(maximum_tokens)
        packed = _Weights(*[t.data_ptr() for t in (
            experts.w13, experts.w13_sf, experts.w2, experts.w2_sf, experts.alpha1,
            experts.alpha2, experts.in_scale_q1, experts.in_scale_q2)])
        handle = ctypes.c_void_p()
        share = shared_scratch._handle if shared_scratch is not None else None
        self._shared = shared_scratch
        with torch.cuda.device(self._device):
            options = _Options((OPTION_NVTX if nvtx else 0) | (OPTION_PAIRS if pairs else 0) |
                               (OPTION_W13_PAIRS if w13_pairs else 0))
            status = library().gevva_moe_create(ctypes.byref(handle), ctypes.byref(packed),
                                                self.maximum_tokens, share, ctypes.byref(options))
        if status != 0:
            raise GevvaMoeError(status, "Nvfp4ExpertRunner")
        self._handle = handle
        self._tokens = 0

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle and library is not None:  # module globals are gone at interpreter shutdown
            library().gevva_moe_destroy(handle)
            self._handle = None

    # -- the reference's five methods ------------------------------------------------
    def launch(self, input, expert_ids, route_weights, output, stream=None):
        """Single token (include/gevva/gpu.hpp:233-234)."""
        self.launch_batch(input, expert_ids, route_weights, output, 1, stream)

    def launch_batch(self, input, expert_ids, route_weights, output, tokens, stream=None):
        _check(input, torch.bfloat16, (tokens, HIDDEN), "input")
        _check(expert_ids, torch.int32, (tokens, TOP_K), "expert_ids")
        _check(route_weights, torch.float32, (tokens, TOP_K), "route_weights")
        _check(output, torch.bfloat16, (tokens, HIDDEN), "output")
        self._launch(input, expert_ids, route_weights, output, tokens, STAGE_ALL, stream)

    def launch_batch_unreduced(self, input, expert_ids, tokens, stream=None):
        _check(input, torch.bfloat16, (tokens, HIDDEN), "input")
        _check(expert_ids, torch.int32, (tokens, TOP_K), "expert_ids")
        self._launch(input, expert_ids, None, None, tokens, STAGE_ALL & ~STAGE_REDUCE, stream)

    def routed_output(self):
        """bf16 [8*tokens, 2816] in sorted-route order, valid until the next launch."""
        ptr = library().gevva_moe_routed_output(self._handle)
        return _view(ptr, (self._tokens * TOP_K, HIDDEN), torch.bfloat16, self._device)

    def inverse_routes(self):
        """int32 [8*tokens]: original route 8*t+k -> sorted row."""
        ptr = library().gevva_moe_inverse_routes(self._handle)
        return _view(ptr, (self._tokens * TOP_K,), torch.int32, self._device)

    # -- additions of this build ------------------------------------------------------
    def _launch(self, input, expert_ids, route_weights, output, tokens, stages, stream):
        with torch.cuda.device(self._device):
            status = library().gevva_moe_launch_stages(
                self._handle, _ptr(input), _ptr(expert_ids), _ptr(route_weights), _ptr(output),
                int(tokens), stages, _stream_handle(stream))
        if status != 0:
            raise GevvaMoeError(status, "launch")
        self._tokens = int(tokens)

    def launch_stages(self, stages, tokens, input=None, expert_ids=None, route_weights=None,
                      output=None, stream=None):
        """Runs a subset of the stages on the runner's scratch (parity tests)."""
        self._launch(input, expert_ids, route_weights, output, tokens, stages, stream)

    def last_status(self):
        """Synchronises, then returns and clears the device status word (0 = ok)."""
        with torch.cuda.device(self._device):
            return library().gevva_moe_last_status(self._handle)

    def check(self):
        status = self.last_status()
        if status != 0:
            raise GevvaMoeError(status, "device status")

    def buffer(self, buffer_id, dtype=torch.uint8):
        """A view of one scratch buffer (gevva_moe_buffer)."""
        ptr, size = ctypes.c_void_p(), ctypes.c_size_t()
        status = library().gevva_moe_buffer(self._handle, buffer_id, ctypes.byref(ptr),
                                            ctypes.byref(size))
        if status != 0:
            raise GevvaMoeError(status, "buffer")
        itemsize = {torch.uint8: 1, torch.int32: 4, torch.bfloat16: 2}[dtype]
        return _view(ptr.value, (size.value // itemsize,), dtype, self._device)


def route_128_top8(logits, expert_scale, activation_scales=None, projection_weight_scale=None,
                   weights=None, ids=None, stream=None):
    """Mirror of route_128_top8_kernel (src/cuda/kernels/routing_sampling.cuh:396-431).

    logits bf16 [rows, ld>=128] (may be a row-padded view), expert_scale bf16 [128].
    Returns (weights f32 [rows,8], ids int32 [rows,8])."""
    rows = logits.shape[0]
    if logits.dtype != torch.bfloat16 or logits.stride(1) != 1 or not logits.is_cuda:
        raise ValueError("logits: expected CUDA bf16 with unit column stride")
    _check(expert_scale, torch.bfloat16, (EXPERTS,), "expert_scale")
    if weights is None:
        weights = torch.empty((rows, TOP_K), dtype=torch.float32, device=logits.device)
    if ids is None:
        ids = torch.empty((rows, TOP_K), dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        status = library().gevva_moe_route(
            _ptr(logits), int(logits.stride(0)) if rows > 1 else max(int(logits.stride(0)), EXPERTS),
            _ptr(expert_scale), _ptr(weights), _ptr(ids), rows, _ptr(activation_scales),
            _ptr(projection_weight_scale), _stream_handle(stream))
    if status != 0:
        raise GevvaMoeError(status, "route_128_top8")
    return weights, ids


def route_project(router_input, router_weight, expert_scale, bias=None, want_logits=False, status_of=None,
                  activation_scales=None, weight_scale=None, weights=None, ids=None, stream=None):
    """Router projection and routing in one kernel (gevva_moe_route_project): what the reference
    does with a library GEMM followed by route_128_top8_kernel (src/cuda/runtime/prefill.cuh:414-422).

    router_input bf16 [rows, 2816] and router_weight bf16 [128, 2816]; or, with activation_scales
    f32 [rows] and weight_scale f32 [1], both as E4M3 bytes (uint8) for the FP8 sidecar's router.
    bias: optional f32 [128].  status_of: a runner whose status word receives a wait timeout.
    Returns (weights f32 [rows,8], ids int32 [rows,8]) and, with want_logits, the bf16 logits."""
    rows = router_input.shape[0]
    fp8 = activation_scales is not None
    dtype = torch.uint8 if fp8 else torch.bfloat16
    _check(router_input, dtype, (rows, HIDDEN), "router_input")
    _check(router_weight, dtype, (EXPERTS, HIDDEN), "router_weight")
    _check(expert_scale, torch.bfloat16, (EXPERTS,), "expert_scale")
    device = router_input.device
    if weights is None:
        weights = torch.empty((rows, TOP_K), dtype=torch.float32, device=device)
    if ids is None:
        ids = torch.empty((rows, TOP_K), dtype=torch.int32, device=device)
    logits = torch.empty((rows, EXPERTS), dtype=torch.bfloat16, device=device) if want_logits else None
    lib = library()
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    lib.gevva_moe_route_project.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, vp, vp]
    lib.gevva_moe_route_project_fp8.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp]
    lib.gevva_moe_status_word.argtypes = [vp]
    lib.gevva_moe_status_word.restype = vp
    status_word = vp(lib.gevva_moe_status_word(status_of._handle)) if status_of is not None else vp(0)
    with torch.cuda.device(device):
        if fp8:
            status = lib.gevva_moe_route_project_fp8(
                _ptr(router_input), _ptr(activation_scales), _ptr(router_weight), _ptr(weight_scale),
                _ptr(expert_scale), _ptr(weights), _ptr(ids), _ptr(logits), rows, status_word,
                _stream_handle(stream))
        else:
            status = lib.gevva_moe_route_project(
                _ptr(router_input), _ptr(router_weight), _ptr(bias), _ptr(expert_scale), _ptr(weights),
                _ptr(ids), _ptr(logits), rows, status_word, _stream_handle(stream))
    if status != 0:
        raise GevvaMoeError(status, "route_project")
    return (weights, ids, logits) if want_logits else (weights, ids)


def pack_experts(weights_fp32, stream=None):
    """fp32 [experts, N, K] -> (codes u8 [E,N,K/2], scales u8 [E,N,K/16], global f32 [E])."""
    experts, n_out, k_in = weights_fp32.shape
    if weights_fp32.dtype != torch.float32 or not weights_fp32.is_contiguous() or not weights_fp32.is_cuda:
        raise ValueError("weights: expected contiguous CUDA float32 [experts, N, K]")
    device = weights_fp32.device
    codes = torch.empty((experts, n_out, k_in // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((experts, n_out, k_in // 16), dtype=torch.uint8, device=device)
    global_scales = torch.empty((experts,), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        status = library().gevva_moe_pack_experts(
            _ptr(weights_fp32), experts, n_out, k_in, _ptr(codes), _ptr(scales),
            _ptr(global_scales), _stream_handle(stream))
    if status != 0:
        raise GevvaMoeError(status, "pack_experts")
    return codes, scales, global_scales


def route_sort_noalloc(expert_ids, stream=None):
    """Sorts routes without any device allocation inside the library.

    For callers that may not allocate on this path: the library's working memory is a
    fixed array in its own image (at most 16384 tokens), and every output is a tensor
    made here by the caller's allocator.  Returns a dict of int32 tensors:
    sorted_experts, sorted_routes, inverse_routes [8*tokens]; expert_offsets,
    scale_row_offsets [129]; status [1] (1 if an id was outside [0,128))."""
    lib = library()
    vp = ctypes.c_void_p
    lib.gevva_moe_route_sort_noalloc.argtypes = [vp, ctypes.c_int, vp, vp, vp, vp, vp, vp, vp]
    lib.gevva_moe_route_sort_noalloc.restype = ctypes.c_int
    tokens = expert_ids.shape[0]
    _check(expert_ids, torch.int32, (tokens, TOP_K), "expert_ids")
    device = expert_ids.device
    routes = tokens * TOP_K
    out = {name: torch.empty(routes, dtype=torch.int32, device=device)
           for name in ("sorted_experts", "sorted_routes", "inverse_routes")}
    out["expert_offsets"] = torch.empty(EXPERTS + 1, dtype=torch.int32, device=device)
    out["scale_row_offsets"] = torch.empty(EXPERTS + 1, dtype=torch.int32, device=device)
    out["status"] = torch.zeros(1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        status = lib.gevva_moe_route_sort_noalloc(
            _ptr(expert_ids), tokens, _ptr(out["sorted_experts"]), _ptr(out["sorted_routes"]),
            _ptr(out["inverse_routes"]), _ptr(out["expert_offsets"]),
            _ptr(out["scale_row_offsets"]), _ptr(out["status"]), _stream_handle(stream))
    if status != 0:
        raise GevvaMoeError(status, "route_sort_noalloc")
    return out
