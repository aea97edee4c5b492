"""Feed-forward steps around the expert path and the dense FP8 GeGLU MLP (ctypes mirror of
the gevva_ff_* / gevva_dense_* entry points), plus the layer wiring of the reference's
layer loop (src/cuda/runtime/prefill.cuh:1200-1250) with attention left out."""
import ctypes
from dataclasses import dataclass

import torch

from .runtime import (EXPERTS, HIDDEN, TOP_K, GevvaMoeError, Nvfp4ExpertRunner, _check, _ptr,
                      _stream_handle, _view, library, route_project)

DENSE = 2112


class _DenseWeights(ctypes.Structure):
    _fields_ = [("gate_up", ctypes.c_void_p), ("down", ctypes.c_void_p), ("gate_scale", ctypes.c_float),
                ("up_scale", ctypes.c_float), ("down_scale", ctypes.c_float)]


def _lib():
    lib = library()
    if getattr(lib, "_gv_ff_ready", False):
        return lib
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.gevva_ff_prepare.argtypes = [vp] * 7 + [i32, vp]
    lib.gevva_ff_finalize.argtypes = [vp] * 10 + [i32, vp, vp, vp]
    lib.gevva_dense_create.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(_DenseWeights), i32]
    lib.gevva_dense_destroy.argtypes = [vp]
    lib.gevva_dense_destroy.restype = None
    lib.gevva_dense_launch.argtypes = [vp, vp, vp, i32, vp]
    lib.gevva_dense_output_scales.argtypes = [vp]
    lib.gevva_dense_output_scales.restype = vp
    lib.gevva_dense_projection_scale.argtypes = [vp]
    lib.gevva_dense_projection_scale.restype = vp
    lib.gevva_dense_buffer.argtypes = [vp, i32, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    lib.gevva_pack_fp8.argtypes = [vp, ctypes.c_size_t, vp, vp, vp]
    lib._gv_ff_ready = True
    return lib


def _status(status, where):
    if status != 0:
        raise GevvaMoeError(status, where)


def pack_fp8(weight_fp32):
    """Per-tensor E4M3 quantisation: returns (uint8 tensor of the same shape, float scale)."""
    w = weight_fp32.contiguous()
    out = torch.empty(w.shape, dtype=torch.uint8, device=w.device)
    scale = torch.empty(1, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _status(_lib().gevva_pack_fp8(_ptr(w), w.numel(), _ptr(out), _ptr(scale), _stream_handle(None)),
                "pack_fp8")
    return out, float(scale.item())


def ff_prepare(x, dense_weight, expert_weight, router_scale):
    rows = x.shape[0]
    _check(x, torch.bfloat16, (rows, HIDDEN), "input")
    outs = [torch.empty_like(x) for _ in range(3)]
    with torch.cuda.device(x.device):
        _status(_lib().gevva_ff_prepare(_ptr(x), _ptr(dense_weight), _ptr(expert_weight), _ptr(router_scale),
                                        _ptr(outs[0]), _ptr(outs[1]), _ptr(outs[2]), rows,
                                        _stream_handle(None)), "ff_prepare")
    return outs  # dense_pre, expert_pre, router_input


def ff_finalize(dense, dense_weight, expert_routes, route_weights, inverse_routes, expert_weight,
                combined_weight, residual, layer_scalar, dense_activation_scales=None,
                dense_projection_scale=None):
    """dense_activation_scales f32 [rows] and dense_projection_scale f32 [1] are CUDA tensors (or both
    None), as the reference kernel takes them."""
    rows = dense.shape[0]
    out = torch.empty_like(residual)
    with torch.cuda.device(dense.device):
        _status(_lib().gevva_ff_finalize(
            _ptr(dense), _ptr(dense_weight), _ptr(expert_routes), _ptr(route_weights), _ptr(inverse_routes),
            _ptr(expert_weight), _ptr(combined_weight), _ptr(residual), _ptr(layer_scalar), _ptr(out), rows,
            _ptr(dense_activation_scales), _ptr(dense_projection_scale), _stream_handle(None)), "ff_finalize")
    return out


class DenseMlp:
    """Dense FP8 GeGLU MLP; launch() returns the unscaled bf16 output and its row scales."""

    def __init__(self, gate_up_fp8, down_fp8, gate_scale, up_scale, down_scale, max_tokens):
        _check(gate_up_fp8, torch.uint8, (2 * DENSE, HIDDEN), "gate_up")
        _check(down_fp8, torch.uint8, (HIDDEN, DENSE), "down")
        self._keep = (gate_up_fp8, down_fp8)
        self.device = gate_up_fp8.device
        self.down_scale = float(down_scale)
        self.max_tokens = max_tokens
        w = _DenseWeights(gate_up_fp8.data_ptr(), down_fp8.data_ptr(), gate_scale, up_scale, down_scale)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _status(_lib().gevva_dense_create(ctypes.byref(handle), ctypes.byref(w), max_tokens), "DenseMlp")
        self._handle = handle
        # f32 [1] on the device, owned by the runner: what ff_finalize takes beside the row scales
        self.projection_scale = _view(_lib().gevva_dense_projection_scale(self._handle), (1,), torch.int32,
                                      self.device).view(torch.float32)

    def __del__(self):
        if getattr(self, "_handle", None):
            _lib().gevva_dense_destroy(self._handle)
            self._handle = None

    def launch(self, x, out=None, stream=None):
        tokens = x.shape[0]
        _check(x, torch.bfloat16, (tokens, HIDDEN), "input")
        if out is None:
            out = torch.empty_like(x)
        with torch.cuda.device(self.device):
            _status(_lib().gevva_dense_launch(self._handle, _ptr(x), _ptr(out), tokens, _stream_handle(stream)),
                    "dense launch")
        scales = _view(_lib().gevva_dense_output_scales(self._handle), (tokens,), torch.int32,
                       self.device).view(torch.float32)
        return out, scales

    def buffer(self, which, dtype):
        ptr, size = ctypes.c_void_p(), ctypes.c_size_t()
        _status(_lib().gevva_dense_buffer(self._handle, which, ctypes.byref(ptr), ctypes.byref(size)), "buffer")
        item = {torch.uint8: 1, torch.int32: 4, torch.bfloat16: 2, torch.float32: 4}[dtype]
        base = torch.int32 if dtype == torch.float32 else dtype
        t = _view(ptr.value, (size.value // item,), base, self.device)
        return t.view(torch.float32) if dtype == torch.float32 else t


@dataclass
class FeedForwardLayer:
    """One layer of the FFN stack: pre-norms + router, experts and dense MLP side by side,
    fused finalize (the wiring of src/cuda/runtime/prefill.cuh:1200-1250)."""
    dense_pre: torch.Tensor        # bf16 [2816] norm weights
    expert_pre: torch.Tensor
    router_scale: torch.Tensor
    router_w: torch.Tensor         # bf16 [128, 2816]
    expert_scale: torch.Tensor     # bf16 [128]
    dense_post: torch.Tensor
    expert_post: torch.Tensor
    combined_post: torch.Tensor
    layer_scalar: torch.Tensor     # bf16 [1]
    experts: Nvfp4ExpertRunner
    dense: DenseMlp

    def forward(self, hidden, aux_stream=None):
        tokens = hidden.shape[0]
        dense_in, expert_in, router_in = ff_prepare(hidden, self.dense_pre, self.expert_pre, self.router_scale)
        weights, ids = route_project(router_in, self.router_w, self.expert_scale, status_of=self.experts)
        main = torch.cuda.current_stream()
        if aux_stream is not None:
            aux_stream.wait_stream(main)
            with torch.cuda.stream(aux_stream):
                dense_out, dense_scales = self.dense.launch(dense_in)
        else:
            dense_out, dense_scales = self.dense.launch(dense_in)
        self.experts.launch_batch_unreduced(expert_in, ids, tokens)
        if aux_stream is not None:
            main.wait_stream(aux_stream)
        return ff_finalize(dense_out, self.dense_post, self.experts.routed_output(), weights,
                           self.experts.inverse_routes(), self.expert_post, self.combined_post, hidden,
                           self.layer_scalar, dense_scales, self.dense.projection_scale)
