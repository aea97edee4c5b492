"""Packed expert sidecar files: reader (over the C ABI) and writer.

The reader mirrors what the reference does with `experts-*.safetensors`: strict header
inspection (src/safetensors.cpp), the 13-tensors-per-layer schema (src/runtime.cpp:222-254)
and the lookup of the eight tensors a runner needs (src/nvfp4_cutlass.cu:1792-1802).  The
writer stands where tools/pack_trtllm_experts.py:134-150 stands (it saves the same names,
dtypes and shapes) so that synthetic layers can be stored and loaded through the same path as
real ones.
"""
import ctypes
import json
import struct

import numpy as np
import torch

from .runtime import EXPERTS, ExpertWeights, GevvaMoeError, library

LAYER_TENSORS = (
    # suffix, numpy dtype, safetensors dtype, shape
    ("w13.weight", np.uint8, "U8", (128, 1408, 1408)),
    ("w13.weight_scale", np.uint8, "U8", (128, 1408, 176)),
    ("w2.weight", np.uint8, "U8", (128, 2816, 352)),
    ("w2.weight_scale", np.uint8, "U8", (128, 2816, 44)),
    ("w13.input_scale", np.float32, "F32", (128,)),
    ("w2.input_scale", np.float32, "F32", (128,)),
    ("w13.weight_scale_2", np.float32, "F32", (128, 2)),
    ("w2.weight_scale_2", np.float32, "F32", (128,)),
    ("g1.alpha", np.float32, "F32", (128,)),
    ("g1.alpha_up", np.float32, "F32", (128,)),
    ("g2.alpha", np.float32, "F32", (128,)),
    ("g1.input_scale_quant", np.float32, "F32", (128,)),
    ("g2.input_scale_quant", np.float32, "F32", (128,)),
)

_NUMPY_DTYPES = {"U8": np.uint8, "I8": np.int8, "BOOL": np.bool_, "U16": np.uint16, "I16": np.int16,
                 "F16": np.float16, "U32": np.uint32, "I32": np.int32, "F32": np.float32,
                 "U64": np.uint64, "I64": np.int64, "F64": np.float64}


class _View(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_char * 16), ("rank", ctypes.c_int), ("shape", ctypes.c_uint64 * 8),
                ("data", ctypes.c_void_p), ("bytes", ctypes.c_uint64)]


class _HostWeights(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in
                ("w13", "w13_sf", "w2", "w2_sf", "alpha1", "alpha2", "in_scale_q1", "in_scale_q2")]


def _bind(lib):
    if getattr(lib, "_sidecar_bound", False):
        return lib
    vp = ctypes.c_void_p
    lib.gevva_sidecar_open.argtypes = [ctypes.POINTER(vp), ctypes.c_char_p]
    lib.gevva_sidecar_open.restype = ctypes.c_int
    lib.gevva_sidecar_close.argtypes = [vp]
    lib.gevva_sidecar_close.restype = None
    lib.gevva_sidecar_tensor_count.argtypes = [vp]
    lib.gevva_sidecar_tensor_count.restype = ctypes.c_int
    lib.gevva_sidecar_tensor.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(_View)]
    lib.gevva_sidecar_tensor.restype = ctypes.c_int
    lib.gevva_sidecar_check_layers.argtypes = [vp, ctypes.c_int]
    lib.gevva_sidecar_check_layers.restype = ctypes.c_int
    lib.gevva_sidecar_layer_weights.argtypes = [vp, ctypes.c_int, ctypes.POINTER(_HostWeights)]
    lib.gevva_sidecar_layer_weights.restype = ctypes.c_int
    lib.gevva_sidecar_error.argtypes = []
    lib.gevva_sidecar_error.restype = ctypes.c_char_p
    lib._sidecar_bound = True
    return lib


class SidecarError(GevvaMoeError):
    pass


def _raise(lib, status, where):
    text = lib.gevva_sidecar_error()
    error = SidecarError(status, where)
    error.args = (f"{where}: {text.decode() if text else 'error'}",)
    raise error


class ExpertSidecar:
    """A mapped sidecar file.  Tensor views are numpy arrays over the read-only mapping and
    must not outlive the object."""

    def __init__(self, path):
        self._lib = _bind(library())
        handle = ctypes.c_void_p()
        status = self._lib.gevva_sidecar_open(ctypes.byref(handle), str(path).encode())
        if status != 0:
            _raise(self._lib, status, "gevva_sidecar_open")
        self._handle = handle

    def close(self):
        handle = getattr(self, "_handle", None)
        if handle:
            self._lib.gevva_sidecar_close(handle)
            self._handle = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return self._lib.gevva_sidecar_tensor_count(self._handle)

    def tensor(self, name):
        view = _View()
        status = self._lib.gevva_sidecar_tensor(self._handle, name.encode(), ctypes.byref(view))
        if status != 0:
            _raise(self._lib, status, "gevva_sidecar_tensor")
        dtype = view.dtype.decode()
        shape = tuple(int(view.shape[i]) for i in range(view.rank))
        if view.bytes == 0:
            return np.zeros(shape, dtype=_NUMPY_DTYPES.get(dtype, np.uint8))
        raw = (ctypes.c_uint8 * view.bytes).from_address(view.data)
        array = np.frombuffer(raw, dtype=np.uint8)
        if dtype in _NUMPY_DTYPES:
            return array.view(_NUMPY_DTYPES[dtype]).reshape(shape)
        return array  # BF16 / F8 have no numpy type: raw bytes

    def check_layers(self, layers=30):
        status = self._lib.gevva_sidecar_check_layers(self._handle, layers)
        if status != 0:
            _raise(self._lib, status, "gevva_sidecar_check_layers")

    def layer_weights(self, layer, device="cuda:0"):
        """The eight tensors of `layer` copied to `device` as an ExpertWeights."""
        host = _HostWeights()
        status = self._lib.gevva_sidecar_layer_weights(self._handle, layer, ctypes.byref(host))
        if status != 0:
            _raise(self._lib, status, "gevva_sidecar_layer_weights")
        prefix = f"layers.{layer}."
        names = ("w13.weight", "w13.weight_scale", "w2.weight", "w2.weight_scale", "g1.alpha",
                 "g2.alpha", "g1.input_scale_quant", "g2.input_scale_quant")
        tensors = [torch.from_numpy(np.array(self.tensor(prefix + name))).to(device) for name in names]
        weights = ExpertWeights(*tensors)
        weights.validate()
        return weights


def write_sidecar(path, layers):
    """Writes a sidecar with the reference's tensor names.  `layers` is a list of dicts keyed by
    the thirteen suffixes of LAYER_TENSORS (numpy arrays or CPU/CUDA torch tensors)."""
    header = {}
    blobs = []
    offset = 0
    for index, layer in enumerate(layers):
        for suffix, np_dtype, st_dtype, shape in LAYER_TENSORS:
            value = layer[suffix]
            if isinstance(value, torch.Tensor):
                value = value.detach().cpu().numpy()
            value = np.ascontiguousarray(value, dtype=np_dtype)
            if value.shape != shape:
                raise ValueError(f"layers.{index}.{suffix}: shape {value.shape}, expected {shape}")
            header[f"layers.{index}.{suffix}"] = {"dtype": st_dtype, "shape": list(shape),
                                                  "data_offsets": [offset, offset + value.nbytes]}
            blobs.append(value)
            offset += value.nbytes
    header["__metadata__"] = {"format": "pt"}
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(text)))
        out.write(text)
        for blob in blobs:
            out.write(blob.tobytes())


def synthetic_layer_tensors(packed, weights, s1, s2):
    """The thirteen tensors of one layer from `make_packed_experts` output, the runner's
    `ExpertWeights` (whose alpha and input_scale_quant vectors are stored as they are) and the
    two static activation scales, following tools/pack_trtllm_experts.py:134-148."""
    ones = np.ones(EXPERTS, dtype=np.float32)
    g13 = packed["g13"].detach().cpu().numpy().astype(np.float32)
    g2 = packed["g2"].detach().cpu().numpy().astype(np.float32)
    return {
        "w13.weight": weights.w13, "w13.weight_scale": weights.w13_sf,
        "w2.weight": weights.w2, "w2.weight_scale": weights.w2_sf,
        "w13.input_scale": ones * np.float32(s1), "w2.input_scale": ones * np.float32(s2),
        "w13.weight_scale_2": np.stack([g13, g13], axis=1), "w2.weight_scale_2": g2,
        "g1.alpha": weights.alpha1, "g1.alpha_up": weights.alpha1, "g2.alpha": weights.alpha2,
        "g1.input_scale_quant": weights.in_scale_q1, "g2.input_scale_quant": weights.in_scale_q2,
    }
