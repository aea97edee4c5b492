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


class _Projection(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("weight_scale", ctypes.c_void_p),
                ("weight_scale_2", ctypes.c_float), ("input_scale", ctypes.c_float)]


class _CheckpointExpert(ctypes.Structure):
    _fields_ = [("gate_proj", _Projection), ("up_proj", _Projection), ("down_proj", _Projection)]


class _SidecarLayer(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in
                ("w13_weight", "w13_weight_scale", "w2_weight", "w2_weight_scale", "w13_input_scale",
                 "w2_input_scale", "w13_weight_scale_2", "w2_weight_scale_2", "g1_alpha", "g1_alpha_up",
                 "g2_alpha", "g1_input_scale_quant", "g2_input_scale_quant")]


def pack_checkpoint_layer(get, layer, experts=EXPERTS, hidden=2816, intermediate=704):
    """The thirteen sidecar tensors of one layer from checkpoint tensors, as
    tools/pack_trtllm_experts.py:88-148 makes them.  `get(name)` returns the checkpoint tensor
    `name` as a numpy array (what safetensors' get_tensor gives): per expert E and projection P in
    gate_proj / up_proj / down_proj,
        model.language_model.layers.{layer}.experts.{E}.{P}.weight          u8 [rows, k/2]
        ...weight_scale  E4M3 bytes [rows, k/16]   ...weight_scale_2, ...input_scale  f32 scalars.
    The work is done by gevva_moe_pack_checkpoint_layer on the host; the result is a dict keyed by
    the suffixes of LAYER_TENSORS, ready for write_sidecar."""
    lib = _bind(library())
    lib.gevva_moe_pack_checkpoint_layer.argtypes = [ctypes.POINTER(_CheckpointExpert), ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_int, ctypes.POINTER(_SidecarLayer)]
    lib.gevva_moe_pack_checkpoint_layer.restype = ctypes.c_int
    keep = []

    def projection(expert, name, rows, k):
        prefix = f"model.language_model.layers.{layer}.experts.{expert}.{name}."
        weight = np.ascontiguousarray(get(prefix + "weight")).view(np.uint8)
        scale = np.ascontiguousarray(get(prefix + "weight_scale")).view(np.uint8)
        if weight.shape != (rows, k // 2) or scale.shape != (rows, k // 16):
            raise ValueError(f"{prefix}: weight {weight.shape}, weight_scale {scale.shape}; expected "
                             f"{(rows, k // 2)} and {(rows, k // 16)}")
        keep.extend((weight, scale))
        return _Projection(weight.ctypes.data, scale.ctypes.data,
                           float(np.asarray(get(prefix + "weight_scale_2"), dtype=np.float32).reshape(())),
                           float(np.asarray(get(prefix + "input_scale"), dtype=np.float32).reshape(())))

    table = (_CheckpointExpert * experts)()
    for e in range(experts):
        table[e] = _CheckpointExpert(projection(e, "gate_proj", intermediate, hidden),
                                     projection(e, "up_proj", intermediate, hidden),
                                     projection(e, "down_proj", hidden, intermediate))
    out = {
        "w13.weight": np.empty((experts, 2 * intermediate, hidden // 2), np.uint8),
        "w13.weight_scale": np.empty((experts, 2 * intermediate, hidden // 16), np.uint8),
        "w2.weight": np.empty((experts, hidden, intermediate // 2), np.uint8),
        "w2.weight_scale": np.empty((experts, hidden, intermediate // 16), np.uint8),
        "w13.input_scale": np.empty(experts, np.float32), "w2.input_scale": np.empty(experts, np.float32),
        "w13.weight_scale_2": np.empty((experts, 2), np.float32), "w2.weight_scale_2": np.empty(experts, np.float32),
        "g1.alpha": np.empty(experts, np.float32), "g1.alpha_up": np.empty(experts, np.float32),
        "g2.alpha": np.empty(experts, np.float32), "g1.input_scale_quant": np.empty(experts, np.float32),
        "g2.input_scale_quant": np.empty(experts, np.float32),
    }
    order = ("w13.weight", "w13.weight_scale", "w2.weight", "w2.weight_scale", "w13.input_scale",
             "w2.input_scale", "w13.weight_scale_2", "w2.weight_scale_2", "g1.alpha", "g1.alpha_up", "g2.alpha",
             "g1.input_scale_quant", "g2.input_scale_quant")
    target = _SidecarLayer(*[out[name].ctypes.data for name in order])
    status = lib.gevva_moe_pack_checkpoint_layer(table, experts, hidden, intermediate, ctypes.byref(target))
    if status != 0:
        _raise(lib, status, "gevva_moe_pack_checkpoint_layer")
    return out


def deinterleave_scales(interleaved):
    """Inverse of the 128-row x 4-group block-scale interleave: sidecar layout [rows, groups] (as
    stored) -> row-major [rows, groups] (as a checkpoint stores weight_scale)."""
    rows, groups = interleaved.shape
    blocks = interleaved.reshape(rows // 128, groups // 4, 32, 4, 4)     # [row block, k block, r%32, (r/32)%4, g%4]
    return np.ascontiguousarray(blocks.transpose(0, 3, 2, 1, 4)).reshape(rows, groups)


def synthetic_checkpoint(packed, s1, s2, layer=0):
    """A checkpoint-format view of `make_packed_experts` output: per-expert gate/up/down tensors
    with row-major block scales, under the checkpoint's tensor names.  Returns get(name)."""
    w13, w13_sf = packed["w13"].cpu().numpy(), packed["w13_sf"].cpu().numpy()
    w2, w2_sf = packed["w2"].cpu().numpy(), packed["w2_sf"].cpu().numpy()
    g13, g2 = packed["g13"].cpu().numpy(), packed["g2"].cpu().numpy()
    inter = w13.shape[1] // 2

    def get(name):
        parts = name.split(".")
        expert, projection, suffix = int(parts[5]), parts[6], parts[7]
        assert int(parts[3]) == layer
        if projection == "down_proj":
            table = {"weight": lambda: w2[expert], "weight_scale": lambda: deinterleave_scales(w2_sf[expert]),
                     "weight_scale_2": lambda: np.float32(g2[expert]), "input_scale": lambda: np.float32(s2)}
        else:
            rows = slice(0, inter) if projection == "up_proj" else slice(inter, 2 * inter)   # w13 = [up; gate]
            table = {"weight": lambda: w13[expert][rows],
                     "weight_scale": lambda: deinterleave_scales(w13_sf[expert])[rows],
                     "weight_scale_2": lambda: np.float32(g13[expert]), "input_scale": lambda: np.float32(s1)}
        return table[suffix]()

    return get


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
