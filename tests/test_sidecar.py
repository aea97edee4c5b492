"""Packed expert sidecar reader: the malformed headers the reference's own safetensors test
rejects (tests/test_safetensors.cpp:46-64) are rejected here, its valid cases map, and the
13-tensor layer schema (src/runtime.cpp:233-252) is enforced.  CPU only."""
import json
import os
import struct

import numpy as np
import pytest

from gevva_b200.sidecar import LAYER_TENSORS, ExpertSidecar, SidecarError

U64_MAX = 2 ** 64 - 1


def tensor(dtype, shape, offsets):
    return {"dtype": dtype, "shape": shape, "data_offsets": offsets}


def write(path, header_text, data_bytes):
    text = header_text.encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(text)))
        out.write(text)
        out.write(b"\0" * data_bytes)


# label, header (JSON text so that fractional and negative literals survive), data bytes
MALFORMED = [
    ("undersized", json.dumps({"x": tensor("BF16", [2816], [0, 2])}), 2),
    ("oversized", json.dumps({"x": tensor("BF16", [1], [0, 4])}), 4),
    ("shape overflow", json.dumps({"x": tensor("U8", [U64_MAX, 2], [0, 0])}), 0),
    ("byte overflow", json.dumps({"x": tensor("BF16", [U64_MAX], [0, 0])}), 0),
    ("unknown dtype", json.dumps({"x": tensor("CUSTOM", [1], [0, 1])}), 1),
    ("unsupported subbyte dtype", json.dumps({"x": tensor("F4", [2], [0, 1])}), 1),
    ("negative shape", '{"x":{"dtype":"U8","shape":[-1],"data_offsets":[0,0]}}', 0),
    ("fractional shape", '{"x":{"dtype":"U8","shape":[1.0],"data_offsets":[0,1]}}', 1),
    ("negative offset", '{"x":{"dtype":"U8","shape":[1],"data_offsets":[-1,0]}}', 1),
    ("fractional offset", '{"x":{"dtype":"U8","shape":[1],"data_offsets":[0.0,1]}}', 1),
    ("overlap", json.dumps({"x": tensor("U8", [2], [0, 2]), "y": tensor("U8", [2], [1, 3])}), 3),
    ("gap", json.dumps({"x": tensor("U8", [1], [0, 1]), "y": tensor("U8", [1], [2, 3])}), 3),
    ("unclaimed bytes", json.dumps({"x": tensor("U8", [1], [0, 1])}), 2),
    ("reversed offsets", json.dumps({"x": tensor("U8", [1], [1, 0])}), 1),
    ("out of file", json.dumps({"x": tensor("U8", [2], [0, 2])}), 1),
    ("extra offset", json.dumps({"x": tensor("U8", [1], [0, 1, 1])}), 1),
    ("shape not array", json.dumps({"x": tensor("U8", 1, [0, 1])}), 1),
    ("header not object", "[]", 0),
    ("metadata not strings", json.dumps({"__metadata__": {"value": 5}}), 0),
    # beyond the reference's list
    ("duplicate key", '{"x":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},'
                      '"x":{"dtype":"U8","shape":[1],"data_offsets":[0,1]}}', 1),
    ("truncated header", '{"x":{"dtype":"U8","shape":[1],"data_offsets":[0,1]}', 1),
    ("missing dtype", '{"x":{"shape":[1],"data_offsets":[0,1]}}', 1),
]


@pytest.mark.parametrize("label,header,data", MALFORMED, ids=[m[0] for m in MALFORMED])
def test_malformed_headers_are_rejected(tmp_path, label, header, data):
    path = tmp_path / "bad.safetensors"
    write(path, header, data)
    with pytest.raises(SidecarError):
        ExpertSidecar(path)


def test_header_length_beyond_file_is_rejected(tmp_path):
    path = tmp_path / "short.safetensors"
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SidecarError):
        ExpertSidecar(path)
    with open(path, "wb") as out:
        out.write(b"\x02\0\0")
    with pytest.raises(SidecarError):
        ExpertSidecar(path)
    with pytest.raises(SidecarError):
        ExpertSidecar(tmp_path / "does-not-exist.safetensors")


def test_valid_scalar_matrix_and_empty_tensors_map(tmp_path):
    path = tmp_path / "ok.safetensors"
    header = {"scalar": tensor("F32", [], [0, 4]), "matrix": tensor("BF16", [2, 2], [4, 12]),
              "empty": tensor("U8", [0, 99], [12, 12]), "__metadata__": {"format": "test"}}
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    payload = struct.pack("<f", 1.5) + bytes(range(8))
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(text)) + text + payload)
    with ExpertSidecar(path) as sidecar:
        assert len(sidecar) == 3
        assert sidecar.tensor("scalar").shape == () and float(sidecar.tensor("scalar")) == 1.5
        assert sidecar.tensor("matrix").tobytes() == bytes(range(8))   # BF16: raw bytes
        assert sidecar.tensor("empty").size == 0
        with pytest.raises(SidecarError):
            sidecar.tensor("absent")
    write(path, "{}", 0)
    with ExpertSidecar(path) as sidecar:
        assert len(sidecar) == 0
        sidecar.check_layers(0)


def sparse_sidecar(path, layers, mutate=None):
    """A sidecar of full-size layers whose data section is a hole in a sparse file."""
    header, offset = {}, 0
    for layer in range(layers):
        for suffix, np_dtype, st_dtype, shape in LAYER_TENSORS:
            size = int(np.prod(shape)) * np.dtype(np_dtype).itemsize
            header[f"layers.{layer}.{suffix}"] = tensor(st_dtype, list(shape), [offset, offset + size])
            offset += size
    if mutate:
        offset = mutate(header, offset)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(text)) + text)
        out.truncate(8 + len(text) + offset)


def test_layer_schema(tmp_path):
    path = tmp_path / "experts.safetensors"
    sparse_sidecar(path, 2)
    with ExpertSidecar(path) as sidecar:
        assert len(sidecar) == 26
        sidecar.check_layers(2)
        with pytest.raises(SidecarError):
            sidecar.check_layers(3)          # a layer is missing
        with pytest.raises(SidecarError):
            sidecar.check_layers(1)          # unexpected extra tensors
        view = sidecar.tensor("layers.1.w2.weight_scale")
        assert view.shape == (128, 2816, 44) and view.dtype == np.uint8

    def wrong_shape(header, offset):
        header["layers.0.g1.alpha"]["dtype"] = "F32"
        entry = header["layers.0.w13.weight_scale_2"]
        entry["shape"] = [2, 128]            # transposed: same bytes, wrong shape
        return offset

    sparse_sidecar(path, 1, wrong_shape)
    with ExpertSidecar(path) as sidecar:
        with pytest.raises(SidecarError, match="w13.weight_scale_2"):
            sidecar.check_layers(1)

    def wrong_dtype(header, offset):
        entry = header["layers.0.g2.alpha"]
        entry["dtype"], entry["shape"] = "I32", [128]
        return offset

    sparse_sidecar(path, 1, wrong_dtype)
    with ExpertSidecar(path) as sidecar:
        with pytest.raises(SidecarError, match="g2.alpha"):
            sidecar.check_layers(1)
