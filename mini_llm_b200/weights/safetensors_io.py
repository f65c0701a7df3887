"""Reading and writing the safetensors container.

Layout of a file: an 8-byte little-endian length N, N bytes of JSON
(``{name: {"dtype", "shape", "data_offsets": [begin, end]}}``, offsets relative
to the end of the header), then the tensors' bytes.  The reference does not
read this format: it exports one raw fp32 file per tensor plus a manifest
(scripts/dump_weights.py:37-53) and opens them by name
(engine/src/tensor_loading.c:6-52).  Here the container is read directly and
each tensor is a zero-copy view into the mapped file.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np


class SafetensorsError(ValueError):
    pass


# dtype tag -> (numpy dtype of the stored bits, bytes per element)
STORED = {
    "F32": (np.dtype("<f4"), 4),
    "F16": (np.dtype("<f2"), 2),
    "BF16": (np.dtype("<u2"), 2),      # bits only: numpy has no bfloat16
    "F64": (np.dtype("<f8"), 8),
    "I64": (np.dtype("<i8"), 8),
    "I32": (np.dtype("<i4"), 4),
    "I16": (np.dtype("<i2"), 2),
    "I8": (np.dtype("i1"), 1),
    "U8": (np.dtype("u1"), 1),
    "BOOL": (np.dtype("u1"), 1),
}


class StoredTensor:
    """One tensor of a file: its tag, shape and the raw bits (a numpy view)."""

    __slots__ = ("name", "dtype", "shape", "bits")

    def __init__(self, name, dtype, shape, bits):
        self.name, self.dtype, self.shape, self.bits = name, dtype, tuple(shape), bits

    @property
    def is_float(self) -> bool:
        return self.dtype in ("F32", "F16", "BF16", "F64")

    @property
    def is_32bit_float(self) -> bool:
        return self.dtype == "F32"


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._handle = open(path, "rb")
        except OSError as error:
            raise SafetensorsError(f"cannot open weights file '{path}': {error.strerror}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > size - 8:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file ({size} bytes): truncated?")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not valid JSON: {error}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + header_len
        self.tensors: dict[str, StoredTensor] = {}
        buffer = memoryview(self._map)
        for name, info in header.items():
            try:
                tag, shape = info["dtype"], info["shape"]
                begin, end = info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            if tag not in STORED:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {tag}")
            np_dtype, width = STORED[tag]
            count = 1
            for extent in shape:
                count *= int(extent)
            if end - begin != count * width:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({tag} {shape}) needs {count * width} bytes, header gives {end - begin}")
            if base + end > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ends at byte {base + end} but the file has {size}: truncated")
            bits = np.frombuffer(buffer, dtype=np_dtype, count=count, offset=base + begin).reshape(shape)
            self.tensors[name] = StoredTensor(name, tag, shape, bits)

    def names(self):
        return list(self.tensors)


def float32_to_bfloat16_bits(values: np.ndarray) -> np.ndarray:
    """Round fp32 to bfloat16 (nearest, ties to even); returns the 16-bit patterns."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = bits + (np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def write_safetensors(path: str, tensors: dict, store_dtype: dict | str = "F32", metadata: dict | None = None):
    """Write ``{name: numpy array}``.  Float arrays are stored as ``store_dtype``
    ("F32" or "BF16"; a dict gives it per name), integer arrays as I32/I64."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    offset = 0
    for name, array in tensors.items():
        array = np.asarray(array)
        tag = store_dtype.get(name, "F32") if isinstance(store_dtype, dict) else store_dtype
        if np.issubdtype(array.dtype, np.floating):
            if tag == "BF16":
                blob = float32_to_bfloat16_bits(array).tobytes()
            elif tag == "F32":
                blob = np.ascontiguousarray(array, dtype="<f4").tobytes()
            elif tag == "F16":
                blob = np.ascontiguousarray(array, dtype="<f2").tobytes()
            else:
                raise SafetensorsError(f"cannot store floats as {tag}")
        elif array.dtype == np.int64:
            tag, blob = "I64", np.ascontiguousarray(array, dtype="<i8").tobytes()
        elif np.issubdtype(array.dtype, np.integer):
            tag, blob = "I32", np.ascontiguousarray(array, dtype="<i4").tobytes()
        else:
            raise SafetensorsError(f"tensor '{name}': cannot store dtype {array.dtype}")
        header[name] = {"dtype": tag, "shape": list(array.shape), "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for blob in blobs:
            handle.write(blob)
