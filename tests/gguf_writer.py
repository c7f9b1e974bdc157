"""Minimal GGUF v3 writer for the tests (the format as documented in the ggml project and as the
reference's reader consumes it, runtime/gguf_loader.cpp:96-134): header, typed key-value metadata,
tensor directory, aligned tensor data."""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _s(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    if vtype == STRING:
        return _s(v)
    if vtype == ARRAY:
        etype, items = v
        return struct.pack("<IQ", etype, len(items)) + b"".join(_value(etype, x) for x in items)
    return struct.pack(_FMT[vtype], v)


def write_gguf(path, metadata, tensors, alignment: int = 32, version: int = 3) -> dict:
    """metadata: list of (key, type, value) -- arrays as (ARRAY, (elem_type, [items]));
    tensors: list of (name, shape (shape[0] contiguous), ggml_type, bytes).  Returns {name: offset}."""
    out = bytearray()
    out += struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(metadata))
    for key, vtype, v in metadata:
        out += _s(key) + struct.pack("<I", vtype) + _value(vtype, v)
    offsets, off = {}, 0
    for name, shape, typ, data in tensors:
        off = (off + alignment - 1) // alignment * alignment
        offsets[name] = off
        out += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", typ, off)
        off += len(bytes(data))
    pad = (-len(out)) % alignment
    out += b"\0" * pad
    base = len(out)
    for name, shape, typ, data in tensors:
        out += b"\0" * (base + offsets[name] - len(out))
        out += bytes(np.ascontiguousarray(data).tobytes() if isinstance(data, np.ndarray) else data)
    with open(path, "wb") as f:
        f.write(out)
    return offsets
