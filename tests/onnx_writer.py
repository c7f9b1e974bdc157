"""A few lines of protobuf wire-format writing: enough to build one-node ONNX models for the
harness tests (the reference's tests do the same in C++, runtime/tests/op_test.cpp:160-371)."""
from __future__ import annotations

import struct

import numpy as np

ONNX_DTYPE = {np.dtype("float32"): 1, np.dtype("uint8"): 2, np.dtype("int8"): 3, np.dtype("int32"): 6,
              np.dtype("int64"): 7, np.dtype("bool"): 9, np.dtype("float16"): 10}


def varint(v: int) -> bytes:
    out = bytearray()
    v &= (1 << 64) - 1
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def field_varint(num: int, v: int) -> bytes:
    return varint(num << 3) + varint(v)


def field_bytes(num: int, payload: bytes) -> bytes:
    return varint((num << 3) | 2) + varint(len(payload)) + payload


def field_str(num: int, s: str) -> bytes:
    return field_bytes(num, s.encode())


def attribute_int(name: str, v: int) -> bytes:
    return field_str(1, name) + field_varint(3, v) + field_varint(20, 2)


def tensor(name: str, arr: np.ndarray) -> bytes:
    out = b"".join(field_varint(1, int(d)) for d in arr.shape)
    out += field_varint(2, ONNX_DTYPE[arr.dtype]) + field_str(8, name) + field_bytes(9, arr.tobytes())
    return out


def value_info(name: str, dtype, shape) -> bytes:
    dims = b"".join(field_bytes(1, field_varint(1, int(d))) for d in shape)
    tensor_type = field_varint(1, ONNX_DTYPE[np.dtype(dtype)]) + field_bytes(2, dims)
    return field_str(1, name) + field_bytes(2, field_bytes(1, tensor_type))


def node(op_type: str, inputs, outputs, name="n0", attrs=(), domain="") -> bytes:
    out = b"".join(field_str(1, i) for i in inputs) + b"".join(field_str(2, o) for o in outputs)
    out += field_str(3, name) + field_str(4, op_type) + b"".join(field_bytes(5, a) for a in attrs)
    if domain:
        out += field_str(7, domain)
    return out


def model(nodes, inputs, outputs, initializers=()) -> bytes:
    g = b"".join(field_bytes(1, n) for n in nodes) + field_str(2, "g")
    g += b"".join(field_bytes(5, t) for t in initializers)
    g += b"".join(field_bytes(11, v) for v in inputs) + b"".join(field_bytes(12, v) for v in outputs)
    opset = field_str(1, "") + field_varint(2, 17)
    return field_varint(1, 8) + field_bytes(7, g) + field_bytes(8, opset)


def matmul_q4k_model(N: int, K: int, x_shape, weights: np.ndarray | None, with_bias: bool, op: str = "MatMulQ4K",
                     block_bytes: int = 144) -> bytes:
    """One MatMulQ4K (or MatMulQ5K / MatMulQ6K: `op`, `block_bytes` 176 / 210) node.  `weights` given: W is an
    initializer; else W is a runtime input."""
    ins = ["X", "W"] + (["Bias"] if with_bias else [])
    n = node(op, ins, ["Y"], attrs=[attribute_int("K", K), attribute_int("N", N)], domain="ai.backpack")
    graph_inputs = [value_info("X", "float32", x_shape)]
    inits = []
    if weights is not None:
        inits.append(tensor("W", weights))
    else:
        graph_inputs.append(value_info("W", "uint8", (N, K // 256 * block_bytes)))
    if with_bias:
        graph_inputs.append(value_info("Bias", "float32", (N,)))
    return model([n], graph_inputs, [value_info("Y", "float32", tuple(x_shape[:-1]) + (N,))], inits)
