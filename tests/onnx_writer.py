"""A minimal ONNX (protobuf) writer for tests: enough of ModelProto to describe small graphs by hand,
so the loader can be exercised without the `onnx` package or any model file."""
import struct

import numpy as np

_ELEM = {np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.int32): 6,
         np.dtype(np.int64): 7, np.dtype(np.bool_): 9, np.dtype(np.float64): 11}


def _varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _int(field: int, value: int) -> bytes:
    return _varint(field << 3) + _varint(value)


def _bytes(field: int, payload: bytes) -> bytes:
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def tensor(name: str, array, typed_fields: bool = False) -> bytes:
    array = np.asarray(array)
    out = b"".join(_int(1, d) for d in array.shape) + _int(2, _ELEM[array.dtype])
    if typed_fields and array.dtype == np.float32:
        out += _bytes(4, array.astype("<f4").tobytes())                 # packed float_data
    elif typed_fields and array.dtype == np.int64:
        out += b"".join(_int(7, int(v)) for v in array.reshape(-1))     # unpacked int64_data
    else:
        out += _bytes(9, array.astype(array.dtype.newbyteorder("<")).tobytes())
    return out + _bytes(8, name.encode())


def _attribute(name: str, value) -> bytes:
    out = _bytes(1, name.encode())
    if isinstance(value, bool):
        raise TypeError("use int for bool attributes")
    if isinstance(value, int):
        return out + _int(3, value) + _int(20, 2)
    if isinstance(value, float):
        return out + _varint((2 << 3) | 5) + struct.pack("<f", value) + _int(20, 1)
    if isinstance(value, str):
        return out + _bytes(4, value.encode()) + _int(20, 3)
    if isinstance(value, np.ndarray):
        return out + _bytes(5, tensor("", value)) + _int(20, 4)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        return out + b"".join(_int(8, v) for v in value) + _int(20, 7)
    raise TypeError(f"unsupported attribute value {value!r}")


def node(op_type: str, inputs, outputs, name: str = "", **attrs) -> bytes:
    out = b"".join(_bytes(1, i.encode()) for i in inputs)
    out += b"".join(_bytes(2, o.encode()) for o in outputs)
    out += _bytes(3, (name or f"{op_type}_{outputs[0]}").encode()) + _bytes(4, op_type.encode())
    return out + b"".join(_bytes(5, _attribute(k, v)) for k, v in attrs.items())


def value_info(name: str, dims, dtype=np.float32) -> bytes:
    dim_msgs = b""
    for d in dims:
        dim_msgs += _bytes(1, _bytes(2, d.encode()) if isinstance(d, str) else _int(1, d))
    tensor_type = _int(1, _ELEM[np.dtype(dtype)]) + _bytes(2, dim_msgs)
    return _bytes(1, name.encode()) + _bytes(2, _bytes(1, tensor_type))


def model(nodes, initializers, inputs, outputs, opset: int = 13) -> bytes:
    graph = b"".join(_bytes(1, n) for n in nodes) + _bytes(2, b"test")
    graph += b"".join(_bytes(5, t) for t in initializers)
    graph += b"".join(_bytes(11, v) for v in inputs) + b"".join(_bytes(12, v) for v in outputs)
    return _int(1, 7) + _bytes(2, b"tests") + _bytes(7, graph) + _bytes(8, _int(2, opset))
