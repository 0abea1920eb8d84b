"""Building blocks of the ONNX loader (`kyanite_b200/onnx.py`): a decoder for the protobuf wire format
of the ModelProto parts the loader reads (the `onnx` Python package is not required), shape-valued
tensors (`SignedSize`, kn-graph/src/onnx/typed_value.rs) and per-node argument tracking
(kn-graph/src/onnx/inputs.rs)."""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .graph import (BATCH, BinaryOp, DType, Graph, ONE, ReduceOp, Shape, Size, SliceRange, UnaryOp, Value,
                    _shape_size, broadcast_shape_symmetric, shape)

__all__ = ["OnnxError", "SignedSize", "parse_model"]


class OnnxError(ValueError):
    """Loading failed; the message names the node (name and op_type) where it applies."""


# --------------------------------------------------------------------------------------
# protobuf wire format
# --------------------------------------------------------------------------------------
def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = 0
    shift = 0
    while True:
        if pos >= len(buf):
            raise OnnxError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        shift += 7
        if b < 0x80:
            return result, pos
        if shift > 70:
            raise OnnxError("varint too long")


def _signed64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= 1 << 63 else v


def _fields(buf: bytes) -> List[Tuple[int, int, Union[int, bytes]]]:
    """(field number, wire type, payload) for every field of one message."""
    out = []
    pos = 0
    n = len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        field, wire = key >> 3, key & 7
        if wire == 0:
            value, pos = _varint(buf, pos)
        elif wire == 1:
            value = buf[pos:pos + 8]
            pos += 8
        elif wire == 2:
            length, pos = _varint(buf, pos)
            value = buf[pos:pos + length]
            if len(value) != length:
                raise OnnxError("truncated length-delimited field")
            pos += length
        elif wire == 5:
            value = buf[pos:pos + 4]
            pos += 4
        else:
            raise OnnxError(f"unsupported protobuf wire type {wire}")
        out.append((field, wire, value))
    return out


def _ints(fields, number: int) -> List[int]:
    """A repeated int64 field, packed or not."""
    out = []
    for f, wire, v in fields:
        if f != number:
            continue
        if wire == 0:
            out.append(_signed64(v))
        else:
            pos = 0
            while pos < len(v):
                x, pos = _varint(v, pos)
                out.append(_signed64(x))
    return out


def _floats(fields, number: int, fmt: str = "f") -> List[float]:
    size = struct.calcsize(fmt)
    out = []
    for f, wire, v in fields:
        if f != number:
            continue
        if len(v) % size != 0:
            raise OnnxError("packed float field with a partial element")
        out.extend(x[0] for x in struct.iter_unpack("<" + fmt, v))
    return out


def _one(fields, number: int, default=None):
    for f, _, v in fields:
        if f == number:
            return v
    return default


def _all(fields, number: int):
    return [v for f, _, v in fields if f == number]


def _string(fields, number: int, default: str = "") -> str:
    v = _one(fields, number)
    return default if v is None else bytes(v).decode("utf-8")


# ONNX TensorProto.DataType -> DType (load.rs:1357-1384); everything else is unsupported
_ONNX_DTYPES = {1: DType.F32, 11: DType.F64, 2: DType.U8, 3: DType.I8, 4: DType.U16, 5: DType.I16,
                6: DType.I32, 7: DType.I64, 12: DType.U32, 13: DType.U64, 9: DType.BOOL}


def _resolve_dtype(data_type: int, what: str) -> DType:
    if data_type not in _ONNX_DTYPES:
        raise OnnxError(f"unsupported ONNX data type {data_type} for {what}")
    return _ONNX_DTYPES[data_type]


@dataclass
class TensorProto:
    name: str
    dims: Tuple[int, ...]
    data_type: int
    array: np.ndarray


def _parse_tensor(buf: bytes, external: Optional[Callable[[str, int, Optional[int]], bytes]] = None) -> TensorProto:
    """TensorProto -> numpy (load.rs:1227-1330): typed fields when present, else `raw_data`."""
    f = _fields(buf)
    name = _string(f, 8)
    dims = tuple(_ints(f, 1))
    data_type = int(_one(f, 2, 0))
    dtype = _resolve_dtype(data_type, f"tensor {name!r}")
    count = int(np.prod(dims, dtype=np.int64)) if dims else 1
    raw = _one(f, 9, b"")
    if int(_one(f, 14, 0)) == 1:     # data_location EXTERNAL
        entries = {}
        for e in _all(f, 13):
            ef = _fields(e)
            entries[_string(ef, 1)] = _string(ef, 2)
        if external is None:
            raise OnnxError(f"tensor {name!r} refers to external data, which is not allowed here")
        length = int(entries["length"]) if "length" in entries else None
        if length is not None and length != count * dtype.size_bytes:
            raise OnnxError(f"external data length mismatch for tensor {name!r}")
        raw = external(entries["location"], int(entries.get("offset", 0)), length or count * dtype.size_bytes)
    npdt = dtype.np
    if dtype == DType.F32 and _all(f, 4):
        arr = np.array(_floats(f, 4, "f"), dtype=npdt)
    elif dtype == DType.F64 and _all(f, 10):
        arr = np.array(_floats(f, 10, "d"), dtype=npdt)
    elif dtype == DType.I64 and _all(f, 7):
        arr = np.array(_ints(f, 7), dtype=npdt)
    elif dtype in (DType.U32, DType.U64) and _all(f, 11):
        arr = np.array([v & ((1 << 64) - 1) for v in _ints(f, 11)], dtype=np.uint64).astype(npdt)
    elif dtype in (DType.I8, DType.I16, DType.I32, DType.U8, DType.U16, DType.BOOL) and _all(f, 5):
        vals = np.array(_ints(f, 5), dtype=np.int64)
        arr = (vals != 0) if dtype == DType.BOOL else vals.astype(npdt)
    elif dtype == DType.BOOL:
        arr = np.frombuffer(bytes(raw), dtype=np.uint8) != 0
    else:
        arr = np.frombuffer(bytes(raw), dtype=npdt.newbyteorder("<")).astype(npdt)
    if arr.size != count:
        raise OnnxError(f"tensor {name!r}: {arr.size} elements for shape {dims}")
    return TensorProto(name, dims, data_type, np.array(arr.reshape(dims), dtype=npdt, order="C", copy=True))


@dataclass
class NodeProto:
    name: str
    op_type: str
    inputs: List[str]
    outputs: List[str]
    attributes: Dict[str, tuple]      # name -> (kind, value); kind in f i s t floats ints


@dataclass
class ValueInfoProto:
    name: str
    elem_type: int
    dims: List[Union[int, str]]       # int for dim_value, str for dim_param


@dataclass
class ModelProto:
    nodes: List[NodeProto]
    initializers: List[TensorProto]
    inputs: List[ValueInfoProto]
    outputs: List[ValueInfoProto]
    opset: int


def _parse_attribute(buf: bytes, external) -> Tuple[str, tuple]:
    f = _fields(buf)
    name = _string(f, 1)
    kind = int(_one(f, 20, 0))
    # AttributeType: FLOAT 1, INT 2, STRING 3, TENSOR 4, FLOATS 6, INTS 7
    if kind == 1 or (kind == 0 and _one(f, 2) is not None):
        return name, ("f", struct.unpack("<f", _one(f, 2))[0])
    if kind == 2 or (kind == 0 and _one(f, 3) is not None):
        return name, ("i", _signed64(_one(f, 3, 0)))
    if kind == 3 or (kind == 0 and _one(f, 4) is not None):
        return name, ("s", bytes(_one(f, 4, b"")).decode("utf-8"))
    if kind == 4 or (kind == 0 and _one(f, 5) is not None):
        return name, ("t", _parse_tensor(_one(f, 5), external))
    if kind == 6:
        return name, ("floats", _floats(f, 7, "f"))
    if kind == 7 or kind == 0:
        return name, ("ints", _ints(f, 8))
    raise OnnxError(f"attribute {name!r} has unsupported type {kind}")


def _parse_value_info(buf: bytes) -> ValueInfoProto:
    f = _fields(buf)
    name = _string(f, 1)
    type_proto = _one(f, 2)
    if type_proto is None:
        raise OnnxError(f"value {name!r} has no type")
    tensor_type = _one(_fields(type_proto), 1)
    if tensor_type is None:
        raise OnnxError(f"value {name!r} is not a tensor")
    tf = _fields(tensor_type)
    elem_type = int(_one(tf, 1, 0))
    shape_proto = _one(tf, 2)
    if shape_proto is None:
        raise OnnxError(f"value {name!r} has no shape")
    dims: List[Union[int, str]] = []
    for d in _all(_fields(shape_proto), 1):
        df = _fields(d)
        if _one(df, 1) is not None:
            dims.append(_signed64(_one(df, 1)))
        elif _one(df, 2) is not None:
            dims.append(_string(df, 2))
        else:
            raise OnnxError(f"value {name!r} has a dimension without value")
    return ValueInfoProto(name, elem_type, dims)


def parse_model(buf: bytes, external=None) -> ModelProto:
    """Decode the parts of a ModelProto the loader needs."""
    model = _fields(buf)
    graph_bytes = _one(model, 7)
    if graph_bytes is None:
        raise OnnxError("model has no graph")
    opset = 0
    for o in _all(model, 8):
        of = _fields(o)
        if _string(of, 1) in ("", "ai.onnx"):
            opset = int(_one(of, 2, 0))
    g = _fields(graph_bytes)
    nodes = []
    for nb in _all(g, 1):
        nf = _fields(nb)
        attrs = dict(_parse_attribute(a, external) for a in _all(nf, 5))
        nodes.append(NodeProto(_string(nf, 3), _string(nf, 4), [bytes(v).decode() for v in _all(nf, 1)],
                               [bytes(v).decode() for v in _all(nf, 2)], attrs))
    return ModelProto(nodes, [_parse_tensor(t, external) for t in _all(g, 5)],
                      [_parse_value_info(v) for v in _all(g, 11)], [_parse_value_info(v) for v in _all(g, 12)], opset)


# --------------------------------------------------------------------------------------
# shape-valued tensors (typed_value.rs:18-22, 116-296)
# --------------------------------------------------------------------------------------
@dataclass(frozen=True)
class SignedSize:
    """`factor * batch_size ** exp` with a signed factor: an element of a shape computation."""
    factor: int
    exp: int = 0

    def __post_init__(self):
        if self.factor == 0 and self.exp != 0:
            object.__setattr__(self, "exp", 0)

    @staticmethod
    def from_size(s: Size) -> "SignedSize":
        return SignedSize(s.factor, s.exp)

    def to_size(self) -> Size:
        if self.factor < 0:
            raise OnnxError(f"size {self} is negative")
        return Size(self.factor, self.exp)

    @property
    def fixed(self) -> Optional[int]:
        return self.factor if self.exp == 0 else None

    def __neg__(self):
        return SignedSize(-self.factor, self.exp)

    def add(self, other: "SignedSize") -> Optional["SignedSize"]:
        if self.factor == 0:
            return other
        if other.factor == 0:
            return self
        if self.exp != other.exp:
            return None
        return SignedSize(self.factor + other.factor, self.exp)

    def sub(self, other: "SignedSize") -> Optional["SignedSize"]:
        return self.add(-other)

    def mul(self, other: "SignedSize") -> "SignedSize":
        return SignedSize(self.factor * other.factor, self.exp + other.exp)

    def floor_div(self, other: "SignedSize") -> Optional["SignedSize"]:
        if self.exp < other.exp or other.factor == 0:
            return None
        # the reference divides two i64 with Rust `/`, which truncates toward zero
        q = abs(self.factor) // abs(other.factor)
        if (self.factor < 0) != (other.factor < 0):
            q = -q
        return SignedSize(q, self.exp - other.exp)

    def __repr__(self):
        s = Size(abs(self.factor), self.exp)
        return ("-" if self.factor < 0 else "") + repr(s)


OnnxValue = Union[Value, np.ndarray]     # a graph value, or an object array of SignedSize


def _size_array(items, shp) -> np.ndarray:
    arr = np.empty(len(items), dtype=object)
    for i, x in enumerate(items):
        arr[i] = x
    return arr.reshape(shp)


def _is_size(x: OnnxValue) -> bool:
    return isinstance(x, np.ndarray)


def _new_size(arr: np.ndarray, graph: Graph) -> OnnxValue:
    """Keep a size tensor only while it mentions the batch size; otherwise it is an I64 constant
    (typed_value.rs:37-45)."""
    flat = list(arr.reshape(-1))
    if any(x.exp != 0 for x in flat):
        return arr
    ints = np.array([x.factor for x in flat], dtype=np.int64).reshape(arr.shape)
    return graph.constant_tensor(ints)


def _as_size(x: OnnxValue, graph: Graph, what: str) -> np.ndarray:
    if _is_size(x):
        return x
    const = graph.as_const(x)
    if const is None:
        raise OnnxError(f"{what}: expected a constant or a shape, got a computed value")
    if const.dtype != np.int64:
        raise OnnxError(f"{what}: expected I64, got {const.dtype}")
    return _size_array([SignedSize(int(v)) for v in const.reshape(-1)], const.shape)


def _as_signed_shape(x: OnnxValue, graph: Graph, what: str) -> List[SignedSize]:
    arr = _as_size(x, graph, what)
    if arr.ndim != 1:
        raise OnnxError(f"{what}: expected a rank-1 shape tensor, got shape {arr.shape}")
    return list(arr)


def _as_shape(x: OnnxValue, graph: Graph, what: str) -> Shape:
    return tuple(s.to_size() for s in _as_signed_shape(x, graph, what))


def _shape_of(x: OnnxValue, graph: Graph) -> Shape:
    return shape(*x.shape) if _is_size(x) else graph[x].shape


def _unwrap_value(x: OnnxValue, what: str) -> Value:
    if _is_size(x):
        raise OnnxError(f"{what}: a batch-dependent shape tensor cannot be used as a value here")
    return x


def _abs_axis(axis: int, rank: int) -> int:
    """load.rs:1386-1394: negative axes count from the end; i64::MAX means `rank`."""
    if axis == (1 << 63) - 1:
        return rank
    if axis < 0:
        if -axis > rank:
            raise OnnxError(f"axis {axis} out of range for rank {rank}")
        return rank + axis
    return axis


class _NodeArgs:
    """Inputs and attributes of one node with use tracking (onnx/inputs.rs): asking twice for the same
    input is a bug, leaving one unused is an error."""

    def __init__(self, node: NodeProto, store: Dict[str, OnnxValue]):
        self.node = node
        self.what = f"node {node.name!r} ({node.op_type})"
        self.inputs: List[Optional[OnnxValue]] = []
        for i, name in enumerate(node.inputs):
            if name == "":
                self.inputs.append(None)      # a missing optional input
            elif name not in store:
                raise OnnxError(f"{self.what}: input {i} {name!r} does not exist")
            else:
                self.inputs.append(store[name])
        self.used_inputs = [x is None for x in self.inputs]
        self.attrs = dict(node.attributes)

    def fail(self, message: str) -> OnnxError:
        return OnnxError(f"{self.what}: {message}")

    # inputs
    def optional(self, index: int) -> Optional[OnnxValue]:
        if index >= len(self.inputs):
            return None
        if self.inputs[index] is not None:
            assert not self.used_inputs[index], f"input {index} of {self.what} used twice"
        self.used_inputs[index] = True
        return self.inputs[index]

    def required(self, index: int) -> OnnxValue:
        v = self.optional(index)
        if v is None:
            raise self.fail(f"missing input {index} (node has {len(self.inputs)})")
        return v

    def value(self, index: int) -> Value:
        return _unwrap_value(self.required(index), self.what)

    def optional_value(self, index: int) -> Optional[Value]:
        v = self.optional(index)
        return None if v is None else _unwrap_value(v, self.what)

    def all_variadic(self) -> List[OnnxValue]:
        out = []
        for i in range(len(self.inputs)):
            v = self.optional(i)
            if v is None:
                raise self.fail(f"variadic input {i} is missing")
            out.append(v)
        return out

    # attributes
    def _take(self, name: str, kind: str, required: bool):
        if name not in self.attrs:
            if required:
                raise self.fail(f"missing attribute {name!r}")
            return None
        k, v = self.attrs.pop(name)
        if kind == "f" and k == "i":
            k, v = "f", float(v)
        if k != kind:
            raise self.fail(f"attribute {name!r} has type {k}, expected {kind}")
        return v

    def take_int(self, name): return self._take(name, "i", True)
    def maybe_int(self, name): return self._take(name, "i", False)
    def take_float(self, name): return self._take(name, "f", True)
    def maybe_float(self, name): return self._take(name, "f", False)
    def take_ints(self, name): return self._take(name, "ints", True)
    def maybe_ints(self, name): return self._take(name, "ints", False)
    def take_string(self, name): return self._take(name, "s", True)
    def maybe_string(self, name): return self._take(name, "s", False)
    def take_tensor(self, name): return self._take(name, "t", True)
    def maybe_tensor(self, name): return self._take(name, "t", False)

    def check_leftovers(self):
        if self.attrs:
            raise self.fail(f"leftover attributes {sorted(self.attrs)}")
        left = [i for i, used in enumerate(self.used_inputs) if not used]
        if left:
            raise self.fail(f"leftover inputs {left}")
