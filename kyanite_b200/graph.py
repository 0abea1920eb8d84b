"""Graph IR builder and wire format.

This is the *input format* of the executor: an SSA DAG of values in topological
order, each with a symbolic shape (`factor * batch^exp` per dim), a dtype and a
creating operation.  The builder mirrors the behaviour of the reference's
`Graph` builder (kn-graph/src/graph.rs:363-1428), including the normalisations
its tests rely on:

* value de-duplication through a back map          (graph.rs:535-574)
* view-of-view collapse                            (graph.rs:632-639)
* permute-of-permute fusion                        (graph.rs:745-755)
* identity-operand skipping in `binary`            (graph.rs:1297-1307)
* gather with a single-valued constant index
  -> slice + repeat                                (graph.rs:872-881)
* trivial slice / cast / reduce skipping           (graph.rs:783-786, 1256-1261, 1168-1171)

`Graph.to_bytes()` serialises the graph into the flat little-endian blob that
crosses the C ABI (`kn_graph_from_blob`).  A host written in another language
emits the same blob by walking its own value list.
"""
from __future__ import annotations

import enum
import math
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np

__all__ = [
    "DType", "Size", "BATCH", "Shape", "SliceRange", "UnaryOp", "BinaryOp", "ReduceOp",
    "OpKind", "Value", "ValueInfo", "Graph", "shape",
]


# --------------------------------------------------------------------------------------
# dtypes (kn-graph/src/dtype.rs:25-37, plus F16 which the reference does not have)
# --------------------------------------------------------------------------------------
class DType(enum.IntEnum):
    F32 = 0
    F64 = 1
    I8 = 2
    I16 = 3
    I32 = 4
    I64 = 5
    U8 = 6
    U16 = 7
    U32 = 8
    U64 = 9
    BOOL = 10
    F16 = 11  # extension: half storage, not present in the reference

    @property
    def np(self) -> np.dtype:
        return _NP_OF[self]

    @property
    def size_bytes(self) -> int:
        return _NP_OF[self].itemsize

    @property
    def is_float(self) -> bool:
        return self in (DType.F32, DType.F64, DType.F16)

    @property
    def is_int(self) -> bool:
        return DType.I8 <= self <= DType.U64

    @property
    def is_signed(self) -> bool:
        return self.is_float or self in (DType.I8, DType.I16, DType.I32, DType.I64)

    @property
    def is_bool(self) -> bool:
        return self == DType.BOOL

    @staticmethod
    def of(np_dtype) -> "DType":
        return _OF_NP[np.dtype(np_dtype)]

    def specials(self):
        """(zero, one, min, max) as numpy scalars; float min/max are -inf/+inf (dtype.rs:134-148)."""
        t = self.np.type
        if self.is_float:
            return t(0), t(1), t(-np.inf), t(np.inf)
        if self.is_bool:
            return t(False), t(True), t(False), t(True)
        info = np.iinfo(self.np)
        return t(0), t(1), t(info.min), t(info.max)


_NP_OF = {
    DType.F32: np.dtype(np.float32), DType.F64: np.dtype(np.float64),
    DType.I8: np.dtype(np.int8), DType.I16: np.dtype(np.int16),
    DType.I32: np.dtype(np.int32), DType.I64: np.dtype(np.int64),
    DType.U8: np.dtype(np.uint8), DType.U16: np.dtype(np.uint16),
    DType.U32: np.dtype(np.uint32), DType.U64: np.dtype(np.uint64),
    DType.BOOL: np.dtype(np.bool_), DType.F16: np.dtype(np.float16),
}
_OF_NP = {v: k for k, v in _NP_OF.items()}


# --------------------------------------------------------------------------------------
# symbolic sizes and shapes (kn-graph/src/shape.rs:27-44, 234-317)
# --------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Size:
    """`factor * batch_size ** exp`; zero is normalised to exp 0."""
    factor: int
    exp: int = 0

    def __post_init__(self):
        if self.factor == 0 and self.exp != 0:
            object.__setattr__(self, "exp", 0)

    @staticmethod
    def of(x: Union["Size", int]) -> "Size":
        return x if isinstance(x, Size) else Size(int(x), 0)

    def eval(self, batch_size: int) -> int:
        return self.factor * batch_size ** self.exp

    @property
    def is_fixed(self) -> bool:
        return self.exp == 0

    def unwrap_fixed(self, what: str = "size") -> int:
        if self.exp != 0:
            raise ValueError(f"{what} must be fixed, but got size {self}")
        return self.factor

    def __mul__(self, other) -> "Size":
        o = Size.of(other)
        return Size(self.factor * o.factor, self.exp + o.exp)

    __rmul__ = __mul__

    def try_add(self, other) -> Optional["Size"]:
        o = Size.of(other)
        if self.factor == 0:
            return o
        if o.factor == 0:
            return self
        if self.exp != o.exp:
            return None
        return Size(self.factor + o.factor, self.exp)

    def __repr__(self):
        if self.exp == 0:
            return str(self.factor)
        b = "B" if self.exp == 1 else f"B^{self.exp}"
        return b if self.factor == 1 else f"{self.factor}{b}"


BATCH = Size(1, 1)
ONE = Size(1, 0)
ZERO = Size(0, 0)

Shape = Tuple[Size, ...]


def shape(*dims) -> Shape:
    """`shape(BATCH, 16, 8, 8)`; also accepts a single iterable."""
    if len(dims) == 1 and not isinstance(dims[0], (Size, int, np.integer)):
        dims = tuple(dims[0])
    return tuple(Size.of(d) for d in dims)


def _shape_size(s: Shape) -> Size:
    r = ONE
    for d in s:
        r = r * d
    return r


def _shape_eval(s: Shape, batch_size: int) -> Tuple[int, ...]:
    return tuple(d.eval(batch_size) for d in s)


def _replace(s: Shape, axis: int, repl: Sequence[Size]) -> Shape:
    return tuple(s[:axis]) + tuple(repl) + tuple(s[axis + 1:])


def _assert_axis(s: Shape, axis: int):
    if not (0 <= axis < len(s)):
        raise ValueError(f"Axis {axis} out of bounds for {s}")


def broadcast_shape_symmetric(left: Shape, right: Shape) -> Shape:
    """Multidirectional broadcasting (graph.rs:1431-1448)."""
    rank = max(len(left), len(right))
    left = (ONE,) * (rank - len(left)) + tuple(left)
    right = (ONE,) * (rank - len(right)) + tuple(right)
    out = []
    for l, r in zip(left, right):
        if l == ONE:
            out.append(r)
        elif r == ONE or l == r:
            out.append(l)
        else:
            raise ValueError(f"Cannot broadcast {l} and {r} in shapes {left} and {right}")
    return tuple(out)


@dataclass(frozen=True)
class SliceRange:
    """`start..end` with `step`; `(end - start) % step == 0` (graph.rs:1549-1595)."""
    start: int
    end: int
    step: int = 1

    def __post_init__(self):
        if self.end < self.start:
            raise ValueError(f"Invalid range {self}: bounds cannot be decreasing")
        if self.step == 0:
            raise ValueError(f"Invalid range {self}: step cannot be 0")
        if (self.end - self.start) % self.step != 0:
            raise ValueError(f"Invalid range {self}: bounds must differ by a multiple of step")

    @staticmethod
    def single(index: int) -> "SliceRange":
        return SliceRange(index, index + 1, 1)

    def assert_in_bounds(self, size: int):
        ok = self.start == self.end or (self.start < size and self.end - (self.step - 1) <= size)
        if not ok:
            raise ValueError(f"{self} out of bounds for axis of size {size}")


class UnaryOp(enum.IntEnum):
    ABS = 0
    NEG = 1
    SIN = 2
    COS = 3
    EXP = 4
    LOG = 5
    SQRT = 6
    SIGMOID = 7
    TANH = 8
    ERF = 9
    MISH = 10
    SOFTPLUS = 11
    VALUE_CAST = 12
    BIT_CAST = 13


UNARY_FLOAT_OPS = [UnaryOp.SIN, UnaryOp.COS, UnaryOp.EXP, UnaryOp.LOG, UnaryOp.SQRT, UnaryOp.SIGMOID,
                   UnaryOp.TANH, UnaryOp.ERF, UnaryOp.MISH, UnaryOp.SOFTPLUS]
UNARY_ALL = [UnaryOp.ABS, UnaryOp.NEG] + UNARY_FLOAT_OPS


class BinaryOp(enum.IntEnum):
    ADD = 0
    SUB = 1
    MUL = 2
    DIV = 3
    MIN = 4
    MAX = 5
    POW = 6


BINARY_ALL = list(BinaryOp)


class ReduceOp(enum.IntEnum):
    SUM = 0
    MEAN = 1
    PROD = 2
    MAX = 3
    MIN = 4


REDUCE_ALL = list(ReduceOp)


class OpKind(enum.IntEnum):
    INPUT = 0
    CONSTANT = 1
    VIEW = 2
    BROADCAST = 3
    PERMUTE = 4
    SLICE = 5
    FLIP = 6
    GATHER = 7
    CONCAT = 8
    CONV = 9
    MATMUL = 10
    UNARY = 11
    BINARY = 12
    SOFTMAX = 13
    LAYERNORM = 14
    REDUCE = 15
    ALL_REDUCE = 16    # extension (no counterpart in the reference): sum over the ranks of a communicator


@dataclass(frozen=True)
class Value:
    index: int
    check: int

    def __repr__(self):
        return f"Value({self.index})"


@dataclass
class ValueInfo:
    shape: Shape
    dtype: DType
    kind: OpKind
    inputs: Tuple[int, ...] = ()
    # op attributes; only the ones that apply are set
    input_index: int = 0                       # INPUT
    tensor: Optional[np.ndarray] = None        # CONSTANT (C-contiguous)
    permutation: Tuple[int, ...] = ()          # PERMUTE
    axis: int = 0                              # SLICE FLIP GATHER CONCAT SOFTMAX LAYERNORM
    range: Optional[SliceRange] = None         # SLICE
    conv: Tuple[int, int, int, int] = (1, 1, 0, 0)   # stride_y, stride_x, padding_y, padding_x
    unary_op: Optional[UnaryOp] = None
    cast_to: Optional[DType] = None            # VALUE_CAST / BIT_CAST target
    binary_op: Optional[BinaryOp] = None
    reduce_op: Optional[ReduceOp] = None
    axes: Tuple[int, ...] = ()                 # REDUCE
    eps: float = 0.0                           # LAYERNORM
    debug_id: str = ""
    non_output_uses: int = 0

    def key(self):
        t = None
        if self.tensor is not None:
            t = (self.tensor.shape, self.tensor.dtype.str, self.tensor.tobytes())
        eps_bits = struct.pack("<f", self.eps)
        return (self.shape, self.dtype, self.kind, self.inputs, self.input_index, t, self.permutation,
                self.axis, self.range, self.conv, self.unary_op, self.cast_to, self.binary_op,
                self.reduce_op, self.axes, eps_bits)


_next_check = [1]


class Graph:
    """Builder for the executor's input graph.  Method names and argument meaning follow the
    reference builder (kn-graph/src/graph.rs)."""

    def __init__(self):
        self.check = _next_check[0]
        _next_check[0] += 1
        self.values: List[ValueInfo] = []
        self._back_map = {}
        self.inputs: List[Value] = []
        self.outputs: List[Value] = []

    # ---------------------------------------------------------------- basic access
    def __getitem__(self, v: Value) -> ValueInfo:
        self._check_contains(v)
        return self.values[v.index]

    def _check_contains(self, v: Value):
        if not isinstance(v, Value) or v.check != self.check or v.index >= len(self.values):
            raise ValueError(f"Value {v!r} does not belong to this graph")

    def _v(self, index: int) -> Value:
        return Value(index, self.check)

    def shape_dtype(self, v: Value) -> Tuple[Shape, DType]:
        info = self[v]
        return info.shape, info.dtype

    def all_values(self) -> List[Value]:
        return [self._v(i) for i in range(len(self.values))]

    def input_shapes(self) -> List[Shape]:
        return [self[v].shape for v in self.inputs]

    def output_shapes(self) -> List[Shape]:
        return [self[v].shape for v in self.outputs]

    def is_hidden(self, v: Value) -> bool:
        return v not in self.inputs and v not in self.outputs

    def is_hidden_with_uses(self, v: Value, users: int) -> bool:
        return self.is_hidden(v) and self[v].non_output_uses == users

    def set_debug_id(self, v: Value, debug_id: str):
        self[v].debug_id = debug_id

    # ---------------------------------------------------------------- constant queries
    def as_single_const(self, v: Value):
        """A numpy scalar if every element of `v` is the same constant (graph.rs:490-527)."""
        info = self[v]
        k = info.kind
        if k == OpKind.INPUT:
            return None
        if k == OpKind.CONSTANT:
            t = info.tensor
            if t.size == 0:
                return None
            flat = t.reshape(-1)
            e = flat[0]
            if t.dtype.kind == "f":
                same = bool(np.all((flat == e) | (np.isnan(flat) & np.isnan(e))))
            else:
                same = bool(np.all(flat == e))
            return e if same else None
        if k in (OpKind.VIEW, OpKind.BROADCAST, OpKind.PERMUTE, OpKind.SLICE, OpKind.FLIP, OpKind.GATHER):
            return self.as_single_const(self._v(info.inputs[0]))
        if k == OpKind.CONCAT:
            if not info.inputs:
                return None
            f = self.as_single_const(self._v(info.inputs[0]))
            if f is None:
                return None
            for i in info.inputs:
                if not self.is_const_filled_with(self._v(i), f):
                    return None
            return f
        if k == OpKind.UNARY:
            x = self.as_single_const(self._v(info.inputs[0]))
            if x is None:
                return None
            return _scalar_unary(info.unary_op, info.cast_to, x)
        if k == OpKind.BINARY:
            l = self.as_single_const(self._v(info.inputs[0]))
            r = self.as_single_const(self._v(info.inputs[1]))
            if l is None or r is None:
                return None
            return _scalar_binary(info.binary_op, l, r)
        return None

    def as_const(self, v: Value) -> Optional[np.ndarray]:
        """The value as a numpy tensor if it depends on constants only (graph.rs:434-474), else None.
        Covers the data-movement ops and elementwise arithmetic, which is what shape computations and
        the model loaders need; contractions, normalisations and reductions of constants return None.
        Shapes with a batch factor are not constant."""
        memo: Dict[int, Optional[np.ndarray]] = {}
        order = [v.index]
        seen = {v.index}
        i = 0
        while i < len(order):       # operands of the cone, iteratively (no recursion limit)
            for j in self.values[order[i]].inputs:
                if j not in seen:
                    seen.add(j)
                    order.append(j)
            i += 1
        for idx in sorted(order):   # operands always precede their users
            info = self.values[idx]
            ops = [memo[j] for j in info.inputs]
            memo[idx] = None
            if any(o is None for o in ops) or not all(d.is_fixed for d in info.shape):
                continue
            out_shape = tuple(d.factor for d in info.shape)
            k = info.kind
            if k == OpKind.CONSTANT:
                res = info.tensor
            elif k == OpKind.VIEW:
                res = ops[0].reshape(out_shape)
            elif k == OpKind.BROADCAST:
                res = np.broadcast_to(ops[0], out_shape)
            elif k == OpKind.PERMUTE:
                res = np.transpose(ops[0], info.permutation)
            elif k == OpKind.SLICE:
                r = info.range
                index = [slice(None)] * ops[0].ndim
                index[info.axis] = slice(r.start, r.end, r.step)
                res = ops[0][tuple(index)]
            elif k == OpKind.FLIP:
                res = np.flip(ops[0], info.axis)
            elif k == OpKind.GATHER:
                indices = ops[1].astype(np.int64)
                size = ops[0].shape[info.axis]
                if indices.size and (indices.min() < 0 or indices.max() >= size):
                    continue
                res = np.take(ops[0], indices.reshape(-1), axis=info.axis)
            elif k == OpKind.CONCAT:
                res = np.concatenate(ops, axis=info.axis) if ops else np.zeros(out_shape, info.dtype.np)
            elif k == OpKind.UNARY:
                res = np.array([_scalar_unary(info.unary_op, info.cast_to, x) for x in ops[0].reshape(-1)],
                               dtype=info.dtype.np)
            elif k == OpKind.BINARY:
                l, r = np.broadcast_arrays(ops[0], ops[1])
                res = np.array([_scalar_binary(info.binary_op, a, b) for a, b in zip(l.reshape(-1), r.reshape(-1))],
                               dtype=info.dtype.np)
            else:
                continue
            memo[idx] = np.array(res, dtype=info.dtype.np, order="C", copy=True).reshape(out_shape)
        return memo[v.index]

    def is_const_filled_with(self, v: Value, expected) -> bool:
        actual = self.as_single_const(v)
        if actual is None:
            return False
        if np.dtype(type(actual)) != np.dtype(type(expected)):
            return False
        if isinstance(actual, np.floating) and np.isnan(actual) and np.isnan(expected):
            return True
        return bool(actual == expected)

    def is_const_zero(self, v: Value) -> bool:
        return self.is_const_filled_with(v, self[v].dtype.specials()[0])

    def is_const_one(self, v: Value) -> bool:
        return self.is_const_filled_with(v, self[v].dtype.specials()[1])

    # ---------------------------------------------------------------- push
    def _push(self, info: ValueInfo) -> Value:
        key = info.key()
        found = self._back_map.get(key)
        if found is not None:
            return self._v(found)
        for i in info.inputs:
            if i >= len(self.values):
                raise ValueError("operand does not belong to this graph")
            self.values[i].non_output_uses += 1
        index = len(self.values)
        self.values.append(info)
        self._back_map[key] = index
        return self._v(index)

    # ---------------------------------------------------------------- leaf values
    def input(self, shp, dtype: DType = DType.F32) -> Value:
        shp = shape(shp)
        v = self._push(ValueInfo(shp, dtype, OpKind.INPUT, input_index=len(self.inputs)))
        self.inputs.append(v)
        return v

    def constant_tensor(self, tensor: np.ndarray) -> Value:
        tensor = np.asarray(tensor)
        if not tensor.flags.c_contiguous:
            tensor = tensor.copy(order="C")  # (ascontiguousarray would turn rank 0 into rank 1)
        dtype = DType.of(tensor.dtype)
        return self._push(ValueInfo(shape(tensor.shape), dtype, OpKind.CONSTANT, tensor=tensor))

    def constant(self, shp, data, dtype: DType = DType.F32) -> Value:
        shp = shape(shp)
        dims = [d.unwrap_fixed("constant shape") for d in shp]
        arr = np.asarray(data, dtype=dtype.np).reshape(dims)
        return self.constant_tensor(arr)

    def scalar(self, value, dtype: DType = DType.F32) -> Value:
        return self.constant_tensor(np.asarray(value, dtype=dtype.np).reshape(()))

    # ---------------------------------------------------------------- restriding ops
    def view(self, input: Value, new_shape) -> Value:
        new_shape = shape(new_shape)
        in_shape, dtype = self.shape_dtype(input)
        if new_shape == in_shape:
            return input
        if _shape_size(in_shape) != _shape_size(new_shape):
            raise ValueError(f"New shape {new_shape} must have the same size as old shape {in_shape}")
        info = self[input]
        inner = self._v(info.inputs[0]) if info.kind == OpKind.VIEW else input
        return self._push(ValueInfo(new_shape, dtype, OpKind.VIEW, inputs=(inner.index,)))

    def broadcast(self, input: Value, new_shape) -> Value:
        new_shape = shape(new_shape)
        in_shape, dtype = self.shape_dtype(input)
        if len(in_shape) > len(new_shape):
            raise ValueError(f"Cannot broadcast to a lower rank shape (from {in_shape} to {new_shape})")
        view_shape = (ONE,) * (len(new_shape) - len(in_shape)) + tuple(in_shape)
        curr = self.view(input, view_shape)
        for v, n in zip(view_shape, new_shape):
            if not (v == n or v == ONE):
                raise ValueError(f"Cannot broadcast from {in_shape} to {new_shape} because of axis ({v}, {n})")
        if view_shape == new_shape:
            return curr
        return self._push(ValueInfo(new_shape, dtype, OpKind.BROADCAST, inputs=(curr.index,)))

    def repeat_unary(self, input: Value, axis: int, count) -> Value:
        count = Size.of(count)
        in_shape, dtype = self.shape_dtype(input)
        if in_shape[axis] != ONE:
            raise ValueError(f"Input shape {in_shape} does not have dim 1 for axis {axis}")
        if count == ONE:
            return input
        new_shape = _replace(in_shape, axis, [count])
        return self._push(ValueInfo(new_shape, dtype, OpKind.BROADCAST, inputs=(input.index,)))

    def flatten(self, input: Value, start_axis: int) -> Value:
        old = self[input].shape
        if start_axis > len(old):
            raise ValueError(f"Flatten start axis {start_axis} out of bounds for {old}")
        flat = _shape_size(old[start_axis:])
        return self.view(input, tuple(old[:start_axis]) + (flat,))

    def permute(self, input: Value, permutation: Sequence[int]) -> Value:
        permutation = tuple(int(p) for p in permutation)
        info = self[input]
        if len(permutation) != len(info.shape):
            raise ValueError(f"Permutation rank must match input shape, got {permutation} and {info.shape}")
        if len(set(permutation)) != len(permutation):
            raise ValueError(f"Permutation cannot contain repeated axis, got {permutation}")
        if any(not (0 <= p < len(info.shape)) for p in permutation):
            raise ValueError(f"Permutation axis out of bounds, got {permutation}")
        if info.kind == OpKind.PERMUTE:
            inner = self._v(info.inputs[0])
            full = tuple(info.permutation[i] for i in permutation)
        else:
            inner, full = input, permutation
        inner_shape = self[inner].shape
        result_shape = tuple(inner_shape[i] for i in full)
        return self._push(ValueInfo(result_shape, info.dtype, OpKind.PERMUTE, inputs=(inner.index,),
                                    permutation=full))

    def slice(self, input: Value, axis: int, range: Union[SliceRange, Tuple[int, ...]]) -> Value:
        if not isinstance(range, SliceRange):
            range = SliceRange(*range)
        info = self[input]
        _assert_axis(info.shape, axis)
        input_size = info.shape[axis].unwrap_fixed("Slice axis length")
        range.assert_in_bounds(input_size)
        new_size = (range.end - range.start) // range.step
        if range == SliceRange(0, input_size, 1):
            return input
        new_shape = _replace(info.shape, axis, [Size(new_size)])
        return self._push(ValueInfo(new_shape, info.dtype, OpKind.SLICE, inputs=(input.index,), axis=axis,
                                    range=range))

    def index(self, input: Value, axis: int, index: int) -> Value:
        new_shape = _replace(self[input].shape, axis, [])
        sliced = self.slice(input, axis, SliceRange.single(index))
        return self.view(sliced, new_shape)

    def flip(self, input: Value, axis: int) -> Value:
        info = self[input]
        _assert_axis(info.shape, axis)
        return self._push(ValueInfo(info.shape, info.dtype, OpKind.FLIP, inputs=(input.index,), axis=axis))

    def repeat(self, input: Value, axis: int, count) -> Value:
        return self._repeat_impl(input, axis, Size.of(count), False)

    def repeat_interleave(self, input: Value, axis: int, count) -> Value:
        return self._repeat_impl(input, axis, Size.of(count), True)

    def _repeat_impl(self, input: Value, axis: int, count: Size, inner: bool) -> Value:
        in_shape = self[input].shape
        _assert_axis(in_shape, axis)
        if in_shape[axis] == ONE:
            return self.repeat_unary(input, axis, count)
        new_size = in_shape[axis] * count
        dummy_axis = axis + 1 if inner else axis
        extra_shape = tuple(in_shape[:dummy_axis]) + (ONE,) + tuple(in_shape[dummy_axis:])
        extra = self.view(input, extra_shape)
        broad = self.repeat_unary(extra, dummy_axis, count)
        return self.view(broad, _replace(in_shape, axis, [new_size]))

    # ---------------------------------------------------------------- indexing ops
    def gather(self, input: Value, axis: int, indices: Value) -> Value:
        in_shape, dtype = self.shape_dtype(input)
        idx_shape, idx_dtype = self.shape_dtype(indices)
        _assert_axis(in_shape, axis)
        if not idx_dtype.is_int:
            raise ValueError(f"Indices must be integers, got {idx_dtype!r}")
        result_shape = _replace(in_shape, axis, idx_shape)
        result_shape_flat = _replace(in_shape, axis, [_shape_size(idx_shape)])
        flat_indices = self.flatten(indices, 0)
        flat_size = self[flat_indices].shape[0]
        single = self.as_single_const(indices)
        if single is not None:
            index = int(single)
            if index < 0:
                raise ValueError("negative constant gather index")
            one = self.slice(input, axis, SliceRange.single(index))
            result_flat = self.repeat(one, axis, flat_size)
            assert self[result_flat].shape == result_shape_flat
        else:
            result_flat = self._push(ValueInfo(result_shape_flat, dtype, OpKind.GATHER,
                                               inputs=(input.index, flat_indices.index), axis=axis))
        return self.view(result_flat, result_shape)

    def concat(self, inputs: Sequence[Value], axis: int, base_shape=None, dtype: Optional[DType] = None) -> Value:
        inputs = list(inputs)
        if base_shape is None:
            if not inputs:
                raise ValueError("Cannot infer concatenation shape without any inputs")
            base_shape = _replace(self[inputs[0]].shape, axis, [ZERO])
        else:
            base_shape = shape(base_shape)
        if dtype is None:
            if not inputs:
                raise ValueError("Cannot infer concatenation dtype without any inputs")
            dtype = self[inputs[0]].dtype
        total = ZERO
        for v in inputs:
            if _replace(self[v].shape, axis, [ZERO]) != base_shape:
                raise ValueError("All concatenated values must match base shape on non-concatenated axes")
            if self[v].dtype != dtype:
                raise ValueError("All concatenated values must have the same dtype")
            total = total.try_add(self[v].shape[axis])
            if total is None:
                raise ValueError("Could not add all concatenation sizes")
        result_shape = _replace(base_shape, axis, [total])
        inputs = [x for x in inputs if _shape_size(self[x].shape) != ZERO]
        if len(inputs) == 1:
            return inputs[0]
        return self._push(ValueInfo(result_shape, dtype, OpKind.CONCAT, inputs=tuple(x.index for x in inputs),
                                    axis=axis))

    def pad(self, input: Value, pad_amount: Sequence[Tuple[int, int]], pad_value: Value) -> Value:
        in_shape, dtype = self.shape_dtype(input)
        pv_shape, pv_dtype = self.shape_dtype(pad_value)
        if len(in_shape) != len(pad_amount):
            raise ValueError("Padding length must match input rank")
        if dtype != pv_dtype:
            raise ValueError("Padding value dtype must match input dtype")
        if pv_shape != ():
            raise ValueError("Padding value must be scalar")
        curr = input
        for i, (before, after) in enumerate(pad_amount):
            cs = self[curr].shape
            b = self.broadcast(pad_value, _replace(cs, i, [Size(before)]))
            a = self.broadcast(pad_value, _replace(cs, i, [Size(after)]))
            curr = self.concat([b, curr, a], i)
        return curr

    # ---------------------------------------------------------------- contractions
    def conv(self, input: Value, filter: Value, stride_y: int, stride_x: int, padding_y: int,
             padding_x: int) -> Value:
        in_shape, in_dtype = self.shape_dtype(input)
        f_shape, f_dtype = self.shape_dtype(filter)
        if in_dtype != f_dtype:
            raise ValueError("Convolution input and filter must have the same dtype")
        if len(in_shape) != 4:
            raise ValueError("Convolution input must have rank 4")
        if len(f_shape) != 4:
            raise ValueError("Convolution filter must have rank 4")
        batch, in_c, in_h, in_w = in_shape
        out_c, in_c_check, k_h, k_w = f_shape
        in_c = in_c.unwrap_fixed("Conv input channels")
        in_h = in_h.unwrap_fixed("Conv input height")
        in_w = in_w.unwrap_fixed("Conv input width")
        out_c = out_c.unwrap_fixed("Conv output channels")
        in_c_check = in_c_check.unwrap_fixed("Filter input channels")
        k_h = k_h.unwrap_fixed("Conv kernel height")
        k_w = k_w.unwrap_fixed("Conv kernel width")
        if k_h % 2 != 1:
            raise ValueError(f"Kernel height must be odd, got {k_h}")
        if k_w % 2 != 1:
            raise ValueError(f"Kernel width must be odd, got {k_w}")
        if in_c != in_c_check:
            raise ValueError("Input channel mismatch")
        if stride_y < 1 or stride_x < 1:
            raise ValueError("Stride must be positive")
        ph, pw = in_h + 2 * padding_y, in_w + 2 * padding_x
        if not (ph >= k_h and pw >= k_w):
            raise ValueError("Kernel must fit inside of padded input")
        out_h = (ph - (k_h - 1) - 1) // stride_y + 1
        out_w = (pw - (k_w - 1) - 1) // stride_x + 1
        out_shape = (batch, Size(out_c), Size(out_h), Size(out_w))
        return self._push(ValueInfo(out_shape, in_dtype, OpKind.CONV, inputs=(input.index, filter.index),
                                    conv=(stride_y, stride_x, padding_y, padding_x)))

    def linear(self, input: Value, weight: Value) -> Value:
        return self.mat_mul(input, self.permute(weight, [1, 0]))

    def mat_mul(self, left: Value, right: Value) -> Value:
        ls, rs = self[left].shape, self[right].shape
        if len(ls) < 2 or len(rs) < 2:
            raise ValueError(f"Matmul operands must have rank >= 2, got shapes {ls} and {rs}")
        l_head, l_tail = ls[:-2], ls[-2:]
        r_head, r_tail = rs[:-2], rs[-2:]
        m, n0 = l_tail
        n1, p = r_tail
        if n0 != n1:
            raise ValueError(f"Inner matmul dimension must match, got shapes {ls} and {rs}")
        head = broadcast_shape_symmetric(l_head, r_head)
        batch = _shape_size(head)
        lb = self.broadcast(left, tuple(head) + tuple(l_tail))
        rb = self.broadcast(right, tuple(head) + tuple(r_tail))
        lf = self.view(lb, (batch,) + tuple(l_tail))
        rf = self.view(rb, (batch,) + tuple(r_tail))
        flat = self.batched_mat_mul(lf, rf)
        return self.view(flat, tuple(head) + (m, p))

    def batched_mat_mul(self, left: Value, right: Value) -> Value:
        ls, ld = self.shape_dtype(left)
        rs, rd = self.shape_dtype(right)
        if ld != rd:
            raise ValueError("Matmul operands must have same dtype")
        if len(ls) != 3 or len(rs) != 3:
            raise ValueError(f"Expected rank 3 shapes, got {ls} and {rs}")
        b0, m, n0 = ls
        b1, n1, p = rs
        if not (b0 == b1 and n0 == n1):
            raise ValueError(f"Batched matmul dimension mismatch, got shapes {ls} and {rs}")
        return self._push(ValueInfo((b0, m, p), ld, OpKind.MATMUL, inputs=(left.index, right.index)))

    # ---------------------------------------------------------------- row ops
    def softmax(self, input: Value, axis: int) -> Value:
        s, d = self.shape_dtype(input)
        if d not in (DType.F32, DType.F16):     # (f16: this repository's storage extension)
            raise ValueError("Softmax input must be f32")
        _assert_axis(s, axis)
        return self._push(ValueInfo(s, d, OpKind.SOFTMAX, inputs=(input.index,), axis=axis))

    def layernorm(self, input: Value, axis: int, eps: float) -> Value:
        s, d = self.shape_dtype(input)
        if d not in (DType.F32, DType.F16):
            raise ValueError("Layernorm input must be f32")
        _assert_axis(s, axis)
        eps = float(np.float32(eps))
        return self._push(ValueInfo(s, d, OpKind.LAYERNORM, inputs=(input.index,), axis=axis, eps=eps))

    def reduce(self, input: Value, axes: Sequence[int], op: ReduceOp) -> Value:
        s, d = self.shape_dtype(input)
        axes = tuple(int(a) for a in axes)
        for a in axes:
            _assert_axis(s, a)
        if len(set(axes)) != len(axes):
            raise ValueError(f"Axes must be unique, got {axes}")
        if op == ReduceOp.MEAN and d != DType.F32:
            raise ValueError("Mean input must be f32")
        if not axes:
            return input
        new_shape = tuple(dim for i, dim in enumerate(s) if i not in axes)
        return self._push(ValueInfo(new_shape, d, OpKind.REDUCE, inputs=(input.index,), axes=axes, reduce_op=op))

    def all_reduce(self, input: Value) -> Value:
        """Extension for tensor-parallel graphs (the reference runs one graph on one device): the element-wise
        sum of `input` over the ranks of the communicator attached to the executor; the value itself when
        there is none.  f32 or f16."""
        s, d = self.shape_dtype(input)
        if d not in (DType.F32, DType.F16):
            raise ValueError(f"all_reduce takes f32 or f16, got {d}")
        return self._push(ValueInfo(s, d, OpKind.ALL_REDUCE, inputs=(input.index,)))

    # ---------------------------------------------------------------- elementwise
    def sigmoid(self, input: Value) -> Value:
        return self.unary(UnaryOp.SIGMOID, input)

    def relu(self, input: Value) -> Value:
        zero, _, _, mx = self[input].dtype.specials()
        return self.clamp(input, zero, mx)

    def clamp(self, input: Value, min, max) -> Value:
        dtype = self[input].dtype
        t = dtype.np.type
        min, max = t(min), t(max)
        _, _, smin, smax = dtype.specials()
        curr = input
        if max != smax:
            curr = self.binary(BinaryOp.MIN, curr, self.scalar(max, dtype))
        if min != smin:
            curr = self.binary(BinaryOp.MAX, curr, self.scalar(min, dtype))
        return curr

    def add(self, l: Value, r: Value) -> Value:
        return self.binary(BinaryOp.ADD, l, r)

    def sub(self, l: Value, r: Value) -> Value:
        return self.binary(BinaryOp.SUB, l, r)

    def mul(self, l: Value, r: Value) -> Value:
        return self.binary(BinaryOp.MUL, l, r)

    def div(self, l: Value, r: Value) -> Value:
        return self.binary(BinaryOp.DIV, l, r)

    def pow(self, l: Value, r: Value) -> Value:
        return self.binary(BinaryOp.POW, l, r)

    def value_cast(self, input: Value, to: DType) -> Value:
        return self.unary(UnaryOp.VALUE_CAST, input, to)

    def bit_cast(self, input: Value, to: DType) -> Value:
        return self.unary(UnaryOp.BIT_CAST, input, to)

    def unary(self, op: UnaryOp, input: Value, cast_to: Optional[DType] = None) -> Value:
        s, in_dtype = self.shape_dtype(input)
        out_dtype = unary_output_dtype(op, in_dtype, cast_to)
        if out_dtype is None:
            raise ValueError(f"Operation {op!r} not supported on dtype {in_dtype!r}")
        if op in (UnaryOp.VALUE_CAST, UnaryOp.BIT_CAST) and out_dtype == in_dtype:
            return input
        if op == UnaryOp.BIT_CAST:
            while self[input].kind == OpKind.UNARY and self[input].unary_op == UnaryOp.BIT_CAST:
                input = self._v(self[input].inputs[0])
        return self._push(ValueInfo(s, out_dtype, OpKind.UNARY, inputs=(input.index,), unary_op=op,
                                    cast_to=cast_to if op in (UnaryOp.VALUE_CAST, UnaryOp.BIT_CAST) else None))

    def binary(self, op: BinaryOp, left: Value, right: Value) -> Value:
        ls, ld = self.shape_dtype(left)
        rs, rd = self.shape_dtype(right)
        result_shape = broadcast_shape_symmetric(ls, rs)
        if ld != rd:
            raise ValueError(f"Binary operation {op!r} requires matching dtypes, got {ld!r} and {rd!r}")
        zero, one, smin, smax = ld.specials()
        if op in (BinaryOp.SUB, BinaryOp.ADD):
            skip = self.is_const_zero(right)
        elif op in (BinaryOp.MUL, BinaryOp.DIV, BinaryOp.POW):
            skip = self.is_const_one(right)
        elif op == BinaryOp.MIN:
            skip = self.is_const_filled_with(right, smax)
        else:
            skip = self.is_const_filled_with(right, smin)
        if skip:
            return left
        l = self.broadcast(left, result_shape)
        r = self.broadcast(right, result_shape)
        return self._push(ValueInfo(result_shape, ld, OpKind.BINARY, inputs=(l.index, r.index), binary_op=op))

    # ---------------------------------------------------------------- composition / outputs
    def call(self, graph: "Graph", inputs: Sequence[Value]) -> List[Value]:
        if len(inputs) != len(graph.inputs):
            raise ValueError("Wrong number of inputs")
        for mine, theirs in zip(inputs, graph.inputs):
            if self[mine].shape != graph[theirs].shape:
                raise ValueError("Wrong input shape")
        mapping = {}
        for i, info in enumerate(graph.values):
            if info.kind == OpKind.INPUT:
                mapping[i] = inputs[info.input_index]
            else:
                copy = ValueInfo(**{**info.__dict__, "inputs": tuple(mapping[j].index for j in info.inputs),
                                    "non_output_uses": 0, "debug_id": ""})
                mapping[i] = self._push(copy)
        return [mapping[v.index] for v in graph.outputs]

    def output(self, v: Value):
        self._check_contains(v)
        self.outputs.append(v)

    def output_all(self, values: Iterable[Value]):
        for v in values:
            self.output(v)

    # ---------------------------------------------------------------- wire format
    def to_bytes(self) -> bytes:
        """Serialise to the C-ABI blob.  Layout (little endian):

        header: magic 'KNG1', u32 value_count, u32 input_count, u32 output_count,
                u32 input value ids..., u32 output value ids...
        value : u8 op, u8 dtype, u16 rank, rank x (u64 factor, u32 batch_exp), then per op:
          INPUT      u32 index
          CONSTANT   u64 byte_count, raw data
          VIEW/BROADCAST/ALL_REDUCE  u32 input
          PERMUTE    u32 input, rank x u32
          SLICE      u32 input, u32 axis, u64 start, u64 end, u64 step
          FLIP       u32 input, u32 axis
          GATHER     u32 input, u32 axis, u32 indices
          CONCAT     u32 count, count x u32, u32 axis
          CONV       u32 input, u32 filter, u32 stride_y, stride_x, padding_y, padding_x
          MATMUL     u32 left, u32 right
          UNARY      u32 input, u8 op, u8 cast dtype (0xff if none)
          BINARY     u32 left, u32 right, u8 op
          SOFTMAX    u32 input, u32 axis
          LAYERNORM  u32 input, u32 axis, f32 eps
          REDUCE     u32 input, u8 op, u32 count, count x u32 axes
        """
        parts = []          # large constants are appended as they are (one copy, in the final join)
        out = bytearray()
        out += b"KNG1"
        out += struct.pack("<III", len(self.values), len(self.inputs), len(self.outputs))
        for v in self.inputs:
            out += struct.pack("<I", v.index)
        for v in self.outputs:
            out += struct.pack("<I", v.index)
        for info in self.values:
            out += struct.pack("<BBH", int(info.kind), int(info.dtype), len(info.shape))
            for d in info.shape:
                out += struct.pack("<QI", d.factor, d.exp)
            k = info.kind
            if k == OpKind.INPUT:
                out += struct.pack("<I", info.input_index)
            elif k == OpKind.CONSTANT:
                raw = np.ascontiguousarray(info.tensor)
                out += struct.pack("<Q", raw.nbytes)
                if raw.nbytes >= 1 << 16:
                    parts.append(bytes(out))
                    parts.append(raw.reshape(-1).view(np.uint8).data)
                    out = bytearray()
                else:
                    out += raw.tobytes()
            elif k in (OpKind.VIEW, OpKind.BROADCAST, OpKind.ALL_REDUCE):
                out += struct.pack("<I", info.inputs[0])
            elif k == OpKind.PERMUTE:
                out += struct.pack("<I", info.inputs[0])
                for p in info.permutation:
                    out += struct.pack("<I", p)
            elif k == OpKind.SLICE:
                out += struct.pack("<IIQQQ", info.inputs[0], info.axis, info.range.start, info.range.end,
                                   info.range.step)
            elif k == OpKind.FLIP:
                out += struct.pack("<II", info.inputs[0], info.axis)
            elif k == OpKind.GATHER:
                out += struct.pack("<III", info.inputs[0], info.axis, info.inputs[1])
            elif k == OpKind.CONCAT:
                out += struct.pack("<I", len(info.inputs))
                for i in info.inputs:
                    out += struct.pack("<I", i)
                out += struct.pack("<I", info.axis)
            elif k == OpKind.CONV:
                out += struct.pack("<IIIIII", info.inputs[0], info.inputs[1], *info.conv)
            elif k == OpKind.MATMUL:
                out += struct.pack("<II", info.inputs[0], info.inputs[1])
            elif k == OpKind.UNARY:
                cast = 0xFF if info.cast_to is None else int(info.cast_to)
                out += struct.pack("<IBB", info.inputs[0], int(info.unary_op), cast)
            elif k == OpKind.BINARY:
                out += struct.pack("<IIB", info.inputs[0], info.inputs[1], int(info.binary_op))
            elif k == OpKind.SOFTMAX:
                out += struct.pack("<II", info.inputs[0], info.axis)
            elif k == OpKind.LAYERNORM:
                out += struct.pack("<IIf", info.inputs[0], info.axis, info.eps)
            elif k == OpKind.REDUCE:
                out += struct.pack("<IBI", info.inputs[0], int(info.reduce_op), len(info.axes))
                for a in info.axes:
                    out += struct.pack("<I", a)
            else:
                raise AssertionError(k)
        parts.append(bytes(out))
        return b"".join(parts)

    def __repr__(self):
        return f"Graph(inputs={self.input_shapes()}, outputs={self.output_shapes()}, values={len(self.values)})"

    def dump(self) -> str:
        lines = ["Graph {"]
        for i, info in enumerate(self.values):
            lines.append(f"  Value({i}) = {info.kind.name} {info.dtype.name} {list(info.shape)} in={list(info.inputs)}"
                         f" uses={info.non_output_uses}")
        lines.append(f"  inputs={self.inputs} outputs={self.outputs}")
        lines.append("}")
        return "\n".join(lines)


def unary_output_dtype(op: UnaryOp, x: DType, cast_to: Optional[DType]) -> Optional[DType]:
    """graph.rs:1613-1647"""
    if op in (UnaryOp.ABS, UnaryOp.NEG):
        return x if x.is_signed else None
    if op in UNARY_FLOAT_OPS:
        return x if x.is_float else None
    if op == UnaryOp.VALUE_CAST:
        return cast_to
    if op == UnaryOp.BIT_CAST:
        if cast_to is None or x.is_bool or cast_to.is_bool:
            return None
        return cast_to if x.size_bytes == cast_to.size_bytes else None
    raise AssertionError(op)


# --------------------------------------------------------------------------------------
# scalar constant folding used only by `as_single_const` (graph.rs:517-520)
# --------------------------------------------------------------------------------------
def _erf_poly(x: float) -> float:
    a = [1.0, 0.0705230784, 0.0422820123, 0.0092705272, 0.0001520143, 0.0002765672, 0.0000430638]
    xa = abs(x)
    d = sum(c * xa ** i for i, c in enumerate(a))
    y = 1.0 - 1.0 / d ** 16
    return math.copysign(y, x) if x != 0 else (x * 0.0 if math.isnan(x) else 0.0 * x)


def _scalar_unary(op: UnaryOp, cast_to: Optional[DType], x):
    t = type(x)
    with np.errstate(all="ignore"):
        if op == UnaryOp.ABS:
            return t(np.abs(x))
        if op == UnaryOp.NEG:
            return t(-x) if t is not np.bool_ else x
        if op == UnaryOp.VALUE_CAST:
            return _value_cast_scalar(x, cast_to)
        if op == UnaryOp.BIT_CAST:
            return np.asarray(x).reshape(1).view(cast_to.np)[0]
        f = {
            UnaryOp.SIN: np.sin, UnaryOp.COS: np.cos, UnaryOp.EXP: np.exp, UnaryOp.LOG: np.log,
            UnaryOp.SQRT: np.sqrt, UnaryOp.TANH: np.tanh,
            UnaryOp.SIGMOID: lambda v: t(1) / (t(1) + np.exp(-v)),
            UnaryOp.ERF: lambda v: t(_erf_poly(float(v))),
            UnaryOp.MISH: lambda v: v * np.tanh(np.log1p(np.exp(v))),
            UnaryOp.SOFTPLUS: lambda v: np.log1p(np.exp(-np.abs(v))) + np.maximum(v, t(0)),
        }[op]
        return t(f(x))


def _value_cast_scalar(x, to: DType):
    """dtype.rs:323-355: widen to (f64, i128), then narrow with wrapping integer casts."""
    src = np.dtype(type(x))
    if src.kind == "f":
        yf = float(x)
        if math.isnan(yf):
            yi = 0
        elif math.isinf(yf):
            yi = (1 << 127) - 1 if yf > 0 else -(1 << 127)
        else:
            yi = max(min(int(yf), (1 << 127) - 1), -(1 << 127))
    else:
        yi = int(x)
        yf = float(yi)
    if to.is_float:
        with np.errstate(all="ignore"):
            return to.np.type(np.float64(yf))
    if to.is_bool:
        return np.bool_(yf != 0.0 or yi != 0)
    bits = to.size_bytes * 8
    yi &= (1 << bits) - 1
    if to.is_signed and yi >= 1 << (bits - 1):
        yi -= 1 << bits
    return to.np.type(yi)


def _scalar_binary(op: BinaryOp, l, r):
    t = type(l)
    with np.errstate(all="ignore"):
        if t is np.bool_:
            return {
                BinaryOp.ADD: np.bool_(l or r), BinaryOp.MUL: np.bool_(l and r),
                BinaryOp.SUB: np.bool_(l and not r), BinaryOp.DIV: np.bool_(l and not r),
                BinaryOp.MIN: np.bool_(l and r), BinaryOp.MAX: np.bool_(l or r),
            }[op]
        if op == BinaryOp.ADD:
            return t(l + r)
        if op == BinaryOp.SUB:
            return t(l - r)
        if op == BinaryOp.MUL:
            return t(l * r)
        if op == BinaryOp.DIV:
            if np.dtype(t).kind == "f":
                return t(l / r)
            q = abs(int(l)) // abs(int(r))
            return t(q if (int(l) < 0) == (int(r) < 0) else -q)
        if op == BinaryOp.MIN:
            return t(np.fmin(l, r))
        if op == BinaryOp.MAX:
            return t(np.fmax(l, r))
        if op == BinaryOp.POW:
            return np.float32(np.power(np.float32(l), np.float32(r)))
    raise AssertionError(op)
