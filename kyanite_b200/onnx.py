"""ONNX model loader: `.onnx` bytes -> `Graph`.

Mirrors the behaviour of the reference loader (kn-graph/src/onnx/load.rs:43-125 for the driver,
:126-1199 for the per-operator lowering, typed_value.rs for shape-valued tensors):

* the axis named `batch_size` becomes `Size.BATCH` (onnx/mod.rs:27-31); other named axes must be given
  through `named_axes`, or whole input shapes through `input_shapes`;
* a value in the ONNX graph is either a graph `Value` or, when it holds sizes that involve the batch size
  (the result of `Shape` and arithmetic on it), a small tensor of `SignedSize` that is evaluated while
  loading and never reaches the graph;
* every attribute and input of a node must be consumed by its lowering, otherwise loading fails
  (load.rs:95-104), so unsupported variants are rejected instead of being silently mis-lowered.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from .graph import (BATCH, BinaryOp, DType, Graph, ONE, ReduceOp, Shape, Size, SliceRange, UnaryOp, Value,
                    _shape_size, broadcast_shape_symmetric, shape)
from .onnx_proto import (ModelProto, OnnxError, OnnxValue, SignedSize, TensorProto, _abs_axis, _as_shape,
                         _as_signed_shape, _as_size, _is_size, _new_size, _NodeArgs, _resolve_dtype, _shape_of,
                         _size_array, parse_model)

__all__ = ["OnnxError", "load_graph_from_onnx_bytes", "load_graph_from_onnx_path", "SUPPORTED_OPS"]

I32_MAX = (1 << 31) - 1
I64_MIN = -(1 << 63)

_UNARY = {"Abs": UnaryOp.ABS, "Neg": UnaryOp.NEG, "Sin": UnaryOp.SIN, "Cos": UnaryOp.COS, "Exp": UnaryOp.EXP,
          "Log": UnaryOp.LOG, "Sqrt": UnaryOp.SQRT, "Sigmoid": UnaryOp.SIGMOID, "Tanh": UnaryOp.TANH,
          "Erf": UnaryOp.ERF, "Mish": UnaryOp.MISH, "Softplus": UnaryOp.SOFTPLUS}
_BINARY = {"Add": BinaryOp.ADD, "Sub": BinaryOp.SUB, "Mul": BinaryOp.MUL, "Div": BinaryOp.DIV,
           "Min": BinaryOp.MIN, "Max": BinaryOp.MAX, "Pow": BinaryOp.POW}
_REDUCE = {"ReduceSum": ReduceOp.SUM, "ReduceMean": ReduceOp.MEAN, "ReduceProd": ReduceOp.PROD,
           "ReduceMin": ReduceOp.MIN, "ReduceMax": ReduceOp.MAX}


def _fixed_dims(s: Shape, what: str) -> List[int]:
    return [d.unwrap_fixed(what) for d in s]


def _replace_dims(s: Shape, axis: int, repl: Sequence[Size]) -> Shape:
    return tuple(s[:axis]) + tuple(repl) + tuple(s[axis + 1:])


def _broadcast_sizes(left: np.ndarray, right: np.ndarray):
    try:
        return np.broadcast_arrays(left, right)
    except ValueError as e:
        raise OnnxError(f"cannot broadcast shape tensors {left.shape} and {right.shape}") from e


# --------------------------------------------------------------------------------------
# per-operator lowering; each handler takes (graph, args) and returns one value or a list
# --------------------------------------------------------------------------------------
def _conv(g: Graph, a: _NodeArgs):
    """load.rs:134-228: 1-D and 2-D convolution, symmetric padding, no dilation, one group; the bias is
    added as a `[1, C, 1, 1]` view so that it fuses into the convolution step."""
    x = a.value(0)
    w = a.value(1)
    bias_raw = a.optional_value(2)
    groups = a.maybe_int("group")
    groups = 1 if groups is None else groups
    kernel_shape = a.take_ints("kernel_shape")
    rank = len(kernel_shape)
    strides = a.maybe_ints("strides") or [1] * rank
    dilations = a.maybe_ints("dilations") or [1] * rank
    auto_pad = a.maybe_string("auto_pad")
    if auto_pad in (None, "NOTSET"):
        pads = list(a.take_ints("pads"))
    elif auto_pad in ("SAME_UPPER", "SAME_LOWER"):
        in_spatial = _fixed_dims(g[x].shape[2:], "conv input spatial dims")
        f_spatial = _fixed_dims(g[w].shape[2:], "conv filter spatial dims")
        lows, highs = [], []
        for i in range(rank):
            total = (in_spatial[i] - 1) * strides[i] + 1 + dilations[i] * (f_spatial[i] - 1) - in_spatial[i]
            small = int(total / 2) if total >= 0 else -((-total) // 2)
            large = total - small
            lo, hi = (small, large) if auto_pad == "SAME_UPPER" else (large, small)
            lows.append(lo)
            highs.append(hi)
        pads = lows + highs
    elif auto_pad == "VALID":
        pads = [0] * (2 * rank)
    else:
        raise a.fail(f"invalid auto_pad value {auto_pad!r}")
    filter_dims = _fixed_dims(g[w].shape, "convolution kernel shape")
    bias = None
    if bias_raw is not None:
        (bias_len,) = g[bias_raw].shape
        bias = g.view(bias_raw, shape(1, bias_len, 1, 1))
    if groups != 1:
        raise a.fail("grouped convolution is not supported")
    if rank == 1:
        if len(pads) != 2 or pads[0] != pads[1] or dilations != [1] or list(strides) != [1]:
            raise a.fail("1-D convolution needs symmetric padding, stride 1, dilation 1")
        if len(filter_dims) != 3 or filter_dims[2] != kernel_shape[0]:
            raise a.fail("kernel_shape does not match the filter")
        x4 = g.view(x, tuple(g[x].shape) + (ONE,))
        w4 = g.view(w, tuple(g[w].shape) + (ONE,))
        y = g.conv(x4, w4, 1, 1, pads[0], 0)
        if bias is not None:
            y = g.add(y, bias)
        return g.view(y, g[y].shape[:3])
    if rank == 2:
        if len(pads) != 4 or pads[0] != pads[2] or pads[1] != pads[3]:
            raise a.fail("asymmetric padding is not supported")
        if list(dilations) != [1, 1]:
            raise a.fail("dilated convolution is not supported")
        if len(filter_dims) != 4 or filter_dims[2:] != list(kernel_shape):
            raise a.fail("kernel_shape does not match the filter")
        y = g.conv(x, w, strides[0], strides[1], pads[0], pads[1])
        return y if bias is None else g.add(y, bias)
    raise a.fail(f"{rank}-D convolution is not supported")


def _clip(g: Graph, a: _NodeArgs):
    """load.rs:229-258: bounds as attributes (old opsets) or as scalar inputs."""
    x = a.value(0)
    lo, hi = a.optional(1), a.optional(2)
    if lo is None and hi is None:
        return g.clamp(x, a.take_float("min"), a.take_float("max"))
    if lo is None or hi is None:
        raise a.fail("Clip must have either 1 or 3 inputs, got 2")
    lo, hi = a_value(a, lo), a_value(a, hi)
    if g[lo].shape != () or g[hi].shape != ():
        raise a.fail("Clip bounds must be scalars")
    return g.binary(BinaryOp.MAX, g.binary(BinaryOp.MIN, x, hi), lo)


def a_value(a: _NodeArgs, v: OnnxValue) -> Value:
    if _is_size(v):
        raise a.fail("a batch-dependent shape tensor cannot be used as a value here")
    return v


def _unary(g: Graph, a: _NodeArgs):
    x = a.value(0)
    if a.node.op_type == "Relu":
        return g.relu(x)
    return g.unary(_UNARY[a.node.op_type], x)


def _size_binary(op: BinaryOp, l: SignedSize, r: SignedSize) -> Optional[SignedSize]:
    if op == BinaryOp.ADD:
        return l.add(r)
    if op == BinaryOp.SUB:
        return l.sub(r)
    if op == BinaryOp.MUL:
        return l.mul(r)
    if op == BinaryOp.DIV:
        return l.floor_div(r)
    return None


def _binary(g: Graph, a: _NodeArgs):
    """load.rs:280-313: values stay values; if either side is a shape tensor both decay to sizes and the
    arithmetic happens while loading (the batch size may cancel out again)."""
    op = _BINARY[a.node.op_type]
    l, r = a.required(0), a.required(1)
    if not _is_size(l) and not _is_size(r):
        return g.binary(op, l, r)
    ls, rs = _broadcast_sizes(_as_size(l, g, a.what), _as_size(r, g, a.what))
    items = []
    for x, y in zip(ls.reshape(-1), rs.reshape(-1)):
        z = _size_binary(op, x, y)
        if z is None:
            raise a.fail(f"cannot evaluate {op.name} between sizes {x} and {y}")
        items.append(z)
    return _new_size(_size_array(items, ls.shape), g)


def _equal(g: Graph, a: _NodeArgs):
    """load.rs:314-343."""
    l, r = a.required(0), a.required(1)
    if not _is_size(l) and not _is_size(r):
        return g.value_cast(g.sub(l, r), DType.BOOL)
    if _is_size(l) and _is_size(r):
        ls, rs = _broadcast_sizes(l, r)
        eq = np.array([x == y for x, y in zip(ls.reshape(-1), rs.reshape(-1))], dtype=np.bool_).reshape(ls.shape)
        return g.constant_tensor(eq)
    # one side mentions the batch size and the other does not: never equal
    out = broadcast_shape_symmetric(_shape_of(l, g), _shape_of(r, g))
    return g.broadcast(g.scalar(False, DType.BOOL), out)


def _where(g: Graph, a: _NodeArgs):
    """load.rs:344-366: constants of equal shape only."""
    cond, x, y = (g.as_const(a.value(i)) for i in range(3))
    if cond is None or x is None or y is None:
        raise a.fail("Where is only supported on constants")
    if cond.dtype != np.bool_ or cond.shape != x.shape or cond.shape != y.shape or x.dtype != y.dtype:
        raise a.fail("Where needs a bool condition and operands of one shape and type")
    return g.constant_tensor(np.where(cond, x, y))


def _flatten(g: Graph, a: _NodeArgs):
    """load.rs:367-394, including the extra leading 1 axis the ONNX spec asks for when axis == 0."""
    x = a.required(0)
    s = _shape_of(x, g)
    rel = a.maybe_int("axis")
    axis = _abs_axis(1 if rel is None else rel, len(s))
    new_shape = list(s[:axis]) + [_shape_size(s[axis:])]
    if axis == 0:
        new_shape.insert(0, ONE)
    if _is_size(x):
        return _new_size(x.reshape(_fixed_dims(new_shape, "size shape")), g)
    return g.view(x, tuple(new_shape))


def _gemm(g: Graph, a: _NodeArgs):
    """load.rs:395-421: only `x @ w.T + b` (alpha = beta = 1, transB = 1)."""
    x, w = a.value(0), a.value(1)
    bias = a.optional_value(2)
    alpha, beta, trans_b = a.take_float("alpha"), a.take_float("beta"), a.take_int("transB")
    if alpha != 1.0 or beta != 1.0 or trans_b == 0:
        raise a.fail("Gemm is only supported with alpha = beta = 1 and transB = 1")
    y = g.linear(x, w)
    if bias is not None:
        (n,) = g[bias].shape
        y = g.add(y, g.view(bias, shape(1, n)))
    return y


def _matmul(g: Graph, a: _NodeArgs):
    return g.mat_mul(a.value(0), a.value(1))


def _einsum(g: Graph, a: _NodeArgs):
    """load.rs:430-461: the two batched-matmul equations."""
    ins = [a_value(a, v) for v in a.all_variadic()]
    eq = a.take_string("equation").replace(" ", "")
    if eq == "bid,bjd->bij" and len(ins) == 2:
        return g.batched_mat_mul(ins[0], g.permute(ins[1], [0, 2, 1]))
    if eq == "bij,bjd->bid" and len(ins) == 2:
        return g.batched_mat_mul(ins[0], ins[1])
    raise a.fail(f"Einsum equation {eq!r} is not supported")


def _batch_norm(g: Graph, a: _NodeArgs):
    """load.rs:463-512: inference-mode batch norm spelled out as sub / div / mul / add on `[1, C, 1...]`
    views, which the optimiser later folds into the neighbouring convolution."""
    x = a.value(0)
    scale, bias, mean, var = (a.value(i) for i in range(1, 5))
    eps = a.take_float("epsilon")
    a.take_float("momentum")
    spatial = a.maybe_int("spatial")
    if spatial not in (None, 1):
        raise a.fail("non-spatial batch normalisation is not supported")
    s = g[x].shape
    if len(s) < 2:
        raise a.fail("BatchNormalization input must have at least rank 2")
    channels = s[1]
    for p in (scale, bias, mean, var):
        if g[p].shape != (channels,):
            raise a.fail("BatchNormalization parameters must have shape [C]")
    exp = tuple(channels if i == 1 else ONE for i in range(len(s)))
    div = g.unary(UnaryOp.SQRT, g.add(g.view(var, exp), g.scalar(np.float32(eps))))
    y = g.binary(BinaryOp.DIV, g.sub(x, g.view(mean, exp)), div)
    return g.add(g.mul(y, g.view(scale, exp)), g.view(bias, exp))


def _norm(g: Graph, a: _NodeArgs):
    """load.rs:513-568: InstanceNormalization (normalise everything after the channel axis) and
    LayerNormalization (everything from `axis` on) as view + layernorm + view + scale + bias."""
    x, scale, bias = a.value(0), a.value(1), a.value(2)
    s = g[x].shape
    if a.node.op_type == "InstanceNormalization":
        eps = a.take_float("epsilon")
        start = 2
        if len(s) < 2:
            raise a.fail("InstanceNormalization input must have at least rank 2")
        exp = tuple(s[1] if i == 1 else ONE for i in range(len(s)))
        scale_b, bias_b = g.view(scale, exp), g.view(bias, exp)
    else:
        axis = a.maybe_int("axis")
        eps = a.maybe_float("epsilon")
        eps = 1e-5 if eps is None else eps
        scale_b, bias_b = g.broadcast(scale, s), g.broadcast(bias, s)
        start = _abs_axis(-1 if axis is None else axis, len(s))
    if len(s) < start:
        raise a.fail(f"input rank must be at least {start}")
    flat = tuple(s[:start]) + (_shape_size(s[start:]),)
    y = g.view(g.layernorm(g.view(x, flat), start, eps), s)
    return g.add(g.mul(y, scale_b), bias_b)


def _constant(g: Graph, a: _NodeArgs):
    return g.constant_tensor(a.take_tensor("value").array)


def _constant_of_shape(g: Graph, a: _NodeArgs):
    """load.rs:575-598."""
    shape_in = a.optional(0)
    out = () if shape_in is None else _as_shape(shape_in, g, a.what)
    t = a.maybe_tensor("value")
    value = g.scalar(np.float32(0)) if t is None else g.constant_tensor(t.array)
    if _shape_size(g[value].shape) != ONE:
        raise a.fail("value must be a one-element tensor")
    return g.broadcast(g.view(value, ()), out)


def _cast(g: Graph, a: _NodeArgs):
    """load.rs:599-612: a shape tensor only survives the no-op cast to I64."""
    x = a.required(0)
    dtype = _resolve_dtype(a.take_int("to"), a.what)
    if _is_size(x):
        if dtype != DType.I64:
            raise a.fail("a shape tensor can only be cast to int64")
        return x
    return g.value_cast(x, dtype)


def _reshape_output_shape(a: _NodeArgs, old: Shape, new: List[SignedSize], allow_zero: bool) -> Shape:
    """load.rs:1421-1472: 0 copies the input dim (unless allowzero), a single -1 takes what is left."""
    old_size = _shape_size(old)
    out: List[Size] = []
    leftover_index = None
    left = old_size
    for i, s in enumerate(new):
        if s == SignedSize(0):
            if allow_zero:
                size = Size(0)
            else:
                if i >= len(old):
                    raise a.fail(f"cannot copy dim {i}: not present in input shape {old}")
                size = old[i]
        elif s == SignedSize(-1):
            if leftover_index is not None:
                raise a.fail("Reshape shape can only contain a single -1")
            leftover_index = i
            out.append(Size(0))
            continue
        else:
            size = s.to_size()
        if size.factor == 0 or left.exp < size.exp or left.factor % size.factor != 0:
            raise a.fail(f"cannot reshape {old} into {new}")
        left = Size(left.factor // size.factor, left.exp - size.exp)
        out.append(size)
    if leftover_index is not None:
        out[leftover_index] = left
    if _shape_size(tuple(out)) != old_size:
        raise a.fail(f"cannot reshape {old} into {new}: sizes differ")
    return tuple(out)


def _reshape(g: Graph, a: _NodeArgs):
    x = a.required(0)
    new = _as_signed_shape(a.required(1), g, a.what)
    allow_zero = bool(a.maybe_int("allowzero") or 0)
    out = _reshape_output_shape(a, _shape_of(x, g), new, allow_zero)
    if _is_size(x):
        return _new_size(x.reshape(_fixed_dims(out, "reshape shape")), g)
    return g.view(x, out)


def _expand(g: Graph, a: _NodeArgs):
    """load.rs:629-644: symmetric broadcast."""
    x = a.required(0)
    target = _as_shape(a.required(1), g, a.what)
    out = broadcast_shape_symmetric(_shape_of(x, g), target)
    if _is_size(x):
        return _new_size(np.broadcast_to(x, _fixed_dims(out, "expand shape")).copy(), g)
    return g.broadcast(x, out)


def _unsqueeze(g: Graph, a: _NodeArgs):
    """load.rs:645-692: axes as input (opset 13+) or attribute, relative to the OUTPUT rank."""
    x = a.required(0)
    axes_in = a.optional(1)
    if axes_in is not None:
        rel = []
        for s in _as_signed_shape(axes_in, g, a.what):
            if s.fixed is None:
                raise a.fail("Unsqueeze axes must be fixed")
            rel.append(s.fixed)
    else:
        rel = list(a.take_ints("axes"))
    in_shape = _shape_of(x, g)
    out_rank = len(in_shape) + len(rel)
    axes = [_abs_axis(r, out_rank) for r in rel]
    if len(set(axes)) != len(axes) or any(ax >= out_rank for ax in axes):
        raise a.fail(f"invalid axes {rel} for input rank {len(in_shape)}")
    it = iter(in_shape)
    out = tuple(ONE if i in axes else next(it) for i in range(out_rank))
    if _is_size(x):
        return _new_size(x.reshape(_fixed_dims(out, "unsqueeze shape")), g)
    return g.view(x, out)


def _transpose(g: Graph, a: _NodeArgs):
    x = a.required(0)
    perm = [int(p) for p in a.take_ints("perm")]
    if _is_size(x):
        return _new_size(np.transpose(x, perm), g)
    return g.permute(x, perm)


def _gather(g: Graph, a: _NodeArgs):
    """load.rs:707-765: negative constant indices wrap around the axis; gathering from a shape tensor
    happens while loading."""
    x = a.required(0)
    indices_raw = a.required(1)
    rel = a.maybe_int("axis")
    in_shape = _shape_of(x, g)
    axis = _abs_axis(0 if rel is None else rel, len(in_shape))
    axis_size = in_shape[axis]
    if _is_size(indices_raw):
        items = []
        for s in indices_raw.reshape(-1):
            if s.factor < 0:
                s = s.add(SignedSize.from_size(axis_size))
                if s is None:
                    raise a.fail("negative gather index cannot be resolved")
            items.append(s)
        indices = _new_size(_size_array(items, indices_raw.shape), g)
    else:
        const = g.as_const(indices_raw)
        if const is not None:
            dim = axis_size.unwrap_fixed("gather dim size")
            wrapped = np.where(const < 0, const + np.array(dim).astype(const.dtype), const) if const.dtype.kind == "i" else const
            indices = g.constant_tensor(np.ascontiguousarray(wrapped).reshape(const.shape))
        else:
            indices = indices_raw       # dynamic indices are assumed to be non-negative
    if _is_size(indices):
        raise a.fail("gather indices depend on the batch size")
    if not _is_size(x):
        return g.gather(x, axis, indices)
    const = g.as_const(indices)
    if const is None:
        raise a.fail("gather from a shape needs constant indices")
    flat = np.take(x, const.reshape(-1).astype(np.int64), axis=axis)
    out_shape = list(x.shape[:axis]) + list(const.shape) + list(x.shape[axis + 1:])
    return _new_size(flat.reshape(out_shape), g)


def _slice(g: Graph, a: _NodeArgs):
    """load.rs:766-851: starts / ends / axes / steps as constant inputs (opset 10+) or attributes;
    positive steps slice, the step -1 full reversal flips; slicing all of a batch axis is a no-op."""
    def get(index: int, name: str) -> Optional[List[int]]:
        v = a.optional(index)
        if v is None:
            ints = a.maybe_ints(name)
            return None if ints is None else list(ints)
        const = g.as_const(a_value(a, v))
        if const is None or const.ndim != 1 or const.dtype not in (np.int64, np.int32):
            raise a.fail(f"Slice operand {name} must be a 1-D integer constant")
        return [int(i) for i in const]

    x = a.required(0)
    starts, ends = get(1, "starts"), get(2, "ends")
    if starts is None or ends is None:
        raise a.fail("missing starts or ends")
    n = len(starts)
    axes = get(3, "axes")
    axes = list(range(n)) if axes is None else axes
    steps = get(4, "steps")
    steps = [1] * n if steps is None else steps
    if not (len(ends) == n and len(axes) == n and len(steps) == n):
        raise a.fail("inconsistent axes count")
    if len(set(axes)) != n:
        raise a.fail(f"Slice axis cannot be repeated, got {axes}")
    in_shape = _shape_of(x, g)
    cur = x
    for i in range(n):
        axis = _abs_axis(axes[i], len(in_shape))
        size = in_shape[axis]
        step = steps[i]
        if step == 0:
            raise a.fail("step cannot be 0")
        if step > 0:
            if not size.is_fixed and starts[i] == 0 and ends[i] == I32_MAX:
                continue
            dim = size.unwrap_fixed("Slice axis size")
            start, end = _abs_axis(starts[i], dim), _abs_axis(ends[i], dim)
            rng = SliceRange(start, end, step)
            if _is_size(cur):
                index = [slice(None)] * cur.ndim
                index[axis] = slice(rng.start, rng.end, rng.step)
                cur = cur[tuple(index)]
            else:
                cur = g.slice(cur, axis, rng)
        else:
            if not (starts[i] == -1 and ends[i] == I64_MIN and step == -1):
                raise a.fail("only the full reversal (start -1, end INT64_MIN, step -1) is supported")
            cur = np.flip(cur, axis) if _is_size(cur) else g.flip(cur, axis)
    return cur


def _concat(g: Graph, a: _NodeArgs):
    ins = a.all_variadic()
    if not ins:
        raise a.fail("must concatenate at least one value")
    axis = _abs_axis(a.take_int("axis"), len(_shape_of(ins[0], g)))
    if any(_is_size(v) for v in ins):
        arrays = [_as_size(v, g, a.what) for v in ins]
        return _new_size(np.concatenate(arrays, axis=axis), g)
    return g.concat(ins, axis)


def _split(g: Graph, a: _NodeArgs):
    """load.rs:874-913: explicit lengths, or two halves (the first takes the extra element)."""
    x = a.required(0)
    split = a.optional(1)
    s = _shape_of(x, g)
    axis = _abs_axis(a.take_int("axis"), len(s))
    if split is None:
        n = s[axis].unwrap_fixed("Split axis length")
        first = (n + 1) // 2
        ranges = [SliceRange(0, first), SliceRange(first, n)]
    else:
        ranges, start = [], 0
        for length in _fixed_dims(_as_shape(split, g, a.what), "split lengths"):
            ranges.append(SliceRange(start, start + length))
            start += length
    out = []
    for r in ranges:
        if _is_size(x):
            index = [slice(None)] * x.ndim
            index[axis] = slice(r.start, r.end)
            out.append(_new_size(x[tuple(index)], g))
        else:
            out.append(g.slice(x, axis, r))
    return out


def _pad(g: Graph, a: _NodeArgs):
    """load.rs:914-971: constant-mode padding as concatenations with a broadcast scalar."""
    x = a.value(0)
    pads = a.value(1)
    constant_value = a.optional(2)
    axes_in = a.optional(3)
    mode = a.maybe_string("mode") or "constant"
    s = g[x].shape
    value = 0.0
    if constant_value is not None:
        c = g.as_single_const(a_value(a, constant_value))
        if c is None or not isinstance(c, np.float32):
            raise a.fail("pad value must be a constant f32")
        value = float(c)
    if axes_in is not None:
        axes = []
        for i in _as_signed_shape(axes_in, g, a.what):
            if i.fixed is None:
                raise a.fail("pad axes must be fixed")
            axes.append(_abs_axis(i.fixed, len(s)))
    else:
        axes = list(range(len(s)))
    pads_const = g.as_const(pads)
    if pads_const is None or pads_const.dtype != np.int64 or pads_const.shape != (2 * len(axes),):
        raise a.fail("pads must be a constant I64 vector of twice the axes count")
    if mode != "constant":
        raise a.fail("only the 'constant' pad mode is supported")
    fill = g.scalar(np.float32(value))
    out = x
    for axis in axes:
        left, right = int(pads_const[axis]), int(pads_const[len(axes) + axis])
        if left < 0 or right < 0:
            raise a.fail("pad values cannot be negative")
        cur = g[out].shape
        blocks = [g.broadcast(fill, _replace_dims(cur, axis, [Size(left)])), out,
                  g.broadcast(fill, _replace_dims(cur, axis, [Size(right)]))]
        out = g.concat(blocks, axis)
    return out


def _shape_op(g: Graph, a: _NodeArgs):
    dims = [SignedSize.from_size(d) for d in _shape_of(a.required(0), g)]
    return _new_size(_size_array(dims, (len(dims),)), g)


def _identity(g: Graph, a: _NodeArgs):
    return a.required(0)


def _softmax(g: Graph, a: _NodeArgs):
    x = a.value(0)
    axis = a.maybe_int("axis")
    return g.softmax(x, _abs_axis(-1 if axis is None else axis, len(g[x].shape)))


def _reduce(g: Graph, a: _NodeArgs):
    """load.rs:995-1024: axes from the attribute (all axes when absent); keepdims defaults to 1."""
    x = a.value(0)
    s = g[x].shape
    axes_attr = a.maybe_ints("axes")
    axes = list(range(len(s))) if axes_attr is None else [_abs_axis(ax, len(s)) for ax in axes_attr]
    keep = a.maybe_int("keepdims")
    keep = True if keep is None else keep != 0
    out = tuple(d if i not in axes else ONE for i, d in enumerate(s) if keep or i not in axes)
    return g.view(g.reduce(x, axes, _REDUCE[a.node.op_type]), out)


def _pool(g: Graph, a: _NodeArgs):
    """load.rs:1025-1109: non-overlapping pooling (stride == kernel, no padding) as view + reduce; a
    remainder is either padded with the reduction's identity (ceil_mode) or sliced off."""
    op = ReduceOp.MAX if a.node.op_type == "MaxPool" else ReduceOp.MEAN
    x = a.value(0)
    strides = list(a.take_ints("strides"))
    kernel = list(a.take_ints("kernel_shape"))
    pads = list(a.take_ints("pads"))
    ceil_mode = bool(a.maybe_int("ceil_mode") or 0)
    auto_pad = a.maybe_string("auto_pad")
    if strides != kernel:
        raise a.fail("pooling with stride != kernel size is not supported")
    if any(p != 0 for p in pads) or auto_pad not in (None, "NOTSET"):
        raise a.fail("pooling with padding is not supported")
    s = g[x].shape
    kept = len(s) - len(kernel)
    pad_amounts = [(0, 0)] * kept
    new_shape = list(s[:kept])
    pooled_axes = []
    slices: List[Optional[SliceRange]] = [None] * kept
    for i, k in enumerate(kernel):
        size = s[kept + i]
        pad, rng = (0, 0), None
        if size.factor % k == 0:
            left = Size(size.factor // k, size.exp)
        elif size.is_fixed:
            rem = size.factor % k
            if ceil_mode:
                pad = (0, k - rem)
                left = Size((size.factor + k - rem) // k)
            else:
                left = Size((size.factor - rem) // k)
                rng = SliceRange(0, left.factor * k, 1)
        else:
            raise a.fail(f"pooling kernel {kernel} does not divide input shape {s}")
        pad_amounts.append(pad)
        new_shape.append(left)
        pooled_axes.append(len(new_shape))
        new_shape.append(Size(k))
        slices.append(rng)
    dtype = g[x].dtype
    zero, one, lo, hi = dtype.specials()
    identity = lo if op == ReduceOp.MAX else zero
    cur = g.pad(x, pad_amounts, g.scalar(identity, dtype))
    for axis, rng in enumerate(slices):
        if rng is not None:
            cur = g.slice(cur, axis, rng)
    return g.reduce(g.view(cur, tuple(new_shape)), pooled_axes, op)


def _global_pool(g: Graph, a: _NodeArgs):
    op = ReduceOp.MAX if a.node.op_type == "GlobalMaxPool" else ReduceOp.MEAN
    x = a.value(0)
    rank = len(g[x].shape)
    if rank < 2:
        raise a.fail(f"unsupported shape {g[x].shape}")
    return g.reduce(x, list(range(2, rank)), op)


def _resize(g: Graph, a: _NodeArgs):
    """load.rs:1130-1192: nearest / floor with constant integer scales = repeat_interleave per axis."""
    x = a.required(0)
    roi = a.optional(1)
    scales = a.optional(2)
    sizes = a.optional(3)
    a.maybe_int("antialias")
    axes = a.maybe_ints("axes")
    a.maybe_string("coordinate_transformation_mode")
    a.take_float("cubic_coeff_a")
    a.maybe_int("exclude_outside")
    a.maybe_float("extrapolation_value")
    policy = a.maybe_string("keep_aspect_ratio_policy") or "stretch"
    mode = a.maybe_string("mode") or "nearest"
    nearest_mode = a.maybe_string("nearest_mode") or "round_prefer_floor"
    if not (mode == "nearest" and nearest_mode == "floor" and roi is None and sizes is None and axes is None
            and policy == "stretch"):
        raise a.fail("the given resize operation is not supported")
    if scales is None:
        raise a.fail("Resize requires scales")
    const = g.as_const(a_value(a, scales))
    x = a_value(a, x)
    rank = len(g[x].shape)
    if const is None or const.dtype != np.float32 or const.shape != (rank,):
        raise a.fail("Resize scales must be a constant f32 vector with one entry per axis")
    out = x
    for axis, scale in enumerate(const):
        if float(int(scale)) != float(scale):
            raise a.fail(f"only integer scales are supported, got {list(const)}")
        out = g.repeat_interleave(out, axis, Size(int(scale)))
    return out


_HANDLERS: Dict[str, Callable[[Graph, _NodeArgs], object]] = {
    "Conv": _conv, "Clip": _clip, "Relu": _unary, "Equal": _equal, "Where": _where, "Flatten": _flatten,
    "Gemm": _gemm, "MatMul": _matmul, "Einsum": _einsum, "BatchNormalization": _batch_norm,
    "InstanceNormalization": _norm, "LayerNormalization": _norm, "Constant": _constant,
    "ConstantOfShape": _constant_of_shape, "Cast": _cast, "Reshape": _reshape, "Expand": _expand,
    "Unsqueeze": _unsqueeze, "Transpose": _transpose, "Gather": _gather, "Slice": _slice, "Concat": _concat,
    "Split": _split, "Pad": _pad, "Shape": _shape_op, "Identity": _identity, "Softmax": _softmax,
    "MaxPool": _pool, "AveragePool": _pool, "GlobalMaxPool": _global_pool, "GlobalAveragePool": _global_pool,
    "Resize": _resize,
}
_HANDLERS.update({name: _unary for name in _UNARY})
_HANDLERS.update({name: _binary for name in _BINARY})
_HANDLERS.update({name: _reduce for name in _REDUCE})
SUPPORTED_OPS = sorted(_HANDLERS)


# --------------------------------------------------------------------------------------
# driver (load.rs:43-125)
# --------------------------------------------------------------------------------------
def _graph_from_model(model: ModelProto, named_axes: Dict[str, Size],
                      input_shapes: Optional[Sequence[Optional[Shape]]]) -> Graph:
    g = Graph()
    store: Dict[str, OnnxValue] = {}

    def define(name: str, value: OnnxValue):
        if name in store:
            raise OnnxError(f"value {name!r} is defined twice")
        store[name] = value

    for t in model.initializers:
        define(t.name, g.constant_tensor(t.array))
    real_index = 0
    for vi in model.inputs:
        if vi.name in store:        # initialisers may be listed among the inputs again
            continue
        dtype = _resolve_dtype(vi.elem_type, f"input {vi.name!r}")
        s = None
        if input_shapes is not None:
            if real_index >= len(input_shapes):
                raise OnnxError(f"no shape given for input {real_index} {vi.name!r}")
            s = input_shapes[real_index]
        if s is None:
            dims = []
            for d in vi.dims:
                if isinstance(d, str):
                    if d not in named_axes:
                        raise OnnxError(f"failed to shape input {real_index} {vi.name!r}: unknown axis {d!r} in {vi.dims}")
                    dims.append(named_axes[d])
                else:
                    dims.append(Size(int(d)))
            s = tuple(dims)
        define(vi.name, g.input(shape(*s), dtype))
        real_index += 1

    for node in model.nodes:
        handler = _HANDLERS.get(node.op_type)
        if handler is None:
            raise OnnxError(f"node {node.name!r}: unsupported operation {node.op_type!r}")
        args = _NodeArgs(node, store)
        first_new = len(g.values)
        try:
            result = handler(g, args)
        except OnnxError:
            raise
        except (ValueError, AssertionError) as e:     # shape / dtype errors from the graph builder
            raise OnnxError(f"{args.what}: {e}") from e
        for index in range(first_new, len(g.values)):
            if not g.values[index].debug_id:
                g.values[index].debug_id = node.name
        results = result if isinstance(result, list) else [result]
        for r in results:
            if _is_size(r) and not any(x.exp != 0 for x in r.reshape(-1)):
                raise AssertionError(f"{args.what}: a fixed shape tensor must be stored as a constant")
        args.check_leftovers()
        if len(results) != len(node.outputs):
            raise OnnxError(f"{args.what}: expected outputs {node.outputs}, got {len(results)}")
        for name, r in zip(node.outputs, results):
            define(name, r)

    for out in model.outputs:
        if out.name not in store:
            raise OnnxError(f"output {out.name!r} does not exist")
        v = store[out.name]
        if _is_size(v):
            raise OnnxError(f"output {out.name!r} is a batch-dependent shape, expected a value")
        g.output(v)
    return g


def load_graph_from_onnx_bytes(buffer: bytes, named_axes: Optional[Dict[str, Size]] = None,
                               input_shapes: Optional[Sequence[Optional[Shape]]] = None,
                               external: Optional[Callable[[str, int, int], bytes]] = None) -> Graph:
    """Load an ONNX model from memory (onnx/mod.rs:39-43).  `batch_size` always names the batch axis;
    `named_axes` adds more names, `input_shapes[i]` (when not None) replaces the declared shape of the i-th
    real input.  Without `external`, a model that refers to external data files is rejected."""
    axes = {"batch_size": BATCH}
    axes.update(named_axes or {})
    return _graph_from_model(parse_model(bytes(buffer), external), axes, input_shapes)


def load_graph_from_onnx_path(path: str, allow_external: bool = False, **kwargs) -> Graph:
    """Load an ONNX file (onnx/mod.rs:27-31).  With `allow_external`, tensor data may live in files next
    to the model (relative locations only, no `..`)."""
    import os
    external = None
    if allow_external:
        base = os.path.dirname(os.path.abspath(path))

        def external(location: str, offset: int, length: int) -> bytes:
            if os.path.isabs(location) or ".." in location.replace("\\", "/").split("/"):
                raise OnnxError(f"external data location {location!r} must be a relative path below the model")
            with open(os.path.join(base, location), "rb") as f:
                f.seek(offset)
                data = f.read(length)
            if len(data) != length:
                raise OnnxError(f"external data file {location!r} is too short")
            return data

    with open(path, "rb") as f:
        return load_graph_from_onnx_bytes(f.read(), external=external, **kwargs)
