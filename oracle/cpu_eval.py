"""CPU oracle: a numpy restatement of the reference's `cpu_eval_graph`.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is the checker
used by `tests/`, by `__graft_entry__.smoke()` and by the `cpu_baseline` / `--impl reference`
legs of `bench.py`.

It follows kn-graph/src/cpu.rs:20-277 operation by operation and takes the same input the
executor takes: the serialised graph blob (see `Graph.to_bytes`), parsed here by an independent
reader.  Element semantics follow kn-graph/src/graph.rs:1649-1815 (`UnaryOp::map`,
`BinaryOp::map`, `ReduceOp::reduce_t`, the 7-term `erf`) and kn-graph/src/dtype.rs:323-392,
726-757 (value/bit casts, Bool arithmetic).

The GEMM inside conv and matmul is `ndarray::dot` in the reference, which dispatches to the
un-vendored `matrixmultiply` crate (version unpinned: the reference ships no Cargo.lock), so its
summation order is not reproducible; numpy's `matmul` stands in for it and results are compared
with the reference's own tolerance rule (kn-cuda-eval/src/tester.rs:28-29).

Pinning: every hand-computed expected output that the reference's tests hold for this path is
replayed against this oracle in `tests/test_oracle_pins.py`.

F16 storage is an extension the reference does not have (kn-graph/src/dtype.rs:25-37 has no half type), so
for it there is nothing to restate and nothing to pin against: PARITY UNPINNED.  The semantics chosen here:
every value of dtype f16 is stored rounded to f16 (round to nearest even); each graph operation on f16
values converts its operands to f32, computes as the f32 operation does (matmul: f32 products and sums;
softmax / layernorm: f32 statistics) and rounds its result to f16 once.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

# tags of the wire format
(OP_INPUT, OP_CONSTANT, OP_VIEW, OP_BROADCAST, OP_PERMUTE, OP_SLICE, OP_FLIP, OP_GATHER, OP_CONCAT, OP_CONV,
 OP_MATMUL, OP_UNARY, OP_BINARY, OP_SOFTMAX, OP_LAYERNORM, OP_REDUCE) = range(16)
OP_ALL_REDUCE = 16   # extension of this repository's IR for tensor-parallel graphs (not in the reference)

NP_DTYPES = [np.float32, np.float64, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32,
             np.uint64, np.bool_, np.float16]
DT_BOOL = 10

(U_ABS, U_NEG, U_SIN, U_COS, U_EXP, U_LOG, U_SQRT, U_SIGMOID, U_TANH, U_ERF, U_MISH, U_SOFTPLUS, U_VALUE_CAST,
 U_BIT_CAST) = range(14)
(B_ADD, B_SUB, B_MUL, B_DIV, B_MIN, B_MAX, B_POW) = range(7)
(R_SUM, R_MEAN, R_PROD, R_MAX, R_MIN) = range(5)


@dataclass
class Node:
    op: int
    dtype: int
    shape: List[Tuple[int, int]]  # (factor, batch_exp)
    inputs: List[int] = field(default_factory=list)
    attr: dict = field(default_factory=dict)


@dataclass
class ParsedGraph:
    nodes: List[Node]
    inputs: List[int]
    outputs: List[int]


class _Reader:
    def __init__(self, data: bytes):
        self.data = data
        self.pos = 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        vals = struct.unpack_from(fmt, self.data, self.pos)
        self.pos += size
        return vals

    def raw(self, n: int) -> bytes:
        b = self.data[self.pos:self.pos + n]
        if len(b) != n:
            raise ValueError("truncated graph blob")
        self.pos += n
        return b


def parse_graph(blob: bytes) -> ParsedGraph:
    r = _Reader(blob)
    if r.raw(4) != b"KNG1":
        raise ValueError("bad graph magic")
    n_values, n_in, n_out = r.take("<III")
    inputs = [r.take("<I")[0] for _ in range(n_in)]
    outputs = [r.take("<I")[0] for _ in range(n_out)]
    nodes = []
    for _ in range(n_values):
        op, dtype, rank = r.take("<BBH")
        shape = [r.take("<QI") for _ in range(rank)]
        node = Node(op, dtype, shape)
        if op == OP_INPUT:
            node.attr["index"] = r.take("<I")[0]
        elif op == OP_CONSTANT:
            n = r.take("<Q")[0]
            dims = [f for f, _ in shape]
            node.attr["tensor"] = np.frombuffer(r.raw(n), dtype=NP_DTYPES[dtype]).reshape(dims)
        elif op in (OP_VIEW, OP_BROADCAST, OP_ALL_REDUCE):
            node.inputs = [r.take("<I")[0]]
        elif op == OP_PERMUTE:
            node.inputs = [r.take("<I")[0]]
            node.attr["perm"] = [r.take("<I")[0] for _ in range(rank)]
        elif op == OP_SLICE:
            i, axis, start, end, step = r.take("<IIQQQ")
            node.inputs = [i]
            node.attr.update(axis=axis, start=start, end=end, step=step)
        elif op == OP_FLIP:
            i, axis = r.take("<II")
            node.inputs = [i]
            node.attr["axis"] = axis
        elif op == OP_GATHER:
            i, axis, idx = r.take("<III")
            node.inputs = [i, idx]
            node.attr["axis"] = axis
        elif op == OP_CONCAT:
            n = r.take("<I")[0]
            node.inputs = [r.take("<I")[0] for _ in range(n)]
            node.attr["axis"] = r.take("<I")[0]
        elif op == OP_CONV:
            i, f, sy, sx, py, px = r.take("<IIIIII")
            node.inputs = [i, f]
            node.attr.update(sy=sy, sx=sx, py=py, px=px)
        elif op == OP_MATMUL:
            node.inputs = list(r.take("<II"))
        elif op == OP_UNARY:
            i, uop, cast = r.take("<IBB")
            node.inputs = [i]
            node.attr.update(op=uop, cast=cast)
        elif op == OP_BINARY:
            l, rr, bop = r.take("<IIB")
            node.inputs = [l, rr]
            node.attr["op"] = bop
        elif op == OP_SOFTMAX:
            i, axis = r.take("<II")
            node.inputs = [i]
            node.attr["axis"] = axis
        elif op == OP_LAYERNORM:
            i, axis, eps = r.take("<IIf")
            node.inputs = [i]
            node.attr.update(axis=axis, eps=np.float32(eps))
        elif op == OP_REDUCE:
            i, rop, n = r.take("<IBI")
            node.inputs = [i]
            node.attr.update(op=rop, axes=[r.take("<I")[0] for _ in range(n)])
        else:
            raise ValueError(f"unknown op tag {op}")
        nodes.append(node)
    if r.pos != len(blob):
        raise ValueError("trailing bytes in graph blob")
    return ParsedGraph(nodes, inputs, outputs)


# --------------------------------------------------------------------------------------
# element semantics
# --------------------------------------------------------------------------------------
_ERF_A = [1.0, 0.0705230784, 0.0422820123, 0.0092705272, 0.0001520143, 0.0002765672, 0.0000430638]


def erf_poly(x: np.ndarray) -> np.ndarray:
    """graph.rs:1789-1815: Abramowitz-Stegun, evaluated in f64, max error 3e-7."""
    x64 = x.astype(np.float64)
    xa = np.abs(x64)
    d = np.zeros_like(xa)
    for i, a in enumerate(_ERF_A):
        d = d + a * xa ** i
    with np.errstate(all="ignore"):
        y = 1.0 - 1.0 / d ** 16
    sign = np.where(np.signbit(x64), -1.0, 1.0)
    sign = np.where(np.isnan(x64), np.nan, sign)
    return (sign * y).astype(x.dtype)


def value_cast(x: np.ndarray, to) -> np.ndarray:
    """dtype.rs:323-355: widen to (f64, i128); floats narrow with `as`, ints wrap."""
    to = np.dtype(to)
    src = x.dtype
    with np.errstate(all="ignore"):
        if src.kind == "b":
            return x.astype(to)
        if to.kind == "f":
            return x.astype(np.float64).astype(to)
        if to.kind == "b":
            if src.kind == "f":
                xf = x.astype(np.float64)
                return (xf != 0.0)
            return x != 0
        # integer target
        if src.kind in "iu":
            return x.astype(to)  # C-style wrap == i128 widen then `as`
        xf = x.astype(np.float64)
        small = np.abs(xf) < 2.0 ** 63
        base = np.where(small, np.trunc(xf), 0.0).astype(np.int64)
        out = base.astype(to)
        big = ~small & ~np.isnan(xf)
        if np.any(big):
            flat_out = out.reshape(-1)
            flat_x = xf.reshape(-1)
            bits = to.itemsize * 8
            for i in np.flatnonzero(big.reshape(-1)):
                v = flat_x[i]
                if np.isinf(v) or abs(v) >= 2.0 ** 127:
                    yi = (1 << 127) - 1 if v > 0 else -(1 << 127)
                else:
                    yi = int(v)
                yi &= (1 << bits) - 1
                if to.kind == "i" and yi >= 1 << (bits - 1):
                    yi -= 1 << bits
                flat_out[i] = yi
            out = flat_out.reshape(out.shape)
        return out


def unary(op: int, cast: int, x: np.ndarray) -> np.ndarray:
    if x.dtype == np.float16 and op not in (U_VALUE_CAST, U_BIT_CAST):
        return unary(op, cast, x.astype(np.float32)).astype(np.float16)    # f16 storage: f32 arithmetic, one rounding
    t = x.dtype.type
    with np.errstate(all="ignore"):
        if op == U_ABS:
            return np.abs(x)
        if op == U_NEG:
            return -x
        if op == U_SIN:
            return np.sin(x)
        if op == U_COS:
            return np.cos(x)
        if op == U_EXP:
            return np.exp(x)
        if op == U_LOG:
            return np.log(x)
        if op == U_SQRT:
            return np.sqrt(x)
        if op == U_SIGMOID:
            return (t(1) / (t(1) + np.exp(-x))).astype(x.dtype)
        if op == U_TANH:
            return np.tanh(x)
        if op == U_ERF:
            return erf_poly(x)
        if op == U_MISH:
            return (x * np.tanh(np.log1p(np.exp(x)))).astype(x.dtype)
        if op == U_SOFTPLUS:
            return (np.log1p(np.exp(-np.abs(x))) + np.fmax(x, t(0))).astype(x.dtype)
        if op == U_VALUE_CAST:
            return value_cast(x, NP_DTYPES[cast])
        if op == U_BIT_CAST:
            return np.array(x, order="C", copy=True).view(NP_DTYPES[cast])
    raise ValueError(f"unknown unary op {op}")


def binary(op: int, l: np.ndarray, r: np.ndarray) -> np.ndarray:
    if l.dtype == np.float16:
        with np.errstate(all="ignore"):
            return binary(op, l.astype(np.float32), r.astype(np.float32)).astype(np.float16)
    with np.errstate(all="ignore"):
        if l.dtype == np.bool_:
            # dtype.rs:726-757 and the derived Ord on DBool
            if op in (B_ADD, B_MAX):
                return l | r
            if op in (B_MUL, B_MIN):
                return l & r
            if op in (B_SUB, B_DIV):
                return l & ~r
            raise ValueError("pow on bool")
        if op == B_ADD:
            return l + r
        if op == B_SUB:
            return l - r
        if op == B_MUL:
            return l * r
        if op == B_DIV:
            if l.dtype.kind == "f":
                return l / r
            if np.any(r == 0):
                raise ZeroDivisionError("integer division by zero")
            if l.dtype.kind == "u":
                return l // r
            # Rust `/` truncates toward zero; numpy `//` floors
            q = np.abs(l.astype(np.int64)) // np.abs(r.astype(np.int64))
            q = np.where((l < 0) != (r < 0), -q, q)
            return q.astype(l.dtype)
        if op == B_MIN:
            return np.fmin(l, r) if l.dtype.kind == "f" else np.minimum(l, r)
        if op == B_MAX:
            return np.fmax(l, r) if l.dtype.kind == "f" else np.maximum(l, r)
        if op == B_POW:
            if l.dtype != np.float32:
                raise ValueError("pow is f32 only")
            return np.power(l, r)
    raise ValueError(f"unknown binary op {op}")


def _identity(op: int, dtype: np.dtype):
    t = dtype.type
    if op in (R_SUM, R_MEAN):
        return t(0)
    if op == R_PROD:
        return t(1)
    if dtype.kind == "f":
        return t(np.inf) if op == R_MIN else t(-np.inf)
    if dtype.kind == "b":
        return t(op == R_MIN)
    info = np.iinfo(dtype)
    return t(info.max) if op == R_MIN else t(info.min)


def reduce_axis(op: int, x: np.ndarray, axis: int) -> np.ndarray:
    """One `lanes(axis)` fold (cpu.rs:263-269, graph.rs:1770-1786), keeping the axis as size 1."""
    ident = _identity(op, x.dtype)
    with np.errstate(all="ignore"):
        if op in (R_SUM, R_MEAN):
            if x.dtype == np.bool_:
                res = np.logical_or.reduce(x, axis=axis, keepdims=True)
            else:
                res = np.add.reduce(x, axis=axis, dtype=x.dtype, keepdims=True)
            if op == R_MEAN:
                res = (res / np.float32(x.shape[axis])).astype(np.float32)
            return res
        if op == R_PROD:
            if x.dtype == np.bool_:
                return np.logical_and.reduce(x, axis=axis, keepdims=True)
            return np.multiply.reduce(x, axis=axis, dtype=x.dtype, keepdims=True)
        if x.dtype.kind == "f":
            f = np.fmin if op == R_MIN else np.fmax
        elif x.dtype.kind == "b":
            f = np.logical_and if op == R_MIN else np.logical_or
        else:
            f = np.minimum if op == R_MIN else np.maximum
        return f.reduce(x, axis=axis, keepdims=True, initial=ident)


def softmax(x: np.ndarray, axis: int) -> np.ndarray:
    """cpu.rs:443-458"""
    if x.dtype == np.float16:
        with np.errstate(all="ignore"):
            return softmax(x.astype(np.float32), axis).astype(np.float16)
    with np.errstate(all="ignore"):
        mx = np.fmax.reduce(x, axis=axis, keepdims=True, initial=np.float32(-np.inf))
        r = np.exp(x - mx)
        s = np.add.reduce(r, axis=axis, keepdims=True, dtype=np.float32)
        return (r / s).astype(np.float32)


def layernorm(x: np.ndarray, axis: int, eps) -> np.ndarray:
    """cpu.rs:461-479: biased variance of the centred values, eps inside the sqrt."""
    if x.dtype == np.float16:
        with np.errstate(all="ignore"):
            return layernorm(x.astype(np.float32), axis, eps).astype(np.float16)
    with np.errstate(all="ignore"):
        n = np.float32(x.shape[axis])
        mean = np.add.reduce(x, axis=axis, keepdims=True, dtype=np.float32) / n
        r = x - mean
        var = np.add.reduce(r * r, axis=axis, keepdims=True, dtype=np.float32) / n
        std = np.sqrt(var + np.float32(eps))
        return (r / std).astype(np.float32)


def convolution(x: np.ndarray, w: np.ndarray, sy: int, sx: int, py: int, px: int) -> np.ndarray:
    """cpu.rs:347-419: im2col with zero padding, one GEMM, cross-correlation."""
    n, c, ih, iw = x.shape
    k, c2, kh, kw = w.shape
    assert c == c2 and kh % 2 == 1 and kw % 2 == 1
    oh = (ih + 2 * py - (kh - 1) - 1) // sy + 1
    ow = (iw + 2 * px - (kw - 1) - 1) // sx + 1
    cols = np.zeros((n, oh, ow, c, kh, kw), dtype=x.dtype)

    def valid(o_count, stride, f, pad, i_count):
        # output positions o with 0 <= o*stride + f - pad < i_count form a contiguous range
        lo = max(0, -((f - pad) // stride)) if f - pad < 0 else 0
        hi = min(o_count, (i_count - 1 - (f - pad)) // stride + 1) if i_count - 1 - (f - pad) >= 0 else 0
        return lo, hi

    for fy in range(kh):
        oy0, oy1 = valid(oh, sy, fy, py, ih)
        if oy1 <= oy0:
            continue
        for fx in range(kw):
            ox0, ox1 = valid(ow, sx, fx, px, iw)
            if ox1 <= ox0:
                continue
            iy0 = oy0 * sy + fy - py
            ix0 = ox0 * sx + fx - px
            src = x[:, :, iy0:iy0 + (oy1 - oy0 - 1) * sy + 1:sy, ix0:ix0 + (ox1 - ox0 - 1) * sx + 1:sx]
            cols[:, oy0:oy1, ox0:ox1, :, fy, fx] = src.transpose(0, 2, 3, 1)
    a = cols.reshape(n * oh * ow, c * kh * kw)
    b = np.ascontiguousarray(w.transpose(1, 2, 3, 0)).reshape(c * kh * kw, k)
    with np.errstate(all="ignore"):
        out = a @ b
    return np.ascontiguousarray(out.reshape(n, oh, ow, k).transpose(0, 3, 1, 2))


def batched_mat_mul(l: np.ndarray, r: np.ndarray) -> np.ndarray:
    """cpu.rs:421-439"""
    assert l.ndim == 3 and r.ndim == 3 and l.shape[0] == r.shape[0] and l.shape[2] == r.shape[1]
    with np.errstate(all="ignore"):
        if l.dtype == np.float16:   # f16 storage: f32 products and sums, one rounding
            return np.matmul(l.astype(np.float32), r.astype(np.float32)).astype(np.float16)
        return np.matmul(l, r)


def gather(x: np.ndarray, axis: int, indices: np.ndarray) -> np.ndarray:
    """cpu.rs:304-333: indices must be non-negative and in range."""
    assert indices.ndim == 1
    idx = indices.astype(np.int64) if indices.dtype != np.uint64 else indices
    if indices.dtype.kind == "i" and np.any(indices < 0):
        raise IndexError("negative gather index")
    if np.any(idx >= x.shape[axis]):
        raise IndexError("Index out of bounds")
    return np.take(x, idx.astype(np.int64), axis=axis)


# --------------------------------------------------------------------------------------
# graph evaluation
# --------------------------------------------------------------------------------------
def cpu_eval_graph(blob, batch_size: int, inputs: Sequence[np.ndarray], keep_all: bool = False,
                   overrides: Optional[dict] = None, wanted: Optional[Sequence[int]] = None, all_reduce=None):
    """Evaluate the graph on the CPU (cpu.rs:20-98).  Returns the list of outputs, each a
    C-contiguous array (cpu.rs:526-535); with `keep_all` also returns every intermediate.

    For layer-wise checks of graphs too large to evaluate whole (the reference tests big graphs
    differentially too, kn-cuda-eval/tests/root/runner.rs:29-55): `overrides` maps value indices to arrays
    that stand in for those values (another executor's result for the layer's input, say) and `wanted`
    lists the value indices to return instead of the graph's outputs.  Only values that `wanted` depends
    on, up to the overridden ones, are computed; graph inputs nothing needs may be passed as None.

    `all_reduce(array) -> array` plays the all-reduce values of a tensor-parallel graph (an extension of this
    repository's IR): the sum over the ranks.  Without it the graph is evaluated as a world of one rank."""
    g = blob if isinstance(blob, ParsedGraph) else parse_graph(blob)
    if len(inputs) != len(g.inputs):
        raise ValueError(f"expected {len(g.inputs)} inputs, got {len(inputs)}")
    overrides = overrides or {}
    targets = list(g.outputs) if wanted is None else list(wanted)

    needed = [False] * len(g.nodes)
    stack = list(targets)
    while stack:
        i = stack.pop()
        if needed[i]:
            continue
        needed[i] = True
        if i not in overrides:
            stack.extend(g.nodes[i].inputs)

    last_use = {}
    for i, node in enumerate(g.nodes):
        if needed[i] and i not in overrides:
            for j in node.inputs:
                last_use[j] = i
    keep = set(targets)

    vals: List[Optional[np.ndarray]] = [None] * len(g.nodes)
    for i, node in enumerate(g.nodes):
        if not needed[i]:
            continue
        out_shape = tuple(f * batch_size ** e for f, e in node.shape)
        np_dtype = np.dtype(NP_DTYPES[node.dtype])
        a = [vals[j] for j in node.inputs] if i not in overrides else []
        op = node.op
        if i in overrides:
            res = np.asarray(overrides[i])
        elif op == OP_INPUT:
            x = np.asarray(inputs[node.attr["index"]])
            if x.dtype != np_dtype:
                raise ValueError(f"input {node.attr['index']}: expected dtype {np_dtype}, got {x.dtype}")
            res = x
        elif op == OP_CONSTANT:
            res = node.attr["tensor"]
        elif op == OP_VIEW:
            res = a[0].reshape(out_shape)
        elif op == OP_BROADCAST:
            res = np.broadcast_to(a[0], out_shape)
        elif op == OP_PERMUTE:
            res = a[0].transpose(node.attr["perm"])
        elif op == OP_SLICE:
            axis = node.attr["axis"]
            end = min(node.attr["end"], a[0].shape[axis])  # cpu.rs:286-302
            sl = [slice(None)] * a[0].ndim
            sl[axis] = slice(node.attr["start"], end, node.attr["step"])
            res = a[0][tuple(sl)]
        elif op == OP_FLIP:
            res = np.flip(a[0], axis=node.attr["axis"])
        elif op == OP_GATHER:
            res = gather(a[0], node.attr["axis"], a[1])
        elif op == OP_CONCAT:
            res = np.concatenate(a, axis=node.attr["axis"]) if a else np.zeros(out_shape, dtype=np_dtype)
        elif op == OP_CONV:
            at = node.attr
            res = convolution(a[0], a[1], at["sy"], at["sx"], at["py"], at["px"])
        elif op == OP_MATMUL:
            res = batched_mat_mul(a[0], a[1])
        elif op == OP_UNARY:
            res = unary(node.attr["op"], node.attr["cast"], a[0])
        elif op == OP_BINARY:
            res = binary(node.attr["op"], a[0], a[1])
        elif op == OP_SOFTMAX:
            res = softmax(a[0], node.attr["axis"])
        elif op == OP_LAYERNORM:
            res = layernorm(a[0], node.attr["axis"], node.attr["eps"])
        elif op == OP_ALL_REDUCE:
            res = np.ascontiguousarray(a[0]) if all_reduce is None else np.asarray(all_reduce(np.ascontiguousarray(a[0])))
        elif op == OP_REDUCE:
            cur = a[0]
            for axis in node.attr["axes"]:
                cur = reduce_axis(node.attr["op"], cur, axis)
            res = cur.reshape(out_shape)
        else:
            raise ValueError(f"unknown op {op}")

        if tuple(res.shape) != out_shape:
            raise AssertionError(f"value {i}: wrong output shape {res.shape}, expected {out_shape}")
        if res.dtype != np_dtype:
            raise AssertionError(f"value {i}: wrong dtype {res.dtype}, expected {np_dtype}")
        vals[i] = res

        if not keep_all and i not in overrides:
            for j in set(node.inputs):
                if last_use.get(j) == i and j not in keep:
                    vals[j] = None

    # (np.ascontiguousarray would promote rank 0 to rank 1)
    outs = [np.array(vals[o], order="C", copy=True) for o in targets]
    if keep_all:
        return outs, vals
    return outs


def assert_tensors_match(expected: Sequence[np.ndarray], actual: Sequence[np.ndarray], tol_abs=1e-3,
                         tol_rel=1e-3, abs_scaled=False) -> Tuple[float, float]:
    """The reference's comparison rule (kn-cuda-eval/src/tester.rs:28-29,216-302): floats mismatch
    iff abs_diff >= tol_abs AND rel_diff >= tol_rel, NaN positions must agree, non-floats must be
    exactly equal.  With `abs_scaled` the absolute threshold of each tensor is
    tol_abs * (largest finite |expected| of that tensor), for reduced-precision operands whose rounding
    error is relative to the summed magnitudes rather than to the (possibly cancelled) result.  There is
    no floor at 1: a tensor of small numbers (a softmax over thousands of entries) is held to its own
    scale.  A tensor that is all zeros keeps the plain tol_abs.
    Returns the (max abs, max rel) float error seen."""
    assert len(expected) == len(actual), f"wrong number of tensors: {len(expected)} vs {len(actual)}"
    max_abs = 0.0
    max_rel = 0.0
    for i, (e, a) in enumerate(zip(expected, actual)):
        e = np.asarray(e)
        a = np.asarray(a)
        assert e.shape == a.shape, f"tensor {i}: shape {a.shape}, expected {e.shape}"
        assert e.dtype == a.dtype, f"tensor {i}: dtype {a.dtype}, expected {e.dtype}"
        if e.dtype.kind != "f":
            bad = np.flatnonzero(e.reshape(-1) != a.reshape(-1))
            assert bad.size == 0, f"tensor {i}: {bad.size} exact mismatches, first at {bad[:5]}"
            continue
        e64 = e.astype(np.float64)
        a64 = a.astype(np.float64)
        nan_e, nan_a = np.isnan(e64), np.isnan(a64)
        assert np.array_equal(nan_e, nan_a), f"tensor {i}: NaN positions differ"
        same = (e64 == a64) | nan_e
        with np.errstate(all="ignore"):
            d = np.where(same, 0.0, np.abs(e64 - a64))
            rel = np.where(same, 0.0, d / np.abs(e64))
        rel = np.where(np.isnan(rel), np.inf, rel)
        tensor_abs = tol_abs
        if abs_scaled:
            finite = np.abs(e64[np.isfinite(e64)])
            scale = float(finite.max()) if finite.size else 0.0
            tensor_abs = tol_abs * scale if scale > 0.0 else tol_abs
        bad = (d >= tensor_abs) & (rel >= tol_rel)
        if bad.any():
            idx = np.argwhere(bad)[:5]
            msg = ", ".join(f"{tuple(j)}: expected {e[tuple(j)]}, got {a[tuple(j)]}" for j in idx)
            raise AssertionError(f"tensor {i}: {int(bad.sum())}/{bad.size} mismatches (abs>={tensor_abs:.3g} and "
                                 f"rel>={tol_rel}; worst abs {float(d[bad].max()):.3g}); {msg}")
        fin = np.isfinite(d)
        if fin.any():
            max_abs = max(max_abs, float(d[fin].max()))
        finr = np.isfinite(rel)
        if finr.any():
            max_rel = max(max_rel, float(rel[finr].max()))
    return max_abs, max_rel
