"""Test graphs re-expressed from the reference's executor test-suite.

Every case is `(name, graph, batch_size, inputs, expected)`; `expected` is a list of arrays where
the reference test holds hand-computed numbers (those pin the oracle), else None (the reference
then compares CPU against GPU on the same data, and so do we).  Sources:
kn-cuda-eval/tests/root/graphs.rs, elementwise.rs, opt.rs; kn-cuda-sys/tests/cublas.rs, fused.rs.
Random inputs use numpy PCG64 (the reference's Rust StdRng stream is not reproducible here and the
values do not matter: both sides see the same arrays).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Callable, List, Optional

import numpy as np

from kyanite_b200.graph import (BATCH, BinaryOp, DType, Graph, OpKind, ReduceOp, Size, SliceRange, UnaryOp,
                                BINARY_ALL, REDUCE_ALL, UNARY_ALL, shape)


@dataclass
class Case:
    name: str
    graph: Graph
    batch_size: int
    inputs: List[np.ndarray]
    expected: Optional[List[np.ndarray]] = None


def f32(shape_, data) -> np.ndarray:
    return np.asarray(data, dtype=np.float32).reshape(shape_)


def linspace(*shape_) -> np.ndarray:
    n = int(np.prod(shape_)) if shape_ else 1
    return np.linspace(-1.0, 1.0, n, dtype=np.float64).astype(np.float32).reshape(shape_)


def arange(n) -> np.ndarray:
    return np.arange(n, dtype=np.float32)


def rng_f32(seed, *shape_) -> np.ndarray:
    return np.random.Generator(np.random.PCG64(seed)).random(shape_, dtype=np.float32)


ELEMENTWISE_TEST_VALUES = np.array(
    [0.0, 0.1, 0.5, 0.8, 1.0, 1.1, 1.5, 1.7, 2.0, 5.0, 6.0, 7.0, -1.0, -1.0, 0.5, 20.0, 80.0, 100.0, 1000.0, -20.0,
     -100.0], dtype=np.float32)

CASES: List[Callable[[], Case]] = []


def case(fn):
    CASES.append(fn)
    return fn


# ------------------------------------------------------------------ graphs.rs
@case
def empty():
    return Case("empty", Graph(), 8, [], [])


@case
def copy():
    g = Graph()
    fixed = g.input(shape(10))
    batch = g.input(shape(BATCH))
    g.output_all([fixed, batch])
    a, b = linspace(10), linspace(8)
    return Case("copy", g, 8, [a, b], [a, b])


@case
def slice_():
    g = Graph()
    x = g.input(shape(10, 4))
    indexed = g.index(x, 1, 0)
    g.output_all([indexed, g.slice(x, 0, SliceRange(0, 2, 1)), g.slice(indexed, 0, SliceRange(0, 2, 1))])
    return Case("slice", g, 0, [linspace(10, 4)])


@case
def flip():
    g = Graph()
    x = g.constant(shape(2, 3), [0, 1, 2, 3, 4, 5])
    first_once = g.flip(x, 0)
    first_twice = g.flip(first_once, 0)
    other_once = g.flip(x, 1)
    other_twice = g.flip(other_once, 1)
    combined = g.flip(first_once, 1)
    g.output_all([first_once, first_twice, other_once, other_twice, combined])
    exp = [f32((2, 3), [3, 4, 5, 0, 1, 2]), f32((2, 3), [0, 1, 2, 3, 4, 5]), f32((2, 3), [2, 1, 0, 5, 4, 3]),
           f32((2, 3), [0, 1, 2, 3, 4, 5]), f32((2, 3), [5, 4, 3, 2, 1, 0])]
    return Case("flip", g, 0, [], exp)


@case
def flip_conv():
    g = Graph()
    x = g.input(shape(2, 4, 8, 8))
    flipped = g.flip(x, 3)
    w = g.constant(shape(4, 4, 3, 3), linspace(4 * 4 * 3 * 3))
    g.output(g.conv(flipped, w, 1, 1, 1, 1))
    return Case("flip_conv", g, 0, [linspace(2, 4, 8, 8)])


def _repeat(interleave: bool):
    g = Graph()
    x = g.input(shape(2, 3))
    f = g.repeat_interleave if interleave else g.repeat
    g.output_all([f(x, 0, Size(0)), f(x, 0, Size(2)), f(x, 1, Size(0)), f(x, 1, Size(2))])
    return Case("repeat_interleave" if interleave else "repeat", g, 0, [rng_f32(0, 2, 3)])


@case
def repeat():
    return _repeat(False)


@case
def repeat_interleave():
    return _repeat(True)


@case
def repeat_manual():
    g = Graph()
    x = g.input(shape(3))
    g.output_all([g.repeat(x, 0, Size(2)), g.repeat_interleave(x, 0, Size(2))])
    return Case("repeat_manual", g, 0, [f32((3,), [1, 2, 3])],
                [f32((6,), [1, 2, 3, 1, 2, 3]), f32((6,), [1, 1, 2, 2, 3, 3])])


@case
def gather_simple_axis_0():
    g = Graph()
    x = g.constant(shape(2, 3), [7.0, 7.1, 7.2, 7.3, 7.4, 7.5])
    idx = g.constant(shape(4), [0, 1, 1, 0], DType.U32)
    g.output(g.gather(x, 0, idx))
    return Case("gather_simple_axis_0", g, 0, [],
                [f32((4, 3), [7.0, 7.1, 7.2, 7.3, 7.4, 7.5, 7.3, 7.4, 7.5, 7.0, 7.1, 7.2])])


@case
def gather_simple_axis_1():
    g = Graph()
    x = g.constant(shape(2, 3), [7.0, 7.1, 7.2, 7.3, 7.4, 7.5])
    idx = g.constant(shape(4), [0, 2, 1, 0], DType.U32)
    g.output(g.gather(x, 1, idx))
    return Case("gather_simple_axis_1", g, 0, [], [f32((2, 4), [7.0, 7.2, 7.1, 7.0, 7.3, 7.5, 7.4, 7.3])])


@case
def gather_complex_axis_0():
    g = Graph()
    x = g.input(shape(3, 2))
    idx = g.constant(shape(2, 2), [0, 1, 1, 2], DType.U32)
    g.output(g.gather(x, 0, idx))
    return Case("gather_complex_axis_0", g, 0, [f32((3, 2), [1.0, 1.2, 2.3, 3.4, 4.5, 5.7])],
                [f32((2, 2, 2), [1.0, 1.2, 2.3, 3.4, 2.3, 3.4, 4.5, 5.7])])


@case
def gather_complex_axis_1():
    g = Graph()
    x = g.input(shape(3, 3))
    idx = g.constant(shape(1, 2), [0, 2], DType.U32)
    g.output(g.gather(x, 1, idx))
    return Case("gather_complex_axis_1", g, 0, [f32((3, 3), [1.0, 1.2, 1.9, 2.3, 3.4, 3.9, 4.5, 5.7, 5.9])],
                [f32((3, 1, 2), [1.0, 1.9, 2.3, 3.9, 4.5, 5.9])])


@case
def gather_size_0():
    g = Graph()
    x = g.input(shape(8, 4))
    idx = g.constant(shape(0), [], DType.U32)
    o0 = g.gather(x, 0, idx)
    o1 = g.gather(x, 1, idx)
    g.output_all([o0, o1])
    assert g[o0].shape == shape(0, 4) and g[o1].shape == shape(8, 0)
    return Case("gather_size_0", g, 0, [linspace(8, 4)])


@case
def gather_as_index():
    g = Graph()
    x = g.input(shape(16, 8, 4))
    index = g.scalar(4, DType.U32)
    indices = g.view(index, shape(1))
    indices_repeat = g.broadcast(indices, shape(3))
    g.output_all([g.gather(x, 1, indices), g.gather(x, 1, indices_repeat)])
    assert all(info.kind != OpKind.GATHER for info in g.values), "gather should have become an index"
    return Case("gather_as_index", g, 0, [rng_f32(0, 16, 8, 4)])


@case
def gather_input_indices():
    # not in the reference suite: runtime indices of a signed type over a middle axis
    g = Graph()
    x = g.input(shape(BATCH, 7, 5))
    idx = g.input(shape(6), DType.I64)
    g.output(g.gather(x, 1, idx))
    return Case("gather_input_indices", g, 3, [rng_f32(3, 3, 7, 5), np.array([6, 0, 3, 3, 1, 5], dtype=np.int64)])


@case
def linear():
    g = Graph()
    x = g.input(shape(1, 4))
    w = g.constant(shape(2, 4), arange(8))
    b = g.constant(shape(1, 2), [-10.0, 10.0])
    lin = g.linear(x, w)
    g.output_all([lin, g.add(lin, b)])
    return Case("linear", g, 0, [f32((1, 4), [0, 1, 2, 3])], [f32((1, 2), [14, 38]), f32((1, 2), [4, 48])])


@case
def linear_sliced():
    g = Graph()
    left = g.input(shape(8, 4))
    ls = g.slice(left, 0, SliceRange(0, 8, 2))
    right = g.input(shape(4, 3))
    g.output(g.mat_mul(ls, right))
    return Case("linear_sliced", g, 0, [linspace(8, 4), linspace(4, 3)])


@case
def mat_mul_broadcast():
    shapes = [((4, 2), (2, 3), (4, 3)), ((8, 4, 2), (2, 3), (8, 4, 3)), ((4, 2), (8, 2, 3), (8, 4, 3)),
              ((8, 4, 2), (8, 2, 3), (8, 4, 3)), ((1, 1, 1, 4, 2), (8, 1, 2, 3), (1, 8, 1, 4, 3))]
    g = Graph()
    inputs = []
    for i, (ls, rs, os) in enumerate(shapes):
        inputs += [rng_f32(2 * i, *ls), rng_f32(2 * i + 1, *rs)]
        res = g.mat_mul(g.input(shape(ls)), g.input(shape(rs)))
        assert g[res].shape == shape(os)
        g.output(res)
    return Case("mat_mul_broadcast", g, 0, inputs)


def _mat_mul_transpose(ta: bool, tb: bool):
    g = Graph()
    sa, sb = [4, 5, 6], [4, 6, 3]
    if ta:
        sa[1], sa[2] = sa[2], sa[1]
    if tb:
        sb[1], sb[2] = sb[2], sb[1]
    a = g.constant(shape(sa), linspace(4 * 5 * 6))
    b = g.constant(shape(sb), linspace(4 * 6 * 3))
    if ta:
        a = g.permute(a, [0, 2, 1])
    if tb:
        b = g.permute(b, [0, 2, 1])
    r = g.batched_mat_mul(a, b)
    assert g[r].shape == shape(4, 5, 3)
    g.output(r)
    return Case(f"mat_mul_transpose_{int(ta)}{int(tb)}", g, 0, [])


for _ta, _tb in itertools.product([True, False], repeat=2):
    CASES.append(lambda ta=_ta, tb=_tb: _mat_mul_transpose(ta, tb))


@case
def cublas_simple():
    # kn-cuda-sys/tests/cublas.rs: 3 x ([1x2] . [2x1])
    g = Graph()
    a = g.constant(shape(3, 1, 2), [1, 2, 3, 4, 5, 6])
    b = g.constant(shape(3, 2, 1), [7, 8, 9, 10, 11, 12])
    g.output(g.batched_mat_mul(a, b))
    return Case("cublas_simple", g, 0, [], [f32((3, 1, 1), [23, 67, 127])])


@case
def fused_all():
    # kn-cuda-sys/tests/fused.rs: act(conv + res + bias) = -1*10 + 3 + 2
    g = Graph()
    x = g.input(shape(1, 1, 1, 1))
    res = g.input(shape(1, 1, 1, 1))
    w = g.constant(shape(1, 1, 1, 1), [10.0])
    b = g.constant(shape(1, 1, 1, 1), [2.0])
    y = g.add(g.add(g.conv(x, w, 1, 1, 0, 0), b), res)
    g.output(y)
    return Case("fused_all", g, 0, [f32((1, 1, 1, 1), [-1]), f32((1, 1, 1, 1), [3])], [f32((1, 1, 1, 1), [-5])])


@case
def horizontal_1x1_conv():
    g = Graph()
    x = g.constant(shape(2, 4, 1, 8), linspace(2 * 4 * 8))
    w = g.constant(shape(3, 4, 1, 1), linspace(3 * 4))
    o = g.conv(x, w, 1, 1, 0, 0)
    assert g[o].shape == shape(2, 3, 1, 8)
    g.output(o)
    return Case("horizontal_1x1_conv", g, 0, [])


@case
def vertical_1x1_conv():
    g = Graph()
    x = g.constant(shape(2, 4, 8, 1), linspace(2 * 4 * 8))
    w = g.constant(shape(3, 4, 1, 1), linspace(3 * 4))
    o = g.conv(x, w, 1, 1, 0, 0)
    assert g[o].shape == shape(2, 3, 8, 1)
    g.output(o)
    return Case("vertical_1x1_conv", g, 0, [])


@case
def fuse_clamp():
    g = Graph()
    c = g.input(shape(BATCH))
    c = g.clamp(c, -5.0, np.inf)
    c = g.clamp(c, -np.inf, 2.0)
    c = g.clamp(c, 0.0, 1.0)
    c = g.clamp(c, -1.0, 2.0)
    g.output(c)
    return Case("fuse_clamp", g, 5, [f32((5,), [-2, 0, 0.5, 1, 2])], [f32((5,), [0, 0, 0.5, 1, 1])])


def _ele_broadcast(op: BinaryOp):
    g = Graph()
    left = g.constant(shape(2, 3, 4), linspace(2 * 3 * 4))
    for s in [(), (1, 1, 1), (2, 3, 4), (2, 1, 4)]:
        right = g.constant(shape(s), linspace(int(np.prod(s))))
        g.output(g.binary(op, left, right))
    return Case(f"ele_broadcast_{op.name}", g, 0, [])


for _op in [BinaryOp.ADD, BinaryOp.SUB, BinaryOp.MUL, BinaryOp.MIN, BinaryOp.MAX]:
    CASES.append(lambda op=_op: _ele_broadcast(op))


@case
def add_broadcast():
    g = Graph()
    left = g.constant(shape(2, 2, 2), [0, 1, 2, 3, 4, 5, 6, 7])
    right = g.constant(shape(1, 2, 2), [0, 1, 2, 3])
    scalar = g.constant(shape(), [10.0])
    g.output_all([g.add(left, right), g.add(right, left), g.add(right, scalar)])
    e01 = f32((2, 2, 2), [0, 2, 4, 6, 4, 6, 8, 10])
    return Case("add_broadcast", g, 0, [], [e01, e01, f32((1, 2, 2), [10, 11, 12, 13])])


@case
def affine_single_element():
    x = f32((8, 1, 1, 1), arange(8))
    expected = ((x + 1.0) * 2.0 * 10.0 + 3.0) * 4.0
    g = Graph()
    cs = shape(1, 1, 1, 1)
    bias_0 = g.constant(cs, [1.0])
    scale_0 = g.constant(cs, [2.0])
    filt = g.constant(cs, [10.0])
    bias_1 = g.constant(cs, [3.0])
    scale_1 = g.constant(cs, [4.0])
    c = g.input(shape(x.shape))
    c = g.add(c, bias_0)
    c = g.mul(c, scale_0)
    c = g.conv(c, filt, 1, 1, 0, 0)
    c = g.add(c, bias_1)
    c = g.mul(c, scale_1)
    g.output(c)
    return Case("affine_single_element", g, 0, [x], [expected])


@case
def affine_add_twice():
    g = Graph()
    x = g.input(shape(BATCH, 1, 1, 1))
    w1 = g.constant(shape(1, 1, 1, 1), [1.0])
    w2 = g.constant(shape(1, 1, 1, 1), [2.0])
    g.output(g.add(g.add(x, w1), w2))
    return Case("affine_add_twice", g, 2, [f32((2, 1, 1, 1), [0, 1])], [f32((2, 1, 1, 1), [3, 4])])


@case
def affine_single_div():
    g = Graph()
    left = g.constant(shape(2, 3), arange(6))
    right = g.scalar(2.0)
    g.output(g.binary(BinaryOp.DIV, left, right))
    return Case("affine_single_div", g, 0, [], [f32((2, 3), [0, 0.5, 1, 1.5, 2, 2.5])])


@case
def affine_multiple_channels():
    x = f32((8, 3, 1, 1), arange(24))
    g = Graph()
    bias_0 = g.constant(shape(1, 3, 1, 1), [1, 2, 3])
    scale_0 = g.constant(shape(1, 3, 1, 1), [2, 3, 4])
    filt = g.constant(shape(2, 3, 1, 1), [10, 20, 30, 40, 50, 60])
    bias_1 = g.constant(shape(1, 2, 1, 1), [3, 4])
    scale_1 = g.constant(shape(1, 2, 1, 1), [4, 5])
    c = g.input(shape(x.shape))
    c = g.add(c, bias_0)
    c = g.mul(c, scale_0)
    c = g.conv(c, filt, 1, 1, 0, 0)
    c = g.add(c, bias_1)
    c = g.mul(c, scale_1)
    g.output(c)
    return Case("affine_multiple_channels", g, 0, [x])


@case
def conv_padding():
    g = Graph()
    i0 = g.input(shape(1, 1, 1, 1))
    i1 = g.input(shape(1, 1, 8, 8))
    w = g.constant(shape(1, 1, 3, 3), arange(9))
    g.output_all([g.conv(i0, w, 1, 1, 1, 1), g.conv(i0, w, 1, 1, 4, 4), g.conv(i1, w, 1, 1, 1, 1),
                  g.conv(i1, w, 1, 1, 4, 1)])
    return Case("conv_padding", g, 0, [f32((1, 1, 1, 1), [1.0]), linspace(1, 1, 8, 8)])


@case
def affine_padding():
    g = Graph()
    w = g.constant(shape(5, 3, 3, 3), linspace(5, 3, 3, 3))
    bias_0 = g.constant(shape(1, 3, 1, 1), linspace(3))
    bias_1 = g.constant(shape(1, 5, 1, 1), linspace(5))
    c = g.input(shape(8, 3, 8, 8))
    c = g.add(c, bias_0)
    c = g.conv(c, w, 1, 1, 1, 1)
    c = g.add(c, bias_1)
    g.output(c)
    return Case("affine_padding", g, 0, [linspace(8, 3, 8, 8)])


def _channel_batchnorm(g: Graph, x):
    c = g[x].shape[1].unwrap_fixed()
    cs = shape(1, c, 1, 1)
    mean = g.constant(cs, linspace(c))
    var = g.constant(cs, linspace(c))
    scale = g.constant(cs, linspace(c))
    bias = g.constant(cs, linspace(c))
    cur = g.add(x, mean)
    cur = g.mul(cur, var)
    cur = g.mul(cur, scale)
    return g.add(cur, bias)


@case
def pre_act_resnet():
    g = Graph()
    x = g.input(shape(8, 3, 8, 8))
    f_init = g.constant(shape(5, 3, 3, 3), linspace(5 * 3 * 3 * 3))
    f_tower = g.constant(shape(5, 5, 3, 3), linspace(5 * 5 * 3 * 3))
    f_policy = g.constant(shape(2, 5, 1, 1), linspace(10))
    tower = g.conv(x, f_init, 1, 1, 1, 1)
    for _ in range(2):
        c = _channel_batchnorm(g, tower)
        c = g.clamp(c, 0.0, 6.0)
        c = g.conv(c, f_tower, 1, 1, 1, 1)
        c = g.clamp(c, 0.0, 6.0)
        c = g.conv(c, f_tower, 1, 1, 1, 1)
        tower = g.add(c, tower)
    policy = g.conv(tower, f_policy, 1, 1, 0, 0)
    g.output_all([tower, policy])
    return Case("pre_act_resnet", g, 0, [linspace(8, 3, 8, 8)])


@case
def fuse_res():
    g = Graph()
    x = g.input(shape(10, 4, 8, 8))
    other = g.input(shape(10, 4, 8, 8))
    w = g.constant(shape(4, 4, 3, 3), linspace(4 * 4 * 3 * 3))
    c = g.conv(x, w, 1, 1, 1, 1)
    c = g.add(c, other)
    c = g.clamp(c, 0.0, np.inf)
    g.output(c)
    return Case("fuse_res", g, 0, [rng_f32(0, 10, 4, 8, 8), rng_f32(1, 10, 4, 8, 8)])


@case
def concat():
    g = Graph()
    a = g.constant(shape(2, 3, 4), linspace(24))
    b = g.constant(shape(2, 1, 4), linspace(8))
    c = g.constant(shape(2, 8, 4), linspace(64))
    g.output(g.concat([a, b, c], 1))
    return Case("concat", g, 0, [])


@case
def pad():
    g = Graph()
    a = g.constant(shape(2, 3, 4), linspace(24))
    zero = g.scalar(0.0)
    g.output(g.pad(a, [(0, 0), (1, 2), (2, 0)], zero))
    return Case("pad", g, 0, [])


@case
def permute():
    g = Graph()
    a = g.constant(shape(2, 3, 4, 5), arange(120))
    for p in itertools.permutations(range(4)):
        g.output(g.permute(a, list(p)))
    return Case("permute", g, 0, [])


@case
def chain():
    child = Graph()
    cx = child.input(shape(2))
    cw = child.constant(shape(1), [2.0])
    child.output(child.mul(cx, cw))
    parent = Graph()
    px = parent.input(shape(2))
    pw = parent.constant(shape(1), [3.0])
    pz = parent.add(px, pw)
    py = parent.call(child, [pz])
    assert len(py) == 1
    parent.output(py[0])
    return Case("chain", parent, 0, [f32((2,), [1, 2])], [f32((2,), [8, 10])])


@case
def repeated_conv():
    g = Graph()
    w0 = g.constant(shape(4, 4, 3, 3), np.linspace(-1, 1, 144))
    w1 = g.constant(shape(4, 4, 3, 3), np.linspace(-2, 2, 144))
    x = g.input(shape(BATCH, 4, 8, 8))
    a = x
    b = x
    for _ in range(4):
        a = g.conv(a, w0, 1, 1, 1, 1)
        b = g.conv(b, w1, 1, 1, 1, 1)
    g.output_all([a, b])
    return Case("repeated_conv", g, 2, [linspace(2, 4, 8, 8)])


@case
def strided_conv():
    g = Graph()
    x = g.input(shape(BATCH, 3, 8, 8))
    w = g.constant(shape(16, 3, 3, 3), rng_f32(0, 16 * 27))
    o = g.conv(x, w, 2, 4, 1, 1)
    assert g[o].shape == shape(BATCH, 16, 4, 2)
    g.output(o)
    return Case("strided_conv", g, 4, [rng_f32(1, 4, 3, 8, 8)])


@case
def softmax():
    g = Graph()
    x = g.input(shape(3, 3))
    r0 = g.softmax(x, 0)
    r1 = g.softmax(x, 1)
    r2 = g.softmax(g.mul(x, g.scalar(2.0)), 0)
    g.output_all([r0, r1, r2])
    return Case("softmax", g, 0, [f32((3, 3), [0, 0, 0, 1, 2, 3, 1, -1, -np.inf])])


@case
def reduce_easy():
    g = Graph()
    x = g.input(shape(4, 3))
    for axis in (0, 1):
        for op in REDUCE_ALL:
            g.output(g.reduce(x, [axis], op))
    return Case("reduce_easy", g, 0, [f32((4, 3), [0, 0, 0, 1, 2, 3, 1, -1, -np.inf, 0, 1, 2])])


@case
def reduce_mixed():
    g = Graph()
    x = g.input(shape(12, 3, 7, 9, 13))
    mixed = g.permute(x, [0, 3, 2, 1, 4])
    g.output(g.reduce(mixed, [1, 2, 4], ReduceOp.SUM))
    return Case("reduce_mixed", g, 0, [linspace(12, 3, 7, 9, 13)])


@case
def reduce_single():
    g = Graph()
    x = g.input(shape(4))
    g.output(g.reduce(x, [0], ReduceOp.SUM))
    return Case("reduce_single", g, 0, [linspace(4)])


@case
def softmax_single():
    g = Graph()
    x = g.input(shape(4))
    g.output(g.softmax(x, 0))
    return Case("softmax_single", g, 0, [linspace(4)])


@case
def layernorm_composed():
    # the unfused graph of graphs.rs:layernorm_fused (the optimizer pass is a separate component)
    eps, axis = 1e-5, 2
    g = Graph()
    x = g.input(shape(BATCH, 8, 32))
    red = shape(BATCH, 8, 1)
    c2 = g.scalar(2.0)
    ceps = g.scalar(eps)
    mean = g.view(g.reduce(x, [axis], ReduceOp.MEAN), red)
    zeroed = g.sub(x, mean)
    var = g.view(g.reduce(g.pow(zeroed, c2), [axis], ReduceOp.MEAN), red)
    std = g.unary(UnaryOp.SQRT, g.add(var, ceps))
    g.output(g.binary(BinaryOp.DIV, zeroed, std))
    return Case("layernorm_composed", g, 2, [linspace(2, 8, 32)])


@case
def layernorm_op():
    # the graph the reference's optimizer reduces layernorm_fused to: Input -> Layernorm
    g = Graph()
    x = g.input(shape(BATCH, 8, 32))
    g.output(g.layernorm(x, 2, 1e-5))
    return Case("layernorm_op", g, 2, [linspace(2, 8, 32)])


@case
def layernorm_residual_scaled():
    # exercises the `alpha0*x0 + alpha1*x1` folding (planner.rs:522-552) on a middle axis
    g = Graph()
    a = g.input(shape(BATCH, 24, 5))
    b = g.input(shape(BATCH, 24, 5))
    s = g.add(g.mul(a, g.scalar(0.5)), g.mul(g.scalar(-2.0), b))
    g.output(g.layernorm(s, 1, 1e-5))
    return Case("layernorm_residual_scaled", g, 3, [rng_f32(5, 3, 24, 5), rng_f32(6, 3, 24, 5)])


@case
def scalar_scalar():
    g = Graph()
    x = g.input(shape())
    g.output(g.unary(UnaryOp.EXP, x))
    return Case("scalar_scalar", g, 0, [f32((), [2.0])])


@case
def split_stride():
    g = Graph()
    n = 4
    x = g.input(shape(2 * n))
    g.output(g.slice(x, 0, SliceRange(1, 2 * n + 1, 2)))
    return Case("split_stride", g, 0, [rng_f32(0, 2 * n)])


def _complex_multiply(new_axis: bool):
    batch, n, axis = 8, 32, 1
    g = Graph()
    a = g.input(shape(batch, n * 2))
    b = g.input(shape(batch, n * 2))
    if new_axis:
        a_s = g.view(a, shape(batch, n, 2))
        b_s = g.view(b, shape(batch, n, 2))
        ar = g.view(g.slice(a_s, axis + 1, SliceRange.single(0)), shape(batch, n))
        ai = g.view(g.slice(a_s, axis + 1, SliceRange.single(1)), shape(batch, n))
        br = g.view(g.slice(b_s, axis + 1, SliceRange.single(0)), shape(batch, n))
        bi = g.view(g.slice(b_s, axis + 1, SliceRange.single(1)), shape(batch, n))
    else:
        ar = g.slice(a, axis, SliceRange(0, n * 2, 2))
        ai = g.slice(a, axis, SliceRange(1, n * 2 + 1, 2))
        br = g.slice(b, axis, SliceRange(0, n * 2, 2))
        bi = g.slice(b, axis, SliceRange(1, n * 2 + 1, 2))
    r = g.sub(g.mul(ar, br), g.mul(ai, bi))
    i = g.add(g.mul(ar, bi), g.mul(ai, br))
    cat = g.concat([g.view(r, shape(batch, n, 1)), g.view(i, shape(batch, n, 1))], axis + 1)
    g.output(g.view(cat, shape(batch, n * 2)))
    xa, xb = rng_f32(0, batch, n * 2), rng_f32(1, batch, n * 2)
    exp = np.empty_like(xa)
    exp[:, 0::2] = xa[:, 0::2] * xb[:, 0::2] - xa[:, 1::2] * xb[:, 1::2]
    exp[:, 1::2] = xa[:, 0::2] * xb[:, 1::2] + xa[:, 1::2] * xb[:, 0::2]
    return Case("complex_multiply_" + ("new_axis" if new_axis else "stride"), g, 0, [xa, xb], [exp])


@case
def complex_multiply_stride():
    return _complex_multiply(False)


@case
def complex_multiply_new_axis():
    return _complex_multiply(True)


# ------------------------------------------------------------------ elementwise.rs
def _rust_unary_f32(op: UnaryOp, x: np.ndarray) -> np.ndarray:
    """Closed forms of `UnaryOp::map` for f32 (graph.rs:1649-1705) evaluated independently of the oracle module."""
    import math
    out = np.empty_like(x)
    a = [1.0, 0.0705230784, 0.0422820123, 0.0092705272, 0.0001520143, 0.0002765672, 0.0000430638]
    for i, v in enumerate(x):
        v = np.float32(v)
        with np.errstate(all="ignore"):
            if op == UnaryOp.ABS:
                r = abs(v)
            elif op == UnaryOp.NEG:
                r = -v
            elif op == UnaryOp.SIN:
                r = np.sin(v)
            elif op == UnaryOp.COS:
                r = np.cos(v)
            elif op == UnaryOp.EXP:
                r = np.exp(v)
            elif op == UnaryOp.LOG:
                r = np.log(v)
            elif op == UnaryOp.SQRT:
                r = np.sqrt(v)
            elif op == UnaryOp.SIGMOID:
                r = np.float32(1) / (np.float32(1) + np.exp(-v))
            elif op == UnaryOp.TANH:
                r = np.tanh(v)
            elif op == UnaryOp.ERF:
                xa = abs(float(v))
                d = sum(c * xa ** k for k, c in enumerate(a))
                r = math.copysign(1.0 - 1.0 / d ** 16, float(v))
            elif op == UnaryOp.MISH:
                r = v * np.tanh(np.log1p(np.exp(v)))
            elif op == UnaryOp.SOFTPLUS:
                r = np.log1p(np.exp(-abs(v))) + max(v, np.float32(0))
            else:
                raise AssertionError(op)
        out[i] = r
    return out


def _unary(op: UnaryOp):
    g = Graph()
    v = ELEMENTWISE_TEST_VALUES
    x = g.input(shape(len(v)))
    g.output(g.unary(op, x))
    return Case(f"unary_{op.name}", g, 0, [v.copy()], [_rust_unary_f32(op, v)])


for _op in UNARY_ALL:
    CASES.append(lambda op=_op: _unary(op))


@case
def unary_fixed():
    g = Graph()
    x = g.input(shape(BATCH))
    g.output(g.unary(UnaryOp.SOFTPLUS, x))
    return Case("unary_fixed", g, 5, [f32((5,), [-2, -1, 0, 1, 2])],
                [f32((5,), [0.126928, 0.313262, 0.693147, 1.313262, 2.126928])])


def _rust_binary_f32(op: BinaryOp, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    with np.errstate(all="ignore"):
        return {
            BinaryOp.ADD: lambda: a + b, BinaryOp.SUB: lambda: a - b, BinaryOp.MUL: lambda: a * b,
            BinaryOp.DIV: lambda: a / b, BinaryOp.POW: lambda: np.power(a, b),
            BinaryOp.MIN: lambda: np.fmin(a, b), BinaryOp.MAX: lambda: np.fmax(a, b),
        }[op]().astype(np.float32)


def _binary(op: BinaryOp):
    g = Graph()
    v = ELEMENTWISE_TEST_VALUES
    n = len(v) * len(v)
    l = g.input(shape(n))
    r = g.input(shape(n))
    g.output(g.binary(op, l, r))
    lt = np.repeat(v, len(v))
    rt = np.tile(v, len(v))
    return Case(f"binary_{op.name}", g, 0, [lt, rt], [_rust_binary_f32(op, lt, rt)])


for _op in BINARY_ALL:
    CASES.append(lambda op=_op: _binary(op))


def _clamp(lo, hi):
    g = Graph()
    v = ELEMENTWISE_TEST_VALUES
    x = g.input(shape(len(v)))
    g.output(g.clamp(x, lo, hi))
    return Case(f"clamp_{lo}_{hi}", g, 0, [v.copy()], [np.clip(v, lo, hi).astype(np.float32)])


for _lo, _hi in itertools.product([-np.inf, 0.0], [np.inf, 6.0]):
    CASES.append(lambda lo=_lo, hi=_hi: _clamp(lo, hi))


@case
def value_cast():
    pairs = [
        (np.uint8(5), np.uint8(5)), (np.uint32(5), np.uint32(5)), (np.float32(5), np.float32(5)),
        (np.uint64(0xdeadbeefdeadbeef), np.uint64(0xdeadbeefdeadbeef)),
        (np.uint8(1), np.uint32(1)), (np.int8(-1), np.uint32(0xFFFFFFFF)),
        (np.uint32(1), np.uint8(1)), (np.int32(-1), np.uint8(255)),
        (np.float32(1), np.uint32(1)), (np.float32(-1), np.int32(-1)), (np.float32(-1), np.int64(-1)),
        (np.float32(-1), np.int8(-1)),
    ]
    g = Graph()
    ins, outs = [], []
    for x, y in pairs:
        xv = g.input(shape(), DType.of(x.dtype))
        g.output(g.value_cast(xv, DType.of(y.dtype)))
        ins.append(np.asarray(x))
        outs.append(np.asarray(y))
    return Case("value_cast", g, 0, ins, outs)


@case
def bit_cast():
    one_bits = np.float32(1).view(np.uint32)
    neg_bits = np.float32(-1).view(np.uint32)
    pairs = [
        (np.uint8(5), np.uint8(5)), (np.uint32(5), np.uint32(5)), (np.float32(5), np.float32(5)),
        (np.uint64(0xdeadbeefdeadbeef), np.uint64(0xdeadbeefdeadbeef)),
        (np.float32(1), one_bits), (np.float32(-1), neg_bits),
    ]
    g = Graph()
    ins, outs = [], []
    for x, y in pairs:
        xv = g.input(shape(), DType.of(x.dtype))
        g.output(g.bit_cast(xv, DType.of(y.dtype)))
        ins.append(np.asarray(x))
        outs.append(np.asarray(y))
    return Case("bit_cast", g, 0, ins, outs)


@case
def int_ops():
    # not in the reference suite: integer / bool arithmetic, wrap-around casts and integer reduce
    g = Graph()
    a = g.input(shape(BATCH, 6), DType.I32)
    b = g.input(shape(BATCH, 6), DType.I32)
    m = g.input(shape(BATCH, 6), DType.BOOL)
    n = g.input(shape(BATCH, 6), DType.BOOL)
    f = g.input(shape(BATCH, 6), DType.F32)
    g.output_all([
        g.add(a, b), g.sub(a, b), g.mul(a, b), g.binary(BinaryOp.MIN, a, b), g.binary(BinaryOp.MAX, a, b),
        g.unary(UnaryOp.ABS, a), g.unary(UnaryOp.NEG, a),
        g.add(m, n), g.mul(m, n), g.sub(m, n),
        g.value_cast(a, DType.I8), g.value_cast(a, DType.U16), g.value_cast(a, DType.F32), g.value_cast(a, DType.BOOL),
        g.value_cast(f, DType.I8), g.value_cast(f, DType.U8), g.value_cast(f, DType.I64), g.value_cast(f, DType.BOOL),
        g.value_cast(f, DType.F64), g.value_cast(m, DType.F32),
        g.reduce(a, [1], ReduceOp.SUM), g.reduce(a, [1], ReduceOp.MAX), g.reduce(a, [1], ReduceOp.MIN),
    ])
    r = np.random.Generator(np.random.PCG64(11))
    av = r.integers(-1000, 1000, (2, 6), dtype=np.int32)
    bv = r.integers(-1000, 1000, (2, 6), dtype=np.int32)
    mv = r.integers(0, 2, (2, 6)).astype(np.bool_)
    nv = r.integers(0, 2, (2, 6)).astype(np.bool_)
    fv = f32((2, 6), [0.0, -0.0, 0.5, -0.5, 1.9, -1.9, 127.0, 128.0, 300.7, -300.7, 65536.0, -3.0e9])
    return Case("int_ops", g, 2, [av, bv, mv, nv, fv])


# ------------------------------------------------------------------ opt.rs
@case
def chained_scalar():
    g = Graph()
    x = g.input(shape(2, 3))
    w1 = g.constant(shape(1, 3), [1, 2, 3])
    w2 = g.constant(shape(2, 1), [0.1, 0.2])
    g.output(g.add(g.mul(x, w1), w2))
    return Case("chained_scalar", g, 0, [np.ones((2, 3), np.float32)], [f32((2, 3), [1.1, 2.1, 3.1, 1.2, 2.2, 3.2])])


def _scalar_topology(kind: str):
    g = Graph()
    x = g.input(shape(2, 3))
    w1 = g.constant(shape(1, 3), rng_f32(0, 3))
    w2 = g.constant(shape(2, 1), rng_f32(1, 2))
    y1 = g.mul(x, w1)
    y2 = g.add(x, w2)
    if kind == "split":
        g.output_all([y1, y2])
    else:
        y3 = g.binary(BinaryOp.MAX, y1, y2)
        g.output_all([y3] if kind == "rejoining" else [y1, y3])
    return Case(f"{kind}_scalar", g, 0, [rng_f32(2, 2, 3)])


for _k in ("split", "rejoining", "inner_used"):
    CASES.append(lambda k=_k: _scalar_topology(k))


def all_cases() -> List[Case]:
    return [fn() for fn in CASES]
