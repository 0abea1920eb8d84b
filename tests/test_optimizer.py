"""Graph optimiser (kyanite_b200/optimizer.py) against the reference's behaviour: its test runner pushes
every graph through `optimize_graph` and requires the same outputs (kn-cuda-eval/tests/root/runner.rs:10-26),
and a few tests look at the shape of the optimised graph (graphs.rs:907-926 layernorm_fused, opt.rs:95-125
gather_cast)."""
import collections
import os

import numpy as np
import pytest

import ref_graphs
from kyanite_b200.graph import BATCH, BinaryOp, DType, Graph, OpKind, ReduceOp, SliceRange, UnaryOp, shape
from kyanite_b200.optimizer import OptimizerSettings, optimize_graph
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

CASES = ref_graphs.all_cases()
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def kinds(graph: Graph):
    return collections.Counter(v.kind for v in graph.values)


def binary_ops(graph: Graph):
    return collections.Counter(v.binary_op for v in graph.values if v.kind == OpKind.BINARY)


def check_same(graph: Graph, optimized: Graph, batch, inputs, tol=1e-3):
    expected = cpu_eval_graph(graph.to_bytes(), batch, inputs)
    actual = cpu_eval_graph(optimized.to_bytes(), batch, inputs)
    assert_tensors_match(expected, actual, tol, tol)
    return expected


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_optimized_reference_graph_matches_oracle(case):
    optimized = optimize_graph(case.graph)
    assert [optimized[v].shape for v in optimized.inputs] == [case.graph[v].shape for v in case.graph.inputs]
    assert [optimized[v].shape for v in optimized.outputs] == [case.graph[v].shape for v in case.graph.outputs]
    expected = check_same(case.graph, optimized, case.batch_size, case.inputs)
    if case.expected is not None:
        assert_tensors_match(case.expected, expected)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_optimized_reference_graph_on_gpu(case):
    from kyanite_b200.executor import MATH_F32, CudaExecutor
    optimized = optimize_graph(case.graph)
    expected = case.expected if case.expected is not None else \
        cpu_eval_graph(case.graph.to_bytes(), case.batch_size, case.inputs)
    with CudaExecutor(0, optimized, case.batch_size, math_mode=MATH_F32) as ex:
        assert_tensors_match(expected, ex.evaluate(case.inputs), 1e-3, 1e-3)


def test_layernorm_collapses_to_two_values():
    case = next(c for c in CASES if c.name == "layernorm_composed")
    optimized = optimize_graph(case.graph)
    assert len(optimized.values) == 2
    out = optimized[optimized.outputs[0]]
    assert out.kind == OpKind.LAYERNORM and out.axis == 2 and abs(out.eps - 1e-5) < 1e-12
    check_same(case.graph, optimized, case.batch_size, case.inputs)
    # switched off, the pattern survives
    kept = optimize_graph(case.graph, OptimizerSettings(fuse_layernorm=False))
    assert kinds(kept)[OpKind.REDUCE] == 2


def test_layernorm_is_not_fused_when_an_inner_value_escapes():
    g = Graph()
    x = g.input(shape(BATCH, 8, 32))
    red = shape(BATCH, 8, 1)
    mean = g.view(g.reduce(x, [2], ReduceOp.MEAN), red)
    zeroed = g.sub(x, mean)
    var = g.view(g.reduce(g.pow(zeroed, g.scalar(2.0)), [2], ReduceOp.MEAN), red)
    std = g.unary(UnaryOp.SQRT, g.add(var, g.scalar(1e-5)))
    g.output(g.binary(BinaryOp.DIV, zeroed, std))
    g.output(zeroed)        # the centred value is also an output
    optimized = optimize_graph(g)
    assert kinds(optimized)[OpKind.LAYERNORM] == 0
    check_same(g, optimized, 2, [rng(1).standard_normal((2, 8, 32)).astype(np.float32)])


def test_clamp_chain_becomes_one_min_and_one_max():
    g = Graph()
    x = g.input(shape(BATCH, 6))
    y = g.binary(BinaryOp.MIN, x, g.scalar(3.0))
    y = g.binary(BinaryOp.MAX, y, g.scalar(-2.0))
    y = g.binary(BinaryOp.MIN, y, g.scalar(1.5))
    y = g.binary(BinaryOp.MAX, y, g.scalar(-1.0))
    g.output(g.unary(UnaryOp.EXP, y))        # the chain itself must be hidden to be followed
    optimized = optimize_graph(g)
    ops = binary_ops(optimized)
    assert ops[BinaryOp.MIN] == 1 and ops[BinaryOp.MAX] == 1
    check_same(g, optimized, 2, [np.linspace(-4, 4, 12, dtype=np.float32).reshape(2, 6)])


def test_div_by_constant_becomes_mul():
    # the divisor must be constant as a whole tensor, so it cannot be broadcast along the batch axis
    # (constants are evaluated without a batch size, kn-graph/src/cpu.rs:116-131)
    g = Graph()
    x = g.input(shape(2, 3))
    g.output(g.binary(BinaryOp.DIV, x, g.constant_tensor(np.array([[2.0, 4.0, -8.0]], np.float32))))
    optimized = optimize_graph(g)
    assert binary_ops(optimized) == {BinaryOp.MUL: 1}
    check_same(g, optimized, 0, [rng(2).standard_normal((2, 3)).astype(np.float32)])
    kept = optimize_graph(g, OptimizerSettings(div_to_mul=False))
    assert binary_ops(kept) == {BinaryOp.DIV: 1}
    batched = Graph()
    xb = batched.input(shape(BATCH, 3))
    batched.output(batched.binary(BinaryOp.DIV, xb, batched.constant_tensor(np.array([[2.0, 4.0, -8.0]], np.float32))))
    assert binary_ops(optimize_graph(batched)) == {BinaryOp.DIV: 1}


def conv_bn_graph(padding: int, bias_before: bool):
    r = rng(3)
    g = Graph()
    x = g.input(shape(BATCH, 4, 6, 6))

    def chan(c, positive=False):
        data = r.standard_normal((1, c, 1, 1)).astype(np.float32)
        return g.constant_tensor(np.abs(data) + 0.5 if positive else data)

    cur = x
    if bias_before:
        cur = g.mul(g.add(cur, chan(4)), chan(4))
    k = 2 * padding + 1
    cur = g.conv(cur, g.constant_tensor(r.standard_normal((5, 4, k, k)).astype(np.float32)), 1, 1, padding, padding)
    cur = g.add(cur, chan(5))
    # batch norm as the ONNX loader spells it
    cur = g.binary(BinaryOp.DIV, g.sub(cur, chan(5)), g.unary(UnaryOp.SQRT, g.add(chan(5, True), g.scalar(1e-5))))
    cur = g.add(g.mul(cur, chan(5)), chan(5))
    g.output(g.relu(cur))
    return g, [r.standard_normal((2, 4, 6, 6)).astype(np.float32)]


def test_conv_batchnorm_folds_into_filter_and_bias():
    g, inputs = conv_bn_graph(padding=1, bias_before=False)
    optimized = optimize_graph(g)
    assert kinds(optimized)[OpKind.CONV] == 1
    assert binary_ops(optimized) == {BinaryOp.ADD: 1, BinaryOp.MAX: 1}       # bias and relu
    check_same(g, optimized, 2, inputs, tol=1e-4)


def test_bias_before_conv():
    # no padding: the bias moves through the convolution and merges with the one behind it
    g, inputs = conv_bn_graph(padding=0, bias_before=True)
    optimized = optimize_graph(g)
    assert binary_ops(optimized) == {BinaryOp.ADD: 1, BinaryOp.MAX: 1}
    check_same(g, optimized, 2, inputs, tol=1e-4)
    # with padding it stays in front (scale and bias), unless forced into a full-size bias map
    g, inputs = conv_bn_graph(padding=1, bias_before=True)
    optimized = optimize_graph(g)
    assert binary_ops(optimized) == {BinaryOp.MUL: 1, BinaryOp.ADD: 2, BinaryOp.MAX: 1}
    check_same(g, optimized, 2, inputs, tol=1e-4)
    forced = optimize_graph(g, OptimizerSettings(force_bias_through_conv=True))
    assert binary_ops(forced) == {BinaryOp.ADD: 1, BinaryOp.MAX: 1}
    bias = next(v for v in forced.values if v.kind == OpKind.CONSTANT and v.tensor.shape == (1, 5, 6, 6))
    assert bias is not None
    check_same(g, forced, 2, inputs, tol=1e-4)


def test_gather_with_cast_index_is_a_slice():
    g = Graph()
    x = g.input(shape(4))
    i = g.value_cast(g.constant_tensor(np.array([0.0], np.float32)), DType.U32)
    g.output(g.gather(x, 0, i))
    optimized = optimize_graph(g)
    out = optimized[optimized.outputs[0]]
    assert out.kind == OpKind.SLICE and out.axis == 0 and out.range == SliceRange.single(0)
    assert out.inputs == (optimized.inputs[0].index,)


def test_dead_values_disappear_and_io_order_is_kept():
    g = Graph()
    a = g.input(shape(BATCH, 2))
    b = g.input(shape(BATCH, 3))          # never used
    g.unary(UnaryOp.EXP, a)               # dead
    y1 = g.unary(UnaryOp.SIN, a)
    y0 = g.unary(UnaryOp.COS, a)
    g.output(y0)
    g.output(y1)
    optimized = optimize_graph(g)
    assert [optimized[v].shape for v in optimized.inputs] == [g[a].shape, g[b].shape]
    assert [optimized[v].unary_op for v in optimized.outputs] == [UnaryOp.COS, UnaryOp.SIN]
    assert len(optimized.values) == 4
    same = optimize_graph(g, OptimizerSettings(optimize=False))
    assert same.to_bytes() == g.to_bytes()


def test_shared_affine_value_is_not_folded_twice():
    g = Graph()
    x = g.input(shape(BATCH, 3, 4, 4))
    w = g.constant_tensor(rng(4).standard_normal((3, 3, 3, 3)).astype(np.float32))
    c = g.conv(x, w, 1, 1, 1, 1)
    b = g.add(c, g.constant_tensor(rng(5).standard_normal((1, 3, 1, 1)).astype(np.float32)))
    g.output(g.relu(b))
    g.output(g.unary(UnaryOp.TANH, b))        # `b` has two users
    optimized = optimize_graph(g)
    assert kinds(optimized)[OpKind.CONV] == 1
    check_same(g, optimized, 2, [rng(6).standard_normal((2, 3, 4, 4)).astype(np.float32)])


@pytest.mark.parametrize("name", ["simple-bn-sttt-1x64", "pre-sttt-4x8", "att-tiny"])
def test_optimized_golden_model(name):
    from kyanite_b200.onnx import load_graph_from_onnx_path
    reference = os.environ.get("KN_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))
    path = os.path.join(reference, "kn-cuda-eval", "tests", "data", name + ".onnx")
    if not os.path.exists(path):
        pytest.skip("needs the reference checkout")
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    inputs = [z[k] for k in sorted(k for k in z.files if k.startswith("input"))]
    expected = [z[k] for k in sorted(k for k in z.files if k.startswith("output"))]
    graph = load_graph_from_onnx_path(path)
    optimized = optimize_graph(graph)
    assert len(optimized.values) < len(graph.values)
    if name == "pre-sttt-4x8":
        # all five batch norms fold away: no division and no square root is left
        assert binary_ops(optimized)[BinaryOp.DIV] == 0
        assert not any(v.kind == OpKind.UNARY and v.unary_op == UnaryOp.SQRT for v in optimized.values)
    assert_tensors_match(expected, cpu_eval_graph(optimized.to_bytes(), int(z["batch"]), inputs), 1e-3, 1e-3)
