"""Stride-1 convolutions with a long reduction as a matmul that reads its windows straight from the channels-last
image (GemmParams::conv_operand, kernels/gemm_persistent.cu): which convolutions the planner routes there (CPU)
and that the result is the oracle's (GPU).  The oracle follows the reference's convolution
(kn-graph/src/cpu.rs `convolution`)."""
import numpy as np
import pytest

from kyanite_b200.executor import FLAG_NO_PERSISTENT_GEMM, MATH_F32, MATH_TF32, CudaExecutor, plan_describe
from kyanite_b200.graph import BATCH, Graph, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def conv_graph(c, k, h, w, r, s, pad, seed=0, relu=True, regroup=None, skip=False):
    """conv + bias (+ skip) (+ relu); `regroup` = groups: the result goes through a group norm, whose [N, groups, rest]
    view a channels-last result cannot offer (the planner takes the view into the step when no activation sits in
    between, so those graphs have none)."""
    rg = rng(seed)
    g = Graph()
    x = g.input(shape(BATCH, c, h, w))
    wgt = (rg.standard_normal((k, c, r, s)) * np.sqrt(2.0 / (c * r * s))).astype(np.float32)
    b = (0.1 * rg.standard_normal((1, k, 1, 1))).astype(np.float32)
    y = g.add(g.conv(x, g.constant_tensor(wgt), 1, 1, pad, pad), g.constant_tensor(b))
    oh, ow = h + 2 * pad - r + 1, w + 2 * pad - s + 1
    if skip:
        y = g.add(y, g.input(shape(BATCH, k, oh, ow)))
    if relu and not regroup:
        y = g.relu(y)
    if regroup:
        y = g.layernorm(g.view(y, shape(BATCH, regroup, k // regroup * oh * ow)), 2, 1e-5)
    g.output(y)
    return g, (oh, ow)


def steps(description):
    return [line for line in description.splitlines() if line.startswith("step")]


def test_long_reduction_convolution_reads_the_image():
    g, _ = conv_graph(320, 320, 64, 64, 3, 3, 1)
    d = plan_describe(g, 2, MATH_TF32)
    assert any("windows read from the image as operand a" in l for l in steps(d)), d
    assert not any(" Im2col " in l for l in steps(d))
    # a view that needs plain NCHW memory: channels x positions, the image is operand b
    g, _ = conv_graph(320, 320, 64, 64, 3, 3, 1, regroup=32)
    d = plan_describe(g, 2, MATH_TF32)
    assert any("windows read from the image as operand b" in l for l in steps(d)), d
    assert not any(" Im2col " in l for l in steps(d))


def test_other_convolutions_keep_their_route():
    # output rows that do not tile the operand tile (width 24), channels not in whole 32-blocks, a strided convolution,
    # the persistent kernel switched off, exact f32: none of them takes the implicit route
    for graph, kwargs in (
        (conv_graph(320, 320, 24, 24, 3, 3, 1)[0], {"math_mode": MATH_TF32}),
        (conv_graph(336, 320, 32, 32, 3, 3, 1)[0], {"math_mode": MATH_TF32}),
        (conv_graph(320, 320, 64, 64, 3, 3, 1)[0], {"math_mode": MATH_TF32, "flags": FLAG_NO_PERSISTENT_GEMM}),
        (conv_graph(320, 320, 64, 64, 3, 3, 1)[0], {"math_mode": MATH_F32}),
    ):
        d = plan_describe(graph, 2, **kwargs)
        assert not any("windows read from the image" in l for l in steps(d)), d


CASES = {
    # name: (c, k, h, w, r, s, pad, batch, kwargs)
    "same_3x3": (256, 128, 16, 16, 3, 3, 1, 2, {}),
    "same_3x3_nchw": (256, 128, 16, 16, 3, 3, 1, 2, {"regroup": 8}),
    "skip_and_bias": (256, 128, 16, 16, 3, 3, 1, 3, {"skip": True}),
    "wide_rows": (256, 96, 8, 32, 3, 3, 1, 2, {"relu": False}),
    "valid_3x3": (256, 128, 18, 18, 3, 3, 0, 2, {}),
    "five_by_five": (96, 128, 16, 16, 5, 5, 2, 2, {}),
    "five_by_five_nchw": (96, 128, 16, 16, 5, 5, 2, 2, {"regroup": 4}),
    "many_tiles": (256, 160, 32, 32, 3, 3, 1, 4, {}),
    "many_tiles_nchw": (256, 160, 32, 32, 3, 3, 1, 4, {"regroup": 32}),
    "row_tail": (256, 128, 12, 32, 3, 3, 1, 2, {}),          # 384 positions: the third tile of 128 is whole, 12 rows of 32
    "position_tail_nchw": (256, 128, 20, 16, 3, 3, 1, 2, {"regroup": 2}),   # 320 positions in column blocks of 160
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_routes(name):
    c, k, h, w, r, s, pad, batch, kw = CASES[name]
    g, _ = conv_graph(c, k, h, w, r, s, pad, **kw)
    d = plan_describe(g, batch, MATH_TF32)
    want = "operand b" if "regroup" in kw else "operand a"
    assert any("windows read from the image as " + want in l for l in steps(d)), d


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_matches_oracle(name):
    c, k, h, w, r, s, pad, batch, kw = CASES[name]
    g, (oh, ow) = conv_graph(c, k, h, w, r, s, pad, seed=3, **kw)
    rg = rng(11)
    inputs = [rg.standard_normal((batch, c, h, w)).astype(np.float32)]
    if kw.get("skip"):
        inputs.append(rg.standard_normal((batch, k, oh, ow)).astype(np.float32))
    expected = cpu_eval_graph(g.to_bytes(), batch, inputs)
    with CudaExecutor(0, g, batch, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
        again = ex.evaluate(inputs)
    # TF32 operands (10-bit mantissa) under a reduction of c * r * s terms: 4e-3 of the largest expected magnitude
    assert_tensors_match(expected, got, 4e-3, 4e-3, abs_scaled=True)
    for a, b in zip(got, again):
        np.testing.assert_array_equal(a, b)


@pytest.mark.gpu
def test_same_result_as_the_materialised_route():
    """Both routes multiply the same TF32-rounded operands tile by tile in the same order of K blocks."""
    c, k, h, w = 320, 320, 32, 32
    g, _ = conv_graph(c, k, h, w, 3, 3, 1, seed=5)
    x = rng(6).standard_normal((2, c, h, w)).astype(np.float32)
    with CudaExecutor(0, g, 2, math_mode=MATH_TF32) as ex:
        implicit = ex.evaluate([x])[0]
    g2, _ = conv_graph(c, k, h, w, 3, 3, 1, seed=5)
    with CudaExecutor(0, g2, 2, math_mode=MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        other = ex.evaluate([x])[0]
    assert_tensors_match([other], [implicit], 1e-3, 1e-3, abs_scaled=True)


def two_convs_with_skip(c, hw, groups, seed=0):
    """y1 = relu(conv(x) + b1) (channels-last result); out = groupnorm-view(conv(y1) + b2 + y1): the second step wants
    plain NCHW memory and gets its skip tensor channels-last."""
    rg = rng(seed)
    g = Graph()
    x = g.input(shape(BATCH, c, hw, hw))

    def conv(t):
        wgt = (rg.standard_normal((c, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
        b = (0.1 * rg.standard_normal((1, c, 1, 1))).astype(np.float32)
        return g.add(g.conv(t, g.constant_tensor(wgt), 1, 1, 1, 1), g.constant_tensor(b))

    y1 = g.relu(conv(x))
    y2 = g.add(conv(y1), y1)
    g.output(g.layernorm(g.view(y2, shape(BATCH, groups, c // groups * hw * hw)), 2, 1e-5))
    return g


def test_skip_tensor_in_the_other_layout_is_copied():
    d = plan_describe(two_convs_with_skip(256, 16, 8), 2, MATH_TF32)
    lines = steps(d)
    assert sum("windows read from the image as operand a" in l for l in lines) == 1, d
    assert sum("windows read from the image as operand b" in l for l in lines) == 1, d


@pytest.mark.gpu
def test_skip_tensor_in_the_other_layout_matches_oracle():
    g = two_convs_with_skip(256, 16, 8, seed=2)
    x = rng(4).standard_normal((2, 256, 16, 16)).astype(np.float32)
    expected = cpu_eval_graph(g.to_bytes(), 2, [x])
    with CudaExecutor(0, g, 2, math_mode=MATH_TF32) as ex:
        got = ex.evaluate([x])
    # the normalised output has unit scale; two chained TF32 convolutions in front of it
    assert_tensors_match(expected, got, 4e-3, 4e-3, abs_scaled=True)
