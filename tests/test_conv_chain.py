"""Runs of 3x3 convolutions merged into the shared-memory-resident chain kernel (kernels/conv_chain.cu):
what the planner merges (CPU) and that the merged kernel computes what the per-layer kernels and the
oracle compute (GPU)."""
import re

import numpy as np
import pytest

from kyanite_b200.configs import resnet_tower
from kyanite_b200.executor import FLAG_NO_CONV_CHAIN, MATH_F32, MATH_TF32, plan_describe
from kyanite_b200.graph import BATCH, Graph, UnaryOp, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def tower(channels, blocks, h, w, c_in, seed=0, residual=True, relu=True, tap_value=False):
    """conv-bias-relu stem, then `blocks` x [conv-bias-relu, conv-bias-(+skip)-relu]."""
    r = rng(seed)
    g = Graph()
    x = g.input(shape(BATCH, c_in, h, w))

    def conv(t, cin, scale=1.0):
        wgt = (r.standard_normal((channels, cin, 3, 3)) * scale * np.sqrt(2.0 / (9 * cin))).astype(np.float32)
        b = (0.1 * r.standard_normal((1, channels, 1, 1))).astype(np.float32)
        return g.add(g.conv(t, g.constant_tensor(wgt), 1, 1, 1, 1), g.constant_tensor(b))

    cur = g.relu(conv(x, c_in))
    extra = None
    for i in range(blocks):
        y = g.relu(conv(cur, channels))
        if tap_value and i == 0:
            extra = y
        y = conv(y, channels, 0.5)
        if residual:
            y = g.add(y, cur)
        cur = g.relu(y) if relu else y
    g.output(cur)
    if extra is not None:
        g.output(g.unary(UnaryOp.TANH, extra))
    return g


def steps(description):
    return [line for line in description.splitlines() if line.startswith("step")]


def test_tower_becomes_one_chain():
    g, _ = resnet_tower()
    d = plan_describe(g, 256, MATH_TF32)
    chains = [l for l in steps(d) if " ConvChain/tc " in l]
    assert len(chains) == 1 and "layers=33" in chains[0]
    assert not any(" Conv/tc " in l and "rs=3x3" in l for l in steps(d))
    # the flag and exact-f32 mode keep one step per layer
    for kwargs in ({"math_mode": MATH_TF32, "flags": FLAG_NO_CONV_CHAIN}, {"math_mode": MATH_F32}):
        d = plan_describe(g, 256, **kwargs)
        assert not any("ConvChain" in l for l in steps(d))
        assert len([l for l in steps(d) if "rs=3x3" in l]) == 33


def test_chain_is_cut_where_an_intermediate_escapes():
    g = tower(32, 3, 8, 8, 32, tap_value=True)
    d = plan_describe(g, 32, MATH_TF32)
    chains = [l for l in steps(d) if " ConvChain/tc " in l]
    # The first conv of block 1 produces a graph output, so a chain would have to end there; but then the
    # stem's result, which the second conv of block 1 adds, would be needed outside that chain while only
    # a chain's last result reaches global memory.  So stem, first and second conv of block 1 stay steps
    # of their own, and the remaining four layers form a chain.
    assert [int(re.search(r"layers=(\d+)", l).group(1)) for l in chains] == [4]
    assert len([l for l in steps(d) if " Conv/tc " in l]) == 3


def test_images_too_large_for_a_chain_stay_per_layer():
    g = tower(32, 1, 19, 19, 8)
    d = plan_describe(g, 8, MATH_TF32)
    assert not any("ConvChain" in l for l in steps(d))


CASES = {
    "tower_8x8_c128": dict(channels=128, blocks=2, h=8, w=8, c_in=21, batch=8),
    "odd_batch": dict(channels=128, blocks=1, h=8, w=8, c_in=128, batch=5),
    "two_images": dict(channels=128, blocks=1, h=8, w=8, c_in=16, batch=2),
    "narrow_64": dict(channels=64, blocks=2, h=8, w=8, c_in=3, batch=6),
    "narrow_32_5x7": dict(channels=32, blocks=2, h=5, w=7, c_in=32, batch=9),
    "wide_board_9x9": dict(channels=96, blocks=1, h=9, w=9, c_in=2, batch=4),
    "tall_12x4": dict(channels=128, blocks=1, h=12, w=4, c_in=40, batch=7),
    "no_residual_no_relu": dict(channels=128, blocks=2, h=8, w=8, c_in=128, batch=4, residual=False, relu=False),
    "escaping_intermediate": dict(channels=64, blocks=2, h=6, w=6, c_in=64, batch=4, tap_value=True),
    "deep": dict(channels=128, blocks=10, h=8, w=8, c_in=21, batch=16),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_chain_matches_oracle_and_per_layer_kernels(name):
    from kyanite_b200.executor import CudaExecutor
    cfg = dict(CASES[name])
    batch = cfg.pop("batch")
    g = tower(seed=hash(name) % 1000, **cfg)
    x = rng(5).standard_normal((batch, cfg["c_in"], cfg["h"], cfg["w"])).astype(np.float32)
    assert any("ConvChain" in l for l in steps(plan_describe(g, batch, MATH_TF32)))
    expected = cpu_eval_graph(g.to_bytes(), batch, [x])
    with CudaExecutor(0, g, batch, math_mode=MATH_TF32) as ex:
        fused = ex.evaluate([x])
        assert_tensors_match(expected, fused, 4e-3, 4e-3, abs_scaled=True)
        for a, b in zip(fused, ex.evaluate([x])):                    # replay is deterministic
            np.testing.assert_array_equal(a, b)
    with CudaExecutor(0, g, batch, math_mode=MATH_TF32, flags=FLAG_NO_CONV_CHAIN) as ex:
        per_layer = ex.evaluate([x])
    # Same operands and the same TF32 rounding points; only the summation order inside a layer differs.
    # That moves a result by an ulp of f32, which now and then flips the TF32 rounding of an activation
    # (2^-11 relative); over tens of layers these flips add up to about 1e-3 of the output scale.
    assert_tensors_match(per_layer, fused, 1e-3, 1e-3, abs_scaled=True)


@pytest.mark.gpu
def test_full_tower_batch_256():
    from kyanite_b200.executor import CudaExecutor
    g, make_inputs = resnet_tower()
    inputs = make_inputs(256, 3)
    with CudaExecutor(0, g, 256, math_mode=MATH_TF32) as ex:
        fused = ex.evaluate(inputs)
    with CudaExecutor(0, g, 256, math_mode=MATH_TF32, flags=FLAG_NO_CONV_CHAIN) as ex:
        per_layer = ex.evaluate(inputs)
    assert_tensors_match(per_layer, fused, 1e-3, 1e-3, abs_scaled=True)
    expected = cpu_eval_graph(g.to_bytes(), 256, inputs)
    assert_tensors_match(expected, fused, 4e-3, 4e-3, abs_scaled=True)


def tower_with_heads(channels, h, w, c_in, head_channels, head_relu, trunk_output=False, seed=0, computed_filter=False):
    """Stem + one residual block, then one 1x1 convolution (+ bias, optional ReLU) per entry of
    `head_channels`, each flattened and run through a softmax so that other steps sit between them."""
    r = rng(seed)
    g = tower(channels, 1, h, w, c_in, seed=seed)
    cur = g.outputs[0]
    g.outputs.clear()
    for k, relu in zip(head_channels, head_relu):
        wgt = g.constant_tensor((r.standard_normal((k, channels, 1, 1)) * np.sqrt(2.0 / channels)).astype(np.float32))
        if computed_filter:
            wgt = g.mul(wgt, g.view(g.input(shape(1)), shape(1, 1, 1, 1)))
        y = g.add(g.conv(cur, wgt, 1, 1, 0, 0), g.constant_tensor((0.1 * r.standard_normal((1, k, 1, 1))).astype(np.float32)))
        if relu:
            y = g.relu(y)
        g.output(y)
        g.output(g.softmax(g.flatten(y, 1), 1))
    if trunk_output:
        g.output(cur)
    return g


def test_pointwise_heads_join_the_chain():
    g, _ = resnet_tower()
    d = steps(plan_describe(g, 256, MATH_TF32))
    assert "heads=73+32 (trunk result not stored)" in d[0] and not any(" Conv/tc " in l for l in d)
    # a trunk that is also a graph output is stored as well
    d = steps(plan_describe(tower_with_heads(64, 8, 8, 8, [5, 70], [True, False], trunk_output=True), 4, MATH_TF32))
    assert "heads=5+70" in d[0] and "not stored" not in d[0] and not any(" Conv/tc " in l for l in d)
    # 128 accumulator lanes: a head that does not fit stays a step of its own
    d = steps(plan_describe(tower_with_heads(32, 8, 8, 8, [100, 40, 20], [False] * 3), 4, MATH_TF32))
    assert "heads=100+20" in d[0] and len([l for l in d if " Conv/tc " in l and "k=40" in l]) == 1
    # a filter computed at run time cannot be laid out by the planner
    d = steps(plan_describe(tower_with_heads(32, 8, 8, 8, [10], [False], computed_filter=True), 4, MATH_TF32))
    assert "heads=" not in d[0] and len([l for l in d if " Conv/tc " in l and "rs=1x1" in l]) == 1


HEAD_CASES = {
    "policy_value": dict(channels=128, h=8, w=8, c_in=21, head_channels=[73, 32], head_relu=[False, False], batch=8),
    "relu_and_plain": dict(channels=128, h=8, w=8, c_in=16, head_channels=[3, 64, 61], head_relu=[True, False, True], batch=5),
    "trunk_kept": dict(channels=64, h=8, w=8, c_in=8, head_channels=[5, 70], head_relu=[True, False], trunk_output=True, batch=6),
    "narrow_trunk_wide_head": dict(channels=32, h=5, w=7, c_in=32, head_channels=[128], head_relu=[False], batch=9),
    "one_left_out": dict(channels=32, h=8, w=8, c_in=8, head_channels=[100, 40, 20], head_relu=[False, True, False], batch=4),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(HEAD_CASES))
def test_heads_match_oracle_and_separate_kernels(name):
    from kyanite_b200.executor import CudaExecutor
    cfg = dict(HEAD_CASES[name])
    batch = cfg.pop("batch")
    g = tower_with_heads(seed=hash(name) % 1000, **cfg)
    x = rng(6).standard_normal((batch, cfg["c_in"], cfg["h"], cfg["w"])).astype(np.float32)
    assert "heads=" in steps(plan_describe(g, batch, MATH_TF32))[0]
    expected = cpu_eval_graph(g.to_bytes(), batch, [x])
    with CudaExecutor(0, g, batch, math_mode=MATH_TF32) as ex:
        fused = ex.evaluate([x])
        assert_tensors_match(expected, fused, 4e-3, 4e-3, abs_scaled=True)
        for a, b in zip(fused, ex.evaluate([x])):
            np.testing.assert_array_equal(a, b)
    with CudaExecutor(0, g, batch, math_mode=MATH_TF32, flags=FLAG_NO_CONV_CHAIN) as ex:
        # Same operands and rounding points, another summation order: the logits differ by about 1e-3 of their
        # scale (see test_chain_matches_oracle_and_per_layer_kernels), and a softmax turns an absolute logit
        # difference into the same RELATIVE difference of its outputs, so those are held to 2.5e-3.
        assert_tensors_match(ex.evaluate([x]), fused, 2.5e-3, 2.5e-3, abs_scaled=True)
