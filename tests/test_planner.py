"""Host-only checks of the planner: every reference graph lowers, fusion produces the step counts
the design promises, and the memory plan reuses buffers."""
import re

import pytest

import ref_graphs
from kyanite_b200.configs import mlp, resnet_tower
from kyanite_b200.executor import FLAG_NO_CONV_CHAIN, MATH_F32, MATH_TF32, KnError, plan_describe
from kyanite_b200.graph import BATCH, DType, Graph, shape

CASES = ref_graphs.all_cases()


def steps_of(text):
    return [l for l in text.splitlines() if l.startswith("step ")]


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_lowers(case):
    text = plan_describe(case.graph, case.batch_size)
    assert text.startswith("plan batch=")


def test_conv_bias_res_relu_is_one_step():
    by = {c.name: c for c in CASES}
    assert len(steps_of(plan_describe(by["fuse_res"].graph, 0, MATH_F32))) == 1       # relu(conv + res)
    assert len(steps_of(plan_describe(by["fused_all"].graph, 0, MATH_F32))) == 1      # conv + bias + res
    assert len(steps_of(plan_describe(by["affine_padding"].graph, 0, MATH_F32))) == 2  # pre-add, then conv + bias
    # on the tensor cores the convolution keeps its fused epilogue; the only extra step is the
    # channels-last copy of an input that is not channels-last yet
    tc = steps_of(plan_describe(by["fuse_res"].graph, 0, MATH_TF32))
    assert [s.split()[2] for s in tc] == ["Scalar", "Conv/tc"] and "+1 relu" in tc[1]


def test_mlp_is_three_gemms_and_a_softmax():
    g, _ = mlp()
    kinds = [s.split()[2] for s in steps_of(plan_describe(g, 8))]
    assert kinds == ["Gemm", "Gemm", "Gemm", "Softmax"]   # the reference plans 7 steps here


def test_resnet_tower_step_list():
    g, _ = resnet_tower(channels=16, blocks=2)
    for mode in (MATH_F32, MATH_TF32):
        # (one step per convolution: the merged chain step is covered by tests/test_conv_chain.py)
        kinds = [s.split()[2] for s in steps_of(plan_describe(g, 4, mode, FLAG_NO_CONV_CHAIN))]
        assert sum(k.startswith("Conv") for k in kinds) == 1 + 2 * 2 + 2
        assert sum(k.startswith("Gemm") for k in kinds) == 2
        assert kinds.count("Softmax") == 2
        # f32: nothing but contractions and softmax; tf32: one channels-last copy of the network input,
        # after which activations stay channels-last from convolution to convolution
        assert kinds.count("Scalar") == (0 if mode == MATH_F32 else 1)
    kinds = [s.split()[2] for s in steps_of(plan_describe(g, 4, MATH_TF32, FLAG_NO_CONV_CHAIN))]
    assert kinds.count("Conv/tc") == 7
    kinds = [s.split()[2] for s in steps_of(plan_describe(g, 4, MATH_TF32))]
    # the five 3x3 convolutions and the two 1x1 head convolutions are one chain step
    assert kinds.count("ConvChain/tc") == 1 and kinds.count("Conv/tc") == 0


def test_arena_reuses_buffers():
    g, _ = resnet_tower(channels=16, blocks=6)
    head = plan_describe(g, 8).splitlines()[0]
    arena = int(re.search(r"arena_bytes=(\d+)", head).group(1))
    total = int(re.search(r"hypo_total=(\d+)", head).group(1))
    peak = int(re.search(r"hypo_peak=(\d+)", head).group(1))
    assert peak <= arena < total / 2


def test_softmax_scale_and_layernorm_residual_fold():
    by = {c.name: c for c in CASES}
    text = plan_describe(by["softmax"].graph, 0)
    assert len(steps_of(text)) == 3                       # the scaled softmax needs no separate multiply
    text = plan_describe(by["layernorm_residual_scaled"].graph, 3)
    assert len(steps_of(text)) == 1 and "+res" in text


def test_unsupported_contraction_dtype_is_reported():
    g = Graph()
    a = g.input(shape(1, 2, 2), DType.I32)
    g.output(g.batched_mat_mul(a, a))
    with pytest.raises(KnError) as e:
        plan_describe(g, 0)
    assert e.value.status == 3


def test_deep_chain_plans():
    # thousands of values in one chain: planning must not depend on the caller's stack size
    g = Graph()
    x = g.input(shape(BATCH, 4))
    cur = x
    for i in range(3000):
        cur = g.softmax(g.add(cur, g.scalar(float(i % 3) + 0.5)), 1)
    g.output(cur)
    assert len(steps_of(plan_describe(g, 2))) == 3000     # each add is the softmax's additive term


def test_gelu_folds_into_the_contraction():
    """x * 0.5 * (1 + erf(x / sqrt(2))) after a linear layer or a convolution is the step's activation, in
    either association of the product; a tanh-free variant with another constant is not."""
    import math
    import numpy as np
    from kyanite_b200.graph import Graph, UnaryOp, shape
    rng = np.random.Generator(np.random.PCG64(0))

    def build(form, scale=1.0 / math.sqrt(2.0)):
        g = Graph()
        x = g.input(shape(64, 32))
        y = g.add(g.linear(x, g.constant_tensor(rng.standard_normal((48, 32)).astype(np.float32))),
                  g.constant_tensor(rng.standard_normal((1, 48)).astype(np.float32)))
        gate = g.add(g.unary(UnaryOp.ERF, g.mul(y, g.scalar(scale))), g.scalar(1.0))
        if form == 0:
            out = g.mul(g.mul(y, g.scalar(0.5)), gate)
        elif form == 1:
            out = g.mul(g.scalar(0.5), g.mul(gate, y))
        else:
            out = g.mul(g.mul(y, gate), g.scalar(0.5))
        g.output(out)
        return g

    for form in range(3):
        for mode in (MATH_F32, MATH_TF32):
            s = steps_of(plan_describe(build(form), 0, mode))
            assert len(s) == 1 and " gelu" in s[0], s
    s = steps_of(plan_describe(build(0, scale=0.5), 0, MATH_TF32))
    assert len(s) == 2 and " gelu" not in s[0]
    # the BERT-shaped encoder: no elementwise step is left for the feed-forward activation
    from kyanite_b200.configs import bert_encoder
    g, _ = bert_encoder(layers=1, hidden=64, heads=4, ffn=128, vocab=100, seq=16)
    text = plan_describe(g, 2, MATH_TF32)
    assert sum(" gelu" in l for l in steps_of(text)) == 1
