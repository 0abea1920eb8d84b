"""Attention head split / merge read in place by the matmuls (GemmOperand4D, kernels/gemm_persistent.cu): the
view - permute - view chains around the attention matmuls cost no copy of the activations when the tensor cores are
used.  Which graphs take the route (CPU) and that the results are the oracle's (GPU).  The reference plans these
chains node by node: a permute is a stride edit, the view after it materialises a copy
(kn-cuda-eval/src/planner.rs:345-357)."""
import math

import numpy as np
import pytest

from kyanite_b200.configs import _attention, bert_encoder
from kyanite_b200.executor import FLAG_NO_PERSISTENT_GEMM, MATH_F32, MATH_TF32, plan_describe
from kyanite_b200.graph import Graph, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def attention_graph(b, s, h, d, seed=0, project=True):
    """q, k, v [b*s, h*d] -> attention over h heads -> (optionally) an output projection with bias."""
    r = rng(seed)
    g = Graph()
    q, k, v = (g.input(shape(b * s, h * d)) for _ in range(3))
    ctx = _attention(g, q, k, v, s, s, h, d, b)
    if project:
        w = (r.standard_normal((1, h * d, h * d)) / math.sqrt(h * d)).astype(np.float32)     # [1, out, in]: K-contiguous
        bias = (0.1 * r.standard_normal((1, 1, h * d))).astype(np.float32)
        ctx = g.add(g.batched_mat_mul(g.view(ctx, shape(1, b * s, h * d)), g.permute(g.constant_tensor(w), [0, 2, 1])),
                    g.constant_tensor(bias))
    g.output(ctx)
    return g


def steps(description):
    return [line for line in description.splitlines() if line.startswith("step")]


def test_bert_layer_keeps_one_copy():
    g, _ = bert_encoder(layers=1)
    lines = steps(plan_describe(g, 4, MATH_TF32))
    assert sum("head split read in place: operands a, b" in l for l in lines) == 1
    assert sum("head merge read in place: operand a" in l for l in lines) == 1
    # what is left is the value matrix made K-contiguous: split and transposition in one copy
    assert sum(" copy " in l for l in lines) == 1
    # exact f32, or the persistent kernel switched off: the chains are copies as before
    assert not any("read in place" in l for l in steps(plan_describe(g, 4, MATH_F32)))
    assert not any("read in place" in l for l in steps(plan_describe(g, 4, MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM)))


CASES = {
    # name: (b, s, h, d, split folded, merge folded)
    "bert_like": (2, 128, 4, 64, True, True),
    "narrow_heads": (3, 256, 2, 32, True, True),
    "wide_heads": (1, 128, 8, 128, True, True),
    "rows_not_a_tile_multiple": (2, 192, 4, 64, True, False),   # 192 % 128 != 0: a tile of the merge would straddle two entries
    "head_dim_not_a_k_block": (2, 128, 3, 24, True, False),     # 24 % 32 != 0: a K block of the merge would straddle two heads
    "short_sequence": (4, 64, 4, 64, True, False),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_routes(name):
    b, s, h, d, split, merge = CASES[name]
    lines = steps(plan_describe(attention_graph(b, s, h, d), 0, MATH_TF32))
    assert any("head split read in place" in l for l in lines) == split, lines
    assert any("head merge read in place" in l for l in lines) == merge, lines


@pytest.mark.gpu
@pytest.mark.parametrize("project", [True, False], ids=["projected", "context_only"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_matches_oracle(name, project):
    from kyanite_b200.executor import CudaExecutor
    b, s, h, d, _, _ = CASES[name]
    g = attention_graph(b, s, h, d, seed=3, project=project)
    r = rng(9)
    inputs = [r.standard_normal((b * s, h * d)).astype(np.float32) for _ in range(3)]
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
    # three chained TF32 contractions (scores, context, projection): 4e-3 of the largest expected magnitude
    assert_tensors_match(expected, got, 4e-3, 4e-3, abs_scaled=True)
    # and the same graph with materialised operands computes the same values up to TF32 rounding of the same operands
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        other = ex.evaluate(inputs)
    assert_tensors_match(other, got, 2e-3, 2e-3, abs_scaled=True)
