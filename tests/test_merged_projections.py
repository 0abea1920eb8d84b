"""Several projections of one tensor (x . W_i + b_i with constant weights and biases: the query / key / value projections
of an attention block) planned as ONE matmul over the concatenated weights, each projection a column slice of its result
(`try_merged_projections` in plan.cpp).  Which graphs take the route (CPU) and that the results are the oracle's (GPU).
The reference plans one matmul and one bias kernel per projection (kn-cuda-eval/src/planner.rs:300-330)."""
import numpy as np
import pytest

from kyanite_b200.configs import bert_encoder
from kyanite_b200.executor import FLAG_NO_PERSISTENT_GEMM, MATH_F32, MATH_TF32, plan_describe
from kyanite_b200.graph import Graph, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def steps(description):
    return [line for line in description.splitlines() if line.startswith("step")]


def projections_graph(m, k, widths, seed=0, with_bias=True, second_input=False, consume="outputs"):
    """x [m, k] -> x . W_i^T + b_i for every width; `consume`: the projections are outputs, or squared and summed
    (elementwise consumers that read the column slices)."""
    r = rng(seed)
    g = Graph()
    x = g.input(shape(m, k))
    other = g.input(shape(m, k)) if second_input else None
    outs = []
    for i, n in enumerate(widths):
        w = (r.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32)
        src = other if (second_input and i == len(widths) - 1) else x
        y = g.linear(src, g.constant_tensor(w))
        if with_bias:
            y = g.add(y, g.constant_tensor((0.1 * r.standard_normal((1, n))).astype(np.float32)))
        outs.append(y)
    if consume == "outputs":
        for y in outs:
            g.output(y)
    else:
        acc = None
        for y in outs:
            t = g.relu(y) if consume == "relu" else g.mul(y, y)
            acc = t if acc is None else g.add(acc, t)
        g.output(acc)
    return g


def merged(lines):
    return [l for l in lines if "projections of one tensor" in l]


def test_bert_layer_projects_queries_keys_and_values_at_once():
    g, _ = bert_encoder(layers=1)
    lines = steps(plan_describe(g, 32, MATH_TF32))
    one = merged(lines)
    assert len(one) == 1 and "n=2304 k=768" in one[0] and "(3 projections of one tensor)" in one[0], lines
    # with their biases: no elementwise step adds one afterwards (only the embedding sum is left as such a step)
    assert sum(l.split()[2] == "Scalar" for l in lines) == 1, lines
    # the attention step reads the three column slices in place
    assert sum("head split read in place: operands a, b, v" in l for l in lines) == 1
    assert sum(" copy " in l for l in lines) == 0
    for mode, flags in ((MATH_F32, 0), (MATH_TF32, FLAG_NO_PERSISTENT_GEMM)):
        assert not merged(steps(plan_describe(g, 32, mode, flags=flags)))


@pytest.mark.parametrize("case", ["three_equal", "three_different", "two", "consumed_as_slices", "no_bias"])
def test_route(case):
    if case == "no_bias":
        g = projections_graph(2048, 256, [256, 256, 256], with_bias=False)    # (read through views only: nothing to fuse into)
    elif case == "three_equal":
        g = projections_graph(2048, 256, [256, 256, 256])
    elif case == "three_different":
        g = projections_graph(2048, 256, [128, 256, 64])
    elif case == "two":
        g = projections_graph(4096, 128, [256, 256])
    else:
        g = projections_graph(2048, 256, [256, 256, 256], consume="sum")
    lines = steps(plan_describe(g, 0, MATH_TF32))
    assert len(merged(lines)) == 1, lines
    assert sum(l.split()[2].startswith("Gemm") for l in lines) == 1, lines


@pytest.mark.parametrize("case", ["no_bias_into_an_activation", "different_inputs", "one_projection", "few_rows", "no_gain"])
def test_stays_separate(case):
    if case == "no_bias_into_an_activation":
        g = projections_graph(2048, 256, [256, 256, 256], with_bias=False, consume="relu")    # relu is each matmul's epilogue
    elif case == "different_inputs":
        g = projections_graph(2048, 256, [256, 256], second_input=True)
    elif case == "one_projection":
        g = projections_graph(2048, 256, [256])
    elif case == "few_rows":
        g = projections_graph(128, 256, [256, 256, 256])
    else:
        g = projections_graph(65536, 256, [512, 512])    # each matmul fills many rounds of tiles on its own
    assert not merged(steps(plan_describe(g, 0, MATH_TF32)))


@pytest.mark.gpu
@pytest.mark.parametrize("with_bias", [True, False], ids=["bias", "no_bias"])
@pytest.mark.parametrize("consume", ["outputs", "sum"])
@pytest.mark.parametrize("m,k,widths", [(2048, 256, [256, 256, 256]), (2048, 256, [128, 256, 64]), (1000, 96, [32, 100, 64, 36]),
                                        (4096, 128, [256, 256])])
def test_matches_oracle(m, k, widths, consume, with_bias):
    from kyanite_b200.executor import CudaExecutor
    if consume == "sum" and (len(set(widths)) > 1 or not with_bias):
        pytest.skip("the sum needs projections of equal width (and reads the matmuls themselves when there is no bias)")
    g = projections_graph(m, k, widths, seed=5, consume=consume, with_bias=with_bias)
    assert merged(steps(plan_describe(g, 0, MATH_TF32)))
    x = rng(6).standard_normal((m, k)).astype(np.float32)
    expected = cpu_eval_graph(g.to_bytes(), 0, [x])
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate([x])
    assert_tensors_match(expected, got, 2e-3, 2e-3, abs_scaled=True)
    # the separately planned matmuls round the same operands the same way
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        other = ex.evaluate([x])
    assert_tensors_match(other, got, 1e-5, 1e-5, abs_scaled=True)
