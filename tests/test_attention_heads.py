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


def test_bert_layer_keeps_no_copy():
    g, _ = bert_encoder(layers=1)
    lines = steps(plan_describe(g, 4, MATH_TF32))
    assert sum("head split read in place: operands a, b, v" in l for l in lines) == 1
    assert sum("head merge read in place: operand a" in l for l in lines) == 1
    # the value matrix is read in place as well (columns contiguous: the MN-major operand of the context MMAs)
    assert sum(" copy " in l for l in lines) == 0
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


# ---------------------------------------------------------------- scores and their softmax in one step
# (kernels/attn_softmax.cu: the scores stay in tensor memory.  The reference runs the matmul, the scaling and the
# softmax as three operations: kn-cuda-eval/src/planner.rs:300-330 and 560-600.)

def scores_graph(b, m, n, k, scale=0.125, seed=0, constant_keys=False, divide=False):
    """softmax(scale * q . keys^T) over the last axis: q [b, m, k] and keys [b, n, k] (K-contiguous, as attention has them)."""
    g = Graph()
    q = g.input(shape(b, m, k))
    if constant_keys:
        keys = g.constant_tensor(rng(seed).standard_normal((b, n, k)).astype(np.float32))
    else:
        keys = g.input(shape(b, n, k))
    scores = g.batched_mat_mul(q, g.permute(keys, [0, 2, 1]))
    if scale is not None:
        scores = g.div(scores, g.scalar(1.0 / scale)) if divide else g.mul(scores, g.scalar(scale))
    g.output(g.softmax(scores, 2))
    return g


def fused_steps(g, mode=MATH_TF32, flags=0):
    return [l for l in steps(plan_describe(g, 0, mode, flags=flags)) if "row softmax" in l]


def test_bert_layer_scores_never_reach_memory():
    g, _ = bert_encoder(layers=1)
    lines = steps(plan_describe(g, 4, MATH_TF32))
    fused = [l for l in lines if " attention " in l]
    assert len(fused) == 1 and "head split read in place: operands a, b, v" in fused[0], lines
    assert "keys=512 k=64 dv=64" in fused[0]
    # neither a softmax step nor a matmul over the probabilities is left
    assert not any("softmax" in l for l in lines), lines
    assert not any("matmul b=48" in l for l in lines), lines
    for mode, flags in ((MATH_F32, 0), (MATH_TF32, FLAG_NO_PERSISTENT_GEMM)):
        other = steps(plan_describe(g, 4, mode, flags=flags))
        assert not any("row softmax" in l or " attention " in l for l in other)


SCORE_SHAPES = {
    # name: (b, m, n, k, scale)
    "one_chunk": (3, 128, 32, 32, 0.2),
    "three_chunks": (2, 256, 96, 64, 0.125),
    "odd_chunk_count_per_group": (2, 128, 160, 64, 0.125),
    "two_halves": (2, 128, 320, 64, 0.125),
    "full_width": (2, 256, 512, 64, 0.125),
    "ragged_rows": (3, 200, 192, 64, 0.125),       # the last row block of an entry is partial
    "long_reduction": (1, 384, 128, 128, 0.09),
    "no_scale": (2, 128, 64, 32, None),
    "more_items_than_ctas": (170, 128, 64, 32, 0.2),   # every CTA walks several items
    "more_items_than_ctas_full_width": (80, 512, 512, 64, 0.125),
}


@pytest.mark.parametrize("name", sorted(SCORE_SHAPES))
def test_scores_route(name):
    b, m, n, k, scale = SCORE_SHAPES[name]
    assert len(fused_steps(scores_graph(b, m, n, k, scale))) == 1
    assert len(fused_steps(scores_graph(b, m, n, k, scale, constant_keys=True))) == 1
    if scale is not None:
        assert len(fused_steps(scores_graph(b, m, n, k, scale, divide=True))) == 1   # scores / sqrt(d), as exported graphs spell it


@pytest.mark.parametrize("case", ["negative_scale", "few_rows", "too_many_keys", "keys_not_a_chunk_multiple", "masked", "softmax_over_rows",
                                  "scores_read_twice"])
def test_scores_stay_two_steps(case):
    b, m, n, k, scale = 2, 128, 128, 64, 0.125
    if case == "negative_scale":
        g = scores_graph(b, m, n, k, -0.125)
    elif case == "few_rows":
        g = scores_graph(b, 64, n, k, scale)
    elif case == "too_many_keys":
        g = scores_graph(b, m, 1024, k, scale)
    elif case == "keys_not_a_chunk_multiple":
        g = scores_graph(b, m, 100, k, scale)
    else:
        g = Graph()
        q, keys = g.input(shape(b, m, k)), g.input(shape(b, n, k))
        scores = g.mul(g.batched_mat_mul(q, g.permute(keys, [0, 2, 1])), g.scalar(scale))
        if case == "masked":
            g.output(g.softmax(g.add(scores, g.input(shape(1, m, n))), 2))
        elif case == "softmax_over_rows":
            g.output(g.softmax(scores, 1))
        else:
            g.output(g.softmax(scores, 2))
            g.output(scores)
    assert fused_steps(g) == []


@pytest.mark.gpu
@pytest.mark.parametrize("constant_keys", [False, True], ids=["input_keys", "constant_keys"])
@pytest.mark.parametrize("name", sorted(SCORE_SHAPES))
def test_scores_match_oracle(name, constant_keys):
    from kyanite_b200.executor import CudaExecutor
    b, m, n, k, scale = SCORE_SHAPES[name]
    g = scores_graph(b, m, n, k, scale, seed=5, constant_keys=constant_keys)
    r = rng(21)
    q = r.standard_normal((b, m, k)).astype(np.float32)
    if scale is None:
        q *= 0.2   # unscaled scores of standard normal operands would make every row one-hot
    inputs = [q] if constant_keys else [q, r.standard_normal((b, n, k)).astype(np.float32)]
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        assert "row softmax" in plan_describe(g, 0, MATH_TF32)
        got = ex.evaluate(inputs)
        again = ex.evaluate(inputs)
    # TF32 operands: a score is off by up to ~1e-2 absolute here, a probability by that relative amount
    assert_tensors_match(expected, got, 2e-2, 2e-2, abs_scaled=True)
    np.testing.assert_allclose(got[0].sum(axis=2), 1.0, rtol=0, atol=1e-5)
    assert np.array_equal(got[0], again[0])
    # the two-step plan rounds the same operands the same way: only the exponential differs (ex2.approx against expf)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        other = ex.evaluate(inputs)
    assert_tensors_match(other, got, 1e-5, 1e-4, abs_scaled=True)


@pytest.mark.gpu
def test_scores_divided_by_a_constant_match_oracle():
    from kyanite_b200.executor import CudaExecutor
    b, m, n, k = 2, 256, 192, 64
    g = scores_graph(b, m, n, k, 0.125, divide=True)
    r = rng(8)
    inputs = [r.standard_normal((b, m, k)).astype(np.float32), r.standard_normal((b, n, k)).astype(np.float32)]
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
    assert_tensors_match(expected, got, 2e-2, 2e-2, abs_scaled=True)


@pytest.mark.gpu
def test_scores_softmax_is_stable_for_large_scores():
    """Rows whose scores are far outside the range of exp: the maximum is subtracted first, as the oracle does."""
    from kyanite_b200.executor import CudaExecutor
    b, m, n, k = 1, 128, 64, 32
    g = scores_graph(b, m, n, k, 1.0)
    r = rng(2)
    q = (30.0 * r.standard_normal((b, m, k))).astype(np.float32)
    keys = (30.0 * r.standard_normal((b, n, k))).astype(np.float32)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate([q, keys])[0]
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got.sum(axis=2), 1.0, rtol=0, atol=1e-5)
    # scores of magnitude ~5000: the winner of a row is the oracle's wherever its margin exceeds the TF32 error
    exact = np.einsum("bmk,bnk->bmn", q.astype(np.float64), keys.astype(np.float64))
    top2 = np.sort(exact, axis=2)[:, :, -2:]
    clear = (top2[:, :, 1] - top2[:, :, 0]) > 50.0
    assert clear.sum() > m // 2
    assert np.array_equal(got.argmax(axis=2)[clear], exact.argmax(axis=2)[clear])


# ---------------------------------------------------------------- scores, softmax and probabilities . V in one step
# (kernels/attention.cu: the probabilities stay in tensor memory as the A operand of the second matmul.)

def context_graph(b, m, n, k, dv, scale=0.125, values_keys_contiguous=True, probabilities_output=False):
    """softmax(scale * q . keys^T) . v: q [b, m, k], keys [b, n, k], v [b, n, dv] (stored as [b, dv, n] if asked)."""
    g = Graph()
    q, keys = g.input(shape(b, m, k)), g.input(shape(b, n, k))
    v = g.permute(g.input(shape(b, dv, n)), [0, 2, 1]) if values_keys_contiguous else g.input(shape(b, n, dv))
    probs = g.softmax(g.mul(g.batched_mat_mul(q, g.permute(keys, [0, 2, 1])), g.scalar(scale)), 2)
    g.output(g.batched_mat_mul(probs, v))
    if probabilities_output:
        g.output(probs)
    return g


CONTEXT_SHAPES = {
    # name: (b, m, n, k, dv)
    "bert_head": (3, 256, 512, 64, 64),
    "narrow_values": (2, 256, 256, 64, 32),
    "narrow_head": (2, 256, 128, 32, 32),
    "one_row_block": (2, 128, 128, 64, 64),
    "keys_only_through_shared_memory": (2, 256, 64, 64, 64),
    "one_chunk_of_keys": (2, 256, 32, 32, 32),
    "three_chunks": (2, 256, 96, 64, 64),
    "ragged_rows": (3, 200, 192, 64, 64),
    "three_row_blocks": (2, 384, 128, 64, 64),
    "long_reduction": (1, 512, 128, 128, 64),
    "more_items_than_ctas": (90, 256, 64, 32, 32),     # every CTA walks several items
    "more_items_than_ctas_full_width": (40, 512, 512, 64, 64),
}


@pytest.mark.parametrize("name", sorted(CONTEXT_SHAPES))
def test_context_route(name):
    b, m, n, k, dv = CONTEXT_SHAPES[name]
    for contiguous in (True, False):
        lines = steps(plan_describe(context_graph(b, m, n, k, dv, values_keys_contiguous=contiguous), 0, MATH_TF32))
        assert sum(" attention " in l for l in lines) == 1 and not any("row softmax" in l for l in lines), lines
        # V is read as it is either way: keys contiguous as a K-major operand, columns contiguous as an MN-major one
        assert sum(" copy " in l for l in lines) == 0, lines


@pytest.mark.parametrize("case", ["wide_values", "values_wider_than_head", "probabilities_read_elsewhere", "few_rows"])
def test_context_stays_a_matmul(case):
    if case == "wide_values":
        g = context_graph(2, 256, 128, 128, 128)
    elif case == "probabilities_read_elsewhere":
        g = context_graph(2, 256, 128, 64, 64, probabilities_output=True)
    elif case == "values_wider_than_head":
        g = context_graph(2, 256, 128, 32, 64)    # V^T takes the place of the keys in shared memory
    else:
        g = context_graph(2, 64, 128, 64, 64)
    lines = steps(plan_describe(g, 0, MATH_TF32))
    assert not any(" attention " in l for l in lines), lines
    if case != "few_rows":
        assert sum("row softmax" in l for l in lines) == 1, lines


@pytest.mark.gpu
@pytest.mark.parametrize("contiguous", [True, False], ids=["keys_contiguous", "columns_contiguous"])
@pytest.mark.parametrize("name", sorted(CONTEXT_SHAPES))
def test_context_matches_oracle(name, contiguous):
    from kyanite_b200.executor import CudaExecutor
    b, m, n, k, dv = CONTEXT_SHAPES[name]
    g = context_graph(b, m, n, k, dv, scale=1.0 / math.sqrt(k), values_keys_contiguous=contiguous)
    r = rng(33)
    inputs = [r.standard_normal((b, m, k)).astype(np.float32), r.standard_normal((b, n, k)).astype(np.float32),
              r.standard_normal((b, dv, n) if contiguous else (b, n, dv)).astype(np.float32)]
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
        again = ex.evaluate(inputs)
    # two chained TF32 contractions: 4e-3 of the largest expected magnitude
    assert_tensors_match(expected, got, 4e-3, 4e-3, abs_scaled=True)
    assert np.array_equal(got[0], again[0])
    # against the same graph planned as separate tensor-core steps (same operand rounding; the probabilities are
    # rounded to TF32 there too, but from their normalised values)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        other = ex.evaluate(inputs)
    assert_tensors_match(other, got, 2e-3, 2e-3, abs_scaled=True)


@pytest.mark.gpu
def test_context_of_one_hot_rows_copies_values():
    """Scores so far apart that every row's softmax is one-hot: the context rows are rows of V (rounded to TF32)."""
    from kyanite_b200.executor import CudaExecutor
    b, m, n, k, dv = 2, 256, 128, 64, 64
    g = context_graph(b, m, n, k, dv, scale=1.0)
    r = rng(4)
    keys = r.standard_normal((b, n, k)).astype(np.float32)
    pick = r.integers(0, n, size=(b, m))
    q = np.stack([40.0 * keys[i][pick[i]] for i in range(b)]).astype(np.float32)
    v = r.standard_normal((b, dv, n)).astype(np.float32)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        got = ex.evaluate([q, keys, v])[0]
    want = np.stack([v[i].T[pick[i]] for i in range(b)])
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-3)


# ---------------------------------------------------------------- seeded random shapes through both attention kernels

def _random_attention_shapes(count, seed):
    r = rng(seed)
    out = []
    while len(out) < count:
        b = int(r.integers(1, 7))
        m = int(r.choice([128, 129, 160, 200, 256, 300, 384, 511, 640]))
        n = 32 * int(r.integers(1, 17))
        k = int(r.choice([32, 64, 96, 128]))
        dv = int(r.choice([32, 64]))
        if (128 + n) * k * 4 + 32768 + 3584 > 227 * 1024:
            continue    # the kernels hold the Q tile and all keys of a head in shared memory
        out.append((b, m, n, k, dv, float(r.choice([0.05, 0.125, 0.3, 1.0])), bool(r.integers(0, 2))))
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("b,m,n,k,dv,scale,keys_contiguous", _random_attention_shapes(24, 77))
def test_random_shapes_match_oracle(b, m, n, k, dv, scale, keys_contiguous):
    """Both kernels on shapes nobody picked: the fused attention step where V fits (dv <= k), else scores + softmax
    followed by a matmul; probabilities as a second output force the scores-only kernel."""
    from kyanite_b200.executor import CudaExecutor
    r = rng(b * 1000003 + m * 1009 + n * 31 + k + dv)
    q = (r.standard_normal((b, m, k)) / math.sqrt(math.sqrt(k))).astype(np.float32)
    keys = (r.standard_normal((b, n, k)) / math.sqrt(math.sqrt(k))).astype(np.float32)
    v = r.standard_normal((b, dv, n) if keys_contiguous else (b, n, dv)).astype(np.float32)
    for probabilities_output in (False, True):
        g = context_graph(b, m, n, k, dv, scale=scale, values_keys_contiguous=keys_contiguous, probabilities_output=probabilities_output)
        lines = steps(plan_describe(g, 0, MATH_TF32))
        fused = any(" attention " in l for l in lines)
        assert fused == (not probabilities_output and dv <= k), lines
        assert fused or any("row softmax" in l for l in lines), lines
        expected = cpu_eval_graph(g.to_bytes(), 0, [q, keys, v])
        with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
            got = ex.evaluate([q, keys, v])
        assert_tensors_match(expected, got, 6e-3, 6e-3, abs_scaled=True)
