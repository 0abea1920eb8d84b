"""F16 storage with f32 accumulation (the storage type of the LLaMA-shaped configuration).  An extension of this
repository's IR: the reference has no half type (kn-graph/src/dtype.rs:25-37) and asserts f32 in matmul, softmax
and layernorm (kn-cuda-eval/src/planner.rs:419,444,608), so there are no reference vectors: PARITY UNPINNED.  The
oracle's semantics (oracle/cpu_eval.py): every f16 value is stored rounded to nearest even, every operation
computes in f32 on the converted operands and rounds once.

Tolerance: the executor rounds at the same points for contractions, softmax, layernorm and single elementwise
operations; inside a fused elementwise kernel it also rounds after every operation.  Sums are formed in another
order than numpy's, so results can differ by one f16 rounding step (2^-11 relative, 4.9e-4) per operation on the
path; comparisons use abs >= tol * max|expected| AND rel >= tol with the tol stated per test."""
import collections

import numpy as np
import pytest

from kyanite_b200 import configs
from kyanite_b200.executor import MATH_F32, MATH_TF32, plan_describe
from kyanite_b200.graph import BATCH, DType, Graph, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def matmul_graph(batch, m, n, k, b_k_major=True):
    g = Graph()
    a = g.input(shape(batch, m, k), DType.F16)
    if b_k_major:
        b = g.permute(g.input(shape(batch, n, k), DType.F16), [0, 2, 1])
    else:
        b = g.input(shape(batch, k, n), DType.F16)
    g.output(g.batched_mat_mul(a, b))
    return g


def matmul_inputs(batch, m, n, k, b_k_major=True, seed=0):
    r = rng(seed)
    a = r.standard_normal((batch, m, k)).astype(np.float16)
    b = r.standard_normal((batch, n, k) if b_k_major else (batch, k, n)).astype(np.float16)
    return [a, b]


def kinds(description):
    return collections.Counter(line.split()[2] for line in description.splitlines() if line.startswith("step"))


def test_oracle_rounds_once_per_operation():
    r = rng(1)
    a = r.standard_normal((1, 8, 300)).astype(np.float16)
    b = r.standard_normal((1, 300, 5)).astype(np.float16)
    g = Graph()
    g.output(g.batched_mat_mul(g.input(shape(1, 8, 300), DType.F16), g.input(shape(1, 300, 5), DType.F16)))
    (got,) = cpu_eval_graph(g.to_bytes(), 1, [a, b])
    exact = a.astype(np.float64) @ b.astype(np.float64)
    assert got.dtype == np.float16
    # f32 accumulation then ONE rounding: within half an f16 step of the exact product (plus f32 summation noise)
    assert np.all(np.abs(got.astype(np.float64) - exact) <= np.abs(exact) * 2.0 ** -11 + 1e-3)
    # elementwise: sigmoid computed in f32, rounded once
    g = Graph()
    g.output(g.sigmoid(g.input(shape(64), DType.F16)))
    x = r.standard_normal(64).astype(np.float16)
    (s,) = cpu_eval_graph(g.to_bytes(), 1, [x])
    np.testing.assert_array_equal(s, (1.0 / (1.0 + np.exp(-x.astype(np.float32)))).astype(np.float16))


def test_planner_uses_tensor_cores_for_f16_matmul():
    d = plan_describe(matmul_graph(1, 256, 512, 1024), 0, MATH_TF32)
    assert kinds(d)["Gemm/tc"] == 1 and " f16" in d
    # few tiles, long K: split along K
    assert "splitk=" in plan_describe(matmul_graph(1, 128, 256, 8192), 0, MATH_TF32)
    # exact-f32 mode keeps f16 matmuls off the tensor cores as well
    assert kinds(plan_describe(matmul_graph(1, 256, 512, 1024), 0, MATH_F32))["Gemm"] == 1
    # an operand that is not K-contiguous gets a K-contiguous copy when the problem is large
    d = plan_describe(matmul_graph(4, 512, 256, 512, b_k_major=False), 0, MATH_TF32)
    assert kinds(d)["Gemm/tc"] == 1 and kinds(d)["Scalar"] == 1


def test_llama_f16_lowers_and_oracle_is_close_to_f32():
    kw = dict(layers=2, d_model=64, heads=4, ffn=96, vocab=100, seq=16)
    g16, make_inputs = configs.llama_decoder(dtype=DType.F16, **kw)
    g32, _ = configs.llama_decoder(**kw)
    ids = make_inputs(2, 1)
    (h,) = cpu_eval_graph(g16.to_bytes(), 2, ids)
    (f,) = cpu_eval_graph(g32.to_bytes(), 2, ids)
    assert h.dtype == np.float16
    assert np.max(np.abs(h.astype(np.float32) - f)) <= 4e-3 * np.max(np.abs(f))
    for mode in (MATH_TF32, MATH_F32):
        assert sum(kinds(plan_describe(g16, 2, mode)).values()) > 0
    # every RMS norm (two per layer and the final one) is ONE step, in the f16 graph (casts around it) and the f32 one:
    # no reduce step and no elementwise step of the pow / mean / sqrt / div / mul subgraph is left
    for g in (g16, g32):
        k = kinds(plan_describe(g, 2, MATH_TF32))
        assert k["RmsNorm"] == 2 * kw["layers"] + 1 and k["Reduce"] == 0, k


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [DType.F16, DType.F32], ids=["f16", "f32"])
@pytest.mark.parametrize("rows,length,with_gain", [(64, 4096, True), (5, 64, False), (3, 16384, True), (7, 100, True)])
def test_rmsnorm_subgraph_matches_oracle(rows, length, with_gain, dtype):
    """The pow / mean / sqrt / div (/ mul) subgraph decoder graphs spell an RMS norm with: fused into one step when
    the row length is a multiple of 8 (at most 16384), planned node by node otherwise; both must agree with the oracle."""
    from kyanite_b200.executor import CudaExecutor
    from kyanite_b200.graph import BinaryOp, ReduceOp, UnaryOp
    r = rng(rows * length)
    g = Graph()
    x = g.input(shape(rows, length), dtype)
    t = g.value_cast(x, DType.F32) if dtype == DType.F16 else x
    ms = g.view(g.reduce(g.pow(t, g.scalar(2.0)), [1], ReduceOp.MEAN), shape(rows, 1))
    y = g.binary(BinaryOp.DIV, t, g.unary(UnaryOp.SQRT, g.add(ms, g.scalar(1e-6))))
    if with_gain:
        y = g.mul(y, g.constant_tensor((1 + 0.1 * r.standard_normal((1, length))).astype(np.float32)))
    g.output(g.value_cast(y, DType.F16) if dtype == DType.F16 else y)
    ins = [(r.standard_normal((rows, length)) * 2).astype(dtype.np)]
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    k = kinds(plan_describe(g, 0))
    assert (k["RmsNorm"] == 1 and len(k) == 1) if length % 8 == 0 else k["RmsNorm"] == 0
    tol = 2e-3 if dtype == DType.F16 else 1e-4
    with CudaExecutor(0, g, 0) as ex:
        assert_tensors_match(expected, ex.evaluate(ins), tol, tol, abs_scaled=True)


# ------------------------------------------------------------------------------------------------ GPU
MATMUL_CASES = {
    # name: (batch, m, n, k, b_k_major)
    "square": (1, 256, 256, 256, True),
    "ragged_m_and_k_tail": (1, 200, 192, 1000, True),
    "wide_n_two_column_blocks": (1, 128, 320, 512, True),
    "batched_scores": (6, 256, 128, 64, True),
    "split_k": (1, 128, 256, 8192, True),
    "b_needs_a_copy": (4, 512, 256, 512, False),
    "small_falls_back_to_simt": (2, 17, 9, 33, True),
    "n_not_multiple_of_8": (1, 256, 100, 256, True),
}


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [MATH_TF32, MATH_F32], ids=["tensor_cores", "simt"])
@pytest.mark.parametrize("name", list(MATMUL_CASES))
def test_f16_matmul_matches_oracle(name, mode):
    from kyanite_b200.executor import CudaExecutor
    batch, m, n, k, b_k_major = MATMUL_CASES[name]
    g = matmul_graph(batch, m, n, k, b_k_major)
    ins = matmul_inputs(batch, m, n, k, b_k_major, seed=len(name))
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    with CudaExecutor(0, g, 0, math_mode=mode) as ex:
        for _ in range(2):
            got = ex.evaluate(ins)
            assert got[0].dtype == np.float16
            # one f16 rounding of an f32-accumulated sum on both sides; the sums differ in order only
            assert_tensors_match(expected, got, 1e-3, 1e-3, abs_scaled=True)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,length,with_mask", [(64, 2048, True), (8, 16384, False), (33, 40, True), (5, 20000, False),
                                                   (300, 128, False)])
def test_f16_softmax_matches_oracle(rows, length, with_mask):
    from kyanite_b200.executor import CudaExecutor
    r = rng(rows + length)
    g = Graph()
    x = g.input(shape(2, rows, length), DType.F16)
    t = g.mul(x, g.scalar(0.125, DType.F16))
    ins = [(r.standard_normal((2, rows, length)) * 4).astype(np.float16)]
    if with_mask:
        mask = np.triu(np.full((rows, length), -np.inf, np.float16), 1).reshape(1, rows, length)
        t = g.add(t, g.constant_tensor(mask))
    g.output(g.softmax(t, 2))
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    assert kinds(plan_describe(g, 0)) == {"Softmax": 1}       # scale and mask are applied as the row is loaded
    with CudaExecutor(0, g, 0) as ex:
        # the oracle rounds scale * x (and + mask) to f16 before the softmax, the kernel does not: one rounding step
        assert_tensors_match(expected, ex.evaluate(ins), 4e-3, 4e-3, abs_scaled=True)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,length", [(64, 4096), (7, 100), (3, 30000)])
def test_f16_layernorm_matches_oracle(rows, length):
    from kyanite_b200.executor import CudaExecutor
    r = rng(rows + length)
    g = Graph()
    g.output(g.layernorm(g.input(shape(rows, length), DType.F16), 1, 1e-5))
    ins = [(r.standard_normal((rows, length)) * 3 + 1).astype(np.float16)]
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    with CudaExecutor(0, g, 0) as ex:
        assert_tensors_match(expected, ex.evaluate(ins), 2e-3, 2e-3, abs_scaled=True)


LLAMA_F16 = {
    "tiny": (dict(layers=2, d_model=64, heads=4, ffn=96, vocab=100, seq=16), 2),
    "tensor_core_sized": (dict(layers=2, d_model=256, heads=4, ffn=512, vocab=512, seq=128), 1),
}


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [MATH_TF32, MATH_F32], ids=["tensor_cores", "simt"])
@pytest.mark.parametrize("name", list(LLAMA_F16))
def test_llama_f16_matches_oracle(name, mode):
    from kyanite_b200.executor import CudaExecutor
    kw, batch = LLAMA_F16[name]
    g, make_inputs = configs.llama_decoder(dtype=DType.F16, **kw)
    ids = make_inputs(batch, 3)
    expected = cpu_eval_graph(g.to_bytes(), batch, ids)
    if name == "tensor_core_sized" and mode == MATH_TF32:
        assert kinds(plan_describe(g, batch, mode))["Gemm/tc"] >= 10
    with CudaExecutor(0, g, batch, math_mode=mode) as ex:
        for _ in range(2):
            # two decoder layers: about 30 f16 roundings on the path of a logit; tolerance 1e-2 of the logits' scale
            assert_tensors_match(expected, ex.evaluate(ids), 1e-2, 1e-2, abs_scaled=True)


def elementwise_f16_graph(kind, rows, cols, broadcast_row=False):
    """One fused elementwise step over f16 operands: `kind` picks the expression."""
    from kyanite_b200.graph import BinaryOp, UnaryOp
    g = Graph()
    a = g.input(shape(rows, cols), DType.F16)
    b = g.input(shape(1, cols) if broadcast_row else shape(rows, cols), DType.F16)
    if broadcast_row:
        b = g.broadcast(b, shape(rows, cols))
    if kind == "add":
        y = g.add(a, b)
    elif kind == "sub_mul":
        y = g.mul(g.sub(a, b), b)
    elif kind == "min_max":
        y = g.binary(BinaryOp.MAX, g.binary(BinaryOp.MIN, a, b), g.unary(UnaryOp.NEG, b))
    elif kind == "rope_like":      # a * b + (-a) * b': two products and a sum, as the rotary embedding step
        c = g.input(shape(rows, cols), DType.F16)
        y = g.add(g.mul(a, b), g.mul(g.unary(UnaryOp.NEG, c), b))
    elif kind == "swiglu":
        y = g.mul(g.mul(g.unary(UnaryOp.SIGMOID, a), a), b)
    else:                          # "div_abs"
        y = g.binary(BinaryOp.DIV, g.unary(UnaryOp.ABS, a), g.add(g.unary(UnaryOp.ABS, b), g.scalar(1.0, DType.F16)))
    g.output(y)
    return g


def test_f16_elementwise_programs_run_on_packed_halves():
    for kind in ("add", "sub_mul", "min_max", "rope_like", "swiglu", "div_abs"):
        d = plan_describe(elementwise_f16_graph(kind, 64, 256), 0)
        assert " half2" in d, (kind, d)
    # a cast inside the program keeps the f32 route
    g = Graph()
    a = g.input(shape(64, 256), DType.F16)
    b = g.input(shape(64, 256), DType.F32)
    g.output(g.add(g.value_cast(a, DType.F32), b))
    assert " half2" not in plan_describe(g, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("broadcast_row", [False, True], ids=["full", "row_broadcast"])
@pytest.mark.parametrize("kind", ["add", "sub_mul", "min_max", "rope_like"])
def test_f16_packed_arithmetic_is_bit_exact(kind, broadcast_row):
    """add / sub / mul / min / max on packed halves: an IEEE half operation rounds the exact result once; the oracle
    computes in f32 and rounds to f16, and that double rounding is innocuous for these operations (24 >= 2 * 11 + 2
    significand bits).  So the comparison is exact, over values that include subnormals, large magnitudes and
    operands of very different exponents."""
    from kyanite_b200.executor import CudaExecutor
    rows, cols = 67, 1000 if kind != "rope_like" else 1024
    cols -= cols % 8
    r = rng(21)

    def halves(shape_):
        x = r.standard_normal(shape_) * np.exp2(r.integers(-20, 12, shape_))
        return x.astype(np.float16)

    inputs = [halves((rows, cols)), halves((1, cols) if broadcast_row else (rows, cols))]
    if kind == "rope_like":
        inputs.append(halves((rows, cols)))
    g = elementwise_f16_graph(kind, rows, cols, broadcast_row)
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)[0]
    with CudaExecutor(0, g, 0) as ex:
        got = ex.evaluate(inputs)[0]
    finite = np.isfinite(expected.astype(np.float32))
    # (the sign of a zero that min / max pick between +0 and -0 is not defined: both zeros count as equal)
    both_zero = (got == 0) & (expected == 0)
    different = (got.view(np.uint16) != expected.view(np.uint16)) & finite & ~both_zero
    assert not different.any(), (int(different.sum()), got[different][:4], expected[different][:4])
    np.testing.assert_array_equal(np.isnan(got.astype(np.float32)), np.isnan(expected.astype(np.float32)))


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["swiglu", "div_abs"])
def test_f16_packed_programs_with_f32_steps_match_oracle(kind):
    """Sigmoid, division: converted, computed in f32 (hardware exponential and reciprocal for the sigmoid) and rounded
    once: within one f16 rounding step of the oracle (tolerance 1e-3 of the tensor's scale)."""
    from kyanite_b200.executor import CudaExecutor
    rows, cols = 40, 2048
    r = rng(5)
    inputs = [r.standard_normal((rows, cols)).astype(np.float16) * np.float16(3), r.standard_normal((rows, cols)).astype(np.float16)]
    g = elementwise_f16_graph(kind, rows, cols)
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    with CudaExecutor(0, g, 0) as ex:
        got = ex.evaluate(inputs)
    assert_tensors_match(expected, got, 1e-3, 1e-3, abs_scaled=True)
