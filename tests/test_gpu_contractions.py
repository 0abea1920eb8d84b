"""Tensor-core contraction kernels against the CPU oracle on shapes the reference suite does not
reach: tiles with ragged edges, channel tails, boards that are not a power of two, 5x5 filters, split-K
matmuls (partial tiles through the step's scratch buffer), channels-last chains with a residual.
Tolerance for TF32 operands: abs >= 4e-3 * (largest |expected| of the tensor) AND rel >= 4e-3 is a mismatch."""
import numpy as np
import pytest

from kyanite_b200.configs import resnet_tower
from kyanite_b200.executor import MATH_F32, MATH_TF32, CudaExecutor, plan_describe
from kyanite_b200.graph import BATCH, Graph, UnaryOp, shape
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

pytestmark = pytest.mark.gpu


def rng(seed, *s):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal(s).astype(np.float32)


def check(g, batch, ins, mode=MATH_TF32, expect=None):
    blob = g.to_bytes()
    if expect is not None:
        assert expect in plan_describe(blob, batch, math_mode=mode)
    want = cpu_eval_graph(blob, batch, ins)
    with CudaExecutor(0, blob, batch, math_mode=mode) as ex:
        for _ in range(2):
            got = ex.evaluate(ins)
            assert_tensors_match(want, got, tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)


@pytest.mark.parametrize("b,m,n,k", [(1, 256, 128, 64), (1, 128, 16, 32), (3, 200, 72, 100), (1, 1000, 300, 36)])
def test_matmul_tiles(b, m, n, k):
    g = Graph()
    a = g.input(shape(b, m, k))
    w = g.input(shape(b, n, k))
    g.output(g.batched_mat_mul(a, g.permute(w, [0, 2, 1])))
    check(g, 0, [rng(1, b, m, k), rng(2, b, n, k)], expect="Gemm/tc")


@pytest.mark.parametrize("b,m,n,k", [(1, 256, 256, 2048), (1, 128, 64, 4096), (2, 130, 40, 1000), (1, 64, 16, 512)])
def test_matmul_split_k(b, m, n, k):
    g = Graph()
    a = g.input(shape(b, m, k))
    w = g.input(shape(b, n, k))
    bias = g.input(shape(1, 1, n))
    g.output(g.relu(g.add(g.batched_mat_mul(a, g.permute(w, [0, 2, 1])), bias)))
    check(g, 0, [rng(1, b, m, k), rng(2, b, n, k), rng(3, 1, 1, n)], expect="splitk=")


@pytest.mark.parametrize("n,c,h,w,k,r,pad", [(4, 32, 8, 8, 128, 3, 1), (8, 3, 8, 8, 5, 3, 1), (2, 21, 8, 8, 16, 1, 0),
                                              (3, 8, 16, 16, 24, 3, 1), (5, 12, 9, 9, 20, 3, 1), (2, 16, 64, 64, 16, 3, 1),
                                              (2, 4, 8, 8, 8, 5, 2), (3, 130, 8, 8, 136, 3, 1)])
def test_conv_shapes(n, c, h, w, k, r, pad):
    g = Graph()
    x = g.input(shape(n, c, h, w))
    wt = g.constant(shape(k, c, r, r), rng(3, k, c, r, r) * 0.1)
    bias = g.constant(shape(1, k, 1, 1), rng(4, k))
    g.output(g.relu(g.add(g.conv(x, wt, 1, 1, pad, pad), bias)))
    check(g, 0, [rng(5, n, c, h, w)], expect="Conv/tc")


def test_channels_last_chain_with_residual_and_runtime_filter():
    # conv -> conv (+ residual) stays channels-last; the second filter is a graph input, so it is
    # rearranged by a copy step instead of on the host
    g = Graph()
    x = g.input(shape(BATCH, 16, 8, 8))
    w2 = g.input(shape(16, 16, 3, 3))
    w1 = g.constant(shape(16, 16, 3, 3), rng(1, 16, 16, 3, 3) * 0.1)
    b1 = g.constant(shape(1, 16, 1, 1), rng(2, 16))
    y = g.relu(g.add(g.conv(x, w1, 1, 1, 1, 1), b1))
    z = g.relu(g.add(g.conv(y, w2, 1, 1, 1, 1), y))
    g.output_all([z, g.flatten(z, 1)])
    check(g, 5, [rng(3, 5, 16, 8, 8), rng(4, 16, 16, 3, 3) * 0.1], expect="Conv/tc")


@pytest.mark.parametrize("mode,tol", [(MATH_F32, 1e-4), (MATH_TF32, 4e-3)])
def test_full_tower(mode, tol):
    g, make_inputs = resnet_tower()
    ins = make_inputs(16, 7)
    want = cpu_eval_graph(g.to_bytes(), 16, ins)
    with CudaExecutor(0, g, 16, math_mode=mode) as ex:
        got = ex.evaluate(ins)
    assert_tensors_match(want, got, tol_abs=tol, tol_rel=tol)


@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32], ids=["f32", "tf32"])
@pytest.mark.parametrize("b,m,n,k", [(1, 256, 3, 256), (1, 7, 1, 33), (4, 50, 8, 1000), (2, 300, 5, 32), (1, 1, 2, 4096)])
def test_matmul_with_few_columns(b, m, n, k, mode):
    """n <= 8 takes the one-warp-per-row kernel: linear-layer operands (K fast in both), a bias and ReLU,
    and a second graph with the operands transposed the other way (K slow)."""
    g = Graph()
    a = g.input(shape(b, m, k))
    w = g.input(shape(b, n, k))
    bias = g.input(shape(1, 1, n))
    g.output(g.relu(g.add(g.batched_mat_mul(a, g.permute(w, [0, 2, 1])), bias)))
    check(g, 0, [rng(1, b, m, k), rng(2, b, n, k), rng(3, 1, 1, n)], mode=mode)
    g = Graph()
    at = g.input(shape(b, k, m))
    w2 = g.input(shape(b, k, n))
    g.output(g.batched_mat_mul(g.permute(at, [0, 2, 1]), w2))
    check(g, 0, [rng(4, b, k, m), rng(5, b, k, n)], mode=mode)


@pytest.mark.parametrize("b,m,n,k", [(1, 5120, 1024, 128), (3, 300, 200, 100), (1, 130, 20, 40), (2, 256, 272, 64),
                                     (1, 257, 18, 96), (1, 4096, 512, 1536), (1, 256, 256, 2048), (2, 130, 40, 1000)])
def test_persistent_matmul_against_one_tile_kernel(b, m, n, k):
    """Matmuls without split-K run on the persistent kernel (one CTA per SM walking the tile list, two
    accumulators in tensor memory); `FLAG_NO_PERSISTENT_GEMM` selects the one-tile-per-CTA kernel instead.
    Both must match the oracle, with a per-column bias, a full residual addend and ReLU in the epilogue, on
    tile lists longer than the grid (160 tiles of 128 x 256), ragged edges, batches and a row length that
    only the one-tile kernel accepts (n = 18), and split-K shapes (the last two), whose partial tiles either
    kernel writes for the reduction kernel."""
    from kyanite_b200.executor import FLAG_NO_PERSISTENT_GEMM
    g = Graph()
    a = g.input(shape(b, m, k))
    w = g.input(shape(b, n, k))
    bias = g.input(shape(1, 1, n))
    res = g.input(shape(b, m, n))
    g.output(g.relu(g.add(g.add(g.batched_mat_mul(a, g.permute(w, [0, 2, 1])), bias), res)))
    ins = [rng(1, b, m, k), rng(2, b, n, k), rng(3, 1, 1, n), rng(4, b, m, n)]
    blob = g.to_bytes()
    want = cpu_eval_graph(blob, 0, ins)
    got = {}
    for flags in (0, FLAG_NO_PERSISTENT_GEMM):
        with CudaExecutor(0, blob, 0, math_mode=MATH_TF32, flags=flags) as ex:
            for _ in range(2):
                got[flags] = ex.evaluate(ins)
                assert_tensors_match(want, got[flags], tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)
    # same operand rounding and the same order of the K blocks in both kernels
    assert_tensors_match(got[0], got[FLAG_NO_PERSISTENT_GEMM], tol_abs=1e-5, tol_rel=1e-5, abs_scaled=True)


@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32], ids=["f32", "tf32"])
@pytest.mark.parametrize("m,n,k", [(300, 200, 100), (256, 256, 2048), (64, 5, 96), (33, 18, 40)])
def test_matmul_with_gelu_epilogue(m, n, k, mode):
    """bias + exact GELU as the matmul's activation: persistent kernel, split-K reduction, few-column kernel,
    one-tile kernel (n = 18), and the exact-f32 kernels."""
    import math
    from kyanite_b200.executor import FLAG_NO_PERSISTENT_GEMM
    from kyanite_b200.graph import UnaryOp
    g = Graph()
    a = g.input(shape(m, k))
    y = g.add(g.linear(a, g.constant_tensor(rng(2, n, k) * 0.2)), g.constant_tensor(rng(3, 1, n)))
    gate = g.add(g.unary(UnaryOp.ERF, g.mul(y, g.scalar(1.0 / math.sqrt(2.0)))), g.scalar(1.0))
    g.output(g.mul(g.mul(y, g.scalar(0.5)), gate))
    assert " gelu" in plan_describe(g.to_bytes(), 0, math_mode=mode)
    check(g, 0, [rng(1, m, k)], mode=mode)
    blob = g.to_bytes()
    want = cpu_eval_graph(blob, 0, [rng(1, m, k)])
    with CudaExecutor(0, blob, 0, math_mode=mode, flags=FLAG_NO_PERSISTENT_GEMM) as ex:
        assert_tensors_match(want, ex.evaluate([rng(1, m, k)]), tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)


def test_conv_with_gelu_epilogue():
    import math
    from kyanite_b200.graph import UnaryOp
    g = Graph()
    x = g.input(shape(BATCH, 24, 8, 8))
    y = g.add(g.conv(x, g.constant_tensor(rng(1, 40, 24, 3, 3) * 0.1), 1, 1, 1, 1), g.constant_tensor(rng(2, 1, 40, 1, 1)))
    gate = g.add(g.unary(UnaryOp.ERF, g.mul(y, g.scalar(1.0 / math.sqrt(2.0)))), g.scalar(1.0))
    z = g.mul(g.mul(y, g.scalar(0.5)), gate)
    # a second convolution after it: the first one must not become part of a chain that only knows ReLU
    g.output(g.relu(g.conv(z, g.constant_tensor(rng(3, 40, 40, 3, 3) * 0.1), 1, 1, 1, 1)))
    d = plan_describe(g.to_bytes(), 3, math_mode=MATH_TF32)
    assert " gelu" in d and "ConvChain" not in d
    check(g, 3, [rng(4, 3, 24, 8, 8)])


def test_matmul_operands_not_contiguous_along_k():
    """probabilities . values of an attention head: B arrives as [batch, k, n] with n contiguous, and here A
    as [batch, k, m] transposed as well.  The planner copies such operands into K-contiguous buffers and
    keeps the tensor-core kernel (the step list shows the copies and a Gemm/tc step)."""
    b, m, n, k = 8, 512, 128, 260
    g = Graph()
    at = g.input(shape(b, k, m))
    v = g.input(shape(b, k, n))
    g.output(g.batched_mat_mul(g.permute(at, [0, 2, 1]), v))
    d = plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)
    assert d.count(" copy ") == 2 and "Gemm/tc" in d
    check(g, 0, [rng(1, b, k, m), rng(2, b, k, n)])
    # small problems are not worth the extra pass
    g = Graph()
    g.output(g.batched_mat_mul(g.input(shape(2, 64, 32)), g.input(shape(2, 32, 32))))
    assert " copy " not in plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)


@pytest.mark.parametrize("n,c,h,w,k,r,stride,pad", [(16, 64, 32, 32, 64, 3, 2, 1), (32, 36, 33, 31, 48, 3, 2, 1), (32, 256, 16, 16, 256, 1, 2, 0),
                                                     (24, 32, 40, 40, 32, 5, 3, 2), (2, 640, 8, 8, 320, 3, 1, 1), (8, 130, 10, 10, 256, 3, 1, 0)])
def test_conv_as_im2col_matmul(n, c, h, w, k, r, stride, pad):
    """Strided convolutions, and convolutions with few output positions under a long reduction, are planned as
    im2col copies + one batched tensor-core matmul whose B operand (the filter) is shared by the batch.
    Epilogue: bias, a per-(image, channel) addend broadcast over the positions, ReLU."""
    g = Graph()
    x = g.input(shape(n, c, h, w))
    t = g.input(shape(n, k, 1, 1))
    y = g.conv(x, g.constant_tensor(rng(1, k, c, r, r) * 0.05), stride, stride, pad, pad)
    oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    y = g.add(g.add(y, g.constant_tensor(rng(2, 1, k, 1, 1))), g.broadcast(t, shape(n, k, oh, ow)))
    g.output(g.relu(y))
    d = plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)
    # (stride 1 over whole 32-channel blocks: the matmul reads the windows from the image, nothing is materialised)
    assert ("via im2col" in d or "windows read from the image" in d) and "Gemm/tc" in d, d
    check(g, 0, [rng(3, n, c, h, w), rng(4, n, k, 1, 1)])
    # exact-f32 mode keeps the convolution kernel
    d32 = plan_describe(g.to_bytes(), 0, math_mode=MATH_F32)
    assert "via im2col" not in d32 and "windows read from the image" not in d32
    check(g, 0, [rng(3, n, c, h, w), rng(4, n, k, 1, 1)], mode=MATH_F32)


@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32], ids=["f32", "tf32"])
@pytest.mark.parametrize("b,m,n,k", [(1, 1, 1280, 1280), (3, 2, 70, 33), (1, 8, 300, 64), (2, 5, 9, 1000)])
def test_matmul_with_few_rows(b, m, n, k, mode):
    """m <= 8 (one token through a linear layer): the one-warp-per-row kernel on the transposed problem."""
    g = Graph()
    a = g.input(shape(b, m, k))
    w = g.input(shape(b, n, k))
    bias = g.input(shape(1, 1, n))
    res = g.input(shape(b, m, n))
    g.output(g.relu(g.add(g.add(g.batched_mat_mul(a, g.permute(w, [0, 2, 1])), bias), res)))
    check(g, 0, [rng(1, b, m, k), rng(2, b, n, k), rng(3, 1, 1, n), rng(4, b, m, n)], mode=mode)


@pytest.mark.parametrize("n,c,h,w,k,r,stride,pad", [(2, 640, 8, 8, 320, 3, 1, 1), (16, 64, 32, 32, 64, 3, 2, 1), (2, 256, 16, 16, 128, 3, 1, 1),
                                                     (32, 32, 32, 32, 128, 3, 2, 1)])
def test_conv_as_im2col_matmul_with_nchw_result(n, c, h, w, k, r, stride, pad):
    """The graph takes the convolution's result through a flat [N, K*OH*OW] view before a per-element term is
    added, which only a plain NCHW result can serve: the matmul then runs channels x positions with the
    filter as the A operand shared by the batch, and the step may be split along K."""
    oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    g = Graph()
    x = g.input(shape(n, c, h, w))
    y = g.conv(x, g.constant_tensor(rng(1, k, c, r, r) * 0.05), stride, stride, pad, pad)
    v = g.view(y, shape(n, k * oh * ow))
    term = g.constant_tensor(rng(2, 1, k * oh * ow))
    g.output(g.relu(g.add(v, g.broadcast(term, shape(n, k * oh * ow)))))
    d = plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)
    assert ("via im2col" in d or "windows read from the image as operand b" in d) and f"m={k} n={oh * ow}" in d, d
    check(g, 0, [rng(3, n, c, h, w)])


@pytest.mark.parametrize("n,c,h,w,k,chained", [(2, 320, 64, 64, 320, False), (12, 96, 40, 24, 136, False), (4, 256, 32, 32, 256, True)])
def test_pointwise_conv_as_matmul(n, c, h, w, k, chained):
    """1x1 stride-1 convolutions are matmuls over the channels: from an NCHW input through one Im2col step (a
    transpose), from the channels-last result of a previous convolution-as-matmul directly."""
    g = Graph()
    x = g.input(shape(n, c, h, w))
    cur, cin = x, c
    if chained:
        cur = g.relu(g.add(g.conv(x, g.constant_tensor(rng(5, c, c, 1, 1) * 0.1), 1, 1, 0, 0), g.constant_tensor(rng(6, 1, c, 1, 1))))
    y = g.add(g.conv(cur, g.constant_tensor(rng(1, k, cin, 1, 1) * 0.1), 1, 1, 0, 0), g.constant_tensor(rng(2, 1, k, 1, 1)))
    g.output(y)
    d = plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)
    steps = [l.split()[2] for l in d.splitlines() if l.startswith("step")]
    assert steps.count("Gemm/tc") == (2 if chained else 1) and steps.count("Im2col") == 1 and "Conv" not in " ".join(steps), d
    check(g, 0, [rng(3, n, c, h, w)])


def test_head_split_and_k_major_copy_are_one_step():
    """values [B, s, h*d] -> heads [B*h, s, d] needs a copy (the head axis moves in front of the sequence axis),
    and as the B operand of probabilities x values a K-contiguous layout: the planner writes that layout
    straight from the projection's output, one transposing copy instead of two passes."""
    B, s, h, d = 4, 256, 6, 64
    g = Graph()
    probs = g.input(shape(B * h, s, s))
    x = g.input(shape(B, s, h * d))
    v = g.view(g.permute(g.view(x, shape(B, s, h, d)), [0, 2, 1, 3]), shape(B * h, s, d))
    g.output(g.batched_mat_mul(probs, v))
    text = plan_describe(g.to_bytes(), 0, math_mode=MATH_TF32)
    kinds = [l.split()[2] for l in text.splitlines() if l.startswith("step")]
    assert kinds == ["Scalar", "Gemm/tc"], text
    check(g, 0, [rng(1, B * h, s, s) * 0.1, rng(2, B, s, h * d)])


PAIR_CASES = {
    # name: (batch, m, n, k, kwargs): at least 74 tiles of 256 rows, so the planner's matmul runs on CTA pairs
    "projection": (1, 8192, 1024, 512, {}),
    "row_tail": (1, 9000, 1024, 264, {"relu": True}),                 # 9000 = 35 x 256 + 40: the last pair's second CTA is past the end
    "column_tail": (1, 8192, 800, 256, {}),                           # 800 = 4 blocks of 224 > 800 - 3 x 224: clipped stores
    "batched": (3, 4000, 1000, 264, {"residual": True}),
    "gelu": (1, 16384, 768, 768, {"gelu": True}),
    "narrow": (1, 20000, 64, 128, {}),                                # one 64-column block: 32 B rows per CTA
}


def pair_graph(batch, m, n, k, relu=False, gelu=False, residual=False, seed=0):
    r = np.random.Generator(np.random.PCG64(seed))
    g = Graph()
    a = g.input(shape(batch, m, k))
    w = g.constant_tensor((r.standard_normal((1, n, k)) / np.sqrt(k)).astype(np.float32))
    y = g.batched_mat_mul(a, g.permute(g.broadcast(w, shape(batch, n, k)), [0, 2, 1]))
    y = g.add(y, g.constant_tensor(r.standard_normal((1, 1, n)).astype(np.float32)))
    inputs = [r.standard_normal((batch, m, k)).astype(np.float32)]
    if residual:
        y = g.add(y, g.input(shape(batch, m, n)))
        inputs.append(r.standard_normal((batch, m, n)).astype(np.float32))
    if relu:
        y = g.relu(y)
    if gelu:
        half = g.scalar(0.5)
        y = g.mul(g.mul(y, half), g.add(g.scalar(1.0), g.unary(UnaryOp.ERF, g.mul(y, g.scalar(float(np.sqrt(0.5)))))))
    g.output(y)
    return g, inputs


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(PAIR_CASES))
def test_matmul_on_cta_pairs(name, monkeypatch):
    """Large matmuls run on CTA pairs (`cta_group::2`: two SMs on one 256-row tile, each loading half of B).  The same
    instructions in the same K order as the one-CTA kernel: the results are bit-identical to it, and within the TF32
    tolerance of the oracle."""
    batch, m, n, k, kw = PAIR_CASES[name]
    g, inputs = pair_graph(batch, m, n, k, **kw)
    results = {}
    for pair in ("1", "0"):
        monkeypatch.setenv("KN_GEMM_PAIR", pair)
        with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
            results[pair] = ex.evaluate(inputs)[0].copy()
    np.testing.assert_array_equal(results["1"], results["0"])
    expected = cpu_eval_graph(g.to_bytes(), 0, inputs)
    assert_tensors_match(expected, [results["1"]], 4e-3, 4e-3, abs_scaled=True)
