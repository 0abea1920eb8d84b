"""ONNX loader (kyanite_b200/onnx.py) and the golden models of the reference's test-suite
(kn-cuda-eval/tests/root/onnx.rs: simple, simple_bn, pre, att_tiny).

The golden outputs come from the framework the models were trained in; they pin the oracle (CPU test) and
the CUDA executor (GPU test) end to end: convolution, batch-norm, clip, residual add, Gemm, softmax,
attention built from MatMul / Transpose / Reshape, and the shape arithmetic around them."""
import os

import numpy as np
import pytest

import onnx_writer as ow
from kyanite_b200.graph import BATCH, DType, OpKind, Size
from kyanite_b200.onnx import SUPPORTED_OPS, OnnxError, load_graph_from_onnx_bytes, load_graph_from_onnx_path
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ["simple-sttt-1x64", "simple-bn-sttt-1x64", "pre-sttt-4x8", "att-tiny"]
# a checkout of the reference project, if there is one: KN_REFERENCE_DIR (tests that need it skip without it)
REFERENCE_DATA = os.path.join(os.environ.get("KN_REFERENCE_DIR", os.path.join(os.sep, "root", "reference")), "kn-cuda-eval", "tests", "data")


def load_golden(name):
    with open(os.path.join(GOLDEN, name + ".kng"), "rb") as f:
        blob = f.read()
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    inputs = [z[k] for k in sorted(k for k in z.files if k.startswith("input"))]
    outputs = [z[k] for k in sorted(k for k in z.files if k.startswith("output"))]
    return blob, int(z["batch"]), inputs, outputs


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_golden_outputs(name):
    blob, batch, inputs, expected = load_golden(name)
    # the reference's own rule for these files (tester.rs:151-154 with TOLERANCE 1e-3)
    assert_tensors_match(expected, cpu_eval_graph(blob, batch, inputs), 1e-3, 1e-3)


@pytest.mark.skipif(not os.path.isdir(REFERENCE_DATA), reason="needs the reference checkout")
@pytest.mark.parametrize("name", NAMES)
def test_loader_reproduces_committed_graph(name):
    graph = load_graph_from_onnx_path(os.path.join(REFERENCE_DATA, name + ".onnx"))
    blob, _, _, _ = load_golden(name)
    assert graph.to_bytes() == blob


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("mode", ["f32", "tf32"])
def test_executor_matches_golden_outputs(name, mode):
    from kyanite_b200.executor import MATH_F32, MATH_TF32, CudaDevice, CudaExecutor
    blob, batch, inputs, expected = load_golden(name)
    ex = CudaExecutor(CudaDevice(0), blob, batch, math_mode=MATH_F32 if mode == "f32" else MATH_TF32)
    for _ in range(2):
        actual = ex.evaluate(inputs)
        if mode == "f32":
            assert_tensors_match(expected, actual, 1e-3, 1e-3)
        else:
            assert_tensors_match(expected, actual, 4e-3, 4e-3, abs_scaled=True)


# --------------------------------------------------------------------------------------
# hand-written models
# --------------------------------------------------------------------------------------
def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def run(model_bytes, batch, inputs, **kwargs):
    graph = load_graph_from_onnx_bytes(model_bytes, **kwargs)
    return graph, cpu_eval_graph(graph.to_bytes(), batch, inputs)


def test_conv_bn_relu_gemm_softmax():
    r = rng(1)
    w = r.standard_normal((4, 3, 3, 3)).astype(np.float32)
    b = r.standard_normal(4).astype(np.float32)
    scale, bias, mean = (r.standard_normal(4).astype(np.float32) for _ in range(3))
    var = r.random(4).astype(np.float32) + 0.5
    fc = r.standard_normal((5, 4 * 6 * 6)).astype(np.float32)
    fcb = r.standard_normal(5).astype(np.float32)
    m = ow.model(
        [ow.node("Conv", ["x", "w", "b"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1],
                 dilations=[1, 1], group=1),
         ow.node("BatchNormalization", ["c", "scale", "bias", "mean", "var"], ["n"], epsilon=1e-5, momentum=0.9),
         ow.node("Relu", ["n"], ["r"]),
         ow.node("Flatten", ["r"], ["f"], axis=1),
         ow.node("Gemm", ["f", "fc", "fcb"], ["l"], alpha=1.0, beta=1.0, transB=1),
         ow.node("Softmax", ["l"], ["y"], axis=1)],
        [ow.tensor("w", w), ow.tensor("b", b), ow.tensor("scale", scale), ow.tensor("bias", bias),
         ow.tensor("mean", mean, typed_fields=True), ow.tensor("var", var), ow.tensor("fc", fc), ow.tensor("fcb", fcb)],
        [ow.value_info("x", ["batch_size", 3, 6, 6])], [ow.value_info("y", ["batch_size", 5])])
    x = r.standard_normal((2, 3, 6, 6)).astype(np.float32)
    graph, (y,) = run(m, 2, [x])
    assert graph[graph.outputs[0]].shape == (BATCH, Size(5))

    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (1, 1), (1, 1)))
    conv = np.zeros((2, 4, 6, 6))
    for dy in range(3):
        for dx in range(3):
            conv += np.einsum("nchw,kc->nkhw", xp[:, :, dy:dy + 6, dx:dx + 6], w[:, :, dy, dx].astype(np.float64))
    conv += b.reshape(1, 4, 1, 1)
    n = (conv - mean.reshape(1, 4, 1, 1)) / np.sqrt(var.reshape(1, 4, 1, 1) + np.float32(1e-5)) * scale.reshape(1, 4, 1, 1) \
        + bias.reshape(1, 4, 1, 1)
    logits = np.maximum(n, 0).reshape(2, -1) @ fc.T.astype(np.float64) + fcb
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    assert_tensors_match([(e / e.sum(axis=1, keepdims=True)).astype(np.float32)], [y], 1e-4, 1e-4)


def test_shape_arithmetic_never_reaches_the_graph():
    """Shape -> Gather -> Unsqueeze -> Concat -> Reshape, the pattern exporters emit for `x.view(B, -1)`,
    plus Mul/Div on sizes where the batch size cancels out again."""
    i64 = np.int64
    m = ow.model(
        [ow.node("Shape", ["x"], ["s"]),
         ow.node("Constant", [], ["zero"], value=np.array(0, dtype=i64)),
         ow.node("Gather", ["s", "zero"], ["b"], axis=0),
         ow.node("Unsqueeze", ["b"], ["b1"], axes=[0]),
         ow.node("Constant", [], ["minus"], value=np.array([-1], dtype=i64)),
         ow.node("Concat", ["b1", "minus"], ["target"], axis=0),
         ow.node("Reshape", ["x", "target"], ["flat"]),
         # (B * 6) / B == 6: a batch-free size again, so it is stored as a plain constant
         ow.node("Constant", [], ["six"], value=np.array(6, dtype=i64)),
         ow.node("Mul", ["b", "six"], ["b6"]),
         ow.node("Div", ["b6", "b"], ["plain"]),
         ow.node("Unsqueeze", ["plain"], ["plain1"], axes=[0]),
         ow.node("Constant", [], ["two"], value=np.array([2], dtype=i64)),
         ow.node("Concat", ["b1", "two", "plain1"], ["target2"], axis=0),
         ow.node("Reshape", ["flat", "target2"], ["y"])],
        [], [ow.value_info("x", ["batch_size", 3, 4])], [ow.value_info("y", ["batch_size", 2, 6])], opset=11)
    x = rng(2).standard_normal((5, 3, 4)).astype(np.float32)
    graph, (y,) = run(m, 5, [x])
    np.testing.assert_array_equal(y, x.reshape(5, 2, 6))
    assert graph[graph.outputs[0]].shape == (BATCH, Size(2), Size(6))
    kinds = {graph.values[i].kind for i in range(len(graph.values))}
    assert kinds <= {OpKind.INPUT, OpKind.VIEW, OpKind.CONSTANT}       # no gather / concat on shapes


def test_slice_split_pad_reduce_transpose():
    i64 = np.int64
    m = ow.model(
        [ow.node("Slice", ["x", "starts", "ends", "axes", "steps"], ["s"]),                # x[:, 1:-1:2, :]
         ow.node("Slice", ["s", "fs", "fe", "fa", "fstep"], ["flipped"]),                  # reverse last axis
         ow.node("Split", ["flipped"], ["lo", "hi"], axis=2),
         ow.node("Transpose", ["hi"], ["t"], perm=[0, 2, 1]),
         ow.node("Pad", ["lo", "pads", "padv"], ["p"], mode="constant"),
         ow.node("ReduceMean", ["p"], ["mean"], axes=[-1], keepdims=0),
         ow.node("ReduceMax", ["x"], ["mx"], axes=[1, 2], keepdims=1)],
        [ow.tensor("starts", np.array([1], i64)), ow.tensor("ends", np.array([-1], i64)),
         ow.tensor("axes", np.array([1], i64)), ow.tensor("steps", np.array([2], i64)),
         ow.tensor("fs", np.array([-1], i64)), ow.tensor("fe", np.array([-(1 << 63)], i64)),
         ow.tensor("fa", np.array([2], i64)), ow.tensor("fstep", np.array([-1], i64)),
         ow.tensor("pads", np.array([0, 0, 1, 0, 0, 2], i64)), ow.tensor("padv", np.array(0.5, np.float32))],
        [ow.value_info("x", ["batch_size", 6, 5])],
        [ow.value_info("t", ["batch_size", 2, 2]), ow.value_info("mean", ["batch_size", 2]),
         ow.value_info("mx", ["batch_size", 1, 1])])
    x = rng(3).standard_normal((3, 6, 5)).astype(np.float32)
    _, (t, mean, mx) = run(m, 3, [x])
    s = x[:, 1:-1:2, :][:, :, ::-1]
    lo, hi = s[:, :, :3], s[:, :, 3:]
    np.testing.assert_array_equal(t, hi.transpose(0, 2, 1))
    p = np.pad(lo, ((0, 0), (0, 0), (1, 2)), constant_values=0.5)
    assert_tensors_match([p.mean(axis=-1)], [mean], 1e-6, 1e-6)
    np.testing.assert_array_equal(mx, x.max(axis=(1, 2), keepdims=True))


def test_pool_resize_layernorm_einsum_clip():
    r = rng(4)
    gamma, beta = r.standard_normal(8).astype(np.float32), r.standard_normal(8).astype(np.float32)
    m = ow.model(
        [ow.node("MaxPool", ["x"], ["mp"], kernel_shape=[2, 2], strides=[2, 2], pads=[0, 0, 0, 0]),
         ow.node("Resize", ["mp", "", "scales"], ["up"], mode="nearest", nearest_mode="floor", cubic_coeff_a=-0.75,
                 coordinate_transformation_mode="asymmetric"),
         ow.node("GlobalAveragePool", ["up"], ["gap"]),
         ow.node("LayerNormalization", ["seq", "gamma", "beta"], ["ln"], axis=-1, epsilon=1e-5),
         ow.node("Einsum", ["ln", "ln"], ["scores"], equation="bid, bjd -> bij"),
         ow.node("Clip", ["scores", "lo", "hi"], ["clipped"])],
        [ow.tensor("scales", np.array([1, 1, 2, 2], np.float32)), ow.tensor("gamma", gamma), ow.tensor("beta", beta),
         ow.tensor("lo", np.array(-1.0, np.float32)), ow.tensor("hi", np.array(2.0, np.float32))],
        [ow.value_info("x", ["batch_size", 2, 5, 4]), ow.value_info("seq", ["batch_size", 3, 8])],
        [ow.value_info("up", ["batch_size", 2, 4, 4]), ow.value_info("gap", ["batch_size", 2]),
         ow.value_info("clipped", ["batch_size", 3, 3])], opset=17)
    x = r.standard_normal((2, 2, 5, 4)).astype(np.float32)
    seq = r.standard_normal((2, 3, 8)).astype(np.float32)
    _, (up, gap, clipped) = run(m, 2, [x, seq])
    mp = x[:, :, :4, :].reshape(2, 2, 2, 2, 2, 2).max(axis=(3, 5))       # floor mode drops the odd row
    up_ref = mp.repeat(2, axis=2).repeat(2, axis=3)
    np.testing.assert_array_equal(up, up_ref)
    assert_tensors_match([up_ref.mean(axis=(2, 3))], [gap], 1e-6, 1e-6)
    mu = seq.mean(-1, keepdims=True)
    ln = (seq - mu) / np.sqrt(((seq - mu) ** 2).mean(-1, keepdims=True) + 1e-5) * gamma + beta
    assert_tensors_match([np.clip(ln @ ln.transpose(0, 2, 1), -1.0, 2.0)], [clipped], 1e-4, 1e-4)


def test_constant_side_ops():
    """Equal / Where / Expand / ConstantOfShape / Cast on constants and shapes."""
    i64 = np.int64
    m = ow.model(
        [ow.node("Shape", ["x"], ["s"]),
         ow.node("Equal", ["s", "s"], ["same"]),                         # shape vs shape
         ow.node("Where", ["same", "a", "b"], ["picked"]),
         ow.node("Cast", ["picked"], ["pf"], to=1),
         ow.node("ConstantOfShape", ["cshape"], ["filled"], value=np.array([3.0], np.float32)),
         ow.node("Expand", ["pf", "eshape"], ["ex"]),
         ow.node("Add", ["ex", "filled"], ["y0"]),
         ow.node("Mul", ["x", "y0"], ["y"])],
        [ow.tensor("a", np.array([10, 20], i64)), ow.tensor("b", np.array([1, 2], i64)),
         ow.tensor("cshape", np.array([1, 2], i64)), ow.tensor("eshape", np.array([1, 2], i64))],
        [ow.value_info("x", ["batch_size", 2])], [ow.value_info("y", ["batch_size", 2])])
    x = rng(5).standard_normal((3, 2)).astype(np.float32)
    _, (y,) = run(m, 3, [x])
    np.testing.assert_allclose(y, x * (np.array([[10.0, 20.0]], np.float32) + 3.0), rtol=1e-6)


def test_named_axes_and_input_shapes():
    m = ow.model([ow.node("Relu", ["x"], ["y"])], [], [ow.value_info("x", ["batch_size", "seq", 4])],
                 [ow.value_info("y", ["batch_size", "seq", 4])])
    with pytest.raises(OnnxError, match="unknown axis 'seq'"):
        load_graph_from_onnx_bytes(m)
    g = load_graph_from_onnx_bytes(m, named_axes={"seq": Size(7)})
    assert g[g.inputs[0]].shape == (BATCH, Size(7), Size(4))
    g = load_graph_from_onnx_bytes(m, input_shapes=[(BATCH, Size(2), Size(4))])
    assert g[g.inputs[0]].shape == (BATCH, Size(2), Size(4))


def test_errors():
    x_in = [ow.value_info("x", ["batch_size", 4])]
    y_out = [ow.value_info("y", ["batch_size", 4])]
    with pytest.raises(OnnxError, match="unsupported operation 'Celu'"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Celu", ["x"], ["y"])], [], x_in, y_out))
    with pytest.raises(OnnxError, match="leftover attributes"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Relu", ["x"], ["y"], alpha=1.0)], [], x_in, y_out))
    with pytest.raises(OnnxError, match="leftover inputs"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Relu", ["x", "x"], ["y"])], [], x_in, y_out))
    with pytest.raises(OnnxError, match="does not exist"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Relu", ["nope"], ["y"])], [], x_in, y_out))
    w = ow.tensor("w", np.zeros((4, 4), np.float32))
    with pytest.raises(OnnxError, match="alpha = beta = 1"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Gemm", ["x", "w"], ["y"], alpha=2.0, beta=1.0, transB=1)],
                                            [w], x_in, y_out))
    with pytest.raises(OnnxError, match="batch-dependent shape"):
        load_graph_from_onnx_bytes(ow.model([ow.node("Shape", ["x"], ["y"])], [], x_in, y_out))
    with pytest.raises(OnnxError, match="unsupported ONNX data type 10"):      # float16
        bad = ow._bytes(1, b"x") + ow._bytes(2, ow._bytes(1, ow._int(1, 10) + ow._bytes(2, b"")))
        load_graph_from_onnx_bytes(ow.model([], [], [bad], []))


def test_supported_ops_cover_the_reference_list():
    expected = {"Conv", "Clip", "Abs", "Neg", "Sin", "Cos", "Exp", "Log", "Sqrt", "Sigmoid", "Relu", "Tanh", "Erf",
                "Mish", "Softplus", "Add", "Sub", "Mul", "Div", "Min", "Max", "Pow", "Equal", "Where", "Flatten",
                "Gemm", "MatMul", "Einsum", "BatchNormalization", "InstanceNormalization", "LayerNormalization",
                "Constant", "ConstantOfShape", "Cast", "Reshape", "Expand", "Unsqueeze", "Transpose", "Gather",
                "Slice", "Concat", "Split", "Pad", "Shape", "Identity", "Softmax", "ReduceSum", "ReduceMean",
                "ReduceProd", "ReduceMin", "ReduceMax", "MaxPool", "AveragePool", "GlobalMaxPool",
                "GlobalAveragePool", "Resize"}
    assert set(SUPPORTED_OPS) == expected
