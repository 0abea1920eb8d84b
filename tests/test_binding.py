"""The `kyanite`-style Python binding (kn-python/src/lib.rs) and the `profile_net` tool
(kn-cuda-eval/src/bin/profile_net.rs) on top of the C ABI."""
import io
import os

import numpy as np
import pytest

import onnx_writer as ow
from kyanite_b200.binding import Graph, infer_batch_size, parse_device
from kyanite_b200.graph import BATCH, Size, shape
from kyanite_b200 import profile_net
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph


def small_model() -> bytes:
    r = np.random.Generator(np.random.PCG64(7))
    w = r.standard_normal((8, 3, 3, 3)).astype(np.float32)
    scale, bias, mean = (r.standard_normal(8).astype(np.float32) for _ in range(3))
    var = r.random(8).astype(np.float32) + 0.5
    fc = r.standard_normal((4, 8 * 5 * 5)).astype(np.float32)
    return ow.model(
        [ow.node("Conv", ["x", "w"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1]),
         ow.node("BatchNormalization", ["c", "scale", "bias", "mean", "var"], ["n"], epsilon=1e-5, momentum=0.9),
         ow.node("Relu", ["n"], ["r"]),
         ow.node("Flatten", ["r"], ["f"], axis=1),
         ow.node("Gemm", ["f", "fc"], ["l"], alpha=1.0, beta=1.0, transB=1),
         ow.node("Softmax", ["l"], ["y"], axis=1)],
        [ow.tensor("w", w), ow.tensor("scale", scale), ow.tensor("bias", bias), ow.tensor("mean", mean),
         ow.tensor("var", var), ow.tensor("fc", fc)],
        [ow.value_info("x", ["batch_size", 3, 5, 5])], [ow.value_info("y", ["batch_size", 4])])


def test_infer_batch_size():
    # kn-graph/src/shape.rs:352-419
    assert infer_batch_size([shape(BATCH, 3), shape(2, BATCH)], [(5, 3), (2, 5)]) == 5
    assert infer_batch_size([shape(4, 3)], [(4, 3)]) is None
    assert infer_batch_size([shape(BATCH * BATCH * 2)], [(18,)]) == 3
    assert infer_batch_size([shape(BATCH, 3)], [(0, 3)]) == 0
    with pytest.raises(ValueError, match="ConstantMismatch"):
        infer_batch_size([shape(BATCH, 3)], [(5, 4)])
    with pytest.raises(ValueError, match="BatchConflict"):
        infer_batch_size([shape(BATCH, 3), shape(BATCH)], [(5, 3), (6,)])
    with pytest.raises(ValueError, match="DifferentLength"):
        infer_batch_size([shape(BATCH, 3)], [(5,)])
    with pytest.raises(ValueError, match="ImpossibleBatchValue"):
        infer_batch_size([shape(Size(2, 1))], [(5,)])


def test_graph_from_bytes_and_optimize():
    g = Graph.from_bytes(small_model())
    opt = g.optimize()
    assert len(opt.inner.values) < len(g.inner.values)
    x = np.zeros((6, 3, 5, 5), np.float32)
    assert g.infer_batch_size([x]) == 6
    with pytest.raises(RuntimeError, match="Could not infer batch size"):
        g.infer_batch_size([np.zeros((6, 3, 5, 4), np.float32)])
    with pytest.raises(RuntimeError):
        Graph.from_bytes(b"\x3a\x05hello")
    assert "Conv" in str(opt) or "conv" in str(opt).lower()


def test_device_strings():
    with pytest.raises(TypeError, match="Invalid device string"):
        parse_device("tpu")
    with pytest.raises(TypeError, match="Invalid device string"):
        parse_device("cuda:x")
    with pytest.raises(RuntimeError, match="no CPU executor"):
        parse_device("cpu")


def test_profile_net_print_needs_no_gpu(tmp_path, capsys):
    path = tmp_path / "m.onnx"
    path.write_bytes(small_model())
    assert profile_net.main([str(path), "--optimize", "--print", "--batch-size", "4"]) == 0
    out = capsys.readouterr().out
    assert "Optimizing graph" in out and "plan batch=4" in out
    assert profile_net.main([str(path), "--print"]) == 2
    assert profile_net.main([str(path), "--cpu", "--batch-size", "4"]) == 2
    zeros = profile_net.dummy_zero_inputs(Graph.from_bytes(small_model()).inner, 3)
    assert [z.shape for z in zeros] == [(3, 3, 5, 5)]


@pytest.mark.gpu
def test_prepare_and_eval():
    g = Graph.from_bytes(small_model())
    x = np.random.Generator(np.random.PCG64(8)).standard_normal((6, 3, 5, 5)).astype(np.float32)
    expected = cpu_eval_graph(g.inner.to_bytes(), 6, [x])
    for graph in (g, g.optimize()):
        prepared = graph.prepare("cuda:0", graph.infer_batch_size([x]))
        assert_tensors_match(expected, prepared.eval([x]), 4e-3, 4e-3, abs_scaled=True)
    with pytest.raises(RuntimeError, match="Invalid CUDA device index"):
        g.prepare("cuda:999", 1)
    assert parse_device("best").cuda_device.index == 0
    with pytest.raises(TypeError, match="Unsupported dtype"):
        g.prepare("cuda", 6).eval([x.astype(np.complex64)])


@pytest.mark.gpu
def test_profile_net_runs(tmp_path):
    path = tmp_path / "m.onnx"
    path.write_bytes(small_model())
    out = io.StringIO()
    g = Graph.from_bytes(small_model()).optimize().inner
    from kyanite_b200.executor import MATH_TF32, CudaDevice
    rate = profile_net.profile_single(CudaDevice(0), g, 16, 20, False, MATH_TF32, out=out)
    assert rate > 0 and "Throughput:" in out.getvalue() and "total" in out.getvalue()
    rate_async = profile_net.profile_single(CudaDevice(0), g, 16, 20, True, MATH_TF32, out=io.StringIO())
    assert rate_async > 0
    assert profile_net.main([str(path), "-o", "-b", "8", "-n", "10"]) == 0
