"""GPU parity: every graph of the reference's executor test-suite (re-expressed in
tests/ref_graphs.py) runs through the C ABI on cuda:0 and is compared with the CPU oracle, or
with the reference's hand-computed numbers where it holds some, under the reference's own rule:
a float mismatches iff abs diff >= 1e-3 AND rel diff >= 1e-3, NaN positions must agree, every
other dtype must be bit-exact (kn-cuda-eval/src/tester.rs:28-29, 216-302).

Both math modes are exercised.  KN_MATH_F32 (exact f32 FMA) is held to the reference's 1e-3 rule.
KN_MATH_TF32 runs contractions on the tensor cores with operands rounded to TF32 (10-bit mantissa,
relative rounding error up to 2^-11 per operand): graphs whose contractions stay on the SIMT path
at these sizes still meet 1e-3; tensor-core ones mismatch iff abs >= 4e-3 * (largest |expected|
of the tensor, no floor at 1) AND rel >= 4e-3 (the rounding error of a contraction scales with the summed
magnitudes, which chained convolutions with cancelling weights make much larger than the result)."""
import numpy as np
import pytest

import ref_graphs
from kyanite_b200.executor import MATH_F32, MATH_TF32, CudaExecutor, plan_describe
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

pytestmark = pytest.mark.gpu

CASES = ref_graphs.all_cases()


@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32], ids=["f32", "tf32"])
@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_reference_graph(case, mode):
    blob = case.graph.to_bytes()
    expected = case.expected if case.expected is not None else cpu_eval_graph(blob, case.batch_size, case.inputs)
    tol = 1e-3
    if mode == MATH_TF32 and "/tc" in plan_describe(blob, case.batch_size, math_mode=mode):
        tol = 4e-3
    with CudaExecutor(0, blob, case.batch_size, math_mode=mode) as ex:
        first = ex.evaluate(case.inputs)
        assert_tensors_match(expected, first, tol_abs=tol, tol_rel=tol, abs_scaled=tol > 1e-3)
        # second call replays the captured CUDA graph
        second = ex.evaluate(case.inputs)
        assert_tensors_match(expected, second, tol_abs=tol, tol_rel=tol, abs_scaled=tol > 1e-3)
    if case.expected is not None:
        # the oracle itself must agree with the reference-held numbers too
        assert_tensors_match(case.expected, cpu_eval_graph(blob, case.batch_size, case.inputs))


@pytest.mark.parametrize("case", [c for c in CASES if c.name in ("pre_act_resnet", "permute", "int_ops", "softmax")],
                         ids=lambda c: c.name)
def test_without_cuda_graph_and_with_profile(case):
    blob = case.graph.to_bytes()
    expected = cpu_eval_graph(blob, case.batch_size, case.inputs)
    with CudaExecutor(0, blob, case.batch_size, math_mode=MATH_F32, use_cuda_graph=False) as ex:
        assert_tensors_match(expected, ex.evaluate(case.inputs))
        ex.set_profile(True)
        assert_tensors_match(expected, ex.evaluate(case.inputs))
        prof = ex.last_profile()
        steps, launches = ex.step_count()
        assert len([l for l in prof.splitlines() if not l.startswith("total")]) == steps
        assert launches >= steps


def test_wrong_inputs_are_rejected():
    case = next(c for c in CASES if c.name == "linear")
    with CudaExecutor(0, case.graph, 0) as ex:
        with pytest.raises(ValueError):
            ex.evaluate([])
        with pytest.raises(ValueError):
            ex.evaluate([np.zeros((2, 4), np.float32)])
        with pytest.raises(ValueError):
            ex.evaluate([np.zeros((1, 4), np.float64)])


def test_missing_device():
    from kyanite_b200.executor import CudaDeviceNotAvailable
    case = next(c for c in CASES if c.name == "linear")
    with pytest.raises(CudaDeviceNotAvailable):
        CudaExecutor(99, case.graph, 0)


def test_gather_out_of_range_writes_zero():
    """The CPU path rejects such indices (kn-graph/src/cpu.rs:309-330); the device path writes 0
    like the reference's kernel (kn-cuda-eval/src/autokernel/gather.cu:46-49)."""
    from kyanite_b200.graph import DType, Graph, shape
    g = Graph()
    x = g.input(shape(4, 3))
    i = g.input(shape(5), DType.I32)
    g.output(g.gather(x, 0, i))
    data = np.arange(12, dtype=np.float32).reshape(4, 3) + 1
    idx = np.array([0, 4, -1, 3, 100], np.int32)
    with CudaExecutor(0, g, 0) as ex:
        out = ex.evaluate([data, idx])[0]
    want = np.stack([data[0], np.zeros(3), np.zeros(3), data[3], np.zeros(3)]).astype(np.float32)
    assert np.array_equal(out, want)


def test_staged_evaluate_matches():
    case = next(c for c in CASES if c.name == "fuse_res")
    expected = cpu_eval_graph(case.graph.to_bytes(), case.batch_size, case.inputs)
    with CudaExecutor(0, case.graph, case.batch_size, math_mode=MATH_F32) as ex:
        for dst, src in zip(ex.host_inputs, case.inputs):
            dst[...] = src
        outs = [o.copy() for o in ex.evaluate_staged()]
        assert_tensors_match(expected, outs)
        # device-resident rerun: no upload, run_async + download only
        ex.run_async()
        ex.download_outputs()
        ex.synchronize()
        assert_tensors_match(expected, [o.copy() for o in ex.host_outputs])


@pytest.mark.parametrize("dims,perm", [((3, 70, 45), (0, 2, 1)), ((2, 5, 33, 64), (0, 3, 1, 2)), ((40, 100), (1, 0)),
                                       ((2, 3, 4, 40, 50), (4, 1, 2, 3, 0)), ((16, 16), (1, 0)), ((1, 300, 17), (0, 2, 1))])
def test_transposing_copies_are_bit_exact(dims, perm):
    """A materialised permutation whose source and destination are contiguous along different axes goes
    through the tiled transposing-copy kernel (32 x 32 tiles through shared memory), for f32 and i32,
    with ragged tile edges and outer axes on both sides; smaller axes stay on the generic kernel."""
    from kyanite_b200.graph import DType, Graph, shape
    r = np.random.Generator(np.random.PCG64(3))
    for dtype, np_dtype in ((DType.F32, np.float32), (DType.I32, np.int32)):
        g = Graph()
        x = g.input(shape(*dims), dtype)
        y = g.permute(x, list(perm))
        g.output(g.view(y, shape(int(np.prod(dims)))))     # a flat view forces the permuted tensor to exist
        data = (r.standard_normal(dims) * 100).astype(np_dtype)
        with CudaExecutor(0, g, 0) as ex:
            (got,) = ex.evaluate([data])
        np.testing.assert_array_equal(got, np.transpose(data, perm).reshape(-1))


@pytest.mark.parametrize("rows,length,mask_kind", [(64, 512, "rows"), (10, 37, "rows"), (3, 9000, "rows"), (8, 256, "full"),
                                                    (8, 64, "per_row_constant"), (4, 2048, "rows")])
def test_softmax_with_scale_and_additive_term(rows, length, mask_kind):
    """softmax(0.125 * x + mask) is one step: the 128-bit kernel (row length a multiple of 4), the scalar
    kernel (37), the streaming kernel (9000); the term broadcast over the batch axis, of full shape, or
    constant along the row."""
    from kyanite_b200.graph import Graph, shape
    r = np.random.Generator(np.random.PCG64(11))
    b = 3
    g = Graph()
    x = g.input(shape(b, rows, length))
    mask_shape = {"rows": (1, rows, length), "full": (b, rows, length), "per_row_constant": (b, rows, 1)}[mask_kind]
    mask = g.input(shape(*mask_shape))
    full = g.broadcast(mask, shape(b, rows, length)) if mask_shape != (b, rows, length) else mask
    g.output(g.softmax(g.add(g.mul(x, g.scalar(0.125)), full), 2))
    text = plan_describe(g, 0)
    assert len([l for l in text.splitlines() if l.startswith("step")]) == 1 and "+term" in text
    m = np.where(r.random(mask_shape) < 0.3, -1e9, 0.0).astype(np.float32)
    m[..., 0] = 0.0   # never a fully masked row
    ins = [(r.standard_normal((b, rows, length)) * 8).astype(np.float32), m]
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    with CudaExecutor(0, g, 0) as ex:
        assert_tensors_match(expected, ex.evaluate(ins))


@pytest.mark.parametrize("rows,length", [(5, 8196), (64, 20480), (3, 40960), (2, 49152), (2, 49156), (2, 81920), (64, 81920), (3, 122880),
                                         (5, 131076), (2, 393216), (2, 393220), (1, 49154), (160, 81920), (80, 122880), (300, 81920)])
def test_layernorm_over_long_rows(rows, length):
    """Group-norm sized rows: 8193..49152 elements run on the one-block-per-row kernel with the row in
    registers (with a second input scaled into the first), up to eight times that on a cluster of eight CTAs per row
    (slices that do not divide evenly, the last CTA's slice short), longer or oddly sized ones on the streaming kernel."""
    from kyanite_b200.graph import Graph, shape
    r = np.random.Generator(np.random.PCG64(21))
    g = Graph()
    a = g.input(shape(rows, length))
    b = g.input(shape(rows, length))
    g.output(g.layernorm(g.add(a, g.mul(b, g.scalar(0.5))), 1, 1e-5))
    ins = [(r.standard_normal((rows, length)) * 3 + 1).astype(np.float32), r.standard_normal((rows, length)).astype(np.float32)]
    expected = cpu_eval_graph(g.to_bytes(), 0, ins)
    with CudaExecutor(0, g, 0) as ex:
        assert_tensors_match(expected, ex.evaluate(ins))


def test_evaluate_in_two_halves_with_two_executors():
    """kn_executor_evaluate_begin / _end: two executors of one graph on one device, the next batch submitted
    before the current one is waited for; results equal those of plain `evaluate`, and the call order is
    checked (begin twice, end without begin)."""
    from kyanite_b200._lib import KnError
    case = next(c for c in CASES if c.name == "fuse_res")
    expected = cpu_eval_graph(case.graph.to_bytes(), case.batch_size, case.inputs)
    with CudaExecutor(0, case.graph, case.batch_size, math_mode=MATH_F32) as a, \
            CudaExecutor(0, case.graph, case.batch_size, math_mode=MATH_F32) as b:
        pair = [a, b]
        for ex in pair:
            for dst, src in zip(ex.host_inputs, case.inputs):
                dst[...] = src
        pair[0].evaluate_staged_begin()
        for i in range(6):
            if i + 1 < 6:
                pair[(i + 1) % 2].evaluate_staged_begin()
            outs = [o.copy() for o in pair[i % 2].evaluate_staged_end()]
            assert_tensors_match(expected, outs)
        with pytest.raises(KnError, match="without evaluate_begin"):
            a.evaluate_staged_end()
        a.evaluate_staged_begin()
        with pytest.raises(KnError, match="in flight"):
            a.evaluate_staged_begin()
        assert_tensors_match(expected, [o.copy() for o in a.evaluate_staged_end()])


def test_expired_wait_is_reported_and_the_executor_stays_usable():
    """Every barrier wait in the tensor-core kernels is bounded.  Here one runs out on purpose, harmlessly
    (kn_executor_selftest_wait_expiry: one thread, a barrier nobody arrives on, 1 ms limit, no tensor memory,
    no copies in flight): the kernel returns, the status word reaches the host as KN_ERR_INTERNAL, the word is
    cleared, and the executor computes the same results before and after, through the captured graph too."""
    import time
    from kyanite_b200 import _lib
    case = next(c for c in CASES if c.name == "fuse_res")
    expected = cpu_eval_graph(case.graph.to_bytes(), case.batch_size, case.inputs)
    lib = _lib.load()
    with CudaExecutor(0, case.graph, case.batch_size) as ex:
        assert_tensors_match(expected, ex.evaluate(case.inputs), 4e-3, 4e-3, abs_scaled=True)
        t0 = time.perf_counter()
        status = lib.kn_executor_selftest_wait_expiry(ex._ptr, 1000)
        elapsed = time.perf_counter() - t0
        assert status == 7, lib.kn_last_error()            # KN_ERR_INTERNAL
        assert b"gave up waiting" in lib.kn_last_error() and b"99" in lib.kn_last_error()
        assert elapsed < 1.0                                # a 1 ms limit, not the 2 s default
        ex.synchronize()                                    # the word was cleared: no stale error
        for _ in range(2):
            assert_tensors_match(expected, ex.evaluate(case.inputs), 4e-3, 4e-3, abs_scaled=True)
        assert lib.kn_executor_selftest_wait_expiry(ex._ptr, 0) == 1      # limit out of range
