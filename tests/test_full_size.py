"""The BERT-base-shaped encoder and the diffusion-UNet-shaped step at their full sizes (hidden 768, 12 layers,
512 tokens, batch 32; channel levels 320/640/1280/1280, 64x64 latents, batch 8) on the GPU, checked against
the CPU oracle.

The oracle cannot run these graphs whole at the full batch in test time, and does not have to: no operation
of either graph mixes batch entries, so the oracle's result for a few batch rows evaluated alone equals its
rows of the full-batch result.  The executor runs the full batch; the oracle runs the same graph
  - end to end on a subset of the batch rows, and
  - layer by layer: every block boundary of the graph is an extra output of the executor, and the oracle
    computes each block from the EXECUTOR's values of everything before it (`overrides` / `wanted` of
    `cpu_eval_graph`), which localises an error to the block that made it.  This is the differential
    method of the reference's own runner (kn-cuda-eval/tests/root/runner.rs:29-55) applied per block.

Tolerances are stated next to each assertion.  TF32 mode: operands of the contractions are rounded to a
10-bit mantissa (relative 2^-11), accumulation is f32."""
import numpy as np
import pytest

from kyanite_b200 import configs
from kyanite_b200.executor import MATH_F32, MATH_TF32, CudaExecutor
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph, parse_graph

pytestmark = pytest.mark.gpu


def _with_tap_outputs(graph, taps):
    """Every tapped value becomes a graph output (once); returns name -> output position."""
    position = {}
    existing = {v.index: i for i, v in enumerate(graph.outputs)}
    for name, v in taps:
        if v.index not in existing:
            graph.output(v)
            existing[v.index] = len(graph.outputs) - 1
        position[name] = existing[v.index]
    return position


def _layerwise(parsed, taps, position, got, rows, sub_inputs, tol, report):
    """Oracle block by block: block i is computed from the executor's values of all other taps."""
    worst = (0.0, 0.0)
    for name, v in taps:
        overrides = {w.index: got[position[n]][rows] for n, w in taps if n != name}
        expected = cpu_eval_graph(parsed, len(rows), sub_inputs, overrides=overrides, wanted=[v.index])
        try:
            max_abs, max_rel = assert_tensors_match(expected, [got[position[name]][rows]], tol, tol, abs_scaled=True)
        except AssertionError as e:
            raise AssertionError(f"block {name}: {e}") from None
        scale = float(np.abs(expected[0]).max())
        report.append((name, max_abs, scale))
        worst = max(worst, (max_abs / scale if scale > 0 else 0.0, max_abs))
    return worst


@pytest.mark.parametrize("mode", [MATH_TF32, MATH_F32], ids=["tf32", "f32"])
def test_bert_base_full_size(mode):
    batch, rows = 32, [0, 31]
    taps = []
    graph, make_inputs = configs.bert_encoder(taps=taps)
    position = _with_tap_outputs(graph, taps)
    inputs = make_inputs(batch, 7)
    blob = graph.to_bytes()
    with CudaExecutor(0, blob, batch, math_mode=mode) as ex:
        got = ex.evaluate(inputs)
    parsed = parse_graph(blob)
    sub_inputs = [inputs[0][rows]]
    # Activations are layer-normalised (O(1), largest about 10).  Stated tolerance per tensor: a value
    # mismatches iff its error is >= tol * (largest |expected|) AND >= tol relative; tol = 4e-3 for TF32
    # operands, 1e-3 for exact f32 (the reference's figure, kn-cuda-eval/src/tester.rs:28-29).
    tol = 4e-3 if mode == MATH_TF32 else 1e-3
    # end to end on two of the 32 sequences: all 12 layers' errors compounded
    expected = cpu_eval_graph(parsed, len(rows), sub_inputs)
    e2e_abs, _ = assert_tensors_match(expected, [g[rows] for g in got], tol, tol, abs_scaled=True)
    report = []
    worst_frac, _ = _layerwise(parsed, taps, position, got, rows, sub_inputs, tol, report)
    # measured bounds, asserted so that a drift shows: one layer's error stays below 5e-4 of the tensor's scale
    # in TF32 mode (1e-5 in exact f32), the compounded end-to-end error below 1e-2 absolute (1e-4 in f32)
    # (measured on a B200: TF32 1.7e-4 per block and 2.6e-3 end to end; exact f32 1.1e-6 and 7.6e-6)
    assert worst_frac <= (5e-4 if mode == MATH_TF32 else 1e-5), report
    assert e2e_abs <= (1e-2 if mode == MATH_TF32 else 1e-4), e2e_abs
    print(f"bert full size mode={mode}: end-to-end max abs {e2e_abs:.3e}; worst block error / scale {worst_frac:.3e}")


def test_unet_full_size():
    batch, rows = 8, [3]
    taps = []
    graph, make_inputs = configs.unet_step(taps=taps)
    position = _with_tap_outputs(graph, taps)
    inputs = make_inputs(batch, 7)
    blob = graph.to_bytes()
    del graph
    with CudaExecutor(0, blob, batch, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
    parsed = parse_graph(blob)
    sub_inputs = [inputs[0][rows], inputs[1], inputs[2][rows]]
    tol = 4e-3
    # end to end on one of the 8 latents (one full oracle pass)
    expected = cpu_eval_graph(parsed, len(rows), sub_inputs)
    e2e_abs, _ = assert_tensors_match(expected, [g[rows] for g in got], tol, tol, abs_scaled=True)
    final_abs, _ = assert_tensors_match(expected[:1], [got[0][rows]], tol, tol, abs_scaled=True)
    final_scale = float(np.abs(expected[0]).max())
    report = []
    worst_frac, _ = _layerwise(parsed, taps, position, got, rows, sub_inputs, tol, report)
    # measured bound for one block (up to 8 contractions with K up to 23 040 in it): error below 1.5e-3 of the
    # block output's scale (measured on a B200: 4.4e-4); the denoised latent end to end within 2e-3 of its scale
    assert worst_frac <= 1.5e-3, report
    assert final_abs <= 2e-3 * final_scale, (final_abs, final_scale)
    print(f"unet full size: end-to-end max abs {e2e_abs:.3e} over all block outputs; final output max abs {final_abs:.3e} "
          f"on a scale of {final_scale:.3e}; worst block error / scale {worst_frac:.3e}")


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_llama_layer_full_width(dtype):
    """One decoder layer of the LLaMA-7B-shaped configuration at full width (d_model 4096, 32 heads of 128, SwiGLU
    11008, 2048 tokens, causal mask, RoPE) plus final norm and a 1000-row slice of the lm head, against the oracle,
    end to end and block by block.  f16: storage f16, accumulation f32 (an extension without reference vectors:
    parity unpinned); f32: TF32 tensor cores."""
    from kyanite_b200.graph import DType
    dt = DType.F16 if dtype == "f16" else DType.F32
    taps = []
    graph, make_inputs = configs.llama_decoder(layers=1, vocab=1000, dtype=dt, taps=taps)
    position = _with_tap_outputs(graph, taps)
    inputs = make_inputs(1, 7)
    blob = graph.to_bytes()
    del graph
    with CudaExecutor(0, blob, 1, math_mode=MATH_TF32) as ex:
        got = ex.evaluate(inputs)
    parsed = parse_graph(blob)
    # f16: about 20 roundings to 11 bits on the path of an output; tf32: operands rounded to 11 bits, f32 sums
    tol = 1e-2 if dtype == "f16" else 4e-3
    expected = cpu_eval_graph(parsed, 1, inputs)
    e2e_abs, _ = assert_tensors_match(expected, got, tol, tol, abs_scaled=True)
    report = []
    worst_frac, _ = _layerwise(parsed, taps, position, got, [0], inputs, tol, report)
    # measured bound, asserted: one block's error stays below 4e-3 of its output's scale
    assert worst_frac <= 4e-3, report
    print(f"llama layer full width {dtype}: end-to-end max abs {e2e_abs:.3e}; worst block error / scale {worst_frac:.3e}")
