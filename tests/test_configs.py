"""The named workload shapes (MLP, ResNet tower, BERT-, LLaMA- and UNet-shaped graphs) at reduced sizes:
the planner lowers each one in both math modes and the CUDA executor agrees with the CPU oracle.

The full-size versions differ only in the size arguments of the same builders, so these cases cover the
operator mix and fusion patterns of each workload at a size the oracle finishes in seconds."""
import collections

import numpy as np
import pytest

from kyanite_b200 import configs
from kyanite_b200.executor import MATH_F32, MATH_TF32, plan_describe
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

SMALL = {
    "mlp": (lambda: configs.mlp(), 8),
    "tower": (lambda: configs.resnet_tower(blocks=2, channels=32), 4),
    "bert": (lambda: configs.bert_encoder(layers=2, hidden=64, heads=4, ffn=128, vocab=100, seq=16), 2),
    "llama": (lambda: configs.llama_decoder(layers=2, d_model=64, heads=4, ffn=96, vocab=100, seq=16), 2),
    "unet": (lambda: configs.unet_step(levels=(32, 64), res_blocks=1, attention_levels=(0,), heads=2, size=16,
                                       ctx_len=5, ctx_dim=24, groups=8), 2),
}


def _kinds(description: str):
    return collections.Counter(line.split()[2] for line in description.splitlines() if line.startswith("step"))


@pytest.mark.parametrize("name", sorted(SMALL))
@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32])
def test_config_lowers(name, mode):
    build, batch = SMALL[name]
    graph, _ = build()
    kinds = _kinds(plan_describe(graph, batch, mode))
    assert sum(kinds.values()) > 0
    if mode == MATH_F32:
        assert not any(k.endswith("/tc") for k in kinds), kinds


def test_transformer_fusion_counts():
    """Per encoder layer: 6 matmul-shaped steps (fused QKV are separate here: 3 + scores + context + out)
    plus 2 feed-forward, 2 layernorms, 1 softmax; the bias/GELU/residual arithmetic must not add more than
    a handful of scalar steps per layer."""
    graph, _ = configs.bert_encoder(layers=2, hidden=64, heads=4, ffn=128, vocab=100, seq=16)
    kinds = _kinds(plan_describe(graph, 2, MATH_F32))
    assert kinds["Gemm"] == 16
    assert kinds["Softmax"] == 2
    assert kinds["Layernorm"] == 5
    assert kinds["Gather"] == 1
    assert kinds["Scalar"] <= 12


def test_oracle_runs_every_config():
    for name, (build, batch) in SMALL.items():
        graph, make_inputs = build()
        outs = cpu_eval_graph(graph.to_bytes(), batch, make_inputs(batch, 1))
        assert all(np.isfinite(o).all() for o in outs if o.dtype.kind == "f"), name


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SMALL))
@pytest.mark.parametrize("mode", [MATH_F32, MATH_TF32])
def test_config_matches_oracle(name, mode):
    from kyanite_b200.executor import CudaDevice, CudaExecutor
    build, batch = SMALL[name]
    graph, make_inputs = build()
    inputs = make_inputs(batch, 3)
    expected = cpu_eval_graph(graph.to_bytes(), batch, inputs)
    ex = CudaExecutor(CudaDevice(0), graph, batch, math_mode=mode)
    for _ in range(2):      # second call replays the captured CUDA graph
        actual = ex.evaluate(inputs)
        if mode == MATH_F32:
            assert_tensors_match(expected, actual, 1e-3, 1e-3)
        else:
            # TF32 operands (10-bit mantissa), f32 accumulation; scaled by the output magnitude
            assert_tensors_match(expected, actual, 4e-3, 4e-3, abs_scaled=True)


@pytest.mark.parametrize("name", ["bert", "unet"])
def test_oracle_block_by_block_equals_whole(name):
    """The plumbing of the full-size GPU tests (tests/test_full_size.py) on small graphs, with the oracle's own
    full-batch result standing in for the executor's: evaluating a subset of batch rows alone, and evaluating
    one block from overridden values of all other block boundaries, reproduce the whole-graph result."""
    from oracle.cpu_eval import parse_graph
    taps = []
    if name == "bert":
        graph, make_inputs = configs.bert_encoder(layers=2, hidden=64, heads=4, ffn=128, vocab=100, seq=16, taps=taps)
    else:
        graph, make_inputs = configs.unet_step(levels=(32, 64), res_blocks=1, attention_levels=(0,), heads=2, size=16,
                                               ctx_len=5, ctx_dim=24, groups=8, taps=taps)
    assert len(taps) >= 3
    for _, v in taps:
        if v.index not in [o.index for o in graph.outputs]:
            graph.output(v)
    out_pos = {o.index: i for i, o in enumerate(graph.outputs)}
    parsed = parse_graph(graph.to_bytes())
    batch, rows = 3, [2]
    inputs = make_inputs(batch, 5)
    whole = cpu_eval_graph(parsed, batch, inputs)
    sub_inputs = [x[rows] if x.shape[:1] == (batch,) else x for x in inputs]
    alone = cpu_eval_graph(parsed, len(rows), sub_inputs)
    assert_tensors_match([w[rows] for w in whole], alone, 1e-5, 1e-5)
    for tap_name, v in taps:
        overrides = {w.index: whole[out_pos[w.index]][rows] for n, w in taps if n != tap_name}
        block = cpu_eval_graph(parsed, len(rows), sub_inputs, overrides=overrides, wanted=[v.index])
        assert_tensors_match([whole[out_pos[v.index]][rows]], block, 1e-5, 1e-5)
    # values nothing needs are not computed: with every tap overridden and one of them wanted, no input is read
    last = taps[-1][1]
    only = cpu_eval_graph(parsed, len(rows), [None] * len(inputs),
                          overrides={w.index: whole[out_pos[w.index]][rows] for _, w in taps}, wanted=[last.index])
    np.testing.assert_array_equal(only[0], whole[out_pos[last.index]][rows])
