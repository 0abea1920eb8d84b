"""Pins the CPU oracle against every hand-computed expected output the reference's own tests hold
for this path (see tests/ref_graphs.py for the sources), and checks that every re-expressed
reference graph at least evaluates with consistent shapes and dtypes."""
import numpy as np
import pytest

import ref_graphs
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

CASES = ref_graphs.all_cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_oracle_case(case):
    outs = cpu_eval_graph(case.graph.to_bytes(), case.batch_size, case.inputs)
    assert len(outs) == len(case.graph.outputs)
    for o, v in zip(outs, case.graph.outputs):
        info = case.graph[v]
        assert o.shape == tuple(d.eval(case.batch_size) for d in info.shape)
        assert o.dtype == info.dtype.np
    if case.expected is not None:
        assert_tensors_match(case.expected, outs)


def test_pinned_count():
    # the number of cases carrying reference-held numbers; guards against silently dropping pins
    assert sum(c.expected is not None for c in CASES) >= 45


def test_layernorm_op_matches_composition():
    by = {c.name: c for c in CASES}
    a, b = by["layernorm_op"], by["layernorm_composed"]
    ra = cpu_eval_graph(a.graph.to_bytes(), 2, a.inputs)
    rb = cpu_eval_graph(b.graph.to_bytes(), 2, b.inputs)
    assert_tensors_match(rb, ra)


def test_gather_rejects_out_of_range():
    from kyanite_b200.graph import DType, Graph, shape
    g = Graph()
    x = g.input(shape(4))
    i = g.input(shape(2), DType.I32)
    g.output(g.gather(x, 0, i))
    with pytest.raises(IndexError):
        cpu_eval_graph(g.to_bytes(), 0, [np.zeros(4, np.float32), np.array([0, 4], np.int32)])
    with pytest.raises(IndexError):
        cpu_eval_graph(g.to_bytes(), 0, [np.zeros(4, np.float32), np.array([-1, 0], np.int32)])
