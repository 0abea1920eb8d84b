"""Regenerates the ONNX golden fixtures of this folder from the reference checkout.

For each model of kn-cuda-eval/tests/data (the models behind kn-cuda-eval/tests/root/onnx.rs) it writes
  <name>.kng   the graph produced by `kyanite_b200.onnx.load_graph_from_onnx_bytes`, in the wire format of
               `Graph.to_bytes()`
  <name>.npz   batch size, inputs and expected outputs decoded from the reference's `<name>.bin`
               (layout: kn-cuda-eval/src/tester.rs:305-345 - one byte batch size, then every input and
               every expected output as little-endian f32 in graph order)
The expected outputs were produced by the framework the models were trained in, not by this repository.

    python tests/golden/make_onnx_golden.py /path/to/reference
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from kyanite_b200.onnx import load_graph_from_onnx_bytes  # noqa: E402

NAMES = ["simple-sttt-1x64", "simple-bn-sttt-1x64", "pre-sttt-4x8", "att-tiny"]


def decode_check_data(graph, raw: bytes):
    batch = raw[0]
    assert (len(raw) - 1) % 4 == 0, "check data must be 1 + 4n bytes"
    data = np.frombuffer(raw[1:], dtype="<f4")
    pos = 0
    groups = []
    for values in (graph.inputs, graph.outputs):
        tensors = []
        for v in values:
            dims = tuple(d.eval(batch) for d in graph[v].shape)
            n = int(np.prod(dims, dtype=np.int64))
            tensors.append(data[pos:pos + n].reshape(dims).astype(np.float32))
            pos += n
        groups.append(tensors)
    assert pos == len(data), f"leftover elements in check data: {len(data) - pos}"
    return batch, groups[0], groups[1]


def main(reference_root: str):
    data_dir = os.path.join(reference_root, "kn-cuda-eval", "tests", "data")
    for name in NAMES:
        with open(os.path.join(data_dir, name + ".onnx"), "rb") as f:
            graph = load_graph_from_onnx_bytes(f.read())
        with open(os.path.join(data_dir, name + ".bin"), "rb") as f:
            batch, inputs, outputs = decode_check_data(graph, f.read())
        with open(os.path.join(HERE, name + ".kng"), "wb") as f:
            f.write(graph.to_bytes())
        arrays = {"batch": np.array(batch, dtype=np.int64)}
        arrays.update({f"input{i}": t for i, t in enumerate(inputs)})
        arrays.update({f"output{i}": t for i, t in enumerate(outputs)})
        np.savez(os.path.join(HERE, name + ".npz"), **arrays)
        print(name, "batch", batch, "values", len(graph.values), [t.shape for t in outputs])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KN_REFERENCE_DIR", os.path.join(os.sep, "root", "reference")))
