"""The graph blob as the Rust shim writes it (rust/kn-cuda-eval-b200/src/serialize.rs, shipped as uncompiled
source: the build image has no Rust toolchain).  What can be checked without a compiler:
  - the tag tables in serialize.rs equal the ones the Python writer and the C++ reader use;
  - rust/kn-b200-sys declares every function of include/kn_b200.h, with the same number of parameters;
  - a blob written by an independent writer that follows the field order documented in serialize.rs is
    byte-identical to `Graph.to_bytes()` for every graph of the reference's test-suite, and the library parses it."""
import ctypes
import os
import re
import struct

import numpy as np
import pytest

import ref_graphs
from kyanite_b200 import _lib
from kyanite_b200.graph import BinaryOp, DType, OpKind, ReduceOp, UnaryOp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SERIALIZE_RS = open(os.path.join(ROOT, "rust", "kn-cuda-eval-b200", "src", "serialize.rs")).read()
SYS_RS = open(os.path.join(ROOT, "rust", "kn-b200-sys", "src", "lib.rs")).read()
HEADER = open(os.path.join(ROOT, "include", "kn_b200.h")).read()


def rust_consts(prefix):
    return {name: int(value, 0) for name, value in re.findall(rf"pub const {prefix}_([A-Z0-9_]+): u8 = (\w+);", SERIALIZE_RS)}


def test_tag_tables_agree():
    ops = rust_consts("OP")
    assert ops == {k.name: int(k) for k in OpKind if k.name != "ALL_REDUCE"}       # the reference's 16 operations
    assert rust_consts("DTYPE") == {d.name: int(d) for d in DType if d.name != "F16"}
    unary = rust_consts("UNARY")
    assert unary == {u.name: int(u) for u in UnaryOp}
    assert rust_consts("BINARY") == {b.name: int(b) for b in BinaryOp}
    assert rust_consts("REDUCE") == {r.name: int(r) for r in ReduceOp}
    # every Operation variant of the reference is matched twice in serialize_graph (tag, payload)
    for variant in ("Input", "Constant", "View", "Broadcast", "Permute", "Slice", "Flip", "Gather", "Concat", "Conv",
                    "MatMul", "Unary", "Binary", "Softmax", "Layernorm", "Reduce"):
        assert len(re.findall(rf"Operation::{variant}\b", SERIALIZE_RS)) >= 2, variant


def c_declarations():
    out = {}
    for name, params in re.findall(r"KN_API[^;(]*?\b(kn_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", HEADER, flags=re.S):
        params = params.strip()
        out[name] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def rust_declarations():
    out = {}
    for name, params in re.findall(r"pub fn (kn_[a-z0-9_]+)\s*\(([^;]*?)\)\s*(?:->[^;]*)?;", SYS_RS, flags=re.S):
        params = params.strip()
        out[name] = 0 if not params else len([p for p in params.split(",") if p.strip()])
    return out


def test_sys_crate_binds_every_header_function():
    c, rust = c_declarations(), rust_declarations()
    assert sorted(c) == sorted(_lib.SIGNATURES)
    assert rust == c


def write_like_the_shim(graph) -> bytes:
    """Independent writer, from the layout table in serialize.rs."""
    out = bytearray(b"KNG1")
    out += struct.pack("<III", len(graph.values), len(graph.inputs), len(graph.outputs))
    for v in list(graph.inputs) + list(graph.outputs):
        out += struct.pack("<I", v.index)
    for info in graph.values:
        out += struct.pack("<BBH", int(info.kind), int(info.dtype), len(info.shape))
        for d in info.shape:
            out += struct.pack("<QI", d.factor, d.exp)
        k = info.kind
        if k == OpKind.INPUT:
            out += struct.pack("<I", info.input_index)
        elif k == OpKind.CONSTANT:
            data = np.ascontiguousarray(info.tensor).tobytes()
            out += struct.pack("<Q", len(data)) + data
        elif k in (OpKind.VIEW, OpKind.BROADCAST):
            out += struct.pack("<I", info.inputs[0])
        elif k == OpKind.PERMUTE:
            out += struct.pack("<I", info.inputs[0]) + b"".join(struct.pack("<I", p) for p in info.permutation)
        elif k == OpKind.SLICE:
            out += struct.pack("<IIQQQ", info.inputs[0], info.axis, info.range.start, info.range.end, info.range.step)
        elif k == OpKind.FLIP:
            out += struct.pack("<II", info.inputs[0], info.axis)
        elif k == OpKind.GATHER:
            out += struct.pack("<III", info.inputs[0], info.axis, info.inputs[1])
        elif k == OpKind.CONCAT:
            out += struct.pack("<I", len(info.inputs)) + b"".join(struct.pack("<I", i) for i in info.inputs)
            out += struct.pack("<I", info.axis)
        elif k == OpKind.CONV:
            out += struct.pack("<IIIIII", info.inputs[0], info.inputs[1], *info.conv)
        elif k == OpKind.MATMUL:
            out += struct.pack("<II", *info.inputs)
        elif k == OpKind.UNARY:
            cast = 0xFF if info.cast_to is None else int(info.cast_to)
            out += struct.pack("<IBB", info.inputs[0], int(info.unary_op), cast)
        elif k == OpKind.BINARY:
            out += struct.pack("<IIB", info.inputs[0], info.inputs[1], int(info.binary_op))
        elif k == OpKind.SOFTMAX:
            out += struct.pack("<II", info.inputs[0], info.axis)
        elif k == OpKind.LAYERNORM:
            out += struct.pack("<IIf", info.inputs[0], info.axis, info.eps)
        elif k == OpKind.REDUCE:
            out += struct.pack("<IBI", info.inputs[0], int(info.reduce_op), len(info.axes))
            out += b"".join(struct.pack("<I", a) for a in info.axes)
        else:
            raise AssertionError(k)
    return bytes(out)


CASES = ref_graphs.all_cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_documented_layout_is_what_the_library_reads(case):
    blob = write_like_the_shim(case.graph)
    assert blob == case.graph.to_bytes()
    lib = _lib.load()
    handle = ctypes.c_void_p()
    assert lib.kn_graph_from_blob(blob, len(blob), ctypes.byref(handle)) == 0, lib.kn_last_error()
    n_in, n_out, n_values = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert lib.kn_graph_io_count(handle, ctypes.byref(n_in), ctypes.byref(n_out), ctypes.byref(n_values)) == 0
    assert (n_in.value, n_out.value, n_values.value) == (len(case.graph.inputs), len(case.graph.outputs), len(case.graph.values))
    lib.kn_graph_destroy(handle)
