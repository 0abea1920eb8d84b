"""The C-ABI library loads without a GPU and exports every function include/kn_b200.h declares;
host-only entry points behave (error codes, plan description, element semantics)."""
import ctypes
import os
import re

import numpy as np
import pytest

from kyanite_b200 import _lib
from kyanite_b200.executor import KnError, plan_describe
from kyanite_b200.graph import BATCH, BinaryOp, DType, Graph, UnaryOp, shape

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "kn_b200.h")).read()
    return sorted(set(re.findall(r"KN_API[^;(]*?\b(kn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    assert declared_functions() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_functions():
        assert getattr(lib, name) is not None
    assert lib.kn_version() >= 1000


def test_bad_blob_is_an_error_not_a_crash():
    lib = _lib.load()
    out = ctypes.c_void_p()
    status = lib.kn_graph_from_blob(b"nonsense-nonsense-nonsense", 26, ctypes.byref(out))
    assert status == 2 and not out.value
    assert b"magic" in lib.kn_last_error()
    # truncated real graph
    g = Graph()
    x = g.input(shape(BATCH, 4))
    g.output(g.unary(UnaryOp.EXP, x))
    blob = g.to_bytes()
    for cut in (len(blob) - 1, len(blob) // 2, 17):
        status = lib.kn_graph_from_blob(blob[:cut], cut, ctypes.byref(out))
        assert status == 2 and not out.value
    with pytest.raises(KnError):
        plan_describe(blob + b"x", 1)


def test_constant_sizes_that_wrap_are_refused():
    """A constant's byte count and shape factors come from the blob; values chosen so that a 64-bit sum or
    product wraps must not pass the size checks."""
    import struct
    lib = _lib.load()
    out = ctypes.c_void_p()

    def blob_with_constant(factors, byte_count, payload):
        b = bytearray(b"KNG1") + struct.pack("<III", 1, 0, 1) + struct.pack("<I", 0)
        b += struct.pack("<BBH", 1, 0, len(factors))        # CONSTANT, f32
        for f in factors:
            b += struct.pack("<QI", f, 0)
        b += struct.pack("<Q", byte_count) + payload
        return bytes(b)

    good = blob_with_constant([2], 8, b"\0" * 8)
    assert lib.kn_graph_from_blob(good, len(good), ctypes.byref(out)) == 0
    lib.kn_graph_destroy(out)
    cases = [
        blob_with_constant([2], 2**64 - 4, b"\0" * 8),            # position + count wraps
        blob_with_constant([2**62, 2**2 + 0, 2], 8, b"\0" * 8),   # product of factors wraps to 0 elements x 4... then 8
        blob_with_constant([2**63, 2, 2], 8, b"\0" * 8),          # 2^65 elements wraps to 0
        blob_with_constant([2**62 + 2], 8, b"\0" * 8),            # elements x 4 bytes wraps to 8
    ]
    for bad in cases:
        out = ctypes.c_void_p()
        assert lib.kn_graph_from_blob(bad, len(bad), ctypes.byref(out)) == 2
        assert not out.value


def test_null_arguments():
    lib = _lib.load()
    assert lib.kn_graph_from_blob(None, 0, None) == 1
    assert lib.kn_executor_run_async(None) == 1
    assert lib.kn_executor_io_count(None, None, None) == 1
    lib.kn_graph_destroy(None)
    lib.kn_executor_destroy(None)


def test_options_struct_size_is_checked():
    lib = _lib.load()
    g = Graph()
    g.output(g.input(shape(2)))
    h = ctypes.c_void_p()
    blob = g.to_bytes()
    assert lib.kn_graph_from_blob(blob, len(blob), ctypes.byref(h)) == 0
    opts = _lib.KnOptions()
    lib.kn_options_default(ctypes.byref(opts))
    opts.struct_size = 3
    needed = ctypes.c_size_t()
    assert lib.kn_plan_describe(h, 1, ctypes.byref(opts), None, 0, ctypes.byref(needed)) == 1
    lib.kn_graph_destroy(h)


def _bits(x):
    x = np.asarray(x)
    if x.dtype == np.bool_:
        return int(bool(x))
    if x.dtype.kind == "i":
        return int(x) & 0xFFFFFFFFFFFFFFFF
    if x.dtype.kind == "u":
        return int(x)
    return int(x.reshape(1).view({2: np.uint16, 4: np.uint32, 8: np.uint64}[x.dtype.itemsize])[0])


def _from_bits(b, np_dtype):
    np_dtype = np.dtype(np_dtype)
    if np_dtype == np.bool_:
        return np.bool_(b != 0)
    if np_dtype.kind in "iu":
        return np.array([b & ((1 << (8 * np_dtype.itemsize)) - 1)], dtype=np.uint64).astype(
            {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[np_dtype.itemsize]).view(np_dtype)[0]
    u = {2: np.uint16, 4: np.uint32, 8: np.uint64}[np_dtype.itemsize]
    return np.array([b & ((1 << (8 * np_dtype.itemsize)) - 1)], dtype=np.uint64).astype(u).view(np_dtype)[0]


CAST_VALUES = {
    DType.F32: [0.0, -0.0, 0.5, -0.5, 1.9, -1.9, 127.0, 128.0, 255.9, 300.7, -300.7, 65536.0, -3.0e9, 3.0e9, 1.0e19,
                -1.0e19, 3.0e38, -3.0e38, np.inf, -np.inf, np.nan],
    DType.F64: [0.0, 1.5, -2.5, 1e10, -1e10, 1e300, np.nan],
    DType.I8: [0, 1, -1, 127, -128], DType.I32: [0, 1, -1, 2 ** 31 - 1, -2 ** 31, 70000],
    DType.I64: [0, -1, 2 ** 63 - 1, -2 ** 63, 2 ** 53 + 1], DType.U8: [0, 1, 255],
    DType.U32: [0, 1, 2 ** 32 - 1], DType.U64: [0, 1, 2 ** 64 - 1, 2 ** 63], DType.BOOL: [False, True],
    DType.F16: [0.0, 1.0, -2.5, 65504.0, 6e-8, np.inf],
}


def test_value_cast_semantics_match_the_oracle():
    """dtype.rs:323-355 through both implementations, including saturation and wrap-around."""
    from oracle.cpu_eval import value_cast
    lib = _lib.load()
    for src, values in CAST_VALUES.items():
        for v in values:
            x = np.asarray(v, dtype=src.np)
            for dst in DType:
                out = ctypes.c_uint64()
                assert lib.kn_scalar_unary(int(UnaryOp.VALUE_CAST), int(src), int(dst), _bits(x), ctypes.byref(out)) == 0
                got = _from_bits(out.value, dst.np)
                want = value_cast(x.reshape(1), dst.np)[0]
                same = (got == want) or (np.isnan(got) and np.isnan(want)) if dst.is_float else got == want
                assert same, f"cast {src.name}->{dst.name} of {v}: got {got}, oracle {want}"


def test_unary_and_binary_semantics_match_the_oracle():
    from oracle import cpu_eval
    lib = _lib.load()
    vals = np.array([0.0, -0.0, 0.1, -1.5, 2.0, 20.0, -100.0, 1000.0, np.inf, -np.inf, np.nan], dtype=np.float32)
    for op in UnaryOp:
        if op in (UnaryOp.VALUE_CAST, UnaryOp.BIT_CAST):
            continue
        want = cpu_eval.unary(int(op), 0xFF, vals)
        for x, w in zip(vals, want):
            out = ctypes.c_uint64()
            assert lib.kn_scalar_unary(int(op), 0, 0, _bits(x), ctypes.byref(out)) == 0
            g = _from_bits(out.value, np.float32)
            assert (np.isnan(g) and np.isnan(w)) or g == w or abs(g - w) <= 2e-6 * max(1.0, abs(w)), (op, x, g, w)
    ints = np.array([0, 1, -1, 7, -7, 127, -128], dtype=np.int8)
    for op in BinaryOp:
        if op == BinaryOp.POW:
            continue
        for a in ints:
            for b in ints:
                if op == BinaryOp.DIV and b == 0:
                    continue
                want = cpu_eval.binary(int(op), np.array([a]), np.array([b]))[0]
                out = ctypes.c_uint64()
                assert lib.kn_scalar_binary(int(op), int(DType.I8), _bits(a), _bits(b), ctypes.byref(out)) == 0
                assert _from_bits(out.value, np.int8) == want, (op, a, b)
    for op in BinaryOp:
        for a in vals:
            for b in vals:
                want = cpu_eval.binary(int(op), np.array([a]), np.array([b]))[0]
                out = ctypes.c_uint64()
                assert lib.kn_scalar_binary(int(op), 0, _bits(a), _bits(b), ctypes.byref(out)) == 0
                g = _from_bits(out.value, np.float32)
                ok = (np.isnan(g) and np.isnan(want)) or g == want or abs(g - want) <= 1e-6 * abs(want)
                assert ok, (op, a, b, g, want)
    for op in (BinaryOp.ADD, BinaryOp.SUB, BinaryOp.MUL, BinaryOp.DIV, BinaryOp.MIN, BinaryOp.MAX):
        for a in (False, True):
            for b in (False, True):
                want = cpu_eval.binary(int(op), np.array([a]), np.array([b]))[0]
                out = ctypes.c_uint64()
                assert lib.kn_scalar_binary(int(op), int(DType.BOOL), int(a), int(b), ctypes.byref(out)) == 0
                assert bool(out.value) == bool(want), (op, a, b)


def test_f16_round_trip_matches_numpy():
    lib = _lib.load()
    r = np.random.Generator(np.random.PCG64(3))
    xs = np.concatenate([r.standard_normal(2000).astype(np.float32) * 10.0 ** r.integers(-9, 6, 2000),
                         np.array([65504.0, 65519.9, 65520.0, 5.96e-8, 2.98e-8, 2.9802325e-08, 6.1e-5, 0.0], np.float32)]).astype(np.float32)
    for x in xs:
        out = ctypes.c_uint64()
        assert lib.kn_scalar_unary(int(UnaryOp.VALUE_CAST), int(DType.F32), int(DType.F16), _bits(x), ctypes.byref(out)) == 0
        with np.errstate(over="ignore"):
            want = np.float32(x).astype(np.float16)
        assert out.value == int(want.reshape(1).view(np.uint16)[0]), x
        back = ctypes.c_uint64()
        assert lib.kn_scalar_unary(int(UnaryOp.VALUE_CAST), int(DType.F16), int(DType.F32), out.value, ctypes.byref(back)) == 0
        assert _from_bits(back.value, np.float32) == np.float32(want) or np.isnan(want)
