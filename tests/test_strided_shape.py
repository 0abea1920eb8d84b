"""The shape / stride algebra of device tensors (kyanite_b200/csrc/strided.cpp) against the cases the reference
pins its own `StridedShape` with (kn-cuda-eval/src/shape.rs:346-431), replayed as numbers through the host-only
`kn_strided_shape` entry point, plus flip / permute / broadcast cases checked against numpy's own strides."""
import ctypes

import numpy as np
import pytest

from kyanite_b200 import _lib

NOTHING, VIEW, SLICE, FLIP, PERMUTE, BROADCAST = range(6)


def run(op, shape, strides, args=()):
    lib = _lib.load()
    arr = lambda xs: (ctypes.c_int64 * max(1, len(xs)))(*xs)
    out_rank, simple, dense = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    out_shape, out_strides = (ctypes.c_int64 * 16)(), (ctypes.c_int64 * 16)()
    status = lib.kn_strided_shape(op, len(shape), arr(shape), arr(strides), len(args), arr(args), ctypes.byref(out_rank), out_shape,
                                  out_strides, ctypes.byref(simple), ctypes.byref(dense))
    if status != 0:
        return status
    n = out_rank.value
    return list(out_shape[:n]), list(out_strides[:n]), bool(simple.value), bool(dense.value)


def test_properties():
    # shape.rs:351-371
    assert run(NOTHING, [2, 3], [3, 1])[2:] == (True, True)
    assert run(NOTHING, [3, 2], [1, 3])[2:] == (False, True)
    assert run(NOTHING, [3, 2], [8, 10])[2:] == (False, False)
    assert run(NOTHING, [2, 3], [3, -1])[2:] == (False, True)


def test_view_cases_of_the_reference():
    # rank zero (shape.rs:384-392)
    assert run(VIEW, [], [], [1, 1, 1])[:2] == ([1, 1, 1], [1, 1, 1])
    # size zero (shape.rs:394-400)
    assert run(VIEW, [2, 3, 0, 5], [0, 0, 0, 2], [0])[:2] == ([0], [1])
    assert run(VIEW, [2, 3, 0, 5], [0, 0, 0, 2], [12, 0])[:2] == ([12, 0], [0, 1])
    # simple strides merge into anything (shape.rs:402-413)
    shape, strides = [2, 3, 4, 3, 2], [72, 24, 6, 2, 1]
    assert run(NOTHING, shape, strides)[2] is True
    assert run(VIEW, shape, strides, [144])[:2] == ([144], [1])
    assert run(VIEW, shape, strides, [72, 2])[:2] == ([72, 2], [2, 1])
    assert run(VIEW, shape, strides, [72, 2, 1, 1, 1])[:2] == ([72, 2, 1, 1, 1], [2, 1, 1, 1, 1])
    # two contiguous groups can be kept apart but not merged (shape.rs:415-421)
    assert run(VIEW, [2, 3, 4], [24, 8, 1], [6, 4])[:2] == ([6, 4], [8, 1])
    assert run(VIEW, [2, 3, 4], [24, 8, 1], [24]) == 5       # KN_ERR_SHAPE: the reference's ViewError


def test_slice_case_of_the_reference():
    # shape.rs:423-430
    assert run(SLICE, [2, 3, 4], [24, 8, 1], [1, 0, 4, 2])[:2] == ([2, 2, 4], [24, 16, 1])


def np_strides(a):
    return [s // a.itemsize for s in a.strides]


def same(result, array, zero_axis=None):
    """Shapes equal, strides equal on every axis longer than one element (the stride of a one-element axis is never
    used, and numpy and the library choose different placeholders for it)."""
    assert not isinstance(result, int), f"status {result}"
    shape, strides = result[:2]
    assert shape == list(array.shape)
    for d, (mine, theirs) in enumerate(zip(strides, np_strides(array))):
        if shape[d] > 1:
            assert mine == theirs, (d, strides, np_strides(array))


@pytest.mark.parametrize("seed", range(6))
def test_against_numpy_strides(seed):
    r = np.random.Generator(np.random.PCG64(seed))
    shape = [int(x) for x in r.integers(1, 5, size=4)]
    base = np.zeros(shape, np.float32)
    strides = np_strides(base)
    perm = [int(x) for x in r.permutation(4)]
    same(run(PERMUTE, shape, strides, perm), base.transpose(perm))
    axis = int(r.integers(0, 4))
    same(run(FLIP, shape, strides, [axis]), np.flip(base, axis))
    start, step = int(r.integers(0, shape[axis])), int(r.integers(1, 3))
    sliced = base[tuple(slice(start, None, step) if d == axis else slice(None) for d in range(4))]
    # (the reference's SliceRange wants (end - start) % step == 0: the end is the one past the last element taken)
    same(run(SLICE, shape, strides, [axis, start, start + step * sliced.shape[axis], step]), sliced)
    assert run(SLICE, [6], [1], [0, 0, 5, 2]) == 5
    ones = list(shape)
    ones[axis] = 1
    small = np.zeros(ones, np.float32)
    same(run(BROADCAST, ones, np_strides(small), shape), np.broadcast_to(small, shape))
    # a view that numpy can make without a copy, the library can make too, with the same strides
    same(run(VIEW, shape, strides, [shape[0] * shape[1], shape[2], shape[3]]), base.reshape(shape[0] * shape[1], shape[2], shape[3]))
    # and a transposed tensor cannot be flattened
    if shape[0] > 1 and shape[1] > 1:
        t = base.transpose(1, 0, 2, 3)
        assert run(VIEW, list(t.shape), np_strides(t), [int(np.prod(shape))]) == 5


def test_arguments_are_checked():
    assert run(7, [2], [1]) == 1
    assert run(FLIP, [2, 3], [3, 1], [2]) == 1
    assert run(VIEW, [2, 3], [3, 1], [5]) == 1
    assert run(PERMUTE, [2, 3], [3, 1], [0, 0]) == 1
    assert run(BROADCAST, [2, 3], [3, 1], [4, 3]) == 1
