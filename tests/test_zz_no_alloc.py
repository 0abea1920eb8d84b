"""`kn_matmul_tf32_static`: the matmul for hosts that may not allocate device memory (a serving loop
with a fixed footprint, a plugin inside a runtime that owns the whole device).  It keeps the split-K
partial sums in an array that is part of the library's device module.  The tests call it through the
C ABI on caller-owned device buffers and compare the result
  - with numpy's `a @ b.T` computed in f64 (independent of any CUDA code), for shapes that take every
    branch of the entry point: ragged m, more than 256 columns (128-wide column tiles), a column count
    that is not a multiple of 4 (scalar stores), a K tail (k not a multiple of 32), one K slice only, and
    a two-stage pipeline under a 128-wide staged tile,
  - with the executor's own split-K matmul (the existing entry point for the same product) on the same
    operands, twice in a row with different data (the array keeps the previous call's contents),
under the tolerance the tensor-core tests use (abs >= 4e-3 * |expected|max AND rel >= 4e-3 is a mismatch).
After the calls the status word of `kn_matmul_tf32_static_status` must read 0.
Collected last on purpose: a failure here stops a `-x` run only after every other test has run."""
import ctypes

import numpy as np
import pytest

from kyanite_b200 import _lib
from kyanite_b200.executor import MATH_TF32, CudaExecutor, plan_describe
from kyanite_b200.graph import Graph, shape
from oracle.cpu_eval import assert_tensors_match

pytestmark = pytest.mark.gpu

M, N, K = 256, 192, 2048


def static_slices(m, n, k):
    """The slicing rule stated in include/kn_b200.h."""
    bn = 128 if n > 256 else min(256, (n + 15) // 16 * 16)
    tiles = ((m + 127) // 128) * ((n + bn - 1) // bn)
    k_blocks = (k + 31) // 32
    s = max(1, min(k_blocks // 4, (96 + tiles - 1) // tiles, 32))
    per_slice = (k_blocks + s - 1) // s
    return (k_blocks + per_slice - 1) // per_slice


def _executor_matmul(a, b):
    m, k = a.shape
    n = b.shape[0]
    g = Graph()
    x = g.input(shape(1, m, k))
    w = g.input(shape(1, n, k))
    g.output(g.batched_mat_mul(x, g.permute(w, [0, 2, 1])))
    assert "splitk=" in plan_describe(g, 0, math_mode=MATH_TF32)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        return ex.evaluate([a[None], b[None]])[0][0]


def _static_matmul(a, b):
    import torch
    lib = _lib.load()
    torch.cuda.set_device(0)
    m, k = a.shape
    n = b.shape[0]
    a_dev = torch.from_numpy(a).cuda()
    b_dev = torch.from_numpy(b).cuda()
    c_dev = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    status = lib.kn_matmul_tf32_static(a_dev.data_ptr(), b_dev.data_ptr(), c_dev.data_ptr(), m, n, k, stream)
    assert status == 0, lib.kn_last_error()
    torch.cuda.synchronize()
    return c_dev.cpu().numpy()


def _status_word():
    code = ctypes.c_int(-1)
    assert _lib.load().kn_matmul_tf32_static_status(ctypes.byref(code)) == 0, _lib.load().kn_last_error()
    return code.value


def test_static_scratch_matmul_matches_executor():
    for seed in (1, 2):   # second call: the scratch array still holds the first call's partial sums
        r = np.random.Generator(np.random.PCG64(seed))
        a = r.standard_normal((M, K)).astype(np.float32)
        b = r.standard_normal((N, K)).astype(np.float32)
        got = _static_matmul(a, b)
        want = _executor_matmul(a, b)
        assert_tensors_match([want], [got], tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)
        exact = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)
        assert_tensors_match([exact], [got], tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)
    assert _status_word() == 0


SHAPES = {
    "ragged_m": (200, 192, 1024),
    "wide_n_128_column_tiles": (128, 384, 512),
    "n_not_multiple_of_4": (130, 50, 512),
    "k_tail": (128, 64, 292),
    "one_slice": (256, 96, 96),
    "two_stages_under_a_wide_tile": (128, 128, 64),
    "large_after_small": (256, 256, 2048),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_static_scratch_matmul_matches_numpy(name):
    m, n, k = SHAPES[name]
    if name == "one_slice" or name == "two_stages_under_a_wide_tile":
        assert static_slices(m, n, k) == 1
    else:
        assert static_slices(m, n, k) > 1
    r = np.random.Generator(np.random.PCG64(len(name)))
    a = r.standard_normal((m, k)).astype(np.float32)
    b = r.standard_normal((n, k)).astype(np.float32)
    exact = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)
    for _ in range(2):
        got = _static_matmul(a, b)
        assert_tensors_match([exact], [got], tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)
    assert _status_word() == 0


def test_static_scratch_limits_are_reported():
    import torch
    lib = _lib.load()
    torch.cuda.set_device(0)
    buf = torch.zeros(1024, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    # 32 slices x 4096 x 4096 partial sums are far beyond the 8 MiB array: refused before any launch
    assert static_slices(4096, 4096, 8192) * 4096 * 4096 * 4 > 8 << 20
    assert lib.kn_matmul_tf32_static(p, p, p, 4096, 4096, 8192, None) == 3
    assert b"static scratch" in lib.kn_last_error()
    assert lib.kn_matmul_tf32_static(p, p, p, 128, 128, 130, None) == 3      # k not a multiple of 4
    assert lib.kn_matmul_tf32_static(None, p, p, 128, 128, 128, None) == 1   # null operand
    assert lib.kn_matmul_tf32_static_status(None) == 1
    torch.cuda.synchronize()
    assert _status_word() == 0
