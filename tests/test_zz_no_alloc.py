"""`kn_matmul_tf32_static`: the matmul for hosts that may not allocate device memory (a serving loop
with a fixed footprint, a plugin inside a runtime that owns the whole device).  It keeps the split-K
partial sums in an array that is part of the library's device module.  The test calls it through the
C ABI on caller-owned device buffers, twice in a row with different data (the array keeps the previous
call's contents), and compares with the executor's own split-K matmul on the same operands, under the
tolerance the tensor-core tests use (abs >= 4e-3 * max(1, |expected|max) AND rel >= 4e-3 mismatches).
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


def _executor_matmul(a, b):
    g = Graph()
    x = g.input(shape(1, M, K))
    w = g.input(shape(1, N, K))
    g.output(g.batched_mat_mul(x, g.permute(w, [0, 2, 1])))
    assert "splitk=" in plan_describe(g, 0, math_mode=MATH_TF32)
    with CudaExecutor(0, g, 0, math_mode=MATH_TF32) as ex:
        return ex.evaluate([a[None], b[None]])[0][0]


def test_static_scratch_matmul_matches_executor():
    import torch
    lib = _lib.load()
    torch.cuda.set_device(0)
    c_dev = torch.empty((M, N), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for seed in (1, 2):   # second call: the scratch array still holds the first call's partial sums
        r = np.random.Generator(np.random.PCG64(seed))
        a = r.standard_normal((M, K)).astype(np.float32)
        b = r.standard_normal((N, K)).astype(np.float32)
        want = _executor_matmul(a, b)
        a_dev = torch.from_numpy(a).cuda()
        b_dev = torch.from_numpy(b).cuda()
        c_dev.fill_(float("nan"))
        status = lib.kn_matmul_tf32_static(a_dev.data_ptr(), b_dev.data_ptr(), c_dev.data_ptr(), M, N, K, stream)
        assert status == 0, lib.kn_last_error()
        torch.cuda.synchronize()
        got = c_dev.cpu().numpy()
        assert_tensors_match([want], [got], tol_abs=4e-3, tol_rel=4e-3, abs_scaled=True)
        # same kernels, same slicing: the two paths should agree far inside that tolerance
        assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want))


def test_static_scratch_limits_are_reported():
    import torch
    lib = _lib.load()
    torch.cuda.set_device(0)
    buf = torch.zeros(1024, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    # 32 slices x 4096 x 4096 partial sums are far beyond the 8 MiB array: refused before any launch
    assert lib.kn_matmul_tf32_static(p, p, p, 4096, 4096, 8192, None) == 3
    assert b"static scratch" in lib.kn_last_error()
    assert lib.kn_matmul_tf32_static(p, p, p, 128, 128, 130, None) == 3      # k not a multiple of 4
    assert lib.kn_matmul_tf32_static(None, p, p, 128, 128, 128, None) == 1   # null operand
    torch.cuda.synchronize()
