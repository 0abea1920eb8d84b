"""ctypes loader for `libkn_b200.so` (declared in include/kn_b200.h).

There is no fallback: if the library has not been built, importing the executor fails with an
instruction to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p)

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libkn_b200.so")

KN_MAX_RANK = 8
KN_OK = 0
STATUS_NAMES = {0: "KN_OK", 1: "KN_ERR_INVALID_ARG", 2: "KN_ERR_BAD_GRAPH", 3: "KN_ERR_UNSUPPORTED", 4: "KN_ERR_CUDA",
                5: "KN_ERR_SHAPE", 6: "KN_ERR_NO_DEVICE", 7: "KN_ERR_INTERNAL"}
KN_MATH_TF32 = 0
KN_MATH_F32 = 1
KN_FLAG_NO_CONV_CHAIN = 1
KN_FLAG_NO_PERSISTENT_GEMM = 2
KN_FLAG_TRACE_GEMM = 4


class KnOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("math_mode", c_int32), ("use_cuda_graph", c_int32), ("flags", c_int32)]


class KnTensorInfo(Structure):
    _fields_ = [("dtype", c_int32), ("rank", c_int32), ("dims", c_int64 * KN_MAX_RANK), ("bytes", c_uint64)]


class KnMemUsage(Structure):
    _fields_ = [("dedicated_bytes", c_uint64), ("shared_bytes", c_uint64), ("zero_bytes", c_uint64),
                ("hypo_peak_bytes", c_uint64), ("hypo_total_bytes", c_uint64)]


# name -> (restype, argtypes); one entry per function declared in include/kn_b200.h
SIGNATURES = {
    "kn_last_error": (c_char_p, []),
    "kn_version": (c_int, []),
    "kn_options_default": (c_int, [POINTER(KnOptions)]),
    "kn_device_count": (c_int, [POINTER(c_int)]),
    "kn_graph_from_blob": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "kn_graph_destroy": (None, [c_void_p]),
    "kn_graph_io_count": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "kn_plan_describe": (c_int, [c_void_p, c_size_t, POINTER(KnOptions), c_void_p, c_size_t, POINTER(c_size_t)]),
    "kn_executor_create": (c_int, [c_int, c_void_p, c_size_t, POINTER(KnOptions), POINTER(c_void_p)]),
    "kn_executor_destroy": (None, [c_void_p]),
    "kn_executor_io_count": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int)]),
    "kn_executor_io_info": (c_int, [c_void_p, c_int, c_int, POINTER(KnTensorInfo)]),
    "kn_executor_evaluate": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p)]),
    "kn_executor_evaluate_begin": (c_int, [c_void_p, POINTER(c_void_p)]),
    "kn_executor_evaluate_end": (c_int, [c_void_p, POINTER(c_void_p)]),
    "kn_executor_run_async": (c_int, [c_void_p]),
    "kn_executor_synchronize": (c_int, [c_void_p]),
    "kn_executor_stream": (c_int, [c_void_p, POINTER(c_void_p)]),
    "kn_executor_host_buffer": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p), POINTER(c_uint64)]),
    "kn_executor_device_buffer": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p), POINTER(c_uint64)]),
    "kn_executor_upload_inputs": (c_int, [c_void_p]),
    "kn_executor_download_outputs": (c_int, [c_void_p]),
    "kn_executor_mem_usage": (c_int, [c_void_p, POINTER(KnMemUsage)]),
    "kn_executor_step_count": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int)]),
    "kn_executor_set_profile": (c_int, [c_void_p, c_int]),
    "kn_executor_last_profile": (c_int, [c_void_p, c_void_p, c_size_t, POINTER(c_size_t)]),
    "kn_executor_time_step": (c_int, [c_void_p, c_int, c_int, POINTER(ctypes.c_float)]),
    "kn_nccl_load": (c_int, [c_char_p]),
    "kn_comm_unique_id": (c_int, [c_void_p, c_size_t]),
    "kn_comm_create": (c_int, [c_int, c_int, c_int, c_void_p, c_size_t, POINTER(c_void_p)]),
    "kn_comm_destroy": (None, [c_void_p]),
    "kn_executor_set_comm": (c_int, [c_void_p, c_void_p]),
    "kn_executor_selftest_wait_expiry": (c_int, [c_void_p, c_uint32]),
    "kn_matmul_tf32_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "kn_matmul_tf32_static_status": (c_int, [POINTER(c_int)]),
    "kn_strided_shape": (c_int, [c_int, c_int, POINTER(c_int64), POINTER(c_int64), c_int, POINTER(c_int64), POINTER(c_int),
                                 POINTER(c_int64), POINTER(c_int64), POINTER(c_int), POINTER(c_int)]),
    "kn_scalar_unary": (c_int, [c_int, c_int, c_int, c_uint64, POINTER(c_uint64)]),
    "kn_scalar_binary": (c_int, [c_int, c_int, c_uint64, c_uint64, POINTER(c_uint64)]),
}

_lib = None


class KnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m kyanite_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError if the library does not export it
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int):
    if status != KN_OK:
        raise KnError(status, load().kn_last_error().decode("utf-8", "replace"))
