"""Host-side mirror of the reference's executor interface, over the C ABI.

    CudaDevice(0)                                   kn-cuda-sys/src/wrapper/handle.rs:38-48
    CudaExecutor(device, graph, batch_size)         kn-cuda-eval/src/executor.rs:61
    executor.evaluate(inputs) -> outputs            kn-cuda-eval/src/executor.rs:117
    executor.run_async()                            kn-cuda-eval/src/executor.rs:199
    Device.cuda(0).prepare(graph, batch).eval(...)  kn-runtime/src/lib.rs:85,120

Same names, argument meaning and error behaviour: wrong input count, shape or dtype raises
(the reference asserts, executor.rs:118-127); a missing device raises `CudaDeviceNotAvailable`.
Everything numerical happens inside `libkn_b200.so`; numpy only carries host buffers.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_size_t, c_uint64, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import KnError, KnMemUsage, KnOptions, KnTensorInfo, check
from .graph import DType, Graph

__all__ = ["Communicator", "CudaDevice", "CudaDeviceNotAvailable", "CudaExecutor", "Device", "PreparedGraph", "MemoryUsage",
           "plan_describe", "KnError", "MATH_TF32", "MATH_F32", "FLAG_NO_CONV_CHAIN", "FLAG_NO_PERSISTENT_GEMM"]

MATH_TF32 = _lib.KN_MATH_TF32
MATH_F32 = _lib.KN_MATH_F32
FLAG_NO_CONV_CHAIN = _lib.KN_FLAG_NO_CONV_CHAIN
FLAG_NO_PERSISTENT_GEMM = _lib.KN_FLAG_NO_PERSISTENT_GEMM


class CudaDeviceNotAvailable(RuntimeError):
    pass


def _options(math_mode: Optional[int], use_cuda_graph: Optional[bool], flags: int = 0) -> KnOptions:
    opts = KnOptions()
    check(_lib.load().kn_options_default(byref(opts)))
    opts.flags = int(flags)
    if math_mode is not None:
        opts.math_mode = int(math_mode)
    if use_cuda_graph is not None:
        opts.use_cuda_graph = 1 if use_cuda_graph else 0
    return opts


class _GraphHandle:
    def __init__(self, graph):
        blob = graph if isinstance(graph, (bytes, bytearray)) else graph.to_bytes()
        self.ptr = c_void_p()
        if isinstance(blob, bytes):
            buf = ctypes.c_char_p(blob)          # the library copies the blob: no second copy here
        else:
            buf = (ctypes.c_char * len(blob)).from_buffer(blob)
        check(_lib.load().kn_graph_from_blob(ctypes.cast(buf, c_void_p), len(blob), byref(self.ptr)))

    def close(self):
        if self.ptr:
            _lib.load().kn_graph_destroy(self.ptr)
            self.ptr = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def plan_describe(graph, batch_size: int, math_mode: Optional[int] = None, flags: int = 0) -> str:
    """Text dump of the planned step list; needs no GPU."""
    lib = _lib.load()
    h = _GraphHandle(graph)
    try:
        opts = _options(math_mode, None, flags)
        needed = c_size_t()
        check(lib.kn_plan_describe(h.ptr, batch_size, byref(opts), None, 0, byref(needed)))
        buf = ctypes.create_string_buffer(needed.value + 1)
        check(lib.kn_plan_describe(h.ptr, batch_size, byref(opts), buf, needed.value + 1, byref(needed)))
        return buf.value.decode()
    finally:
        h.close()


@dataclass(frozen=True)
class CudaDevice:
    index: int = 0

    def __post_init__(self):
        if not (0 <= self.index < CudaDevice.device_count()):
            raise CudaDeviceNotAvailable(f"CUDA device {self.index} not available")

    @staticmethod
    def device_count() -> int:
        n = c_int()
        check(_lib.load().kn_device_count(byref(n)))
        return n.value

    @staticmethod
    def all() -> List["CudaDevice"]:
        return [CudaDevice(i) for i in range(CudaDevice.device_count())]


@dataclass
class MemoryUsage:
    dedicated_bytes: int
    shared_bytes: int
    zero_bytes: int
    hypo_peak_bytes: int
    hypo_total_bytes: int


def bundled_nccl_path() -> Optional[str]:
    """Path of the NCCL library that ships with the Python environment (the `nvidia-nccl` wheel), if any."""
    import importlib.util
    import os
    spec = importlib.util.find_spec("nvidia")
    for root in (spec.submodule_search_locations if spec and spec.submodule_search_locations else []):
        path = os.path.join(root, "nccl", "lib", "libnccl.so.2")
        if os.path.exists(path):
            return path
    return None


class Communicator:
    """One rank of an NCCL communicator for the all-reduce steps of tensor-parallel graphs
    (kn_comm_unique_id / kn_comm_create).  Rank 0 makes the id with `Communicator.unique_id()` and the host
    program sends the 128 bytes to the other ranks; every rank then constructs its `Communicator`, which
    returns once all ranks have."""

    def __init__(self, device: int, rank: int, world: int, unique_id: bytes):
        self._lib = _lib.load()
        self._ptr = c_void_p()
        self.device, self.rank, self.world = int(device), int(rank), int(world)
        Communicator.load_library()
        buf = ctypes.create_string_buffer(bytes(unique_id), len(unique_id))
        check(self._lib.kn_comm_create(self.device, self.rank, self.world, ctypes.cast(buf, c_void_p), len(unique_id),
                                       byref(self._ptr)))

    @staticmethod
    def load_library(path: Optional[str] = None):
        lib = _lib.load()
        path = path or bundled_nccl_path()
        check(lib.kn_nccl_load(path.encode() if path else None))

    @staticmethod
    def unique_id() -> bytes:
        Communicator.load_library()
        buf = ctypes.create_string_buffer(128)
        check(_lib.load().kn_comm_unique_id(ctypes.cast(buf, c_void_p), 128))
        return buf.raw

    def close(self):
        if getattr(self, "_ptr", None):
            self._lib.kn_comm_destroy(self._ptr)
            self._ptr = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CudaExecutor:
    def __init__(self, device, graph, batch_size: int, math_mode: Optional[int] = None,
                 use_cuda_graph: Optional[bool] = None, flags: int = 0):
        self._lib = _lib.load()
        self._ptr = c_void_p()
        index = device.index if isinstance(device, CudaDevice) else int(device)
        self.device = index
        self.batch_size = int(batch_size)
        h = _GraphHandle(graph)
        try:
            opts = _options(math_mode, use_cuda_graph, flags)
            status = self._lib.kn_executor_create(index, h.ptr, self.batch_size, byref(opts), byref(self._ptr))
            if status == 6:
                raise CudaDeviceNotAvailable(self._lib.kn_last_error().decode())
            check(status)
        finally:
            h.close()
        n_in, n_out = c_int(), c_int()
        check(self._lib.kn_executor_io_count(self._ptr, byref(n_in), byref(n_out)))
        self._in_info = [self._io_info(0, i) for i in range(n_in.value)]
        self._out_info = [self._io_info(1, i) for i in range(n_out.value)]
        self.host_inputs = [self._host_array(0, i) for i in range(n_in.value)]
        self.host_outputs = [self._host_array(1, i) for i in range(n_out.value)]

    # ---------------------------------------------------------------- info
    def _io_info(self, is_output: int, index: int):
        info = KnTensorInfo()
        check(self._lib.kn_executor_io_info(self._ptr, is_output, index, byref(info)))
        shape = tuple(info.dims[d] for d in range(info.rank))
        return shape, DType(info.dtype), int(info.bytes)

    def _host_array(self, is_output: int, index: int) -> np.ndarray:
        """numpy view of the pinned staging buffer (no copy)."""
        shape, dtype, nbytes = (self._out_info if is_output else self._in_info)[index]
        ptr, size = c_void_p(), c_uint64()
        check(self._lib.kn_executor_host_buffer(self._ptr, is_output, index, byref(ptr), byref(size)))
        if nbytes == 0:
            return np.zeros(shape, dtype=dtype.np)
        raw = (ctypes.c_uint8 * nbytes).from_address(ptr.value)
        return np.frombuffer(raw, dtype=dtype.np).reshape(shape)

    @property
    def input_shapes(self):
        return [s for s, _, _ in self._in_info]

    @property
    def output_shapes(self):
        return [s for s, _, _ in self._out_info]

    @property
    def mem_usage(self) -> MemoryUsage:
        u = KnMemUsage()
        check(self._lib.kn_executor_mem_usage(self._ptr, byref(u)))
        return MemoryUsage(u.dedicated_bytes, u.shared_bytes, u.zero_bytes, u.hypo_peak_bytes, u.hypo_total_bytes)

    def step_count(self):
        steps, launches = c_int(), c_int()
        check(self._lib.kn_executor_step_count(self._ptr, byref(steps), byref(launches)))
        return steps.value, launches.value

    def device_buffer(self, is_output: bool, index: int):
        ptr, size = c_void_p(), c_uint64()
        check(self._lib.kn_executor_device_buffer(self._ptr, int(is_output), index, byref(ptr), byref(size)))
        return ptr.value, size.value

    def stream(self) -> int:
        s = c_void_p()
        check(self._lib.kn_executor_stream(self._ptr, byref(s)))
        return s.value or 0

    # ---------------------------------------------------------------- running
    def evaluate(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        """Copies inputs to the device, runs the graph, returns fresh host arrays."""
        if len(inputs) != len(self._in_info):
            raise ValueError(f"Wrong input count, expected {len(self._in_info)} but got {len(inputs)}")
        arrays = []
        for i, (x, (shape, dtype, _)) in enumerate(zip(inputs, self._in_info)):
            x = np.asarray(x)
            if tuple(x.shape) != shape:
                raise ValueError(f"Wrong shape for input {i}: expected {shape}, got {tuple(x.shape)}")
            if x.dtype != dtype.np:
                raise ValueError(f"Wrong dtype for input {i}: expected {dtype.np}, got {x.dtype}")
            if not x.flags.c_contiguous:
                x = x.copy(order="C")   # `as_standard_layout` (executor.rs:135)
            arrays.append(x)
        outs = [np.empty(shape, dtype=dtype.np) for shape, dtype, _ in self._out_info]
        in_ptrs = (c_void_p * max(1, len(arrays)))(*[a.ctypes.data for a in arrays])
        out_ptrs = (c_void_p * max(1, len(outs)))(*[o.ctypes.data for o in outs])
        check(self._lib.kn_executor_evaluate(self._ptr, in_ptrs, out_ptrs))
        return outs

    def evaluate_begin(self, inputs: Sequence[np.ndarray]):
        """First half of `evaluate` with caller-owned input arrays (C-contiguous, right shape and dtype; checked):
        the library copies them to its pinned staging, then enqueues upload, steps and download without
        waiting (kn_executor_evaluate_begin).  The arrays may be reused as soon as this returns."""
        if len(inputs) != len(self._in_info):
            raise ValueError(f"Wrong input count, expected {len(self._in_info)} but got {len(inputs)}")
        for i, (x, (shape, dtype, _)) in enumerate(zip(inputs, self._in_info)):
            if tuple(x.shape) != shape or x.dtype != dtype.np or not x.flags.c_contiguous:
                raise ValueError(f"input {i}: expected a C-contiguous {dtype.np} array of shape {shape}")
        in_ptrs = (c_void_p * max(1, len(inputs)))(*[a.ctypes.data if a.size else None for a in inputs])
        check(self._lib.kn_executor_evaluate_begin(self._ptr, in_ptrs))

    def evaluate_end(self) -> List[np.ndarray]:
        """Second half: waits for the evaluation started by `evaluate_begin` and returns the outputs as views
        of the executor's pinned staging, valid until the next evaluation (the reference's `evaluate`
        returns borrowed tensors too, kn-cuda-eval/src/executor.rs:194)."""
        return self.evaluate_staged_end()

    def evaluate_staged(self) -> List[np.ndarray]:
        """`evaluate` on the pinned staging buffers: the caller has filled `host_inputs` and reads
        `host_outputs` (valid until the next call); no extra host copies."""
        in_ptrs = (c_void_p * max(1, len(self.host_inputs)))(
            *[a.ctypes.data if a.size else None for a in self.host_inputs])
        out_ptrs = (c_void_p * max(1, len(self.host_outputs)))(
            *[a.ctypes.data if a.size else None for a in self.host_outputs])
        check(self._lib.kn_executor_evaluate(self._ptr, in_ptrs, out_ptrs))
        return self.host_outputs

    def evaluate_staged_begin(self):
        """First half of `evaluate_staged`: enqueue upload, steps and download, do not wait.  With two
        executors on one device, `b.evaluate_staged_begin(); a.evaluate_staged_end()` keeps the GPU and both
        copy engines busy (kn_executor_evaluate_begin / _end)."""
        in_ptrs = (c_void_p * max(1, len(self.host_inputs)))(
            *[a.ctypes.data if a.size else None for a in self.host_inputs])
        check(self._lib.kn_executor_evaluate_begin(self._ptr, in_ptrs))

    def evaluate_staged_end(self) -> List[np.ndarray]:
        out_ptrs = (c_void_p * max(1, len(self.host_outputs)))(
            *[a.ctypes.data if a.size else None for a in self.host_outputs])
        check(self._lib.kn_executor_evaluate_end(self._ptr, out_ptrs))
        return self.host_outputs

    def set_comm(self, comm: Optional["Communicator"]):
        """Attaches the communicator the graph's all-reduce values sum over (None: a world of one rank)."""
        check(self._lib.kn_executor_set_comm(self._ptr, comm._ptr if comm is not None else None))
        self._comm = comm   # keep it alive as long as the executor uses it

    def upload_inputs(self):
        check(self._lib.kn_executor_upload_inputs(self._ptr))

    def download_outputs(self):
        check(self._lib.kn_executor_download_outputs(self._ptr))

    def run_async(self):
        check(self._lib.kn_executor_run_async(self._ptr))

    def synchronize(self):
        check(self._lib.kn_executor_synchronize(self._ptr))

    # ---------------------------------------------------------------- profiling
    def set_profile(self, enable: bool):
        check(self._lib.kn_executor_set_profile(self._ptr, int(enable)))

    def last_profile(self) -> str:
        needed = c_size_t()
        check(self._lib.kn_executor_last_profile(self._ptr, None, 0, byref(needed)))
        buf = ctypes.create_string_buffer(needed.value + 1)
        check(self._lib.kn_executor_last_profile(self._ptr, buf, needed.value + 1, byref(needed)))
        return buf.value.decode()

    def time_step(self, step: int, launches: int = 20) -> float:
        """Average microseconds of one launch of step `step`, launched `launches` times back to back."""
        us = ctypes.c_float()
        check(self._lib.kn_executor_time_step(self._ptr, step, launches, byref(us)))
        return us.value

    def close(self):
        if getattr(self, "_ptr", None):
            self.host_inputs = []
            self.host_outputs = []
            self._lib.kn_executor_destroy(self._ptr)
            self._ptr = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class PreparedGraph:
    """kn-runtime/src/lib.rs:48-51,120-126"""

    def __init__(self, executor: CudaExecutor):
        self.executor = executor

    def eval(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        return self.executor.evaluate(inputs)


class Device:
    """kn-runtime/src/lib.rs:68-93.  Only the CUDA variant exists here: the CPU executor of the
    reference is not part of this library."""

    def __init__(self, cuda_device: CudaDevice):
        self.cuda_device = cuda_device

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        return Device(CudaDevice(index))

    @staticmethod
    def best() -> "Device":
        if CudaDevice.device_count() == 0:
            raise CudaDeviceNotAvailable("no CUDA device; this library has no CPU executor")
        return Device(CudaDevice(0))

    def prepare(self, graph: Graph, batch_size: int, **kwargs) -> PreparedGraph:
        return PreparedGraph(CudaExecutor(self.cuda_device, graph, batch_size, **kwargs))
