"""B200-native CUDA executor for Kyanite's graph IR.

`graph` holds the input format (IR builder + wire format); `executor` mirrors the reference's
`CudaExecutor` / `Device::prepare` interface over the C ABI declared in include/kn_b200.h.
"""
from .graph import (BATCH, BinaryOp, DType, Graph, OpKind, ReduceOp, Size, SliceRange, UnaryOp, Value, shape)

__all__ = ["BATCH", "BinaryOp", "DType", "Graph", "OpKind", "ReduceOp", "Size", "SliceRange", "UnaryOp", "Value",
           "shape"]
