//! `serialize_graph`: walks `graph.values()` (kn-graph/src/graph.rs:391-394, topological order) and writes one
//! record per `ValueInfo` (graph.rs:95-101), covering all 16 `Operation` variants (graph.rs:106-162), in the
//! layout `kn_graph_from_blob` parses (kyanite_b200/csrc/ir.cpp).  A Rust `&Graph` cannot cross a C boundary;
//! this blob is how the graph reaches the library.
//!
//! Layout, little endian:
//!
//! ```text
//! header  b"KNG1", u32 value_count, u32 input_count, u32 output_count,
//!         input_count x u32 value index, output_count x u32 value index
//! value   u8 operation tag, u8 dtype tag, u16 rank, rank x (u64 fixed_factor, u32 batch_exp), then
//!   0  Input      u32 index
//!   1  Constant   u64 byte_count, the elements in standard (row-major) layout; Bool as one byte 0/1
//!   2  View       u32 input
//!   3  Broadcast  u32 input
//!   4  Permute    u32 input, rank x u32 permutation
//!   5  Slice      u32 input, u32 axis, u64 start, u64 end, u64 step
//!   6  Flip       u32 input, u32 axis
//!   7  Gather     u32 input, u32 axis, u32 indices
//!   8  Concat     u32 count, count x u32 input, u32 axis
//!   9  Conv       u32 input, u32 filter, u32 stride_y, u32 stride_x, u32 padding_y, u32 padding_x
//!   10 MatMul     u32 left, u32 right
//!   11 Unary      u32 input, u8 unary tag, u8 cast dtype tag (0xff unless ValueCast / BitCast)
//!   12 Binary     u32 left, u32 right, u8 binary tag
//!   13 Softmax    u32 input, u32 axis
//!   14 Layernorm  u32 input, u32 axis, f32 eps
//!   15 Reduce     u32 input, u8 reduce tag, u32 count, count x u32 axis
//! ```
//! (Tag 16, AllReduce: u32 input, is an extension the reference's `Graph` cannot express; only graphs built
//! for tensor-parallel execution contain it.)
//!
//! dtype tags are `DType`'s declaration order (kn-graph/src/dtype.rs:25-37); unary, binary and reduce tags are
//! the declaration orders of `UnaryOp`, `BinaryOp`, `ReduceOp` (graph.rs:172-217).
//!
//! Uncompiled source: the image this repository is built in has no Rust toolchain.

use kn_graph::dtype::{DTensor, DType};
use kn_graph::graph::{BinaryOp, Graph, Operation, ReduceOp, UnaryOp};

pub const OP_INPUT: u8 = 0;
pub const OP_CONSTANT: u8 = 1;
pub const OP_VIEW: u8 = 2;
pub const OP_BROADCAST: u8 = 3;
pub const OP_PERMUTE: u8 = 4;
pub const OP_SLICE: u8 = 5;
pub const OP_FLIP: u8 = 6;
pub const OP_GATHER: u8 = 7;
pub const OP_CONCAT: u8 = 8;
pub const OP_CONV: u8 = 9;
pub const OP_MATMUL: u8 = 10;
pub const OP_UNARY: u8 = 11;
pub const OP_BINARY: u8 = 12;
pub const OP_SOFTMAX: u8 = 13;
pub const OP_LAYERNORM: u8 = 14;
pub const OP_REDUCE: u8 = 15;

pub const DTYPE_F32: u8 = 0;
pub const DTYPE_F64: u8 = 1;
pub const DTYPE_I8: u8 = 2;
pub const DTYPE_I16: u8 = 3;
pub const DTYPE_I32: u8 = 4;
pub const DTYPE_I64: u8 = 5;
pub const DTYPE_U8: u8 = 6;
pub const DTYPE_U16: u8 = 7;
pub const DTYPE_U32: u8 = 8;
pub const DTYPE_U64: u8 = 9;
pub const DTYPE_BOOL: u8 = 10;

pub const UNARY_ABS: u8 = 0;
pub const UNARY_NEG: u8 = 1;
pub const UNARY_SIN: u8 = 2;
pub const UNARY_COS: u8 = 3;
pub const UNARY_EXP: u8 = 4;
pub const UNARY_LOG: u8 = 5;
pub const UNARY_SQRT: u8 = 6;
pub const UNARY_SIGMOID: u8 = 7;
pub const UNARY_TANH: u8 = 8;
pub const UNARY_ERF: u8 = 9;
pub const UNARY_MISH: u8 = 10;
pub const UNARY_SOFTPLUS: u8 = 11;
pub const UNARY_VALUE_CAST: u8 = 12;
pub const UNARY_BIT_CAST: u8 = 13;

pub const BINARY_ADD: u8 = 0;
pub const BINARY_SUB: u8 = 1;
pub const BINARY_MUL: u8 = 2;
pub const BINARY_DIV: u8 = 3;
pub const BINARY_MIN: u8 = 4;
pub const BINARY_MAX: u8 = 5;
pub const BINARY_POW: u8 = 6;

pub const REDUCE_SUM: u8 = 0;
pub const REDUCE_MEAN: u8 = 1;
pub const REDUCE_PROD: u8 = 2;
pub const REDUCE_MAX: u8 = 3;
pub const REDUCE_MIN: u8 = 4;

pub const NO_CAST: u8 = 0xff;

pub fn dtype_tag(dtype: DType) -> u8 {
    match dtype {
        DType::F32 => DTYPE_F32,
        DType::F64 => DTYPE_F64,
        DType::I8 => DTYPE_I8,
        DType::I16 => DTYPE_I16,
        DType::I32 => DTYPE_I32,
        DType::I64 => DTYPE_I64,
        DType::U8 => DTYPE_U8,
        DType::U16 => DTYPE_U16,
        DType::U32 => DTYPE_U32,
        DType::U64 => DTYPE_U64,
        DType::Bool => DTYPE_BOOL,
    }
}

pub fn dtype_from_tag(tag: i32) -> DType {
    match tag as u8 {
        DTYPE_F32 => DType::F32,
        DTYPE_F64 => DType::F64,
        DTYPE_I8 => DType::I8,
        DTYPE_I16 => DType::I16,
        DTYPE_I32 => DType::I32,
        DTYPE_I64 => DType::I64,
        DTYPE_U8 => DType::U8,
        DTYPE_U16 => DType::U16,
        DTYPE_U32 => DType::U32,
        DTYPE_U64 => DType::U64,
        DTYPE_BOOL => DType::Bool,
        other => panic!("the library reported a dtype tag ({}) that kn-graph has no type for", other),
    }
}

/// (unary tag, cast dtype tag)
fn unary_tags(op: UnaryOp) -> (u8, u8) {
    match op {
        UnaryOp::Abs => (UNARY_ABS, NO_CAST),
        UnaryOp::Neg => (UNARY_NEG, NO_CAST),
        UnaryOp::Sin => (UNARY_SIN, NO_CAST),
        UnaryOp::Cos => (UNARY_COS, NO_CAST),
        UnaryOp::Exp => (UNARY_EXP, NO_CAST),
        UnaryOp::Log => (UNARY_LOG, NO_CAST),
        UnaryOp::Sqrt => (UNARY_SQRT, NO_CAST),
        UnaryOp::Sigmoid => (UNARY_SIGMOID, NO_CAST),
        UnaryOp::Tanh => (UNARY_TANH, NO_CAST),
        UnaryOp::Erf => (UNARY_ERF, NO_CAST),
        UnaryOp::Mish => (UNARY_MISH, NO_CAST),
        UnaryOp::Softplus => (UNARY_SOFTPLUS, NO_CAST),
        UnaryOp::ValueCast(to) => (UNARY_VALUE_CAST, dtype_tag(to)),
        UnaryOp::BitCast(to) => (UNARY_BIT_CAST, dtype_tag(to)),
    }
}

fn binary_tag(op: BinaryOp) -> u8 {
    match op {
        BinaryOp::Add => BINARY_ADD,
        BinaryOp::Sub => BINARY_SUB,
        BinaryOp::Mul => BINARY_MUL,
        BinaryOp::Div => BINARY_DIV,
        BinaryOp::Min => BINARY_MIN,
        BinaryOp::Max => BINARY_MAX,
        BinaryOp::Pow => BINARY_POW,
    }
}

fn reduce_tag(op: ReduceOp) -> u8 {
    match op {
        ReduceOp::Sum => REDUCE_SUM,
        ReduceOp::Mean => REDUCE_MEAN,
        ReduceOp::Prod => REDUCE_PROD,
        ReduceOp::Max => REDUCE_MAX,
        ReduceOp::Min => REDUCE_MIN,
    }
}

fn put_u16(out: &mut Vec<u8>, v: usize) {
    out.extend_from_slice(&u16::try_from(v).expect("rank above 65535").to_le_bytes());
}
fn put_u32(out: &mut Vec<u8>, v: usize) {
    out.extend_from_slice(&u32::try_from(v).expect("index above u32::MAX").to_le_bytes());
}
fn put_u64(out: &mut Vec<u8>, v: usize) {
    out.extend_from_slice(&(v as u64).to_le_bytes());
}

/// The elements of a constant in standard layout, as the bytes the library uploads.
fn put_tensor(out: &mut Vec<u8>, tensor: &DTensor) {
    macro_rules! pod {
        ($inner:expr) => {{
            let std = $inner.as_standard_layout();
            let bytes: &[u8] = bytemuck::cast_slice(std.as_slice().expect("standard layout is contiguous"));
            put_u64(out, bytes.len());
            out.extend_from_slice(bytes);
        }};
    }
    match tensor {
        DTensor::F32(t) => pod!(t),
        DTensor::F64(t) => pod!(t),
        DTensor::I8(t) => pod!(t),
        DTensor::I16(t) => pod!(t),
        DTensor::I32(t) => pod!(t),
        DTensor::I64(t) => pod!(t),
        DTensor::U8(t) => pod!(t),
        DTensor::U16(t) => pod!(t),
        DTensor::U32(t) => pod!(t),
        DTensor::U64(t) => pod!(t),
        DTensor::Bool(t) => {
            put_u64(out, t.len());
            out.extend(t.iter().map(|b| b.0 as u8));   // ndarray iterates in logical (row-major) order
        }
    }
}

pub fn serialize_graph(graph: &Graph) -> Vec<u8> {
    let mut out = Vec::new();
    out.extend_from_slice(b"KNG1");
    put_u32(&mut out, graph.values().count());
    put_u32(&mut out, graph.inputs().len());
    put_u32(&mut out, graph.outputs().len());
    for v in graph.inputs() {
        put_u32(&mut out, v.index());
    }
    for v in graph.outputs() {
        put_u32(&mut out, v.index());
    }

    for value in graph.values() {
        let info = &graph[value];
        let tag = match &info.operation {
            Operation::Input { .. } => OP_INPUT,
            Operation::Constant { .. } => OP_CONSTANT,
            Operation::View { .. } => OP_VIEW,
            Operation::Broadcast { .. } => OP_BROADCAST,
            Operation::Permute { .. } => OP_PERMUTE,
            Operation::Slice { .. } => OP_SLICE,
            Operation::Flip { .. } => OP_FLIP,
            Operation::Gather { .. } => OP_GATHER,
            Operation::Concat { .. } => OP_CONCAT,
            Operation::Conv { .. } => OP_CONV,
            Operation::MatMul { .. } => OP_MATMUL,
            Operation::Unary { .. } => OP_UNARY,
            Operation::Binary { .. } => OP_BINARY,
            Operation::Softmax { .. } => OP_SOFTMAX,
            Operation::Layernorm { .. } => OP_LAYERNORM,
            Operation::Reduce { .. } => OP_REDUCE,
        };
        out.push(tag);
        out.push(dtype_tag(info.dtype));
        put_u16(&mut out, info.shape.rank());
        for size in &info.shape.dims {
            let (factor, exp) = size.components_factor_exp();
            put_u64(&mut out, factor);
            out.extend_from_slice(&exp.to_le_bytes());
        }

        match &info.operation {
            &Operation::Input { index } => put_u32(&mut out, index),
            Operation::Constant { tensor } => put_tensor(&mut out, tensor.inner()),
            &Operation::View { input } | &Operation::Broadcast { input } => put_u32(&mut out, input.index()),
            Operation::Permute { input, permutation } => {
                put_u32(&mut out, input.index());
                for &p in permutation {
                    put_u32(&mut out, p);
                }
            }
            &Operation::Slice { input, axis, range } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, axis);
                put_u64(&mut out, range.start);
                put_u64(&mut out, range.end);
                put_u64(&mut out, range.step);
            }
            &Operation::Flip { input, axis } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, axis);
            }
            &Operation::Gather { input, axis, indices } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, axis);
                put_u32(&mut out, indices.index());
            }
            Operation::Concat { inputs, axis } => {
                put_u32(&mut out, inputs.len());
                for v in inputs {
                    put_u32(&mut out, v.index());
                }
                put_u32(&mut out, *axis);
            }
            Operation::Conv { input, filter, details } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, filter.index());
                put_u32(&mut out, details.stride_y);
                put_u32(&mut out, details.stride_x);
                put_u32(&mut out, details.padding_y);
                put_u32(&mut out, details.padding_x);
            }
            &Operation::MatMul { left, right } => {
                put_u32(&mut out, left.index());
                put_u32(&mut out, right.index());
            }
            &Operation::Unary { input, op } => {
                put_u32(&mut out, input.index());
                let (unary, cast) = unary_tags(op);
                out.push(unary);
                out.push(cast);
            }
            &Operation::Binary { left, right, op } => {
                put_u32(&mut out, left.index());
                put_u32(&mut out, right.index());
                out.push(binary_tag(op));
            }
            &Operation::Softmax { input, axis } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, axis);
            }
            &Operation::Layernorm { input, axis, eps } => {
                put_u32(&mut out, input.index());
                put_u32(&mut out, axis);
                out.extend_from_slice(&eps.into_inner().to_le_bytes());
            }
            Operation::Reduce { input, axes, op } => {
                put_u32(&mut out, input.index());
                out.push(reduce_tag(*op));
                put_u32(&mut out, axes.len());
                for &a in axes {
                    put_u32(&mut out, a);
                }
            }
        }
    }
    out
}
