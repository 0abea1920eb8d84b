// Host-side mirror of the graph IR the executor consumes (the reference's `Graph`, `ValueInfo`,
// `Operation`: kn-graph/src/graph.rs:77-217) and the reader of its serialised form.
#pragma once
#include <memory>
#include <optional>

#include "common.h"

namespace kn {

// 0..15 are the reference's `Operation` variants (kn-graph/src/graph.rs:106-162); AllReduce is an extension
// for tensor-parallel graphs (the reference runs one graph on one device): the element-wise sum of the value
// over the ranks of the communicator attached to the executor, the value itself when there is none.
enum class OpKind : uint8_t {
    Input = 0, Constant, View, Broadcast, Permute, Slice, Flip, Gather, Concat, Conv, MatMul, Unary, Binary,
    Softmax, Layernorm, Reduce, AllReduce, COUNT
};
const char* op_name(OpKind k);

// `factor * batch^exp` (kn-graph/src/shape.rs:37-44)
struct Size {
    uint64_t factor = 0;
    uint32_t exp = 0;
    int64_t eval(int64_t batch) const;
};

// A single element of any dtype, kept as raw bits.
struct Scalar {
    DType dtype = DType::F32;
    uint64_t bits = 0;
    static Scalar f32(float v);
    float as_f32() const;
    double as_f64_value() const;   // numeric value converted to double (any dtype)
    bool operator==(const Scalar& o) const;   // NaN equals NaN, -0 equals +0 for floats
};

struct ValueInfo {
    OpKind op = OpKind::Input;
    DType dtype = DType::F32;
    std::vector<Size> shape;
    std::vector<int> inputs;

    int input_index = 0;                       // Input
    const uint8_t* const_data = nullptr;       // Constant: points into Graph::blob
    size_t const_bytes = 0;
    std::vector<int> permutation;              // Permute
    int axis = 0;                              // Slice Flip Gather Concat Softmax Layernorm
    int64_t slice_start = 0, slice_end = 0, slice_step = 1;
    int stride_y = 1, stride_x = 1, pad_y = 0, pad_x = 0;   // Conv
    UnaryOp unary_op = UnaryOp::Abs;
    DType cast_from = DType::F32;              // Unary casts: dtype of the operand
    BinaryOp binary_op = BinaryOp::Add;
    ReduceOp reduce_op = ReduceOp::Sum;
    std::vector<int> axes;                     // Reduce
    float eps = 0.f;                           // Layernorm

    int non_output_uses = 0;                   // recomputed on load (graph.rs:549-552)
};

struct Graph {
    std::vector<uint8_t> blob;                 // owns constant payloads
    std::vector<ValueInfo> values;
    std::vector<int> inputs, outputs;

    static std::unique_ptr<Graph> parse(const void* bytes, size_t len);

    std::vector<int64_t> eval_shape(int v, int64_t batch) const;
    bool is_input(int v) const;
    bool is_output(int v) const;
    bool is_hidden(int v) const { return !is_input(v) && !is_output(v); }
    // hidden and used by exactly `users` operations (graph.rs:421-423)
    bool is_hidden_with_uses(int v, int users) const { return is_hidden(v) && values[v].non_output_uses == users; }

    // `Some(c)` if every element of `v` equals the same constant (graph.rs:490-527)
    std::optional<Scalar> as_single_const(int v) const;
    bool is_const_zero(int v) const;
};

// scalar evaluation on the host with the executor's element semantics
Scalar host_unary(UnaryOp op, DType from, DType to, Scalar x);
Scalar host_binary(BinaryOp op, Scalar a, Scalar b);

}  // namespace kn
