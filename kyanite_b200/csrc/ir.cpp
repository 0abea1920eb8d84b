#include "ir.h"

#include <cmath>

#include "kn_b200.h"
#include "scalar_ops.h"

namespace kn {

void fail(int code, const std::string& msg) { throw Error(code, msg); }

const char* dtype_name(DType d) {
    static const char* names[] = {"f32", "f64", "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "bool", "f16"};
    return (int)d < 12 ? names[(int)d] : "?";
}

const char* op_name(OpKind k) {
    static const char* names[] = {"Input", "Constant", "View", "Broadcast", "Permute", "Slice", "Flip", "Gather",
                                  "Concat", "Conv", "MatMul", "Unary", "Binary", "Softmax", "Layernorm", "Reduce", "AllReduce"};
    return (int)k < (int)OpKind::COUNT ? names[(int)k] : "?";
}

int64_t Size::eval(int64_t batch) const {
    int64_t r = (int64_t)factor;
    for (uint32_t i = 0; i < exp; i++) r *= batch;
    return r;
}

Scalar Scalar::f32(float v) { return Scalar{DType::F32, f32_to_bits(v)}; }
float Scalar::as_f32() const { return bits_to_f32(bits); }

double Scalar::as_f64_value() const {
    if (dtype_is_float(dtype)) return float_value(dtype, bits);
    if (dtype == DType::U64) return (double)bits;
    return (double)(int64_t)bits;
}

bool Scalar::operator==(const Scalar& o) const {
    if (dtype != o.dtype) return false;
    if (dtype_is_float(dtype)) {
        double a = float_value(dtype, bits), b = float_value(o.dtype, o.bits);
        if (a != a && b != b) return true;
        return a == b;
    }
    return bits == o.bits;
}

Scalar host_unary(UnaryOp op, DType from, DType to, Scalar x) { return Scalar{to, unary_bits(op, from, to, x.bits)}; }
Scalar host_binary(BinaryOp op, Scalar a, Scalar b) { return Scalar{a.dtype, binary_bits(op, a.dtype, a.bits, b.bits)}; }

namespace {

struct Reader {
    const uint8_t* p;
    size_t len, pos = 0;
    template <typename T>
    T take() {
        KN_CHECK(pos + sizeof(T) <= len, KN_ERR_BAD_GRAPH, "graph blob truncated");
        T v;
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    uint32_t u32() { return take<uint32_t>(); }
};

int checked_operand(Reader& r, size_t current) {
    uint32_t v = r.u32();
    KN_CHECK(v < current, KN_ERR_BAD_GRAPH, "graph blob: operand does not precede its user");
    return (int)v;
}

}  // namespace

std::unique_ptr<Graph> Graph::parse(const void* bytes, size_t len) {
    KN_CHECK(bytes != nullptr && len >= 16, KN_ERR_BAD_GRAPH, "graph blob too short");
    auto g = std::make_unique<Graph>();
    g->blob.assign((const uint8_t*)bytes, (const uint8_t*)bytes + len);
    Reader r{g->blob.data(), len};
    KN_CHECK(memcmp(r.p, "KNG1", 4) == 0, KN_ERR_BAD_GRAPH, "graph blob: bad magic");
    r.pos = 4;
    uint32_t n_values = r.u32(), n_in = r.u32(), n_out = r.u32();
    KN_CHECK((size_t)n_values <= len && (size_t)n_in <= len && (size_t)n_out <= len, KN_ERR_BAD_GRAPH,
             "graph blob: counts exceed blob size");
    for (uint32_t i = 0; i < n_in; i++) g->inputs.push_back((int)r.u32());
    for (uint32_t i = 0; i < n_out; i++) g->outputs.push_back((int)r.u32());
    for (int v : g->inputs) KN_CHECK(v >= 0 && (uint32_t)v < n_values, KN_ERR_BAD_GRAPH, "graph blob: bad input id");
    for (int v : g->outputs) KN_CHECK(v >= 0 && (uint32_t)v < n_values, KN_ERR_BAD_GRAPH, "graph blob: bad output id");

    g->values.reserve(n_values);
    for (uint32_t i = 0; i < n_values; i++) {
        ValueInfo info;
        uint8_t op = r.take<uint8_t>(), dt = r.take<uint8_t>();
        uint16_t rank = r.take<uint16_t>();
        KN_CHECK(op < (uint8_t)OpKind::COUNT, KN_ERR_BAD_GRAPH, "graph blob: unknown operation tag");
        KN_CHECK(dt < (uint8_t)DType::COUNT, KN_ERR_BAD_GRAPH, "graph blob: unknown dtype tag");
        info.op = (OpKind)op;
        info.dtype = (DType)dt;
        for (int d = 0; d < rank; d++) {
            Size s;
            s.factor = r.take<uint64_t>();
            s.exp = r.u32();
            info.shape.push_back(s);
        }
        switch (info.op) {
            case OpKind::Input:
                info.input_index = (int)r.u32();
                break;
            case OpKind::Constant: {
                uint64_t n = r.take<uint64_t>();
                // (n and the shape factors come from the blob: compare without letting a sum or product wrap)
                KN_CHECK(n <= (uint64_t)(len - r.pos), KN_ERR_BAD_GRAPH, "graph blob: constant payload truncated");
                const uint64_t elem_size = (uint64_t)dtype_size(info.dtype);
                uint64_t elems = 1;
                for (auto& s : info.shape) {
                    KN_CHECK(s.exp == 0, KN_ERR_BAD_GRAPH, "graph blob: constant with batch-dependent shape");
                    KN_CHECK(s.factor == 0 || elems <= (uint64_t)len / s.factor, KN_ERR_BAD_GRAPH,
                             "graph blob: constant shape larger than the blob");
                    elems *= s.factor;
                }
                KN_CHECK(elems <= (uint64_t)len / elem_size && elems * elem_size == n, KN_ERR_BAD_GRAPH,
                         "graph blob: constant size mismatch");
                info.const_data = r.p + r.pos;
                info.const_bytes = n;
                r.pos += n;
                break;
            }
            case OpKind::View: case OpKind::Broadcast:
                info.inputs = {checked_operand(r, i)};
                break;
            case OpKind::AllReduce:
                info.inputs = {checked_operand(r, i)};
                KN_CHECK(g->values[info.inputs[0]].dtype == info.dtype && (info.dtype == DType::F32 || info.dtype == DType::F16),
                         KN_ERR_BAD_GRAPH, "graph blob: all-reduce takes f32 or f16 and keeps the dtype");
                break;
            case OpKind::Permute:
                info.inputs = {checked_operand(r, i)};
                for (int d = 0; d < rank; d++) info.permutation.push_back((int)r.u32());
                break;
            case OpKind::Slice:
                info.inputs = {checked_operand(r, i)};
                info.axis = (int)r.u32();
                info.slice_start = (int64_t)r.take<uint64_t>();
                info.slice_end = (int64_t)r.take<uint64_t>();
                info.slice_step = (int64_t)r.take<uint64_t>();
                KN_CHECK(info.slice_step >= 1 && info.slice_end >= info.slice_start, KN_ERR_BAD_GRAPH,
                         "graph blob: invalid slice range");
                break;
            case OpKind::Flip:
                info.inputs = {checked_operand(r, i)};
                info.axis = (int)r.u32();
                break;
            case OpKind::Gather: {
                int in = checked_operand(r, i);
                info.axis = (int)r.u32();
                int idx = checked_operand(r, i);
                info.inputs = {in, idx};
                break;
            }
            case OpKind::Concat: {
                uint32_t n = r.u32();
                KN_CHECK(n <= len, KN_ERR_BAD_GRAPH, "graph blob: concat count");
                for (uint32_t k = 0; k < n; k++) info.inputs.push_back(checked_operand(r, i));
                info.axis = (int)r.u32();
                break;
            }
            case OpKind::Conv: {
                int in = checked_operand(r, i), f = checked_operand(r, i);
                info.inputs = {in, f};
                info.stride_y = (int)r.u32();
                info.stride_x = (int)r.u32();
                info.pad_y = (int)r.u32();
                info.pad_x = (int)r.u32();
                KN_CHECK(info.stride_y >= 1 && info.stride_x >= 1, KN_ERR_BAD_GRAPH, "graph blob: conv stride");
                break;
            }
            case OpKind::MatMul: {
                int a = checked_operand(r, i), b = checked_operand(r, i);
                info.inputs = {a, b};
                break;
            }
            case OpKind::Unary: {
                info.inputs = {checked_operand(r, i)};
                uint8_t uop = r.take<uint8_t>();
                (void)r.take<uint8_t>();   // cast target repeats the value dtype
                KN_CHECK(uop <= (uint8_t)UnaryOp::BitCast, KN_ERR_BAD_GRAPH, "graph blob: unknown unary op");
                info.unary_op = (UnaryOp)uop;
                info.cast_from = g->values[info.inputs[0]].dtype;
                break;
            }
            case OpKind::Binary: {
                int a = checked_operand(r, i), b = checked_operand(r, i);
                info.inputs = {a, b};
                uint8_t bop = r.take<uint8_t>();
                KN_CHECK(bop <= (uint8_t)BinaryOp::Pow, KN_ERR_BAD_GRAPH, "graph blob: unknown binary op");
                info.binary_op = (BinaryOp)bop;
                break;
            }
            case OpKind::Softmax:
                info.inputs = {checked_operand(r, i)};
                info.axis = (int)r.u32();
                break;
            case OpKind::Layernorm:
                info.inputs = {checked_operand(r, i)};
                info.axis = (int)r.u32();
                info.eps = r.take<float>();
                break;
            case OpKind::Reduce: {
                info.inputs = {checked_operand(r, i)};
                uint8_t rop = r.take<uint8_t>();
                KN_CHECK(rop <= (uint8_t)ReduceOp::Min, KN_ERR_BAD_GRAPH, "graph blob: unknown reduce op");
                info.reduce_op = (ReduceOp)rop;
                uint32_t n = r.u32();
                KN_CHECK(n <= 64, KN_ERR_BAD_GRAPH, "graph blob: reduce axes count");
                for (uint32_t k = 0; k < n; k++) info.axes.push_back((int)r.u32());
                break;
            }
            default:
                fail(KN_ERR_BAD_GRAPH, "graph blob: unknown operation");
        }
        // axis sanity against the operand rank
        if (!info.inputs.empty()) {
            size_t in_rank = g->values[info.inputs[0]].shape.size();
            switch (info.op) {
                case OpKind::Slice: case OpKind::Flip: case OpKind::Gather: case OpKind::Softmax: case OpKind::Layernorm:
                    KN_CHECK((size_t)info.axis < in_rank, KN_ERR_BAD_GRAPH, "graph blob: axis out of range");
                    break;
                case OpKind::Concat:
                    KN_CHECK((size_t)info.axis < info.shape.size(), KN_ERR_BAD_GRAPH, "graph blob: axis out of range");
                    break;
                case OpKind::Reduce:
                    for (int a : info.axes) KN_CHECK((size_t)a < in_rank, KN_ERR_BAD_GRAPH, "graph blob: axis out of range");
                    break;
                case OpKind::Permute:
                    KN_CHECK(info.permutation.size() == in_rank, KN_ERR_BAD_GRAPH, "graph blob: permutation rank");
                    for (int a : info.permutation) KN_CHECK((size_t)a < in_rank, KN_ERR_BAD_GRAPH, "graph blob: permutation axis");
                    break;
                default: break;
            }
        }
        for (int in : info.inputs) g->values[in].non_output_uses++;
        g->values.push_back(std::move(info));
    }
    KN_CHECK(r.pos == len, KN_ERR_BAD_GRAPH, "graph blob: trailing bytes");
    for (size_t k = 0; k < g->inputs.size(); k++) {
        const ValueInfo& info = g->values[g->inputs[k]];
        KN_CHECK(info.op == OpKind::Input && info.input_index == (int)k, KN_ERR_BAD_GRAPH,
                 "graph blob: input list does not match Input values");
    }
    return g;
}

std::vector<int64_t> Graph::eval_shape(int v, int64_t batch) const {
    std::vector<int64_t> r;
    for (auto& s : values[v].shape) r.push_back(s.eval(batch));
    return r;
}

bool Graph::is_input(int v) const {
    for (int i : inputs) if (i == v) return true;
    return false;
}
bool Graph::is_output(int v) const {
    for (int i : outputs) if (i == v) return true;
    return false;
}

std::optional<Scalar> Graph::as_single_const(int v) const {
    // iterative for the pass-through chain, recursive only at Unary/Binary/Concat forks
    while (true) {
        const ValueInfo& info = values[v];
        switch (info.op) {
            case OpKind::Input: return std::nullopt;
            case OpKind::Constant: {
                size_t es = dtype_size(info.dtype);
                size_t n = info.const_bytes / es;
                if (n == 0) return std::nullopt;
                Scalar first{info.dtype, load_bits(info.const_data, info.dtype, 0)};
                for (size_t i = 1; i < n; i++) {
                    Scalar e{info.dtype, load_bits(info.const_data, info.dtype, (int64_t)i)};
                    if (!(e == first)) return std::nullopt;
                }
                return first;
            }
            case OpKind::View: case OpKind::Broadcast: case OpKind::Permute: case OpKind::Slice: case OpKind::Flip:
            case OpKind::Gather:
                v = info.inputs[0];
                continue;
            case OpKind::Concat: {
                if (info.inputs.empty()) return std::nullopt;
                auto f = as_single_const(info.inputs[0]);
                if (!f) return std::nullopt;
                for (int in : info.inputs) {
                    auto o = as_single_const(in);
                    if (!o || !(*o == *f)) return std::nullopt;
                }
                return f;
            }
            case OpKind::Unary: {
                auto x = as_single_const(info.inputs[0]);
                if (!x) return std::nullopt;
                return host_unary(info.unary_op, info.cast_from, info.dtype, *x);
            }
            case OpKind::Binary: {
                auto a = as_single_const(info.inputs[0]);
                if (!a) return std::nullopt;
                auto b = as_single_const(info.inputs[1]);
                if (!b) return std::nullopt;
                return host_binary(info.binary_op, *a, *b);
            }
            default: return std::nullopt;
        }
    }
}

bool Graph::is_const_zero(int v) const {
    auto c = as_single_const(v);
    if (!c) return false;
    if (dtype_is_float(c->dtype)) return float_value(c->dtype, c->bits) == 0.0;
    return c->bits == 0;
}

}  // namespace kn
