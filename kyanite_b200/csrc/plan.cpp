#include "plan.h"

#include <pthread.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <map>
#include <optional>
#include <sstream>

#include "scalar_ops.h"
#include "tc.h"

namespace kn {

const char* step_kind_name(StepKind k) {
    static const char* names[] = {"Scalar", "Reduce", "Softmax", "Layernorm", "Gather", "Gemm", "Conv", "ConvChain", "Im2col", "AllReduce", "RmsNorm"};
    return (int)k < (int)StepKind::COUNT ? names[(int)k] : "?";
}

// ------------------------------------------------------------------------------------------------
// PlanTensor
// ------------------------------------------------------------------------------------------------
PlanTensor PlanTensor::with(StridedShape s, int64_t extra_offset) const {
    PlanTensor r = *this;
    r.ss = std::move(s);
    r.offset += extra_offset;
    return r;
}

PlanTensor PlanTensor::slice(int axis, int64_t start, int64_t end, int64_t step) const {
    StridedShape s = ss.slice(axis, start, end, step);
    // an empty slice addresses nothing; keep the offset inside the buffer
    int64_t extra = s.shape[axis] == 0 ? 0 : start * ss.strides[axis];
    return with(std::move(s), extra);
}

PlanTensor PlanTensor::flip(int axis) const {
    StridedShape s = ss.flip(axis);
    int64_t len = ss.shape[axis];
    int64_t extra = len == 0 ? 0 : (len - 1) * ss.strides[axis];
    return with(std::move(s), extra);
}

std::string PlanTensor::str() const {
    return std::string(dtype_name(dtype)) + "@b" + std::to_string(buf) + "+" + std::to_string(offset) + ss.str();
}

namespace {

double touched_bytes(const PlanTensor& t) {
    double n = 1;
    for (int i = 0; i < t.ss.rank(); i++)
        if (t.ss.strides[i] != 0 || t.ss.shape[i] == 0) n *= (double)t.ss.shape[i];
    return n * dtype_size(t.dtype);
}

// Merge axes that are contiguous for every operand and drop unit axes, so kernels decode as few
// coordinates per element as possible.  `strides[o]` are per-operand strides over `dims`.
void coalesce_axes(std::vector<int64_t>& dims, std::vector<std::vector<int64_t>>& strides) {
    std::vector<int64_t> nd;
    std::vector<std::vector<int64_t>> ns(strides.size());
    for (size_t d = 0; d < dims.size(); d++) {
        if (dims[d] == 1) continue;
        bool merged = false;
        if (!nd.empty()) {
            bool can = true;
            for (size_t o = 0; o < strides.size(); o++)
                if (ns[o].back() != strides[o][d] * dims[d]) { can = false; break; }
            if (can) {
                nd.back() *= dims[d];
                for (size_t o = 0; o < strides.size(); o++) ns[o].back() = strides[o][d];
                merged = true;
            }
        }
        if (!merged) {
            nd.push_back(dims[d]);
            for (size_t o = 0; o < strides.size(); o++) ns[o].push_back(strides[o][d]);
        }
    }
    if (nd.empty()) {
        nd.push_back(1);
        for (auto& s : ns) s.push_back(0);
    }
    dims = std::move(nd);
    strides = std::move(ns);
}

// slot reference while a scalar program is being built: loads and instructions are numbered
// separately and merged into one slot space at the end
struct Ref {
    bool is_load = false;
    int index = -1;
};

struct ScalarBlock {
    std::vector<PlanTensor> loads;
    struct PendingInstr {
        ScalarInstr in;
        Ref a, b;
    };
    std::vector<PendingInstr> instrs;
    std::map<int, Ref> value_ref;   // graph value -> slot (common sub-expressions evaluate once)

    Ref load(const PlanTensor& t) {
        for (size_t i = 0; i < loads.size(); i++)
            if (loads[i].same_storage(t)) return Ref{true, (int)i};
        loads.push_back(t);
        return Ref{true, (int)loads.size() - 1};
    }
    Ref constant(Scalar c) {
        PendingInstr p{};
        p.in.kind = 0;
        p.in.dtype = (uint8_t)c.dtype;
        p.in.from = (uint8_t)c.dtype;
        p.in.imm = c.bits;
        instrs.push_back(p);
        return Ref{false, (int)instrs.size() - 1};
    }
    Ref unary(UnaryOp op, DType from, DType to, Ref a) {
        PendingInstr p{};
        p.in.kind = 1;
        p.in.op = (uint8_t)op;
        p.in.dtype = (uint8_t)to;
        p.in.from = (uint8_t)from;
        p.a = a;
        instrs.push_back(p);
        return Ref{false, (int)instrs.size() - 1};
    }
    Ref binary(BinaryOp op, DType d, Ref a, Ref b) {
        PendingInstr p{};
        p.in.kind = 2;
        p.in.op = (uint8_t)op;
        p.in.dtype = (uint8_t)d;
        p.in.from = (uint8_t)d;
        p.a = a;
        p.b = b;
        instrs.push_back(p);
        return Ref{false, (int)instrs.size() - 1};
    }
};

class Planner {
   public:
    Planner(const Graph& g, int64_t batch, const kn_options& opts, Plan& plan)
        : g_(g), batch_(batch), opts_(opts), plan_(plan), map_(g.values.size()), chain_cache_(g.values.size(), -2),
          users_(g.values.size()) {
        for (size_t v = 0; v < g.values.size(); v++)
            for (int in : g.values[v].inputs) users_[in].push_back((int)v);
    }

    void run() {
        plan_.batch = batch_;
        plan_.opts = opts_;
        plan_.inputs.resize(g_.inputs.size());
        // every graph input gets a buffer, used or not (planner.rs:117-121)
        for (int v : g_.inputs) visit(v);
        for (int v : g_.outputs) {
            PlanTensor t = ensure_simple(visit(v), v);
            buffer(t.buf).always_live = true;
            plan_.outputs.push_back(t);
            plan_.output_shapes.push_back(t.ss.shape);
        }
        for (auto& t : plan_.inputs) plan_.input_shapes.push_back(t.ss.shape);
        fuse_conv_chains();
        drop_unused_constants();
        assign_memory();
    }

   private:
    const Graph& g_;
    int64_t batch_;
    kn_options opts_;
    Plan& plan_;
    std::vector<std::optional<PlanTensor>> map_;
    std::vector<int> chain_cache_;
    std::vector<std::vector<int>> users_;

    BufferInfo& buffer(int b) { return plan_.buffers[b]; }

    std::vector<int64_t> shape_of(int v) const {
        std::vector<int64_t> s = g_.eval_shape(v, batch_);
        for (int64_t d : s) KN_CHECK(d >= 0, KN_ERR_SHAPE, "negative dimension");
        return s;
    }

    // ---------------------------------------------------------------- buffers
    PlanTensor alloc_shared(const std::vector<int64_t>& shape, DType dtype, int value) {
        BufferInfo b;
        b.kind = BufKind::Shared;
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        b.bytes = (size_t)n * dtype_size(dtype);
        b.value = value;
        plan_.buffers.push_back(b);
        PlanTensor t;
        t.buf = (int)plan_.buffers.size() - 1;
        t.dtype = dtype;
        t.ss = StridedShape::simple(shape);
        return t;
    }

    PlanTensor alloc_const(const std::vector<int64_t>& shape, DType dtype, int value, const uint8_t* data,
                           std::shared_ptr<std::vector<uint8_t>> owned) {
        BufferInfo b;
        b.kind = BufKind::Const;
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        b.bytes = (size_t)n * dtype_size(dtype);
        b.value = value;
        b.host_data = owned ? owned->data() : data;
        b.owned = std::move(owned);
        plan_.buffers.push_back(b);
        PlanTensor t;
        t.buf = (int)plan_.buffers.size() - 1;
        t.dtype = dtype;
        t.ss = StridedShape::simple(shape);
        return t;
    }

    // ---------------------------------------------------------------- steps
    void push_step(Step&& s) {
        for (auto& t : s.operands) KN_CHECK(t.ss.rank() <= 64, KN_ERR_INTERNAL, "operand rank");
        s.alg_bytes = 0;
        for (size_t i = 0; i < s.operands.size(); i++) {
            bool dup = false;
            for (size_t j = 0; j < i; j++) dup = dup || s.operands[j].same_storage(s.operands[i]);
            if (!dup) s.alg_bytes += touched_bytes(s.operands[i]);
        }
        plan_.steps.push_back(std::move(s));
    }

    // Emit one fused elementwise kernel.  `stores` pairs a destination tensor with the slot to write.
    void emit_scalar(ScalarBlock& block, const std::vector<std::pair<PlanTensor, Ref>>& stores, int value,
                     const std::string& desc) {
        KN_CHECK(!stores.empty(), KN_ERR_INTERNAL, "scalar step without a store");
        const std::vector<int64_t>& shape = stores[0].first.ss.shape;
        int64_t total = 1;
        for (int64_t d : shape) total *= d;
        if (total == 0) return;

        Step s;
        s.kind = StepKind::Scalar;
        s.value = value;
        s.desc = desc;
        for (auto& t : block.loads) {
            KN_CHECK(t.ss.shape == shape, KN_ERR_INTERNAL, "scalar operand shape mismatch");
            s.operands.push_back(t);
            s.writes.push_back(0);
        }
        for (auto& st : stores) {
            KN_CHECK(st.first.ss.shape == shape, KN_ERR_INTERNAL, "scalar store shape mismatch");
            s.operands.push_back(st.first);
            s.writes.push_back(1);
        }
        KN_CHECK((int)s.operands.size() <= SCALAR_MAX_OPERANDS, KN_ERR_UNSUPPORTED, "too many operands in one fused elementwise step");
        KN_CHECK((int)block.instrs.size() <= SCALAR_MAX_INSTR, KN_ERR_UNSUPPORTED, "fused elementwise program too long");

        std::vector<int64_t> dims = shape;
        std::vector<std::vector<int64_t>> strides;
        for (auto& t : s.operands) strides.push_back(t.ss.strides);
        coalesce_axes(dims, strides);
        KN_CHECK((int)dims.size() <= DEV_MAX_RANK, KN_ERR_UNSUPPORTED,
                 "elementwise step needs more than 8 non-mergeable axes");

        ScalarParams& p = s.scalar;
        p.rank = (int)dims.size();
        p.n_operands = (int)s.operands.size();
        p.n_loads = (int)block.loads.size();
        p.n_instr = (int)block.instrs.size();
        p.n_stores = (int)stores.size();
        p.total = total;
        for (int d = 0; d < p.rank; d++) p.dims[d] = dims[d];
        for (int o = 0; o < p.n_operands; o++) {
            p.dtype[o] = (uint8_t)s.operands[o].dtype;
            for (int d = 0; d < p.rank; d++) p.strides[o][d] = strides[o][d];
        }
        auto slot_of = [&](Ref r) { return r.is_load ? r.index : p.n_loads + r.index; };
        for (int l = 0; l < p.n_loads; l++) p.load_operand[l] = (uint8_t)l;
        for (int k = 0; k < p.n_instr; k++) {
            ScalarInstr in = block.instrs[k].in;
            if (in.kind >= 1) in.a = (uint8_t)slot_of(block.instrs[k].a);
            if (in.kind == 2) in.b = (uint8_t)slot_of(block.instrs[k].b);
            p.instr[k] = in;
        }
        for (int st = 0; st < p.n_stores; st++) {
            p.store_operand[st] = (uint8_t)(p.n_loads + st);
            p.store_slot[st] = (uint8_t)slot_of(stores[st].second);
        }

        // 128-bit path: all f32, innermost axis contiguous (or broadcast for loads), 16-byte aligned
        bool vec = dims.back() % 4 == 0;
        for (int k = 0; k < p.n_instr && vec; k++)
            vec = p.instr[k].dtype == (uint8_t)DType::F32 && p.instr[k].from == (uint8_t)DType::F32;
        for (int o = 0; o < p.n_operands && vec; o++) {
            const PlanTensor& t = s.operands[o];
            int64_t inner = strides[o].back();
            bool is_store = o >= p.n_loads;
            if (t.dtype != DType::F32 || !(inner == 1 || (inner == 0 && !is_store))) { vec = false; break; }
            if (inner == 1) {
                if (t.offset % 4 != 0) vec = false;
                for (int d = 0; d + 1 < p.rank; d++)
                    if (strides[o][d] % 4 != 0) vec = false;
            }
        }
        p.vec4 = vec ? 1 : 0;
        if (!vec && dims.back() % 8 == 0) {
            // f16 / f32 mix (half-storage graphs): the eight-elements-per-access kernel
            bool vec8 = true, any_half = false;
            for (int k = 0; k < p.n_instr && vec8; k++) {
                const DType d = (DType)p.instr[k].dtype, f = (DType)p.instr[k].from;
                vec8 = (d == DType::F32 || d == DType::F16) && (f == DType::F32 || f == DType::F16) &&
                       !(p.instr[k].kind == 1 && (UnaryOp)p.instr[k].op == UnaryOp::BitCast);
            }
            for (int o = 0; o < p.n_operands && vec8; o++) {
                const PlanTensor& t = s.operands[o];
                const int64_t inner = strides[o].back();
                const bool is_store = o >= p.n_loads;
                if (t.dtype != DType::F32 && t.dtype != DType::F16) { vec8 = false; break; }
                any_half = any_half || t.dtype == DType::F16;
                if (!(inner == 1 || (inner == 0 && !is_store))) { vec8 = false; break; }
                const int64_t align = t.dtype == DType::F16 ? 8 : 4;
                if (inner == 1) {
                    if (t.offset % align != 0) vec8 = false;
                    for (int d = 0; d + 1 < p.rank; d++)
                        if (strides[o][d] % align != 0) vec8 = false;
                } else if (t.offset % 1 != 0) {
                    vec8 = false;
                }
            }
            if (vec8 && any_half) p.vec4 = 3;
        }
        // the accumulator-program kernel computes element offsets in 32 bits and keeps four operand addresses
        // in registers: non-negative strides, no operand may reach 2^31 elements from its start
        const bool mixed = p.vec4 == 3;
        bool small = (vec || mixed) && total < (1ll << 31) && p.n_operands <= (mixed ? 6 : 4);   // (the kernel's register operands)
        for (int o = 0; o < p.n_operands && small; o++) {
            int64_t reach = 0;
            for (int d = 0; d < p.rank; d++) {
                if (strides[o][d] < 0) small = false;
                reach += (dims[d] - 1) * strides[o][d];
            }
            if (reach >= (1ll << 31) - 16) small = false;
        }
        if (small && allocate_registers(p)) {
            p.vec4 = mixed ? 4 : 2;
            // every operand and every value f16: the program runs on packed halves (mode 5)
            bool all_half = mixed;
            for (int o = 0; o < p.n_operands && all_half; o++) all_half = (DType)p.dtype[o] == DType::F16;
            for (int k = 0; k < p.n_instr && all_half; k++)
                all_half = (DType)p.instr[k].dtype == DType::F16 && (DType)p.instr[k].from == DType::F16;
            if (all_half) p.vec4 = 5;
        }
        push_step(std::move(s));
    }

    // Turns the slot program into an accumulator program (ScalarParams::micro).  Every micro-op leaves its
    // result in the accumulator; an operand is read from the accumulator when it was computed by the
    // micro-op just before, from a constant folded into the operation, or else from a numbered spill slot
    // that its defining micro-op copies the result to.  All loads come first (so they are in flight
    // together), slots are recycled after a value's last use.  False if more than 8 slots would be live.
    //   kind 0 acc = imm                      3 acc = load operand `a`
    //   kind 1 acc = unary(A)                 4 store A -> operand `b`
    //   kind 2 acc = binary(A, B)             5 acc = binary(A, imm)     6 acc = binary(imm, A)
    // A / B: `a` / `b` = 255 means the accumulator, otherwise a slot; `pad` low byte = slot to copy the result to, or
    // 255; `pad` bit 8 = the result goes to f16 stores only, so the store's rounding is the op's rounding and the
    // kernel need not round the f16-typed result itself.
    static bool allocate_registers(ScalarParams& p) {
        const int kAcc = 255;
        const int n_values = p.n_loads + p.n_instr;
        auto is_const = [&](int v) { return v >= p.n_loads && p.instr[v - p.n_loads].kind == 0; };
        struct Op {
            ScalarInstr m;
            int result = -1, src_a = -1, src_b = -1;   // value ids
        };
        std::vector<Op> ops;
        std::vector<int> const_op(n_values, -1);   // constant used as a value -> op that materialises it
        auto materialise_const = [&](int v) {
            if (const_op[v] >= 0) return;
            Op o;
            o.m.kind = 0;
            o.m.imm = p.instr[v - p.n_loads].imm;
            o.m.dtype = p.instr[v - p.n_loads].dtype;   // how to read `imm`
            o.result = v;
            const_op[v] = (int)ops.size();
            ops.push_back(o);
        };
        // pass 1: order of the micro-ops
        for (int l = 0; l < p.n_loads; l++) {
            Op o;
            o.m.kind = 3;
            o.m.a = p.load_operand[l];
            o.result = l;
            ops.push_back(o);
        }
        for (int k = 0; k < p.n_instr; k++) {
            const ScalarInstr& in = p.instr[k];
            if (in.kind == 0) continue;
            Op o;
            o.m = in;
            o.result = p.n_loads + k;
            if (in.kind == 1) {
                if (is_const(in.a)) materialise_const(in.a);
                o.src_a = in.a;
            } else if (is_const(in.b) && !is_const(in.a)) {
                o.m.kind = 5;
                o.m.imm = p.instr[in.b - p.n_loads].imm;
                o.src_a = in.a;
                // x ^ 2 is the square: exact, and far cheaper than the general power function
                if (in.op == (uint8_t)BinaryOp::Pow && in.dtype == (uint8_t)DType::F32 && o.m.imm == 0x40000000ull) {
                    o.m.kind = 2;
                    o.m.op = (uint8_t)BinaryOp::Mul;
                    o.src_b = in.a;
                }
            } else if (is_const(in.a) && !is_const(in.b)) {
                o.m.kind = 6;
                o.m.imm = p.instr[in.a - p.n_loads].imm;
                o.src_a = in.b;
            } else {
                if (is_const(in.a)) materialise_const(in.a);
                if (is_const(in.b)) materialise_const(in.b);
                o.src_a = in.a;
                o.src_b = in.b;
            }
            ops.push_back(o);
        }
        for (int st = 0; st < p.n_stores; st++) {
            const int v = p.store_slot[st];
            if (is_const(v)) materialise_const(v);
            Op o;
            o.m.kind = 4;
            o.m.b = p.store_operand[st];
            o.src_a = v;
            ops.push_back(o);
        }
        if ((int)ops.size() > SCALAR_MAX_INSTR + 2 * SCALAR_MAX_OPERANDS) return false;
        // pass 2: a value needs a slot unless its only uses are operands of the op right after its definition
        std::vector<int> def(n_values, -1), last_use(n_values, -1);
        std::vector<uint8_t> needs_slot(n_values, 0);
        for (int i = 0; i < (int)ops.size(); i++)
            if (ops[i].result >= 0) def[ops[i].result] = i;
        for (int i = 0; i < (int)ops.size(); i++)
            for (int v : {ops[i].src_a, ops[i].src_b}) {
                if (v < 0) continue;
                if (def[v] < 0) return false;   // (cannot happen: every used value has a defining op)
                last_use[v] = std::max(last_use[v], i);
                if (i != def[v] + 1) needs_slot[v] = 1;
            }
        std::vector<int> slot_of(n_values, -1);
        std::vector<int> free_slots;
        std::vector<std::vector<int>> expiring(ops.size() + 1);
        int n_regs = 0;
        for (int i = 0; i < (int)ops.size(); i++) {
            // operands are read before the result is written: slots whose last reader is this op are free again
            for (int v : expiring[i]) free_slots.push_back(slot_of[v]);
            Op& o = ops[i];
            o.m.pad = (uint16_t)kAcc;
            auto where = [&](int v) -> int { return (i == def[v] + 1) ? kAcc : slot_of[v]; };
            if (o.m.kind == 4) {
                o.m.a = (uint8_t)where(o.src_a);
            } else if (o.m.kind != 0 && o.m.kind != 3) {
                if (o.src_a >= 0) o.m.a = (uint8_t)where(o.src_a);
                if (o.src_b >= 0) o.m.b = (uint8_t)where(o.src_b);
            }
            const int v = o.result;
            if (v >= 0 && needs_slot[v] && last_use[v] > i) {
                int s;
                if (!free_slots.empty()) {
                    s = free_slots.back();
                    free_slots.pop_back();
                } else if (n_regs < 8) {
                    s = n_regs++;
                } else {
                    return false;
                }
                slot_of[v] = s;
                o.m.pad = (uint16_t)s;
                expiring[last_use[v]].push_back(v);
            }
        }
        // results that only f16 stores read
        std::vector<uint8_t> read_by_other(n_values, 0), read_by_store(n_values, 0);
        for (const Op& o : ops) {
            if (o.m.kind == 4) {
                if (o.src_a >= 0) ((DType)p.dtype[o.m.b] == DType::F16 ? read_by_store : read_by_other)[o.src_a] = 1;
            } else {
                for (int v : {o.src_a, o.src_b})
                    if (v >= 0) read_by_other[v] = 1;
            }
        }
        for (Op& o : ops)
            if (o.result >= 0 && o.m.kind != 0 && o.m.kind != 3 && o.m.kind != 4 && read_by_store[o.result] && !read_by_other[o.result])
                o.m.pad |= 0x100;
        p.n_micro = (int)ops.size();
        for (int i = 0; i < p.n_micro; i++) p.micro[i] = ops[i].m;
        p.n_regs = n_regs;
        return true;
    }


    void emit_copy(const PlanTensor& src, const PlanTensor& dst, int value) {
        ScalarBlock block;
        Ref r = block.load(src);
        emit_scalar(block, {{dst, r}}, value, "copy");
    }

    PlanTensor ensure_simple(const PlanTensor& t, int value) {
        if (t.ss.has_simple_strides()) return t;
        PlanTensor dense = alloc_shared(t.ss.shape, t.dtype, value);
        emit_copy(t, dense, value);
        return dense;
    }

    // ---------------------------------------------------------------- visiting
    PlanTensor visit(int v) {
        if (map_[v]) return *map_[v];
        PlanTensor t = visit_new(v);
        KN_CHECK(t.ss.shape == shape_of(v), KN_ERR_INTERNAL, "planned shape differs from graph shape");
        KN_CHECK(t.dtype == g_.values[v].dtype, KN_ERR_INTERNAL, "planned dtype differs from graph dtype");
        map_[v] = t;
        return t;
    }

    PlanTensor visit_new(int v) {
        if (auto fused = try_fused_attention_context(v)) return *fused;
        if (auto fused = try_fused_contraction(v)) return *fused;
        if (auto fused = try_fused_rmsnorm(v)) return *fused;
        const ValueInfo& info = g_.values[v];
        std::vector<int64_t> shape = shape_of(v);
        switch (info.op) {
            case OpKind::Input: {
                PlanTensor t = alloc_shared(shape, info.dtype, v);
                buffer(t.buf).always_live = true;
                plan_.inputs[info.input_index] = t;
                return t;
            }
            case OpKind::Constant:
                return alloc_const(shape, info.dtype, v, info.const_data, nullptr);
            case OpKind::View: {
                PlanTensor in = visit(info.inputs[0]);
                if (auto s = in.ss.view(shape)) return in.with(*s);
                PlanTensor dense = alloc_shared(in.ss.shape, in.dtype, v);
                emit_copy(in, dense, v);
                auto s = dense.ss.view(shape);
                KN_CHECK(s.has_value(), KN_ERR_INTERNAL, "view of a dense tensor failed");
                return dense.with(*s);
            }
            case OpKind::Broadcast: {
                PlanTensor in = visit(info.inputs[0]);
                return in.with(in.ss.broadcast(shape));
            }
            case OpKind::Permute: {
                PlanTensor in = visit(info.inputs[0]);
                return in.with(in.ss.permute(info.permutation));
            }
            case OpKind::Slice: {
                PlanTensor in = visit(info.inputs[0]);
                return in.slice(info.axis, info.slice_start, info.slice_end, info.slice_step);
            }
            case OpKind::Flip: {
                PlanTensor in = visit(info.inputs[0]);
                return in.flip(info.axis);
            }
            case OpKind::Gather: return visit_gather(v);
            case OpKind::Concat: {
                std::vector<PlanTensor> ins;
                for (int i : info.inputs) ins.push_back(visit(i));
                PlanTensor out = alloc_shared(shape, info.dtype, v);
                int64_t start = 0;
                for (auto& in : ins) {
                    int64_t n = in.ss.shape[info.axis];
                    emit_copy(in, out.slice(info.axis, start, start + n, 1), v);
                    start += n;
                }
                KN_CHECK(start == shape[info.axis], KN_ERR_SHAPE, "concat sizes do not add up");
                return out;
            }
            case OpKind::MatMul:
                if (info.dtype == DType::F16) return visit_matmul_f16(v);
                fail(KN_ERR_UNSUPPORTED, "MatMul is only supported for f32 and f16 operands");
            case OpKind::Conv:
                fail(KN_ERR_UNSUPPORTED, "Conv is only supported for f32 operands");
            case OpKind::Unary: case OpKind::Binary: return visit_scalar(v);
            case OpKind::Softmax:
                if (auto fused = try_fused_attention_scores(v)) return *fused;
                return visit_softmax(v);
            case OpKind::Layernorm: return visit_layernorm(v);
            case OpKind::Reduce: return visit_reduce(v);
            case OpKind::AllReduce: {
                // the collective library wants dense buffers; the result is a buffer of its own, so the step is the
                // same whether or not other steps still read the partial sum
                PlanTensor in = ensure_simple(visit(info.inputs[0]), v);
                PlanTensor out = alloc_shared(shape, info.dtype, v);
                Step s;
                s.kind = StepKind::AllReduce;
                s.value = v;
                s.operands = {in, out};
                s.writes = {0, 1};
                s.all_reduce.count = out.ss.size();
                s.all_reduce.dtype = (uint8_t)info.dtype;
                s.desc = "allreduce sum count=" + std::to_string(out.ss.size()) + " " + dtype_name(info.dtype);
                if (out.ss.size() != 0) {
                    push_step(std::move(s));
                    plan_.collectives++;
                }
                return out;
            }
            default: fail(KN_ERR_INTERNAL, "unknown operation");
        }
    }

    // ---------------------------------------------------------------- elementwise fusion
    // (kn-cuda-eval/src/planner.rs:835-923.)  Differences from the reference: a value whose users
    // are not all inside this expression is materialised once and loaded instead of being
    // recomputed per user, shared sub-expressions inside the block evaluate once, and a block that
    // outgrows the kernel's program size is split at a sub-expression.
    PlanTensor visit_scalar(int root) {
        // count edges from Unary/Binary nodes reachable from the root, to find values used only here
        std::map<int, int> tree_uses;
        {
            std::vector<int> stack{root};
            std::map<int, bool> seen;
            while (!stack.empty()) {
                int x = stack.back();
                stack.pop_back();
                if (seen[x]) continue;
                seen[x] = true;
                const ValueInfo& xi = g_.values[x];
                if (xi.op != OpKind::Unary && xi.op != OpKind::Binary) continue;
                for (int in : xi.inputs) {
                    tree_uses[in]++;
                    stack.push_back(in);
                }
            }
        }
        // Inline as deep as the kernel's program and operand limits allow; on overflow retry with a
        // shallower cut (operands materialised by a failed attempt stay planned and are reused).
        static const int kDepths[] = {1 << 20, 12, 6, 3, 1, 0};
        for (int max_depth : kDepths) {
            ScalarBlock block;
            Ref r = build_scalar(root, 0, max_depth, block, tree_uses);
            if ((int)block.loads.size() + 1 > SCALAR_MAX_OPERANDS || (int)block.instrs.size() > SCALAR_MAX_INSTR) continue;
            PlanTensor out = alloc_shared(shape_of(root), g_.values[root].dtype, root);
            emit_scalar(block, {{out, r}}, root, "fused");
            return out;
        }
        fail(KN_ERR_INTERNAL, "elementwise operation does not fit one kernel");
    }

    Ref build_scalar(int v, int depth, int max_depth, ScalarBlock& block, const std::map<int, int>& tree_uses) {
        const bool is_root = depth == 0;
        if (!is_root) {
            auto cached = block.value_ref.find(v);
            if (cached != block.value_ref.end()) return cached->second;
            if (map_[v]) return block.load(*map_[v]);
        }
        const ValueInfo& info = g_.values[v];
        bool is_scalar_op = info.op == OpKind::Unary || info.op == OpKind::Binary;
        Ref result;
        if (!is_root && !is_scalar_op) {
            if (auto c = g_.as_single_const(v)) result = block.constant(*c);
            else result = block.load(visit(v));
        } else if (!is_root && (depth > max_depth || !can_inline(v, tree_uses))) {
            if (auto c = g_.as_single_const(v)) result = block.constant(*c);
            else result = block.load(visit(v));
        } else if (info.op == OpKind::Unary) {
            Ref a = build_scalar(info.inputs[0], depth + 1, max_depth, block, tree_uses);
            result = block.unary(info.unary_op, info.cast_from, info.dtype, a);
        } else {
            Ref a = build_scalar(info.inputs[0], depth + 1, max_depth, block, tree_uses);
            Ref b = build_scalar(info.inputs[1], depth + 1, max_depth, block, tree_uses);
            result = block.binary(info.binary_op, info.dtype, a, b);
        }
        block.value_ref[v] = result;
        return result;
    }

    bool can_inline(int v, const std::map<int, int>& tree_uses) {
        if (!g_.is_hidden(v)) return false;
        auto it = tree_uses.find(v);
        int in_tree = it == tree_uses.end() ? 0 : it->second;
        if (g_.values[v].non_output_uses != in_tree) return false;
        // a contraction epilogue takes precedence over inlining (planner.rs:881-893)
        if (match_epilogue(v).has_value()) return false;
        return true;
    }

    // ---------------------------------------------------------------- contraction + epilogue
    bool is_contraction(int v) const {
        const ValueInfo& info = g_.values[v];
        if (info.dtype != DType::F32) return false;
        if (info.op == OpKind::Conv) return info.shape.size() == 4;
        if (info.op == OpKind::MatMul) return true;
        return false;
    }
    bool fusable(int v) const { return g_.is_hidden_with_uses(v, 1); }

    // The contraction a chain of single-use Add / View nodes ends in, or -1.
    int chain_end(int v) {
        if (chain_cache_[v] != -2) return chain_cache_[v];
        const ValueInfo& info = g_.values[v];
        int r = -1;
        if (is_contraction(v)) {
            r = v;
        } else if (info.dtype == DType::F32 && info.op == OpKind::View) {
            int in = info.inputs[0];
            if (fusable(in)) r = chain_end(in);
        } else if (info.dtype == DType::F32 && info.op == OpKind::Binary && info.binary_op == BinaryOp::Add) {
            for (int side : info.inputs) {
                if (fusable(side)) {
                    int e = chain_end(side);
                    if (e >= 0) { r = e; break; }
                }
            }
        }
        chain_cache_[v] = r;
        return r;
    }

    struct Epilogue {
        int contraction = -1;
        Activation act = Activation::None;
        std::vector<int> addends;
    };

    // `root` = y * 0.5 * (1 + erf(y * sqrt(1/2))) as a product tree in any association, every node of it
    // hidden and used by this expression only (y itself twice: as a factor and inside erf): returns y, else -1.
    int match_gelu(int root) {
        const ValueInfo& ri = g_.values[root];
        if (ri.dtype != DType::F32 || ri.op != OpKind::Binary || ri.binary_op != BinaryOp::Mul) return -1;
        // flatten the product
        std::vector<int> factors, stack = {ri.inputs[1], ri.inputs[0]};
        while (!stack.empty()) {
            const int v = stack.back();
            stack.pop_back();
            const ValueInfo& vi = g_.values[v];
            if (vi.op == OpKind::Binary && vi.binary_op == BinaryOp::Mul && fusable(v) && !g_.as_single_const(v)) {
                stack.push_back(vi.inputs[1]);
                stack.push_back(vi.inputs[0]);
            } else {
                factors.push_back(v);
            }
            if (factors.size() > 3) return -1;
        }
        if (factors.size() != 3) return -1;
        int half = -1, y = -1, gate = -1;
        for (int v : factors) {
            auto c = g_.as_single_const(v);
            const ValueInfo& vi = g_.values[v];
            if (c && half < 0 && c->as_f32() == 0.5f) half = v;
            else if (vi.op == OpKind::Binary && vi.binary_op == BinaryOp::Add && fusable(v) && gate < 0 && !c) gate = v;
            else if (y < 0) y = v;
            else return -1;
        }
        if (half < 0 || y < 0 || gate < 0) return -1;
        // gate = 1 + erf(y * c)
        const ValueInfo& gi = g_.values[gate];
        int erf = -1;
        for (int side = 0; side < 2; side++) {
            auto one = g_.as_single_const(gi.inputs[side]);
            if (one && one->as_f32() == 1.0f) erf = gi.inputs[1 - side];
        }
        if (erf < 0) return -1;
        const ValueInfo& ei = g_.values[erf];
        if (ei.op != OpKind::Unary || ei.unary_op != UnaryOp::Erf || !fusable(erf)) return -1;
        const int arg = ei.inputs[0];
        const ValueInfo& ai = g_.values[arg];
        if (ai.op != OpKind::Binary || ai.binary_op != BinaryOp::Mul || !fusable(arg)) return -1;
        bool scaled = false;
        for (int side = 0; side < 2; side++) {
            auto c = g_.as_single_const(ai.inputs[side]);
            if (c && std::fabs(c->as_f32() - 0.70710678f) < 1e-6f && ai.inputs[1 - side] == y) scaled = true;
        }
        if (!scaled) return -1;
        // y feeds exactly the product and the erf argument, has the product's shape, and is a hidden value
        if (!g_.is_hidden_with_uses(y, 2) || g_.values[y].dtype != DType::F32 || shape_of(y) != shape_of(root)) return -1;
        return y;
    }

    // Matches  (relu | gelu)?( add*( view?( conv | matmul ) ) )  rooted at `root`
    // (generalises try_visit_fused_conv, kn-cuda-eval/src/planner.rs:669-833, to MatMul and to
    // addends of any broadcast shape).
    std::optional<Epilogue> match_epilogue(int root) {
        const ValueInfo& ri = g_.values[root];
        if (ri.dtype != DType::F32) return std::nullopt;
        Epilogue e;
        int curr = root;
        if (int y = match_gelu(root); y >= 0) {
            if (chain_end(y) < 0) return std::nullopt;
            curr = y;
            e.act = Activation::Gelu;
        } else if (ri.op == OpKind::Binary && ri.binary_op == BinaryOp::Max) {
            int l = ri.inputs[0], r = ri.inputs[1];
            if (g_.is_const_zero(r) && fusable(l) && chain_end(l) >= 0) { curr = l; e.act = Activation::Relu; }
            else if (g_.is_const_zero(l) && fusable(r) && chain_end(r) >= 0) { curr = r; e.act = Activation::Relu; }
            else return std::nullopt;
        }
        if (chain_end(curr) < 0) return std::nullopt;
        while (!is_contraction(curr)) {
            // (a node below the root that is planned already, as one of several projections computed by one matmul,
            // is read, not recomputed)
            if (curr != root && map_[curr]) return std::nullopt;
            const ValueInfo& ci = g_.values[curr];
            if (ci.op == OpKind::View) {
                curr = ci.inputs[0];
            } else {   // Add: continue on the side that reaches the contraction
                int l = ci.inputs[0], r = ci.inputs[1];
                int cont, other;
                if (fusable(l) && chain_end(l) >= 0) { cont = l; other = r; }
                else { cont = r; other = l; }
                if (e.addends.size() == 2) return std::nullopt;
                e.addends.push_back(other);
                curr = cont;
            }
        }
        if (curr != root && map_[curr]) return std::nullopt;
        e.contraction = curr;
        return e;
    }

    // ---------------------------------------------------------------- attention head split / merge read in place
    // Attention graphs spell the head split as view [B*S, H*D] -> [B, S, H, D], permute [0, 2, 1, 3], view -> [B*H, S, D]
    // and the merge as the same three nodes the other way round.  Neither result is expressible with strides (two
    // batch-like axes of the source with unrelated strides would have to merge), so planned node by node each costs a
    // copy of the activations.  A matmul operand of that form is instead read in place through a 4-D tensor map
    // (GemmOperand4D): this finds the source and the four extents.
    struct HeadChain {
        int src = -1;
        int64_t B = 0, S = 0, H = 0, D = 0;
        bool merge = false;
    };
    std::optional<HeadChain> match_head_chain(int v) {
        auto strip = [](std::vector<int64_t> s) {
            while (s.size() > 2 && s.front() == 1) s.erase(s.begin());
            return s;
        };
        if (map_[v]) return std::nullopt;                      // already materialised: use that
        const std::vector<int64_t> target = strip(shape_of(v));
        int cur = v;
        while (g_.values[cur].op == OpKind::View && !map_[cur]) cur = g_.values[cur].inputs[0];
        const ValueInfo& pi = g_.values[cur];
        if (cur == v || pi.op != OpKind::Permute || map_[cur] || pi.permutation != std::vector<int>{0, 2, 1, 3}) return std::nullopt;
        const int w = pi.inputs[0];
        if (g_.values[w].op != OpKind::View) return std::nullopt;
        const std::vector<int64_t> a = shape_of(w);            // [a0, a1, a2, a3] before the permute
        if (a.size() != 4) return std::nullopt;
        int src = w;
        while (g_.values[src].op == OpKind::View && !map_[src]) src = g_.values[src].inputs[0];
        const std::vector<int64_t> from = strip(shape_of(src));
        for (int64_t d : a)
            if (d < 1) return std::nullopt;
        HeadChain c;
        c.src = src;
        if (from == std::vector<int64_t>{a[0] * a[1], a[2] * a[3]} && target == std::vector<int64_t>{a[0] * a[2], a[1], a[3]}) {
            c.B = a[0]; c.S = a[1]; c.H = a[2]; c.D = a[3];
            c.merge = false;
            return c;
        }
        if (from == std::vector<int64_t>{a[0] * a[1], a[2], a[3]} && target == std::vector<int64_t>{a[0] * a[2], a[1] * a[3]}) {
            c.B = a[0]; c.H = a[1]; c.S = a[2]; c.D = a[3];
            c.merge = true;
            return c;
        }
        return std::nullopt;
    }
    // The 4-D description of a matmul operand that is such a chain (rows x K, K contiguous), or nothing.  `as_b`: the
    // operand is B, given in the graph as [batch, K, rows], so the chain sits under a permute [0, 2, 1].
    // Sets `source` to the planned source tensor (visited here) on success.
    bool head_chain_operand(int value, bool as_b, DType dtype, GemmOperand4D* out, PlanTensor* source, int64_t* batch, int64_t* rows,
                            int64_t* k) {
        if (opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM) return false;
        if (as_b) {
            const ValueInfo& vi = g_.values[value];
            if (map_[value] || vi.op != OpKind::Permute || vi.permutation != std::vector<int>{0, 2, 1}) return false;
            value = vi.inputs[0];
        }
        if (shape_of(value).size() != 3) return false;
        auto c = match_head_chain(value);
        if (!c) return false;
        const int64_t block_k = dtype == DType::F16 ? 64 : 32, align = dtype == DType::F16 ? 8 : 4;
        if (g_.values[c->src].dtype != dtype || c->D % align != 0 || c->B > 65535 || c->H > 65535) return false;
        GemmOperand4D o{};
        o.enabled = 1;
        o.dims[0] = c->D; o.dims[1] = c->S; o.dims[2] = c->H; o.dims[3] = c->B;
        o.strides[0] = 1;
        if (!c->merge) {
            // [B*S, H*D] read as [B*H, S, D]
            o.strides[1] = c->H * c->D; o.strides[2] = c->D; o.strides[3] = c->S * c->H * c->D;
            o.kd = (int32_t)c->D; o.rd = (int32_t)c->S; o.bi = (int32_t)c->H;
            *batch = c->B * c->H; *rows = c->S; *k = c->D;
            if (c->S < 64) return false;
        } else {
            // [B*H, S, D] read as [B*S, H*D]: the K offset is split into (head, offset), whole K blocks per head, and a
            // tile's rows must lie inside one batch entry
            if (as_b || c->D % block_k != 0 || (c->D & (c->D - 1)) != 0 || c->S % 128 != 0) return false;
            o.strides[1] = c->D; o.strides[2] = c->S * c->D; o.strides[3] = c->H * c->S * c->D;
            o.kd = (int32_t)c->D; o.rd = (int32_t)c->S; o.bi = 1;
            *batch = 1; *rows = c->B * c->S; *k = c->H * c->D;
        }
        PlanTensor t = visit(c->src);
        if (t.offset % align != 0) return false;   // (the source is planned either way)
        if (!t.ss.has_simple_strides()) {
            // a head split of a column slice of a wider matrix (one of several projections computed as one matmul):
            // the rows are further apart, nothing else changes
            if (c->merge) return false;
            auto rows = t.ss.view({c->B * c->S, c->H * c->D});   // (whatever leading axes the source has)
            if (!rows || rows->strides[1] != 1 || rows->strides[0] < c->H * c->D || rows->strides[0] % align != 0) return false;
            o.strides[1] = rows->strides[0];
            o.strides[3] = c->S * rows->strides[0];
        }
        *out = o;
        *source = t;
        return true;
    }

    // ---------------------------------------------------------------- attention scores + softmax as one step
    // softmax over the last axis of (scale *) a batched matmul whose rows are at most 512 long (the scores of an
    // attention head over up to 512 keys), every node in between used by this expression only: ONE tensor-core step
    // that keeps the scores in tensor memory and writes the probabilities (kernels/attn_softmax.cu), instead of a
    // matmul that writes the scores and a softmax that reads and writes them again.
    //
    // With `context` (a matmul whose left operand is that softmax and nothing else reads it, V of 32 or 64 columns) the
    // step goes on to probabilities . V: the probabilities never reach memory either (kernels/attention.cu).
    std::optional<PlanTensor> try_fused_attention_scores(int v) { return plan_attention(v, -1); }

    std::optional<PlanTensor> try_fused_attention_context(int v) {
        const ValueInfo& mi = g_.values[v];
        if (mi.op != OpKind::MatMul || mi.dtype != DType::F32 || shape_of(v).size() != 3) return std::nullopt;
        const int sv = mi.inputs[0];
        if (g_.values[sv].op != OpKind::Softmax || !fusable(sv) || map_[sv] || mi.inputs[1] == sv) return std::nullopt;
        const std::vector<int64_t> ps = shape_of(sv), vs = shape_of(mi.inputs[1]);
        if (ps.size() != 3 || vs.size() != 3 || vs[0] != ps[0]) return std::nullopt;
        const int q = plan_attention_query(sv);
        if (q < 0 || !attention_fits(ps[0], ps[1], ps[2], shape_of(q)[2], vs[2])) return std::nullopt;
        return plan_attention(sv, v);
    }

    // the left operand of the scores matmul if `v` is a softmax the fused attention steps take, else -1
    int plan_attention_query(int v) {
        const ValueInfo& si = g_.values[v];
        if (si.dtype != DType::F32 || opts_.math_mode != KN_MATH_TF32 || (opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM)) return -1;
        if (shape_of(v).size() != 3 || si.axis != 2) return -1;
        float scale = 1.0f;
        const int y = peel_positive_scale(si.inputs[0], &scale);
        if (y < 0) return -1;
        const ValueInfo& ci = g_.values[y];
        if (ci.op != OpKind::MatMul || ci.dtype != DType::F32 || !fusable(y) || map_[y] || shape_of(y) != shape_of(v)) return -1;
        return ci.inputs[0];
    }

    // `y`, or what `y` scales if it is x * c, c * x or x / c with a positive finite constant c that only this expression
    // reads (the attention kernels take the row maximum before scaling); -1 if it scales by anything else.
    int peel_positive_scale(int y, float* scale) {
        const ValueInfo& mi = g_.values[y];
        if (mi.op != OpKind::Binary || !fusable(y) || map_[y]) return y;
        if (mi.binary_op != BinaryOp::Mul && mi.binary_op != BinaryOp::Div) return y;
        auto c0 = g_.as_single_const(mi.inputs[0]), c1 = g_.as_single_const(mi.inputs[1]);
        float c;
        int other;
        if (c1) c = c1->as_f32(), other = mi.inputs[0];
        else if (c0 && mi.binary_op == BinaryOp::Mul) c = c0->as_f32(), other = mi.inputs[1];
        else return -1;
        if (mi.binary_op == BinaryOp::Div) c = 1.0f / c;
        if (!(c > 0.0f) || !std::isfinite(c)) return -1;
        *scale = c;
        return other;
    }

    std::optional<PlanTensor> plan_attention(int v, int context) {
        const ValueInfo& si = g_.values[v];
        if (si.dtype != DType::F32 || opts_.math_mode != KN_MATH_TF32 || (opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM)) return std::nullopt;
        const std::vector<int64_t> shape = shape_of(v);
        if (shape.size() != 3 || si.axis != 2) return std::nullopt;
        float scale = 1.0f;
        const int y = peel_positive_scale(si.inputs[0], &scale);
        if (y < 0) return std::nullopt;
        const ValueInfo& ci = g_.values[y];
        if (ci.op != OpKind::MatMul || ci.dtype != DType::F32 || !fusable(y) || map_[y] || shape_of(y) != shape) return std::nullopt;
        const int64_t batch = shape[0], m = shape[1], n = shape[2];
        const int64_t k = shape_of(ci.inputs[0])[2];
        if (!attn_softmax_fits(batch, m, n, k)) return std::nullopt;
        // operands: head splits read in place, or K-contiguous matrices as they are
        GemmOperand4D a4{}, b4{};
        int64_t ob = 0, orows = 0, ok_ = 0;
        PlanTensor x, w;
        if (!(head_chain_operand(ci.inputs[0], false, DType::F32, &a4, &x, &ob, &orows, &ok_) && a4.kd == k && ob == batch && orows == m))
            a4 = GemmOperand4D{};
        if (!a4.enabled) x = visit(ci.inputs[0]);
        if (!(head_chain_operand(ci.inputs[1], true, DType::F32, &b4, &w, &ob, &orows, &ok_) && b4.kd == k && ob == batch && orows == n))
            b4 = GemmOperand4D{};
        if (!b4.enabled) w = visit(ci.inputs[1]);
        PlanTensor xc = x, wc = w;   // what the shape checks see
        if (a4.enabled) xc.ss = StridedShape({batch, m, k}, {m * k, k, 1}), xc.offset = 0;
        if (b4.enabled) wc.ss = StridedShape({batch, k, n}, {n * k, 1, k}), wc.offset = 0;
        if (xc.ss.rank() != 3 || wc.ss.rank() != 3 || !gemm_fits_tensor_core(xc, wc) || xc.ss.strides[0] == 0 || wc.ss.strides[0] == 0)
            return std::nullopt;   // (the operands are planned either way; the matmul and the softmax stay two steps)
        PlanTensor values;
        GemmOperand4D v4{};
        bool values_mn = false;
        int64_t dv = 0;
        if (context >= 0) {
            // V [batch, keys, dv]: a head split read in place or a tensor with its columns contiguous (the MN-major B
            // operand of the context MMAs), or one with its keys contiguous (K-major); anything else gets a copy
            const int vin = g_.values[context].inputs[1];
            dv = shape_of(vin)[2];
            if (head_chain_operand(vin, false, DType::F32, &v4, &values, &ob, &orows, &ok_) && v4.kd == dv && ob == batch && orows == n) {
                values_mn = true;
            } else {
                v4 = GemmOperand4D{};
                values = visit(vin);
                const auto& vs = values.ss.strides;
                if (vs[2] == 1 && vs[1] % 4 == 0 && vs[0] % 4 == 0 && (batch == 1 || vs[0] != 0) && values.offset % 4 == 0) {
                    values_mn = true;
                } else {
                    values = k_major_b(values, vin);
                    const auto& st = values.ss.strides;
                    if (st[1] != 1 || st[2] % 4 != 0 || st[0] % 4 != 0 || (batch > 1 && st[0] == 0) || values.offset % 4 != 0)
                        return std::nullopt;   // (planned as separate steps; V stays planned)
                }
            }
        }
        if (context >= 0) {
            // the softmax and its matmul are part of this step: nothing else reads them (checked by the caller)
            PlanTensor out = alloc_shared({batch, m, dv}, DType::F32, context);
            Step s;
            s.kind = StepKind::Gemm;
            s.value = context;
            s.tensor_core = true;
            s.operands = {x, w, out, values};
            s.writes = {0, 0, 1, 0};
            GemmParams& p = s.gemm;
            p.batch = batch;
            p.m = m;
            p.n = n;
            p.k = k;
            p.a4 = a4;
            p.b4 = b4;
            for (int i = 0; i < 3; i++) {
                if (!a4.enabled) p.sa[i] = x.ss.strides[i];
                if (!b4.enabled) p.sb[i] = w.ss.strides[i];
                p.sc[i] = out.ss.strides[i];
            }
            p.values_mn = values_mn ? 1 : 0;
            p.v4 = v4;
            if (values_mn && !v4.enabled) {
                for (int i = 0; i < 3; i++) p.values_strides[i] = values.ss.strides[i];   // V [batch][keys][dv]
            } else if (!values_mn) {
                p.values_strides[0] = values.ss.strides[0];   // V^T [batch][dv][keys]
                p.values_strides[1] = values.ss.strides[2];
                p.values_strides[2] = values.ss.strides[1];
            }
            p.values_cols = dv;
            p.splits = 1;
            p.row_softmax = 2;
            p.softmax_scale = scale;
            s.flops = 2.0 * (double)batch * (double)m * (double)n * (double)(k + dv);
            s.desc = "attention b=" + std::to_string(batch) + " m=" + std::to_string(m) + " keys=" + std::to_string(n) + " k=" + std::to_string(k) +
                     " dv=" + std::to_string(dv) + " tf32 (scores and probabilities stay in tensor memory)";
            if (a4.enabled || b4.enabled || v4.enabled) {
                std::string which;
                for (const char* name : {a4.enabled ? "a" : "", b4.enabled ? "b" : "", v4.enabled ? "v" : ""})
                    if (*name) which += (which.empty() ? "" : ", ") + std::string(name);
                s.desc += std::string(" (head split read in place: operand") + (which.size() > 1 ? "s " : " ") + which + ")";
            }
            push_step(std::move(s));
            return out;
        }
        PlanTensor out = alloc_shared(shape, DType::F32, v);
        Step s;
        s.kind = StepKind::Gemm;
        s.value = v;
        s.tensor_core = true;
        s.operands = {x, w, out};
        s.writes = {0, 0, 1};
        GemmParams& p = s.gemm;
        p.batch = batch;
        p.m = m;
        p.n = n;
        p.k = k;
        p.a4 = a4;
        p.b4 = b4;
        for (int i = 0; i < 3; i++) {
            if (!a4.enabled) p.sa[i] = x.ss.strides[i];
            if (!b4.enabled) p.sb[i] = w.ss.strides[i];
            p.sc[i] = out.ss.strides[i];
        }
        p.splits = 1;
        p.row_softmax = 1;
        p.softmax_scale = scale;
        s.flops = 2.0 * (double)batch * (double)m * (double)n * (double)k;
        s.desc = "matmul b=" + std::to_string(batch) + " m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" + std::to_string(k) +
                 " +0 tf32 row softmax";
        if (a4.enabled || b4.enabled)
            s.desc += std::string(" (head split read in place: operand") + (a4.enabled && b4.enabled ? "s a, b" : (a4.enabled ? " a" : " b")) + ")";
        push_step(std::move(s));
        return out;
    }

    // ---------------------------------------------------------------- projections of one tensor as one matmul
    // x . W1 + b1, x . W2 + b2, ... (the query / key / value projections of an attention block) with constant weights
    // and biases: ONE matmul x . [W1 W2 ...] + [b1 b2 ...] into one buffer of which every projection is a column
    // slice.  Three matmuls of 16384 x 768 x 768 are 2.6 rounds of tiles each on 74 CTA pairs, with the first loads and
    // the last epilogue exposed three times; one of 16384 x 2304 x 768 is 7.8 rounds.  The weights and biases are
    // concatenated here, on the host, once.
    struct Projection {
        int root, matmul;
        PlanTensor weight, bias;   // constants: [1, K, N] and anything that broadcasts to [1, 1, N]
        bool has_bias;
        int64_t n;
    };
    // `v` is read, through any views / permutes / slices (the head split of an attention block), by matmuls only: no
    // bias, residual or activation that would have been its epilogue
    void ensure_readers() {
        if (!readers_.empty()) return;
        readers_.resize(g_.values.size());
        matmuls_of_.resize(g_.values.size());
        for (int u = 0; u < (int)g_.values.size(); u++) {
            for (int in : g_.values[u].inputs) readers_[in].push_back(u);
            if (g_.values[u].op == OpKind::MatMul) matmuls_of_[g_.values[u].inputs[0]].push_back(u);
        }
    }
    bool only_contraction_readers(int v) {
        ensure_readers();
        for (int u : readers_[v]) {
            const OpKind op = g_.values[u].op;
            if (op == OpKind::View || op == OpKind::Permute || op == OpKind::Slice) {
                if (!only_contraction_readers(u)) return false;
            } else if (op != OpKind::MatMul) {
                return false;
            }
        }
        return true;
    }
    std::vector<std::vector<int>> readers_, matmuls_of_;   // per value: the values that read it; the matmuls whose left operand it is
    // a constant seen through operations that only edit strides: planning it emits no step
    bool is_constant_view(int v) const {
        for (;;) {
            const ValueInfo& vi = g_.values[v];
            if (vi.op == OpKind::Constant) return true;
            if (vi.op != OpKind::View && vi.op != OpKind::Permute && vi.op != OpKind::Broadcast && vi.op != OpKind::Slice && vi.op != OpKind::Flip)
                return false;
            v = vi.inputs[0];
        }
    }
    std::optional<Projection> as_projection(int root, int x) {
        if (map_[root] || g_.values[root].dtype != DType::F32) return std::nullopt;
        auto e = match_epilogue(root);
        if (!e || e->act != Activation::None || e->addends.size() > 1) return std::nullopt;
        const ValueInfo& ci = g_.values[e->contraction];
        if (ci.op != OpKind::MatMul || ci.dtype != DType::F32 || map_[e->contraction] || ci.inputs[0] != x) return std::nullopt;
        // [1, M, N] out of the matmul; the sum may be over a view of it that keeps the columns ([M, N])
        const std::vector<int64_t> shape = shape_of(e->contraction), rs = shape_of(root);
        int64_t root_elems = 1;
        for (int64_t d : rs) root_elems *= d;
        if (shape.size() != 3 || shape[0] != 1 || rs.empty() || rs.back() != shape[2] || root_elems != shape[1] * shape[2]) return std::nullopt;
        Projection p;
        p.has_bias = !e->addends.empty();
        if (!is_constant_view(ci.inputs[1]) || (p.has_bias && !is_constant_view(e->addends[0]))) return std::nullopt;
        p.root = root;
        p.matmul = e->contraction;
        p.n = shape[2];
        p.weight = visit(ci.inputs[1]);
        auto is_host_const = [&](const PlanTensor& t) {
            const BufferInfo& b = plan_.buffers[t.buf];
            return b.kind == BufKind::Const && b.host_data != nullptr && t.dtype == DType::F32;
        };
        if (!is_host_const(p.weight) || p.weight.ss.rank() != 3 || p.n % 4 != 0) return std::nullopt;
        if (!p.has_bias) return p;
        p.bias = visit(e->addends[0]);
        if (!is_host_const(p.bias)) return std::nullopt;
        // the bias must be one value per column
        const std::vector<int64_t>& bs = p.bias.ss.shape;
        if (bs.empty() || bs.back() != p.n) return std::nullopt;
        for (size_t d = 0; d + 1 < bs.size(); d++)
            if (bs[d] != 1 && p.bias.ss.strides[d] != 0) return std::nullopt;
        return p;
    }

    std::optional<PlanTensor> try_merged_projections(int root) {
        if (opts_.math_mode != KN_MATH_TF32 || (opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM)) return std::nullopt;
        auto head = match_epilogue(root);
        if (!head || g_.values[head->contraction].op != OpKind::MatMul) return std::nullopt;
        const int x = g_.values[head->contraction].inputs[0];
        auto first = as_projection(root, x);
        if (!first) return std::nullopt;
        const std::vector<int64_t> xs = shape_of(x);
        const int64_t m = xs[1], k = xs[2];
        if (m < 256 || k % 4 != 0) return std::nullopt;
        // the other projections of x: an Add over a MatMul of x that nothing else reads
        std::vector<Projection> all{*first};
        ensure_readers();
        for (int mm : matmuls_of_[x]) {
            if (all.size() >= 8) break;
            if (map_[mm]) continue;
            bool seen = false;
            for (auto& have : all) seen = seen || have.matmul == mm;
            if (seen) continue;
            // the sum over it (through views that nothing else reads), or the matmul itself if only matmuls read it
            int cur = mm;
            while (readers_[cur].size() == 1 && g_.values[readers_[cur][0]].op == OpKind::View && fusable(cur)) cur = readers_[cur][0];
            int candidate = -1;
            if (readers_[cur].size() == 1 && fusable(cur)) {
                const ValueInfo& ri = g_.values[readers_[cur][0]];
                if (ri.op == OpKind::Binary && ri.binary_op == BinaryOp::Add) candidate = readers_[cur][0];
            }
            if (candidate < 0 && only_contraction_readers(mm)) candidate = mm;
            if (candidate < 0 || candidate == root || map_[candidate]) continue;
            if (auto p = as_projection(candidate, x))
                if (p->matmul == mm) all.push_back(*p);
        }
        if (all.size() < 2) return std::nullopt;
        int64_t n_total = 0;
        for (auto& p : all) n_total += p.n;
        // only where the separate matmuls leave CTA pairs idle in their last round of 256 x 256 tiles
        auto rounds = [&](int64_t n) { return (double)(((m + 255) / 256) * ((n + 255) / 256)) / 74.0; };
        double separate = 0;
        for (auto& p : all) separate += std::ceil(rounds(p.n));
        if (std::ceil(rounds(n_total)) >= separate || n_total > (1 << 20)) return std::nullopt;
        // (a result of few tiles under a long reduction is cut along K by the planner: not here)
        if (((m + 127) / 128) * ((n_total + 255) / 256) < 74 && k >= 512) return std::nullopt;
        bool any_bias = false;
        for (auto& p : all) any_bias = any_bias || p.has_bias;
        PlanTensor xt = visit(x);
        if (xt.ss.rank() != 3 || xt.ss.strides[2] != 1 || !tma_stride_ok(m, xt.ss.strides[1]) || xt.offset % 4 != 0) return std::nullopt;
        // [n_total][k] with k contiguous, and the biases side by side
        auto wdata = std::make_shared<std::vector<uint8_t>>((size_t)(n_total * k) * 4);
        auto bdata = std::make_shared<std::vector<uint8_t>>((size_t)n_total * 4);
        float* wd = (float*)wdata->data();
        float* bd = (float*)bdata->data();
        int64_t col = 0;
        for (auto& p : all) {
            if (p.weight.ss.shape[1] != k || p.weight.ss.shape[2] != p.n) return std::nullopt;
            const float* ws = (const float*)plan_.buffers[p.weight.buf].host_data + p.weight.offset;
            const float* bs = p.has_bias ? (const float*)plan_.buffers[p.bias.buf].host_data + p.bias.offset : nullptr;
            const int64_t sk = p.weight.ss.strides[1], sn = p.weight.ss.strides[2], sb = p.has_bias ? p.bias.ss.strides.back() : 0;
            for (int64_t j = 0; j < p.n; j++) {
                for (int64_t i = 0; i < k; i++) wd[(col + j) * k + i] = ws[i * sk + j * sn];
                bd[col + j] = bs ? bs[j * sb] : 0.0f;
            }
            col += p.n;
        }
        PlanTensor w = alloc_const({1, n_total, k}, DType::F32, all[0].matmul, nullptr, wdata);
        w = w.with(w.ss.permute({0, 2, 1}));                                  // logical [1, k, n_total], k contiguous
        PlanTensor bias;
        if (any_bias) {
            bias = alloc_const({1, 1, n_total}, DType::F32, all[0].root, nullptr, bdata);
            bias = bias.with(StridedShape({1, m, n_total}, {0, 0, 1}));
        }
        PlanTensor out = alloc_shared({1, m, n_total}, DType::F32, root);
        if (!gemm_fits_tensor_core(xt, w)) return std::nullopt;
        Step s;
        s.kind = StepKind::Gemm;
        s.value = root;
        s.tensor_core = true;
        s.operands = {xt, w, out};
        s.writes = {0, 0, 1};
        if (any_bias) {
            s.operands.push_back(bias);
            s.writes.push_back(0);
        }
        GemmParams& p = s.gemm;
        p.batch = 1;
        p.m = m;
        p.n = n_total;
        p.k = k;
        for (int i = 0; i < 3; i++) {
            p.sa[i] = xt.ss.strides[i];
            p.sb[i] = w.ss.strides[i];
            p.sc[i] = out.ss.strides[i];
            if (any_bias) p.s1[i] = bias.ss.strides[i];
        }
        p.splits = 1;
        s.flops = 2.0 * (double)m * (double)n_total * (double)k;
        s.desc = "matmul b=1 m=" + std::to_string(m) + " n=" + std::to_string(n_total) + " k=" + std::to_string(k) + (any_bias ? " +1" : " +0") + " tf32 (" +
                 std::to_string(all.size()) + " projections of one tensor)";
        push_step(std::move(s));
        // every projection is a column slice of the result, seen in the shape of its sum
        col = 0;
        PlanTensor mine;
        for (auto& pr : all) {
            PlanTensor slice = out.slice(2, col, col + pr.n, 1);
            auto shaped = slice.ss.view(shape_of(pr.root));
            KN_CHECK(shaped.has_value(), KN_ERR_INTERNAL, "column slice of merged projections is not viewable");
            slice = slice.with(*shaped);
            if (pr.root == root) mine = slice;
            else map_[pr.root] = slice;
            col += pr.n;
        }
        return mine;
    }

    std::optional<PlanTensor> try_fused_contraction(int root) {
        if (auto merged = try_merged_projections(root)) return *merged;
        auto m = match_epilogue(root);
        if (!m) return std::nullopt;
        const ValueInfo& ci = g_.values[m->contraction];
        std::vector<int64_t> native = shape_of(m->contraction);
        std::vector<int64_t> root_shape = shape_of(root);

        // operands first (they may emit steps of their own), then this step
        // (a matmul operand that is an attention head split or merge is read in place: tensor cores only)
        GemmOperand4D a4{}, b4{};
        int64_t a4_batch = 0, a4_rows = 0, a4_k = 0, b4_batch = 0, b4_rows = 0, b4_k = 0;
        PlanTensor x, w;
        const bool heads_ok = ci.op == OpKind::MatMul && native.size() == 3 && native[2] >= 16 && native[2] % 4 == 0 &&
                              (ci.dtype == DType::F16 || (ci.dtype == DType::F32 && opts_.math_mode == KN_MATH_TF32));
        if (!(heads_ok && head_chain_operand(ci.inputs[0], false, ci.dtype, &a4, &x, &a4_batch, &a4_rows, &a4_k) &&
              a4_batch * 1 == native[0] * 1 && a4_rows == native[1]))
            a4 = GemmOperand4D{};
        if (!a4.enabled) x = visit(ci.inputs[0]);
        if (!(heads_ok && head_chain_operand(ci.inputs[1], true, ci.dtype, &b4, &w, &b4_batch, &b4_rows, &b4_k) && b4_batch == native[0] &&
              b4_rows == native[2]))
            b4 = GemmOperand4D{};
        if (!b4.enabled) w = visit(ci.inputs[1]);
        std::vector<PlanTensor> addends;
        for (int a : m->addends) {
            PlanTensor t = visit(a);
            auto s = t.ss.view(native);
            if (!s) {
                if (m->contraction == root) fail(KN_ERR_INTERNAL, "bare contraction with addends");
                return std::nullopt;   // planned unfused instead
            }
            addends.push_back(t.with(*s));
        }
        PlanTensor out;
        bool tensor_core = false, as_gemm = false;
        PlanTensor conv_view;   // as_gemm: the matmul's output seen as [N, K, OH, OW]
        ConvGemm implicit;      // as_gemm with an implicit operand (implicit.implicit != 0)
        if (opts_.math_mode == KN_MATH_TF32) {
            if (ci.op == OpKind::MatMul && (a4.enabled || b4.enabled)) {
                // operands read in place: the other operand must be fine as it is, and the addends ones the persistent
                // kernel's epilogue takes (per row, per column, or per element with contiguous rows); else back to
                // materialised operands
                PlanTensor xc = x, wc = w;   // what the shape checks see
                if (a4.enabled) xc.ss = StridedShape({a4_batch, a4_rows, a4_k}, {a4_rows * a4_k, a4_k, 1}), xc.offset = 0;
                if (b4.enabled) wc.ss = StridedShape({b4_batch, b4_k, b4_rows}, {b4_rows * b4_k, 1, b4_k}), wc.offset = 0;
                bool ok = xc.ss.rank() == 3 && wc.ss.rank() == 3 && xc.ss.shape[2] == wc.ss.shape[1] && gemm_fits_tensor_core(xc, wc);
                for (const PlanTensor& t : addends) {
                    const auto& st = t.ss.strides;
                    if (!(st[1] == 0 || st[2] == 1 || st[2] == 0)) ok = false;
                }
                if (ok) {
                    tensor_core = true;
                } else {
                    a4 = GemmOperand4D{};
                    b4 = GemmOperand4D{};
                    x = visit(ci.inputs[0]);
                    w = visit(ci.inputs[1]);
                }
            }
            if (ci.op == OpKind::MatMul) {
                // An operand that is not contiguous along K (the value matrix of an attention head arrives as
                // [batch, k, n] with n contiguous) gets a transposing copy: the exact-f32 kernel this would
                // otherwise fall back to is some twenty times slower than copy + tensor cores.
                if (!a4.enabled && !b4.enabled) {
                    if (!gemm_fits_tensor_core(x, w) && gemm_worth_a_copy(x, w)) {
                        PlanTensor x2 = k_major_a(x, ci.inputs[0]), w2 = k_major_b(w, ci.inputs[1]);
                        if (gemm_fits_tensor_core(x2, w2)) {
                            x = x2;
                            w = w2;
                        }
                    }
                    tensor_core = gemm_fits_tensor_core(x, w);
                }
            }
            else if (auto g = conv_as_gemm(ci, x, w, native, addends, root)) {
                // im2col + batched matmul (see conv_as_gemm); from here on this is a matmul step
                x = g->a;
                w = g->b;
                out = g->c;
                addends = g->addends;
                conv_view = g->result;
                as_gemm = true;
                tensor_core = true;
                implicit = *g;
            }
            else tensor_core = conv_fits_tensor_core(ci, x, w, native);
        }
        if (tensor_core && ci.op == OpKind::Conv && !as_gemm) {
            x = channels_last(x, ci.inputs[0]);
            w = tap_major_filter(w, ci.inputs[1]);
            // keep the activation channels-last while it flows from convolution to convolution
            if (root_shape == native && native[1] % 4 == 0 && feeds_tensor_core_conv(root)) {
                out = alloc_shared({native[0], native[2], native[3], native[1]}, DType::F32, root);
                out = out.with(out.ss.permute({0, 3, 1, 2}));
            }
        }
        if (out.buf < 0) out = alloc_shared(native, DType::F32, root);

        Step s;
        s.value = root;
        s.tensor_core = tensor_core;
        s.operands = {x, w, out};
        s.writes = {0, 0, 1};
        for (auto& a : addends) {
            s.operands.push_back(a);
            s.writes.push_back(0);
        }
        if (ci.op == OpKind::MatMul || as_gemm) {
            s.kind = StepKind::Gemm;
            GemmParams& p = s.gemm;
            if (implicit.implicit != 0) {
                // the image tensor stands for operand a or b: its strides go to the convolution fields
                const PlanTensor& img = implicit.implicit == 1 ? x : w;
                p.batch = implicit.batch;
                p.m = implicit.m;
                p.n = implicit.n;
                p.k = implicit.k;
                p.conv_operand = implicit.implicit;
                p.conv_c = (int32_t)img.ss.shape[1];
                p.conv_h = (int32_t)img.ss.shape[2];
                p.conv_w = (int32_t)img.ss.shape[3];
                p.conv_ow = (int32_t)native[3];
                const std::vector<int64_t> filter_shape = shape_of(ci.inputs[1]);
                p.conv_r = (int32_t)filter_shape[2];
                p.conv_s = (int32_t)filter_shape[3];
                p.conv_pad_y = ci.pad_y;
                p.conv_pad_x = ci.pad_x;
                p.conv_strides[0] = img.ss.strides[0];
                p.conv_strides[1] = img.ss.strides[2];
                p.conv_strides[2] = img.ss.strides[3];
            } else if (a4.enabled || b4.enabled) {
                // attention head split / merge read in place: the source tensors stand for the operands
                p.batch = native[0];
                p.m = native[1];
                p.n = native[2];
                p.k = a4.enabled ? a4_k : x.ss.shape[2];
                p.a4 = a4;
                p.b4 = b4;
            } else {
                KN_CHECK(x.ss.rank() == 3 && w.ss.rank() == 3, KN_ERR_SHAPE, "matmul operands must have rank 3");
                p.batch = x.ss.shape[0];
                p.m = x.ss.shape[1];
                p.k = x.ss.shape[2];
                p.n = w.ss.shape[2];
                KN_CHECK(w.ss.shape[0] == p.batch && w.ss.shape[1] == p.k, KN_ERR_SHAPE, "matmul operand shapes differ");
            }
            for (int i = 0; i < 3; i++) {
                if (implicit.implicit != 1 && !a4.enabled) p.sa[i] = x.ss.strides[i];
                if (implicit.implicit != 2 && !b4.enabled) p.sb[i] = w.ss.strides[i];
                p.sc[i] = out.ss.strides[i];
                if (addends.size() > 0) p.s1[i] = addends[0].ss.strides[i];
                if (addends.size() > 1) p.s2[i] = addends[1].ss.strides[i];
            }
            p.act = (int32_t)m->act;
            p.splits = 1;
            if (tensor_core) {
                // A contraction with few output tiles but a long K would leave most SMs idle: cut K into
                // slices computed by separate CTAs.  Their partial tiles go to a scratch buffer of the
                // arena (live only during this step) and a second small kernel sums them.
                const int64_t n_blocks = (p.n + 255) / 256;   // the persistent kernel's column blocks
                const int64_t bn = std::min<int64_t>(((p.n + n_blocks - 1) / n_blocks + 31) / 32 * 32, 256);
                const int64_t tiles = ((p.m + 127) / 128) * ((p.n + bn - 1) / bn) * p.batch;
                const int64_t k_blocks = (p.k + 31) / 32;
                if (tiles < 74 && k_blocks >= 16) {
                    // aim at one CTA per SM
                    int64_t splits = std::min<int64_t>(std::min<int64_t>(k_blocks / 4, (148 + tiles - 1) / tiles), 32);
                    if (splits > 1) {
                        const int64_t per = (k_blocks + splits - 1) / splits;
                        splits = (k_blocks + per - 1) / per;
                        p.splits = (int32_t)splits;
                        PlanTensor scratch = alloc_shared({p.batch, splits, p.m, p.n}, DType::F32, root);
                        s.operands.push_back(scratch);
                        s.writes.push_back(1);
                        s.launches = 2;
                    }
                }
            }
            s.flops = 2.0 * (double)p.batch * (double)p.m * (double)p.n * (double)p.k;
            s.desc = "matmul b=" + std::to_string(p.batch) + " m=" + std::to_string(p.m) + " n=" + std::to_string(p.n) +
                     " k=" + std::to_string(p.k);
        } else {
            KN_CHECK(x.ss.rank() == 4 && w.ss.rank() == 4, KN_ERR_SHAPE, "conv operands must have rank 4");
            s.kind = StepKind::Conv;
            ConvParams& p = s.conv;
            p.n = (int32_t)x.ss.shape[0];
            p.c = (int32_t)x.ss.shape[1];
            p.h = (int32_t)x.ss.shape[2];
            p.w = (int32_t)x.ss.shape[3];
            p.k = (int32_t)w.ss.shape[0];
            p.r = (int32_t)w.ss.shape[2];
            p.s = (int32_t)w.ss.shape[3];
            KN_CHECK(w.ss.shape[1] == p.c, KN_ERR_SHAPE, "conv channel mismatch");
            p.stride_y = ci.stride_y;
            p.stride_x = ci.stride_x;
            p.pad_y = ci.pad_y;
            p.pad_x = ci.pad_x;
            p.oh = (int32_t)native[2];
            p.ow = (int32_t)native[3];
            KN_CHECK(native[0] == p.n && native[1] == p.k, KN_ERR_SHAPE, "conv output shape mismatch");
            KN_CHECK((p.h + 2 * p.pad_y - p.r) / p.stride_y + 1 == p.oh && (p.w + 2 * p.pad_x - p.s) / p.stride_x + 1 == p.ow,
                     KN_ERR_SHAPE, "conv output extent does not match stride and padding");
            for (int i = 0; i < 4; i++) {
                p.s_in[i] = x.ss.strides[i];
                p.s_f[i] = w.ss.strides[i];
                p.s_out[i] = out.ss.strides[i];
                if (addends.size() > 0) p.s1[i] = addends[0].ss.strides[i];
                if (addends.size() > 1) p.s2[i] = addends[1].ss.strides[i];
            }
            p.act = (int32_t)m->act;
            s.flops = 2.0 * (double)p.n * p.k * p.c * p.r * p.s * p.oh * p.ow;
            s.desc = "conv n=" + std::to_string(p.n) + " c=" + std::to_string(p.c) + " hw=" + std::to_string(p.h) + "x" +
                     std::to_string(p.w) + " k=" + std::to_string(p.k) + " rs=" + std::to_string(p.r) + "x" + std::to_string(p.s);
        }
        s.desc += std::string(" +") + std::to_string(addends.size()) +
                  (m->act == Activation::Relu ? " relu" : (m->act == Activation::Gelu ? " gelu" : ""));
        if (tensor_core) s.desc += " tf32";
        if (s.kind == StepKind::Gemm && s.gemm.splits > 1) s.desc += " splitk=" + std::to_string(s.gemm.splits);
        int64_t total = 1;
        for (int64_t d : native) total *= d;
        if (a4.enabled || b4.enabled)
            s.desc += std::string(" (head ") + ((a4.enabled && a4.bi == 1) ? "merge" : "split") + " read in place: operand" +
                      (a4.enabled && b4.enabled ? "s a, b" : (a4.enabled ? " a" : " b")) + ")";
        if (as_gemm && implicit.implicit != 0)
            s.desc += std::string(" (conv, windows read from the image as operand ") + (implicit.implicit == 1 ? "a" : "b") + ")";
        else if (as_gemm) s.desc += " (conv via im2col, stride " + std::to_string(ci.stride_y) + "x" + std::to_string(ci.stride_x) + ")";
        if (total != 0) push_step(std::move(s));

        if (as_gemm) out = conv_view;
        auto rs = out.ss.view(root_shape);
        KN_CHECK(rs.has_value(), KN_ERR_INTERNAL, "view of a dense contraction output failed");
        return out.with(*rs);
    }

    // ---------------------------------------------------------------- root-mean-square norm
    // The IR has no RMS norm; decoder graphs compose it as
    //     t = x (f32), or value_cast(x, f32) for f16 storage
    //     y = t / broadcast(sqrt(view(mean(pow(t, 2), last axis)) + eps)) [* broadcast(gain)]   [value_cast(y, f16)]
    // which planned node by node is five steps that move the activations five times.  Matched here from its last node
    // (every node in between hidden and used by this expression only, `t` by the power and the division only) and
    // emitted as ONE RmsNorm step: one read, one write.  The kernel multiplies by 1/sqrt(..) where the graph divides
    // by sqrt(..): a difference of an f32 rounding step.
    std::optional<PlanTensor> try_fused_rmsnorm(int root) {
        auto is_binary = [&](int v, BinaryOp op) { return g_.values[v].op == OpKind::Binary && g_.values[v].binary_op == op; };
        auto is_cast_to = [&](int v, DType to) {
            const ValueInfo& i = g_.values[v];
            return i.op == OpKind::Unary && i.unary_op == UnaryOp::ValueCast && i.dtype == to;
        };
        const ValueInfo& ri = g_.values[root];
        int cur = root;
        DType out_dtype = DType::F32;
        if (is_cast_to(root, DType::F16)) {
            out_dtype = DType::F16;
            cur = ri.inputs[0];
            if (!fusable(cur) || map_[cur]) return std::nullopt;
        }
        if (g_.values[cur].dtype != DType::F32) return std::nullopt;
        // optional gain
        int gain = -1, div = cur;
        if (is_binary(cur, BinaryOp::Mul)) {
            const ValueInfo& mi = g_.values[cur];
            for (int side = 0; side < 2 && gain < 0; side++) {
                const int d = mi.inputs[side], b = mi.inputs[1 - side];
                if (is_binary(d, BinaryOp::Div) && fusable(d) && !map_[d] && g_.values[b].op == OpKind::Broadcast) {
                    div = d;
                    gain = g_.values[b].inputs[0];
                }
            }
            if (gain < 0) return std::nullopt;
        }
        if (!is_binary(div, BinaryOp::Div)) return std::nullopt;
        const ValueInfo& di = g_.values[div];
        const int t = di.inputs[0], br = di.inputs[1];
        if (g_.values[br].op != OpKind::Broadcast || !fusable(br) || map_[br]) return std::nullopt;
        const int sq = g_.values[br].inputs[0];
        const ValueInfo& si = g_.values[sq];
        if (si.op != OpKind::Unary || si.unary_op != UnaryOp::Sqrt || !fusable(sq) || map_[sq]) return std::nullopt;
        const int add = si.inputs[0];
        if (!is_binary(add, BinaryOp::Add) || !fusable(add) || map_[add]) return std::nullopt;
        int view = -1;
        float eps = 0.f;
        for (int side = 0; side < 2 && view < 0; side++) {
            auto c = g_.as_single_const(g_.values[add].inputs[1 - side]);
            if (c && c->dtype == DType::F32 && g_.values[g_.values[add].inputs[side]].op == OpKind::View) {
                view = g_.values[add].inputs[side];
                eps = c->as_f32();
            }
        }
        if (view < 0 || !fusable(view) || map_[view]) return std::nullopt;
        const int red = g_.values[view].inputs[0];
        const ValueInfo& rdi = g_.values[red];
        const int rank = (int)g_.values[t].shape.size();
        if (rdi.op != OpKind::Reduce || rdi.reduce_op != ReduceOp::Mean || rdi.axes.size() != 1 || rdi.axes[0] != rank - 1 || rank < 1 ||
            !fusable(red) || map_[red])
            return std::nullopt;
        const int pw = rdi.inputs[0];
        if (!is_binary(pw, BinaryOp::Pow) || !fusable(pw) || map_[pw] || g_.values[pw].inputs[0] != t) return std::nullopt;
        auto two = g_.as_single_const(g_.values[pw].inputs[1]);
        if (!two || two->dtype != DType::F32 || two->as_f32() != 2.0f) return std::nullopt;
        if (g_.values[t].dtype != DType::F32) return std::nullopt;
        if (shape_of(view) != [&] { auto s = shape_of(t); s.back() = 1; return s; }()) return std::nullopt;
        if (shape_of(root) != shape_of(t)) return std::nullopt;
        // `t` itself is read, unless it is a cast from f16 that only this expression uses: then the f16 value is read
        int source = t;
        if (is_cast_to(t, DType::F32) && g_.values[g_.values[t].inputs[0]].dtype == DType::F16 && g_.is_hidden_with_uses(t, 2) && !map_[t])
            source = g_.values[t].inputs[0];
        if (gain >= 0) {
            // one f32 value per position of the last axis, the same for every row
            const std::vector<int64_t> gs = shape_of(gain);
            bool per_column = g_.values[gain].dtype == DType::F32 && gs.size() == shape_of(t).size() && gs.back() == shape_of(t).back();
            for (size_t d = 0; per_column && d + 1 < gs.size(); d++) per_column = gs[d] == 1;
            if (!per_column) return std::nullopt;
        }
        const std::vector<int64_t> sh = shape_of(t);
        const int64_t len = sh.back();
        int64_t rows = 1;
        for (size_t d = 0; d + 1 < sh.size(); d++) rows *= sh[d];
        if (len % 8 != 0 || len > 16384 || rows > 0x7FFFFFFFll) return std::nullopt;

        // from here on steps are emitted: nothing may fail any more
        PlanTensor in = source == t ? visit(t) : visit(source);
        const int64_t in_align = in.dtype == DType::F16 ? 8 : 4;
        auto flat = in.ss.view({rows, len});
        if (!flat || flat->strides[1] != 1 || (rows > 1 && flat->strides[0] % in_align != 0) || in.offset % in_align != 0) {
            in = ensure_simple_copy(in, source);
            flat = in.ss.view({rows, len});
            KN_CHECK(flat.has_value(), KN_ERR_INTERNAL, "view of a dense tensor failed");
        }
        std::optional<PlanTensor> g_t;
        int64_t gain_stride = 0;
        if (gain >= 0) {
            PlanTensor gt = visit(gain);
            gain_stride = gt.ss.strides.back();
            g_t = gt;
        }
        PlanTensor out = alloc_shared(sh, out_dtype, root);
        Step s;
        s.kind = StepKind::RmsNorm;
        s.value = root;
        s.operands = {in, out};
        s.writes = {0, 1};
        if (g_t) {
            s.operands.push_back(*g_t);
            s.writes.push_back(0);
        }
        s.rms.rows = rows;
        s.rms.len = len;
        s.rms.in_row_stride = rows > 1 ? flat->strides[0] : len;
        s.rms.out_row_stride = len;
        s.rms.gain_stride = gain_stride;
        s.rms.eps = eps;
        s.rms.in_half = in.dtype == DType::F16 ? 1 : 0;
        s.rms.out_half = out_dtype == DType::F16 ? 1 : 0;
        s.desc = "rmsnorm rows=" + std::to_string(rows) + " len=" + std::to_string(len) + (g_t ? " *gain" : "") + " " +
                 dtype_name(in.dtype) + "->" + dtype_name(out_dtype);
        if (out.ss.size() != 0) push_step(std::move(s));
        return out;
    }
    PlanTensor ensure_simple_copy(const PlanTensor& t, int value) {
        PlanTensor dense = alloc_shared(t.ss.shape, t.dtype, value);
        emit_copy(t, dense, value);
        return dense;
    }

    // ---------------------------------------------------------------- f16 storage (an extension: the reference has no half type)
    // A [b, m, k] and B [b, k, n] of f16, both contiguous along k, every other stride a multiple of 16 bytes (8 elements),
    // and an output the persistent kernel can store through the copy engine (n a multiple of 8, at least 16)
    bool gemm_f16_fits_tensor_core(const PlanTensor& a, const PlanTensor& b) const {
        if (a.ss.rank() != 3 || b.ss.rank() != 3) return false;
        const int64_t batch = a.ss.shape[0], m = a.ss.shape[1], k = a.ss.shape[2], n = b.ss.shape[2];
        auto ok = [](int64_t dim, int64_t stride) { return dim <= 1 || (stride > 0 && stride % 8 == 0); };
        if (batch < 1 || batch > 65535 || m < 64 || n < 16 || n % 8 != 0 || k < 16) return false;
        if (k > 1 && (a.ss.strides[2] != 1 || b.ss.strides[1] != 1)) return false;
        if (!ok(m, a.ss.strides[1]) || !(ok(batch, a.ss.strides[0]) || a.ss.strides[0] == 0)) return false;
        if (!ok(n, b.ss.strides[2]) || !(ok(batch, b.ss.strides[0]) || b.ss.strides[0] == 0)) return false;
        if (a.offset % 8 != 0 || b.offset % 8 != 0) return false;
        if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return false;
        return true;
    }
    // `t` [b, rows, k] as it is when K-contiguous and aligned, else copied into a K-contiguous buffer
    // (`transposed`: t is [b, k, rows], the copy is stored [b, rows, k_pad] and viewed back as [b, k, rows])
    PlanTensor k_major_f16(const PlanTensor& t, bool transposed, int value) {
        const int k_axis = transposed ? 1 : 2, other = transposed ? 2 : 1;
        auto ok = [](int64_t dim, int64_t stride) { return dim <= 1 || (stride > 0 && stride % 8 == 0); };
        if ((t.ss.shape[k_axis] <= 1 || t.ss.strides[k_axis] == 1) && ok(t.ss.shape[other], t.ss.strides[other]) &&
            (ok(t.ss.shape[0], t.ss.strides[0]) || t.ss.strides[0] == 0) && t.offset % 8 == 0)
            return t;
        const int64_t k = t.ss.shape[k_axis], k_pad = (k + 7) / 8 * 8;
        PlanTensor dense = alloc_shared({t.ss.shape[0], t.ss.shape[other], k_pad}, DType::F16, value);
        PlanTensor dst = transposed ? dense.with(dense.ss.permute({0, 2, 1})).slice(1, 0, k, 1) : dense.slice(2, 0, k, 1);
        emit_copy(t, dst, value);
        return dst;
    }

    // MatMul on f16 values: f16 operands, f32 accumulation, the result rounded to f16 once.  No epilogue fusion (the
    // graphs that use f16 have bias-free projections).  Tensor cores (kind::f16) when the persistent kernel takes the
    // shape, else the SIMT kernel with conversion on load.
    PlanTensor visit_matmul_f16(int v) {
        const ValueInfo& info = g_.values[v];
        PlanTensor x = visit(info.inputs[0]);
        PlanTensor w = visit(info.inputs[1]);
        KN_CHECK(x.dtype == DType::F16 && w.dtype == DType::F16, KN_ERR_UNSUPPORTED, "f16 matmul needs f16 operands");
        KN_CHECK(x.ss.rank() == 3 && w.ss.rank() == 3, KN_ERR_SHAPE, "matmul operands must have rank 3");
        std::vector<int64_t> native = shape_of(v);
        bool tensor_core = false;
        if (opts_.math_mode == KN_MATH_TF32) {
            if (!gemm_f16_fits_tensor_core(x, w) && gemm_worth_a_copy(x, w)) {
                PlanTensor x2 = k_major_f16(x, false, info.inputs[0]), w2 = k_major_f16(w, true, info.inputs[1]);
                if (gemm_f16_fits_tensor_core(x2, w2)) {
                    x = x2;
                    w = w2;
                }
            }
            tensor_core = gemm_f16_fits_tensor_core(x, w);
        }
        PlanTensor out = alloc_shared(native, DType::F16, v);
        Step s;
        s.value = v;
        s.kind = StepKind::Gemm;
        s.tensor_core = tensor_core;
        s.operands = {x, w, out};
        s.writes = {0, 0, 1};
        GemmParams& p = s.gemm;
        p.half = 1;
        p.batch = x.ss.shape[0];
        p.m = x.ss.shape[1];
        p.k = x.ss.shape[2];
        p.n = w.ss.shape[2];
        KN_CHECK(w.ss.shape[0] == p.batch && w.ss.shape[1] == p.k, KN_ERR_SHAPE, "matmul operand shapes differ");
        for (int i = 0; i < 3; i++) {
            p.sa[i] = x.ss.strides[i];
            p.sb[i] = w.ss.strides[i];
            p.sc[i] = out.ss.strides[i];
        }
        p.act = 0;
        p.splits = 1;
        if (tensor_core) {
            // few output tiles under a long K: slices of K on separate CTAs, f32 partial sums in a scratch buffer
            const int64_t n_blocks = (p.n + 255) / 256;
            const int64_t bn = std::min<int64_t>(((p.n + n_blocks - 1) / n_blocks + 31) / 32 * 32, 256);
            const int64_t tiles = ((p.m + 127) / 128) * ((p.n + bn - 1) / bn) * p.batch;
            const int64_t k_blocks = (p.k + 63) / 64;
            if (tiles < 74 && k_blocks >= 16 && p.n % 4 == 0) {
                int64_t splits = std::min<int64_t>(std::min<int64_t>(k_blocks / 4, (148 + tiles - 1) / tiles), 32);
                if (splits > 1) {
                    const int64_t per = (k_blocks + splits - 1) / splits;
                    splits = (k_blocks + per - 1) / per;
                    p.splits = (int32_t)splits;
                    PlanTensor scratch = alloc_shared({p.batch, splits, p.m, p.n}, DType::F32, v);
                    s.operands.push_back(scratch);
                    s.writes.push_back(1);
                    s.launches = 2;
                }
            }
        }
        s.flops = 2.0 * (double)p.batch * (double)p.m * (double)p.n * (double)p.k;
        s.desc = "matmul b=" + std::to_string(p.batch) + " m=" + std::to_string(p.m) + " n=" + std::to_string(p.n) + " k=" +
                 std::to_string(p.k) + " +0 f16" + (p.splits > 1 ? " splitk=" + std::to_string(p.splits) : "");
        if (out.ss.size() != 0) push_step(std::move(s));
        return out;
    }

    // ---------------------------------------------------------------- tensor-core eligibility
    static bool tma_stride_ok(int64_t dim, int64_t stride) { return dim <= 1 || (stride > 0 && stride % 4 == 0); }

    // A [b, m, k] and B [b, k, n] both contiguous along k, every other stride a multiple of 16 bytes
    bool gemm_fits_tensor_core(const PlanTensor& a, const PlanTensor& b) const {
        if (a.ss.rank() != 3 || b.ss.rank() != 3) return false;
        const int64_t batch = a.ss.shape[0], m = a.ss.shape[1], k = a.ss.shape[2], n = b.ss.shape[2];
        if (batch < 1 || batch > 65535 || m < 64 || n < 8 || k < 8) return false;
        if (k > 1 && (a.ss.strides[2] != 1 || b.ss.strides[1] != 1)) return false;
        if (!tma_stride_ok(m, a.ss.strides[1]) || !(tma_stride_ok(batch, a.ss.strides[0]) || a.ss.strides[0] == 0)) return false;
        // (a B shared by every batch entry, batch stride 0, is loaded with batch coordinate 0)
        if (!tma_stride_ok(n, b.ss.strides[2]) || !(tma_stride_ok(batch, b.ss.strides[0]) || b.ss.strides[0] == 0)) return false;
        if (a.offset % 4 != 0 || b.offset % 4 != 0) return false;
        if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return false;
        return true;
    }

    // shapes the tensor-core kernels take, large enough that an extra pass over an operand pays off
    bool gemm_worth_a_copy(const PlanTensor& a, const PlanTensor& b) const {
        if (a.ss.rank() != 3 || b.ss.rank() != 3) return false;
        const int64_t batch = a.ss.shape[0], m = a.ss.shape[1], k = a.ss.shape[2], n = b.ss.shape[2];
        if (batch < 1 || batch > 65535 || m < 64 || n < 32 || k < 32) return false;
        return 2.0 * (double)batch * (double)m * (double)n * (double)k >= 2e8;
    }
    bool k_major_ok(const PlanTensor& t, int k_axis, int other_axis) const {
        const auto& sh = t.ss.shape;
        const auto& st = t.ss.strides;
        return (sh[k_axis] <= 1 || st[k_axis] == 1) && tma_stride_ok(sh[other_axis], st[other_axis]) && tma_stride_ok(sh[0], st[0]) &&
               t.offset % 4 == 0;
    }
    // A [b, m, k] with k contiguous: `a` itself, or a copy of it
    PlanTensor k_major_a(const PlanTensor& a, int value) {
        if (k_major_ok(a, 2, 1)) return a;
        const int64_t k_pad = (a.ss.shape[2] + 3) / 4 * 4;
        PlanTensor dense = alloc_shared({a.ss.shape[0], a.ss.shape[1], k_pad}, DType::F32, value);
        PlanTensor dst = dense.slice(2, 0, a.ss.shape[2], 1);
        emit_copy(a, dst, value);
        return dst;
    }
    // B [b, k, n] with k contiguous (stored as [b, n, k_pad]): `b` itself, or a transposed copy of it
    PlanTensor k_major_b(const PlanTensor& b, int value) {
        if (k_major_ok(b, 1, 2)) return b;
        const int64_t k_pad = (b.ss.shape[1] + 3) / 4 * 4;
        PlanTensor dense = alloc_shared({b.ss.shape[0], b.ss.shape[2], k_pad}, DType::F32, value);
        PlanTensor dst = dense.with(dense.ss.permute({0, 2, 1})).slice(1, 0, b.ss.shape[1], 1);
        // `b` itself is often the product of a copy (the head split [B, s, h, d] -> [B*h, s, d] cannot be a view)
        // that nothing else reads: copy from that copy's source straight into the K-contiguous buffer
        if (!plan_.steps.empty() && g_.is_hidden_with_uses(value, 1)) {
            const Step& last = plan_.steps.back();
            if (last.kind == StepKind::Scalar && last.desc.rfind("copy", 0) == 0 && last.value == value && last.operands.size() == 2 &&
                last.writes[1] && !last.writes[0] && last.operands[1].buf == b.buf && last.operands[1].offset == 0 && b.offset == 0 &&
                last.operands[1].ss.has_simple_strides() && b.ss.has_simple_strides() && last.operands[1].ss.size() == b.ss.size() &&
                last.operands[0].dtype == DType::F32) {
                if (auto v = dst.ss.view(last.operands[1].ss.shape)) {
                    const PlanTensor src = last.operands[0];
                    plan_.steps.pop_back();
                    emit_copy(src, dst.with(*v), value);
                    return dst;
                }
            }
        }
        emit_copy(b, dst, value);
        return dst;
    }

    // A convolution the tensor-core convolution kernels do not take (stride > 1) or take badly (a handful
    // of output positions under a long reduction: one M tile, so a handful of CTAs walk K = C*R*S serially)
    // as im2col + batched matmul: the input is gathered into [N, OH*OW, R*S*C_pad] by one Im2col step (zeros
    // for taps outside the image and for padding channels), the constant filter is laid out as
    // [K, R*S*C_pad] on the host, and the matmul (persistent kernel, split-K when there are few tiles)
    // writes [N, OH*OW, K], which the rest of the plan sees as a channels-last [N, K, OH, OW] tensor.
    struct ConvGemm {
        PlanTensor a, b, c, result;
        std::vector<PlanTensor> addends;
        // implicit route: operand `implicit` (1 = a, 2 = b) is the channels-last image tensor itself, the matmul reads
        // the windows straight from it (GemmParams::conv_operand); dims of the matmul it stands for
        int implicit = 0;
        int64_t batch = 0, m = 0, n = 0, k = 0;
    };
    std::optional<ConvGemm> conv_as_gemm(const ValueInfo& ci, const PlanTensor& x, const PlanTensor& w, const std::vector<int64_t>& native,
                                         const std::vector<PlanTensor>& addends, int root) {
        if (x.ss.rank() != 4 || w.ss.rank() != 4 || native.size() != 4) return std::nullopt;
        const int64_t N = x.ss.shape[0], C = x.ss.shape[1], H = x.ss.shape[2], W = x.ss.shape[3];
        const int64_t K = w.ss.shape[0], R = w.ss.shape[2], S = w.ss.shape[3], OH = native[2], OW = native[3];
        const int64_t sy = ci.stride_y, sx = ci.stride_x, py = ci.pad_y, px = ci.pad_x;
        const bool strided = sy != 1 || sx != 1;
        const bool few_positions = N * OH * OW <= 512 && C * R * S >= 1024;
        // a 1x1 convolution IS a matmul over the channels; the generic convolution kernel stores its result
        // one row per thread, which the matmul kernels' staged epilogues do not
        const bool pointwise = R == 1 && S == 1;
        // a long reduction over many channels: the convolution kernels' 128-channel tiles and row-per-thread
        // epilogue reach about 0.2 of the tensor peak there, im2col + the persistent matmul about 0.5, which
        // pays for writing the R*S times larger matrix as long as that stays a few hundred MB
        // (the limit is on the materialised matrix; the implicit route below has none, its operand tile rows being whole
        // output rows is checked there)
        const bool may_be_implicit = !strided && C % 32 == 0 && OW <= 256 && 128 % OW == 0 && OH * OW >= 64 &&
                                     !(opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM);
        const bool long_k = C * R * S >= 2048 && (may_be_implicit || N * OH * OW * R * S * C * 4 <= (256ll << 20));
        if (!strided && !few_positions && !pointwise && !long_k) return std::nullopt;
        if (N < 1 || N > 65535 || OH * OW < 64 || K < 16 || K % 4 != 0 || C < 1 || R * S > 64) return std::nullopt;
        if (2.0 * (double)N * OH * OW * K * C * R * S < 2e8) return std::nullopt;
        const ValueInfo& wi = g_.values[ci.inputs[1]];
        if (wi.op != OpKind::Constant || !w.ss.has_simple_strides() || w.offset != 0) return std::nullopt;
        // Two orientations.  positions x channels: the result is channels-last in memory, which the next
        // tensor-core convolution wants.  If the value the graph asks for (a view of the result, say the
        // [N, groups, ...] view a group norm takes) cannot be expressed on that layout, channels x positions:
        // the filter is the A operand (shared by the batch), the result is plain NCHW.
        const bool nchw = !StridedShape({N, K, OH, OW}, {OH * OW * K, 1, OW * K, K}).view(shape_of(root)).has_value();
        if (nchw && (K < 64 || OH * OW < 16 || (OH * OW) % 4 != 0)) return std::nullopt;
        // addends as [N, OH*OW, K] or [N, K, OH*OW]
        ConvGemm g;
        for (const PlanTensor& t : addends) {
            const auto& st = t.ss.strides;
            int64_t row;
            if (OH * OW == 1 || (st[2] == 0 && st[3] == 0)) row = 0;
            else if (OH == 1) row = st[3];
            else if (OW == 1) row = st[2];
            else if (st[2] == OW * st[3]) row = st[3];
            else return std::nullopt;
            if (nchw) g.addends.push_back(t.with(StridedShape({N, K, OH * OW}, {st[0], st[1], row})));
            else g.addends.push_back(t.with(StridedShape({N, OH * OW, K}, {st[0], row, st[1]})));
        }
        const int64_t taps = R * S, c_pad = (C + 3) / 4 * 4, kk = taps * c_pad;
        // the filter as [K, taps * c_pad], rounded to TF32 like the other tensor-core filters
        auto data = std::make_shared<std::vector<uint8_t>>((size_t)(K * kk) * 4, 0);
        {
            const uint8_t* src = wi.const_data;
            uint32_t* dst = (uint32_t*)data->data();
            for (int64_t k = 0; k < K; k++)
                for (int64_t c = 0; c < C; c++)
                    for (int64_t t = 0; t < taps; t++) {
                        uint32_t bits;
                        memcpy(&bits, src + 4 * ((k * C + c) * taps + t), 4);
                        if ((bits & 0x7F800000u) != 0x7F800000u) bits = (bits + 0x1000u) & 0xFFFFE000u;
                        dst[k * kk + t * c_pad + c] = bits;
                    }
        }
        PlanTensor wmat = alloc_const({K, kk}, DType::F32, ci.inputs[1], nullptr, data);
        if (nchw) g.a = wmat.with(StridedShape({N, K, kk}, {0, kk, 1}));
        else g.b = wmat.with(StridedShape({N, kk, K}, {0, 1, kk}));
        // Implicit route: a stride-1 convolution over whole 32-channel blocks whose output rows tile the matmul
        // kernel's operand tiles reads its windows straight from the channels-last image (one pass over the input to
        // make it channels-last, if it is not) instead of from a materialised [positions, R*S*C] matrix, which is
        // R*S times the input, written once and read once.
        {
            const int64_t rows = nchw ? gemm_persistent_bn(OH * OW) : 128;
            // (positions x channels with fewer than 128 positions per image: half of every 128-row tile is empty either
            // way, the matrix is small, and the materialised route measured slightly faster: 29 against 32 us for
            // 2 x 8x8 positions, 1280 channels)
            const bool fits = !strided && !pointwise && c_pad == C && C % 32 == 0 && OW <= 256 && rows % OW == 0 && OH * OW >= (nchw ? 64 : 128) &&
                              !(opts_.flags & KN_FLAG_NO_PERSISTENT_GEMM) && H <= 32768 && W <= 32768;
            if (fits) {
                PlanTensor xcl = channels_last(x, ci.inputs[0]);
                const auto& cs = xcl.ss.strides;
                if ((C <= 1 || cs[1] == 1) && cs[3] % 4 == 0 && cs[2] % 4 == 0 && (N <= 1 || cs[0] % 4 == 0) && cs[3] > 0 && cs[2] > 0) {
                    g.implicit = nchw ? 2 : 1;
                    g.batch = N;
                    g.k = kk;
                    // The persistent kernel is the only one that reads an implicit operand, and its epilogue takes an
                    // addend per row, per column, or per element with contiguous rows.  Anything else (a skip
                    // tensor that is channels-last where the result is not, or the other way round) is copied
                    // into the result's layout first: one pass over a tensor the size of the result.
                    for (PlanTensor& t : g.addends) {
                        const auto& st = t.ss.strides;
                        if (st[1] == 0 || st[2] == 1 || st[2] == 0) continue;
                        PlanTensor dense = alloc_shared(t.ss.shape, DType::F32, root);
                        emit_copy(t, dense, root);
                        t = dense;
                    }
                    if (nchw) {
                        g.b = xcl;
                        g.m = K;
                        g.n = OH * OW;
                        g.c = alloc_shared({N, K, OH * OW}, DType::F32, root);
                        g.result = g.c.with(StridedShape({N, K, OH, OW}, {K * OH * OW, OH * OW, OW, 1}));
                    } else {
                        g.a = xcl;
                        g.m = OH * OW;
                        g.n = K;
                        g.c = alloc_shared({N, OH * OW, K}, DType::F32, root);
                        g.result = g.c.with(StridedShape({N, K, OH, OW}, {OH * OW * K, 1, OW * K, K}));
                    }
                    return g;
                }
            }
        }
        // (a long-reduction convolution that did not take the implicit route after all: the size limit applies)
        if (!strided && !few_positions && !pointwise && N * OH * OW * R * S * C * 4 > (256ll << 20)) return std::nullopt;
        // im2col (not needed for a 1x1 stride-1 convolution of a channels-last tensor: that is the matrix already)
        PlanTensor col;
        const auto& xs = x.ss.strides;
        if (pointwise && !strided && py == 0 && px == 0 && c_pad == C && (C <= 1 || xs[1] == 1) && xs[2] == W * xs[3] && xs[3] % 4 == 0 &&
            xs[3] >= C && (N <= 1 || xs[0] % 4 == 0) && x.offset % 4 == 0) {
            col = x.with(StridedShape({N, OH * OW, kk}, {xs[0], xs[3], 1}));
        } else {
            col = alloc_shared({N, OH * OW, kk}, DType::F32, root);
        }
        if (col.buf != x.buf || col.offset != x.offset) {
            Step st;
            st.kind = StepKind::Im2col;
            st.value = root;
            st.operands = {x, col};
            st.writes = {0, 1};
            Im2colParams& ip = st.im2col;
            ip.n = (int32_t)N; ip.c = (int32_t)C; ip.h = (int32_t)H; ip.w = (int32_t)W;
            ip.r = (int32_t)R; ip.s = (int32_t)S; ip.oh = (int32_t)OH; ip.ow = (int32_t)OW;
            ip.stride_y = (int32_t)sy; ip.stride_x = (int32_t)sx; ip.pad_y = (int32_t)py; ip.pad_x = (int32_t)px;
            ip.c_pad = (int32_t)c_pad;
            for (int d = 0; d < 4; d++) ip.s_in[d] = x.ss.strides[d];
            st.desc = "im2col n=" + std::to_string(N) + " c=" + std::to_string(C) + " hw=" + std::to_string(H) + "x" + std::to_string(W) +
                      " rs=" + std::to_string(R) + "x" + std::to_string(S) + " -> " + std::to_string(OH) + "x" + std::to_string(OW);
            push_step(std::move(st));
        }
        if (nchw) {
            g.b = col.with(StridedShape({N, kk, OH * OW}, {col.ss.strides[0], 1, col.ss.strides[1]}));
            g.c = alloc_shared({N, K, OH * OW}, DType::F32, root);
            g.result = g.c.with(StridedShape({N, K, OH, OW}, {K * OH * OW, OH * OW, OW, 1}));
        } else {
            g.a = col;
            g.c = alloc_shared({N, OH * OW, K}, DType::F32, root);
            g.result = g.c.with(StridedShape({N, K, OH, OW}, {OH * OW * K, 1, OW * K, K}));
        }
        if (!gemm_fits_tensor_core(g.a, g.b)) return std::nullopt;
        return g;
    }

    bool conv_fits_tensor_core(const ValueInfo& ci, const PlanTensor& x, const PlanTensor& w, const std::vector<int64_t>& out) const {
        if (ci.stride_y != 1 || ci.stride_x != 1) return false;
        if (x.ss.rank() != 4 || w.ss.rank() != 4) return false;
        const int64_t positions = out[0] * out[2] * out[3];
        if (positions < 128 || out[1] < 4 || x.ss.shape[1] < 1) return false;
        if (out[2] > 32768 || out[3] > 32768 || out[0] > (1 << 24) || w.ss.shape[2] * w.ss.shape[3] > 1024) return false;
        return true;
    }

    bool value_is_tensor_core_conv_input(int conv, int input) {
        const ValueInfo& ci = g_.values[conv];
        if (ci.op != OpKind::Conv || ci.inputs[0] != input || ci.dtype != DType::F32) return false;
        if (ci.stride_y != 1 || ci.stride_x != 1) return false;
        std::vector<int64_t> o = shape_of(conv);
        return o[0] * o[2] * o[3] >= 128 && o[1] >= 4;
    }
    bool feeds_tensor_core_conv(int v) {
        for (int u : users_[v])
            if (value_is_tensor_core_conv_input(u, v)) return true;
        return false;
    }

    // The convolution kernel reads its input as (C, W, H, N) with channels contiguous.  A tensor that
    // already is channels-last (the output of a previous tensor-core convolution) is used in place.
    PlanTensor channels_last(const PlanTensor& x, int value) {
        const auto& sh = x.ss.shape;
        const auto& st = x.ss.strides;
        bool ok = (sh[1] <= 1 || st[1] == 1) && tma_stride_ok(sh[3], st[3]) && tma_stride_ok(sh[2], st[2]) &&
                  tma_stride_ok(sh[0], st[0]) && x.offset % 4 == 0;
        if (ok) return x;
        const int64_t c_pad = (sh[1] + 3) / 4 * 4;
        PlanTensor dense = alloc_shared({sh[0], sh[2], sh[3], c_pad}, DType::F32, value);
        PlanTensor nhwc = dense.with(dense.ss.permute({0, 3, 1, 2}));   // logical [N, C_pad, H, W]
        PlanTensor dst = nhwc.slice(1, 0, sh[1], 1);                    // the real channels; pad lanes are never read
        emit_copy(x, dst, value);
        return dst;
    }

    // Filter [K, C, R, S] -> [R*S][K][C_pad] rounded to TF32 (round to nearest, ties away).  Constant
    // filters are rearranged here on the host, once; computed filters get a strided copy step.
    PlanTensor tap_major_filter(const PlanTensor& w, int value) {
        const int64_t K = w.ss.shape[0], C = w.ss.shape[1], R = w.ss.shape[2], S = w.ss.shape[3];
        const int64_t c_pad = (C + 3) / 4 * 4;
        const ValueInfo& wi = g_.values[value];
        if (wi.op == OpKind::Constant && w.ss.has_simple_strides() && w.offset == 0) {
            auto data = std::make_shared<std::vector<uint8_t>>((size_t)(R * S * K * c_pad) * 4, 0);
            const uint32_t* src = (const uint32_t*)wi.const_data;
            uint32_t* dst = (uint32_t*)data->data();
            for (int64_t k = 0; k < K; k++)
                for (int64_t c = 0; c < C; c++)
                    for (int64_t r = 0; r < R; r++)
                        for (int64_t s2 = 0; s2 < S; s2++) {
                            uint32_t bits;
                            memcpy(&bits, (const uint8_t*)src + 4 * (((k * C + c) * R + r) * S + s2), 4);
                            if ((bits & 0x7F800000u) != 0x7F800000u) bits = (bits + 0x1000u) & 0xFFFFE000u;
                            dst[((r * S + s2) * K + k) * c_pad + c] = bits;
                        }
            PlanTensor t = alloc_const({R, S, K, c_pad}, DType::F32, value, nullptr, data);
            return t.with(t.ss.permute({2, 3, 0, 1})).slice(1, 0, C, 1);   // logical [K, C, R, S]
        }
        PlanTensor dense = alloc_shared({R, S, K, c_pad}, DType::F32, value);
        PlanTensor dst = dense.with(dense.ss.permute({2, 3, 0, 1})).slice(1, 0, C, 1);
        emit_copy(w, dst, value);
        return dst;
    }

    // ---------------------------------------------------------------- gather
    PlanTensor visit_gather(int v) {
        const ValueInfo& info = g_.values[v];
        PlanTensor in = visit(info.inputs[0]);
        PlanTensor idx = visit(info.inputs[1]);
        KN_CHECK(idx.ss.rank() == 1 && dtype_is_int(idx.dtype), KN_ERR_BAD_GRAPH, "gather indices must be a rank-1 integer tensor");
        PlanTensor out = alloc_shared(shape_of(v), info.dtype, v);
        KN_CHECK(out.ss.rank() <= DEV_MAX_RANK, KN_ERR_UNSUPPORTED, "gather rank above 8");
        Step s;
        s.kind = StepKind::Gather;
        s.value = v;
        s.operands = {in, idx, out};
        s.writes = {0, 0, 1};
        GatherParams& p = s.gather;
        p.rank = out.ss.rank();
        p.axis = info.axis;
        p.elem_size = dtype_size(info.dtype);
        p.idx_dtype = (uint8_t)idx.dtype;
        p.total = out.ss.size();
        p.axis_in_size = in.ss.shape[info.axis];
        p.idx_stride = idx.ss.strides[0];
        for (int d = 0; d < p.rank; d++) {
            p.out_dims[d] = out.ss.shape[d];
            p.in_strides[d] = in.ss.strides[d];
            p.out_strides[d] = out.ss.strides[d];
        }
        s.desc = "gather axis=" + std::to_string(info.axis);
        if (p.total != 0) push_step(std::move(s));
        return out;
    }

    // ---------------------------------------------------------------- scale / sum peeling
    // `const * x` -> (const, x)   (kn-cuda-eval/src/planner.rs:584-604)
    std::pair<float, PlanTensor> visit_scalable(int v) {
        const ValueInfo& info = g_.values[v];
        if (info.op == OpKind::Binary && info.binary_op == BinaryOp::Mul && (info.dtype == DType::F32 || info.dtype == DType::F16) &&
            !map_[v]) {
            if (auto c = g_.as_single_const(info.inputs[0])) return {(float)c->as_f64_value(), visit(info.inputs[1])};
            if (auto c = g_.as_single_const(info.inputs[1])) return {(float)c->as_f64_value(), visit(info.inputs[0])};
        }
        return {1.0f, visit(v)};
    }

    void fill_rows(RowParams& p, const PlanTensor& in, const PlanTensor& out, int axis) {
        KN_CHECK(in.ss.rank() - 1 <= DEV_MAX_RANK, KN_ERR_UNSUPPORTED, "row kernel rank above 9");
        p.outer_rank = 0;
        p.rows = 1;
        for (int d = 0; d < in.ss.rank(); d++) {
            if (d == axis) continue;
            if (in.ss.shape[d] == 1) continue;
            p.outer_dims[p.outer_rank] = in.ss.shape[d];
            p.in_strides[p.outer_rank] = in.ss.strides[d];
            p.out_strides[p.outer_rank] = out.ss.strides[d];
            p.outer_rank++;
            p.rows *= in.ss.shape[d];
        }
        p.len = in.ss.shape[axis];
        p.in_axis_stride = in.ss.strides[axis];
        p.out_axis_stride = out.ss.strides[axis];
    }

    PlanTensor visit_softmax(int v) {
        const ValueInfo& info = g_.values[v];
        KN_CHECK(info.dtype == DType::F32 || info.dtype == DType::F16, KN_ERR_UNSUPPORTED, "softmax needs f32 or f16");
        // softmax(c * x + mask): the scale and the additive term (an attention mask, usually a broadcast view)
        // are applied as the row is loaded instead of by an elementwise step of their own
        float scale = 1.f;
        PlanTensor in;
        std::optional<PlanTensor> term;
        const int input = info.inputs[0];
        const ValueInfo& ii = g_.values[input];
        if (ii.op == OpKind::Binary && ii.binary_op == BinaryOp::Add && ii.dtype == info.dtype && fusable(input) && !map_[input] &&
            !match_epilogue(input)) {
            auto [s0, t0] = visit_scalable(ii.inputs[0]);
            auto [s1, t1] = visit_scalable(ii.inputs[1]);
            if (s1 == 1.f && t0.ss.shape == t1.ss.shape) { scale = s0; in = t0; term = t1; }
            else if (s0 == 1.f && t0.ss.shape == t1.ss.shape) { scale = s1; in = t1; term = t0; }
        }
        if (!term) std::tie(scale, in) = visit_scalable(input);
        PlanTensor out = alloc_shared(shape_of(v), info.dtype, v);
        Step s;
        s.kind = StepKind::Softmax;
        s.value = v;
        s.operands = {in, out};
        s.writes = {0, 1};
        fill_rows(s.row, in, out, info.axis);
        if (term) {
            s.operands.push_back(*term);
            s.writes.push_back(0);
            int r = 0;
            for (int d = 0; d < in.ss.rank(); d++) {
                if (d == info.axis || in.ss.shape[d] == 1) continue;
                s.row.in1_strides[r++] = term->ss.strides[d];
            }
            s.row.in1_axis_stride = term->ss.strides[info.axis];
        }
        s.row.scale = scale;
        s.row.half = info.dtype == DType::F16 ? 1 : 0;
        s.desc = "softmax rows=" + std::to_string(s.row.rows) + " len=" + std::to_string(s.row.len) + (term ? " +term" : "");
        if (out.ss.size() != 0) push_step(std::move(s));
        return out;
    }

    // `a*x + b*y` -> the layernorm kernel's two inputs (kn-cuda-eval/src/planner.rs:522-552)
    PlanTensor visit_layernorm(int v) {
        const ValueInfo& info = g_.values[v];
        KN_CHECK(info.dtype == DType::F32 || info.dtype == DType::F16, KN_ERR_UNSUPPORTED, "layernorm needs f32 or f16");
        int input = info.inputs[0];
        const ValueInfo& ii = g_.values[input];
        float a0 = 1.f, a1 = 0.f;
        PlanTensor x0;
        std::optional<PlanTensor> x1;
        if (ii.op == OpKind::Binary && ii.binary_op == BinaryOp::Add && !map_[input]) {
            auto [s0, t0] = visit_scalable(ii.inputs[0]);
            auto [s1, t1] = visit_scalable(ii.inputs[1]);
            if (t0.ss == t1.ss) {
                a0 = s0; a1 = s1; x0 = t0; x1 = t1;
            } else {
                x0 = visit(input);
            }
        } else {
            auto [s0, t0] = visit_scalable(input);
            a0 = s0;
            x0 = t0;
        }
        PlanTensor out = alloc_shared(shape_of(v), info.dtype, v);
        Step s;
        s.kind = StepKind::Layernorm;
        s.value = v;
        s.operands = {x0, out};
        s.writes = {0, 1};
        if (x1) {
            s.operands.push_back(*x1);
            s.writes.push_back(0);
        }
        fill_rows(s.row, x0, out, info.axis);
        s.row.alpha0 = a0;
        s.row.alpha1 = a1;
        s.row.eps = info.eps;
        s.row.half = info.dtype == DType::F16 ? 1 : 0;
        s.desc = "layernorm rows=" + std::to_string(s.row.rows) + " len=" + std::to_string(s.row.len) + (x1 ? " +res" : "");
        if (out.ss.size() != 0) push_step(std::move(s));
        return out;
    }

    PlanTensor visit_reduce(int v) {
        const ValueInfo& info = g_.values[v];
        PlanTensor in = visit(info.inputs[0]);
        PlanTensor out = alloc_shared(shape_of(v), info.dtype, v);
        Step s;
        s.kind = StepKind::Reduce;
        s.value = v;
        s.operands = {in, out};
        s.writes = {0, 1};
        ReduceParams& p = s.reduce;
        p.dtype = (uint8_t)info.dtype;
        p.op = (uint8_t)info.reduce_op;
        if (info.reduce_op == ReduceOp::Mean) KN_CHECK(info.dtype == DType::F32, KN_ERR_UNSUPPORTED, "mean needs f32");
        std::vector<int64_t> kd, ki, ko, rd, rs;
        int out_axis = 0;
        for (int d = 0; d < in.ss.rank(); d++) {
            bool reduced = std::find(info.axes.begin(), info.axes.end(), d) != info.axes.end();
            if (reduced) {
                rd.push_back(in.ss.shape[d]);
                rs.push_back(in.ss.strides[d]);
            } else {
                kd.push_back(in.ss.shape[d]);
                ki.push_back(in.ss.strides[d]);
                ko.push_back(out.ss.strides[out_axis++]);
            }
        }
        {
            std::vector<std::vector<int64_t>> st{ki, ko};
            coalesce_axes(kd, st);
            ki = st[0];
            ko = st[1];
            std::vector<std::vector<int64_t>> rt{rs};
            coalesce_axes(rd, rt);
            rs = rt[0];
        }
        KN_CHECK((int)kd.size() <= DEV_MAX_RANK && (int)rd.size() <= DEV_MAX_RANK, KN_ERR_UNSUPPORTED, "reduce rank above 8");
        p.kept_rank = (int)kd.size();
        p.red_rank = (int)rd.size();
        p.n_out = 1;
        p.n_red = 1;
        for (int d = 0; d < p.kept_rank; d++) {
            p.kept_dims[d] = kd[d];
            p.kept_in_strides[d] = ki[d];
            p.kept_out_strides[d] = ko[d];
            p.n_out *= kd[d];
        }
        for (int d = 0; d < p.red_rank; d++) {
            p.red_dims[d] = rd[d];
            p.red_strides[d] = rs[d];
            p.n_red *= rd[d];
        }
        p.mean_scale = (float)p.n_red;
        s.desc = "reduce out=" + std::to_string(p.n_out) + " red=" + std::to_string(p.n_red);
        if (out.ss.size() != 0) push_step(std::move(s));
        return out;
    }

    // ---------------------------------------------------------------- convolution chains
    // A run of consecutive tensor-core steps conv3x3(stride 1, same padding) -> [+bias] [+skip] [relu],
    // each reading the previous one's result and none of whose intermediate results is needed
    // elsewhere, becomes ONE ConvChain step: the activations of a group of whole images stay in the
    // shared memory of one SM from the first layer to the last (a 3x3 convolution of an image depends on
    // that image only), so per layer only the filter crosses from L2.  The skip operand of a residual
    // block must be the tensor the kernel currently holds: the chain's input, or the latest result
    // that a later layer of the chain adds.
    struct ChainLayer {
        size_t step;
        int bias_operand = -1, res_operand = -1;
    };
    struct ChainHead {
        size_t step;
        int bias_operand = -1;
    };

    // every operand once; the trunk's result only if the chain stores it
    static void chain_alg_bytes(Step& s) {
        bool stored = false;
        for (int l = 0; l < s.chain.n_layers; l++) stored = stored || (s.chain.flags[l] & kChainFlagStore);
        s.alg_bytes = 0;
        for (size_t o = 0; o < s.operands.size(); o++)
            if (o != 1 || stored) s.alg_bytes += touched_bytes(s.operands[o]);
    }

    bool chain_candidate(const Step& s, ChainLayer& l) const {
        if (s.kind != StepKind::Conv || !s.tensor_core) return false;
        const ConvParams& c = s.conv;
        if (c.r != 3 || c.s != 3 || c.pad_y != 1 || c.pad_x != 1 || c.stride_y != 1 || c.stride_x != 1) return false;
        if (c.k > 128 || c.c > 128 || c.oh != c.h || c.ow != c.w) return false;
        if (c.act != (int32_t)Activation::None && c.act != (int32_t)Activation::Relu) return false;
        if (!tc_chain_geometry(c.h, c.w, c.n, 4, nullptr)) return false;
        // the filter must be a planner-made tap-major constant [3][3][K][C_pad] whose bytes are still on the host
        const PlanTensor& w = s.operands[1];
        const BufferInfo& wb = plan_.buffers[w.buf];
        const int64_t c_pad = (c.c + 3) / 4 * 4;
        if (wb.kind != BufKind::Const || !wb.owned || w.offset != 0) return false;
        if (w.ss.strides[0] != c_pad || (c.c > 1 && w.ss.strides[1] != 1) || w.ss.strides[2] != 3 * c.k * c_pad ||
            w.ss.strides[3] != c.k * c_pad)
            return false;
        for (size_t o = 3; o < s.operands.size(); o++) {
            const PlanTensor& a = s.operands[o];
            const BufferInfo& ab = plan_.buffers[a.buf];
            const auto& st = a.ss.strides;
            if (st[0] == 0 && st[2] == 0 && st[3] == 0 && ab.kind == BufKind::Const && ab.host_data != nullptr && l.bias_operand < 0)
                l.bias_operand = (int)o;
            else if (l.res_operand < 0)
                l.res_operand = (int)o;
            else
                return false;
        }
        return true;
    }

    // A later 1x1 convolution of the chain's last result, with constant filter and bias: it can run as
    // part of the chain's pointwise last layer (ConvChainParams: heads).
    bool head_candidate(const Step& s, const Step& last, int& bias_operand) const {
        if (s.kind != StepKind::Conv || !s.tensor_core || s.operands.size() < 3 || s.operands.size() > 4) return false;
        const ConvParams& c = s.conv;
        if (c.r != 1 || c.s != 1 || c.pad_y != 0 || c.pad_x != 0 || c.stride_y != 1 || c.stride_x != 1) return false;
        if (c.c != last.conv.k || c.n != last.conv.n || c.h != last.conv.h || c.w != last.conv.w || c.k > 128) return false;
        if (!s.operands[0].same_storage(last.operands[2])) return false;
        if (c.act != (int32_t)Activation::None && c.act != (int32_t)Activation::Relu) return false;
        const BufferInfo& wb = plan_.buffers[s.operands[1].buf];
        if (wb.kind != BufKind::Const || wb.host_data == nullptr) return false;
        bias_operand = -1;
        if (s.operands.size() == 4) {
            const PlanTensor& a = s.operands[3];
            const BufferInfo& ab = plan_.buffers[a.buf];
            const auto& st = a.ss.strides;
            if (!(st[0] == 0 && st[2] == 0 && st[3] == 0 && ab.kind == BufKind::Const && ab.host_data != nullptr)) return false;
            bias_operand = 3;
        }
        return true;
    }

    bool buffer_used_outside(int buf, size_t first, size_t last, const std::vector<uint8_t>* skip = nullptr) const {
        if (plan_.buffers[buf].always_live) return true;
        for (size_t i = 0; i < plan_.steps.size(); i++) {
            if (i >= first && i <= last) continue;
            if (skip && (*skip)[i]) continue;
            for (auto& t : plan_.steps[i].operands)
                if (t.buf == buf) return true;
        }
        return false;
    }

    void fuse_conv_chains() {
        if (opts_.math_mode != KN_MATH_TF32 || (opts_.flags & KN_FLAG_NO_CONV_CHAIN)) return;
        std::vector<Step>& steps = plan_.steps;
        std::vector<Step> result;
        std::vector<uint8_t> consumed(steps.size(), 0);   // 1x1 convolutions that became heads of an earlier chain
        size_t i = 0;
        while (i < steps.size()) {
            if (consumed[i]) {
                i++;
                continue;
            }
            // longest run starting at i
            std::vector<ChainLayer> layers;
            for (size_t j = i; j < steps.size() && layers.size() < (size_t)kMaxChainLayers; j++) {
                ChainLayer l;
                l.step = j;
                if (!chain_candidate(steps[j], l)) break;
                if (!layers.empty()) {
                    const Step& prev = steps[j - 1];
                    if (!steps[j].operands[0].same_storage(prev.operands[2])) break;
                    if (steps[j].conv.n != prev.conv.n || steps[j].conv.h != prev.conv.h || steps[j].conv.w != prev.conv.w) break;
                }
                layers.push_back(l);
            }
            // the held tensor: follow the skip connections, cut where one does not match
            size_t len = 0;
            std::vector<uint8_t> hold(layers.size(), 0);
            if (!layers.empty()) {
                PlanTensor held = steps[layers[0].step].operands[0];
                for (size_t a = 0; a < layers.size(); a++) {
                    const Step& s = steps[layers[a].step];
                    if (layers[a].res_operand >= 0 && !s.operands[layers[a].res_operand].same_storage(held)) break;
                    for (size_t b = a + 1; b < layers.size(); b++) {
                        const Step& later = steps[layers[b].step];
                        if (layers[b].res_operand >= 0 && later.operands[layers[b].res_operand].same_storage(s.operands[2])) hold[a] = 1;
                    }
                    if (hold[a]) held = s.operands[2];
                    len = a + 1;
                }
                // an intermediate result that something else reads must reach global memory: end the chain there
                // (a cut moves later layers outside, which may expose earlier results in turn: repeat)
                for (bool changed = true; changed;) {
                    changed = false;
                    for (size_t a = 0; a + 1 < len; a++) {
                        if (buffer_used_outside(steps[layers[a].step].operands[2].buf, layers[0].step, layers[len - 1].step)) {
                            len = a + 1;
                            changed = true;
                            break;
                        }
                    }
                }
                // the tensor held at the end must not be required after a cut (it never is: cuts only shorten)
            }
            if (len < 2) {
                result.push_back(std::move(steps[i]));
                i++;
                continue;
            }
            // 1x1 convolutions of the chain's result anywhere later in the plan become heads of a pointwise
            // last layer (their inputs are the result and constants, so they can run this early)
            std::vector<ChainHead> heads;
            if (len < (size_t)kMaxChainLayers) {
                const Step& last = steps[layers[len - 1].step];
                int channels = 0;
                for (size_t j = layers[len - 1].step + 1; j < steps.size() && heads.size() < (size_t)kMaxChainHeads; j++) {
                    ChainHead h;
                    h.step = j;
                    if (consumed[j] || !head_candidate(steps[j], last, h.bias_operand)) continue;
                    if (channels + steps[j].conv.k > 128) continue;
                    channels += steps[j].conv.k;
                    heads.push_back(h);
                }
            }
            for (auto& h : heads) consumed[h.step] = 1;
            const bool store_trunk = heads.empty() || buffer_used_outside(steps[layers[len - 1].step].operands[2].buf, layers[0].step,
                                                                           layers[len - 1].step, &consumed);
            Step chain = make_chain_step(steps, layers, hold, len, heads, store_trunk);
            // The chain reads its input through element strides, so a copy that only exists to make the
            // input channels-last for the per-layer kernel is skipped: read the copy's source instead.
            if (!result.empty()) {
                const Step& prev = result.back();
                const size_t prev_index = layers[0].step - 1;
                if (prev.kind == StepKind::Scalar && prev.desc == "copy" && prev.operands.size() == 2 && prev.writes[1] &&
                    prev.operands[1].same_storage(chain.operands[0]) && prev.operands[0].dtype == DType::F32 &&
                    prev.operands[0].ss.shape == chain.operands[0].ss.shape &&
                    !buffer_used_outside(prev.operands[1].buf, prev_index, layers[len - 1].step)) {
                    chain.operands[0] = prev.operands[0];
                    for (int d = 0; d < 4; d++) chain.chain.s_in[d] = chain.operands[0].ss.strides[d];
                    chain_alg_bytes(chain);
                    result.pop_back();
                }
            }
            result.push_back(std::move(chain));
            i += len;
        }
        steps = std::move(result);
    }

    Step make_chain_step(const std::vector<Step>& steps, const std::vector<ChainLayer>& layers, const std::vector<uint8_t>& hold,
                         size_t len, const std::vector<ChainHead>& heads, bool store_trunk) {
        const Step& first = steps[layers[0].step];
        const Step& last = steps[layers[len - 1].step];
        Step s;
        s.kind = StepKind::ConvChain;
        s.tensor_core = true;
        s.value = last.value;
        ConvChainParams& p = s.chain;
        p.n = first.conv.n;
        p.c_in = first.conv.c;
        p.k = first.conv.k;
        p.h = first.conv.h;
        p.w = first.conv.w;
        const size_t n_layers = len + (heads.empty() ? 0 : 1);
        p.n_layers = (int32_t)n_layers;
        int64_t n_tiles = 0;
        for (size_t a = 0; a < len; a++) {
            const ConvParams& c = steps[layers[a].step].conv;
            KN_CHECK(c.k == p.k && (a == 0 || c.c == p.k), KN_ERR_INTERNAL, "convolution chain with changing width");
            p.c_blocks[a] = (uint8_t)((c.c + 31) / 32);
            n_tiles += 9 * p.c_blocks[a];
            p.flags[a] = (uint8_t)((c.act == (int32_t)Activation::Relu ? kChainFlagRelu : 0) |
                                   (layers[a].res_operand >= 0 ? kChainFlagAddHeld : 0) | (hold[a] ? kChainFlagHold : 0));
            s.flops += steps[layers[a].step].flops;
        }
        if (store_trunk) p.flags[len - 1] |= kChainFlagStore;
        if (!heads.empty()) {
            p.c_blocks[len] = (uint8_t)((p.k + 31) / 32);
            p.flags[len] = kChainFlagPointwise;
            n_tiles += p.c_blocks[len];
        }
        // filter tiles: [tile][128][32] f32 (already TF32), zero beyond the real channels
        auto tiles = std::make_shared<std::vector<uint8_t>>((size_t)n_tiles * 128 * 32 * 4, 0);
        auto bias = std::make_shared<std::vector<uint8_t>>(n_layers * 128 * 4, 0);
        float* tp = (float*)tiles->data();
        float* bp = (float*)bias->data();
        int64_t tile = 0;
        for (size_t a = 0; a < len; a++) {
            const Step& st = steps[layers[a].step];
            const ConvParams& c = st.conv;
            const int64_t c_pad = (c.c + 3) / 4 * 4;
            const float* src = (const float*)plan_.buffers[st.operands[1].buf].owned->data();   // [tap][K][c_pad]
            for (int tap = 0; tap < 9; tap++)
                for (int cb = 0; cb < p.c_blocks[a]; cb++, tile++)
                    for (int k = 0; k < c.k; k++)
                        for (int ch = cb * 32; ch < std::min<int>(c.c, cb * 32 + 32); ch++)
                        {
                            // stored exactly as the tile sits in shared memory (rows of 128 bytes whose 16-byte
                            // chunks are XOR-swizzled with the row number), so a linear bulk copy delivers it
                            const int col = ch - cb * 32;
                            const int64_t pos = (int64_t)k * 32 + ((((col >> 2) ^ (k & 7)) << 2) | (col & 3));
                            tp[tile * 128 * 32 + pos] = src[((int64_t)tap * c.k + k) * c_pad + ch];
                        }
            if (layers[a].bias_operand >= 0) {
                const PlanTensor& b = st.operands[layers[a].bias_operand];
                const float* bsrc = (const float*)plan_.buffers[b.buf].host_data;
                for (int k = 0; k < c.k; k++) bp[a * 128 + k] = bsrc[b.offset + (int64_t)k * b.ss.strides[1]];
            }
        }
        // the pointwise last layer: the heads' filters below one another (rows = output channels)
        p.n_heads = (int32_t)heads.size();
        std::vector<PlanTensor> head_outputs;
        int row0 = 0;
        for (size_t hi = 0; hi < heads.size(); hi++) {
            const Step& st = steps[heads[hi].step];
            const ConvParams& c = st.conv;
            const PlanTensor& w = st.operands[1];
            const float* src = (const float*)plan_.buffers[w.buf].host_data;
            for (int k = 0; k < c.k; k++)
                for (int ch = 0; ch < c.c; ch++) {
                    float v = src[w.offset + (int64_t)k * w.ss.strides[0] + (int64_t)ch * w.ss.strides[1]];
                    uint32_t bits;
                    memcpy(&bits, &v, 4);
                    if ((bits & 0x7F800000u) != 0x7F800000u) bits = (bits + 0x1000u) & 0xFFFFE000u;
                    memcpy(&v, &bits, 4);
                    const int row = row0 + k, cb = ch / 32, col = ch % 32;
                    const int64_t pos = (int64_t)row * 32 + ((((col >> 2) ^ (row & 7)) << 2) | (col & 3));
                    tp[(tile + cb) * 128 * 32 + pos] = v;
                }
            if (heads[hi].bias_operand >= 0) {
                const PlanTensor& b = st.operands[heads[hi].bias_operand];
                const float* bsrc = (const float*)plan_.buffers[b.buf].host_data;
                for (int k = 0; k < c.k; k++) bp[len * 128 + row0 + k] = bsrc[b.offset + (int64_t)k * b.ss.strides[1]];
            }
            p.head_begin[hi] = row0;
            p.head_relu[hi] = c.act == (int32_t)Activation::Relu;
            for (int d = 0; d < 4; d++) p.head_s_out[hi][d] = st.operands[2].ss.strides[d];
            head_outputs.push_back(st.operands[2]);
            row0 += c.k;
            s.flops += st.flops;
        }
        p.head_begin[heads.size()] = row0;
        PlanTensor t_tiles = alloc_const({n_tiles, 128, 32}, DType::F32, s.value, nullptr, tiles);
        PlanTensor t_bias = alloc_const({(int64_t)n_layers, 128}, DType::F32, s.value, nullptr, bias);
        // operand 1 is the trunk's result; when nothing reads it, it is neither stored nor allocated (the slot
        // then repeats the first head's output)
        s.operands = {first.operands[0], store_trunk ? last.operands[2] : head_outputs[0], t_tiles, t_bias};
        s.writes = {0, 1, 0, 0};
        for (auto& t : head_outputs) {
            s.operands.push_back(t);
            s.writes.push_back(1);
        }
        for (int d = 0; d < 4; d++) {
            p.s_in[d] = first.operands[0].ss.strides[d];
            p.s_out[d] = last.operands[2].ss.strides[d];
        }
        s.desc = "convchain layers=" + std::to_string(len) + " n=" + std::to_string(p.n) + " c=" + std::to_string(p.c_in) + " hw=" +
                 std::to_string(p.h) + "x" + std::to_string(p.w) + " k=" + std::to_string(p.k) + " rs=3x3 tf32";
        if (!heads.empty()) {
            s.desc += " heads=";
            for (size_t hi = 0; hi < heads.size(); hi++) s.desc += (hi ? "+" : "") + std::to_string(p.head_begin[hi + 1] - p.head_begin[hi]);
            if (!store_trunk) s.desc += " (trunk result not stored)";
        }
        chain_alg_bytes(s);
        return s;
    }

    // Constants no step reads any more (a raw filter whose tap-major copy is used instead, filters
    // folded into a chain) are not uploaded.
    void drop_unused_constants() {
        std::vector<uint8_t> used(plan_.buffers.size(), 0);
        for (auto& s : plan_.steps)
            for (auto& t : s.operands) used[t.buf] = 1;
        for (auto& t : plan_.outputs) used[t.buf] = 1;
        for (auto& t : plan_.inputs) used[t.buf] = 1;
        for (size_t b = 0; b < plan_.buffers.size(); b++) {
            BufferInfo& bi = plan_.buffers[b];
            if (bi.kind == BufKind::Const && !used[b]) {
                bi.bytes = 0;
                bi.host_data = nullptr;
                bi.owned.reset();
            }
        }
    }

    // ---------------------------------------------------------------- memory
    // Live ranges over step indices, then offsets inside one arena: buffers are placed largest
    // first at the lowest offset that does not collide with an already placed buffer whose live
    // range overlaps.  (The reference reuses only buffers of identical size and gives each its own
    // cudaMalloc: kn-cuda-eval/src/planner.rs:134-228.)
    void assign_memory() {
        auto& bufs = plan_.buffers;
        for (size_t i = 0; i < plan_.steps.size(); i++) {
            for (auto& t : plan_.steps[i].operands) {
                BufferInfo& b = bufs[t.buf];
                b.first_step = std::min(b.first_step, (int)i);
                b.last_step = std::max(b.last_step, (int)i);
            }
        }
        const int n_steps = (int)plan_.steps.size();
        for (auto& b : bufs) {
            if (b.always_live) {
                b.first_step = -1;
                b.last_step = n_steps;
            }
        }
        auto align = [](size_t x) { return (x + 255) & ~(size_t)255; };

        // constants: packed back to back
        size_t coff = 0;
        for (auto& b : bufs) {
            if (b.kind != BufKind::Const) continue;
            b.arena_offset = (int64_t)coff;
            coff += align(std::max<size_t>(b.bytes, 1));
            plan_.mem.dedicated_bytes += b.bytes;
        }
        plan_.const_bytes = coff;

        std::vector<int> order;
        for (size_t i = 0; i < bufs.size(); i++) {
            BufferInfo& b = bufs[i];
            if (b.kind != BufKind::Shared) continue;
            plan_.mem.hypo_total_bytes += b.bytes;
            if (b.last_step < b.first_step) {   // never touched by a step
                if (!b.always_live) { b.arena_offset = 0; continue; }
            }
            order.push_back((int)i);
        }
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return bufs[a].bytes > bufs[b].bytes; });
        std::vector<int> placed;
        size_t arena = 0;
        for (int bi : order) {
            BufferInfo& b = bufs[bi];
            size_t size = align(std::max<size_t>(b.bytes, 1));
            std::vector<std::pair<size_t, size_t>> busy;
            for (int pj : placed) {
                BufferInfo& o = bufs[pj];
                if (o.last_step < b.first_step || b.last_step < o.first_step) continue;
                busy.push_back({(size_t)o.arena_offset, (size_t)o.arena_offset + align(std::max<size_t>(o.bytes, 1))});
            }
            std::sort(busy.begin(), busy.end());
            size_t off = 0;
            for (auto& iv : busy) {
                if (off + size <= iv.first) break;
                off = std::max(off, iv.second);
            }
            b.arena_offset = (int64_t)off;
            arena = std::max(arena, off + size);
            placed.push_back(bi);
        }
        plan_.arena_bytes = arena;
        plan_.mem.shared_bytes = arena;

        // lower bound on the arena: the largest set of simultaneously live buffers
        std::vector<int64_t> delta(n_steps + 3, 0);
        for (int bi : order) {
            BufferInfo& b = bufs[bi];
            delta[b.first_step + 1] += (int64_t)b.bytes;
            delta[b.last_step + 2] -= (int64_t)b.bytes;
        }
        int64_t live = 0, peak = 0;
        for (int64_t d : delta) {
            live += d;
            peak = std::max(peak, live);
        }
        plan_.mem.hypo_peak_bytes = (uint64_t)peak;
        plan_.mem.zero_bytes = 0;

        // every operand must stay inside its buffer
        for (auto& s : plan_.steps) {
            for (auto& t : s.operands) {
                int64_t lo, hi;
                t.ss.extent(&lo, &hi);
                if (t.ss.size() == 0) continue;
                int64_t es = dtype_size(t.dtype);
                KN_CHECK(t.offset + lo >= 0 && (t.offset + hi + 1) * es <= (int64_t)bufs[t.buf].bytes, KN_ERR_INTERNAL,
                         "operand reaches outside its buffer: " + t.str());
            }
        }
    }
};

struct PlanJob {
    const Graph* g;
    int64_t batch;
    kn_options opts;
    Plan* plan;
    int code = 0;
    std::string msg;
};

void* plan_thread(void* arg) {
    PlanJob* job = (PlanJob*)arg;
    try {
        Planner p(*job->g, job->batch, job->opts, *job->plan);
        p.run();
    } catch (const Error& e) {
        job->code = e.code;
        job->msg = e.what();
    } catch (const std::exception& e) {
        job->code = KN_ERR_INTERNAL;
        job->msg = e.what();
    }
    return nullptr;
}

}  // namespace

std::unique_ptr<Plan> make_plan(const Graph& graph, int64_t batch, const kn_options& opts) {
    KN_CHECK(batch >= 0, KN_ERR_INVALID_ARG, "negative batch size");
    auto plan = std::make_unique<Plan>();
    PlanJob job{&graph, batch, opts, plan.get()};
    // The lowering recurses along operand chains; deep graphs (thousands of values in a chain) need
    // more stack than a caller's thread may have, so it runs on a thread with a large stack.
    pthread_attr_t attr;
    pthread_attr_init(&attr);
    pthread_attr_setstacksize(&attr, (size_t)512 << 20);
    pthread_t th;
    int rc = pthread_create(&th, &attr, plan_thread, &job);
    pthread_attr_destroy(&attr);
    if (rc != 0) {
        plan_thread(&job);
    } else {
        pthread_join(th, nullptr);
    }
    if (job.code != 0) fail(job.code, job.msg);
    return plan;
}

std::string Plan::describe() const {
    std::ostringstream os;
    os << "plan batch=" << batch << " steps=" << steps.size() << " buffers=" << buffers.size() << " arena_bytes=" << arena_bytes
       << " const_bytes=" << const_bytes << " hypo_peak=" << mem.hypo_peak_bytes << " hypo_total=" << mem.hypo_total_bytes << "\n";
    for (size_t i = 0; i < steps.size(); i++) {
        const Step& s = steps[i];
        os << "step " << i << " " << step_kind_name(s.kind) << (s.tensor_core ? "/tc" : "") << " value=" << s.value << " " << s.desc;
        if (s.kind == StepKind::Scalar)
            os << " loads=" << s.scalar.n_loads << " instr=" << s.scalar.n_instr << " rank=" << s.scalar.rank
               << (s.scalar.vec4 >= 3 ? " vec8" : (s.scalar.vec4 ? " vec4" : ""))
               << ((s.scalar.vec4 == 2 || s.scalar.vec4 >= 4) ? " acc" : "") << (s.scalar.vec4 == 5 ? " half2" : "");
        os << " bytes=" << (uint64_t)s.alg_bytes << " flops=" << (uint64_t)s.flops << " [";
        for (size_t o = 0; o < s.operands.size(); o++) os << (o ? " " : "") << (s.writes[o] ? "w:" : "r:") << s.operands[o].str();
        os << "]\n";
    }
    for (size_t i = 0; i < inputs.size(); i++) os << "input " << i << " " << inputs[i].str() << "\n";
    for (size_t i = 0; i < outputs.size(); i++) os << "output " << i << " " << outputs[i].str() << "\n";
    return os.str();
}

}  // namespace kn
