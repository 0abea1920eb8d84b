// The planner: lowers a Graph at a concrete batch size into a list of kernel steps over planned
// buffers.  Pure host code (no CUDA calls), so it can be inspected and tested without a device.
// Counterpart of the reference's `Planner` / `Plan` / `Step` (kn-cuda-eval/src/planner.rs:45-272,
// step.rs:18-402).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "ir.h"
#include "kernels.h"
#include "kn_b200.h"
#include "strided.h"

namespace kn {

enum class BufKind : uint8_t { Const, Shared, Zero };

struct BufferInfo {
    BufKind kind = BufKind::Shared;
    size_t bytes = 0;
    int value = -1;                    // graph value this buffer was created for (debugging)
    const uint8_t* host_data = nullptr;   // Const: bytes to upload (points into the graph blob or `owned`)
    std::shared_ptr<std::vector<uint8_t>> owned;   // Const data produced by the planner itself
    int first_step = 1 << 30, last_step = -1;
    bool always_live = false;          // graph inputs and outputs
    int64_t arena_offset = -1;         // Shared: byte offset inside the arena; Const: inside the constant block
};

// A device tensor: buffer + element offset + dtype + strided shape.  View-like graph operations only
// edit this descriptor (kn-cuda-eval/src/offset_tensor.rs:10-108).
struct PlanTensor {
    int buf = -1;
    int64_t offset = 0;   // in elements
    DType dtype = DType::F32;
    StridedShape ss;

    PlanTensor with(StridedShape s, int64_t extra_offset = 0) const;
    PlanTensor slice(int axis, int64_t start, int64_t end, int64_t step) const;
    PlanTensor flip(int axis) const;
    bool same_storage(const PlanTensor& o) const {
        return buf == o.buf && offset == o.offset && dtype == o.dtype && ss == o.ss;
    }
    std::string str() const;
};

struct TcLaunch;   // tensor maps and launch geometry of a tensor-core step (kernels/contract_tc.cu)

enum class StepKind : uint8_t { Scalar = 0, Reduce, Softmax, Layernorm, Gather, Gemm, Conv, ConvChain, Im2col, AllReduce, RmsNorm, COUNT };
const char* step_kind_name(StepKind k);

struct Step {
    StepKind kind = StepKind::Scalar;
    int value = -1;                     // graph value the step produces
    std::vector<PlanTensor> operands;   // in the order the kernel's pointers are patched
    std::vector<uint8_t> writes;        // per operand: 1 if the step writes it
    bool tensor_core = false;           // Gemm / Conv: tcgen05 kernel instead of the SIMT one
    std::shared_ptr<TcLaunch> tc;       // built by tc_prepare_step once device pointers exist
    int launches = 1;
    double alg_bytes = 0;               // distinct operand bytes touched once (roofline numerator)
    double flops = 0;
    std::string desc;

    ScalarParams scalar{};
    ReduceParams reduce{};
    RowParams row{};
    GatherParams gather{};
    GemmParams gemm{};
    ConvParams conv{};
    ConvChainParams chain{};
    Im2colParams im2col{};
    AllReduceParams all_reduce{};
    RmsNormParams rms{};
};

struct Plan {
    int64_t batch = 0;
    kn_options opts{};
    std::vector<BufferInfo> buffers;
    std::vector<Step> steps;
    std::vector<PlanTensor> inputs;    // dense, one per graph input
    std::vector<PlanTensor> outputs;   // dense, one per graph output
    std::vector<std::vector<int64_t>> input_shapes, output_shapes;
    size_t arena_bytes = 0, const_bytes = 0, zero_bytes = 0;
    int collectives = 0;               // AllReduce steps
    kn_mem_usage mem{};

    std::string describe() const;
};

// Throws kn::Error.  `graph` must outlive the plan (constant payloads are referenced, not copied).
std::unique_ptr<Plan> make_plan(const Graph& graph, int64_t batch, const kn_options& opts);

}  // namespace kn
