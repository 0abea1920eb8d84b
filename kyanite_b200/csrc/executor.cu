// The executor and the C ABI.  Counterpart of `CudaExecutor` (kn-cuda-eval/src/executor.rs:20-325):
// owns the arena, the uploaded constants, pinned staging for inputs and outputs, the stream and the
// captured CUDA graph of the step list.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "comm.h"
#include "ir.h"
#include "kernels.h"
#include "kn_b200.h"
#include "plan.h"
#include "scalar_ops.h"
#include "tc.h"
#include "kernels/tc_ptx.cuh"

namespace kn {

// One thread waits, through the same bounded wait every tensor-core kernel uses, on a barrier that nobody
// arrives on: the wait runs out after `limit_cycles`, raises the status word and the kernel returns.  No tensor
// memory, no copies in flight: nothing is left behind.  (kn_executor_selftest_wait_expiry)
__global__ void wait_expiry_kernel(uint32_t* status, long long limit_cycles, uint32_t code) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abandon;
    if (threadIdx.x == 0) {
        tcp::mbar_init(tcp::smem_u32(&bar), 1);
        abandon = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) tcp::mbar_wait(tcp::smem_u32(&bar), 0, &abandon, status, code, limit_cycles);
}

namespace {

thread_local std::string g_last_error;

#define KN_CUDA(expr)                                                                                   \
    do {                                                                                                \
        cudaError_t err__ = (expr);                                                                     \
        if (err__ != cudaSuccess)                                                                       \
            ::kn::fail(KN_ERR_CUDA, std::string(#expr) + " failed: " + cudaGetErrorString(err__));      \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device) {
        cudaGetDevice(&prev);
        KN_CUDA(cudaSetDevice(device));
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace

void set_last_error(const std::string& message) { g_last_error = message; }

struct Executor {
    int device = 0;
    std::unique_ptr<Plan> plan;
    cudaStream_t stream = nullptr;
    uint8_t* arena = nullptr;
    uint8_t* consts = nullptr;
    uint32_t* status_dev = nullptr;    // raised by a kernel whose bounded wait expired
    uint32_t* status_host = nullptr;   // pinned mirror
    std::vector<void*> pinned_in, pinned_out;
    std::vector<size_t> bytes_in, bytes_out;
    std::vector<DType> dtype_in, dtype_out;
    cudaGraphExec_t graph_exec = nullptr;        // the step list
    cudaGraphExec_t eval_graph_exec = nullptr;   // uploads + step list + downloads (see capture_evaluate)
    cudaStream_t side_stream = nullptr;          // capture-time fork for early output copies
    bool profile = false;
    std::vector<float> step_us;
    int launches = 0;
    Comm* comm = nullptr;              // not owned; AllReduce steps sum over its ranks (null: a world of one)

    ~Executor() {
        // the caller's current device is left as it was (a host may share the thread with other CUDA users)
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (graph_exec) cudaGraphExecDestroy(graph_exec);
        if (eval_graph_exec) cudaGraphExecDestroy(eval_graph_exec);
        if (side_stream) cudaStreamDestroy(side_stream);
        for (void* p : pinned_in) if (p) cudaFreeHost(p);
        for (void* p : pinned_out) if (p) cudaFreeHost(p);
        if (arena) cudaFree(arena);
        if (consts) cudaFree(consts);
        if (status_dev) cudaFree(status_dev);
        if (status_host) cudaFreeHost(status_host);
        if (stream) cudaStreamDestroy(stream);
        if (prev >= 0) cudaSetDevice(prev);
    }

    uint8_t* device_ptr(const PlanTensor& t) const {
        const BufferInfo& b = plan->buffers[t.buf];
        uint8_t* base = b.kind == BufKind::Const ? consts : arena;
        return base + b.arena_offset + t.offset * dtype_size(t.dtype);
    }

    void patch_pointers() {
        launches = 0;
        for (Step& s : plan->steps) {
            std::vector<void*> ptr;
            for (auto& t : s.operands) ptr.push_back(device_ptr(t));
            switch (s.kind) {
                case StepKind::Scalar:
                    for (size_t i = 0; i < ptr.size(); i++) s.scalar.ptr[i] = ptr[i];
                    break;
                case StepKind::Reduce:
                    s.reduce.in = ptr[0];
                    s.reduce.out = ptr[1];
                    break;
                case StepKind::Softmax:
                    s.row.in0 = (const float*)ptr[0];
                    s.row.in1 = ptr.size() > 2 ? (const float*)ptr[2] : nullptr;   // additive term
                    s.row.out = (float*)ptr[1];
                    break;
                case StepKind::Layernorm:
                    s.row.in0 = (const float*)ptr[0];
                    s.row.out = (float*)ptr[1];
                    s.row.in1 = ptr.size() > 2 ? (const float*)ptr[2] : nullptr;
                    break;
                case StepKind::Gather:
                    s.gather.in = ptr[0];
                    s.gather.idx = ptr[1];
                    s.gather.out = ptr[2];
                    break;
                case StepKind::Gemm:
                    s.gemm.a = (const float*)ptr[0];
                    s.gemm.b = (const float*)ptr[1];
                    s.gemm.c = (float*)ptr[2];
                    s.gemm.scratch = nullptr;
                    if (s.gemm.splits > 1) {   // the split-K scratch buffer is the last operand
                        s.gemm.scratch = (float*)ptr.back();
                        ptr.pop_back();
                    }
                    s.gemm.add1 = ptr.size() > 3 ? (const float*)ptr[3] : nullptr;
                    s.gemm.add2 = ptr.size() > 4 ? (const float*)ptr[4] : nullptr;
                    if (s.gemm.row_softmax == 2) {   // fused attention: the fourth operand is V^T, there are no addends
                        s.gemm.values = s.gemm.add1;
                        s.gemm.add1 = nullptr;
                    }
                    break;
                case StepKind::Conv:
                    s.conv.in = (const float*)ptr[0];
                    s.conv.filter = (const float*)ptr[1];
                    s.conv.out = (float*)ptr[2];
                    s.conv.add1 = ptr.size() > 3 ? (const float*)ptr[3] : nullptr;
                    s.conv.add2 = ptr.size() > 4 ? (const float*)ptr[4] : nullptr;
                    break;
                case StepKind::Im2col:
                    s.im2col.in = (const float*)ptr[0];
                    s.im2col.col = (float*)ptr[1];
                    break;
                case StepKind::RmsNorm:
                    s.rms.in = ptr[0];
                    s.rms.out = ptr[1];
                    s.rms.gain = ptr.size() > 2 ? (const float*)ptr[2] : nullptr;
                    break;
                case StepKind::AllReduce:
                    s.all_reduce.in = ptr[0];
                    s.all_reduce.out = ptr[1];
                    break;
                case StepKind::ConvChain:
                    s.chain.in = (const float*)ptr[0];
                    s.chain.out = (float*)ptr[1];
                    s.chain.tiles = (const float*)ptr[2];
                    s.chain.bias = (const float*)ptr[3];
                    for (int h = 0; h < s.chain.n_heads; h++) s.chain.head_out[h] = (float*)ptr[4 + h];
                    break;
                default: fail(KN_ERR_INTERNAL, "unknown step kind");
            }
            if (s.tensor_core)
                tc_prepare_step(s, status_dev, plan->opts.flags, (plan->opts.flags & KN_FLAG_TRACE_GEMM) ? status_host + 4 : nullptr);
            launches += s.launches;
        }
    }

    void launch_step(const Step& s) {
        int err = 0;
        switch (s.kind) {
            case StepKind::Scalar: err = launch_scalar(s.scalar, stream); break;
            case StepKind::Reduce: err = launch_reduce(s.reduce, stream); break;
            case StepKind::Softmax: err = launch_softmax(s.row, stream); break;
            case StepKind::Layernorm: err = launch_layernorm(s.row, stream); break;
            case StepKind::Gather: err = launch_gather(s.gather, stream); break;
            case StepKind::Gemm: err = s.tensor_core ? tc_launch_step(s, stream) : launch_gemm_simt(s.gemm, stream); break;
            case StepKind::Conv: err = s.tensor_core ? tc_launch_step(s, stream) : launch_conv_simt(s.conv, stream); break;
            case StepKind::ConvChain: err = tc_launch_step(s, stream); break;
            case StepKind::Im2col: err = launch_im2col(s.im2col, stream); break;
            case StepKind::RmsNorm: err = launch_rmsnorm(s.rms, stream); break;
            case StepKind::AllReduce: {
                const AllReduceParams& a = s.all_reduce;
                if (comm != nullptr && comm->world > 1)
                    comm_all_reduce_sum(comm, a.in, a.out, (size_t)a.count, (DType)a.dtype, stream);
                else   // one rank: the sum is the value
                    err = (int)cudaMemcpyAsync(a.out, a.in, (size_t)a.count * dtype_size((DType)a.dtype), cudaMemcpyDeviceToDevice, stream);
                break;
            }
            default: fail(KN_ERR_INTERNAL, "unknown step kind");
        }
        if (err != 0)
            fail(KN_ERR_CUDA, std::string("launch of step ") + step_kind_name(s.kind) + " (" + s.desc + ") failed: " +
                                  cudaGetErrorString((cudaError_t)err));
    }

    void run_async() {
        if (plan->steps.empty()) return;
        if (profile) {
            std::vector<cudaEvent_t> ev(plan->steps.size() + 1, nullptr);
            try {
                for (auto& e : ev) KN_CUDA(cudaEventCreate(&e));
                KN_CUDA(cudaEventRecord(ev[0], stream));
                for (size_t i = 0; i < plan->steps.size(); i++) {
                    launch_step(plan->steps[i]);
                    KN_CUDA(cudaEventRecord(ev[i + 1], stream));
                }
                KN_CUDA(cudaStreamSynchronize(stream));
                step_us.assign(plan->steps.size(), 0.f);
                for (size_t i = 0; i < plan->steps.size(); i++) {
                    float ms = 0;
                    KN_CUDA(cudaEventElapsedTime(&ms, ev[i], ev[i + 1]));
                    step_us[i] = ms * 1000.f;
                }
            } catch (...) {
                for (auto& e : ev) if (e) cudaEventDestroy(e);
                throw;
            }
            for (auto& e : ev) cudaEventDestroy(e);
            return;
        }
        if (use_graph()) {
            if (!graph_exec) {
                cudaGraph_t graph = nullptr;
                KN_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
                try {
                    for (const Step& s : plan->steps) launch_step(s);
                } catch (...) {
                    cudaStreamEndCapture(stream, &graph);
                    if (graph) cudaGraphDestroy(graph);
                    throw;
                }
                KN_CUDA(cudaStreamEndCapture(stream, &graph));
                cudaError_t err = cudaGraphInstantiate(&graph_exec, graph, 0);
                cudaGraphDestroy(graph);
                KN_CUDA(err);
            }
            KN_CUDA(cudaGraphLaunch(graph_exec, stream));
        } else {
            for (const Step& s : plan->steps) launch_step(s);
        }
    }

    // The step list is captured into a CUDA graph and replayed, except when it contains collectives that go
    // through NCCL: those are enqueued call by call, so that a rank that fails between steps cannot leave a
    // captured collective half-issued on the others.
    bool use_graph() const { return plan->opts.use_cuda_graph && !(plan->collectives > 0 && comm != nullptr && comm->world > 1); }

    void upload_inputs() {
        for (size_t i = 0; i < pinned_in.size(); i++)
            if (bytes_in[i])
                KN_CUDA(cudaMemcpyAsync(device_ptr(plan->inputs[i]), pinned_in[i], bytes_in[i], cudaMemcpyHostToDevice, stream));
    }
    void download_outputs() {
        for (size_t i = 0; i < pinned_out.size(); i++)
            if (bytes_out[i])
                KN_CUDA(cudaMemcpyAsync(pinned_out[i], device_ptr(plan->outputs[i]), bytes_out[i], cudaMemcpyDeviceToHost, stream));
        KN_CUDA(cudaMemcpyAsync(status_host, status_dev, 4, cudaMemcpyDeviceToHost, stream));
    }
    void check_status() {
        if (*status_host != 0) {
            uint32_t code = *status_host;
            *status_host = 0;
            cudaMemsetAsync(status_dev, 0, 4, stream);
            fail(KN_ERR_INTERNAL, "a kernel gave up waiting on a barrier (code " + std::to_string(code) + ")");
        }
    }

    // One graph for a whole `evaluate`: input copies, the steps, output copies.  An output that is complete
    // before the last step (the large policy tensor of a two-headed network, say) starts its way back to
    // the host on a forked branch right after the step that produces it, so the copy overlaps the rest
    // of the step list instead of following it.
    void capture_evaluate() {
        const size_t n_steps = plan->steps.size();
        // last step that writes each output's buffer (-1: none, e.g. an output that is an input or a constant)
        std::vector<int> producer(plan->outputs.size(), -1);
        for (size_t o = 0; o < plan->outputs.size(); o++)
            for (size_t i = 0; i < n_steps; i++)
                for (size_t k = 0; k < plan->steps[i].operands.size(); k++)
                    if (plan->steps[i].writes[k] && plan->steps[i].operands[k].buf == plan->outputs[o].buf) producer[o] = (int)i;
        if (!side_stream) KN_CUDA(cudaStreamCreateWithFlags(&side_stream, cudaStreamNonBlocking));
        std::vector<cudaEvent_t> events;
        auto new_event = [&]() {
            cudaEvent_t e;
            KN_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            events.push_back(e);
            return e;
        };
        auto copy_out = [&](size_t o, cudaStream_t st) {
            if (bytes_out[o])
                KN_CUDA(cudaMemcpyAsync(pinned_out[o], device_ptr(plan->outputs[o]), bytes_out[o], cudaMemcpyDeviceToHost, st));
        };
        cudaGraph_t graph = nullptr;
        KN_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        try {
            upload_inputs();
            bool forked = false;
            for (size_t i = 0; i < n_steps; i++) {
                launch_step(plan->steps[i]);
                if (i + 1 == n_steps) break;
                for (size_t o = 0; o < producer.size(); o++) {
                    if (producer[o] != (int)i || bytes_out[o] == 0) continue;
                    cudaEvent_t e = new_event();
                    KN_CUDA(cudaEventRecord(e, stream));
                    KN_CUDA(cudaStreamWaitEvent(side_stream, e, 0));
                    copy_out(o, side_stream);
                    forked = true;
                }
            }
            for (size_t o = 0; o < producer.size(); o++)
                if (n_steps == 0 || producer[o] < 0 || producer[o] == (int)n_steps - 1) copy_out(o, stream);
            KN_CUDA(cudaMemcpyAsync(status_host, status_dev, 4, cudaMemcpyDeviceToHost, stream));
            if (forked) {
                cudaEvent_t e = new_event();
                KN_CUDA(cudaEventRecord(e, side_stream));
                KN_CUDA(cudaStreamWaitEvent(stream, e, 0));
            }
        } catch (...) {
            cudaStreamEndCapture(stream, &graph);
            if (graph) cudaGraphDestroy(graph);
            for (cudaEvent_t e : events) cudaEventDestroy(e);
            throw;
        }
        cudaError_t end = cudaStreamEndCapture(stream, &graph);
        for (cudaEvent_t e : events) cudaEventDestroy(e);
        KN_CUDA(end);
        cudaError_t err = cudaGraphInstantiate(&eval_graph_exec, graph, 0);
        cudaGraphDestroy(graph);
        KN_CUDA(err);
    }

    void evaluate(const void* const* inputs, void* const* outputs) {
        evaluate_begin(inputs);
        evaluate_end(outputs);
    }

    bool in_flight = false;   // evaluate_begin without its evaluate_end

    void evaluate_begin(const void* const* inputs) {
        KN_CHECK(!in_flight, KN_ERR_INVALID_ARG, "evaluate_begin while an evaluation is in flight");
        KN_CUDA(cudaStreamSynchronize(stream));
        for (size_t i = 0; i < pinned_in.size(); i++) {
            KN_CHECK(inputs != nullptr && (inputs[i] != nullptr || bytes_in[i] == 0), KN_ERR_INVALID_ARG, "null input buffer");
            if (bytes_in[i] && inputs[i] != pinned_in[i]) memcpy(pinned_in[i], inputs[i], bytes_in[i]);
        }
        if (use_graph() && !profile) {
            if (!eval_graph_exec) capture_evaluate();
            KN_CUDA(cudaGraphLaunch(eval_graph_exec, stream));
        } else {
            upload_inputs();
            run_async();
            download_outputs();
        }
        in_flight = true;
    }

    void evaluate_end(void* const* outputs) {
        KN_CHECK(in_flight, KN_ERR_INVALID_ARG, "evaluate_end without evaluate_begin");
        in_flight = false;
        {
            cudaError_t done = cudaStreamSynchronize(stream);
            if (done != cudaSuccess && (plan->opts.flags & KN_FLAG_TRACE_GEMM)) {
                std::string m = std::string("cudaStreamSynchronize failed: ") + cudaGetErrorString(done) + "; matmul progress markers:";
                for (int i = 0; i < 8; i++) m += " " + std::to_string(status_host[4 + i]);
                fail(KN_ERR_CUDA, m);
            }
            KN_CUDA(done);
        }
        check_status();
        for (size_t i = 0; i < pinned_out.size(); i++) {
            KN_CHECK(outputs != nullptr && (outputs[i] != nullptr || bytes_out[i] == 0), KN_ERR_INVALID_ARG, "null output buffer");
            if (dtype_out[i] == DType::Bool) {
                const uint8_t* b = (const uint8_t*)pinned_out[i];
                for (size_t k = 0; k < bytes_out[i]; k++)
                    KN_CHECK(b[k] <= 1, KN_ERR_INTERNAL, "bool output holds a value other than 0 or 1");
            }
            if (bytes_out[i] && outputs[i] != pinned_out[i]) memcpy(outputs[i], pinned_out[i], bytes_out[i]);
        }
    }
};

static std::unique_ptr<Executor> create_executor(int device, const Graph& graph, size_t batch, const kn_options& opts) {
    int count = 0;
    cudaError_t cerr = cudaGetDeviceCount(&count);
    if (cerr != cudaSuccess || count == 0)
        fail(KN_ERR_NO_DEVICE, std::string("no CUDA device available: ") + cudaGetErrorString(cerr));
    KN_CHECK(device >= 0 && device < count, KN_ERR_NO_DEVICE, "CUDA device " + std::to_string(device) + " not available");

    auto ex = std::make_unique<Executor>();
    ex->device = device;
    DeviceGuard guard(device);
    ex->plan = make_plan(graph, (int64_t)batch, opts);
    Plan& plan = *ex->plan;
    KN_CUDA(cudaStreamCreateWithFlags(&ex->stream, cudaStreamNonBlocking));
    KN_CUDA(cudaMalloc((void**)&ex->arena, std::max<size_t>(plan.arena_bytes, 256)));
    KN_CUDA(cudaMalloc((void**)&ex->consts, std::max<size_t>(plan.const_bytes, 256)));
    KN_CUDA(cudaMalloc((void**)&ex->status_dev, 256));
    KN_CUDA(cudaMemset(ex->status_dev, 0, 256));
    KN_CUDA(cudaHostAlloc((void**)&ex->status_host, 64, cudaHostAllocDefault));
    memset(ex->status_host, 0, 64);   // word 0: status mirror; words 4..11: matmul progress markers (KN_FLAG_TRACE_GEMM)
    if (plan.const_bytes) {
        // constants cross to the device once, here (kn-cuda-eval/src/planner.rs:331-344)
        std::vector<uint8_t> staging(plan.const_bytes, 0);
        for (auto& b : plan.buffers)
            if (b.kind == BufKind::Const && b.bytes) memcpy(staging.data() + b.arena_offset, b.host_data, b.bytes);
        KN_CUDA(cudaMemcpy(ex->consts, staging.data(), plan.const_bytes, cudaMemcpyHostToDevice));
    }
    for (auto& b : plan.buffers) {   // host copies are no longer needed
        b.host_data = nullptr;
        b.owned.reset();
    }
    for (size_t i = 0; i < plan.inputs.size(); i++) {
        size_t bytes = (size_t)plan.inputs[i].ss.size() * dtype_size(plan.inputs[i].dtype);
        void* p = nullptr;
        KN_CUDA(cudaHostAlloc(&p, std::max<size_t>(bytes, 16), cudaHostAllocDefault));
        memset(p, 0, std::max<size_t>(bytes, 16));
        ex->pinned_in.push_back(p);
        ex->bytes_in.push_back(bytes);
        ex->dtype_in.push_back(plan.inputs[i].dtype);
    }
    for (size_t i = 0; i < plan.outputs.size(); i++) {
        size_t bytes = (size_t)plan.outputs[i].ss.size() * dtype_size(plan.outputs[i].dtype);
        void* p = nullptr;
        KN_CUDA(cudaHostAlloc(&p, std::max<size_t>(bytes, 16), cudaHostAllocDefault));
        memset(p, 0, std::max<size_t>(bytes, 16));
        ex->pinned_out.push_back(p);
        ex->bytes_out.push_back(bytes);
        ex->dtype_out.push_back(plan.outputs[i].dtype);
    }
    KN_CUDA(cudaMemsetAsync(ex->arena, 0, std::max<size_t>(plan.arena_bytes, 256), ex->stream));
    ex->patch_pointers();
    KN_CUDA(cudaStreamSynchronize(ex->stream));
    return ex;
}

}  // namespace kn

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
struct kn_graph {
    std::unique_ptr<kn::Graph> g;
};
struct kn_executor {
    std::unique_ptr<kn::Executor> e;
};
struct kn_comm {
    kn::Comm* c = nullptr;
};

namespace {

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return KN_OK;
    } catch (const kn::Error& e) {
        kn::g_last_error = e.what();
        return e.code;
    } catch (const std::bad_alloc&) {
        kn::g_last_error = "out of host memory";
        return KN_ERR_INTERNAL;
    } catch (const std::exception& e) {
        kn::g_last_error = e.what();
        return KN_ERR_INTERNAL;
    }
}

kn_options resolve_options(const kn_options* opts) {
    kn_options o;
    kn_options_default(&o);
    if (opts) {
        KN_CHECK(opts->struct_size == sizeof(kn_options), KN_ERR_INVALID_ARG, "kn_options.struct_size does not match this library");
        KN_CHECK(opts->math_mode == KN_MATH_TF32 || opts->math_mode == KN_MATH_F32, KN_ERR_INVALID_ARG, "unknown math mode");
        o = *opts;
    }
    return o;
}

int write_text(const std::string& text, char* buf, size_t cap, size_t* needed) {
    if (needed) *needed = text.size();
    if (buf && cap) {
        size_t n = std::min(cap - 1, text.size());
        memcpy(buf, text.data(), n);
        buf[n] = 0;
    }
    return KN_OK;
}

}  // namespace

extern "C" {

const char* kn_last_error(void) { return kn::g_last_error.c_str(); }

int kn_version(void) { return 1000; }

int kn_options_default(kn_options* opts) {
    if (!opts) return KN_ERR_INVALID_ARG;
    opts->struct_size = sizeof(kn_options);
    opts->math_mode = KN_MATH_TF32;
    opts->use_cuda_graph = 1;
    opts->flags = 0;
    return KN_OK;
}

int kn_device_count(int* count) {
    return guarded([&] {
        KN_CHECK(count != nullptr, KN_ERR_INVALID_ARG, "null count");
        int n = 0;
        cudaError_t err = cudaGetDeviceCount(&n);
        if (err != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        *count = n;
    });
}

int kn_graph_from_blob(const void* bytes, size_t len, kn_graph** out) {
    return guarded([&] {
        KN_CHECK(out != nullptr, KN_ERR_INVALID_ARG, "null out pointer");
        *out = nullptr;
        auto g = kn::Graph::parse(bytes, len);
        *out = new kn_graph{std::move(g)};
    });
}

void kn_graph_destroy(kn_graph* graph) { delete graph; }

int kn_graph_io_count(const kn_graph* graph, int* n_inputs, int* n_outputs, int* n_values) {
    return guarded([&] {
        KN_CHECK(graph != nullptr, KN_ERR_INVALID_ARG, "null graph");
        if (n_inputs) *n_inputs = (int)graph->g->inputs.size();
        if (n_outputs) *n_outputs = (int)graph->g->outputs.size();
        if (n_values) *n_values = (int)graph->g->values.size();
    });
}

int kn_plan_describe(const kn_graph* graph, size_t batch_size, const kn_options* opts, char* buf, size_t cap, size_t* needed) {
    return guarded([&] {
        KN_CHECK(graph != nullptr, KN_ERR_INVALID_ARG, "null graph");
        kn_options o = resolve_options(opts);
        auto plan = kn::make_plan(*graph->g, (int64_t)batch_size, o);
        write_text(plan->describe(), buf, cap, needed);
    });
}

int kn_executor_create(int device, const kn_graph* graph, size_t batch_size, const kn_options* opts, kn_executor** out) {
    return guarded([&] {
        KN_CHECK(out != nullptr, KN_ERR_INVALID_ARG, "null out pointer");
        *out = nullptr;
        KN_CHECK(graph != nullptr, KN_ERR_INVALID_ARG, "null graph");
        kn_options o = resolve_options(opts);
        auto e = kn::create_executor(device, *graph->g, batch_size, o);
        *out = new kn_executor{std::move(e)};
    });
}

void kn_executor_destroy(kn_executor* exec) { delete exec; }

int kn_executor_io_count(const kn_executor* exec, int* n_inputs, int* n_outputs) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        if (n_inputs) *n_inputs = (int)exec->e->plan->inputs.size();
        if (n_outputs) *n_outputs = (int)exec->e->plan->outputs.size();
    });
}

static const kn::PlanTensor& io_tensor(const kn_executor* exec, int is_output, int index) {
    KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
    const auto& list = is_output ? exec->e->plan->outputs : exec->e->plan->inputs;
    KN_CHECK(index >= 0 && (size_t)index < list.size(), KN_ERR_INVALID_ARG, "input/output index out of range");
    return list[index];
}

int kn_executor_io_info(const kn_executor* exec, int is_output, int index, kn_tensor_info* info) {
    return guarded([&] {
        KN_CHECK(info != nullptr, KN_ERR_INVALID_ARG, "null info");
        const kn::PlanTensor& t = io_tensor(exec, is_output, index);
        KN_CHECK(t.ss.rank() <= KN_MAX_RANK, KN_ERR_UNSUPPORTED, "input/output rank above 8");
        info->dtype = (int32_t)t.dtype;
        info->rank = t.ss.rank();
        for (int d = 0; d < KN_MAX_RANK; d++) info->dims[d] = d < t.ss.rank() ? t.ss.shape[d] : 1;
        info->bytes = (uint64_t)t.ss.size() * kn::dtype_size(t.dtype);
    });
}

int kn_executor_evaluate(kn_executor* exec, const void* const* inputs, void* const* outputs) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->evaluate(inputs, outputs);
    });
}

int kn_executor_evaluate_begin(kn_executor* exec, const void* const* inputs) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->evaluate_begin(inputs);
    });
}

int kn_executor_evaluate_end(kn_executor* exec, void* const* outputs) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->evaluate_end(outputs);
    });
}

int kn_executor_run_async(kn_executor* exec) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->run_async();
    });
}

int kn_executor_synchronize(kn_executor* exec) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        KN_CUDA(cudaMemcpyAsync(exec->e->status_host, exec->e->status_dev, 4, cudaMemcpyDeviceToHost, exec->e->stream));
        KN_CUDA(cudaStreamSynchronize(exec->e->stream));
        exec->e->check_status();
    });
}

int kn_executor_stream(kn_executor* exec, void** stream) {
    return guarded([&] {
        KN_CHECK(exec != nullptr && stream != nullptr, KN_ERR_INVALID_ARG, "null argument");
        *stream = (void*)exec->e->stream;
    });
}

int kn_executor_host_buffer(kn_executor* exec, int is_output, int index, void** ptr, uint64_t* bytes) {
    return guarded([&] {
        io_tensor(exec, is_output, index);
        if (ptr) *ptr = is_output ? exec->e->pinned_out[index] : exec->e->pinned_in[index];
        if (bytes) *bytes = is_output ? exec->e->bytes_out[index] : exec->e->bytes_in[index];
    });
}

int kn_executor_device_buffer(kn_executor* exec, int is_output, int index, void** ptr, uint64_t* bytes) {
    return guarded([&] {
        const kn::PlanTensor& t = io_tensor(exec, is_output, index);
        if (ptr) *ptr = exec->e->device_ptr(t);
        if (bytes) *bytes = is_output ? exec->e->bytes_out[index] : exec->e->bytes_in[index];
    });
}

int kn_executor_upload_inputs(kn_executor* exec) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->upload_inputs();
    });
}

int kn_executor_download_outputs(kn_executor* exec) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::DeviceGuard guard(exec->e->device);
        exec->e->download_outputs();
    });
}

int kn_executor_mem_usage(const kn_executor* exec, kn_mem_usage* usage) {
    return guarded([&] {
        KN_CHECK(exec != nullptr && usage != nullptr, KN_ERR_INVALID_ARG, "null argument");
        *usage = exec->e->plan->mem;
    });
}

int kn_executor_step_count(const kn_executor* exec, int* steps, int* launches) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        if (steps) *steps = (int)exec->e->plan->steps.size();
        if (launches) *launches = exec->e->launches;
    });
}

int kn_executor_set_profile(kn_executor* exec, int enable) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        exec->e->profile = enable != 0;
    });
}

int kn_executor_last_profile(kn_executor* exec, char* buf, size_t cap, size_t* needed) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        const kn::Plan& plan = *exec->e->plan;
        std::ostringstream os;
        double total[(int)kn::StepKind::COUNT] = {0};
        double total_tc = 0;
        const auto& us = exec->e->step_us;
        for (size_t i = 0; i < plan.steps.size() && i < us.size(); i++) {
            const kn::Step& s = plan.steps[i];
            os << i << " " << kn::step_kind_name(s.kind) << (s.tensor_core ? "/tc" : "") << " " << us[i] << " "
               << (uint64_t)s.alg_bytes << " " << (uint64_t)s.flops << " " << s.desc << "\n";
            total[(int)s.kind] += us[i];
            if (s.tensor_core) total_tc += us[i];
        }
        for (int k = 0; k < (int)kn::StepKind::COUNT; k++)
            os << "total " << kn::step_kind_name((kn::StepKind)k) << " " << total[k] << "\n";
        os << "total tensor_core " << total_tc << "\n";
        write_text(os.str(), buf, cap, needed);
    });
}

int kn_executor_time_step(kn_executor* exec, int step, int launches, float* microseconds) {
    return guarded([&] {
        KN_CHECK(exec != nullptr && microseconds != nullptr, KN_ERR_INVALID_ARG, "null argument");
        kn::Executor& e = *exec->e;
        KN_CHECK(step >= 0 && (size_t)step < e.plan->steps.size(), KN_ERR_INVALID_ARG, "step index out of range");
        KN_CHECK(launches >= 1 && launches <= 100000, KN_ERR_INVALID_ARG, "launch count out of range");
        kn::DeviceGuard guard(e.device);
        cudaEvent_t a, b;
        KN_CUDA(cudaEventCreate(&a));
        KN_CUDA(cudaEventCreate(&b));
        try {
            e.launch_step(e.plan->steps[step]);   // warm
            KN_CUDA(cudaEventRecord(a, e.stream));
            for (int i = 0; i < launches; i++) e.launch_step(e.plan->steps[step]);
            KN_CUDA(cudaEventRecord(b, e.stream));
            KN_CUDA(cudaStreamSynchronize(e.stream));
            float ms = 0;
            KN_CUDA(cudaEventElapsedTime(&ms, a, b));
            *microseconds = ms * 1000.f / (float)launches;
        } catch (...) {
            cudaEventDestroy(a);
            cudaEventDestroy(b);
            throw;
        }
        cudaEventDestroy(a);
        cudaEventDestroy(b);
    });
}

int kn_nccl_load(const char* path) {
    return guarded([&] { kn::nccl_load(path); });
}

int kn_comm_unique_id(void* id, size_t id_bytes) {
    return guarded([&] {
        KN_CHECK(id != nullptr && id_bytes == KN_COMM_ID_BYTES, KN_ERR_INVALID_ARG, "the id buffer must be KN_COMM_ID_BYTES long");
        kn::comm_unique_id(id);
    });
}

int kn_comm_create(int device, int rank, int world, const void* id, size_t id_bytes, kn_comm** out) {
    return guarded([&] {
        KN_CHECK(out != nullptr, KN_ERR_INVALID_ARG, "null out pointer");
        *out = nullptr;
        KN_CHECK(id != nullptr && id_bytes == KN_COMM_ID_BYTES, KN_ERR_INVALID_ARG, "the id buffer must be KN_COMM_ID_BYTES long");
        kn::Comm* c = kn::comm_create(device, rank, world, id);
        *out = new kn_comm{c};
    });
}

void kn_comm_destroy(kn_comm* comm) {
    if (!comm) return;
    kn::comm_destroy(comm->c);
    delete comm;
}

int kn_executor_set_comm(kn_executor* exec, kn_comm* comm) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        kn::Executor& e = *exec->e;
        KN_CHECK(!e.in_flight, KN_ERR_INVALID_ARG, "an evaluation is in flight");
        KN_CHECK(comm == nullptr || comm->c->device == e.device, KN_ERR_INVALID_ARG, "communicator and executor are on different devices");
        kn::DeviceGuard guard(e.device);
        KN_CUDA(cudaStreamSynchronize(e.stream));
        // graphs captured under the previous setting would replay the wrong kind of step
        if (e.graph_exec) { cudaGraphExecDestroy(e.graph_exec); e.graph_exec = nullptr; }
        if (e.eval_graph_exec) { cudaGraphExecDestroy(e.eval_graph_exec); e.eval_graph_exec = nullptr; }
        e.comm = comm ? comm->c : nullptr;
    });
}

int kn_executor_selftest_wait_expiry(kn_executor* exec, uint32_t limit_us) {
    return guarded([&] {
        KN_CHECK(exec != nullptr, KN_ERR_INVALID_ARG, "null executor");
        KN_CHECK(limit_us >= 1 && limit_us <= 100000, KN_ERR_INVALID_ARG, "limit must be 1 .. 100000 microseconds");
        kn::Executor& e = *exec->e;
        KN_CHECK(!e.in_flight, KN_ERR_INVALID_ARG, "an evaluation is in flight");
        kn::DeviceGuard guard(e.device);
        int khz = 0;
        KN_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, e.device));
        const long long cycles = (long long)limit_us * (long long)(khz > 0 ? khz : 2000000) / 1000ll;
        kn::wait_expiry_kernel<<<1, 32, 0, e.stream>>>(e.status_dev, cycles, 99u);
        KN_CUDA(cudaGetLastError());
        KN_CUDA(cudaMemcpyAsync(e.status_host, e.status_dev, 4, cudaMemcpyDeviceToHost, e.stream));
        KN_CUDA(cudaStreamSynchronize(e.stream));
        e.check_status();   // throws KN_ERR_INTERNAL: the expected outcome
    });
}

int kn_strided_shape(int op, int rank, const int64_t* shape, const int64_t* strides, int n_args, const int64_t* args, int* out_rank,
                     int64_t* out_shape, int64_t* out_strides, int* simple, int* dense) {
    return guarded([&] {
        KN_CHECK(rank >= 0 && rank <= 16 && n_args >= 0 && n_args <= 16, KN_ERR_INVALID_ARG, "rank or argument count above 16");
        KN_CHECK((rank == 0 || (shape != nullptr && strides != nullptr)) && (n_args == 0 || args != nullptr), KN_ERR_INVALID_ARG, "null array");
        std::vector<int64_t> sh(shape, shape + rank), st(strides, strides + rank), a(args, args + n_args);
        for (int64_t d : sh) KN_CHECK(d >= 0, KN_ERR_INVALID_ARG, "negative extent");
        kn::StridedShape s(sh, st), r;
        auto axis = [&](int i) {
            KN_CHECK(n_args > i && a[i] >= 0 && a[i] < rank, KN_ERR_INVALID_ARG, "axis out of range");
            return (int)a[i];
        };
        switch (op) {
            case 0: r = s; break;
            case 1: {
                for (int64_t d : a) KN_CHECK(d >= 0, KN_ERR_INVALID_ARG, "negative extent");
                int64_t n = 1;
                for (int64_t d : a) n *= d;
                KN_CHECK(n == s.size(), KN_ERR_INVALID_ARG, "a view keeps the element count");
                auto v = s.view(a);
                KN_CHECK(v.has_value(), KN_ERR_SHAPE, "cannot view " + s.str() + " as the requested shape without a copy");
                r = *v;
                break;
            }
            case 2:
                KN_CHECK(n_args == 4 && a[3] >= 1 && a[1] >= 0 && a[2] >= a[1], KN_ERR_INVALID_ARG, "slice takes axis, start, end >= start, step >= 1");
                r = s.slice(axis(0), a[1], a[2], a[3]);
                break;
            case 3: r = s.flip(axis(0)); break;
            case 4: {
                KN_CHECK(n_args == rank, KN_ERR_INVALID_ARG, "permutation length differs from the rank");
                std::vector<int> perm;
                std::vector<bool> seen(rank, false);
                for (int i = 0; i < rank; i++) {
                    const int p = axis(i);
                    KN_CHECK(!seen[p], KN_ERR_INVALID_ARG, "not a permutation");
                    seen[p] = true;
                    perm.push_back(p);
                }
                r = s.permute(perm);
                break;
            }
            case 5:
                KN_CHECK(n_args == rank, KN_ERR_INVALID_ARG, "broadcast keeps the rank");
                for (int i = 0; i < rank; i++)
                    KN_CHECK(a[i] == sh[i] || sh[i] == 1, KN_ERR_INVALID_ARG, "only axes of size 1 can be broadcast");
                r = s.broadcast(a);
                break;
            default: kn::fail(KN_ERR_INVALID_ARG, "unknown operation");
        }
        if (out_rank) *out_rank = r.rank();
        for (int i = 0; i < r.rank(); i++) {
            if (out_shape) out_shape[i] = r.shape[i];
            if (out_strides) out_strides[i] = r.strides[i];
        }
        if (simple) *simple = r.has_simple_strides() ? 1 : 0;
        if (dense) *dense = r.has_dense_strides() ? 1 : 0;
    });
}

int kn_scalar_unary(int unary_op, int from_dtype, int to_dtype, uint64_t x, uint64_t* out) {
    return guarded([&] {
        KN_CHECK(out != nullptr, KN_ERR_INVALID_ARG, "null out");
        KN_CHECK(unary_op >= 0 && unary_op <= (int)kn::UnaryOp::BitCast, KN_ERR_INVALID_ARG, "unknown unary op");
        KN_CHECK(from_dtype >= 0 && from_dtype < (int)kn::DType::COUNT && to_dtype >= 0 && to_dtype < (int)kn::DType::COUNT,
                 KN_ERR_INVALID_ARG, "unknown dtype");
        *out = kn::unary_bits((kn::UnaryOp)unary_op, (kn::DType)from_dtype, (kn::DType)to_dtype, x);
    });
}

int kn_scalar_binary(int binary_op, int dtype, uint64_t a, uint64_t b, uint64_t* out) {
    return guarded([&] {
        KN_CHECK(out != nullptr, KN_ERR_INVALID_ARG, "null out");
        KN_CHECK(binary_op >= 0 && binary_op <= (int)kn::BinaryOp::Pow, KN_ERR_INVALID_ARG, "unknown binary op");
        KN_CHECK(dtype >= 0 && dtype < (int)kn::DType::COUNT, KN_ERR_INVALID_ARG, "unknown dtype");
        *out = kn::binary_bits((kn::BinaryOp)binary_op, (kn::DType)dtype, a, b);
    });
}

}  // extern "C"
