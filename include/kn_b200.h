/* kn_b200.h -- C ABI of the B200-native executor for Kyanite's graph IR.
 *
 * The entry points below are what a host binding (Rust FFI, ctypes, cgo ...) binds in place of the
 * reference's CUDA stack for this path: the `CudaExecutor` of kn-cuda-eval together with the
 * kn-cuda-sys bindings underneath it (cuDNN, cuBLAS, NVRTC, cudart).  Each declaration cites the
 * reference interface it replaces as `path:line` inside the reference project.
 *
 * Conventions
 *  - every function returns a `kn_status`; on failure `kn_last_error()` holds a message for the
 *    calling thread.  Nothing aborts the process (the reference panics instead:
 *    kn-cuda-sys/src/wrapper/status.rs:17-32; a binding that wants that behaviour panics on a
 *    non-zero status).
 *  - an executor is used by one thread at a time but may move between threads; different
 *    executors (devices) may run concurrently (kn-cuda-eval/src/executor.rs:39-41).
 *  - the library selects the executor's device itself on every entry.
 *  - all tensors crossing the boundary are dense, row-major ("standard layout") host arrays of the
 *    dtype reported by `kn_executor_io_info`.
 */
#ifndef KN_B200_H
#define KN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KN_API __attribute__((visibility("default")))
#else
#define KN_API
#endif

typedef enum kn_status {
    KN_OK = 0,
    KN_ERR_INVALID_ARG = 1, /* null pointer, index out of range, wrong struct size */
    KN_ERR_BAD_GRAPH = 2,   /* malformed graph blob */
    KN_ERR_UNSUPPORTED = 3, /* valid graph the executor cannot run (rank / dtype limits) */
    KN_ERR_CUDA = 4,        /* a CUDA runtime or driver call failed; message holds the CUDA error */
    KN_ERR_SHAPE = 5,       /* shapes inconsistent for the given batch size */
    KN_ERR_NO_DEVICE = 6,   /* requested device does not exist (CudaDeviceNotAvailable) */
    KN_ERR_INTERNAL = 7
} kn_status;

/* dtype tags: the reference's `DType` in declaration order (kn-graph/src/dtype.rs:25-37) plus F16 */
typedef enum kn_dtype {
    KN_F32 = 0, KN_F64, KN_I8, KN_I16, KN_I32, KN_I64, KN_U8, KN_U16, KN_U32, KN_U64, KN_BOOL, KN_F16
} kn_dtype;

/* how f32 contractions (MatMul, Conv) are computed */
typedef enum kn_math_mode {
    KN_MATH_TF32 = 0, /* tcgen05 tensor cores, TF32 operands, f32 accumulate (default).  This is what
                         the reference's cuDNN convolutions use on Ampere-and-later GPUs. */
    KN_MATH_F32 = 1   /* exact f32 FMA on the SIMT pipes (what the reference's cublasSgemm uses) */
} kn_math_mode;

typedef struct kn_options {
    uint32_t struct_size;   /* = sizeof(kn_options) */
    int32_t math_mode;      /* kn_math_mode */
    int32_t use_cuda_graph; /* 1: capture the step list once and replay it (default), 0: launch steps */
    int32_t flags;          /* bit set of KN_FLAG_*, 0 by default */
} kn_options;

/* keep every convolution its own step: do not merge runs of stride-1 3x3 convolutions into the
   shared-memory-resident chain kernel (for A/B comparison and tests) */
#define KN_FLAG_NO_CONV_CHAIN 1
/* matrix multiplies use the one-tile-per-CTA kernel instead of the persistent one (A/B comparison and tests) */
#define KN_FLAG_NO_PERSISTENT_GEMM 2

/* post-mortem aid: the persistent matmul kernel records how far its roles got in pinned host memory, and a CUDA
   failure reported by kn_executor_evaluate / _end carries those markers in its message */
#define KN_FLAG_TRACE_GEMM 4

#define KN_MAX_RANK 8

typedef struct kn_tensor_info {
    int32_t dtype; /* kn_dtype */
    int32_t rank;
    int64_t dims[KN_MAX_RANK];
    uint64_t bytes;
} kn_tensor_info;

/* kn-cuda-eval/src/planner.rs:67-81 `MemoryUsage` */
typedef struct kn_mem_usage {
    uint64_t dedicated_bytes;  /* constants */
    uint64_t shared_bytes;     /* the activation arena actually allocated */
    uint64_t zero_bytes;
    uint64_t hypo_peak_bytes;  /* lower bound: largest sum of simultaneously live buffers */
    uint64_t hypo_total_bytes; /* sum of all shared buffers if nothing were reused */
} kn_mem_usage;

typedef struct kn_graph kn_graph;
typedef struct kn_executor kn_executor;

/* Message of the last failure on this thread; never NULL. */
KN_API const char* kn_last_error(void);

/* Library ABI version (major * 1000 + minor). */
KN_API int kn_version(void);

/* Fills a default option block. */
KN_API int kn_options_default(kn_options* opts);

/* Number of CUDA devices.  Replaces `CudaDevice::all` / `cudaGetDeviceCount`
 * (kn-cuda-sys/src/wrapper/handle.rs:38-48). */
KN_API int kn_device_count(int* count);

/* Builds the graph from its serialised form (see kyanite_b200/graph.py `Graph.to_bytes` for the
 * layout).  The reference passes `&Graph` by reference inside one Rust process
 * (kn-cuda-eval/src/executor.rs:61); a Rust value cannot cross a C boundary, so the binding walks
 * `graph.values()` (kn-graph/src/graph.rs:391-394) and serialises each `ValueInfo`.
 * The blob is copied; the caller may free it afterwards. */
KN_API int kn_graph_from_blob(const void* bytes, size_t len, kn_graph** out);
KN_API void kn_graph_destroy(kn_graph* graph);
KN_API int kn_graph_io_count(const kn_graph* graph, int* n_inputs, int* n_outputs, int* n_values);

/* Host-only: lowers the graph for `batch_size` and writes a text description of the step list and
 * memory plan into `buf` (NUL-terminated, truncated to `cap`); `*needed` receives the full length.
 * Touches no CUDA API.  Mirrors the reference's `Debug` dump of a `CudaExecutor`
 * (kn-cuda-eval/src/executor.rs:269-289). */
KN_API int kn_plan_describe(const kn_graph* graph, size_t batch_size, const kn_options* opts, char* buf, size_t cap,
                     size_t* needed);

/* `CudaExecutor::new(device, &graph, batch_size)` (kn-cuda-eval/src/executor.rs:61-110): plans the
 * graph, allocates the arena, uploads constants, allocates pinned staging for inputs and outputs.
 * The graph handle may be destroyed afterwards. */
KN_API int kn_executor_create(int device, const kn_graph* graph, size_t batch_size, const kn_options* opts,
                       kn_executor** out);
KN_API void kn_executor_destroy(kn_executor* exec);

KN_API int kn_executor_io_count(const kn_executor* exec, int* n_inputs, int* n_outputs);
/* Shape and dtype of input/output `index` at this executor's batch size
 * (`graph.input_shapes()` / `output_shapes()` evaluated, kn-cuda-eval/src/executor.rs:118-127). */
KN_API int kn_executor_io_info(const kn_executor* exec, int is_output, int index, kn_tensor_info* info);

/* `CudaExecutor::evaluate(&inputs) -> &[DTensor]` (kn-cuda-eval/src/executor.rs:117-195):
 * copies every input to the device, runs all steps, copies every output back and waits.
 * `inputs[i]` / `outputs[i]` are host buffers of `kn_executor_io_info(..).bytes` bytes.  Passing
 * the executor's own staging pointer (kn_executor_host_buffer) for an entry skips the extra host
 * copy for it.  Bool outputs are validated to be 0/1 (executor.rs:181-189). */
KN_API int kn_executor_evaluate(kn_executor* exec, const void* const* inputs, void* const* outputs);
/* `evaluate` in two halves, for hosts that keep several executors of one device busy at once (the
 * reference's self-play and server loops run several executor threads per GPU; here one thread can do it):
 * `begin` stages the inputs and enqueues upload, steps and download on the executor's stream without waiting,
 * `end` waits, checks the status word and hands out the outputs.  While executor A computes, executor B's
 * upload and A's previous download use the copy engines.  One evaluation per executor may be in flight. */
KN_API int kn_executor_evaluate_begin(kn_executor* exec, const void* const* inputs);
KN_API int kn_executor_evaluate_end(kn_executor* exec, void* const* outputs);

/* `CudaExecutor::run_async` (kn-cuda-eval/src/executor.rs:199-258): enqueues the steps on the
 * executor's stream without touching host memory; inputs are whatever the device input buffers hold. */
KN_API int kn_executor_run_async(kn_executor* exec);
/* `stream().synchronize()` (kn-cuda-sys/src/wrapper/handle.rs:128-132) */
KN_API int kn_executor_synchronize(kn_executor* exec);
/* The `cudaStream_t` the steps run on, as an opaque pointer (`CudaExecutor::stream`, executor.rs:263-265). */
KN_API int kn_executor_stream(kn_executor* exec, void** stream);

/* Pinned host staging buffer of input/output `index` (the reference keeps these private:
 * kn-cuda-eval/src/executor.rs:74-95). */
KN_API int kn_executor_host_buffer(kn_executor* exec, int is_output, int index, void** ptr, uint64_t* bytes);
/* Device buffer of input/output `index` (`device_inputs` / `device_outputs`, executor.rs:27-28).
 * Outputs may be strided views in the reference; here they are always dense. */
KN_API int kn_executor_device_buffer(kn_executor* exec, int is_output, int index, void** ptr, uint64_t* bytes);
/* Asynchronous halves of `evaluate`: staging -> device for all inputs, device -> staging for all outputs. */
KN_API int kn_executor_upload_inputs(kn_executor* exec);
KN_API int kn_executor_download_outputs(kn_executor* exec);

/* `executor.mem_usage` (kn-cuda-eval/src/executor.rs:33, planner.rs:67-81) */
KN_API int kn_executor_mem_usage(const kn_executor* exec, kn_mem_usage* usage);
/* Number of steps and of kernel launches one `run_async` issues. */
KN_API int kn_executor_step_count(const kn_executor* exec, int* steps, int* launches);

/* `set_profile` / `last_profile` (kn-cuda-eval/src/executor.rs:43-58, 208-257, 291-325): with
 * profiling on, the next `run_async`/`evaluate` launches step by step (no graph replay) with a CUDA
 * event pair around each step.  `kn_executor_last_profile` writes one line per step
 * (`index kind microseconds algorithmic_bytes flops description`) followed by per-kind totals. */
KN_API int kn_executor_set_profile(kn_executor* exec, int enable);
KN_API int kn_executor_last_profile(kn_executor* exec, char* buf, size_t cap, size_t* needed);
/* Launches step `step` alone `launches` times back to back between one pair of CUDA events on the
 * executor's stream and returns the average duration of one launch in microseconds.  The step reads
 * and rewrites whatever its buffers currently hold.  (The per-step figures of `last_profile` include
 * the event and launch gaps of a one-by-one run; this one does not.)  No reference counterpart. */
KN_API int kn_executor_time_step(kn_executor* exec, int step, int launches, float* microseconds);

/* Tensor-parallel graphs.  No counterpart in the reference, which runs one graph on one device.
 *
 * A graph may contain all-reduce values (operation tag 16 of the blob: one operand, same shape and dtype,
 * f32 or f16): the element-wise sum of the operand over the ranks of a communicator, one rank = one
 * process with its own executor on its own GPU, every rank running a graph with the same sequence of
 * all-reduce values of the same sizes.  The planner turns each into a step of the step list and the
 * executor hands the arena buffers to ncclAllReduce on its own stream, between the kernels before and
 * after it; nothing crosses host memory.  Without a communicator (or with one rank) the step is a
 * device-to-device copy.  With a communicator of several ranks the step list is launched step by step
 * instead of being replayed from a captured CUDA graph.
 *
 * NCCL is bound at run time: the library opens `libnccl.so.2` itself (the copy already loaded into the
 * process if there is one, else `path` of kn_nccl_load, else the dynamic loader's search path).
 * kn_nccl_load is optional and idempotent.
 *
 * Setting up: rank 0 calls kn_comm_unique_id and sends the KN_COMM_ID_BYTES to every rank by any means
 * (a file, a socket, MPI ...); every rank then calls kn_comm_create (collective: it returns once all
 * `world` ranks have called it) and kn_executor_set_comm.  A communicator must outlive the executors
 * that use it; several executors of one device may share one, as long as their evaluations do not
 * overlap. */
#define KN_COMM_ID_BYTES 128
typedef struct kn_comm kn_comm;
KN_API int kn_nccl_load(const char* path);
KN_API int kn_comm_unique_id(void* id, size_t id_bytes);
KN_API int kn_comm_create(int device, int rank, int world, const void* id, size_t id_bytes, kn_comm** out);
KN_API void kn_comm_destroy(kn_comm* comm);
/* Attaches `comm` (may be NULL: back to a world of one) to the executor.  Not while an evaluation is in flight. */
KN_API int kn_executor_set_comm(kn_executor* exec, kn_comm* comm);

/* Self-test of the bounded waits, with no counterpart in the reference.  Every barrier wait inside the
 * tensor-core kernels gives up after a cycle limit, raises the executor's status word and lets the
 * kernel return, and the next synchronising call reports KN_ERR_INTERNAL.  In normal operation no wait
 * expires, so this entry point makes one expire on purpose, harmlessly: a one-thread kernel waits
 * through the same routine, with a limit of `limit_us` microseconds (1 .. 100000), on a barrier in its own
 * shared memory that nothing arrives on.  It holds no tensor memory and has no copies in flight.
 * Returns KN_ERR_INTERNAL (the status path works, message "a kernel gave up waiting ... (code 99)") or
 * KN_OK (the expiry went unreported: a defect).  The status word is cleared and the executor stays usable. */
KN_API int kn_executor_selftest_wait_expiry(kn_executor* exec, uint32_t limit_us);

/* Matrix multiply that allocates nothing.  No counterpart in the reference.
 *
 *     C[m][n] = sum_k A[m][k] * B[n][k]        (A, B, C dense row-major f32 in DEVICE memory)
 *
 * For callers that cannot allocate device memory: a serving loop with a fixed memory footprint, a
 * plugin callback inside a runtime that owns every byte of the device, a context whose pool is
 * already handed out.  It runs a split-K tensor-core matmul (the executor's one-tile kernel and its
 * reduction kernel; TF32 operands rounded to nearest, f32 accumulation) with the per-slice partial
 * sums kept in a fixed array inside the library's device module instead of an allocated buffer; it
 * calls no cudaMalloc / cudaFree and no allocating library routine.  The kernels are enqueued on
 * `stream` (a cudaStream_t, may be NULL for the default stream) of the CURRENT device and the call
 * returns without waiting.
 *
 *  - Limit: slices * m * n * 4 bytes <= KN_STATIC_SCRATCH_BYTES; larger problems are rejected with
 *    KN_ERR_UNSUPPORTED and a message that states the need.  k must be a multiple of 4; A and B
 *    16-byte aligned.  `slices` follows from the shape alone, by this rule (integer arithmetic):
 *        bn       = n > 256 ? 128 : min(256, n rounded up to a multiple of 16)
 *        tiles    = ceil(m / 128) * ceil(n / bn)
 *        k_blocks = ceil(k / 32)
 *        s        = clamp(min(k_blocks / 4, ceil(96 / tiles)), 1, 32)
 *        slices   = ceil(k_blocks / ceil(k_blocks / s))          (no empty slice)
 *    (The executor's planner slices its own matmuls by a different rule; only this one applies here.)
 *  - The array costs KN_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, for
 *    the life of the process.
 *  - The first call on a device looks up the array's device address and opts the kernel in to large
 *    shared memory; make that first call outside any stream capture.
 *  - All calls share the one array (it keeps the previous call's partial sums; every element a call
 *    reads it has written first, so nothing needs clearing).  Two calls whose kernels may overlap on
 *    the GPU (different streams, or different threads) race on it: serialise them. */
#define KN_STATIC_SCRATCH_BYTES (8u << 20)
KN_API int kn_matmul_tf32_static(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                 void* stream);
/* Companion of kn_matmul_tf32_static (no counterpart in the reference either).  Every barrier wait in
 * the kernels is bounded; a CTA whose wait runs out gives up its part of the result and raises a status
 * word that lives next to the scratch array.  kn_matmul_tf32_static itself returns before the kernels
 * run, so it cannot report that: after synchronising the stream, call this to learn whether any call
 * since the last query gave up.  `*code` receives 0 (every result is complete) or the code of the wait
 * that expired (the affected C is then incomplete: run the call again); the word is cleared.  Reads
 * the CURRENT device's word with a 4-byte copy; allocates nothing. */
KN_API int kn_matmul_tf32_static_status(int* code);

/* Host-only: the shape / stride algebra every view-like operation of the planner goes through (the reference's
 * `StridedShape`, kn-cuda-eval/src/shape.rs:11-344), exported so that its rules can be tested as numbers.
 * Strides are in elements and may be zero (broadcast) or negative (flip).
 *   op 0  nothing (flags of the input)          op 3  flip(axis)             args = {axis}
 *   op 1  view(new shape)  args = new shape     op 4  permute(permutation)   args = permutation
 *   op 2  slice(axis, start, end, step)         op 5  broadcast(new shape)   args = new shape
 * The result (at most 16 axes) goes to out_rank / out_shape / out_strides, `*simple` and `*dense` receive
 * the result's has_simple_strides / has_dense_strides flags (shape.rs:34-72).  A view that needs a copy returns
 * KN_ERR_SHAPE (the reference's `ViewError`). */
KN_API int kn_strided_shape(int op, int rank, const int64_t* shape, const int64_t* strides, int n_args, const int64_t* args,
                            int* out_rank, int64_t* out_shape, int64_t* out_strides, int* simple, int* dense);

/* Host-only element semantics, exported so the scalar rules can be tested without a device:
 * applies one unary / binary operation to 64-bit canonical element patterns. */
KN_API int kn_scalar_unary(int unary_op, int from_dtype, int to_dtype, uint64_t x, uint64_t* out);
KN_API int kn_scalar_binary(int binary_op, int dtype, uint64_t a, uint64_t b, uint64_t* out);

#ifdef __cplusplus
}
#endif
#endif /* KN_B200_H */
