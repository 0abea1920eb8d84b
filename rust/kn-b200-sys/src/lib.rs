//! Raw bindings to `libkn_b200.so`: one declaration per function of `include/kn_b200.h`, in the header's
//! order, with the header's names.  See the header for what each function replaces in the reference.
//!
//! Uncompiled source: the image this repository is built in has no Rust toolchain.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_void};

pub const KN_OK: c_int = 0;
pub const KN_ERR_INVALID_ARG: c_int = 1;
pub const KN_ERR_BAD_GRAPH: c_int = 2;
pub const KN_ERR_UNSUPPORTED: c_int = 3;
pub const KN_ERR_CUDA: c_int = 4;
pub const KN_ERR_SHAPE: c_int = 5;
pub const KN_ERR_NO_DEVICE: c_int = 6;
pub const KN_ERR_INTERNAL: c_int = 7;

pub const KN_MATH_TF32: i32 = 0;
pub const KN_MATH_F32: i32 = 1;

pub const KN_FLAG_NO_CONV_CHAIN: i32 = 1;
pub const KN_FLAG_NO_PERSISTENT_GEMM: i32 = 2;
pub const KN_FLAG_TRACE_GEMM: i32 = 4;

pub const KN_MAX_RANK: usize = 8;
pub const KN_COMM_ID_BYTES: usize = 128;
pub const KN_STATIC_SCRATCH_BYTES: usize = 8 << 20;

#[repr(C)]
#[derive(Debug, Copy, Clone)]
pub struct kn_options {
    pub struct_size: u32,
    pub math_mode: i32,
    pub use_cuda_graph: i32,
    pub flags: i32,
}

#[repr(C)]
#[derive(Debug, Copy, Clone)]
pub struct kn_tensor_info {
    pub dtype: i32,
    pub rank: i32,
    pub dims: [i64; KN_MAX_RANK],
    pub bytes: u64,
}

#[repr(C)]
#[derive(Debug, Copy, Clone, Default)]
pub struct kn_mem_usage {
    pub dedicated_bytes: u64,
    pub shared_bytes: u64,
    pub zero_bytes: u64,
    pub hypo_peak_bytes: u64,
    pub hypo_total_bytes: u64,
}

#[repr(C)]
pub struct kn_graph {
    _private: [u8; 0],
}
#[repr(C)]
pub struct kn_executor {
    _private: [u8; 0],
}
#[repr(C)]
pub struct kn_comm {
    _private: [u8; 0],
}

extern "C" {
    pub fn kn_last_error() -> *const c_char;
    pub fn kn_version() -> c_int;
    pub fn kn_options_default(opts: *mut kn_options) -> c_int;
    pub fn kn_device_count(count: *mut c_int) -> c_int;

    pub fn kn_graph_from_blob(bytes: *const c_void, len: usize, out: *mut *mut kn_graph) -> c_int;
    pub fn kn_graph_destroy(graph: *mut kn_graph);
    pub fn kn_graph_io_count(graph: *const kn_graph, n_inputs: *mut c_int, n_outputs: *mut c_int, n_values: *mut c_int) -> c_int;
    pub fn kn_plan_describe(graph: *const kn_graph, batch_size: usize, opts: *const kn_options, buf: *mut c_char, cap: usize,
                            needed: *mut usize) -> c_int;

    pub fn kn_executor_create(device: c_int, graph: *const kn_graph, batch_size: usize, opts: *const kn_options,
                              out: *mut *mut kn_executor) -> c_int;
    pub fn kn_executor_destroy(exec: *mut kn_executor);
    pub fn kn_executor_io_count(exec: *const kn_executor, n_inputs: *mut c_int, n_outputs: *mut c_int) -> c_int;
    pub fn kn_executor_io_info(exec: *const kn_executor, is_output: c_int, index: c_int, info: *mut kn_tensor_info) -> c_int;

    pub fn kn_executor_evaluate(exec: *mut kn_executor, inputs: *const *const c_void, outputs: *const *mut c_void) -> c_int;
    pub fn kn_executor_evaluate_begin(exec: *mut kn_executor, inputs: *const *const c_void) -> c_int;
    pub fn kn_executor_evaluate_end(exec: *mut kn_executor, outputs: *const *mut c_void) -> c_int;
    pub fn kn_executor_run_async(exec: *mut kn_executor) -> c_int;
    pub fn kn_executor_synchronize(exec: *mut kn_executor) -> c_int;
    pub fn kn_executor_stream(exec: *mut kn_executor, stream: *mut *mut c_void) -> c_int;

    pub fn kn_executor_host_buffer(exec: *mut kn_executor, is_output: c_int, index: c_int, ptr: *mut *mut c_void, bytes: *mut u64) -> c_int;
    pub fn kn_executor_device_buffer(exec: *mut kn_executor, is_output: c_int, index: c_int, ptr: *mut *mut c_void, bytes: *mut u64) -> c_int;
    pub fn kn_executor_upload_inputs(exec: *mut kn_executor) -> c_int;
    pub fn kn_executor_download_outputs(exec: *mut kn_executor) -> c_int;

    pub fn kn_executor_mem_usage(exec: *const kn_executor, usage: *mut kn_mem_usage) -> c_int;
    pub fn kn_executor_step_count(exec: *const kn_executor, steps: *mut c_int, launches: *mut c_int) -> c_int;

    pub fn kn_executor_set_profile(exec: *mut kn_executor, enable: c_int) -> c_int;
    pub fn kn_executor_last_profile(exec: *mut kn_executor, buf: *mut c_char, cap: usize, needed: *mut usize) -> c_int;
    pub fn kn_executor_time_step(exec: *mut kn_executor, step: c_int, launches: c_int, microseconds: *mut f32) -> c_int;

    pub fn kn_nccl_load(path: *const c_char) -> c_int;
    pub fn kn_comm_unique_id(id: *mut c_void, id_bytes: usize) -> c_int;
    pub fn kn_comm_create(device: c_int, rank: c_int, world: c_int, id: *const c_void, id_bytes: usize, out: *mut *mut kn_comm) -> c_int;
    pub fn kn_comm_destroy(comm: *mut kn_comm);
    pub fn kn_executor_set_comm(exec: *mut kn_executor, comm: *mut kn_comm) -> c_int;

    pub fn kn_executor_selftest_wait_expiry(exec: *mut kn_executor, limit_us: u32) -> c_int;

    pub fn kn_matmul_tf32_static(a: *const f32, b: *const f32, c: *mut f32, m: i64, n: i64, k: i64, stream: *mut c_void) -> c_int;
    pub fn kn_matmul_tf32_static_status(code: *mut c_int) -> c_int;

    pub fn kn_strided_shape(op: c_int, rank: c_int, shape: *const i64, strides: *const i64, n_args: c_int, args: *const i64,
                            out_rank: *mut c_int, out_shape: *mut i64, out_strides: *mut i64, simple: *mut c_int, dense: *mut c_int) -> c_int;

    pub fn kn_scalar_unary(unary_op: c_int, from_dtype: c_int, to_dtype: c_int, x: u64, out: *mut u64) -> c_int;
    pub fn kn_scalar_binary(binary_op: c_int, dtype: c_int, a: u64, b: u64, out: *mut u64) -> c_int;
}
