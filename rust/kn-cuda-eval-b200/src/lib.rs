//! `kn-cuda-eval`'s public executor API on `libkn_b200.so`: same type and method names, same argument meaning
//! and the same panics on misuse as the reference (kn-cuda-eval/src/executor.rs, kn-cuda-sys/src/wrapper/handle.rs),
//! so that `kn-runtime`'s `Device::Cuda` / `PreparedGraph::Cuda` (kn-runtime/src/lib.rs:68-126) and every other
//! caller compile against it unchanged.
//!
//! Uncompiled source: the image this repository is built in has no Rust toolchain.

pub mod serialize;

use std::ffi::{c_void, CStr};
use std::os::raw::c_int;
use std::ptr::{null, null_mut};

use kn_b200_sys as sys;
use kn_graph::dtype::{DBool, DTensor, DType, Tensor};
use kn_graph::graph::Graph;

pub use serialize::serialize_graph;

fn last_error() -> String {
    unsafe { CStr::from_ptr(sys::kn_last_error()).to_string_lossy().into_owned() }
}

/// The reference panics on any CUDA or planning failure (kn-cuda-sys/src/wrapper/status.rs:17-32); so does this.
#[track_caller]
fn check(status: c_int) {
    if status != sys::KN_OK {
        panic!("kn_b200 error {}: {}", status, last_error());
    }
}

// ------------------------------------------------------------------------------------------------
// CudaDevice (kn-cuda-sys/src/wrapper/handle.rs:27-70)
// ------------------------------------------------------------------------------------------------
#[derive(Debug, Copy, Clone, Eq, PartialEq, Hash)]
pub struct CudaDevice(i32);

#[derive(Debug)]
pub struct CudaDeviceNotAvailable;

pub fn cuda_device_count() -> i32 {
    let mut n: c_int = 0;
    check(unsafe { sys::kn_device_count(&mut n) });
    n
}

impl CudaDevice {
    pub fn new(device: i32) -> Result<Self, CudaDeviceNotAvailable> {
        if 0 <= device && device < cuda_device_count() {
            Ok(CudaDevice(device))
        } else {
            Err(CudaDeviceNotAvailable)
        }
    }

    pub fn all() -> impl Iterator<Item = Self> {
        (0..cuda_device_count()).map(CudaDevice)
    }

    pub fn inner(self) -> i32 {
        self.0
    }
}

/// The stream the steps run on, as the raw `cudaStream_t` (the reference hands out its own `CudaStream`
/// wrapper, kn-cuda-eval/src/executor.rs:263-265).
#[derive(Debug, Copy, Clone)]
pub struct CudaStream(pub *mut c_void);

impl CudaStream {
    pub fn inner(&self) -> *mut c_void {
        self.0
    }
}

// ------------------------------------------------------------------------------------------------
// MemoryUsage, Profile (kn-cuda-eval/src/planner.rs:67-81, executor.rs:43-58)
// ------------------------------------------------------------------------------------------------
#[derive(Debug, Copy, Clone)]
pub struct MemoryUsage {
    pub dedicated_bytes: usize,
    pub shared_bytes: usize,
    pub zero_bytes: usize,
    pub hypo_shared_bytes_peak: usize,
    pub hypo_shared_bytes_total: usize,
}

#[derive(Default, Debug, Clone)]
pub struct Profile {
    /// One line per step: `index kind microseconds algorithmic_bytes flops description`.
    pub steps: Vec<String>,

    pub conv: f32,
    pub mat_mul: f32,
    pub scalar_op: f32,
    pub reduce_op: f32,
    pub softmax_op: f32,
    pub layernorm_op: f32,
    pub gather_op: f32,

    pub total_cpu: f32,
    pub total_gpu: f32,
    pub timing_overhead: f32,
}

/// Shape and dtype of a device-side input or output (what callers read from the reference's
/// `device_inputs` / `device_outputs`, executor.rs:27-28) together with its device address.
#[derive(Debug, Clone)]
pub struct DeviceTensorInfo {
    pub shape: Vec<usize>,
    pub dtype: DType,
    pub ptr: *mut c_void,
    pub bytes: usize,
}

// ------------------------------------------------------------------------------------------------
// CudaExecutor (kn-cuda-eval/src/executor.rs:20-37)
// ------------------------------------------------------------------------------------------------
pub struct CudaExecutor {
    raw: *mut sys::kn_executor,
    stream: CudaStream,

    pub device_inputs: Vec<DeviceTensorInfo>,
    pub device_outputs: Vec<DeviceTensorInfo>,

    pub batch_size: usize,
    pub mem_usage: MemoryUsage,

    profile: bool,
    last_profile: Option<Profile>,

    tensor_outputs: Vec<DTensor>,
}

// The library allows an executor to move between threads as long as one thread uses it at a time
// (include/kn_b200.h, conventions); the reference makes the same claim (executor.rs:39-41).
unsafe impl Send for CudaExecutor {}

fn zeros(dtype: DType, shape: &[usize]) -> DTensor {
    match dtype {
        DType::F32 => DTensor::F32(Tensor::zeros(shape)),
        DType::F64 => DTensor::F64(Tensor::zeros(shape)),
        DType::I8 => DTensor::I8(Tensor::zeros(shape)),
        DType::I16 => DTensor::I16(Tensor::zeros(shape)),
        DType::I32 => DTensor::I32(Tensor::zeros(shape)),
        DType::I64 => DTensor::I64(Tensor::zeros(shape)),
        DType::U8 => DTensor::U8(Tensor::zeros(shape)),
        DType::U16 => DTensor::U16(Tensor::zeros(shape)),
        DType::U32 => DTensor::U32(Tensor::zeros(shape)),
        DType::U64 => DTensor::U64(Tensor::zeros(shape)),
        DType::Bool => DTensor::Bool(Tensor::from_elem(shape, DBool(false))),
    }
}

/// Pointer to the first element of a tensor in standard layout and its length in bytes.
fn host_bytes_mut(t: &mut DTensor) -> (*mut c_void, usize) {
    macro_rules! raw {
        ($inner:expr, $size:expr) => {{
            let n = $inner.len() * $size;
            ($inner.as_slice_mut().expect("output tensors are in standard layout").as_mut_ptr() as *mut c_void, n)
        }};
    }
    match t {
        DTensor::F32(x) => raw!(x, 4),
        DTensor::F64(x) => raw!(x, 8),
        DTensor::I8(x) => raw!(x, 1),
        DTensor::I16(x) => raw!(x, 2),
        DTensor::I32(x) => raw!(x, 4),
        DTensor::I64(x) => raw!(x, 8),
        DTensor::U8(x) => raw!(x, 1),
        DTensor::U16(x) => raw!(x, 2),
        DTensor::U32(x) => raw!(x, 4),
        DTensor::U64(x) => raw!(x, 8),
        DTensor::Bool(x) => raw!(x, 1),   // DBool is repr(transparent) over bool; the library writes only 0 / 1
    }
}

impl CudaExecutor {
    /// `CudaExecutor::new(device, &graph, batch_size)` (executor.rs:61-110): plans the graph, allocates device
    /// memory, uploads the constants.
    pub fn new(device: CudaDevice, graph: &Graph, batch_size: usize) -> Self {
        Self::with_options(device, graph, batch_size, None)
    }

    /// `options`: `None` for the defaults (TF32 tensor-core contractions, captured CUDA graph).
    pub fn with_options(device: CudaDevice, graph: &Graph, batch_size: usize, options: Option<sys::kn_options>) -> Self {
        let blob = serialize_graph(graph);
        let mut raw_graph: *mut sys::kn_graph = null_mut();
        check(unsafe { sys::kn_graph_from_blob(blob.as_ptr() as *const c_void, blob.len(), &mut raw_graph) });
        drop(blob);   // the library keeps its own copy

        let mut raw: *mut sys::kn_executor = null_mut();
        let opts_ptr = options.as_ref().map_or(null(), |o| o as *const sys::kn_options);
        let status = unsafe { sys::kn_executor_create(device.inner(), raw_graph, batch_size, opts_ptr, &mut raw) };
        unsafe { sys::kn_graph_destroy(raw_graph) };
        check(status);

        let (mut n_in, mut n_out): (c_int, c_int) = (0, 0);
        check(unsafe { sys::kn_executor_io_count(raw, &mut n_in, &mut n_out) });
        let io = |is_output: c_int, index: c_int| -> DeviceTensorInfo {
            let mut info = sys::kn_tensor_info { dtype: 0, rank: 0, dims: [0; sys::KN_MAX_RANK], bytes: 0 };
            check(unsafe { sys::kn_executor_io_info(raw, is_output, index, &mut info) });
            let mut ptr: *mut c_void = null_mut();
            let mut bytes: u64 = 0;
            check(unsafe { sys::kn_executor_device_buffer(raw, is_output, index, &mut ptr, &mut bytes) });
            DeviceTensorInfo {
                shape: info.dims[..info.rank as usize].iter().map(|&d| d as usize).collect(),
                dtype: serialize::dtype_from_tag(info.dtype),
                ptr,
                bytes: bytes as usize,
            }
        };
        let device_inputs: Vec<_> = (0..n_in).map(|i| io(0, i)).collect();
        let device_outputs: Vec<_> = (0..n_out).map(|i| io(1, i)).collect();
        let tensor_outputs = device_outputs.iter().map(|t| zeros(t.dtype, &t.shape)).collect();

        let mut usage = sys::kn_mem_usage::default();
        check(unsafe { sys::kn_executor_mem_usage(raw, &mut usage) });
        let mut stream: *mut c_void = null_mut();
        check(unsafe { sys::kn_executor_stream(raw, &mut stream) });

        CudaExecutor {
            raw,
            stream: CudaStream(stream),
            device_inputs,
            device_outputs,
            batch_size,
            mem_usage: MemoryUsage {
                dedicated_bytes: usage.dedicated_bytes as usize,
                shared_bytes: usage.shared_bytes as usize,
                zero_bytes: usage.zero_bytes as usize,
                hypo_shared_bytes_peak: usage.hypo_peak_bytes as usize,
                hypo_shared_bytes_total: usage.hypo_total_bytes as usize,
            },
            profile: false,
            last_profile: None,
            tensor_outputs,
        }
    }

    pub fn stream(&self) -> &CudaStream {
        &self.stream
    }

    /// `evaluate(&inputs) -> &[DTensor]` (executor.rs:117-195): copies the inputs to the device, runs every step,
    /// copies the outputs back and waits.  Panics on a wrong input count, shape or dtype like the reference.
    pub fn evaluate(&mut self, inputs: &[DTensor]) -> &[DTensor] {
        assert_eq!(inputs.len(), self.device_inputs.len(), "Wrong input count");
        for (i, (input, tensor)) in inputs.iter().zip(&self.device_inputs).enumerate() {
            assert_eq!(input.shape(), &tensor.shape[..], "Wrong shape for input {}", i);
            assert_eq!(input.dtype(), tensor.dtype, "Wrong dtype for input {}", i);
        }

        // inputs in standard layout (executor.rs:135), kept alive until the call has returned
        let standard: Vec<DTensor> = inputs.iter().map(standard_layout).collect();
        let in_ptrs: Vec<*const c_void> = standard.iter().map(host_ptr).collect();
        let mut out_ptrs: Vec<*mut c_void> = Vec::with_capacity(self.tensor_outputs.len());
        for t in &mut self.tensor_outputs {
            out_ptrs.push(host_bytes_mut(t).0);
        }
        check(unsafe { sys::kn_executor_evaluate(self.raw, in_ptrs.as_ptr(), out_ptrs.as_ptr()) });
        if self.profile {
            self.last_profile = Some(self.read_profile());
        }
        &self.tensor_outputs
    }

    /// `run_async` (executor.rs:199-258): enqueues the steps on the executor's stream; the inputs are whatever the
    /// device input buffers hold.  Unsafe for the reference's reason: nothing waits for the device.
    pub unsafe fn run_async(&mut self) {
        check(sys::kn_executor_run_async(self.raw));
        if self.profile {
            self.last_profile = Some(self.read_profile());
        }
    }

    pub fn synchronize(&mut self) {
        check(unsafe { sys::kn_executor_synchronize(self.raw) });
    }

    pub fn set_profile(&mut self, profile: bool) {
        self.profile = profile;
        check(unsafe { sys::kn_executor_set_profile(self.raw, profile as c_int) });
    }

    pub fn last_profile(&self) -> Option<&Profile> {
        self.last_profile.as_ref()
    }

    fn read_profile(&mut self) -> Profile {
        let mut needed: usize = 0;
        check(unsafe { sys::kn_executor_last_profile(self.raw, null_mut(), 0, &mut needed) });
        let mut buf = vec![0u8; needed + 1];
        check(unsafe { sys::kn_executor_last_profile(self.raw, buf.as_mut_ptr() as *mut _, buf.len(), &mut needed) });
        let text = String::from_utf8_lossy(&buf[..needed]).into_owned();

        let mut profile = Profile::default();
        for line in text.lines() {
            let parts: Vec<&str> = line.split_whitespace().collect();
            if parts.len() == 3 && parts[0] == "total" {
                // the reference reports seconds (executor.rs:291-325); the library reports microseconds
                let seconds = parts[2].parse::<f32>().unwrap_or(0.0) * 1e-6;
                match parts[1] {
                    "Conv" | "ConvChain" | "Im2col" => profile.conv += seconds,
                    "Gemm" => profile.mat_mul += seconds,
                    "Scalar" => profile.scalar_op += seconds,
                    "Reduce" => profile.reduce_op += seconds,
                    "Softmax" => profile.softmax_op += seconds,
                    "Layernorm" => profile.layernorm_op += seconds,
                    "Gather" => profile.gather_op += seconds,
                    _ => {}
                }
            } else if parts.first().map_or(false, |p| p.chars().all(|c| c.is_ascii_digit())) {
                profile.steps.push(line.to_owned());
            }
        }
        profile.total_gpu = profile.conv + profile.mat_mul + profile.scalar_op + profile.reduce_op + profile.softmax_op
            + profile.layernorm_op + profile.gather_op;
        profile
    }
}

fn standard_layout(t: &DTensor) -> DTensor {
    match t {
        DTensor::F32(x) => DTensor::F32(x.as_standard_layout().to_shared()),
        DTensor::F64(x) => DTensor::F64(x.as_standard_layout().to_shared()),
        DTensor::I8(x) => DTensor::I8(x.as_standard_layout().to_shared()),
        DTensor::I16(x) => DTensor::I16(x.as_standard_layout().to_shared()),
        DTensor::I32(x) => DTensor::I32(x.as_standard_layout().to_shared()),
        DTensor::I64(x) => DTensor::I64(x.as_standard_layout().to_shared()),
        DTensor::U8(x) => DTensor::U8(x.as_standard_layout().to_shared()),
        DTensor::U16(x) => DTensor::U16(x.as_standard_layout().to_shared()),
        DTensor::U32(x) => DTensor::U32(x.as_standard_layout().to_shared()),
        DTensor::U64(x) => DTensor::U64(x.as_standard_layout().to_shared()),
        DTensor::Bool(x) => DTensor::Bool(x.as_standard_layout().to_shared()),
    }
}

fn host_ptr(t: &DTensor) -> *const c_void {
    match t {
        DTensor::F32(x) => x.as_ptr() as *const c_void,
        DTensor::F64(x) => x.as_ptr() as *const c_void,
        DTensor::I8(x) => x.as_ptr() as *const c_void,
        DTensor::I16(x) => x.as_ptr() as *const c_void,
        DTensor::I32(x) => x.as_ptr() as *const c_void,
        DTensor::I64(x) => x.as_ptr() as *const c_void,
        DTensor::U8(x) => x.as_ptr() as *const c_void,
        DTensor::U16(x) => x.as_ptr() as *const c_void,
        DTensor::U32(x) => x.as_ptr() as *const c_void,
        DTensor::U64(x) => x.as_ptr() as *const c_void,
        DTensor::Bool(x) => x.as_ptr() as *const c_void,
    }
}

impl Drop for CudaExecutor {
    fn drop(&mut self) {
        unsafe { sys::kn_executor_destroy(self.raw) };
    }
}

impl std::fmt::Debug for CudaExecutor {
    /// The step list and memory plan, like the reference's `Debug` (executor.rs:269-289).
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        f.debug_struct("CudaExecutor")
            .field("batch_size", &self.batch_size)
            .field("mem_usage", &self.mem_usage)
            .field("device_inputs", &self.device_inputs)
            .field("device_outputs", &self.device_outputs)
            .field("profile", &self.profile)
            .finish()
    }
}
