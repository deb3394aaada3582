//! `backend::cuda` — sage's device boundary on the B200 library (`libsagecuda.so`, `include/sage_cuda.h`).
//!
//! Replaces the stub at `src/backend/cuda.rs` (a `rustacuda` device list and an nvcc-to-PTX helper).
//! Selected with the existing `cuda` cargo feature (`Cargo.toml:18-19`); `Data::Cuda` (`src/tensor.rs:569-574`)
//! holds a `CudaMemory`, and the `unimplemented!()` arms at `src/tensor.rs:221,291,307` and
//! `src/session/device.rs:261` become the calls below.
//!
//! NOT COMPILED in this repository's build image (no Rust toolchain).  Every call below is
//! exercised with the same argument conventions through ctypes by `tests/test_gpu_abi_ops.py`.

pub mod ffi;

use super::{Backend, BackendError, DataType, MemStats, ReduceKind, TensorView, Window};
use ffi::*;
use std::ffi::{CStr, CString};
use std::os::raw::c_void;
use std::ptr;
use std::rc::Rc;

/// Owns the `sage_ctx`; shared by every `CudaMemory` allocated from it so that a tensor can outlive
/// the `Context` struct the way `Rc<RefCell<Pool>>` lets it today (`src/session/memory.rs:174`).
#[derive(Debug)]
struct CtxHandle(*mut sage_ctx);

impl Drop for CtxHandle {
    fn drop(&mut self) {
        unsafe { sage_ctx_destroy(self.0) };
    }
}

/// Device memory: `Drop` returns the block to the library's pool (stream-ordered), as
/// `Drop for OpenClMemory` does (`src/session/memory.rs:685-692`).
#[derive(Debug)]
pub struct CudaMemory {
    ctx: Rc<CtxHandle>,
    buf: *mut sage_buf,
    bytes: usize,
}

impl CudaMemory {
    pub fn size(&self) -> usize {
        self.bytes
    }
}

impl Drop for CudaMemory {
    fn drop(&mut self) {
        unsafe { sage_free(self.ctx.0, self.buf) };
    }
}

pub struct CudaBackend {
    ctx: Rc<CtxHandle>,
}

fn dtype_code(d: DataType) -> i32 {
    match d {
        DataType::Float => SAGE_F32,
        DataType::Int => SAGE_I32,
        DataType::Uint => SAGE_U32,
    }
}

fn window(w: Window) -> sage_window {
    let p = |v: [usize; 2]| [v[0] as i32, v[1] as i32];
    sage_window { ker: p(w.ker), stride: p(w.stride), pad: p(w.pad), dil: p(w.dil) }
}

/// `Tensor` -> `sage_tensor`: the same extents / strides / offset in elements.
fn desc(t: &TensorView<CudaMemory>) -> sage_tensor {
    let mut d = sage_tensor {
        buf: t.mem.buf,
        dtype: dtype_code(t.dtype),
        ndim: t.extents.len() as i32,
        extents: [0; SAGE_MAX_DIMS],
        strides: [0; SAGE_MAX_DIMS],
        offset: t.offset as i64,
    };
    for (i, (&e, &s)) in t.extents.iter().zip(t.strides.iter()).enumerate() {
        d.extents[i] = e as i64;
        d.strides[i] = s as i64;
    }
    d
}

impl CudaBackend {
    /// Status code -> `Result`; `SAGE_ERR_OOM` carries the sizes `Program::exec` wants for its
    /// evict-and-retry loop (`src/session.rs:259-331`).
    fn check(&self, status: i32) -> Result<(), BackendError> {
        if status == SAGE_OK {
            return Ok(());
        }
        let msg = unsafe { CStr::from_ptr(sage_last_error(self.ctx.0)) }.to_string_lossy().into_owned();
        Err(match status {
            SAGE_ERR_OOM => {
                let (mut needed, mut total) = (0u64, 0u64);
                unsafe { sage_last_oom(self.ctx.0, &mut needed, &mut total) };
                BackendError::OutOfMemory { mem_needed: needed as usize, mem_total: total as usize }
            }
            SAGE_ERR_INVALID | SAGE_ERR_UNSUPPORTED => BackendError::Shape(msg),
            SAGE_ERR_COMPILE => BackendError::Compile(msg),
            _ => BackendError::Device(msg),
        })
    }

    /// `Context::get_program` + `KernelProgram::kernel` + `Kernel::launch` (`src/session/context.rs:62-90`,
    /// `src/session/device.rs:215-318`) for operators that bring their own CUDA C source.
    pub fn launch(&mut self, cuda_src: &str, kernel: &str, grid: [u32; 3], block: [u32; 3], smem: u32, args: &[sage_arg]) -> Result<(), BackendError> {
        let src = CString::new(cuda_src).map_err(|e| BackendError::Compile(e.to_string()))?;
        let name = CString::new(kernel).map_err(|e| BackendError::Compile(e.to_string()))?;
        let mut module = ptr::null_mut();
        self.check(unsafe { sage_module_get(self.ctx.0, src.as_ptr(), &mut module) })?;
        self.check(unsafe { sage_launch(self.ctx.0, module, name.as_ptr(), grid.as_ptr(), block.as_ptr(), smem, args.as_ptr(), args.len() as i32) })
    }

    /// The fused row composites the evaluator may use instead of the reference's 4-7 kernels
    /// (`src/ops/nn.rs:42-100`); `x` and `y` contiguous, `rows * inner` elements.
    pub fn softmax(&mut self, x: &TensorView<CudaMemory>, rows: usize, inner: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_softmax(self.ctx.0, &desc(x), rows as i64, inner as i64, &desc(y)) })
    }
    pub fn log_sum_exp(&mut self, x: &TensorView<CudaMemory>, rows: usize, inner: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_log_sum_exp(self.ctx.0, &desc(x), rows as i64, inner as i64, &desc(y)) })
    }
    #[allow(clippy::too_many_arguments)]
    pub fn layer_norm(&mut self, x: &TensorView<CudaMemory>, rows: usize, inner: usize, gamma: &TensorView<CudaMemory>,
                      beta: &TensorView<CudaMemory>, eps: f32, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_layer_norm(self.ctx.0, &desc(x), rows as i64, inner as i64, &desc(gamma), &desc(beta), eps, &desc(y)) })
    }
    /// `max_pool_2d` / `avg_pool_2d` (`src/ops/conv.rs:143-165`) without the column tensor.
    pub fn pool2d(&mut self, is_max: bool, x: &TensorView<CudaMemory>, w: Window, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_pool2d(self.ctx.0, is_max as i32, &desc(x), &window(w), &desc(y)) })
    }
    /// `conv_2d` (`src/ops/conv.rs:61-96`) as an implicit GEMM on the tensor cores.
    pub fn conv2d(&mut self, x: &TensorView<CudaMemory>, filter: &TensorView<CudaMemory>, w: Window, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_conv2d_nhwc(self.ctx.0, &desc(x), &desc(filter), &window(w), &desc(y)) })
    }
    /// Device-side status word: kernels with bounded waits set bits here instead of trapping.
    pub fn status_word(&mut self) -> Result<u32, BackendError> {
        let mut w = 0u32;
        self.check(unsafe { sage_status_word(self.ctx.0, &mut w) })?;
        Ok(w)
    }
}

impl Backend for CudaBackend {
    type Memory = CudaMemory;

    fn device_list() -> Vec<String> {
        let mut n = 0i32;
        unsafe { sage_device_count(&mut n) };
        (0..n)
            .map(|i| {
                let mut name = [0 as std::os::raw::c_char; 256];
                unsafe { sage_device_name(i, name.as_mut_ptr(), name.len()) };
                unsafe { CStr::from_ptr(name.as_ptr()) }.to_string_lossy().into_owned()
            })
            .collect()
    }

    fn with_device(idx: usize) -> Result<Self, BackendError> {
        let mut opts = sage_ctx_opts { mem_capacity_bytes: 0, use_cache: 1, ref_compat: 1, pattern_fusion: 1, gemm_backend: 0 };
        unsafe { sage_ctx_opts_default(&mut opts) };
        let mut ctx = ptr::null_mut();
        let status = unsafe { sage_ctx_create(idx as i32, &opts, &mut ctx) };
        if status != SAGE_OK {
            return Err(BackendError::Device(format!("sage_ctx_create({idx}) failed with status {status}")));
        }
        Ok(CudaBackend { ctx: Rc::new(CtxHandle(ctx)) })
    }

    fn alloc(&mut self, _dtype: DataType, size: usize) -> Result<CudaMemory, BackendError> {
        let bytes = size * 4; // every element type is 4 bytes wide (device.rs:73-81)
        let mut buf = ptr::null_mut();
        self.check(unsafe { sage_alloc(self.ctx.0, bytes, &mut buf) })?;
        Ok(CudaMemory { ctx: self.ctx.clone(), buf, bytes })
    }

    fn mem_stats(&self) -> MemStats {
        let mut s = sage_mem_stats_t::default();
        unsafe { sage_mem_stats(self.ctx.0, &mut s) };
        MemStats { capacity: s.capacity as usize, mem_total: s.mem_total as usize, mem_used: s.mem_used as usize, mem_peak: s.mem_peak as usize }
    }

    fn write(&mut self, dst: &CudaMemory, host: &[u8]) -> Result<(), BackendError> {
        self.check(unsafe { sage_upload(self.ctx.0, dst.buf, 0, host.as_ptr() as *const c_void, host.len()) })
    }
    fn read(&mut self, src: &CudaMemory, host: &mut [u8]) -> Result<(), BackendError> {
        self.check(unsafe { sage_download(self.ctx.0, src.buf, 0, host.as_mut_ptr() as *mut c_void, host.len()) })
    }
    fn fill_zero(&mut self, dst: &CudaMemory) -> Result<(), BackendError> {
        self.check(unsafe { sage_memset(self.ctx.0, dst.buf, 0, 0, dst.bytes) })
    }

    fn map(&mut self, expr: &str, x: &[TensorView<CudaMemory>], y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        let e = CString::new(expr).map_err(|e| BackendError::Compile(e.to_string()))?;
        let xs: Vec<sage_tensor> = x.iter().map(desc).collect();
        self.check(unsafe { sage_map(self.ctx.0, e.as_ptr(), xs.as_ptr(), xs.len() as i32, &desc(y)) })
    }
    fn reduce(&mut self, kind: ReduceKind, x: &TensorView<CudaMemory>, axes: &[usize], y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        let k = match kind {
            ReduceKind::Sum => 0,
            ReduceKind::Prod => 1,
            ReduceKind::Max => 2,
            ReduceKind::Min => 3,
        };
        let ax: Vec<i32> = axes.iter().map(|&a| a as i32).collect();
        self.check(unsafe { sage_reduce(self.ctx.0, k, &desc(x), ax.as_ptr(), ax.len() as i32, &desc(y)) })
    }
    fn reduce_arg(&mut self, is_max: bool, x: &TensorView<CudaMemory>, axis: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_reduce_arg(self.ctx.0, is_max as i32, &desc(x), axis as i32, &desc(y)) })
    }
    fn gather(&mut self, x: &TensorView<CudaMemory>, ind: &TensorView<CudaMemory>, axis: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_gather(self.ctx.0, &desc(x), &desc(ind), axis as i32, &desc(y)) })
    }
    fn scatter(&mut self, x: &TensorView<CudaMemory>, ind: &TensorView<CudaMemory>, axis: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_scatter(self.ctx.0, &desc(x), &desc(ind), axis as i32, &desc(y)) })
    }
    fn unslice(&mut self, x: &TensorView<CudaMemory>, axis: usize, start: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_unslice(self.ctx.0, &desc(x), axis as i32, start as i64, &desc(y)) })
    }
    fn concat(&mut self, xs: &[TensorView<CudaMemory>], axis: usize, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        let d: Vec<sage_tensor> = xs.iter().map(desc).collect();
        self.check(unsafe { sage_concat(self.ctx.0, d.as_ptr(), d.len() as i32, axis as i32, &desc(y)) })
    }
    fn gemm_batched(&mut self, trans_a: bool, trans_b: bool, m: usize, n: usize, k: usize, batch: usize,
                    a: &TensorView<CudaMemory>, lda: usize, stride_a: usize,
                    b: &TensorView<CudaMemory>, ldb: usize, stride_b: usize,
                    c: &TensorView<CudaMemory>, ldc: usize, stride_c: usize) -> Result<(), BackendError> {
        self.check(unsafe {
            sage_gemm_strided_batched(self.ctx.0, trans_a as i32, trans_b as i32, m as i64, n as i64, k as i64,
                                      a.mem.buf, a.offset as i64, lda as i64, stride_a as i64,
                                      b.mem.buf, b.offset as i64, ldb as i64, stride_b as i64,
                                      c.mem.buf, c.offset as i64, ldc as i64, stride_c as i64, batch as i64)
        })
    }
    fn im2col(&mut self, x: &TensorView<CudaMemory>, w: Window, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_im2col(self.ctx.0, &desc(x), &window(w), &desc(y)) })
    }
    fn col2im(&mut self, x: &TensorView<CudaMemory>, w: Window, y: &TensorView<CudaMemory>) -> Result<(), BackendError> {
        self.check(unsafe { sage_col2im(self.ctx.0, &desc(x), &window(w), &desc(y)) })
    }
    fn sync(&mut self) -> Result<(), BackendError> {
        self.check(unsafe { sage_sync(self.ctx.0) })
    }
}
