//! The device boundary of sage as a trait.
//!
//! sage today has no such trait: `src/backend.rs` is three `mod` lines and every operator's
//! `compute()` calls the concrete OpenCL types of `src/session/device.rs` / `memory.rs` directly
//! (`Context::alloc`, `Buffer::{read, write, fill}`, `KernelProgram::kernel`, `Kernel::launch`).
//! This file names those calls once, so that `backend::opencl` (the existing code) and
//! `backend::cuda` (this crate: the B200 library behind `include/sage_cuda.h`) can both stand
//! behind `Context`.  Nothing above `src/session` changes: `Var`, `grad()`, `Operator::fuse`,
//! `Program::compile/exec`, `layers::*` and `models::*` keep building and scheduling the graph.
//!
//! NOT COMPILED in the build image of this repository (no Rust toolchain there); the Python test
//! `tests/test_gpu_abi_ops.py` exercises the same entry points with the same argument
//! conventions through ctypes, and `tests/test_rust_binding.py` checks this crate's `extern "C"`
//! block against the header.

pub mod cuda;

use std::fmt::Debug;

/// Element types sage can store: all 4 bytes (`src/session/device.rs:73-81`, `src/tensor/data.rs:13-30`).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum DataType {
    Float,
    Int,
    Uint,
}

/// `Error` of `src/error.rs:5-13`; only `Memory` is recoverable (`Program::exec`, `src/session.rs:259-331`).
#[derive(Debug)]
pub enum BackendError {
    /// `MemoryError::OutOfMemory { mem_needed, mem_total }` — `src/session/memory.rs:45-54`
    OutOfMemory { mem_needed: usize, mem_total: usize },
    Device(String),
    Shape(String),
    Compile(String),
}

/// A strided view of device memory: the reference's `Tensor` = buffer + `Shape{extents, strides, offset}`
/// (`src/tensor.rs:106-110`, `src/shape.rs:37-43`), offsets and strides in elements, stride 0 = broadcast.
pub struct TensorView<'a, M> {
    pub mem: &'a M,
    pub dtype: DataType,
    pub extents: &'a [usize],
    pub strides: &'a [usize],
    pub offset: usize,
}

/// Window parameters of `im2col` / `col2im` / pooling; every pair is `[w, h]` like `SizedExtent<2>`
/// (`src/ops/conv.rs:83,205-209`).
#[derive(Clone, Copy, Debug)]
pub struct Window {
    pub ker: [usize; 2],
    pub stride: [usize; 2],
    pub pad: [usize; 2],
    pub dil: [usize; 2],
}

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum ReduceKind {
    Sum,
    Prod,
    Max,
    Min,
}

/// Counters of `Allocator::{capacity, mem_total, mem_peak, mem_used}` (`src/session/memory.rs:184-198`).
#[derive(Clone, Copy, Debug, Default)]
pub struct MemStats {
    pub capacity: usize,
    pub mem_total: usize,
    pub mem_used: usize,
    pub mem_peak: usize,
}

/// One device + one in-order queue + one allocator, single-threaded like `Context`
/// (`Rc<RefCell<Pool>>`, `src/session/memory.rs:174`).  One method per row of the boundary.
pub trait Backend: Sized {
    /// Device memory handle; dropping it returns the block to the pool (`Drop for OpenClMemory`,
    /// `src/session/memory.rs:685-692`).
    type Memory: Debug;

    // ---- Device::get_list / get_first_gpu — src/session/device.rs:26-43
    fn device_list() -> Vec<String>;
    // ---- Context::with_device — src/session/context.rs:43-52
    fn with_device(idx: usize) -> Result<Self, BackendError>;

    // ---- Context::alloc -> Allocator::alloc -> Device::alloc_buffer — context.rs:119-137, memory.rs:200-208
    fn alloc(&mut self, dtype: DataType, size: usize) -> Result<Self::Memory, BackendError>;
    fn mem_stats(&self) -> MemStats;
    // ---- Buffer::write / read / fill — device.rs:111-164
    fn write(&mut self, dst: &Self::Memory, host: &[u8]) -> Result<(), BackendError>;
    fn read(&mut self, src: &Self::Memory, host: &mut [u8]) -> Result<(), BackendError>;
    fn fill_zero(&mut self, dst: &Self::Memory) -> Result<(), BackendError>;

    // ---- {Nullary,Unary,Binary,Ternary,Variadic}MapOperator::compute — src/ops/map.rs:898-1175.
    // `expr` is what map_fn() returns: a C expression over x0..x{n-1}.
    fn map(&mut self, expr: &str, x: &[TensorView<Self::Memory>], y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    // ---- ReduceOperator::compute / ReduceArgOperator::compute — src/ops/reduce.rs:258-325, 372-431
    fn reduce(&mut self, kind: ReduceKind, x: &TensorView<Self::Memory>, axes: &[usize], y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    fn reduce_arg(&mut self, is_max: bool, x: &TensorView<Self::Memory>, axis: usize, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    // ---- Gather / Scatter / Unslice / Concat ::compute — src/ops/core.rs:571-934
    fn gather(&mut self, x: &TensorView<Self::Memory>, ind: &TensorView<Self::Memory>, axis: usize, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    fn scatter(&mut self, x: &TensorView<Self::Memory>, ind: &TensorView<Self::Memory>, axis: usize, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    fn unslice(&mut self, x: &TensorView<Self::Memory>, axis: usize, start: usize, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    fn concat(&mut self, xs: &[TensorView<Self::Memory>], axis: usize, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    // ---- Gemm::compute_direct / GemmBatched::compute_direct — src/ops/gemm.rs:176-250, 338-421.
    // Row-major C[batch][M, N] = op(A) op(B); leading dimensions and batch strides in elements.
    #[allow(clippy::too_many_arguments)]
    fn gemm_batched(&mut self, trans_a: bool, trans_b: bool, m: usize, n: usize, k: usize, batch: usize,
                    a: &TensorView<Self::Memory>, lda: usize, stride_a: usize,
                    b: &TensorView<Self::Memory>, ldb: usize, stride_b: usize,
                    c: &TensorView<Self::Memory>, ldc: usize, stride_c: usize) -> Result<(), BackendError>;
    // ---- Im2col::compute / Col2im::compute — src/ops/conv.rs:289-374, 404-498
    fn im2col(&mut self, x: &TensorView<Self::Memory>, w: Window, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;
    fn col2im(&mut self, x: &TensorView<Self::Memory>, w: Window, y: &TensorView<Self::Memory>) -> Result<(), BackendError>;

    /// Blocks until everything enqueued so far has run (the reference's only synchronisation point
    /// is `Buffer::read`, device.rs:111-129).
    fn sync(&mut self) -> Result<(), BackendError>;
}
