//! `qlora-cuda`: CUDA (B200, sm_100a) backend for QLoRA operations, a sibling of `qlora-wgpu`.
//!
//! The crate exports the items `qlora-wgpu` exports (qlora-wgpu/src/lib.rs:25-32) with the same
//! names and signatures, so a caller switches backends by changing one `use` line:
//!
//! ```ignore
//! // use qlora_wgpu::{GpuContext, gpu_qlora_forward, gpu_qlora_backward};
//! use qlora_cuda::{GpuContext, gpu_qlora_forward, gpu_qlora_backward};
//! ```
//!
//! Host code stays Rust; the arithmetic runs in hand-written CUDA kernels behind the C ABI of
//! `libqlora_cuda.so` (`src/ffi.rs` mirrors `include/qlora_cuda.h`).  One deliberate difference:
//! there is NO CPU fallback.  `GpuContext::try_new_blocking` never returns `Ok(None)`, and passing
//! `None` as the context is `Err(QloraError::Gpu(..))` where `qlora-wgpu` would compute on the CPU
//! (qlora-wgpu/src/kernels.rs:48-50).
//!
//! This crate was written on a machine without a Rust toolchain and has not been compiled.

pub mod context;
pub mod ffi;
pub mod kernels;
pub mod resident;

pub use context::{GpuContext, Precision};
pub use kernels::{
    gpu_dequantize, gpu_matmul, gpu_matmul_trans_a, gpu_matmul_trans_b, gpu_qlora_backward,
    gpu_qlora_forward,
};
pub use resident::{Bf16Grads, CudaPagedAdam, CudaQloraLinear, StepBuffers};
