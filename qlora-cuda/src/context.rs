//! The CUDA counterpart of `qlora_wgpu::GpuContext` (qlora-wgpu/src/context.rs:18-79).

use std::ffi::CStr;
use std::os::raw::c_int;
use std::ptr;

use qlora_core::QloraError;

use crate::ffi;

/// Arithmetic of the layer GEMMs (QLC_PRECISION_* in include/qlora_cuda.h).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Precision {
    /// Tensor cores where the shape allows it; the fp32 slice entry points then use TF32.
    Auto,
    /// fp32 kernels in the CPU reference's accumulation order: bit-exact, any shape.
    Fp32Exact,
    /// bf16 operands, fp32 accumulation (relative Frobenius error <= 5e-3).
    Bf16,
    /// fp32 operands read as tf32, fp32 accumulation (<= 1e-3).
    Tf32,
}

/// One CUDA device and stream.  Unlike the WGPU backend there is no CPU fallback behind it.
pub struct GpuContext {
    raw: *mut ffi::qlc_ctx,
}

// The library allows one context per host thread; a context may move between threads.
unsafe impl Send for GpuContext {}

/// Turns a status code of the C ABI into the matching `QloraError` variant, with the library's
/// message for the calling thread (its display prefix, e.g. "gpu error: ", is stripped because
/// `QloraError`'s `Display` adds it again).
pub(crate) fn check(status: c_int) -> Result<(), QloraError> {
    if status == ffi::QLC_OK {
        return Ok(());
    }
    let full = unsafe { CStr::from_ptr(ffi::qlc_last_error_message()) }
        .to_string_lossy()
        .into_owned();
    let msg = match full.split_once(": ") {
        Some((_, rest)) => rest.to_string(),
        None => full,
    };
    Err(match status {
        ffi::QLC_ERR_SHAPE_MISMATCH => QloraError::ShapeMismatch(msg),
        ffi::QLC_ERR_INVALID_CONFIG => QloraError::InvalidConfig(msg),
        _ => QloraError::Gpu(msg),
    })
}

impl GpuContext {
    /// Same name and shape as `qlora_wgpu::GpuContext::try_new_blocking` so that callers compile
    /// unchanged.  The WGPU backend answers `Ok(None)` without an adapter and lets callers fall back
    /// to the CPU; this backend has no CPU path, so a missing or non-B200 device is `Err(Gpu(..))`
    /// and `Ok(None)` is never returned.
    pub fn try_new_blocking() -> Result<Option<Self>, QloraError> {
        Self::on_device(0).map(Some)
    }

    /// A context on CUDA device `device`.
    pub fn on_device(device: i32) -> Result<Self, QloraError> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::qlc_ctx_create(device as c_int, &mut raw) })?;
        Ok(Self { raw })
    }

    pub fn set_precision(&self, p: Precision) -> Result<(), QloraError> {
        let code = match p {
            Precision::Auto => ffi::QLC_PRECISION_AUTO,
            Precision::Fp32Exact => ffi::QLC_PRECISION_FP32_EXACT,
            Precision::Bf16 => ffi::QLC_PRECISION_BF16,
            Precision::Tf32 => ffi::QLC_PRECISION_TF32,
        };
        check(unsafe { ffi::qlc_ctx_set_precision(self.raw, code) })
    }

    /// SMs the one-wave weight GEMMs leave free for kernels of other streams (a collective that overlaps them).
    pub fn set_reserved_sms(&self, sms: i32) -> Result<(), QloraError> {
        check(unsafe { ffi::qlc_ctx_set_reserved_sms(self.raw, sms) })
    }

    /// Blocks until the asynchronous submission that returned `ticket` has delivered its outputs to host memory.
    pub fn wait(&self, ticket: u64) -> Result<(), QloraError> {
        check(unsafe { ffi::qlc_ctx_wait(self.raw, ticket) })
    }

    /// Waits for everything queued on the context's stream and reports a status raised by a kernel.
    pub fn synchronize(&self) -> Result<(), QloraError> {
        check(unsafe { ffi::qlc_ctx_synchronize(self.raw) })
    }

    pub(crate) fn raw(&self) -> *mut ffi::qlc_ctx {
        self.raw
    }
}

impl Drop for GpuContext {
    fn drop(&mut self) {
        unsafe {
            ffi::qlc_ctx_destroy(self.raw);
        }
    }
}

/// `ctx = None` selects the CPU reference in the WGPU backend (qlora-wgpu/src/kernels.rs:48-50).
/// Here it is an error.
pub(crate) fn require(ctx: Option<&GpuContext>) -> Result<&GpuContext, QloraError> {
    ctx.ok_or_else(|| QloraError::Gpu("a GPU context is required (this backend has no CPU fallback)".to_string()))
}
