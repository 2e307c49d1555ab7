//! Device-resident forms for callers that keep a layer or an optimiser across steps (the WGPU backend
//! re-uploads everything on every call, qlora-wgpu/src/kernels.rs:56-93).

use std::ptr;

use qlora_core::{AdamConfig, AdamStats, QloraError, QloraGrads, QloraLinear, QuantConfig};

use crate::context::{check, GpuContext};
use crate::ffi;
use crate::kernels::DeviceLayer;

/// `QloraLinear` whose NF4 weight and adapter stay in device memory.
pub struct CudaQloraLinear<'c> {
    ctx: &'c GpuContext,
    dev: DeviceLayer,
    in_dim: usize,
    out_dim: usize,
    rank: usize,
}

impl<'c> CudaQloraLinear<'c> {
    /// From a host layer (`QloraLinear::new` / `from_quantized`, qlora-core/src/qlora.rs:41-83).
    pub fn from_layer(ctx: &'c GpuContext, layer: &QloraLinear) -> Result<Self, QloraError> {
        Ok(Self {
            ctx,
            dev: DeviceLayer::upload(ctx, layer)?,
            in_dim: layer.in_dim(),
            out_dim: layer.out_dim(),
            rank: layer.adapter().map_or(0, |a| a.rank()),
        })
    }

    /// Quantises on the host with `qlora-core` and uploads (`QloraLinear::new`, qlora.rs:41-64).
    pub fn new(
        ctx: &'c GpuContext,
        weight: &[f32],
        out_dim: usize,
        in_dim: usize,
        quant: &QuantConfig,
        adapter: Option<qlora_core::LoraAdapter>,
    ) -> Result<Self, QloraError> {
        let host = QloraLinear::new(weight, out_dim, in_dim, quant, adapter)?;
        Self::from_layer(ctx, &host)
    }

    pub fn in_dim(&self) -> usize {
        self.in_dim
    }
    pub fn out_dim(&self) -> usize {
        self.out_dim
    }

    /// `QloraLinear::forward` (qlora.rs:86-107).
    pub fn forward(&self, x: &[f32], batch: usize) -> Result<Vec<f32>, QloraError> {
        let mut y = vec![0.0f32; batch * self.out_dim];
        check(unsafe {
            ffi::qlc_qlora_forward(self.ctx.raw(), self.dev.raw, x.as_ptr(), x.len(), batch, y.as_mut_ptr())
        })?;
        Ok(y)
    }

    /// `QloraLinear::backward` (qlora.rs:116-165).
    pub fn backward(&self, x: &[f32], dy: &[f32], batch: usize) -> Result<QloraGrads, QloraError> {
        let mut grad_x = vec![0.0f32; batch * self.in_dim];
        let mut grad_a = (self.rank > 0).then(|| vec![0.0f32; self.rank * self.in_dim]);
        let mut grad_b = (self.rank > 0).then(|| vec![0.0f32; self.out_dim * self.rank]);
        let pa = grad_a.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
        let pb = grad_b.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
        check(unsafe {
            ffi::qlc_qlora_backward(
                self.ctx.raw(),
                self.dev.raw,
                x.as_ptr(),
                x.len(),
                dy.as_ptr(),
                dy.len(),
                batch,
                grad_x.as_mut_ptr(),
                pa,
                pb,
            )
        })?;
        Ok(QloraGrads { grad_a, grad_b, grad_x })
    }

    /// Forward and backward of one batch of bf16 activations (raw bf16 bit patterns) in one call: the same results
    /// as `gpu_qlora_forward` followed by `gpu_qlora_backward` (kernels.rs:262-353), but X crosses the host link once.
    pub fn forward_backward_bf16(&self, x: &[u16], dy: &[u16], batch: usize) -> Result<(Vec<u16>, Bf16Grads), QloraError> {
        if x.len() != batch * self.in_dim || dy.len() != batch * self.out_dim {
            return Err(QloraError::ShapeMismatch(format!(
                "x.len() = {}, dy.len() = {} but batch*in_dim = {}, batch*out_dim = {}",
                x.len(), dy.len(), batch * self.in_dim, batch * self.out_dim
            )));
        }
        let mut y = vec![0u16; batch * self.out_dim];
        let mut grad_x = vec![0u16; batch * self.in_dim];
        let mut grad_a = (self.rank > 0).then(|| vec![0.0f32; self.rank * self.in_dim]);
        let mut grad_b = (self.rank > 0).then(|| vec![0.0f32; self.out_dim * self.rank]);
        let pa = grad_a.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
        let pb = grad_b.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
        check(unsafe {
            ffi::qlc_qlora_forward_backward_host(
                self.ctx.raw(),
                self.dev.raw,
                x.as_ptr().cast(),
                dy.as_ptr().cast(),
                ffi::QLC_DTYPE_BF16,
                batch,
                y.as_mut_ptr().cast(),
                grad_x.as_mut_ptr().cast(),
                pa,
                pb,
            )
        })?;
        Ok((y, Bf16Grads { grad_a, grad_b, grad_x }))
    }

    /// The same call without waiting: the buffers of `io` must stay untouched until `GpuContext::wait(ticket)` has
    /// returned.  A caller that keeps two submissions in flight, each on its own `StepBuffers`, keeps the host link
    /// busy in both directions.
    ///
    /// # Safety
    /// `io` is borrowed by the device until the ticket has been waited for.
    pub unsafe fn submit_forward_backward_bf16(&self, io: &mut StepBuffers, batch: usize) -> Result<u64, QloraError> {
        let mut ticket = 0u64;
        check(ffi::qlc_qlora_forward_backward_host_async(
            self.ctx.raw(),
            self.dev.raw,
            io.x.as_ptr().cast(),
            io.dy.as_ptr().cast(),
            ffi::QLC_DTYPE_BF16,
            batch,
            io.y.as_mut_ptr().cast(),
            io.grad_x.as_mut_ptr().cast(),
            io.grad_a.as_mut_ptr(),
            io.grad_b.as_mut_ptr(),
            &mut ticket,
        ))?;
        Ok(ticket)
    }

    /// `LoraAdapter::set_weights` through `adapter_mut` (lora.rs:70-83, qlora.rs:175-177).
    pub fn set_adapter_weights(&mut self, a: &[f32], b: &[f32]) -> Result<(), QloraError> {
        check(unsafe { ffi::qlc_layer_set_weights(self.dev.raw, a.as_ptr(), a.len(), b.as_ptr(), b.len()) })
    }
}

/// Gradients of the bf16 calls: `grad_x` as bf16 bit patterns, adapter gradients in fp32 (`QloraGrads`, qlora.rs:13-20).
pub struct Bf16Grads {
    pub grad_a: Option<Vec<f32>>,
    pub grad_b: Option<Vec<f32>>,
    pub grad_x: Vec<u16>,
}

/// Host buffers of one asynchronous step (allocate them page-locked for full link speed).
pub struct StepBuffers {
    pub x: Vec<u16>,
    pub dy: Vec<u16>,
    pub y: Vec<u16>,
    pub grad_x: Vec<u16>,
    pub grad_a: Vec<f32>,
    pub grad_b: Vec<f32>,
}

/// `Adam8bit` (qlora-core/src/optim.rs:143-204) with its 8-bit state on the device, or paged through
/// pinned host memory when `max_resident_pages` is smaller than the number of state pages.
pub struct CudaPagedAdam<'c> {
    _ctx: &'c GpuContext,
    raw: *mut ffi::qlc_adam,
}

impl<'c> CudaPagedAdam<'c> {
    /// `Adam8bit::new` (optim.rs:155-161).
    pub fn new(ctx: &'c GpuContext, config: AdamConfig) -> Result<Self, QloraError> {
        let cfg = ffi::qlc_adam_config {
            lr: config.lr,
            beta1: config.beta1,
            beta2: config.beta2,
            eps: config.eps,
            block_size: config.block_size,
            max_resident_pages: config.max_resident_pages,
        };
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::qlc_adam_create(ctx.raw(), &cfg, &mut raw) })?;
        Ok(Self { _ctx: ctx, raw })
    }

    /// `Adam8bit::step` (optim.rs:164-199): parameters are updated in place.
    pub fn step(&mut self, params: &mut [&mut [f32]], grads: &[&[f32]]) -> Result<AdamStats, QloraError> {
        if params.len() != grads.len() {
            return Err(QloraError::ShapeMismatch(format!(
                "params.len() = {} but grads.len() = {}",
                params.len(),
                grads.len()
            )));
        }
        let p_ptrs: Vec<*mut f32> = params.iter_mut().map(|p| p.as_mut_ptr()).collect();
        let p_lens: Vec<usize> = params.iter().map(|p| p.len()).collect();
        let g_ptrs: Vec<*const f32> = grads.iter().map(|g| g.as_ptr()).collect();
        let g_lens: Vec<usize> = grads.iter().map(|g| g.len()).collect();
        let mut stats = ffi::qlc_adam_stats::default();
        check(unsafe {
            ffi::qlc_adam_step(
                self.raw,
                p_ptrs.len(),
                p_ptrs.as_ptr(),
                p_lens.as_ptr(),
                g_ptrs.as_ptr(),
                g_lens.as_ptr(),
                &mut stats,
            )
        })?;
        Ok(AdamStats {
            pages_streamed: stats.pages_streamed,
            state_bytes: stats.state_bytes,
        })
    }

    /// `Adam8bit::state_bytes` (optim.rs:201-204).
    pub fn state_bytes(&self) -> usize {
        unsafe { ffi::qlc_adam_state_bytes(self.raw) }
    }
}

impl Drop for CudaPagedAdam<'_> {
    fn drop(&mut self) {
        unsafe {
            ffi::qlc_adam_destroy(self.raw);
        }
    }
}
