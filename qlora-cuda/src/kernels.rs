//! The six free functions of `qlora_wgpu::kernels` (qlora-wgpu/src/kernels.rs:44-353) on CUDA.
//! They keep the reference's stateless convention: host slices in, fresh `Vec<f32>` out, the weight
//! uploaded for the call.  For weights that stay on the device between calls use `CudaQloraLinear`.

use std::ptr;

use qlora_core::{QloraError, QloraGrads, QloraLinear, QuantizedTensor};

use crate::context::{check, require, GpuContext};
use crate::ffi;

/// A quantised tensor in device memory, built from a host `QuantizedTensor` the way the WGPU backend
/// uploads one: packed codes plus decoded fp32 block scales (kernels.rs:56-72).
pub(crate) struct DeviceTensor {
    pub(crate) raw: *mut ffi::qlc_qtensor,
}

impl DeviceTensor {
    pub(crate) fn upload(ctx: &GpuContext, q: &QuantizedTensor) -> Result<Self, QloraError> {
        let scales = q.block_scales();
        let codes = q.codes();
        let mut raw = ptr::null_mut();
        check(unsafe {
            ffi::qlc_qtensor_from_raw_parts(
                ctx.raw(),
                q.rows(),
                q.cols(),
                q.block_size(),
                codes.as_ptr(),
                codes.len(),
                scales.as_ptr(),
                scales.len(),
                &mut raw,
            )
        })?;
        Ok(Self { raw })
    }
}

impl Drop for DeviceTensor {
    fn drop(&mut self) {
        unsafe {
            ffi::qlc_qtensor_destroy(self.raw);
        }
    }
}

/// A layer handle that lives for one call.
pub(crate) struct DeviceLayer {
    pub(crate) raw: *mut ffi::qlc_layer,
    _weight: DeviceTensor,
}

impl DeviceLayer {
    pub(crate) fn upload(ctx: &GpuContext, layer: &QloraLinear) -> Result<Self, QloraError> {
        let weight = DeviceTensor::upload(ctx, layer.weight())?;
        let mut raw = ptr::null_mut();
        let status = match layer.adapter() {
            Some(ad) => unsafe {
                ffi::qlc_layer_create(
                    ctx.raw(),
                    weight.raw,
                    ad.a().as_ptr(),
                    ad.a().len(),
                    ad.b().as_ptr(),
                    ad.b().len(),
                    ad.rank(),
                    ad.alpha(),
                    &mut raw,
                )
            },
            None => unsafe {
                ffi::qlc_layer_create(ctx.raw(), weight.raw, ptr::null(), 0, ptr::null(), 0, 0, 0.0, &mut raw)
            },
        };
        check(status)?;
        Ok(Self { raw, _weight: weight })
    }
}

impl Drop for DeviceLayer {
    fn drop(&mut self) {
        unsafe {
            ffi::qlc_layer_destroy(self.raw);
        }
    }
}

/// `gpu_dequantize` (kernels.rs:44-103): bit-identical to `QuantizedTensor::dequantize`.
pub fn gpu_dequantize(ctx: Option<&GpuContext>, q: &QuantizedTensor) -> Result<Vec<f32>, QloraError> {
    let ctx = require(ctx)?;
    let n = q.num_elements();
    let mut out = vec![0.0f32; n];
    if n == 0 {
        return Ok(out);
    }
    let t = DeviceTensor::upload(ctx, q)?;
    check(unsafe { ffi::qlc_dequantize(ctx.raw(), t.raw, out.as_mut_ptr(), out.len()) })?;
    Ok(out)
}

type GemmFn = unsafe extern "C" fn(
    *mut ffi::qlc_ctx,
    *const f32,
    usize,
    *const f32,
    usize,
    usize,
    usize,
    usize,
    *mut f32,
) -> std::os::raw::c_int;

fn gemm(
    f: GemmFn,
    ctx: Option<&GpuContext>,
    a: &[f32],
    b: &[f32],
    m: usize,
    k: usize,
    n: usize,
    out_len: usize,
) -> Result<Vec<f32>, QloraError> {
    let ctx = require(ctx)?;
    let mut c = vec![0.0f32; out_len];
    check(unsafe { f(ctx.raw(), a.as_ptr(), a.len(), b.as_ptr(), b.len(), m, k, n, c.as_mut_ptr()) })?;
    Ok(c)
}

/// `gpu_matmul` (kernels.rs:140-176): `C(m,n) = A(m,k)·B(k,n)`.
pub fn gpu_matmul(
    ctx: Option<&GpuContext>,
    a: &[f32],
    b: &[f32],
    m: usize,
    k: usize,
    n: usize,
) -> Result<Vec<f32>, QloraError> {
    gemm(ffi::qlc_matmul, ctx, a, b, m, k, n, m * n)
}

/// `gpu_matmul_trans_b` (kernels.rs:180-216): `C(m,n) = A(m,k)·B(n,k)^T`.
pub fn gpu_matmul_trans_b(
    ctx: Option<&GpuContext>,
    a: &[f32],
    b: &[f32],
    m: usize,
    k: usize,
    n: usize,
) -> Result<Vec<f32>, QloraError> {
    gemm(ffi::qlc_matmul_trans_b, ctx, a, b, m, k, n, m * n)
}

/// `gpu_matmul_trans_a` (kernels.rs:220-257): `C(k,n) = A(m,k)^T·B(m,n)`.
pub fn gpu_matmul_trans_a(
    ctx: Option<&GpuContext>,
    a: &[f32],
    b: &[f32],
    m: usize,
    k: usize,
    n: usize,
) -> Result<Vec<f32>, QloraError> {
    gemm(ffi::qlc_matmul_trans_a, ctx, a, b, m, k, n, k * n)
}

/// `gpu_qlora_forward` (kernels.rs:262-296).
pub fn gpu_qlora_forward(
    ctx: Option<&GpuContext>,
    layer: &QloraLinear,
    x: &[f32],
    batch: usize,
) -> Result<Vec<f32>, QloraError> {
    let ctx = require(ctx)?;
    let dev = DeviceLayer::upload(ctx, layer)?;
    let mut y = vec![0.0f32; batch * layer.out_dim()];
    check(unsafe { ffi::qlc_qlora_forward(ctx.raw(), dev.raw, x.as_ptr(), x.len(), batch, y.as_mut_ptr()) })?;
    Ok(y)
}

/// `gpu_qlora_backward` (kernels.rs:301-353).
pub fn gpu_qlora_backward(
    ctx: Option<&GpuContext>,
    layer: &QloraLinear,
    x: &[f32],
    dy: &[f32],
    batch: usize,
) -> Result<QloraGrads, QloraError> {
    let ctx = require(ctx)?;
    let dev = DeviceLayer::upload(ctx, layer)?;
    let mut grad_x = vec![0.0f32; batch * layer.in_dim()];
    let (mut grad_a, mut grad_b) = match layer.adapter() {
        Some(ad) => (
            Some(vec![0.0f32; ad.rank() * layer.in_dim()]),
            Some(vec![0.0f32; layer.out_dim() * ad.rank()]),
        ),
        None => (None, None),
    };
    let pa = grad_a.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
    let pb = grad_b.as_mut().map_or(ptr::null_mut(), |v| v.as_mut_ptr());
    check(unsafe {
        ffi::qlc_qlora_backward(
            ctx.raw(),
            dev.raw,
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
