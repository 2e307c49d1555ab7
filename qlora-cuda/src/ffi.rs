//! Raw bindings to the C ABI of libqlora_cuda.so (include/qlora_cuda.h).  One declaration per entry
//! point this crate uses; names, argument order and types follow the header exactly.

#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_float, c_int, c_void};

pub const QLC_OK: c_int = 0;
pub const QLC_ERR_SHAPE_MISMATCH: c_int = 1;
pub const QLC_ERR_INVALID_CONFIG: c_int = 2;
pub const QLC_ERR_GPU: c_int = 3;

pub const QLC_DTYPE_F32: c_int = 0;
pub const QLC_DTYPE_BF16: c_int = 1;

pub const QLC_PRECISION_AUTO: c_int = 0;
pub const QLC_PRECISION_FP32_EXACT: c_int = 1;
pub const QLC_PRECISION_BF16: c_int = 2;
pub const QLC_PRECISION_TF32: c_int = 3;

#[repr(C)]
pub struct qlc_ctx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qlc_qtensor {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qlc_layer {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qlc_adam {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qlc_comm {
    _private: [u8; 0],
}
pub const QLC_COMM_ID_BYTES: usize = 128;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct qlc_adam_config {
    pub lr: c_float,
    pub beta1: c_float,
    pub beta2: c_float,
    pub eps: c_float,
    pub block_size: usize,
    pub max_resident_pages: usize,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct qlc_adam_stats {
    pub pages_streamed: usize,
    pub state_bytes: usize,
}

extern "C" {
    pub fn qlc_last_error_message() -> *const c_char;

    pub fn qlc_ctx_create(device: c_int, out: *mut *mut qlc_ctx) -> c_int;
    pub fn qlc_ctx_destroy(ctx: *mut qlc_ctx) -> c_int;
    pub fn qlc_ctx_set_precision(ctx: *mut qlc_ctx, precision: c_int) -> c_int;
    pub fn qlc_ctx_set_reserved_sms(ctx: *mut qlc_ctx, sms: c_int) -> c_int;
    pub fn qlc_ctx_synchronize(ctx: *mut qlc_ctx) -> c_int;
    pub fn qlc_ctx_stream(ctx: *mut qlc_ctx) -> *mut c_void;

    pub fn qlc_quantize_nf4(
        ctx: *mut qlc_ctx,
        weights: *const c_float,
        weights_len: usize,
        rows: usize,
        cols: usize,
        block_size: usize,
        double_quant: c_int,
        out: *mut *mut qlc_qtensor,
    ) -> c_int;
    pub fn qlc_qtensor_from_raw_parts(
        ctx: *mut qlc_ctx,
        rows: usize,
        cols: usize,
        block_size: usize,
        codes: *const u8,
        codes_len: usize,
        scales: *const c_float,
        scales_len: usize,
        out: *mut *mut qlc_qtensor,
    ) -> c_int;
    pub fn qlc_qtensor_destroy(q: *mut qlc_qtensor) -> c_int;
    pub fn qlc_qtensor_codes(q: *const qlc_qtensor, out: *mut u8, out_len: usize) -> c_int;
    pub fn qlc_qtensor_block_scales(q: *const qlc_qtensor, out: *mut c_float, out_len: usize) -> c_int;
    pub fn qlc_dequantize(ctx: *mut qlc_ctx, q: *const qlc_qtensor, out: *mut c_float, out_len: usize) -> c_int;

    pub fn qlc_matmul(
        ctx: *mut qlc_ctx,
        a: *const c_float,
        a_len: usize,
        b: *const c_float,
        b_len: usize,
        m: usize,
        k: usize,
        n: usize,
        c: *mut c_float,
    ) -> c_int;
    pub fn qlc_matmul_trans_b(
        ctx: *mut qlc_ctx,
        a: *const c_float,
        a_len: usize,
        b: *const c_float,
        b_len: usize,
        m: usize,
        k: usize,
        n: usize,
        c: *mut c_float,
    ) -> c_int;
    pub fn qlc_matmul_trans_a(
        ctx: *mut qlc_ctx,
        a: *const c_float,
        a_len: usize,
        b: *const c_float,
        b_len: usize,
        m: usize,
        k: usize,
        n: usize,
        c: *mut c_float,
    ) -> c_int;

    pub fn qlc_layer_create(
        ctx: *mut qlc_ctx,
        weight: *mut qlc_qtensor,
        a: *const c_float,
        a_len: usize,
        b: *const c_float,
        b_len: usize,
        r: usize,
        alpha: c_float,
        out: *mut *mut qlc_layer,
    ) -> c_int;
    pub fn qlc_layer_destroy(layer: *mut qlc_layer) -> c_int;
    pub fn qlc_layer_set_weights(
        layer: *mut qlc_layer,
        a: *const c_float,
        a_len: usize,
        b: *const c_float,
        b_len: usize,
    ) -> c_int;

    pub fn qlc_qlora_forward(
        ctx: *mut qlc_ctx,
        layer: *mut qlc_layer,
        x: *const c_float,
        x_len: usize,
        batch: usize,
        y: *mut c_float,
    ) -> c_int;
    pub fn qlc_qlora_backward(
        ctx: *mut qlc_ctx,
        layer: *mut qlc_layer,
        x: *const c_float,
        x_len: usize,
        dy: *const c_float,
        dy_len: usize,
        batch: usize,
        grad_x: *mut c_float,
        grad_a: *mut c_float,
        grad_b: *mut c_float,
    ) -> c_int;
    pub fn qlc_qlora_forward_dev(
        ctx: *mut qlc_ctx,
        layer: *mut qlc_layer,
        d_x: *const c_void,
        dtype: c_int,
        batch: usize,
        d_y: *mut c_void,
    ) -> c_int;
    pub fn qlc_qlora_backward_dev(
        ctx: *mut qlc_ctx,
        layer: *mut qlc_layer,
        d_x: *const c_void,
        d_dy: *const c_void,
        dtype: c_int,
        batch: usize,
        d_grad_x: *mut c_void,
        d_grad_a: *mut c_float,
        d_grad_b: *mut c_float,
    ) -> c_int;

    pub fn qlc_adam_config_default(cfg: *mut qlc_adam_config);
    pub fn qlc_adam_create(ctx: *mut qlc_ctx, cfg: *const qlc_adam_config, out: *mut *mut qlc_adam) -> c_int;
    pub fn qlc_adam_destroy(opt: *mut qlc_adam) -> c_int;
    pub fn qlc_adam_step(
        opt: *mut qlc_adam,
        n_tensors: usize,
        params: *const *mut c_float,
        param_lens: *const usize,
        grads: *const *const c_float,
        grad_lens: *const usize,
        stats: *mut qlc_adam_stats,
    ) -> c_int;
    pub fn qlc_adam_state_bytes(opt: *const qlc_adam) -> usize;

    // bf16 / fp32 host buffers through the row-slab pipelines; forward + backward of one batch in one call
    // (X crosses the host link once), synchronous and asynchronous (ticket) forms
    pub fn qlc_qlora_forward_host(ctx: *mut qlc_ctx, layer: *mut qlc_layer, x: *const c_void, dtype: c_int, batch: usize, y: *mut c_void) -> c_int;
    pub fn qlc_qlora_backward_host(ctx: *mut qlc_ctx, layer: *mut qlc_layer, x: *const c_void, dy: *const c_void, dtype: c_int, batch: usize, grad_x: *mut c_void, grad_a: *mut c_float, grad_b: *mut c_float) -> c_int;
    pub fn qlc_qlora_forward_backward_host(ctx: *mut qlc_ctx, layer: *mut qlc_layer, x: *const c_void, dy: *const c_void, dtype: c_int, batch: usize, y: *mut c_void, grad_x: *mut c_void, grad_a: *mut c_float, grad_b: *mut c_float) -> c_int;
    pub fn qlc_qlora_forward_backward_host_async(ctx: *mut qlc_ctx, layer: *mut qlc_layer, x: *const c_void, dy: *const c_void, dtype: c_int, batch: usize, y: *mut c_void, grad_x: *mut c_void, grad_a: *mut c_float, grad_b: *mut c_float, ticket: *mut u64) -> c_int;
    pub fn qlc_ctx_wait(ctx: *mut qlc_ctx, ticket: u64) -> c_int;

    // optimiser state to and from host memory (checkpoint / resume)
    pub fn qlc_adam_get_state(opt: *mut qlc_adam, index: usize, numel: *mut usize, step: *mut u64, m_codes: *mut u8, v_codes: *mut u8, m_scales: *mut c_float, v_scales: *mut c_float) -> c_int;
    pub fn qlc_adam_set_state(opt: *mut qlc_adam, index: usize, numel: usize, step: u64, m_codes: *const u8, v_codes: *const u8, m_scales: *const c_float, v_scales: *const c_float) -> c_int;

    // gradient exchange between the ranks of a data-parallel job (NCCL, loaded at first use)
    pub fn qlc_comm_unique_id(id_out: *mut u8, id_len: usize) -> c_int;
    pub fn qlc_comm_init(ctx: *mut qlc_ctx, nranks: c_int, rank: c_int, id: *const u8, id_len: usize, out: *mut *mut qlc_comm) -> c_int;
    pub fn qlc_comm_allreduce_sum_f32(comm: *mut qlc_comm, d_buf: *mut c_float, count: usize) -> c_int;
    pub fn qlc_allreduce_lora_grads(comm: *mut qlc_comm, layer: *mut qlc_layer) -> c_int;
    pub fn qlc_comm_destroy(comm: *mut qlc_comm) -> c_int;
}
