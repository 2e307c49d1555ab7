/*
 * qlora_cuda.h — C ABI of libqlora_cuda.so, the B200 (sm_100a) implementation of the
 * QloraLinear hot path of VkQLoRA.rs.
 *
 * This is the surface a `qlora-cuda` Rust crate (sitting beside the reference's
 * `qlora-wgpu`) binds with an `extern "C"` block, and the surface the Python module with
 * the reference's PyO3 entry points calls through ctypes.  Every entry point cites the
 * reference interface it replaces (paths are relative to the reference repository).
 *
 * Conventions
 *  - Every function returns an int status: QLC_OK, or one of the three error kinds of the
 *    reference's `QloraError` (qlora-core/src/error.rs:7-26).  The human-readable message
 *    of the last failure on the calling thread is returned by qlc_last_error_message().
 *  - There is NO CPU fallback: without a usable CUDA device every call fails with
 *    QLC_ERR_GPU (the reference's `None`-context fallback, qlora-wgpu/src/kernels.rs:48-50,
 *    is deliberately not reproduced).
 *  - All matrices are row-major.  W:(out_dim,in_dim)  X:(batch,in_dim)  Y,dY:(batch,out_dim)
 *    A:(r,in_dim)  B:(out_dim,r).
 *  - Functions without a `_dev` suffix take HOST pointers, are synchronous, and copy data
 *    both ways (the reference's Vec<f32>/&[f32] convention).  `_dev` functions take DEVICE
 *    pointers, enqueue work on the context's stream and return without synchronising.
 *  - The caller owns every buffer it passes; the library owns handles.  No pointer is kept
 *    after a call returns unless it is a handle.
 *  - A context is bound to one device and one stream; use one context per host thread.
 */
#ifndef QLORA_CUDA_H_
#define QLORA_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* qlora-core/src/error.rs:7-26 — QloraError::{ShapeMismatch, InvalidConfig, Gpu}. */
#define QLC_OK 0
#define QLC_ERR_SHAPE_MISMATCH 1
#define QLC_ERR_INVALID_CONFIG 2
#define QLC_ERR_GPU 3

/* Element types of device / host activation buffers. */
#define QLC_DTYPE_F32 0
#define QLC_DTYPE_BF16 1
#define QLC_DTYPE_F16 2 /* accepted by qlc_quantize_nf4_typed only */

/* Arithmetic used by the layer GEMMs.
 *  AUTO       : tensor-core path (bf16 operands, fp32 accumulate) for every quantised layer with a LoRA
 *               rank <= 256.  Layers with block_size 32, 64, 128 or 256 and in_dim / out_dim multiples of
 *               64 run the fused kernels (the NF4 weight tile is decoded inside the GEMM); any other
 *               dimensions or block size run through a zero-padded bf16 copy of the layer (2 bytes per
 *               weight of extra device memory, built at the layer's first call).  Larger ranks take the
 *               exact fp32 path.  Exception: the reference-named fp32 host entry points
 *               qlc_qlora_forward / qlc_qlora_backward use TF32 instead of bf16 on fused-kernel shapes and
 *               the exact fp32 path on all others, so that they keep the reference's GPU-vs-CPU
 *               tolerances (max abs diff 1e-3 / 1e-2, qlora-wgpu/tests/gpu_parity.rs:59,
 *               gpu_backward.rs:88-96) at every shape.
 *  FP32_EXACT : fp32 SIMT kernels that reproduce the reference's CPU accumulation order
 *               bit-for-bit (any shape, any block size).
 *  BF16       : force the tensor-core path; a layer it does not take (rank > 256) fails with QLC_ERR_GPU.
 *  TF32       : tensor-core path with fp32 operands read as tf32 (fp32 accumulate), for a relative
 *               Frobenius error <= 1e-3, about half the speed of BF16.  Fused-kernel shapes only: other
 *               layers are multiplied in exact fp32 in this mode.  fp32 activations are consumed as they
 *               are (bf16 ones are widened first). */
#define QLC_PRECISION_AUTO 0
#define QLC_PRECISION_FP32_EXACT 1
#define QLC_PRECISION_BF16 2
#define QLC_PRECISION_TF32 3

typedef struct qlc_ctx qlc_ctx;         /* replaces qlora_wgpu::GpuContext (qlora-wgpu/src/context.rs:18-28) */
typedef struct qlc_qtensor qlc_qtensor; /* replaces qlora_core::QuantizedTensor (qlora-core/src/quant.rs:93-101) */
typedef struct qlc_layer qlc_layer;     /* replaces qlora_core::QloraLinear (qlora-core/src/qlora.rs:33-37) */
typedef struct qlc_adam qlc_adam;       /* replaces qlora_core::Adam8bit (qlora-core/src/optim.rs:147-151) */

/* Message of the last error raised on this thread (never NULL).  Display text follows
 * qlora-core/src/error.rs:17-23 ("shape mismatch: ...", "invalid config: ...", "gpu error: ..."). */
const char *qlc_last_error_message(void);

/* ---- context ----------------------------------------------------------------------- */

/* GpuContext::try_new_blocking (qlora-wgpu/src/context.rs:33-79).  Fails with QLC_ERR_GPU
 * when `device` is not a usable CUDA device (no silent CPU fallback). */
int qlc_ctx_create(int device, qlc_ctx **out);
/* Drops the creator's reference.  Layers and optimisers created on the context keep it alive; its
 * stream and scratch memory are released when the last of them is destroyed. */
int qlc_ctx_destroy(qlc_ctx *ctx);
int qlc_ctx_set_precision(qlc_ctx *ctx, int precision);
/* The weight GEMMs run as ONE wave of CTA pairs, one pair per two SMs, each pair walking its share of the tiles.
 * A kernel of another stream that holds an SM when such a GEMM starts (a collective of the gradient exchange,
 * for instance) keeps one pair from starting until it ends, and that pair's tiles wait with it.  A host that
 * overlaps such kernels with the layer passes reserves their SMs here: the GEMMs then use (SMs - sms) / 2 pairs.
 * sms is rounded down to an even number; 0 (the default) uses every SM.  No counterpart in the reference. */
int qlc_ctx_set_reserved_sms(qlc_ctx *ctx, int sms);
/* Blocks until everything enqueued on the context's stream has finished, then reports any
 * device-side status raised by the kernels (e.g. a bounded wait that gave up). */
int qlc_ctx_synchronize(qlc_ctx *ctx);
/* The context's cudaStream_t, for callers that interleave their own work. */
void *qlc_ctx_stream(qlc_ctx *ctx);
/* Copies between host memory and device memory in the context's stream order (asynchronous for pinned host
 * memory; complete after qlc_ctx_synchronize), for hosts that link no CUDA runtime of their own - e.g. to read
 * a layer's device gradient bucket (qlc_layer_grad_bucket) after an all-reduce.  (No counterpart in the
 * reference: its buffers never outlive a call.) */
int qlc_ctx_copy_to_host(qlc_ctx *ctx, void *dst, const void *d_src, size_t bytes);
int qlc_ctx_copy_to_device(qlc_ctx *ctx, void *d_dst, const void *src, size_t bytes);
/* Number of kernels this context has launched since creation (diagnostics / benchmarks). */
uint64_t qlc_ctx_launch_count(const qlc_ctx *ctx);

/* Per-kernel timing for benchmarks (no counterpart in the reference, whose compute pass is created
 * with `timestamp_writes: None`, qlora-wgpu/src/kernels.rs:381-384).  While enabled, the tensor-core
 * GEMM launches of this context are bracketed by CUDA events on the context's stream.
 * qlc_ctx_profile_read synchronises, then returns for kernel slot `slot` the summed device time in
 * milliseconds and the number of launches since the last read, and clears the slot.
 * Slots: 0 = forward GEMM (X·deq(W)^T + LoRA), 1 = backward dX GEMM (dY·deq(W) + LoRA),
 *        2 = skinny LoRA products (X·A^T, dY·B), 3 = token-contracted gradient products. */
#define QLC_PROFILE_SLOTS 4
int qlc_ctx_profile_enable(qlc_ctx *ctx, int enable);
int qlc_ctx_profile_read(qlc_ctx *ctx, int slot, double *total_ms, uint64_t *launches);

/* ---- NF4 quantisation -------------------------------------------------------------- */

/* QuantizedTensor::quantize(weights, rows, cols, &QuantConfig{block_size, double_quant})
 * (qlora-core/src/quant.rs:104-154; config validation :72-79).  `weights_len` is the slice
 * length and must equal rows*cols. */
int qlc_quantize_nf4(qlc_ctx *ctx, const float *weights, size_t weights_len, size_t rows, size_t cols,
                     size_t block_size, int double_quant, qlc_qtensor **out);
/* Same, reading rows*cols fp32 weights that already live in device memory. */
/* Same for host weights stored as fp32, bf16 or fp16 (checkpoint dtypes): the raw values are uploaded and
 * widened to fp32 on the device (exact for all three), then quantised - the codes equal those of widening on the
 * host first, which is what the reference's loader does (qlora-io/src/safetensors.rs:82-99 then quant.rs:104). */
int qlc_quantize_nf4_typed(qlc_ctx *ctx, const void *weights, int dtype, size_t rows, size_t cols, size_t block_size,
                           int double_quant, qlc_qtensor **out);
int qlc_quantize_nf4_dev(qlc_ctx *ctx, const float *d_weights, size_t rows, size_t cols, size_t block_size,
                         int double_quant, qlc_qtensor **out);
/* Re-runs QuantizedTensor::quantize (quant.rs:104-154) on new rows*cols fp32 device weights INTO an existing
 * tensor of the same shape and configuration (no allocation; asynchronous).  The reference has no in-place
 * form; this is the call to use when weights are re-quantised repeatedly, and what the benchmark times. */
int qlc_qtensor_requantize_dev(qlc_ctx *ctx, qlc_qtensor *q, const float *d_weights);
/* QuantizedTensor::from_raw_parts (qlora-core/src/quant.rs:171-207): plain fp32 scales. */
int qlc_qtensor_from_raw_parts(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, const uint8_t *codes,
                               size_t codes_len, const float *scales, size_t scales_len, qlc_qtensor **out);
/* A double-quantised tensor from its stored payload: packed nibbles, the 8-bit absmax codes and the fp32
 * second-level absmax, exactly the three arrays of ScaleStore::Int8 (qlora-core/src/quant.rs:84-101) that
 * qlc_qtensor_codes / _absmax_codes / _absmax2 return.  The reference has no constructor for this form (its
 * from_raw_parts always yields fp32 scales, quant.rs:171-207); this one lets a saved NF4 payload come back
 * bit for bit, 8-bit scales included.  Length checks as from_raw_parts, plus absmax2_len == ceil(blocks/256). */
int qlc_qtensor_from_double_quant_parts(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, const uint8_t *codes,
                                        size_t codes_len, const uint8_t *absmax_codes, size_t absmax_codes_len,
                                        const float *absmax2, size_t absmax2_len, qlc_qtensor **out);
int qlc_qtensor_destroy(qlc_qtensor *q);

typedef struct qlc_qtensor_info {
    size_t rows;          /* QuantizedTensor::rows          quant.rs:242 */
    size_t cols;          /* QuantizedTensor::cols          quant.rs:245 */
    size_t block_size;    /* QuantizedTensor::block_size    quant.rs:248 */
    size_t num_elements;  /* QuantizedTensor::num_elements  quant.rs:224 */
    size_t num_blocks;    /* QuantizedTensor::num_blocks    quant.rs:251 */
    size_t codes_len;     /* ceil(num_elements / 2)         quant.rs:255 */
    size_t absmax2_len;   /* ceil(num_blocks / 256), 0 without double quant */
    size_t storage_bytes; /* QuantizedTensor::storage_bytes quant.rs:229-235 */
    int double_quant;     /* QuantizedTensor::uses_double_quant quant.rs:238 */
} qlc_qtensor_info;
int qlc_qtensor_get_info(const qlc_qtensor *q, qlc_qtensor_info *info);
/* QuantizedTensor::codes (quant.rs:255): packed nibbles, element 2i = low nibble of byte i. */
int qlc_qtensor_codes(const qlc_qtensor *q, uint8_t *out, size_t out_len);
/* The 8-bit absmax codes and fp32 second-level absmax of a double-quantised tensor
 * (private ScaleStore::Int8 fields, quant.rs:84-89).  QLC_ERR_INVALID_CONFIG without double quant. */
int qlc_qtensor_absmax_codes(const qlc_qtensor *q, uint8_t *out, size_t out_len);
int qlc_qtensor_absmax2(const qlc_qtensor *q, float *out, size_t out_len);
/* QuantizedTensor::block_scales (quant.rs:212-221): decoded fp32 scale per block. */
int qlc_qtensor_block_scales(const qlc_qtensor *q, float *out, size_t out_len);
/* Device addresses of the payload (NULL where absent); valid until the tensor is destroyed. */
int qlc_qtensor_device_ptrs(const qlc_qtensor *q, const uint8_t **d_codes, const uint8_t **d_absmax_codes,
                            const float **d_absmax2, const float **d_scales_f32);
/* gpu_dequantize (qlora-wgpu/src/kernels.rs:44-103) == QuantizedTensor::dequantize
 * (quant.rs:157-167): out has rows*cols fp32 values, bit-exact. */
int qlc_dequantize(qlc_ctx *ctx, const qlc_qtensor *q, float *out, size_t out_len);
/* Device output, fp32 (bit-exact) or bf16 (= round-to-nearest-even of the fp32 value). */
int qlc_dequantize_dev(qlc_ctx *ctx, const qlc_qtensor *q, void *d_out, int dtype);

/* ---- plain row-major GEMMs (fp32, exact reference accumulation order) -------------- */

/* gpu_matmul (kernels.rs:140-176) == lora::matmul (lora.rs:129-142): C(m,n) = A(m,k)·B(k,n). */
int qlc_matmul(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k,
               size_t n, float *c);
/* gpu_matmul_trans_b (kernels.rs:180-216) == lora::matmul_trans_b (lora.rs:169-183): C(m,n) = A(m,k)·B(n,k)^T. */
int qlc_matmul_trans_b(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k,
                       size_t n, float *c);
/* gpu_matmul_trans_a (kernels.rs:220-257) == lora::matmul_trans_a (lora.rs:148-162): C(k,n) = A(m,k)^T·B(m,n). */
int qlc_matmul_trans_a(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k,
                       size_t n, float *c);

/* ---- QloraLinear ------------------------------------------------------------------- */

/* QloraLinear::from_quantized(weight, Some(LoraAdapter::new(a, b, in_dim, out_dim, r, alpha)))
 * (qlora.rs:67-83, lora.rs:28-61).  Pass a == NULL and b == NULL (r ignored) for a layer
 * without an adapter.  The layer keeps a reference to `weight`; destroying the tensor handle
 * afterwards is safe.  A and B are copied. */
int qlc_layer_create(qlc_ctx *ctx, qlc_qtensor *weight, const float *a, size_t a_len, const float *b, size_t b_len,
                     size_t r, float alpha, qlc_layer **out);
/* QloraLinear::new (qlora.rs:41-64): quantise an fp32 (out_dim, in_dim) weight, then as above. */
int qlc_layer_create_from_fp32(qlc_ctx *ctx, const float *weight, size_t weight_len, size_t out_dim, size_t in_dim,
                               size_t block_size, int double_quant, const float *a, size_t a_len, const float *b,
                               size_t b_len, size_t r, float alpha, qlc_layer **out);
int qlc_layer_destroy(qlc_layer *layer);
/* LoraAdapter::set_weights via QloraLinear::adapter_mut (lora.rs:70-83, qlora.rs:175-177). */
int qlc_layer_set_weights(qlc_layer *layer, const float *a, size_t a_len, const float *b, size_t b_len);
/* Same with device fp32 sources (r*in_dim and out_dim*r values), stream-ordered. */
int qlc_layer_set_weights_dev(qlc_layer *layer, const float *d_a, const float *d_b);
/* Device pointers of the layer's fp32 A (r*in_dim) and B (out_dim*r): an optimiser can update them in place
 * (qlc_adam_step_dev); call qlc_layer_adapter_updated afterwards (stream-ordered) so that the operand copies
 * the kernels read follow.  The reference instead rebuilds LoraAdapter and QloraLinear from host vectors every
 * step (qlora-core/examples/train_lora.rs:26-47). */
int qlc_layer_adapter_dev(qlc_layer *layer, float **d_a, float **d_b);
int qlc_layer_adapter_updated(qlc_layer *layer);
/* QloraLinear::{in_dim,out_dim} (qlora.rs:178-183), LoraAdapter::{rank,alpha} (lora.rs:111-116); rank 0 = no adapter. */
int qlc_layer_dims(const qlc_layer *layer, size_t *out_dim, size_t *in_dim, size_t *rank, float *alpha);
/* QloraLinear::weight (qlora.rs:167-169): borrowed handle, owned by the layer. */
qlc_qtensor *qlc_layer_weight(qlc_layer *layer);

/* gpu_qlora_forward (kernels.rs:262-296) == QloraLinear::forward (qlora.rs:86-107).
 * x: batch*in_dim fp32 (x_len is the slice length), y: batch*out_dim fp32. */
int qlc_qlora_forward(qlc_ctx *ctx, qlc_layer *layer, const float *x, size_t x_len, size_t batch, float *y);
/* gpu_qlora_backward (kernels.rs:301-353) == QloraLinear::backward (qlora.rs:116-165).
 * grad_x: batch*in_dim; grad_a: r*in_dim; grad_b: out_dim*r.  grad_a/grad_b may be NULL, and
 * are not written for a layer without an adapter (QloraGrads::{grad_a,grad_b} == None). */
int qlc_qlora_backward(qlc_ctx *ctx, qlc_layer *layer, const float *x, size_t x_len, const float *dy, size_t dy_len,
                       size_t batch, float *grad_x, float *grad_a, float *grad_b);
/* Host-buffer variants that take/return activations as `dtype` (fp32 or bf16) and stream the
 * copies through the context's pinned staging buffers; gradients of A and B stay fp32. */
int qlc_qlora_forward_host(qlc_ctx *ctx, qlc_layer *layer, const void *x, int dtype, size_t batch, void *y);
int qlc_qlora_backward_host(qlc_ctx *ctx, qlc_layer *layer, const void *x, const void *dy, int dtype, size_t batch,
                            void *grad_x, float *grad_a, float *grad_b);
/* Forward and backward of one batch in one call, for callers that hold X and dY together (a benchmark step, or
 * a backward pass replayed with a stored upstream gradient): the same results as qlc_qlora_forward_host followed
 * by qlc_qlora_backward_host, but X crosses the host link once instead of twice and one row-slab pipeline
 * (copy in | forward + backward | copy out) serves both passes.  The reference's two stateless calls upload X
 * twice (qlora-wgpu/src/kernels.rs:262-267 and 301-307 each take x); those calls remain.  grad_a / grad_b may
 * both be NULL: the gradients then go to the layer's device bucket (qlc_layer_grad_bucket) and stay there, e.g.
 * for an all-reduce; with a host pointer given the pipelined form accumulates them in its own staging memory and
 * leaves the layer's bucket alone. */
int qlc_qlora_forward_backward_host(qlc_ctx *ctx, qlc_layer *layer, const void *x, const void *dy, int dtype,
                                    size_t batch, void *y, void *grad_x, float *grad_a, float *grad_b);
/* The same call without waiting: it returns once the copies and kernels are queued and hands out a ticket;
 * qlc_ctx_wait(ctx, ticket) blocks until that submission's outputs are in host memory (qlc_ctx_synchronize
 * waits for all of them and reports any kernel status).  A caller that keeps two submissions in flight, each with
 * its own host buffers, hides the start and the end of one step's copies behind the other's: the host link stays
 * busy in both directions.  Every host buffer of a submission must stay valid and untouched until its ticket has
 * been waited for.  Shapes the pipeline does not take (see above) run synchronously and return a finished ticket. */
int qlc_qlora_forward_backward_host_async(qlc_ctx *ctx, qlc_layer *layer, const void *x, const void *dy, int dtype,
                                          size_t batch, void *y, void *grad_x, float *grad_a, float *grad_b,
                                          uint64_t *ticket);
int qlc_ctx_wait(qlc_ctx *ctx, uint64_t ticket);
/* Device-pointer variants: activations (x, dy, y, grad_x) are `dtype`; d_grad_a / d_grad_b are
 * fp32 device buffers (may be NULL).  Asynchronous on the context's stream. */
int qlc_qlora_forward_dev(qlc_ctx *ctx, qlc_layer *layer, const void *d_x, int dtype, size_t batch, void *d_y);
int qlc_qlora_backward_dev(qlc_ctx *ctx, qlc_layer *layer, const void *d_x, const void *d_dy, int dtype,
                           size_t batch, void *d_grad_x, float *d_grad_a, float *d_grad_b);

/* Forward pass for callers that cannot allocate device memory.  (No counterpart in the reference: its
 * GPU path creates fresh buffers for every operation, qlora-wgpu/src/kernels.rs:62-93.)
 *
 * Some hosts of this library must not trigger cudaMalloc/cudaFree while they run: a serving or training
 * process that has already given every spare byte of device memory to its own pool and would fail or
 * fragment on a late driver allocation, and step loops that cannot afford the device-wide
 * synchronisation a driver allocation or free implies.  qlc_qlora_forward_dev may grow the context's
 * scratch arena (a cudaMalloc) when it meets a larger batch; this variant never does.  Its only
 * scratch - the rank-padded LoRA intermediate, 128 bytes per row - is a fixed 1 MiB array compiled
 * into the library and present on every GPU that loads it until the process exits.
 *
 *  - Same arithmetic and result as qlc_qlora_forward_dev with QLC_DTYPE_BF16: d_x is (batch, in_dim)
 *    bf16, d_y is (batch, out_dim) bf16, both device pointers, 16-byte aligned; asynchronous on the
 *    context's stream.
 *  - Limits: batch <= 8192 rows per call (more fails with QLC_ERR_INVALID_CONFIG and a message saying
 *    so; split larger batches), and the layer must be eligible for the tensor-core path (block_size 32, 64, 128 or 256,
 *    in_dim and out_dim multiples of 64, rank <= 64).
 *  - The call makes no cudaMalloc, cudaFree or other allocating CUDA call.  The first call on each
 *    device additionally looks up the array's device address (cudaGetSymbolAddress); make that first
 *    call during start-up, before any stream capture.  The two diagnostics of this library do allocate
 *    and must stay off for this guarantee: per-kernel timing (qlc_ctx_profile_enable creates CUDA
 *    events as it goes) and the QLC_GEMM_TIMING environment variable (a device buffer per launch).
 *  - All calls on a device share the one array, in every context and stream.  Two such calls whose
 *    kernels overlap on the GPU race on it; serialise them (one stream, or events).  Nothing has to be
 *    cleared between calls: each call rewrites every scratch row it later reads. */
int qlc_qlora_forward_dev_noalloc(qlc_ctx *ctx, qlc_layer *layer, const void *d_x, size_t batch, void *d_y);

/* ---- paged 8-bit Adam --------------------------------------------------------------- */

/* AdamConfig (qlora-core/src/optim.rs:33-58).  max_resident_pages == SIZE_MAX keeps every
 * state page on the device (the reference default, usize::MAX).  An optimiser that holds more pages than
 * max_resident_pages keeps ALL of its state in pinned host memory; the step kernel then reads and writes the
 * pages in place over the host link (nothing of the state is resident on the device), or, with the environment
 * variable QLC_ADAM_PAGED_MODE=slots (hybrid), copies them through min(max_resident_pages, 8) device slots in both
 * directions (on the way in only).  Results are bit-identical in every mode. */
typedef struct qlc_adam_config {
    float lr;
    float beta1;
    float beta2;
    float eps;
    size_t block_size;
    size_t max_resident_pages;
} qlc_adam_config;
/* AdamStats (optim.rs:136-141). */
typedef struct qlc_adam_stats {
    size_t pages_streamed;
    size_t state_bytes;
} qlc_adam_stats;

/* AdamConfig::default (optim.rs:48-58). */
void qlc_adam_config_default(qlc_adam_config *cfg);
/* Adam8bit::new (optim.rs:155-161; validation :61-80). */
int qlc_adam_create(qlc_ctx *ctx, const qlc_adam_config *cfg, qlc_adam **out);
int qlc_adam_destroy(qlc_adam *opt);
/* Adam8bit::step (optim.rs:164-199) on HOST parameter / gradient slices: params[i] has
 * param_lens[i] values and is updated in place; grads[i] has grad_lens[i] values. */
int qlc_adam_step(qlc_adam *opt, size_t n_tensors, float *const *params, const size_t *param_lens,
                  const float *const *grads, const size_t *grad_lens, qlc_adam_stats *stats);
/* Same on DEVICE parameter / gradient buffers (lens[i] values each); asynchronous. */
int qlc_adam_step_dev(qlc_adam *opt, size_t n_tensors, float *const *d_params, const float *const *d_grads,
                      const size_t *lens, qlc_adam_stats *stats);
/* Arithmetic of the step kernel (no counterpart in the reference).  Default (0): every operation of
 * optim.rs:227-241 is reproduced with IEEE rounding in the reference's order - parameters and 8-bit state
 * are bit-identical to qlora-core.  1: hardware reciprocal / square-root approximations and fused
 * multiply-adds - parameters agree to ~1e-6 relative per step, state codes differ only next to rounding
 * boundaries, and the kernel runs at memory speed.  Applies to tensors with block_size 256. */
int qlc_adam_set_fast_math(qlc_adam *opt, int enable);
/* Adam8bit::state_bytes (optim.rs:201-204). */
size_t qlc_adam_state_bytes(const qlc_adam *opt);
/* Raw state of tensor `index` (ParamState, optim.rs:104-112), for checkpointing and tests:
 * m_codes/v_codes have numel bytes, m_scales/v_scales have ceil(numel/block_size) floats.
 * Any output pointer may be NULL. */
int qlc_adam_get_state(qlc_adam *opt, size_t index, size_t *numel, uint64_t *step, uint8_t *m_codes,
                       uint8_t *v_codes, float *m_scales, float *v_scales);
/* Restores the raw state of tensor `index` (the inverse of qlc_adam_get_state; ParamState, optim.rs:104-126):
 * numel elements, the tensor's step counter, and the four arrays with the lengths qlc_adam_get_state
 * documents.  States are restored in order: `index` may name an existing state (replaced, re-created when
 * numel differs) or the next one to be created.  A step after restoring continues bit for bit as if the
 * optimiser had never been saved.  (The reference keeps ParamState private and has no save / restore.) */
int qlc_adam_set_state(qlc_adam *opt, size_t index, size_t numel, uint64_t step, const uint8_t *m_codes,
                       const uint8_t *v_codes, const float *m_scales, const float *v_scales);
/* Bytes of optimiser state currently resident in device memory / parked in pinned host memory,
 * and the number of bytes the last step moved over the host link in each direction. */
int qlc_adam_paging_info(const qlc_adam *opt, size_t *device_bytes, size_t *host_bytes, size_t *h2d_bytes_last_step,
                         size_t *d2h_bytes_last_step);

/* ---- multi-GPU (token rows sharded across ranks, W_q / A / B replicated) ------------- */

/* Sum-all-reduce of the concatenated LoRA gradients is done by the host framework's NCCL
 * communicator on the buffers returned here: one contiguous fp32 device bucket holding
 * grad_a (r*in_dim) followed by grad_b (out_dim*r), owned by the layer, which
 * qlc_qlora_backward_dev fills when d_grad_a == qlc_layer_grad_bucket(...) is passed.
 * (No counterpart in the reference: it has no multi-device path.) */
int qlc_layer_grad_bucket(qlc_layer *layer, float **d_bucket, size_t *n_floats);

/* The exchange step for hosts without a communicator of their own: NCCL (loaded with dlopen at first use;
 * QLC_NCCL_LIBRARY overrides the library path), one communicator per context, all-reduce in stream order on
 * qlc_ctx_stream(ctx).  Rank 0 creates the id and passes its QLC_COMM_ID_BYTES bytes to the other ranks by
 * any host channel; every rank then calls qlc_comm_init (collective).  Failures are QLC_ERR_GPU.
 * A process keeps one libnccl.so.2: if a framework with its own NCCL (PyTorch) is loaded too, load it first.
 * (No counterpart in the reference: it has no multi-device path.) */
#define QLC_COMM_ID_BYTES 128
typedef struct qlc_comm qlc_comm;
int qlc_comm_unique_id(unsigned char *id_out, size_t id_len);
int qlc_comm_init(qlc_ctx *ctx, int nranks, int rank, const unsigned char *id, size_t id_len, qlc_comm **out);
/* In-place sum over ranks of `count` floats at d_buf (device pointer). */
int qlc_comm_allreduce_sum_f32(qlc_comm *comm, float *d_buf, size_t count);
/* In-place sum over ranks of the layer's grad_a || grad_b bucket (qlc_layer_grad_bucket). */
int qlc_allreduce_lora_grads(qlc_comm *comm, qlc_layer *layer);
/* The same sum for n buffers at once (d_bufs[i] holds counts[i] floats), issued as one NCCL group so that the
 * library can fuse them into few launches; stream-ordered on the communicator's context. */
int qlc_comm_allreduce_sum_f32_many(qlc_comm *comm, float *const *d_bufs, const size_t *counts, size_t n);
/* Number of ranks of the communicator (0 for a null handle) and the context it was created on. */
int qlc_comm_nranks(const qlc_comm *comm);
qlc_ctx *qlc_comm_context(const qlc_comm *comm);
int qlc_comm_destroy(qlc_comm *comm);

/* ---- one training step of a layer, entirely on the device ------------------------------ */

/* backward (gradients into the layer's bucket) -> sum over ranks when `comm` is not NULL -> 8-bit Adam on the
 * layer's A and B in place (tensor 0 = A, tensor 1 = B of `adam`, which must be used for this layer only) ->
 * refresh of the operand copies.  Everything is stream-ordered on qlc_ctx_stream(ctx); nothing returns to the
 * host.  One call replaces the body of the reference's training loop after the loss
 * (qlora-core/examples/train_lora.rs:41-46: backward, collect grads, opt.step, rebuild the layer). */
int qlc_train_step_dev(qlc_ctx *ctx, qlc_layer *layer, qlc_adam *adam, qlc_comm *comm, const void *d_x,
                       const void *d_dy, int dtype, size_t batch, void *d_grad_x);

/* ---- the caller of the path: Llama decoder with QLoRA adapters (qlora-model/src/llama.rs) ------- */

/* LlamaConfig (llama.rs:13-43).  Head dimension hidden/heads must be 64. */
typedef struct qlc_llama_config {
    size_t hidden, layers, heads, kv_heads, intermediate, vocab;
    float rms_eps, rope_theta;
} qlc_llama_config;
/* ProjKind (llama.rs:44-54) */
#define QLC_LLAMA_Q 0
#define QLC_LLAMA_K 1
#define QLC_LLAMA_V 2
#define QLC_LLAMA_O 3
#define QLC_LLAMA_GATE 4
#define QLC_LLAMA_UP 5
#define QLC_LLAMA_DOWN 6
#define QLC_LLAMA_PROJ_COUNT 7
typedef struct qlc_llama qlc_llama; /* replaces qlora_model::LlamaModel (llama.rs:167-172) */

/* embed: (vocab, hidden) fp32, also the tied LM head; final_norm: (hidden).  Replaces LlamaModel::from_tensors
 * (llama.rs:203-307) together with qlc_llama_set_layer / qlc_llama_attach_adapter. */
int qlc_llama_create(qlc_ctx *ctx, const qlc_llama_config *cfg, const float *embed, const float *final_norm,
                     qlc_llama **out);
int qlc_llama_destroy(qlc_llama *model);
/* weights[QLC_LLAMA_*]: the seven (out, in) fp32 matrices of the block (llama.rs:250-297); every one is
 * NF4-quantised on the GPU (the reference quantises only adapter targets and keeps the others in fp32). */
int qlc_llama_set_layer(qlc_llama *model, size_t layer, const float *attn_norm, const float *mlp_norm,
                        const float *const *weights, size_t block_size, int double_quant);
/* Same, quantising only the projections with quantize[QLC_LLAMA_*] != 0; the others stay frozen fp32 matrices
 * (Proj::Raw, llama.rs:87-93, 236-238: the reference quantises only adapter targets) and are multiplied as they
 * are: in fp32 in the FP32_EXACT and TF32 modes, rounded to bf16 on the tensor-core path. */
int qlc_llama_set_layer_mixed(qlc_llama *model, size_t layer, const float *attn_norm, const float *mlp_norm,
                              const float *const *weights, const int *quantize, size_t block_size, int double_quant);
/* a: (r, in), b: (out, r) of the adapter on projection `kind` (llama.rs:228-242).  A raw projection is quantised
 * first (block 64, double quantisation: QuantConfig::default()), as the reference's loader does for targets. */
int qlc_llama_attach_adapter(qlc_llama *model, size_t layer, int kind, const float *a, const float *b, size_t r,
                             float alpha);
qlc_layer *qlc_llama_projection(qlc_llama *model, size_t layer, int kind);
/* LlamaModel::forward (llama.rs:310-326) for n_seq sequences of seq_len token ids (ids: n_seq*seq_len host
 * values); logits: host (n_seq*seq_len, vocab) or NULL. */
int qlc_llama_forward(qlc_llama *model, const uint32_t *ids, size_t n_seq, size_t seq_len, float *logits);
/* LlamaModel::backward (llama.rs:385-412): dlogits host (n_seq*seq_len, vocab); the adapter gradients are left
 * in each adapter layer's gradient bucket (qlc_llama_adapter_grads / qlc_layer_grad_bucket). */
int qlc_llama_backward(qlc_llama *model, const uint32_t *ids, const float *dlogits, size_t n_seq, size_t seq_len);
/* forward, softmax cross-entropy against `targets` averaged over all positions (llama.rs:487-514), backward;
 * logits and dlogits never leave the device. */
int qlc_llama_loss_backward(qlc_llama *model, const uint32_t *ids, const uint32_t *targets, size_t n_seq,
                            size_t seq_len, float *loss);
/* qlc_llama_loss_backward + one 8-bit Adam step over all adapter matrices in the reference loop's order (layers
 * reversed, projections in kind order, A then B: qlora-model/examples/train_smollm.rs:42-72) + operand refresh. */
int qlc_llama_train_step(qlc_llama *model, qlc_adam *adam, const uint32_t *ids, const uint32_t *targets, size_t n_seq,
                         size_t seq_len, float *loss);
/* The data-parallel form of qlc_llama_train_step: every rank runs it on its own sequences (the same n_seq and
 * seq_len on every rank).  The loss gradient is scaled by 1 / (tokens of ALL ranks), the adapter gradients of
 * all layers are summed over the ranks of `comm` (one NCCL group, stream-ordered after the backward pass), and
 * every rank then takes the same optimiser step, so adapters that start equal stay equal.  `comm` must live on
 * the model's context.  *loss is the mean over this rank's tokens. */
int qlc_llama_train_step_dp(qlc_llama *model, qlc_adam *adam, qlc_comm *comm, const uint32_t *ids, const uint32_t *targets,
                            size_t n_seq, size_t seq_len, float *loss);
int qlc_llama_adapter_grads(qlc_llama *model, size_t layer, int kind, float *grad_a, float *grad_b);
int qlc_llama_adapter_weights(qlc_llama *model, size_t layer, int kind, float *a, float *b);

/* ---- self-tests (no counterpart in the reference) ----------------------------------------------------- */

/* Runs the quantise kernels' code-selection routine (15 decision thresholds on the divided target) over the
 * `count` consecutive fp32 bit patterns starting at `first_bits`, read as targets t = w / absmax, and returns
 * the codes two per byte (pattern first_bits + 2i in the low nibble of out[i]); out_len == ceil(count / 2).
 * The parity tests compare this with the 16-way scan of qlora-core/src/quant.rs:263-278 for EVERY target in
 * [-1, 1]. */
int qlc_selftest_nf4_codes_of_targets(qlc_ctx *ctx, uint32_t first_bits, size_t count, uint8_t *out, size_t out_len);
/* Runs the block-64 quantise kernel's fast code selection (approximate quotient w * rcp(absmax), 32-bin table,
 * exact redo inside a guard band around the bin's threshold) for every weight bit pattern in
 * [first_bits, first_bits + count) against the block absmax `absmax`, and compares each code with the code of
 * the IEEE quotient w / absmax (what quant.rs:264 computes), on the device.  Returns the number of differing
 * weights (must be 0), the number of 8-weight groups that took the exact redo, and the first differing bit
 * pattern. */
int qlc_selftest_nf4_fast_path(qlc_ctx *ctx, float absmax, uint32_t first_bits, uint64_t count, uint64_t *mismatches,
                               uint64_t *redone, uint32_t *first_mismatch_bits);
/* The exact Adam kernel computes its per-element square roots and its division with branch-free sequences
 * (hardware approximation + exact FMA residual corrections) when all operands lie in the middle of the exponent
 * range, and with the IEEE intrinsics otherwise.  This compares the two on the device:
 *   which == 0: the square-root sequence against the IEEE square root for the `count` fp32 bit patterns from
 *               `first_bits` (the kernel uses it for values in [2^-80, 2^80]; the tests sweep all of them);
 *   which == 1: the division sequence against IEEE division for `count` operand pairs from a seeded generator
 *               covering the kernel's operand windows (|numerator| in [2^-70, 2^70], denominator in [2^-40, 2^41]).
 * Returns the number of differing results (must be 0) and the index of the first. */
int qlc_selftest_adam_math(qlc_ctx *ctx, int which, uint32_t first_bits, uint64_t count, uint64_t seed,
                           uint64_t *mismatches, uint64_t *first_mismatch);
/* Failure-path test: enqueues a one-CTA kernel (no TMA, no tensor memory) whose thread 0 waits, with the
 * bounded wait of the tensor-core kernels, on an mbarrier nobody arrives on.  After `limit_cycles` SM clock
 * cycles (1 .. 1e8) the wait gives up, stores (code 1, site 99, block 0) in the context's status word and the
 * kernel returns normally.  Tensor-core kernels queued behind it return at once; the next
 * qlc_ctx_synchronize fails with QLC_ERR_GPU naming the site, clears the status, and the context works again. */
int qlc_selftest_wait_timeout(qlc_ctx *ctx, uint64_t limit_cycles);

#ifdef __cplusplus
}
#endif
#endif /* QLORA_CUDA_H_ */
