// C-ABI entry points: contexts, quantised tensors, QloraLinear layers and the host-pointer
// wrappers.  Host-side validation mirrors the reference's checks and error kinds
// (qlora-core/src/{quant,lora,qlora}.rs; cited per function in include/qlora_cuda.h).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>
#include <string>

#include "common.cuh"

namespace qlc {

static thread_local std::string t_last_error;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    // Display prefixes of QloraError (qlora-core/src/error.rs:17-23).
    const char *prefix = code == QLC_ERR_SHAPE_MISMATCH ? "shape mismatch: "
                         : code == QLC_ERR_INVALID_CONFIG ? "invalid config: "
                                                          : "gpu error: ";
    t_last_error = std::string(prefix) + buf;
    return code;
}

int ctx_workspace(qlc_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->ws_bytes) {
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->ws) cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
        const size_t want = (bytes + (1u << 20)) & ~(size_t)((1u << 20) - 1);
        QLC_CUDA(cudaMalloc(&ctx->ws, want));
        ctx->ws_bytes = want;
    }
    *out = ctx->ws;
    return QLC_OK;
}

int ctx_pinned(qlc_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->pin_bytes) {
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->pin) cudaFreeHost(ctx->pin);
        ctx->pin = nullptr;
        ctx->pin_bytes = 0;
        QLC_CUDA(cudaHostAlloc(&ctx->pin, bytes, cudaHostAllocDefault));
        ctx->pin_bytes = bytes;
    }
    *out = ctx->pin;
    return QLC_OK;
}

// Zeroed counters for kernels whose last-arriving CTA finishes a tile; every such kernel leaves them zero.
// Two sets, because a kernel of each kind may be in flight at the same time (main and side stream).
int ctx_tile_counters(qlc_ctx *ctx, int set, size_t count, int **out) {
    if (count > ctx->tile_counters_cap[set]) {
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->d_tile_counters[set]) cudaFree(ctx->d_tile_counters[set]);
        ctx->d_tile_counters[set] = nullptr;
        ctx->tile_counters_cap[set] = 0;
        const size_t want = (count + 1023) & ~(size_t)1023;
        QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&ctx->d_tile_counters[set]), want * sizeof(int)));
        QLC_CUDA(cudaMemset(ctx->d_tile_counters[set], 0, want * sizeof(int)));
        ctx->tile_counters_cap[set] = want;
    }
    *out = ctx->d_tile_counters[set];
    return QLC_OK;
}

// Waits (on the host) until the copies of earlier asynchronous host-buffer submissions have ended: they run on the
// copy streams, which the context's main stream does not cover.
static int fused_quiesce(qlc_ctx *ctx) {
    if (!ctx->fused_open) return QLC_OK;
    QLC_CUDA(cudaStreamSynchronize(ctx->copy_stream));
    QLC_CUDA(cudaStreamSynchronize(ctx->d2h_stream));
    ctx->fused_open = false;
    return QLC_OK;
}

static int ctx_io_grow(qlc_ctx *ctx, size_t bytes);
int ctx_io(qlc_ctx *ctx, size_t bytes, void **out) {
    QLC_TRY(fused_quiesce(ctx));  // the staging area is about to be reused by a synchronous entry point
    QLC_TRY(ctx_io_grow(ctx, bytes));
    *out = ctx->io;
    return QLC_OK;
}
static int ctx_io_grow(qlc_ctx *ctx, size_t bytes) {
    if (bytes > ctx->io_bytes) {
        QLC_TRY(fused_quiesce(ctx));
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->io) cudaFree(ctx->io);
        ctx->io = nullptr;
        ctx->io_bytes = 0;
        const size_t want = (bytes + (1u << 20)) & ~(size_t)((1u << 20) - 1);
        QLC_CUDA(cudaMalloc(&ctx->io, want));
        ctx->io_bytes = want;
    }
    return QLC_OK;
}

static cudaEvent_t prof_event(qlc_ctx *ctx) {
    if (!ctx->prof_pool.empty()) {
        cudaEvent_t e = ctx->prof_pool.back();
        ctx->prof_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

void prof_begin(qlc_ctx *ctx, int slot, cudaStream_t stream) {
    if (!ctx->profiling) return;
    qlc_ctx::ProfEvent pe{slot, prof_event(ctx), prof_event(ctx)};
    cudaEventRecord(pe.start, stream ? stream : ctx->stream);
    ctx->prof_pending.push_back(pe);
}

void prof_end(qlc_ctx *ctx, cudaStream_t stream) {
    if (!ctx->profiling || ctx->prof_pending.empty()) return;
    cudaEventRecord(ctx->prof_pending.back().stop, stream ? stream : ctx->stream);
}

namespace {

// A temporary device buffer for the synchronous host-pointer entry points.
struct DevBuf {
    void *p = nullptr;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    int alloc(size_t bytes) {
        QLC_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
        return QLC_OK;
    }
    template <class T> T *as() { return static_cast<T *>(p); }
};

int sync_and_check(qlc_ctx *ctx) {
    QLC_TRY(fused_quiesce(ctx));
    QLC_CUDA(cudaStreamSynchronize(ctx->stream));
    DeviceStatus s;
    QLC_CUDA(cudaMemcpy(&s, ctx->d_status, sizeof(s), cudaMemcpyDeviceToHost));
    if (s.code != 0) {
        QLC_CUDA(cudaMemset(ctx->d_status, 0, sizeof(DeviceStatus)));
        return fail(QLC_ERR_GPU, "kernel reported status %d at site %d (block %d, detail %d)", s.code, s.where,
                    s.block, s.detail);
    }
    return QLC_OK;
}

bool mul_overflows(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }

}  // namespace

int alloc_qtensor(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, bool dq, qlc_qtensor **out) {
    qlc_qtensor *q = new (std::nothrow) qlc_qtensor();
    if (!q) return fail(QLC_ERR_GPU, "out of host memory");
    q->device = ctx->device;
    q->rows = rows;
    q->cols = cols;
    q->block_size = block_size;
    q->n = rows * cols;
    q->nb = ceil_div(q->n, block_size);
    q->dq = dq;
    const size_t codes_len = (q->n + 1) / 2;
    const size_t codes_alloc = ((codes_len + 15) & ~(size_t)15) + 16;  // whole 128-bit reads stay in bounds
    int st = QLC_OK;
    auto chk = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == QLC_OK) st = fail(QLC_ERR_GPU, "%s: %s", what, cudaGetErrorString(e));
    };
    chk(cudaMalloc(&q->d_codes, codes_alloc), "cudaMalloc(codes)");
    if (st == QLC_OK) chk(cudaMemsetAsync(q->d_codes, 0, codes_alloc, ctx->stream), "cudaMemset(codes)");
    if (dq) {
        if (st == QLC_OK) chk(cudaMalloc(&q->d_absmax_codes, q->nb + 16), "cudaMalloc(absmax codes)");
        if (st == QLC_OK)
            chk(cudaMalloc(&q->d_absmax2, (ceil_div(q->nb, kDoubleQuantBlock) + 1) * sizeof(float)),
                "cudaMalloc(absmax2)");
    } else {
        if (st == QLC_OK) chk(cudaMalloc(&q->d_scales_f32, (q->nb + 1) * sizeof(float)), "cudaMalloc(scales)");
    }
    if (st != QLC_OK) {
        qlc_qtensor_destroy(q);
        return st;
    }
    *out = q;
    return QLC_OK;
}

namespace {

void qtensor_retain(qlc_qtensor *q) { q->refs += 1; }

}  // namespace
// The fp32 (tf32-rounded) padded adapter copies of the TF32 mode: created on first use, refreshed after
// every change of A / B.
int layer_tf32_operands(qlc_layer *L) {
    if (L->r == 0 || L->pad32_valid) return QLC_OK;
    if (!L->d_a_pad32) {
        QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&L->d_a_pad32), (L->r_pad * L->in_dim + 4) * 4));
        QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&L->d_b_pad32), (L->out_dim * L->r_pad + 4) * 4));
        QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&L->d_bt_pad32), (L->out_dim * L->r_pad + 4) * 4));
    }
    QLC_TRY(launch_pad_to_tf32(L->ctx, L->d_a, L->r, L->in_dim, L->d_a_pad32, L->r_pad, L->in_dim, 0));
    QLC_TRY(launch_pad_to_tf32(L->ctx, L->d_b, L->out_dim, L->r, L->d_b_pad32, L->out_dim, L->r_pad, 0));
    QLC_TRY(launch_pad_to_tf32(L->ctx, L->d_b, L->out_dim, L->r, L->d_bt_pad32, L->r_pad, L->out_dim, 1));
    L->pad32_valid = true;
    return QLC_OK;
}

int layer_create_raw(qlc_ctx *ctx, const float *d_weight, size_t out_dim, size_t in_dim, qlc_layer **out) {
    qlc_layer *L = new (std::nothrow) qlc_layer();
    if (!L) return fail(QLC_ERR_GPU, "out of host memory");
    L->ctx = ctx;
    ctx->refs += 1;
    L->in_dim = in_dim;
    L->out_dim = out_dim;
    const size_t n = out_dim * in_dim;
    int st = QLC_OK;
    if (cudaMalloc(reinterpret_cast<void **>(&L->d_w_raw), (n + 4) * 4) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void **>(&L->d_w_raw_bf16), (n + 8) * 2) != cudaSuccess)
        st = fail(QLC_ERR_GPU, "out of device memory for a raw (%zu, %zu) projection", out_dim, in_dim);
    if (st == QLC_OK && n &&
        cudaMemcpyAsync(L->d_w_raw, d_weight, n * 4, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
        st = fail(QLC_ERR_GPU, "copy of the raw weight failed");
    if (st == QLC_OK) st = launch_convert_f32_to_bf16(ctx, L->d_w_raw, L->d_w_raw_bf16, n);
    if (st != QLC_OK) {
        qlc_layer_destroy(L);
        return st;
    }
    *out = L;
    return QLC_OK;
}

}  // namespace qlc

using namespace qlc;

extern "C" {

const char *qlc_last_error_message(void) { return t_last_error.c_str(); }

int qlc_ctx_create(int device, qlc_ctx **out) {
    if (!out) return fail(QLC_ERR_INVALID_CONFIG, "null output pointer");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(QLC_ERR_GPU, "no usable CUDA device (%s); this library has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    if (device < 0 || device >= count) return fail(QLC_ERR_GPU, "device %d out of range (count %d)", device, count);
    QLC_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    QLC_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(QLC_ERR_GPU, "device %d is sm_%d%d; this library is built for sm_100a (B200) only", device,
                    prop.major, prop.minor);
    qlc_ctx *ctx = new (std::nothrow) qlc_ctx();
    if (!ctx) return fail(QLC_ERR_GPU, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->umma_smem_optin = (int)prop.sharedMemPerBlockOptin;
    // The context's stream outranks its side stream: thread blocks of a kernel on the side stream only take
    // SMs that no pending block of the main stream's kernels can use (the last, partial wave of a weight GEMM).
    int prio_least = 0, prio_greatest = 0;
    QLC_CUDA(cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest));
    QLC_CUDA(cudaStreamCreateWithPriority(&ctx->stream, cudaStreamNonBlocking, prio_greatest));
    QLC_CUDA(cudaStreamCreateWithPriority(&ctx->side_stream, cudaStreamNonBlocking, prio_least));
    QLC_CUDA(cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming));
    QLC_CUDA(cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming));
    QLC_CUDA(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    QLC_CUDA(cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    for (int p = 0; p < 2; ++p) {
        QLC_CUDA(cudaEventCreateWithFlags(&ctx->ev_in_free[p], cudaEventDisableTiming));
        QLC_CUDA(cudaEventCreateWithFlags(&ctx->ev_out_free[p], cudaEventDisableTiming));
    }
    QLC_CUDA(cudaMalloc(&ctx->d_status, sizeof(DeviceStatus)));
    QLC_CUDA(cudaMemset(ctx->d_status, 0, sizeof(DeviceStatus)));
    *out = ctx;
    return QLC_OK;
}

int qlc_ctx_destroy(qlc_ctx *ctx) {
    if (!ctx) return QLC_OK;
    // Layers and optimisers keep their context alive: the storage is released with the last reference.
    if (--ctx->refs > 0) return QLC_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamSynchronize(ctx->d2h_stream);  // copies out of asynchronous host-buffer submissions read the staging area
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->io) cudaFree(ctx->io);
    for (auto &pe : ctx->prof_pending) {
        cudaEventDestroy(pe.start);
        cudaEventDestroy(pe.stop);
    }
    for (cudaEvent_t e : ctx->prof_pool) cudaEventDestroy(e);
    if (ctx->pin) cudaFreeHost(ctx->pin);
    if (ctx->d_status) cudaFree(ctx->d_status);
    for (int p = 0; p < 2; ++p) {
        cudaEventDestroy(ctx->ev_in_free[p]);
        cudaEventDestroy(ctx->ev_out_free[p]);
    }
    cudaStreamDestroy(ctx->stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaStreamSynchronize(ctx->d2h_stream);
    cudaStreamDestroy(ctx->d2h_stream);
    cudaStreamSynchronize(ctx->side_stream);
    cudaStreamDestroy(ctx->side_stream);
    cudaEventDestroy(ctx->ev_fork);
    cudaEventDestroy(ctx->ev_join);
    for (cudaEvent_t e : ctx->chunk_events) cudaEventDestroy(e);
    for (cudaEvent_t e : ctx->ticket_ev)
        if (e) cudaEventDestroy(e);
    for (int *p : ctx->d_tile_counters)
        if (p) cudaFree(p);
    delete ctx;
    return QLC_OK;
}

int qlc_ctx_set_precision(qlc_ctx *ctx, int precision) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (precision < QLC_PRECISION_AUTO || precision > QLC_PRECISION_TF32)
        return fail(QLC_ERR_INVALID_CONFIG, "unknown precision %d", precision);
    ctx->precision = precision;
    return QLC_OK;
}

int qlc_ctx_set_reserved_sms(qlc_ctx *ctx, int sms) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (sms < 0 || sms > ctx->sm_count / 2)
        return fail(QLC_ERR_INVALID_CONFIG, "reserved SMs must be in [0, %d]", ctx->sm_count / 2);
    ctx->reserved_sms = sms & ~1;  // whole pairs
    return QLC_OK;
}

int qlc_ctx_synchronize(qlc_ctx *ctx) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    QLC_CUDA(cudaSetDevice(ctx->device));
    return sync_and_check(ctx);
}

int qlc_ctx_profile_enable(qlc_ctx *ctx, int enable) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    ctx->profiling = enable != 0;
    return QLC_OK;
}

int qlc_ctx_profile_read(qlc_ctx *ctx, int slot, double *total_ms, uint64_t *launches) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (slot < 0 || slot >= QLC_PROFILE_SLOTS) return fail(QLC_ERR_INVALID_CONFIG, "profile slot %d out of range", slot);
    QLC_CUDA(cudaSetDevice(ctx->device));
    QLC_CUDA(cudaStreamSynchronize(ctx->stream));
    for (auto &pe : ctx->prof_pending) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, pe.start, pe.stop) == cudaSuccess) {
            ctx->prof_ms[pe.slot] += ms;
            ctx->prof_launches[pe.slot] += 1;
        }
        ctx->prof_pool.push_back(pe.start);
        ctx->prof_pool.push_back(pe.stop);
    }
    ctx->prof_pending.clear();
    if (total_ms) *total_ms = ctx->prof_ms[slot];
    if (launches) *launches = ctx->prof_launches[slot];
    ctx->prof_ms[slot] = 0.0;
    ctx->prof_launches[slot] = 0;
    return QLC_OK;
}

int qlc_ctx_copy_to_host(qlc_ctx *ctx, void *dst, const void *d_src, size_t bytes) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (bytes == 0) return QLC_OK;
    if (!dst || !d_src) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    QLC_CUDA(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return QLC_OK;
}

int qlc_ctx_copy_to_device(qlc_ctx *ctx, void *d_dst, const void *src, size_t bytes) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (bytes == 0) return QLC_OK;
    if (!d_dst || !src) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    QLC_CUDA(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return QLC_OK;
}

void *qlc_ctx_stream(qlc_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
uint64_t qlc_ctx_launch_count(const qlc_ctx *ctx) { return ctx ? ctx->launches : 0; }

// ---- quantised tensors -----------------------------------------------------------------------

static int quantize_common(qlc_ctx *ctx, const float *weights, bool on_device, size_t weights_len, size_t rows,
                           size_t cols, size_t block_size, int double_quant, qlc_qtensor **out) {
    if (!ctx || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (block_size == 0) return fail(QLC_ERR_INVALID_CONFIG, "block_size must be > 0");  // quant.rs:72-79
    size_t n = 0;
    if (mul_overflows(rows, cols, &n)) return fail(QLC_ERR_INVALID_CONFIG, "rows*cols overflow");  // :111-113
    if (!on_device && weights_len != n)
        return fail(QLC_ERR_SHAPE_MISMATCH, "weights.len() = %zu but rows*cols = %zu", weights_len, n);  // :114-119
    if (n && !weights) return fail(QLC_ERR_INVALID_CONFIG, "null weights");
    QLC_CUDA(cudaSetDevice(ctx->device));
    qlc_qtensor *q = nullptr;
    QLC_TRY(alloc_qtensor(ctx, rows, cols, block_size, double_quant != 0, &q));
    int st = QLC_OK;
    if (on_device) {
        st = launch_quantize_nf4(ctx, weights, q);
    } else {
        DevBuf w;
        st = w.alloc(n * sizeof(float));
        if (st == QLC_OK && n) {
            cudaError_t e = cudaMemcpyAsync(w.p, weights, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
            if (e != cudaSuccess) st = fail(QLC_ERR_GPU, "cudaMemcpyAsync(weights): %s", cudaGetErrorString(e));
        }
        if (st == QLC_OK) st = launch_quantize_nf4(ctx, w.as<float>(), q);
        if (st == QLC_OK) st = sync_and_check(ctx);
    }
    if (st != QLC_OK) {
        qlc_qtensor_destroy(q);
        return st;
    }
    *out = q;
    return QLC_OK;
}

int qlc_quantize_nf4(qlc_ctx *ctx, const float *weights, size_t weights_len, size_t rows, size_t cols,
                     size_t block_size, int double_quant, qlc_qtensor **out) {
    return quantize_common(ctx, weights, false, weights_len, rows, cols, block_size, double_quant, out);
}

int qlc_quantize_nf4_typed(qlc_ctx *ctx, const void *weights, int dtype, size_t rows, size_t cols, size_t block_size,
                           int double_quant, qlc_qtensor **out) {
    if (!ctx || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16 && dtype != QLC_DTYPE_F16)
        return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    size_t n = 0;
    if (mul_overflows(rows, cols, &n)) return fail(QLC_ERR_INVALID_CONFIG, "rows*cols overflow");  // quant.rs:111-113
    if (dtype == QLC_DTYPE_F32) return qlc_quantize_nf4(ctx, static_cast<const float *>(weights), n, rows, cols, block_size, double_quant, out);
    if (block_size == 0) return fail(QLC_ERR_INVALID_CONFIG, "block_size must be > 0");  // quant.rs:72-79
    if (n && !weights) return fail(QLC_ERR_INVALID_CONFIG, "null weights");
    QLC_CUDA(cudaSetDevice(ctx->device));
    void *raw = nullptr;
    float *wide = nullptr;
    QLC_CUDA(cudaMalloc(&raw, n * 2 + 16));
    if (cudaMalloc(reinterpret_cast<void **>(&wide), n * 4 + 16) != cudaSuccess) {
        cudaFree(raw);
        return fail(QLC_ERR_GPU, "out of device memory for the widened weights (%zu bytes)", n * 4);
    }
    int st = QLC_OK;
    if (n && cudaMemcpyAsync(raw, weights, n * 2, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
        st = fail(QLC_ERR_GPU, "upload of the weights failed");
    if (st == QLC_OK)
        st = dtype == QLC_DTYPE_BF16 ? launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(raw), wide, n)
                                     : launch_convert_f16_to_f32(ctx, raw, wide, n);
    if (st == QLC_OK) st = quantize_common(ctx, wide, true, 0, rows, cols, block_size, double_quant, out);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(raw);
    cudaFree(wide);
    return st;
}

int qlc_quantize_nf4_dev(qlc_ctx *ctx, const float *d_weights, size_t rows, size_t cols, size_t block_size,
                         int double_quant, qlc_qtensor **out) {
    return quantize_common(ctx, d_weights, true, 0, rows, cols, block_size, double_quant, out);
}

int qlc_qtensor_requantize_dev(qlc_ctx *ctx, qlc_qtensor *q, const float *d_weights) {
    if (!ctx || !q) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (q->n && !d_weights) return fail(QLC_ERR_INVALID_CONFIG, "null weights");
    if (q->device != ctx->device) return fail(QLC_ERR_GPU, "tensor lives on device %d, context on %d", q->device, ctx->device);
    QLC_CUDA(cudaSetDevice(ctx->device));
    return launch_quantize_nf4(ctx, d_weights, q);
}

int qlc_qtensor_from_raw_parts(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, const uint8_t *codes,
                               size_t codes_len, const float *scales, size_t scales_len, qlc_qtensor **out) {
    if (!ctx || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (block_size == 0) return fail(QLC_ERR_INVALID_CONFIG, "block_size must be > 0");  // quant.rs:178-182
    size_t n = 0;
    if (mul_overflows(rows, cols, &n)) return fail(QLC_ERR_INVALID_CONFIG, "rows*cols overflow");
    if (codes_len != (n + 1) / 2)  // quant.rs:186-192
        return fail(QLC_ERR_SHAPE_MISMATCH, "codes.len() = %zu but ceil(rows*cols/2) = %zu", codes_len, (n + 1) / 2);
    if (scales_len != ceil_div(n, block_size))  // quant.rs:193-199
        return fail(QLC_ERR_SHAPE_MISMATCH, "scales.len() = %zu but ceil(rows*cols/block_size) = %zu", scales_len,
                    ceil_div(n, block_size));
    if ((codes_len && !codes) || (scales_len && !scales)) return fail(QLC_ERR_INVALID_CONFIG, "null payload");
    QLC_CUDA(cudaSetDevice(ctx->device));
    qlc_qtensor *q = nullptr;
    QLC_TRY(alloc_qtensor(ctx, rows, cols, block_size, false, &q));
    cudaError_t e = cudaSuccess;
    if (codes_len) e = cudaMemcpyAsync(q->d_codes, codes, codes_len, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && scales_len)
        e = cudaMemcpyAsync(q->d_scales_f32, scales, scales_len * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        qlc_qtensor_destroy(q);
        return fail(QLC_ERR_GPU, "upload of raw parts: %s", cudaGetErrorString(e));
    }
    *out = q;
    return QLC_OK;
}

int qlc_qtensor_from_double_quant_parts(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, const uint8_t *codes,
                                        size_t codes_len, const uint8_t *absmax_codes, size_t absmax_codes_len,
                                        const float *absmax2, size_t absmax2_len, qlc_qtensor **out) {
    if (!ctx || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (block_size == 0) return fail(QLC_ERR_INVALID_CONFIG, "block_size must be > 0");
    size_t n = 0;
    if (mul_overflows(rows, cols, &n)) return fail(QLC_ERR_INVALID_CONFIG, "rows*cols overflow");
    const size_t nb = ceil_div(n, block_size), n2 = ceil_div(nb, kDoubleQuantBlock);
    if (codes_len != (n + 1) / 2)
        return fail(QLC_ERR_SHAPE_MISMATCH, "codes.len() = %zu but ceil(rows*cols/2) = %zu", codes_len, (n + 1) / 2);
    if (absmax_codes_len != nb)
        return fail(QLC_ERR_SHAPE_MISMATCH, "absmax_codes.len() = %zu but ceil(rows*cols/block_size) = %zu",
                    absmax_codes_len, nb);
    if (absmax2_len != n2)
        return fail(QLC_ERR_SHAPE_MISMATCH, "absmax2.len() = %zu but ceil(num_blocks/256) = %zu", absmax2_len, n2);
    if ((codes_len && !codes) || (nb && !absmax_codes) || (n2 && !absmax2))
        return fail(QLC_ERR_INVALID_CONFIG, "null payload");
    QLC_CUDA(cudaSetDevice(ctx->device));
    qlc_qtensor *q = nullptr;
    QLC_TRY(alloc_qtensor(ctx, rows, cols, block_size, true, &q));
    cudaError_t e = cudaSuccess;
    if (codes_len) e = cudaMemcpyAsync(q->d_codes, codes, codes_len, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && nb) e = cudaMemcpyAsync(q->d_absmax_codes, absmax_codes, nb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && n2) e = cudaMemcpyAsync(q->d_absmax2, absmax2, n2 * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        qlc_qtensor_destroy(q);
        return fail(QLC_ERR_GPU, "upload of the payload: %s", cudaGetErrorString(e));
    }
    *out = q;
    return QLC_OK;
}

int qlc_qtensor_destroy(qlc_qtensor *q) {
    if (!q) return QLC_OK;
    if (--q->refs > 0) return QLC_OK;
    cudaSetDevice(q->device);
    cudaFree(q->d_codes);
    cudaFree(q->d_absmax_codes);
    cudaFree(q->d_absmax2);
    cudaFree(q->d_scales_f32);
    delete q;
    return QLC_OK;
}

int qlc_qtensor_get_info(const qlc_qtensor *q, qlc_qtensor_info *info) {
    if (!q || !info) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    info->rows = q->rows;
    info->cols = q->cols;
    info->block_size = q->block_size;
    info->num_elements = q->n;
    info->num_blocks = q->nb;
    info->codes_len = (q->n + 1) / 2;
    info->absmax2_len = q->dq ? ceil_div(q->nb, kDoubleQuantBlock) : 0;
    info->double_quant = q->dq ? 1 : 0;
    // quant.rs:229-235
    info->storage_bytes = info->codes_len + (q->dq ? q->nb + info->absmax2_len * 4 : q->nb * 4);
    return QLC_OK;
}

static int copy_out(const qlc_qtensor *q, const void *d_src, size_t want_bytes, void *out, size_t out_bytes,
                    const char *what) {
    if (out_bytes != want_bytes)
        return fail(QLC_ERR_SHAPE_MISMATCH, "%s: output holds %zu bytes but the tensor has %zu", what, out_bytes,
                    want_bytes);
    if (want_bytes == 0) return QLC_OK;
    if (!out) return fail(QLC_ERR_INVALID_CONFIG, "null output");
    QLC_CUDA(cudaSetDevice(q->device));
    QLC_CUDA(cudaMemcpy(out, d_src, want_bytes, cudaMemcpyDeviceToHost));
    return QLC_OK;
}

int qlc_qtensor_codes(const qlc_qtensor *q, uint8_t *out, size_t out_len) {
    if (!q) return fail(QLC_ERR_INVALID_CONFIG, "null tensor");
    return copy_out(q, q->d_codes, (q->n + 1) / 2, out, out_len, "codes");
}

int qlc_qtensor_absmax_codes(const qlc_qtensor *q, uint8_t *out, size_t out_len) {
    if (!q) return fail(QLC_ERR_INVALID_CONFIG, "null tensor");
    if (!q->dq) return fail(QLC_ERR_INVALID_CONFIG, "tensor is not double-quantized");
    return copy_out(q, q->d_absmax_codes, q->nb, out, out_len, "absmax codes");
}

int qlc_qtensor_absmax2(const qlc_qtensor *q, float *out, size_t out_len) {
    if (!q) return fail(QLC_ERR_INVALID_CONFIG, "null tensor");
    if (!q->dq) return fail(QLC_ERR_INVALID_CONFIG, "tensor is not double-quantized");
    const size_t n2 = ceil_div(q->nb, kDoubleQuantBlock);
    return copy_out(q, q->d_absmax2, n2 * 4, out, out_len * 4, "absmax2");
}

int qlc_qtensor_device_ptrs(const qlc_qtensor *q, const uint8_t **d_codes, const uint8_t **d_absmax_codes,
                            const float **d_absmax2, const float **d_scales_f32) {
    if (!q) return fail(QLC_ERR_INVALID_CONFIG, "null tensor");
    if (d_codes) *d_codes = q->d_codes;
    if (d_absmax_codes) *d_absmax_codes = q->d_absmax_codes;
    if (d_absmax2) *d_absmax2 = q->d_absmax2;
    if (d_scales_f32) *d_scales_f32 = q->d_scales_f32;
    return QLC_OK;
}

// The two getters below need a context (they launch a kernel); they use a private one-shot
// stream-less path: a temporary context-free launch on the legacy default stream is avoided by
// requiring a context in qlc_dequantize and by decoding scales through it as well.
int qlc_dequantize(qlc_ctx *ctx, const qlc_qtensor *q, float *out, size_t out_len) {
    if (!ctx || !q) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (out_len != q->n) return fail(QLC_ERR_SHAPE_MISMATCH, "out.len() = %zu but rows*cols = %zu", out_len, q->n);
    if (q->n == 0) return QLC_OK;  // kernels.rs:51-54
    if (!out) return fail(QLC_ERR_INVALID_CONFIG, "null output");
    QLC_CUDA(cudaSetDevice(ctx->device));
    DevBuf d;
    QLC_TRY(d.alloc(q->n * sizeof(float)));
    QLC_TRY(launch_dequantize(ctx, q, d.p, QLC_DTYPE_F32));
    QLC_CUDA(cudaMemcpyAsync(out, d.p, q->n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    return sync_and_check(ctx);
}

int qlc_dequantize_dev(qlc_ctx *ctx, const qlc_qtensor *q, void *d_out, int dtype) {
    if (!ctx || !q) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (q->n && !d_out) return fail(QLC_ERR_INVALID_CONFIG, "null output");
    QLC_CUDA(cudaSetDevice(ctx->device));
    return launch_dequantize(ctx, q, d_out, dtype);
}

int qlc_qtensor_block_scales(const qlc_qtensor *q, float *out, size_t out_len) {
    if (!q) return fail(QLC_ERR_INVALID_CONFIG, "null tensor");
    if (out_len != q->nb) return fail(QLC_ERR_SHAPE_MISMATCH, "out.len() = %zu but num_blocks = %zu", out_len, q->nb);
    if (q->nb == 0) return QLC_OK;
    if (!out) return fail(QLC_ERR_INVALID_CONFIG, "null output");
    if (!q->dq) return copy_out(q, q->d_scales_f32, q->nb * 4, out, out_len * 4, "scales");
    // Decode on the device with a throw-away context so the arithmetic is the kernels' own.
    qlc_ctx *ctx = nullptr;
    QLC_TRY(qlc_ctx_create(q->device, &ctx));
    DevBuf d;
    int st = d.alloc(q->nb * 4);
    if (st == QLC_OK) st = launch_decode_block_scales(ctx, q, d.as<float>());
    if (st == QLC_OK) {
        cudaError_t e = cudaMemcpyAsync(out, d.p, q->nb * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) st = fail(QLC_ERR_GPU, "cudaMemcpyAsync: %s", cudaGetErrorString(e));
    }
    if (st == QLC_OK) st = sync_and_check(ctx);
    qlc_ctx_destroy(ctx);
    return st;
}

// ---- plain GEMMs -------------------------------------------------------------------------------

typedef int (*exact_fn)(qlc_ctx *, const float *, const float *, size_t, size_t, size_t, float *);

static int host_gemm(qlc_ctx *ctx, exact_fn fn, const char *name, const float *a, size_t a_len, size_t a_want,
                     const float *b, size_t b_len, size_t b_want, size_t m, size_t k, size_t n, size_t c_len,
                     float *c) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (c_len == 0) return QLC_OK;  // kernels.rs:151-153 — empty output
    if (a_len != a_want || b_len != b_want)
        return fail(QLC_ERR_SHAPE_MISMATCH, "%s: a.len() = %zu, b.len() = %zu, expected %zu and %zu", name, a_len,
                    b_len, a_want, b_want);
    if (!c || (a_len && !a) || (b_len && !b)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    DevBuf da, db, dc;
    QLC_TRY(da.alloc(a_len * 4));
    QLC_TRY(db.alloc(b_len * 4));
    QLC_TRY(dc.alloc(c_len * 4));
    if (a_len) QLC_CUDA(cudaMemcpyAsync(da.p, a, a_len * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (b_len) QLC_CUDA(cudaMemcpyAsync(db.p, b, b_len * 4, cudaMemcpyHostToDevice, ctx->stream));
    QLC_TRY(fn(ctx, da.as<float>(), db.as<float>(), m, k, n, dc.as<float>()));
    QLC_CUDA(cudaMemcpyAsync(c, dc.p, c_len * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return sync_and_check(ctx);
}

int qlc_matmul(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k, size_t n,
               float *c) {
    return host_gemm(ctx, exact_matmul, "gpu_matmul", a, a_len, m * k, b, b_len, k * n, m, k, n, m * n, c);
}
int qlc_matmul_trans_b(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k,
                       size_t n, float *c) {
    return host_gemm(ctx, exact_matmul_trans_b, "gpu_matmul_trans_b", a, a_len, m * k, b, b_len, n * k, m, k, n,
                     m * n, c);
}
int qlc_matmul_trans_a(qlc_ctx *ctx, const float *a, size_t a_len, const float *b, size_t b_len, size_t m, size_t k,
                       size_t n, float *c) {
    return host_gemm(ctx, exact_matmul_trans_a, "gpu_matmul_trans_a", a, a_len, m * k, b, b_len, m * n, m, k, n,
                     k * n, c);
}

// ---- layers ----------------------------------------------------------------------------------------

static int refresh_padded_adapter(qlc_layer *L) {
    if (L->r == 0 || !L->d_a_pad) return QLC_OK;
    QLC_TRY(launch_pad_to_bf16(L->ctx, L->d_a, L->r, L->in_dim, L->d_a_pad, L->r_pad, L->in_dim));
    QLC_TRY(launch_pad_to_bf16(L->ctx, L->d_b, L->out_dim, L->r, L->d_b_pad, L->out_dim, L->r_pad));
    QLC_TRY(launch_pad_transpose_to_bf16(L->ctx, L->d_b, L->out_dim, L->r, L->d_bt_pad, L->r_pad, L->out_dim));
    L->pad32_valid = false;  // rebuilt by the next TF32-mode call
    L->shadow_valid = false; // and the padded copy's adapter matrices by the next tensor-core call
    return QLC_OK;
}


int qlc_layer_create(qlc_ctx *ctx, qlc_qtensor *weight, const float *a, size_t a_len, const float *b, size_t b_len,
                     size_t r, float alpha, qlc_layer **out) {
    if (!ctx || !weight || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    const size_t in_dim = weight->cols, out_dim = weight->rows;
    const bool has_adapter = (a != nullptr) || (b != nullptr);
    if (has_adapter) {
        if (!a || !b) return fail(QLC_ERR_INVALID_CONFIG, "lora_a and lora_b must be given together");
        if (r == 0) return fail(QLC_ERR_INVALID_CONFIG, "rank r must be > 0");  // lora.rs:36-38
        if (a_len != r * in_dim)                                                 // lora.rs:39-45
            return fail(QLC_ERR_SHAPE_MISMATCH, "a.len() = %zu but r*in_dim = %zu", a_len, r * in_dim);
        if (b_len != out_dim * r)                                                // lora.rs:46-52
            return fail(QLC_ERR_SHAPE_MISMATCH, "b.len() = %zu but out_dim*r = %zu", b_len, out_dim * r);
    } else {
        r = 0;
    }
    if (weight->device != ctx->device) return fail(QLC_ERR_GPU, "weight lives on device %d, context on %d", weight->device, ctx->device);
    QLC_CUDA(cudaSetDevice(ctx->device));
    qlc_layer *L = new (std::nothrow) qlc_layer();
    if (!L) return fail(QLC_ERR_GPU, "out of host memory");
    L->ctx = ctx;
    ctx->refs += 1;
    L->w = weight;
    qtensor_retain(weight);
    L->in_dim = in_dim;
    L->out_dim = out_dim;
    L->r = r;
    L->alpha = alpha;
    int st = QLC_OK;
    auto chk = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == QLC_OK) st = fail(QLC_ERR_GPU, "%s: %s", what, cudaGetErrorString(e));
    };
    if (r > 0) {
        L->r_pad = (r + 63) / 64 * 64;
        chk(cudaMalloc(&L->d_a, (r * in_dim + 1) * 4), "cudaMalloc(A)");
        chk(cudaMalloc(&L->d_b, (out_dim * r + 1) * 4), "cudaMalloc(B)");
        chk(cudaMalloc(&L->d_a_pad, (L->r_pad * in_dim + 8) * 2), "cudaMalloc(A bf16)");
        chk(cudaMalloc(&L->d_b_pad, (out_dim * L->r_pad + 8) * 2), "cudaMalloc(B bf16)");
        chk(cudaMalloc(&L->d_bt_pad, (out_dim * L->r_pad + 8) * 2), "cudaMalloc(B^T bf16)");
        chk(cudaMalloc(&L->d_grad_bucket, (r * in_dim + out_dim * r + 1) * 4), "cudaMalloc(grad bucket)");
        if (st == QLC_OK && a_len) chk(cudaMemcpyAsync(L->d_a, a, a_len * 4, cudaMemcpyHostToDevice, ctx->stream), "upload A");
        if (st == QLC_OK && b_len) chk(cudaMemcpyAsync(L->d_b, b, b_len * 4, cudaMemcpyHostToDevice, ctx->stream), "upload B");
        if (st == QLC_OK) st = refresh_padded_adapter(L);
        if (st == QLC_OK) st = sync_and_check(ctx);
    }
    if (st != QLC_OK) {
        qlc_layer_destroy(L);
        return st;
    }
    *out = L;
    return QLC_OK;
}

int qlc_layer_create_from_fp32(qlc_ctx *ctx, const float *weight, size_t weight_len, size_t out_dim, size_t in_dim,
                               size_t block_size, int double_quant, const float *a, size_t a_len, const float *b,
                               size_t b_len, size_t r, float alpha, qlc_layer **out) {
    qlc_qtensor *q = nullptr;
    QLC_TRY(qlc_quantize_nf4(ctx, weight, weight_len, out_dim, in_dim, block_size, double_quant, &q));
    const int st = qlc_layer_create(ctx, q, a, a_len, b, b_len, r, alpha, out);
    qlc_qtensor_destroy(q);  // the layer holds its own reference on success
    return st;
}

int qlc_layer_destroy(qlc_layer *L) {
    if (!L) return QLC_OK;
    cudaSetDevice(L->ctx->device);
    cudaStreamSynchronize(L->ctx->stream);
    umma_layer_release(L);
    cudaFree(L->d_a);
    cudaFree(L->d_b);
    cudaFree(L->d_a_pad);
    cudaFree(L->d_b_pad);
    cudaFree(L->d_bt_pad);
    cudaFree(L->d_a_pad32);
    cudaFree(L->d_b_pad32);
    cudaFree(L->d_bt_pad32);
    cudaFree(L->d_grad_bucket);
    cudaFree(L->d_w_raw);
    cudaFree(L->d_w_raw_bf16);
    qlc_qtensor_destroy(L->w);
    qlc_ctx_destroy(L->ctx);
    delete L;
    return QLC_OK;
}

int qlc_layer_set_weights(qlc_layer *L, const float *a, size_t a_len, const float *b, size_t b_len) {
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "null layer");
    if (L->r == 0) return fail(QLC_ERR_INVALID_CONFIG, "layer has no adapter");
    if (a_len != L->r * L->in_dim || b_len != L->out_dim * L->r)  // lora.rs:71-80
        return fail(QLC_ERR_SHAPE_MISMATCH, "set_weights: got (%zu, %zu), expected (%zu, %zu)", a_len, b_len,
                    L->r * L->in_dim, L->out_dim * L->r);
    if ((a_len && !a) || (b_len && !b)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(L->ctx->device));
    if (a_len) QLC_CUDA(cudaMemcpyAsync(L->d_a, a, a_len * 4, cudaMemcpyHostToDevice, L->ctx->stream));
    if (b_len) QLC_CUDA(cudaMemcpyAsync(L->d_b, b, b_len * 4, cudaMemcpyHostToDevice, L->ctx->stream));
    QLC_TRY(refresh_padded_adapter(L));
    return sync_and_check(L->ctx);
}

int qlc_layer_set_weights_dev(qlc_layer *L, const float *d_a, const float *d_b) {
    if (!L || !d_a || !d_b) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (L->r == 0) return fail(QLC_ERR_INVALID_CONFIG, "layer has no adapter");
    QLC_CUDA(cudaSetDevice(L->ctx->device));
    if (d_a != L->d_a)
        QLC_CUDA(cudaMemcpyAsync(L->d_a, d_a, L->r * L->in_dim * 4, cudaMemcpyDeviceToDevice, L->ctx->stream));
    if (d_b != L->d_b)
        QLC_CUDA(cudaMemcpyAsync(L->d_b, d_b, L->out_dim * L->r * 4, cudaMemcpyDeviceToDevice, L->ctx->stream));
    return refresh_padded_adapter(L);
}

int qlc_layer_adapter_dev(qlc_layer *L, float **d_a, float **d_b) {
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "null layer");
    if (L->r == 0) return fail(QLC_ERR_INVALID_CONFIG, "layer has no adapter");
    if (d_a) *d_a = L->d_a;
    if (d_b) *d_b = L->d_b;
    return QLC_OK;
}

int qlc_layer_adapter_updated(qlc_layer *L) {
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "null layer");
    if (L->r == 0) return fail(QLC_ERR_INVALID_CONFIG, "layer has no adapter");
    QLC_CUDA(cudaSetDevice(L->ctx->device));
    return refresh_padded_adapter(L);
}

int qlc_train_step_dev(qlc_ctx *ctx, qlc_layer *L, qlc_adam *adam, qlc_comm *comm, const void *d_x, const void *d_dy,
                       int dtype, size_t batch, void *d_grad_x) {
    if (!ctx || !L || !adam) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (L->r == 0) return fail(QLC_ERR_INVALID_CONFIG, "layer has no adapter to train");
    const size_t na = L->r * L->in_dim, nb = L->out_dim * L->r;
    float *ga = L->d_grad_bucket, *gb = L->d_grad_bucket + na;
    QLC_TRY(qlc_qlora_backward_dev(ctx, L, d_x, d_dy, dtype, batch, d_grad_x, ga, gb));
    if (comm) QLC_TRY(qlc_allreduce_lora_grads(comm, L));
    float *params[2] = {L->d_a, L->d_b};
    const float *grads[2] = {ga, gb};
    const size_t lens[2] = {na, nb};
    QLC_TRY(qlc_adam_step_dev(adam, 2, params, grads, lens, nullptr));
    return refresh_padded_adapter(L);
}

int qlc_layer_dims(const qlc_layer *L, size_t *out_dim, size_t *in_dim, size_t *rank, float *alpha) {
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "null layer");
    if (out_dim) *out_dim = L->out_dim;
    if (in_dim) *in_dim = L->in_dim;
    if (rank) *rank = L->r;
    if (alpha) *alpha = L->alpha;
    return QLC_OK;
}

qlc_qtensor *qlc_layer_weight(qlc_layer *L) { return L ? L->w : nullptr; }

int qlc_layer_grad_bucket(qlc_layer *L, float **d_bucket, size_t *n_floats) {
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "null layer");
    if (d_bucket) *d_bucket = L->d_grad_bucket;
    if (n_floats) *n_floats = L->r * (L->in_dim + L->out_dim);
    return QLC_OK;
}

// Handles are bound to the device they were created on: a layer of another GPU's context would make this
// GPU's kernels dereference foreign device pointers.
static int same_device(const qlc_ctx *ctx, const qlc_layer *L) {
    const int wdev = L->w ? L->w->device : L->ctx->device;
    if (L->ctx->device != ctx->device || wdev != ctx->device)
        return fail(QLC_ERR_GPU, "layer lives on device %d (weight on %d), context on %d", L->ctx->device, wdev, ctx->device);
    return QLC_OK;
}

// Which arithmetic a call uses (see QLC_PRECISION_* in the header).
static int pick_path(qlc_ctx *ctx, const qlc_layer *L, bool *use_umma) {
    const bool ok = umma_supported(L);
    if (ctx->precision == QLC_PRECISION_FP32_EXACT ||
        (ctx->precision == QLC_PRECISION_TF32 && (!L->w || !umma_fused_supported(L)))) {
        // TF32 exists in the fused kernels only: raw projections and layers that run through a padded copy are
        // multiplied in exact fp32 in that mode (more precise than asked for, slower)
        *use_umma = false;
    } else if (ctx->precision == QLC_PRECISION_BF16 || ctx->precision == QLC_PRECISION_TF32) {
        if (!ok)
            return fail(QLC_ERR_GPU,
                        "the tensor-core path takes LoRA ranks up to 256 and dimensions below 2^30 "
                        "(got block %zu, in %zu, out %zu, r %zu)",
                        L->w ? L->w->block_size : (size_t)0, L->in_dim, L->out_dim, L->r);
        *use_umma = true;
    } else {
        *use_umma = ok;
    }
    return QLC_OK;
}

static inline size_t a256(size_t b) { return (b + 255) & ~(size_t)255; }

int qlc_qlora_forward_dev(qlc_ctx *ctx, qlc_layer *L, const void *d_x, int dtype, size_t batch, void *d_y) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16) return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    if (batch == 0 || L->out_dim == 0) return QLC_OK;
    if (!d_y || (L->in_dim && !d_x)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    bool use_umma = false;
    QLC_TRY(pick_path(ctx, L, &use_umma));
    const size_t nx = batch * L->in_dim, ny = batch * L->out_dim;
    if (use_umma && ctx->precision == QLC_PRECISION_TF32) {
        // fp32 operands read as tf32 by the tensor cores, which would truncate them: fp32 activations are
        // rounded to tf32 into a staging buffer first; bf16 activations are widened (exactly representable).
        float *xf = nullptr;
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xf), a256(nx * 4), ctx->stream));
        int st = dtype == QLC_DTYPE_F32 ? launch_round_to_tf32(ctx, static_cast<const float *>(d_x), xf, nx)
                                        : launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_x), xf, nx);
        if (st == QLC_OK) st = umma_qlora_forward(ctx, L, xf, batch, d_y, dtype, true);
        cudaFreeAsync(xf, ctx->stream);
        return st;
    }
    if (use_umma) {
        if (dtype == QLC_DTYPE_BF16)
            return umma_qlora_forward(ctx, L, static_cast<const __nv_bfloat16 *>(d_x), batch, d_y, dtype);
        // fp32 activations: round X to bf16 in a staging buffer owned by the layer pass.
        __nv_bfloat16 *xb = nullptr;
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xb), a256(nx * 2), ctx->stream));
        int st = launch_convert_f32_to_bf16(ctx, static_cast<const float *>(d_x), xb, nx);
        if (st == QLC_OK) st = umma_qlora_forward(ctx, L, xb, batch, d_y, dtype);
        cudaFreeAsync(xb, ctx->stream);
        return st;
    }
    if (dtype == QLC_DTYPE_F32)
        return exact_qlora_forward(ctx, L, static_cast<const float *>(d_x), batch, static_cast<float *>(d_y));
    // bf16 activations on the exact path: widen, compute in fp32, round the result.
    float *xf = nullptr, *yf = nullptr;
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xf), a256(nx * 4), ctx->stream));
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&yf), a256(ny * 4), ctx->stream));
    int st = launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_x), xf, nx);
    if (st == QLC_OK) st = exact_qlora_forward(ctx, L, xf, batch, yf);
    if (st == QLC_OK) st = launch_convert_f32_to_bf16(ctx, yf, static_cast<__nv_bfloat16 *>(d_y), ny);
    cudaFreeAsync(xf, ctx->stream);
    cudaFreeAsync(yf, ctx->stream);
    return st;
}

int qlc_qlora_forward_dev_noalloc(qlc_ctx *ctx, qlc_layer *L, const void *d_x, size_t batch, void *d_y) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (batch == 0 || L->out_dim == 0) return QLC_OK;
    if (!d_x || !d_y) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    if (!L->w || !umma_fused_supported(L))
        return fail(QLC_ERR_INVALID_CONFIG,
                    "qlc_qlora_forward_dev_noalloc needs a tensor-core-eligible layer (block_size 32, 64, 128 or 256, in_dim and "
                    "out_dim multiples of 64, rank <= 64); got block %zu, in %zu, out %zu, r %zu",
                    L->w ? L->w->block_size : (size_t)0, L->in_dim, L->out_dim, L->r);
    QLC_CUDA(cudaSetDevice(ctx->device));
    return umma_qlora_forward_noalloc(ctx, L, static_cast<const __nv_bfloat16 *>(d_x), batch, d_y);
}

int qlc_qlora_backward_dev(qlc_ctx *ctx, qlc_layer *L, const void *d_x, const void *d_dy, int dtype, size_t batch,
                           void *d_gx, float *d_ga, float *d_gb) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16) return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    QLC_CUDA(cudaSetDevice(ctx->device));
    bool use_umma = false;
    QLC_TRY(pick_path(ctx, L, &use_umma));
    const size_t nx = batch * L->in_dim, ny = batch * L->out_dim;
    if (batch == 0) {
        // No rows: grad_x is empty and the token-contracted gradients are zero.
        if (L->r && d_ga) QLC_CUDA(cudaMemsetAsync(d_ga, 0, L->r * L->in_dim * 4, ctx->stream));
        if (L->r && d_gb) QLC_CUDA(cudaMemsetAsync(d_gb, 0, L->out_dim * L->r * 4, ctx->stream));
        return QLC_OK;
    }
    if ((nx && (!d_x || !d_gx)) || (ny && !d_dy)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    if (use_umma && ctx->precision == QLC_PRECISION_TF32) {
        float *xf = nullptr, *dyf = nullptr;
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xf), a256(nx * 4), ctx->stream));
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dyf), a256(ny * 4), ctx->stream));
        int st = QLC_OK;
        if (dtype == QLC_DTYPE_F32) {
            st = launch_round_to_tf32(ctx, static_cast<const float *>(d_x), xf, nx);
            if (st == QLC_OK) st = launch_round_to_tf32(ctx, static_cast<const float *>(d_dy), dyf, ny);
        } else {
            st = launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_x), xf, nx);
            if (st == QLC_OK) st = launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_dy), dyf, ny);
        }
        if (st == QLC_OK) st = umma_qlora_backward(ctx, L, xf, dyf, batch, d_gx, dtype, d_ga, d_gb, 0, true);
        cudaFreeAsync(xf, ctx->stream);
        cudaFreeAsync(dyf, ctx->stream);
        return st;
    }
    if (use_umma) {
        if (dtype == QLC_DTYPE_BF16)
            return umma_qlora_backward(ctx, L, static_cast<const __nv_bfloat16 *>(d_x),
                                       static_cast<const __nv_bfloat16 *>(d_dy), batch, d_gx, dtype, d_ga, d_gb);
        __nv_bfloat16 *xb = nullptr, *dyb = nullptr;
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xb), a256(nx * 2), ctx->stream));
        QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dyb), a256(ny * 2), ctx->stream));
        int st = launch_convert_f32_to_bf16(ctx, static_cast<const float *>(d_x), xb, nx);
        if (st == QLC_OK) st = launch_convert_f32_to_bf16(ctx, static_cast<const float *>(d_dy), dyb, ny);
        if (st == QLC_OK) st = umma_qlora_backward(ctx, L, xb, dyb, batch, d_gx, dtype, d_ga, d_gb);
        cudaFreeAsync(xb, ctx->stream);
        cudaFreeAsync(dyb, ctx->stream);
        return st;
    }
    if (dtype == QLC_DTYPE_F32)
        return exact_qlora_backward(ctx, L, static_cast<const float *>(d_x), static_cast<const float *>(d_dy), batch,
                                    static_cast<float *>(d_gx), d_ga, d_gb);
    float *xf = nullptr, *dyf = nullptr, *gxf = nullptr;
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&xf), a256(nx * 4), ctx->stream));
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dyf), a256(ny * 4), ctx->stream));
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&gxf), a256(nx * 4), ctx->stream));
    int st = launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_x), xf, nx);
    if (st == QLC_OK) st = launch_convert_bf16_to_f32(ctx, static_cast<const __nv_bfloat16 *>(d_dy), dyf, ny);
    if (st == QLC_OK) st = exact_qlora_backward(ctx, L, xf, dyf, batch, gxf, d_ga, d_gb);
    if (st == QLC_OK) st = launch_convert_f32_to_bf16(ctx, gxf, static_cast<__nv_bfloat16 *>(d_gx), nx);
    cudaFreeAsync(xf, ctx->stream);
    cudaFreeAsync(dyf, ctx->stream);
    cudaFreeAsync(gxf, ctx->stream);
    return st;
}

static size_t dtype_size(int dtype) { return dtype == QLC_DTYPE_BF16 ? 2 : 4; }

// Row slabs of the pipelined host entry points: while slab i computes, slab i+1 is copied in and slab i-1 is
// copied out (three streams, events in between), so a host-link-bound call costs about max(in, out) instead of
// in + compute + out.  Rows are independent for Y and dX; grad_a / grad_b accumulate slab after slab in a
// fixed order.
static const size_t kSlabRows = getenv("QLC_SLAB_ROWS") ? (size_t)atoi(getenv("QLC_SLAB_ROWS")) : 2048;  // diagnostics override

// The first copy in and the last copy out have nothing to overlap with, so the slabs ramp up and down: a quarter
// and a half slab at either end, full slabs in between (8192 rows: 512, 1024, 2048, 2048, 1024, 1024, 512; a
// third ramp step measured no better).
// `streaming`: the caller keeps several submissions in flight, so the ends of one submission's copies overlap its
// neighbours' and the ramp (shorter slabs at both ends, which shorten a lone call's exposed first copy in and last
// copy out) would only add small, less efficient transfers.
static std::vector<size_t> slab_schedule(size_t batch, bool streaming = false) {
    // streaming: two slabs per submission - fewer, larger copies carry more (8192 rows: 3.44 / 3.13 / 3.02 ms per
    // step with 1024- / 2048- / 4096-row slabs), and one split is enough to overlap a submission's own stages
    const size_t S = streaming && batch / 2 > kSlabRows ? ((batch / 2 + 255) & ~(size_t)255) : kSlabRows;
    std::vector<size_t> rows, ramp;
    static const bool flat_env = getenv("QLC_FLAT_SLABS") != nullptr;  // diagnostics: equal slabs
    const bool flat = flat_env || streaming;
    size_t ramp_rows = 0;
    for (size_t r = S / 4; r && r < S; r *= 2) {
        ramp.push_back(r);
        ramp_rows += r;
    }
    if (flat || ramp.empty() || batch < 2 * ramp_rows + S) {
        for (size_t r0 = 0; r0 < batch; r0 += S) rows.push_back(r0 + S <= batch ? S : batch - r0);
        return rows;
    }
    rows = ramp;
    size_t mid = batch - 2 * ramp_rows;
    for (; mid >= S; mid -= S) rows.push_back(S);
    if (mid) rows.push_back(mid);
    for (size_t k = ramp.size(); k-- > 0;) rows.push_back(ramp[k]);
    return rows;
}

static int chunk_event(qlc_ctx *ctx, size_t i, cudaEvent_t *out) {
    while (ctx->chunk_events.size() <= i) {
        cudaEvent_t e = nullptr;
        QLC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->chunk_events.push_back(e);
    }
    *out = ctx->chunk_events[i];
    return QLC_OK;
}

static int finish_pipelined(qlc_ctx *ctx) {
    QLC_CUDA(cudaStreamSynchronize(ctx->d2h_stream));
    QLC_CUDA(cudaStreamSynchronize(ctx->copy_stream));
    return sync_and_check(ctx);
}

int qlc_qlora_forward_host(qlc_ctx *ctx, qlc_layer *L, const void *x, int dtype, size_t batch, void *y) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16) return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    const size_t es = dtype_size(dtype), nx = batch * L->in_dim, ny = batch * L->out_dim;
    if (ny == 0) return QLC_OK;
    if (!y || (nx && !x)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    void *io = nullptr;
    QLC_TRY(ctx_io(ctx, a256(nx * es) + a256(ny * es), &io));
    char *dx = static_cast<char *>(io), *dy = static_cast<char *>(io) + a256(nx * es);
    bool use_umma = false;
    QLC_TRY(pick_path(ctx, L, &use_umma));
    if (!use_umma || batch < 2 * kSlabRows) {
        if (nx) QLC_CUDA(cudaMemcpyAsync(dx, x, nx * es, cudaMemcpyHostToDevice, ctx->stream));
        QLC_TRY(qlc_qlora_forward_dev(ctx, L, dx, dtype, batch, dy));
        QLC_CUDA(cudaMemcpyAsync(y, dy, ny * es, cudaMemcpyDeviceToHost, ctx->stream));
        return sync_and_check(ctx);
    }
    QLC_CUDA(cudaStreamSynchronize(ctx->stream));  // earlier work on the context is done before the side streams start
    const std::vector<size_t> sched = slab_schedule(batch);
    size_t r0 = 0;
    for (size_t c = 0; c < sched.size(); r0 += sched[c], ++c) {
        const size_t rows = sched[c];
        const size_t ox = r0 * L->in_dim * es, oy = r0 * L->out_dim * es;
        cudaEvent_t in_done, out_ready;
        QLC_TRY(chunk_event(ctx, 2 * c, &in_done));
        QLC_TRY(chunk_event(ctx, 2 * c + 1, &out_ready));
        QLC_CUDA(cudaMemcpyAsync(dx + ox, static_cast<const char *>(x) + ox, rows * L->in_dim * es, cudaMemcpyHostToDevice,
                                 ctx->copy_stream));
        QLC_CUDA(cudaEventRecord(in_done, ctx->copy_stream));
        QLC_CUDA(cudaStreamWaitEvent(ctx->stream, in_done, 0));
        QLC_TRY(qlc_qlora_forward_dev(ctx, L, dx + ox, dtype, rows, dy + oy));
        QLC_CUDA(cudaEventRecord(out_ready, ctx->stream));
        QLC_CUDA(cudaStreamWaitEvent(ctx->d2h_stream, out_ready, 0));
        QLC_CUDA(cudaMemcpyAsync(static_cast<char *>(y) + oy, dy + oy, rows * L->out_dim * es, cudaMemcpyDeviceToHost,
                                 ctx->d2h_stream));
    }
    return finish_pipelined(ctx);
}

int qlc_qlora_backward_host(qlc_ctx *ctx, qlc_layer *L, const void *x, const void *dy, int dtype, size_t batch,
                            void *grad_x, float *grad_a, float *grad_b) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16) return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    const size_t es = dtype_size(dtype), nx = batch * L->in_dim, ny = batch * L->out_dim;
    const size_t na = L->r * L->in_dim, nb = L->out_dim * L->r;
    if ((nx && (!x || !grad_x)) || (ny && !dy)) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    void *io = nullptr;
    QLC_TRY(ctx_io(ctx, 2 * a256(nx * es) + a256(ny * es), &io));
    char *dx = static_cast<char *>(io), *ddy = static_cast<char *>(io) + a256(nx * es);
    char *dgx = static_cast<char *>(io) + a256(nx * es) + a256(ny * es);
    float *d_ga = L->r ? L->d_grad_bucket : nullptr;
    float *d_gb = L->r ? L->d_grad_bucket + na : nullptr;
    bool use_umma = false;
    QLC_TRY(pick_path(ctx, L, &use_umma));
    if (!use_umma || dtype != QLC_DTYPE_BF16 || batch < 2 * kSlabRows || ctx->precision == QLC_PRECISION_TF32) {
        if (nx) QLC_CUDA(cudaMemcpyAsync(dx, x, nx * es, cudaMemcpyHostToDevice, ctx->stream));
        if (ny) QLC_CUDA(cudaMemcpyAsync(ddy, dy, ny * es, cudaMemcpyHostToDevice, ctx->stream));
        QLC_TRY(qlc_qlora_backward_dev(ctx, L, dx, ddy, dtype, batch, dgx, d_ga, d_gb));
        if (nx) QLC_CUDA(cudaMemcpyAsync(grad_x, dgx, nx * es, cudaMemcpyDeviceToHost, ctx->stream));
    } else {
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        const std::vector<size_t> sched = slab_schedule(batch);
        size_t r0 = 0;
        for (size_t c = 0; c < sched.size(); r0 += sched[c], ++c) {
            const size_t rows = sched[c];
            const size_t ox = r0 * L->in_dim * es, oy = r0 * L->out_dim * es;
            cudaEvent_t in_done, out_ready;
            QLC_TRY(chunk_event(ctx, 2 * c, &in_done));
            QLC_TRY(chunk_event(ctx, 2 * c + 1, &out_ready));
            QLC_CUDA(cudaMemcpyAsync(dx + ox, static_cast<const char *>(x) + ox, rows * L->in_dim * es,
                                     cudaMemcpyHostToDevice, ctx->copy_stream));
            QLC_CUDA(cudaMemcpyAsync(ddy + oy, static_cast<const char *>(dy) + oy, rows * L->out_dim * es,
                                     cudaMemcpyHostToDevice, ctx->copy_stream));
            QLC_CUDA(cudaEventRecord(in_done, ctx->copy_stream));
            QLC_CUDA(cudaStreamWaitEvent(ctx->stream, in_done, 0));
            QLC_TRY(umma_qlora_backward(ctx, L, reinterpret_cast<const __nv_bfloat16 *>(dx + ox),
                                        reinterpret_cast<const __nv_bfloat16 *>(ddy + oy), rows, dgx + ox, dtype, d_ga, d_gb,
                                        c > 0 ? 1 : 0));
            QLC_CUDA(cudaEventRecord(out_ready, ctx->stream));
            QLC_CUDA(cudaStreamWaitEvent(ctx->d2h_stream, out_ready, 0));
            QLC_CUDA(cudaMemcpyAsync(static_cast<char *>(grad_x) + ox, dgx + ox, rows * L->in_dim * es,
                                     cudaMemcpyDeviceToHost, ctx->d2h_stream));
        }
    }
    if (L->r && grad_a && na) QLC_CUDA(cudaMemcpyAsync(grad_a, d_ga, na * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (L->r && grad_b && nb) QLC_CUDA(cudaMemcpyAsync(grad_b, d_gb, nb * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return finish_pipelined(ctx);
}

// Queues forward + backward of one batch (host buffers) without waiting for any of it; *pipelined tells whether the
// slab pipeline was used (false: the two synchronous calls ran and everything is already complete).
// Diagnostics (QLC_HOST_PIPE_TIMING=1): device-side time stamps of every stage of the fused host pipeline, printed
// four submissions later (by then they have completed; nothing waits for them).  One line per row slab.
struct PipeTimeline {
    std::vector<cudaEvent_t> ev;
    size_t used = 0, slabs = 0;
    uint64_t submission = 0;
};
static PipeTimeline g_pipe_tl[4];
static cudaEvent_t g_pipe_base = nullptr;
static uint64_t g_pipe_n = 0;
constexpr size_t kPipeMarks = 8;  // per slab: h2d begin/end, compute begin, fwd end, bwd end, d2h begin, y out, dX out
static void pipe_timeline_print(PipeTimeline &t) {
    if (!t.used || cudaEventQuery(t.ev[t.used - 1]) != cudaSuccess) return;
    fprintf(stderr, "[qlc host pipe] submission %llu, ms since the first one: slab | h2d begin, end | compute begin, fwd end, bwd end | d2h begin, Y out, dX out\n",
            (unsigned long long)t.submission);
    for (size_t c = 0; c < t.slabs; ++c) {
        float ms[kPipeMarks];
        for (size_t k = 0; k < kPipeMarks; ++k) cudaEventElapsedTime(&ms[k], g_pipe_base, t.ev[c * kPipeMarks + k]);
        fprintf(stderr, "[qlc host pipe]   %2zu | %8.3f %8.3f | %8.3f %8.3f %8.3f | %8.3f %8.3f %8.3f\n", c, ms[0], ms[1], ms[2], ms[3],
                ms[4], ms[5], ms[6], ms[7]);
    }
    t.used = 0;
}

static int fused_submit(qlc_ctx *ctx, qlc_layer *L, const void *x, const void *dy, int dtype, size_t batch, void *y,
                        void *grad_x, float *grad_a, float *grad_b, bool streaming, bool *pipelined) {
    *pipelined = false;
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    QLC_TRY(same_device(ctx, L));
    if (dtype != QLC_DTYPE_F32 && dtype != QLC_DTYPE_BF16) return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
    const size_t es = dtype_size(dtype), nx = batch * L->in_dim, ny = batch * L->out_dim;
    const size_t na = L->r * L->in_dim, nb = L->out_dim * L->r;
    if ((nx && (!x || !grad_x)) || (ny && (!dy || !y))) return fail(QLC_ERR_INVALID_CONFIG, "null buffer");
    QLC_CUDA(cudaSetDevice(ctx->device));
    bool use_umma = false;
    QLC_TRY(pick_path(ctx, L, &use_umma));
    if (!use_umma || dtype != QLC_DTYPE_BF16 || batch < 2 * kSlabRows || ctx->precision == QLC_PRECISION_TF32 || !L->w ||
        !umma_fused_supported(L)) {
        // no pipelined form for this case: the two stateless calls, one after the other
        QLC_TRY(qlc_qlora_forward_host(ctx, L, x, dtype, batch, y));
        return qlc_qlora_backward_host(ctx, L, x, dy, dtype, batch, grad_x, grad_a, grad_b);
    }
    *pipelined = true;
    // Two sets of device staging buffers, used by consecutive submissions in turn: a submission's copies in never
    // wait for the previous submission's compute, and its compute never waits for the previous submission's copies
    // out - with two submissions in flight the host link stays busy in both directions without a gap.
    const size_t g_bytes = a256((na + nb + 1) * 4);
    const size_t set_bytes = 2 * a256(nx * es) + 2 * a256(ny * es) + g_bytes;
    QLC_TRY(ctx_io_grow(ctx, 2 * set_bytes));
    const int p = (int)(ctx->fused_submissions++ & 1);
    char *dx = static_cast<char *>(ctx->io) + p * set_bytes, *ddy = dx + a256(nx * es), *dyo = ddy + a256(ny * es),
         *dgx = dyo + a256(ny * es);
    // Gradients wanted on the host are accumulated in this set's own bucket and leave on the copy-out stream; with
    // grad_a == grad_b == NULL they go to the layer's bucket (qlc_layer_grad_bucket) and stay on the device.
    const bool grads_out = L->r && (grad_a || grad_b);
    float *g_stage = reinterpret_cast<float *>(dgx + a256(nx * es));
    float *d_ga = L->r ? (grads_out ? g_stage : L->d_grad_bucket) : nullptr;
    float *d_gb = L->r ? d_ga + na : nullptr;
    QLC_CUDA(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_in_free[p], 0));  // staged inputs of set p: read two submissions ago
    QLC_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_out_free[p], 0));      // staged outputs of set p: copied out two submissions ago
    const std::vector<size_t> sched = slab_schedule(batch, streaming);
    static const bool timing = getenv("QLC_HOST_PIPE_TIMING") != nullptr;
    PipeTimeline *tl = nullptr;
    if (timing) {
        tl = &g_pipe_tl[g_pipe_n % 4];
        pipe_timeline_print(*tl);
        if (!g_pipe_base) {
            QLC_CUDA(cudaEventCreate(&g_pipe_base));
            QLC_CUDA(cudaEventRecord(g_pipe_base, ctx->stream));
        }
        while (tl->ev.size() < sched.size() * kPipeMarks) {
            cudaEvent_t e = nullptr;
            QLC_CUDA(cudaEventCreate(&e));
            tl->ev.push_back(e);
        }
        tl->slabs = sched.size();
        tl->used = sched.size() * kPipeMarks;
        tl->submission = g_pipe_n++;
    }
    auto mark = [&](size_t c, size_t k, cudaStream_t st) {
        if (tl) cudaEventRecord(tl->ev[c * kPipeMarks + k], st);
    };
    size_t r0 = 0;
    for (size_t c = 0; c < sched.size(); r0 += sched[c], ++c) {
        const size_t rows = sched[c];
        const size_t ox = r0 * L->in_dim * es, oy = r0 * L->out_dim * es;
        cudaEvent_t in_done, y_ready, gx_ready;
        QLC_TRY(chunk_event(ctx, 3 * c, &in_done));
        QLC_TRY(chunk_event(ctx, 3 * c + 1, &y_ready));
        QLC_TRY(chunk_event(ctx, 3 * c + 2, &gx_ready));
        mark(c, 0, ctx->copy_stream);
        QLC_CUDA(cudaMemcpyAsync(dx + ox, static_cast<const char *>(x) + ox, rows * L->in_dim * es, cudaMemcpyHostToDevice,
                                 ctx->copy_stream));
        QLC_CUDA(cudaMemcpyAsync(ddy + oy, static_cast<const char *>(dy) + oy, rows * L->out_dim * es, cudaMemcpyHostToDevice,
                                 ctx->copy_stream));
        QLC_CUDA(cudaEventRecord(in_done, ctx->copy_stream));
        mark(c, 1, ctx->copy_stream);
        QLC_CUDA(cudaStreamWaitEvent(ctx->stream, in_done, 0));
        mark(c, 2, ctx->stream);
        QLC_TRY(umma_qlora_forward(ctx, L, dx + ox, rows, dyo + oy, dtype));
        QLC_CUDA(cudaEventRecord(y_ready, ctx->stream));
        mark(c, 3, ctx->stream);
        QLC_TRY(umma_qlora_backward(ctx, L, reinterpret_cast<const __nv_bfloat16 *>(dx + ox),
                                    reinterpret_cast<const __nv_bfloat16 *>(ddy + oy), rows, dgx + ox, dtype, d_ga, d_gb,
                                    c > 0 ? 1 : 0));
        QLC_CUDA(cudaEventRecord(gx_ready, ctx->stream));
        mark(c, 4, ctx->stream);
        QLC_CUDA(cudaStreamWaitEvent(ctx->d2h_stream, y_ready, 0));
        mark(c, 5, ctx->d2h_stream);
        QLC_CUDA(cudaMemcpyAsync(static_cast<char *>(y) + oy, dyo + oy, rows * L->out_dim * es, cudaMemcpyDeviceToHost,
                                 ctx->d2h_stream));
        mark(c, 6, ctx->d2h_stream);
        QLC_CUDA(cudaStreamWaitEvent(ctx->d2h_stream, gx_ready, 0));
        QLC_CUDA(cudaMemcpyAsync(static_cast<char *>(grad_x) + ox, dgx + ox, rows * L->in_dim * es, cudaMemcpyDeviceToHost,
                                 ctx->d2h_stream));
        mark(c, 7, ctx->d2h_stream);
    }
    QLC_CUDA(cudaEventRecord(ctx->ev_in_free[p], ctx->stream));  // end of this submission's compute
    // (the copy-out stream has waited for the last slab's backward pass, which ends with the gradient contractions)
    if (grads_out && grad_a && na) QLC_CUDA(cudaMemcpyAsync(grad_a, d_ga, na * 4, cudaMemcpyDeviceToHost, ctx->d2h_stream));
    if (grads_out && grad_b && nb) QLC_CUDA(cudaMemcpyAsync(grad_b, d_gb, nb * 4, cudaMemcpyDeviceToHost, ctx->d2h_stream));
    QLC_CUDA(cudaEventRecord(ctx->ev_out_free[p], ctx->d2h_stream));  // end of this submission
    ctx->fused_open = true;
    return QLC_OK;
}

int qlc_qlora_forward_backward_host(qlc_ctx *ctx, qlc_layer *L, const void *x, const void *dy, int dtype, size_t batch,
                                    void *y, void *grad_x, float *grad_a, float *grad_b) {
    bool pipelined = false;
    QLC_TRY(fused_submit(ctx, L, x, dy, dtype, batch, y, grad_x, grad_a, grad_b, false, &pipelined));
    return pipelined ? sync_and_check(ctx) : QLC_OK;
}

int qlc_qlora_forward_backward_host_async(qlc_ctx *ctx, qlc_layer *L, const void *x, const void *dy, int dtype,
                                          size_t batch, void *y, void *grad_x, float *grad_a, float *grad_b,
                                          uint64_t *ticket) {
    if (!ticket) return fail(QLC_ERR_INVALID_CONFIG, "null ticket");
    bool pipelined = false;
    QLC_TRY(fused_submit(ctx, L, x, dy, dtype, batch, y, grad_x, grad_a, grad_b, true, &pipelined));
    const uint64_t t = ctx->tickets_issued;
    cudaEvent_t &ev = ctx->ticket_ev[t % qlc_ctx::kTickets];
    if (!ev) QLC_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    // the copy-out stream ends a pipelined submission (it has waited for all of its compute)
    QLC_CUDA(cudaEventRecord(ev, pipelined ? ctx->d2h_stream : ctx->stream));
    ctx->tickets_issued = t + 1;
    *ticket = t;
    return QLC_OK;
}

int qlc_ctx_wait(qlc_ctx *ctx, uint64_t ticket) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (ticket >= ctx->tickets_issued) return fail(QLC_ERR_INVALID_CONFIG, "ticket %llu was never issued", (unsigned long long)ticket);
    QLC_CUDA(cudaSetDevice(ctx->device));
    // An old ticket's event has been re-recorded by a later submission on the same stream: waiting for that one
    // waits for the older submission too.
    QLC_CUDA(cudaEventSynchronize(ctx->ticket_ev[ticket % qlc_ctx::kTickets]));
    return QLC_OK;
}

// The reference-named fp32 entry points (qlc_qlora_forward / qlc_qlora_backward) promise the reference's
// GPU-vs-CPU agreement (max abs diff < 1e-3 forward, < 1e-2 gradients: qlora-wgpu/tests/gpu_parity.rs:59,
// gpu_backward.rs:88-96), which bf16 operands do not keep at in_dim in the thousands.  Under
// QLC_PRECISION_AUTO they therefore compute in TF32 where the tensor-core path takes the shape and in exact
// fp32 elsewhere, so the precision class does not change with the shape; bf16 is an explicit choice
// (qlc_ctx_set_precision) or comes with the bf16 / device entry points.
struct Fp32CallPrecision {
    qlc_ctx *ctx;
    int saved;
    Fp32CallPrecision(qlc_ctx *c, const qlc_layer *L) : ctx(c), saved(c->precision) {
        if (saved == QLC_PRECISION_AUTO) ctx->precision = umma_fused_supported(L) ? QLC_PRECISION_TF32 : QLC_PRECISION_FP32_EXACT;
    }
    ~Fp32CallPrecision() { ctx->precision = saved; }
};

int qlc_qlora_forward(qlc_ctx *ctx, qlc_layer *L, const float *x, size_t x_len, size_t batch, float *y) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (x_len != batch * L->in_dim)  // qlora.rs:89-95
        return fail(QLC_ERR_SHAPE_MISMATCH, "x.len() = %zu but batch*in_dim = %zu", x_len, batch * L->in_dim);
    const Fp32CallPrecision scope(ctx, L);
    return qlc_qlora_forward_host(ctx, L, x, QLC_DTYPE_F32, batch, y);
}

int qlc_qlora_backward(qlc_ctx *ctx, qlc_layer *L, const float *x, size_t x_len, const float *dy, size_t dy_len,
                       size_t batch, float *grad_x, float *grad_a, float *grad_b) {
    if (!ctx || !L) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (x_len != batch * L->in_dim)  // qlora.rs:119-125
        return fail(QLC_ERR_SHAPE_MISMATCH, "x.len() = %zu but batch*in_dim = %zu", x_len, batch * L->in_dim);
    if (dy_len != batch * L->out_dim)  // qlora.rs:126-132
        return fail(QLC_ERR_SHAPE_MISMATCH, "dy.len() = %zu but batch*out_dim = %zu", dy_len, batch * L->out_dim);
    const Fp32CallPrecision scope(ctx, L);
    return qlc_qlora_backward_host(ctx, L, x, dy, QLC_DTYPE_F32, batch, grad_x, grad_a, grad_b);
}

}  // extern "C"
