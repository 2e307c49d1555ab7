// Shared declarations of libqlora_cuda: status handling, handle layouts, kernel launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <vector>

#include "../../../include/qlora_cuda.h"

namespace qlc {

// ---- status ---------------------------------------------------------------------------
// Records the message (thread-local) and returns `code` so call sites can `return fail(...)`.
int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define QLC_CUDA(expr)                                                                       \
    do {                                                                                     \
        cudaError_t qlc_e_ = (expr);                                                         \
        if (qlc_e_ != cudaSuccess)                                                           \
            return ::qlc::fail(QLC_ERR_GPU, "%s: %s", #expr, cudaGetErrorString(qlc_e_));    \
    } while (0)

#define QLC_TRY(expr)                 \
    do {                              \
        int qlc_s_ = (expr);          \
        if (qlc_s_ != QLC_OK) return qlc_s_; \
    } while (0)

// Number of 256-scale super-blocks of double quantisation (qlora-core/src/quant.rs:50).
constexpr size_t kDoubleQuantBlock = 256;

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// ---- device-side status word -----------------------------------------------------------
// Kernels never trap: a bounded wait that gives up, or a failed self-check, stores a
// non-zero code here (device memory) and returns.  qlc_ctx_synchronize reads it back and reports it.
struct DeviceStatus {
    int code;      // 0 = fine
    int where;     // site id of the first failure
    int block;     // blockIdx.x of the reporter
    int detail;    // site-specific
};

enum StatusCode : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,   // an mbarrier wait hit its iteration/time limit
};

}  // namespace qlc

// ---- handle layouts (opaque to C callers) ------------------------------------------------
struct qlc_ctx {
    int refs = 1;  // the creator's reference + one per live layer / optimiser bound to this context
    int device = -1;
    cudaStream_t stream = nullptr;       // all kernels of this context
    cudaStream_t copy_stream = nullptr;  // host-to-device copies of the pipelined *_host entry points
    int *d_tile_counters[2] = {nullptr, nullptr};  // zeroed ints for kernels whose last-arriving CTA finishes a tile
    size_t tile_counters_cap[2] = {0, 0};
    cudaStream_t side_stream = nullptr;  // lowest priority: work that fills SMs the main stream leaves idle
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t d2h_stream = nullptr;   // device-to-host copies of the pipelined *_host entry points
    std::vector<cudaEvent_t> chunk_events;  // reused by the pipelined *_host entry points
    // Asynchronous host-buffer calls (forward + backward of one batch): consecutive submissions alternate between
    // two sets of device staging buffers.  ev_in_free[p]: the compute of the last submission that used set p has
    // ended (its staged inputs may be overwritten); ev_out_free[p]: that submission's copies out have ended.
    cudaEvent_t ev_in_free[2] = {nullptr, nullptr}, ev_out_free[2] = {nullptr, nullptr};
    uint64_t fused_submissions = 0;
    bool fused_open = false;  // copies of such submissions may still run on the copy streams
    // completion tickets of the asynchronous host-buffer calls: a ring of events, ticket t -> ticket_ev[t % 8]
    static constexpr int kTickets = 8;
    cudaEvent_t ticket_ev[kTickets] = {nullptr};
    uint64_t tickets_issued = 0;
    int precision = QLC_PRECISION_AUTO;
    int sm_count = 0;
    int reserved_sms = 0;  // SMs the one-wave (persistent) kernels leave free for kernels of other streams (qlc_ctx_set_reserved_sms)
    uint64_t launches = 0;
    qlc::DeviceStatus *d_status = nullptr;  // device memory, read back by qlc_ctx_synchronize
    // Scratch arena for intermediates of the layer passes (T1, Ds, split partials, staged
    // activations).  Grown on demand; never shrinks.
    void *ws = nullptr;
    size_t ws_bytes = 0;
    // Pinned host staging for the *_host entry points.
    void *pin = nullptr;
    size_t pin_bytes = 0;
    int umma_smem_optin = 0;  // max dynamic smem per block
    // Device staging of activations for the *_host entry points (grown on demand).
    void *io = nullptr;
    size_t io_bytes = 0;
    // Optional per-kernel event timing (qlc_ctx_profile_*).
    bool profiling = false;
    struct ProfEvent {
        int slot;
        cudaEvent_t start, stop;
    };
    std::vector<ProfEvent> prof_pending;
    std::vector<cudaEvent_t> prof_pool;
    double prof_ms[QLC_PROFILE_SLOTS] = {0, 0, 0, 0};
    uint64_t prof_launches[QLC_PROFILE_SLOTS] = {0, 0, 0, 0};
};

struct qlc_qtensor {
    int refs = 1;
    int device = -1;
    size_t rows = 0, cols = 0, block_size = 0;
    size_t n = 0, nb = 0;
    bool dq = false;
    uint8_t *d_codes = nullptr;         // ceil(n/2) bytes, allocation padded & zero-filled to 16 B
    uint8_t *d_absmax_codes = nullptr;  // nb bytes (dq)
    float *d_absmax2 = nullptr;         // ceil(nb/256) (dq)
    float *d_scales_f32 = nullptr;      // nb (not dq)
};

struct qlc_layer {
    qlc_ctx *ctx = nullptr;
    qlc_qtensor *w = nullptr;  // null for a raw (unquantised) projection, which the model code creates
    // Raw projection (qlora-model/src/llama.rs:87-93, Proj::Raw): the frozen (out_dim, in_dim) weight as fp32
    // (exact and TF32 modes) and rounded to bf16 (tensor-core path).  Never has an adapter.
    float *d_w_raw = nullptr;
    __nv_bfloat16 *d_w_raw_bf16 = nullptr;
    size_t in_dim = 0, out_dim = 0, r = 0;
    float alpha = 0.f;
    float *d_a = nullptr;  // (r, in_dim) fp32
    float *d_b = nullptr;  // (out_dim, r) fp32
    // bf16 operand copies for the tensor-core path, rank padded with zeros to r_pad (multiple of 64):
    __nv_bfloat16 *d_a_pad = nullptr;  // (r_pad, in_dim)
    __nv_bfloat16 *d_b_pad = nullptr;  // (out_dim, r_pad)
    __nv_bfloat16 *d_bt_pad = nullptr; // (r_pad, out_dim): B transposed, for the dY·B product
    // the same three as fp32 values rounded to tf32, for the TF32 mode (allocated on first use)
    float *d_a_pad32 = nullptr, *d_b_pad32 = nullptr, *d_bt_pad32 = nullptr;
    bool pad32_valid = false;
    size_t r_pad = 0;
    float *d_grad_bucket = nullptr;  // r*in_dim + out_dim*r fp32
    // Cached tensor maps (opaque blobs, built lazily by the tensor-core path).
    void *tmaps = nullptr;
    // Layers the fused kernels do not take (dimensions no multiple of 64, other block sizes): a padded bf16 copy of
    // the layer, built at the first tensor-core call (umma_gemm.cu); its adapter copies follow every change of A / B.
    qlc_layer *shadow = nullptr;
    bool shadow_valid = false;
};

namespace qlc {

// ---- launchers implemented in the .cu files -------------------------------------------------
// quant_kernels.cu
int launch_quantize_nf4(qlc_ctx *ctx, const float *d_w, qlc_qtensor *q);
int alloc_qtensor(qlc_ctx *ctx, size_t rows, size_t cols, size_t block_size, bool dq, qlc_qtensor **out);  // empty payload
int launch_dequantize(qlc_ctx *ctx, const qlc_qtensor *q, void *d_out, int dtype);
int launch_decode_block_scales(qlc_ctx *ctx, const qlc_qtensor *q, float *d_out);
int launch_refresh_adapters(qlc_ctx *ctx, qlc_layer *const *layers, size_t n);
int launch_convert_f32_to_bf16(qlc_ctx *ctx, const float *d_in, __nv_bfloat16 *d_out, size_t n);
int launch_convert_bf16_to_f32(qlc_ctx *ctx, const __nv_bfloat16 *d_in, float *d_out, size_t n);
// Pads a row-major (rows, cols) fp32 matrix to bf16 (rows_pad, cols_pad), zero filled.
int launch_convert_f16_to_f32(qlc_ctx *ctx, const void *d_in, float *d_out, size_t n);
int launch_round_to_tf32(qlc_ctx *ctx, const float *d_in, float *d_out, size_t n);
int launch_pad_to_tf32(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, float *d_out, size_t out_rows,
                       size_t out_cols, int transposed);
int launch_pad_to_bf16(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, __nv_bfloat16 *d_out,
                       size_t rows_pad, size_t cols_pad);
// Same for the transpose: out (cols_pad, rows_pad) = in(rows, cols)^T, zero filled.
int launch_pad_transpose_to_bf16(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, __nv_bfloat16 *d_out,
                                 size_t cols_pad, size_t rows_pad);

// self-tests of the code selection (quant_kernels.cu)
int selftest_codes_of_targets(qlc_ctx *ctx, uint32_t first_bits, size_t count, uint8_t *d_out);
int selftest_fast_path(qlc_ctx *ctx, float absmax, uint32_t first_bits, unsigned long long count,
                       unsigned long long *d_out3);

// gemm_exact.cu — fp32 SIMT, reference accumulation order
int exact_matmul(qlc_ctx *ctx, const float *d_a, const float *d_b, size_t m, size_t k, size_t n, float *d_c);
int exact_matmul_trans_b(qlc_ctx *ctx, const float *d_a, const float *d_b, size_t m, size_t k, size_t n, float *d_c);
int exact_matmul_trans_a(qlc_ctx *ctx, const float *d_a, const float *d_b, size_t m, size_t k, size_t n, float *d_c);
int exact_qlora_forward(qlc_ctx *ctx, qlc_layer *layer, const float *d_x, size_t batch, float *d_y);
int exact_qlora_backward(qlc_ctx *ctx, qlc_layer *layer, const float *d_x, const float *d_dy, size_t batch,
                         float *d_gx, float *d_ga, float *d_gb);

// umma_gemm.cu — tcgen05 / TMEM / TMA tensor-core path
bool umma_supported(const qlc_layer *layer);        // the tensor-core path takes this layer (fused kernels or padded copy)
bool umma_fused_supported(const qlc_layer *layer);  // ... through the fused kernels (TF32 needs these)
int umma_qlora_forward(qlc_ctx *ctx, qlc_layer *layer, const void *d_x, size_t batch, void *d_y, int y_dtype,
                       bool tf32 = false);
// accumulate != 0: grad_a / grad_b receive this slab's contribution on top of their current contents.
// tf32: d_x / d_dy are fp32 and every product runs on the tensor cores in tf32.
int umma_qlora_backward(qlc_ctx *ctx, qlc_layer *layer, const void *d_x, const void *d_dy, size_t batch, void *d_gx,
                        int gx_dtype, float *d_ga, float *d_gb, int accumulate = 0, bool tf32 = false);
void umma_layer_release(qlc_layer *layer);
int attention_tc_forward(qlc_ctx *ctx, const __nv_bfloat16 *qr, const __nv_bfloat16 *kr, const __nv_bfloat16 *v, float *o,
                         __nv_bfloat16 *o_b, float *lse, size_t n_seq, size_t seq_len, size_t heads, size_t kv_heads);
int attention_tc_backward(qlc_ctx *ctx, const __nv_bfloat16 *qr, const __nv_bfloat16 *kr, const __nv_bfloat16 *v,
                          const float *o, const float *d_o, const __nv_bfloat16 *o_b, __nv_bfloat16 *d_o_b, const float *lse,
                          float *delta, float *dqr, float *dkr, float *dv, __nv_bfloat16 *dv_b, float *dk_parts, float *dv_parts,
                          size_t n_seq, size_t seq_len, size_t heads, size_t kv_heads, qlc_ctx *dq_ctx = nullptr,
                          cudaEvent_t ev_fork = nullptr, cudaEvent_t ev_join = nullptr);
size_t attention_tc_stat_stride(size_t seq_len);
int attention_tc_init_stats(qlc_ctx *ctx, float *lse, float *delta, size_t n_seq, size_t seq_len, size_t heads);
// ---- programmatic dependent launch ------------------------------------------------------------------------------
// A kernel launched through launch_pdl may start while the kernel before it in the stream is still running: its
// CTAs are scheduled as SMs free up, run whatever precedes pdl_wait() (barrier set-up, TMEM allocation), and
// pdl_wait() then blocks until the earlier kernel has completed and its writes are visible.  Every kernel
// launched this way calls pdl_wait() before its first access to memory another kernel may have written, and
// pdl_trigger() at its top so that the kernel after it gets the same head start.  In a kernel launched the plain
// way both are no-ops.  Environment variable QLC_NO_PDL turns the attribute off (diagnostics).
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled();
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

int make_map_bf16(void *map_out, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows);
int umma_gemm_bf16(qlc_ctx *ctx, const __nv_bfloat16 *d_a, const __nv_bfloat16 *d_b, bool b_is_kn, void *d_c, size_t M,
                   size_t N, size_t K, bool c_bf16 = false);
int umma_qlora_forward_noalloc(qlc_ctx *ctx, qlc_layer *layer, const __nv_bfloat16 *d_x, size_t batch, void *d_y);

// Scratch arena: returns a pointer to at least `bytes` bytes of device scratch (256-B aligned).
// The arena is a single region; callers carve it up themselves.  May reallocate (synchronises).
int ctx_workspace(qlc_ctx *ctx, size_t bytes, void **out);
int ctx_pinned(qlc_ctx *ctx, size_t bytes, void **out);
int ctx_io(qlc_ctx *ctx, size_t bytes, void **out);
int ctx_tile_counters(qlc_ctx *ctx, int set, size_t count, int **out);
int layer_tf32_operands(qlc_layer *layer);
// A layer that multiplies by a plain (out_dim, in_dim) fp32 device matrix, copied; no quantisation, no adapter.
int layer_create_raw(qlc_ctx *ctx, const float *d_weight, size_t out_dim, size_t in_dim, qlc_layer **out);
// Event bracketing of a launch when profiling is enabled (no-ops otherwise).
void prof_begin(qlc_ctx *ctx, int slot, cudaStream_t stream = nullptr);
void prof_end(qlc_ctx *ctx, cudaStream_t stream = nullptr);

}  // namespace qlc
