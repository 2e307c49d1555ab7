// fp32 SIMT GEMMs that reproduce the reference's CPU arithmetic bit-for-bit, for any shape,
// block size and scale format.  They back the plain gpu_matmul* entry points and the
// QloraLinear passes whenever the tensor-core path does not apply (or FP32_EXACT is selected).
//
// Bit-exactness rests on three facts about the reference loops (qlora-core/src/lora.rs):
//   matmul          :129-142  c[i][j] starts at 0 and receives a[i][p]*b[p][j] for p ascending;
//   matmul_trans_a  :148-162  acc = 0; acc += a[p][i]*b[p][j] for p ascending;
//   matmul_trans_b  :169-183  acc = 0; acc += a[i][p]*b[j][p] for p ascending;
// i.e. every output is a sequential fp32 sum over the contraction index with separately rounded
// multiply and add (Rust never fuses them).  The kernels below keep exactly that order per
// output (tiles are visited with p ascending, the ragged last tile is not padded) and use
// __fmul_rn/__fadd_rn; this file is also compiled with -fmad=false.
#include "common.cuh"

namespace qlc {
namespace {

__constant__ float c_nf4_levels_x[16] = {
    (float)-1.0,
    (float)-0.6961928009986877,
    (float)-0.5250730514526367,
    (float)-0.39491748809814453,
    (float)-0.28444138169288635,
    (float)-0.18477343022823334,
    (float)-0.09105003625154495,
    (float)0.0,
    (float)0.07958029955625534,
    (float)0.16093020141124725,
    (float)0.24611230194568634,
    (float)0.33791524171829224,
    (float)0.44070982933044434,
    (float)0.5626170039176941,
    (float)0.7229568362236023,
    (float)1.0,
};

// Element accessors: operator()(row, col) of the logical operand.
struct RowMajor {  // M(r, c) = p[r * ld + c]
    const float *p;
    size_t ld;
    __device__ __forceinline__ float operator()(size_t r, size_t c) const { return p[r * ld + c]; }
};
struct Transposed {  // M(r, c) = p[c * ld + r]
    const float *p;
    size_t ld;
    __device__ __forceinline__ float operator()(size_t r, size_t c) const { return p[c * ld + r]; }
};
// Dequantised weight element idx = NF4_LEVELS[nibble] * scale[idx / block] (quant.rs:157-167),
// with the per-block scales already decoded exactly as block_scales() does (quant.rs:212-221).
struct DequantW {
    const uint8_t *codes;
    const float *scales;
    size_t block_size;
    __device__ __forceinline__ float at(size_t idx) const {
        const uint32_t byte = codes[idx >> 1];
        const uint32_t c = (idx & 1) ? (byte >> 4) : (byte & 15u);
        return __fmul_rn(c_nf4_levels_x[c], scales[idx / block_size]);
    }
};
struct DequantRowMajor {  // W(r, c), W stored (rows, ld)
    DequantW w;
    size_t ld;
    __device__ __forceinline__ float operator()(size_t r, size_t c) const { return w.at(r * ld + c); }
};
struct DequantTransposed {  // W^T(r, c) = W(c, r)
    DequantW w;
    size_t ld;
    __device__ __forceinline__ float operator()(size_t r, size_t c) const { return w.at(c * ld + r); }
};

// C(M,N)[i][j] = sum_{p=0..K-1} A(i,p) * B(p,j), sequential in p.
template <class LA, class LB>
__global__ void __launch_bounds__(256)
exact_gemm_kernel(LA la, LB lb, size_t M, size_t N, size_t K, float *__restrict__ C) {
    __shared__ float sa[16][17];
    __shared__ float sb[16][17];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t row = (size_t)blockIdx.y * 16 + ty;
    const size_t col = (size_t)blockIdx.x * 16 + tx;
    float acc = 0.0f;
    for (size_t p0 = 0; p0 < K; p0 += 16) {
        sa[ty][tx] = (row < M && p0 + tx < K) ? la(row, p0 + tx) : 0.0f;
        sb[ty][tx] = (p0 + ty < K && col < N) ? lb(p0 + ty, col) : 0.0f;
        __syncthreads();
        const int pmax = (K - p0 < 16) ? (int)(K - p0) : 16;
        for (int p = 0; p < pmax; ++p) acc = __fadd_rn(acc, __fmul_rn(sa[ty][p], sb[p][tx]));
        __syncthreads();
    }
    if (row < M && col < N) C[row * N + col] = acc;
}

template <class LA, class LB>
int launch_exact(qlc_ctx *ctx, LA la, LB lb, size_t M, size_t N, size_t K, float *C) {
    if (M == 0 || N == 0) return QLC_OK;
    const size_t gx = ceil_div(N, 16), gy = ceil_div(M, 16);
    if (gy > 65535) return fail(QLC_ERR_GPU, "exact GEMM: %zu output rows exceed the launch limit", M);
    dim3 grid((unsigned)gx, (unsigned)gy);
    exact_gemm_kernel<LA, LB><<<grid, 256, 0, ctx->stream>>>(la, lb, M, N, K, C);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

__global__ void scale_kernel(const float *__restrict__ in, float s, float *__restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(in[i], s);
}
// y += t * s   (lora.rs:98-101 then qlora.rs:101-105)
__global__ void add_scaled_kernel(float *__restrict__ y, const float *__restrict__ t, float s, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(y[i], __fmul_rn(t[i], s));
}
// g += d   (qlora.rs:154-156)
__global__ void add_kernel(float *__restrict__ g, const float *__restrict__ d, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) g[i] = __fadd_rn(g[i], d[i]);
}

inline unsigned g1(size_t n) { return (unsigned)ceil_div(n, 256); }
inline size_t align256(size_t b) { return (b + 255) & ~(size_t)255; }

}  // namespace

int exact_matmul(qlc_ctx *ctx, const float *a, const float *b, size_t m, size_t k, size_t n, float *c) {
    return launch_exact(ctx, RowMajor{a, k}, RowMajor{b, n}, m, n, k, c);
}
int exact_matmul_trans_b(qlc_ctx *ctx, const float *a, const float *b, size_t m, size_t k, size_t n, float *c) {
    return launch_exact(ctx, RowMajor{a, k}, Transposed{b, k}, m, n, k, c);
}
// C(k,n) = A(m,k)^T · B(m,n): output rows = k, contraction = m.
int exact_matmul_trans_a(qlc_ctx *ctx, const float *a, const float *b, size_t m, size_t k, size_t n, float *c) {
    return launch_exact(ctx, Transposed{a, k}, RowMajor{b, n}, k, n, m, c);
}

// QloraLinear::forward (qlora.rs:86-107) in the reference's exact order.
int exact_qlora_forward(qlc_ctx *ctx, qlc_layer *L, const float *x, size_t batch, float *y) {
    // raw projection: Y = X·W^T on the fp32 weight (qlora-model/src/llama.rs:101-105)
    if (!L->w) return exact_matmul_trans_b(ctx, x, L->d_w_raw, batch, L->in_dim, L->out_dim, y);
    const qlc_qtensor *q = L->w;
    const size_t in = L->in_dim, out = L->out_dim, r = L->r;
    const size_t b_scales = align256(q->nb * 4), b_t1 = align256(batch * r * 4), b_t2 = align256(batch * out * 4);
    void *ws = nullptr;
    QLC_TRY(ctx_workspace(ctx, b_scales + b_t1 + b_t2, &ws));
    float *scales = static_cast<float *>(ws);
    float *t1 = reinterpret_cast<float *>(static_cast<char *>(ws) + b_scales);
    float *t2 = reinterpret_cast<float *>(static_cast<char *>(ws) + b_scales + b_t1);
    QLC_TRY(launch_decode_block_scales(ctx, q, scales));
    DequantW dw{q->d_codes, scales, q->block_size};
    QLC_TRY(launch_exact(ctx, RowMajor{x, in}, DequantTransposed{dw, in}, batch, out, in, y));
    if (r > 0 && batch * out > 0) {
        QLC_TRY(exact_matmul_trans_b(ctx, x, L->d_a, batch, in, r, t1));
        QLC_TRY(exact_matmul_trans_b(ctx, t1, L->d_b, batch, r, out, t2));
        const float s = L->alpha / (float)r;  // lora.rs:64-66
        add_scaled_kernel<<<g1(batch * out), 256, 0, ctx->stream>>>(y, t2, s, batch * out);
        ctx->launches += 1;
        QLC_CUDA(cudaGetLastError());
    }
    return QLC_OK;
}

// QloraLinear::backward (qlora.rs:116-165) in the reference's exact order.
int exact_qlora_backward(qlc_ctx *ctx, qlc_layer *L, const float *x, const float *dy, size_t batch, float *gx,
                         float *ga, float *gb) {
    // raw projection: dX = dY·W (qlora-model/src/llama.rs:119-123)
    if (!L->w) return exact_matmul(ctx, dy, L->d_w_raw, batch, L->out_dim, L->in_dim, gx);
    const qlc_qtensor *q = L->w;
    const size_t in = L->in_dim, out = L->out_dim, r = L->r;
    const size_t b_scales = align256(q->nb * 4), b_dys = align256(batch * out * 4), b_t1 = align256(batch * r * 4),
                 b_ds = align256(batch * r * 4), b_dxl = align256(batch * in * 4), b_ga = align256(r * in * 4),
                 b_gb = align256(out * r * 4);
    void *ws = nullptr;
    QLC_TRY(ctx_workspace(ctx, b_scales + b_dys + b_t1 + b_ds + b_dxl + b_ga + b_gb, &ws));
    char *p = static_cast<char *>(ws);
    float *scales = reinterpret_cast<float *>(p); p += b_scales;
    float *dys = reinterpret_cast<float *>(p); p += b_dys;
    float *t1 = reinterpret_cast<float *>(p); p += b_t1;
    float *ds = reinterpret_cast<float *>(p); p += b_ds;
    float *dxl = reinterpret_cast<float *>(p); p += b_dxl;
    float *ga_tmp = reinterpret_cast<float *>(p); p += b_ga;
    float *gb_tmp = reinterpret_cast<float *>(p);
    QLC_TRY(launch_decode_block_scales(ctx, q, scales));
    DequantW dw{q->d_codes, scales, q->block_size};
    // grad_x = dY · W
    QLC_TRY(launch_exact(ctx, RowMajor{dy, out}, DequantRowMajor{dw, in}, batch, in, out, gx));
    if (r == 0) return QLC_OK;
    if (!ga) ga = ga_tmp;
    if (!gb) gb = gb_tmp;
    const float s = L->alpha / (float)r;
    if (batch * out > 0) {
        scale_kernel<<<g1(batch * out), 256, 0, ctx->stream>>>(dy, s, dys, batch * out);
        ctx->launches += 1;
        QLC_CUDA(cudaGetLastError());
    }
    QLC_TRY(exact_matmul_trans_b(ctx, x, L->d_a, batch, in, r, t1));   // T1 = X·A^T
    QLC_TRY(exact_matmul_trans_a(ctx, dys, t1, batch, out, r, gb));    // dB = dYs^T·T1
    QLC_TRY(exact_matmul(ctx, dys, L->d_b, batch, out, r, ds));        // Ds = dYs·B
    QLC_TRY(exact_matmul_trans_a(ctx, ds, x, batch, r, in, ga));       // dA = Ds^T·X
    QLC_TRY(exact_matmul(ctx, ds, L->d_a, batch, r, in, dxl));         // Ds·A
    if (batch * in > 0) {
        add_kernel<<<g1(batch * in), 256, 0, ctx->stream>>>(gx, dxl, batch * in);
        ctx->launches += 1;
        QLC_CUDA(cudaGetLastError());
    }
    return QLC_OK;
}

}  // namespace qlc
