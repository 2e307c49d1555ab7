// Llama decoder around the QLoRA linears: the caller of the hot path (qlora-model/src/llama.rs).
//
// Reference semantics reproduced here:
//   llama.rs:310-326  forward   embedding gather, decoder blocks, final RMSNorm, tied LM head
//   llama.rs:385-412  backward  only adapter matrices get gradients; base weights are frozen
//   llama.rs:417-468  block     x += O(attn(RoPE(Q(n1 x)), RoPE(K(n1 x)), V(n1 x)));  x += Down(silu(Gate(n2 x)) * Up(n2 x))
//   llama.rs:605-630  rmsnorm_backward (dx only: norm weights are frozen)
//   llama.rs:633-792  causal grouped-query attention with rotate-half RoPE, and its backward
//   llama.rs:487-514  softmax cross-entropy, mean over positions
// The reference runs one sequence at a time in scalar fp32 on the CPU.  Here n_seq sequences of equal length
// share the row dimension of every linear (token t = sequence * seq_len + position), the seven projections of
// a block are QloraLinear layers of this library (NF4 weights, tensor-core or exact path as the context's
// precision says), and everything between them is the CUDA below, in fp32.  Head dimension 64 only.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <new>
#include <vector>

#include <chrono>

#include "common.cuh"

namespace qlc {
namespace {

constexpr int kHeadDim = 64;

// ---- small row-wise kernels ----------------------------------------------------------------------
__global__ void embed_gather_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ embed,
                                    float *__restrict__ x, size_t tokens, int h, uint32_t vocab) {
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    if (t >= tokens) return;
    const uint32_t id = ids[t] < vocab ? ids[t] : vocab - 1;  // ids are validated on the host; never read outside
    for (int j = threadIdx.x; j < h; j += blockDim.x) x[t * h + j] = embed[(size_t)id * h + j];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// y = x / sqrt(mean(x^2) + eps) * w, one warp per row (llama.rs:730-740).  With `res` the row normalised is
// x + res (the residual addition before the norm, llama.rs:447, 461), and the sum is stored to `sum_out`.
// The result goes to y (fp32) and / or y_b (bf16).
__global__ void rmsnorm_fwd_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps,
                                   float *__restrict__ y, size_t rows, int h, __nv_bfloat16 *__restrict__ y_b,
                                   const float *__restrict__ res, float *__restrict__ sum_out) {
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float *xr = x + row * h;
    float ss = 0.0f;
    if (res) {
        for (int j = lane; j < h; j += 32) {
            const float v = xr[j] + res[row * h + j];
            sum_out[row * h + j] = v;
            ss += v * v;
        }
        xr = sum_out + row * h;  // each lane re-reads only what it wrote itself
    } else {
        for (int j = lane; j < h; j += 32) ss += xr[j] * xr[j];
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)h + eps);
    for (int j = lane; j < h; j += 32) {
        const float v = xr[j] * r * w[j];
        if (y) y[row * h + j] = v;
        if (y_b) y_b[row * h + j] = __float2bfloat16_rn(v);
    }
}

// dx = dy*w*r + 2*x/h*ds with ds = sum(dy*x*w) * (-0.5) / ss * r  (llama.rs:605-630); out = dx (+ add)
__global__ void rmsnorm_bwd_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                   const float *__restrict__ dy, float eps, const float *__restrict__ add,
                                   float *__restrict__ out, size_t rows, int h, __nv_bfloat16 *__restrict__ out_b,
                                   const float *__restrict__ dy2, const float *__restrict__ dy3,
                                   float *__restrict__ dy_sum) {
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float *xr = x + row * h, *dyr = dy + row * h;
    float sq = 0.0f, dot = 0.0f;
    if (dy2) {
        // the gradient of the normalised row is the sum of the gradients from the linears that read it
        // (llama.rs:571-573, 597-599); the sum is kept in dy_sum, each lane re-reading only its own elements
        for (int j = lane; j < h; j += 32) {
            float d = dyr[j] + dy2[row * h + j];
            if (dy3) d += dy3[row * h + j];
            dy_sum[row * h + j] = d;
            sq += xr[j] * xr[j];
            dot += d * xr[j] * w[j];
        }
        dyr = dy_sum + row * h;
    } else {
        for (int j = lane; j < h; j += 32) {
            sq += xr[j] * xr[j];
            dot += dyr[j] * xr[j] * w[j];
        }
    }
    sq = warp_sum(sq);
    dot = warp_sum(dot);
    const float ss = sq / (float)h + eps;
    const float r = 1.0f / sqrtf(ss);
    const float ds = dot * (-0.5f / ss * r);
    for (int j = lane; j < h; j += 32) {
        const float v = dyr[j] * w[j] * r + 2.0f * xr[j] / (float)h * ds;
        const float res = add ? v + add[row * h + j] : v;
        out[row * h + j] = res;
        if (out_b) out_b[row * h + j] = __float2bfloat16_rn(res);  // the next linear's dY operand
    }
}

// The two norm kernels of the bf16 pipeline (h is a multiple of 64, so every lane handles h / 64 element pairs).
// Forward: s = x + res (res is a branch output, bf16; null for the very first norm), stored to sum_out when res
// is given; y_b = bf16(s / rms(s) * w), optionally also y (fp32).
__global__ void pipe_norm_fwd_kernel(const float2 *__restrict__ x, const __nv_bfloat162 *__restrict__ res,
                                     float2 *__restrict__ sum_out, const float2 *__restrict__ w, float eps,
                                     float2 *__restrict__ y, __nv_bfloat162 *__restrict__ y_b, size_t rows, int h2) {
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float2 *xr = x + row * h2;
    float ss = 0.0f;
    if (res) {
        for (int j = lane; j < h2; j += 32) {
            const float2 a = xr[j], b = __bfloat1622float2(res[row * h2 + j]);
            const float2 v = make_float2(a.x + b.x, a.y + b.y);
            sum_out[row * h2 + j] = v;
            ss += v.x * v.x + v.y * v.y;
        }
        xr = sum_out + row * h2;  // each lane re-reads only what it wrote itself
    } else {
        for (int j = lane; j < h2; j += 32) {
            const float2 a = xr[j];
            ss += a.x * a.x + a.y * a.y;
        }
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)(2 * h2) + eps);
    for (int j = lane; j < h2; j += 32) {
        const float2 a = xr[j], g = w[j];
        const float2 v = make_float2(a.x * r * g.x, a.y * r * g.y);
        if (y) y[row * h2 + j] = v;
        if (y_b) y_b[row * h2 + j] = __floats2bfloat162_rn(v.x, v.y);
    }
}
// Backward: dy = dy1 + dy2 (+ dy3), the bf16 input gradients of the linears that read the normalised row;
// out = rmsnorm_backward(x, dy) + add (the residual gradient), out_b its bf16 copy (the next linear's dY).
__global__ void pipe_norm_bwd_kernel(const float2 *__restrict__ x, const float2 *__restrict__ w,
                                     const __nv_bfloat162 *__restrict__ dy1, const __nv_bfloat162 *__restrict__ dy2,
                                     const __nv_bfloat162 *__restrict__ dy3, float eps, const float2 *__restrict__ add,
                                     float2 *__restrict__ out, __nv_bfloat162 *__restrict__ out_b, size_t rows, int h2) {
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const size_t at = row * h2;
    auto dy_at = [&](int j) {
        float2 d = __bfloat1622float2(dy1[at + j]);
        if (dy2) {
            const float2 e = __bfloat1622float2(dy2[at + j]);
            d.x += e.x;
            d.y += e.y;
        }
        if (dy3) {
            const float2 f = __bfloat1622float2(dy3[at + j]);
            d.x += f.x;
            d.y += f.y;
        }
        return d;
    };
    float sq = 0.0f, dot = 0.0f;
    for (int j = lane; j < h2; j += 32) {
        const float2 a = x[at + j], g = w[j], d = dy_at(j);
        sq += a.x * a.x + a.y * a.y;
        dot += d.x * a.x * g.x + d.y * a.y * g.y;
    }
    sq = warp_sum(sq);
    dot = warp_sum(dot);
    const float h = (float)(2 * h2);
    const float ss = sq / h + eps;
    const float r = 1.0f / sqrtf(ss);
    const float ds = dot * (-0.5f / ss * r);
    for (int j = lane; j < h2; j += 32) {
        const float2 a = x[at + j], g = w[j], d = dy_at(j), q = add[at + j];
        const float2 v = make_float2(d.x * g.x * r + 2.0f * a.x / h * ds + q.x, d.y * g.y * r + 2.0f * a.y / h * ds + q.y);
        out[at + j] = v;
        out_b[at + j] = __floats2bfloat162_rn(v.x, v.y);
    }
}

// Rotate-half RoPE on (tokens, heads, 64) (llama.rs:814-820); inverse applies the transposed rotation
// (llama.rs:706-724).  Position = token index modulo seq_len.
__device__ __forceinline__ float as_f32(float v) { return v; }
__device__ __forceinline__ float as_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename TIn>
__global__ void rope_kernel(const TIn *__restrict__ x, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                            float *__restrict__ y, size_t tokens, int heads, int seq_len, int inverse,
                            __nv_bfloat16 *__restrict__ yb) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (token, head, pair)
    const size_t total = tokens * heads * (kHeadDim / 2);
    if (i >= total) return;
    const int j = (int)(i % (kHeadDim / 2));
    const size_t th = i / (kHeadDim / 2);
    const size_t t = th / heads;
    const int pos = (int)(t % seq_len);
    const float c = cos_t[pos * (kHeadDim / 2) + j], s0 = sin_t[pos * (kHeadDim / 2) + j];
    const float s = inverse ? -s0 : s0;
    const float a = as_f32(x[th * kHeadDim + j]), b = as_f32(x[th * kHeadDim + j + kHeadDim / 2]);
    const float lo = a * c - b * s, hi = b * c + a * s;
    if (y) {
        y[th * kHeadDim + j] = lo;
        y[th * kHeadDim + j + kHeadDim / 2] = hi;
    }
    if (yb) {  // bf16 copy for the tensor-core attention kernels
        yb[th * kHeadDim + j] = __float2bfloat16_rn(lo);
        yb[th * kHeadDim + j + kHeadDim / 2] = __float2bfloat16_rn(hi);
    }
}

__global__ void swiglu_fwd_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ act,
                                  size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i];
    act[i] = g / (1.0f + expf(-g)) * up[i];  // silu(g) * u  (llama.rs:455-457, 516-518)
}
__global__ void swiglu_bwd_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                  const float *__restrict__ d_act, float *__restrict__ dg, float *__restrict__ du, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i], s = 1.0f / (1.0f + expf(-g));
    dg[i] = d_act[i] * up[i] * (s * (1.0f + g * (1.0f - s)));  // llama.rs:557-560, 524-528
    du[i] = d_act[i] * (g * s);
}
// The same two on bf16 storage, 8 elements per thread (n is a multiple of 8: the MLP width is a multiple of 64).
__device__ __forceinline__ void unpack8(const uint4 &u, float (&f)[8]) {
    const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
}
// The pipeline's RoPE: q and k in one launch, bf16 out, eight pairs per thread (128-bit accesses).  Thread
// (token, head, j8) rotates elements 8*j8 .. 8*j8 + 7 of the head's low half against the same elements of its high
// half; heads 0 .. heads-1 are q's, the following kv_heads are k's.
__device__ __forceinline__ void load8(const float *p, float (&f)[8]) {
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <typename TIn>
__global__ void rope_qk_kernel(const TIn *__restrict__ xq, const TIn *__restrict__ xk, const float *__restrict__ cos_t,
                               const float *__restrict__ sin_t, __nv_bfloat16 *__restrict__ yq, __nv_bfloat16 *__restrict__ yk,
                               size_t tokens, int heads, int kv_heads, int seq_len, int inverse) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_token = (heads + kv_heads) * 4;
    if (i >= tokens * per_token) return;
    const size_t t = i / per_token;
    const int rem = (int)(i % per_token), hh = rem >> 2, j0 = (rem & 3) * 8;
    const bool is_q = hh < heads;
    const size_t at = is_q ? (t * heads + hh) * kHeadDim + j0 : (t * kv_heads + (hh - heads)) * kHeadDim + j0;
    const TIn *x = is_q ? xq : xk;
    __nv_bfloat16 *y = is_q ? yq : yk;
    const int pos = (int)(t % seq_len);
    float a[8], b[8], c[8], sn[8], lo[8], hi[8];
    load8(x + at, a);
    load8(x + at + kHeadDim / 2, b);
    load8(cos_t + pos * (kHeadDim / 2) + j0, c);
    load8(sin_t + pos * (kHeadDim / 2) + j0, sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float s1 = inverse ? -sn[e] : sn[e];
        lo[e] = a[e] * c[e] - b[e] * s1;
        hi[e] = b[e] * c[e] + a[e] * s1;
    }
    *reinterpret_cast<uint4 *>(y + at) = pack8(lo);
    *reinterpret_cast<uint4 *>(y + at + kHeadDim / 2) = pack8(hi);
}

// End of the attention backward pass in the bf16 pipeline, one launch: dq = inverse RoPE of dqr; dk = inverse RoPE
// of (sum of the group's per-head dK partials, in head order) / sqrt(64); dv = sum of the dV partials; all three
// written as bf16, the dY operands of the q / k / v projections' backward GEMMs.  Thread layout as rope_qk_kernel,
// plus a third range of threads for dv (8 values each).
__global__ void attn_bwd_finish_kernel(const float *__restrict__ dqr, const float *__restrict__ dk_parts,
                                       const float *__restrict__ dv_parts, size_t part_stride, int parts,
                                       const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                       __nv_bfloat16 *__restrict__ dq_b, __nv_bfloat16 *__restrict__ dk_b,
                                       __nv_bfloat16 *__restrict__ dv_b, size_t tokens, int heads, int kv_heads, int seq_len,
                                       size_t ld_q, size_t ld_kv) {  // row strides of dq_b and of dk_b / dv_b (elements)
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_token = (heads + kv_heads) * 4 + kv_heads * 8;
    if (i >= tokens * per_token) return;
    const size_t t = i / per_token;
    const int rem = (int)(i % per_token);
    if (rem >= (heads + kv_heads) * 4) {  // dv: plain sum
        const size_t at = t * kv_heads * kHeadDim + (size_t)(rem - (heads + kv_heads) * 4) * 8;
        float acc[8], x[8];
        load8(dv_parts + at, acc);
        for (int p = 1; p < parts; ++p) {
            load8(dv_parts + (size_t)p * part_stride + at, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += x[e];
        }
        *reinterpret_cast<uint4 *>(dv_b + t * ld_kv + (size_t)(rem - (heads + kv_heads) * 4) * 8) = pack8(acc);
        return;
    }
    const int hh = rem >> 2, j0 = (rem & 3) * 8;
    const bool is_q = hh < heads;
    const size_t at = is_q ? (t * heads + hh) * kHeadDim + j0 : (t * kv_heads + (hh - heads)) * kHeadDim + j0;
    float a[8], b[8], c[8], sn[8], lo[8], hi[8];
    if (is_q) {
        load8(dqr + at, a);
        load8(dqr + at + kHeadDim / 2, b);
    } else {
        float x[8];
        load8(dk_parts + at, a);
        load8(dk_parts + at + kHeadDim / 2, b);
        for (int p = 1; p < parts; ++p) {
            load8(dk_parts + (size_t)p * part_stride + at, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] += x[e];
            load8(dk_parts + (size_t)p * part_stride + at + kHeadDim / 2, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) b[e] += x[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a[e] *= 0.125f;
            b[e] *= 0.125f;
        }
    }
    const int pos = (int)(t % seq_len);
    load8(cos_t + pos * (kHeadDim / 2) + j0, c);
    load8(sin_t + pos * (kHeadDim / 2) + j0, sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) {  // the transposed rotation (llama.rs:706-724)
        lo[e] = a[e] * c[e] + b[e] * sn[e];
        hi[e] = b[e] * c[e] - a[e] * sn[e];
    }
    __nv_bfloat16 *y = is_q ? dq_b + t * ld_q + (size_t)hh * kHeadDim + j0 : dk_b + t * ld_kv + (size_t)(hh - heads) * kHeadDim + j0;
    *reinterpret_cast<uint4 *>(y) = pack8(lo);
    *reinterpret_cast<uint4 *>(y + kHeadDim / 2) = pack8(hi);
}

// Forward RoPE of the merged q | k | v projection's output (rows of ld elements: q heads, k heads, v heads): q and k
// rotated into their own matrices, v copied into its own (the attention kernels read three dense matrices).
__global__ void rope_qkv_kernel(const __nv_bfloat16 *__restrict__ qkv, size_t ld, const float *__restrict__ cos_t,
                                const float *__restrict__ sin_t, __nv_bfloat16 *__restrict__ yq, __nv_bfloat16 *__restrict__ yk,
                                __nv_bfloat16 *__restrict__ yv, size_t tokens, int heads, int kv_heads, int seq_len) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_token = (heads + kv_heads) * 4 + kv_heads * 8;
    if (i >= tokens * per_token) return;
    const size_t t = i / per_token;
    const int rem = (int)(i % per_token);
    const __nv_bfloat16 *row = qkv + t * ld;
    if (rem >= (heads + kv_heads) * 4) {  // v: 8 values per thread
        const size_t c = (size_t)(rem - (heads + kv_heads) * 4) * 8;
        *reinterpret_cast<uint4 *>(yv + t * kv_heads * kHeadDim + c) =
            *reinterpret_cast<const uint4 *>(row + (size_t)(heads + kv_heads) * kHeadDim + c);
        return;
    }
    const int hh = rem >> 2, j0 = (rem & 3) * 8;
    const bool is_q = hh < heads;
    const __nv_bfloat16 *x = row + (size_t)hh * kHeadDim + j0;  // k heads follow the q heads in the row
    __nv_bfloat16 *y = is_q ? yq + (t * heads + hh) * kHeadDim + j0 : yk + (t * kv_heads + (hh - heads)) * kHeadDim + j0;
    const int pos = (int)(t % seq_len);
    float a[8], b[8], c[8], sn[8], lo[8], hi[8];
    load8(x, a);
    load8(x + kHeadDim / 2, b);
    load8(cos_t + pos * (kHeadDim / 2) + j0, c);
    load8(sin_t + pos * (kHeadDim / 2) + j0, sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        lo[e] = a[e] * c[e] - b[e] * sn[e];
        hi[e] = b[e] * c[e] + a[e] * sn[e];
    }
    *reinterpret_cast<uint4 *>(y) = pack8(lo);
    *reinterpret_cast<uint4 *>(y + kHeadDim / 2) = pack8(hi);
}

// The merged q | k | v layer's adapter operands (zero-padded bf16 A, B and B^T) from the projections' own fp32 A / B:
// A_m stacks the A matrices, B_m holds each B in its rows and rank columns, zeros elsewhere.
struct QkvRefresh {
    const float *a[3], *b[3];
    uint32_t r[3], out[3];  // ranks and output widths of q, k, v
    __nv_bfloat16 *a_pad, *b_pad, *bt_pad;
    uint32_t r_pad, in_dim, out_m;
};
constexpr int kQkvBatch = 24;
struct QkvRefreshBatch {
    int n;
    QkvRefresh d[kQkvBatch];
};
__global__ void qkv_refresh_kernel(const QkvRefreshBatch batch) {
    pdl_trigger();
    pdl_wait();
    const QkvRefresh &d = batch.d[blockIdx.y];
    const size_t na = (size_t)d.r_pad * d.in_dim, nb = (size_t)d.out_m * d.r_pad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < na + 2 * nb; i += (size_t)gridDim.x * blockDim.x) {
        float val = 0.0f;
        if (i < na) {
            const uint32_t r = (uint32_t)(i / d.in_dim), c = (uint32_t)(i % d.in_dim);
            uint32_t r0 = 0;
            for (int sgm = 0; sgm < 3; ++sgm) {
                if (r < r0 + d.r[sgm]) {
                    val = d.a[sgm][(size_t)(r - r0) * d.in_dim + c];
                    break;
                }
                r0 += d.r[sgm];
            }
            d.a_pad[i] = __float2bfloat16_rn(val);
            continue;
        }
        const bool transposed = i >= na + nb;
        const size_t j = i - na - (transposed ? nb : 0);
        const uint32_t row = transposed ? (uint32_t)(j % d.out_m) : (uint32_t)(j / d.r_pad);
        const uint32_t c = transposed ? (uint32_t)(j / d.out_m) : (uint32_t)(j % d.r_pad);
        uint32_t o0 = 0, r0 = 0;
        for (int sgm = 0; sgm < 3; ++sgm) {
            if (row < o0 + d.out[sgm]) {
                if (c >= r0 && c < r0 + d.r[sgm]) val = d.b[sgm][(size_t)(row - o0) * d.r[sgm] + (c - r0)];
                break;
            }
            o0 += d.out[sgm];
            r0 += d.r[sgm];
        }
        (transposed ? d.bt_pad : d.b_pad)[j] = __float2bfloat16_rn(val);
    }
}

// The merged layer's adapter gradients back into the projections' own gradient buckets (grad_A, then grad_B):
// grad_A of a projection is its rows of the merged grad_A; grad_B its rows and rank columns of the merged grad_B.
struct QkvScatter {
    const float *ga_m, *gb_m;
    float *bucket[3];
    uint32_t r[3], out[3];
    uint32_t r_m, in_dim;
};
struct QkvScatterBatch {
    int n;
    QkvScatter d[kQkvBatch];
};
__global__ void qkv_scatter_kernel(const QkvScatterBatch batch) {
    pdl_trigger();
    pdl_wait();
    const QkvScatter &d = batch.d[blockIdx.y];
    size_t total = 0;
    for (int sgm = 0; sgm < 3; ++sgm) total += (size_t)d.r[sgm] * (d.in_dim + d.out[sgm]);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t k = i;
        uint32_t o0 = 0, r0 = 0;
        for (int sgm = 0; sgm < 3; ++sgm) {
            const size_t na = (size_t)d.r[sgm] * d.in_dim, nb = (size_t)d.out[sgm] * d.r[sgm];
            if (k < na + nb) {
                if (k < na) {
                    d.bucket[sgm][k] = d.ga_m[(size_t)r0 * d.in_dim + k];  // rows r0.. of the merged grad_A, contiguous
                } else {
                    const size_t j = k - na, row = j / d.r[sgm], c = j % d.r[sgm];
                    d.bucket[sgm][k] = d.gb_m[(size_t)(o0 + row) * d.r_m + r0 + c];
                }
                break;
            }
            k -= na + nb;
            o0 += d.out[sgm];
            r0 += d.r[sgm];
        }
    }
}

// gate / up (and dg / du below) are read with a row stride of ld8 16-byte words, cols8 words per row: two (T, I)
// matrices (ld8 == cols8) or the two halves of one (T, 2I) matrix (ld8 == 2 * cols8); act and d_act are (T, I).
__global__ void swiglu_fwd_bf16_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up, uint4 *__restrict__ act,
                                       size_t n8, uint32_t cols8, uint32_t ld8) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const size_t row = i / cols8, at = row * ld8 + (i - row * cols8);
    float g[8], u[8], a[8];
    unpack8(gate[at], g);
    unpack8(up[at], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = g[e] / (1.0f + __expf(-g[e])) * u[e];
    act[i] = pack8(a);
}
__global__ void swiglu_bwd_bf16_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up,
                                       const uint4 *__restrict__ d_act, uint4 *__restrict__ dg, uint4 *__restrict__ du,
                                       size_t n8, uint32_t cols8, uint32_t ld8) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const size_t row = i / cols8, at = row * ld8 + (i - row * cols8);
    float g[8], u[8], d[8], og[8], ou[8];
    unpack8(gate[at], g);
    unpack8(up[at], u);
    unpack8(d_act[i], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float sg = 1.0f / (1.0f + __expf(-g[e]));
        og[e] = d[e] * u[e] * (sg * (1.0f + g[e] * (1.0f - sg)));
        ou[e] = d[e] * (g[e] * sg);
    }
    dg[at] = pack8(og);
    du[at] = pack8(ou);
}
// out may be one of the inputs (element i only depends on element i)
__global__ void add_kernel(const float *a, const float *b, const float *c, float *out, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = c ? a[i] + b[i] + c[i] : a[i] + b[i];
}

// ---- attention (causal, grouped-query, head dim 64) ----------------------------------------------------
// Layout: q / o / dq are (tokens, heads*64), k / v / dk / dv are (tokens, kv_heads*64); rows of one sequence
// are contiguous.  A CTA owns 64 consecutive positions of one (sequence, head).
constexpr int kAttnRows = 64, kAttnThreads = 256;

// ---- register-tiled products -----------------------------------------------------------------------------------
// The attention kernels below work on 64 x 64 tiles with 256 threads arranged 16 x 16: thread (ty, tx) owns the
// 4 x 4 block (rows 4ty.., columns 4tx..) of every product, and a product C = A·B^T is computed from the two
// operands stored TRANSPOSED in shared memory ([contraction index][row]), so that one 128-bit load per operand
// feeds 16 FMAs.  A tile that is produced by threads in the (row, column) arrangement and consumed as a
// transposed operand (P, dS) is stored with its 4-row groups XOR-swizzled by the key group, which makes both
// the stores and the broadcast loads free of bank conflicts.
constexpr int kTile = 64;
typedef float Tile[kTile][kTile];

// dst[c][r] = src[r][c] for a 64 x 64 tile of a row-major matrix (row stride ld); rows >= valid read zero.
__device__ __forceinline__ void load_tile_transposed(Tile &dst, const float *src, size_t ld, int valid) {
    for (int i = threadIdx.x; i < kTile * (kTile / 4); i += kAttnThreads) {
        const int r = i & 63, c = (i >> 6) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < valid) v = *reinterpret_cast<const float4 *>(src + (size_t)r * ld + c);
        dst[c + 0][r] = v.x;
        dst[c + 1][r] = v.y;
        dst[c + 2][r] = v.z;
        dst[c + 3][r] = v.w;
    }
}
__device__ __forceinline__ void load_tile_rowmajor(Tile &dst, const float *src, size_t ld, int valid) {
    for (int i = threadIdx.x; i < kTile * (kTile / 4); i += kAttnThreads) {
        const int r = i >> 4, c = (i & 15) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < valid) v = *reinterpret_cast<const float4 *>(src + (size_t)r * ld + c);
        *reinterpret_cast<float4 *>(&dst[r][c]) = v;
    }
}
// acc[i][j] += sum_d At[d][4ty+i] * Bt[d][4tx+j]
__device__ __forceinline__ void tile_mma(float (&acc)[4][4], const Tile &At, const Tile &Bt, int ty, int tx) {
#pragma unroll 8
    for (int d = 0; d < kTile; ++d) {
        const float4 a = *reinterpret_cast<const float4 *>(&At[d][4 * ty]);
        const float4 b = *reinterpret_cast<const float4 *>(&Bt[d][4 * tx]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
}
// Stores this thread's 4 x 4 block of a (row, key) tile transposed and swizzled: element (row 4ty+i, key 4tx+j)
// goes to dst[4tx+j][4*(ty ^ tx) + i].
__device__ __forceinline__ void store_block_swizzled(Tile &dst, const float (&blk)[4][4], int ty, int tx) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4 *>(&dst[4 * tx + j][4 * (ty ^ tx)]) = make_float4(blk[0][j], blk[1][j], blk[2][j], blk[3][j]);
}
// acc[i][j] += sum_k Pt[k][rows 4ty+i, swizzled] * B[k][4tx+j]   (Pt as written by store_block_swizzled)
__device__ __forceinline__ void tile_mma_swizzled(float (&acc)[4][4], const Tile &Pt, const Tile &B, int ty, int tx) {
#pragma unroll 8
    for (int k = 0; k < kTile; ++k) {
        const float4 a = *reinterpret_cast<const float4 *>(&Pt[k][4 * (ty ^ (k >> 2))]);
        const float4 b = *reinterpret_cast<const float4 *>(&B[k][4 * tx]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
}
// reductions over the 16 threads (one half-warp) that share the rows 4ty..4ty+3
__device__ __forceinline__ float row_max16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float row_sum16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Forward: for each key tile S = Q K^T (scaled, causal mask), running row maximum m and sum l, P = exp(S - m),
// O = O * exp(m_old - m) + P V.  lse = m + log(l) is kept for the backward pass.
// Shared memory: Q^T, K^T (re-used for P^T), V - 48 KiB.
__global__ void __launch_bounds__(kAttnThreads)
attn_fwd_kernel(const float *__restrict__ qr, const float *__restrict__ kr, const float *__restrict__ v,
                float *__restrict__ o, float *__restrict__ lse, int seq_len, int heads, int kv_heads) {
    extern __shared__ __align__(16) float attn_smem[];
    Tile &sQt = *reinterpret_cast<Tile *>(attn_smem);
    Tile &sKt = *reinterpret_cast<Tile *>(attn_smem + kTile * kTile);  // K^T, then P^T
    Tile &sV = *reinterpret_cast<Tile *>(attn_smem + 2 * kTile * kTile);
    const int qb = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int kvh = head / (heads / kv_heads);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int q0 = qb * kTile;
    const size_t tok0 = (size_t)seq * seq_len;
    const size_t ldq = (size_t)heads * kHeadDim, ldk = (size_t)kv_heads * kHeadDim;
    const float scale = 1.0f / sqrtf((float)kHeadDim);
    load_tile_transposed(sQt, qr + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
    float m[4], l[4], oacc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) oacc[i][j] = 0.0f;
    }
    for (int kb = 0; kb <= qb; ++kb) {
        const int k0 = kb * kTile;
        __syncthreads();  // the previous tile's P^T and V have been consumed (and Q^T is in place)
        load_tile_transposed(sKt, kr + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
        load_tile_rowmajor(sV, v + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
        __syncthreads();
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
        tile_mma(s, sQt, sKt, ty, tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qpos = q0 + 4 * ty + i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kpos = k0 + 4 * tx + j;
                s[i][j] = (kpos <= qpos && kpos < seq_len) ? s[i][j] * scale : -INFINITY;  // causal
                mx = fmaxf(mx, s[i][j]);
            }
            const float mn = fmaxf(m[i], row_max16(mx));  // every row sees at least one key in every tile it visits
            const float corr = expf(m[i] - mn);
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s[i][j] = expf(s[i][j] - mn);
                sum += s[i][j];
            }
            l[i] = l[i] * corr + row_sum16(sum);
            m[i] = mn;
#pragma unroll
            for (int j = 0; j < 4; ++j) oacc[i][j] *= corr;
        }
        __syncthreads();  // everybody is done with K^T
        store_block_swizzled(sKt, s, ty, tx);
        __syncthreads();
        tile_mma_swizzled(oacc, sKt, sV, ty, tx);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qpos = q0 + 4 * ty + i;
        if (qpos >= seq_len) continue;
        const float inv = 1.0f / l[i];
        *reinterpret_cast<float4 *>(o + (tok0 + qpos) * ldq + head * kHeadDim + 4 * tx) =
            make_float4(oacc[i][0] * inv, oacc[i][1] * inv, oacc[i][2] * inv, oacc[i][3] * inv);
        if (tx == 0) lse[(tok0 + qpos) * heads + head] = m[i] + logf(l[i]);
    }
}

// Backward, query side: delta_i = do_i . o_i,  p_ij = exp(s_ij - lse_i),  ds_ij = p_ij (do_i . v_j - delta_i) scale,
// dq_i = sum_j ds_ij k_j  (llama.rs:674-704, in the rotated frame).
// Shared memory: Q^T, dO^T (once); per key tile K^T, V^T (re-used for dS^T), K - 80 KiB.
constexpr size_t kAttnDqSmem = 5 * sizeof(Tile);
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dq_kernel(const float *__restrict__ qr, const float *__restrict__ kr, const float *__restrict__ v,
                   const float *__restrict__ o, const float *__restrict__ d_o, const float *__restrict__ lse,
                   float *__restrict__ delta, float *__restrict__ dqr, int seq_len, int heads, int kv_heads) {
    extern __shared__ __align__(16) float attn_smem[];
    Tile &sQt = *reinterpret_cast<Tile *>(attn_smem);
    Tile &sGt = *reinterpret_cast<Tile *>(attn_smem + 1 * kTile * kTile);  // dO^T
    Tile &sKt = *reinterpret_cast<Tile *>(attn_smem + 2 * kTile * kTile);
    Tile &sVt = *reinterpret_cast<Tile *>(attn_smem + 3 * kTile * kTile);  // V^T, then dS^T
    Tile &sK = *reinterpret_cast<Tile *>(attn_smem + 4 * kTile * kTile);
    const int qb = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int kvh = head / (heads / kv_heads);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int q0 = qb * kTile;
    const size_t tok0 = (size_t)seq * seq_len;
    const size_t ldq = (size_t)heads * kHeadDim, ldk = (size_t)kv_heads * kHeadDim;
    const float scale = 1.0f / sqrtf((float)kHeadDim);
    load_tile_transposed(sQt, qr + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
    load_tile_transposed(sGt, d_o + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
    float dl[4], L[4], acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qpos = q0 + 4 * ty + i;
        float part = 0.0f;
        L[i] = 0.0f;
        if (qpos < seq_len) {
            const size_t idx = (tok0 + qpos) * ldq + head * kHeadDim + 4 * tx;
            const float4 a = *reinterpret_cast<const float4 *>(d_o + idx), b = *reinterpret_cast<const float4 *>(o + idx);
            part = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
            L[i] = lse[(tok0 + qpos) * heads + head];
        }
        dl[i] = row_sum16(part);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    }
    for (int kb = 0; kb <= qb; ++kb) {
        const int k0 = kb * kTile;
        __syncthreads();
        load_tile_transposed(sKt, kr + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
        load_tile_transposed(sVt, v + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
        load_tile_rowmajor(sK, kr + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
        __syncthreads();
        float s[4][4], dp[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.0f;
        tile_mma(s, sQt, sKt, ty, tx);
        tile_mma(dp, sGt, sVt, ty, tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qpos = q0 + 4 * ty + i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kpos = k0 + 4 * tx + j;
                const bool on = kpos <= qpos && qpos < seq_len;
                s[i][j] = on ? expf(s[i][j] * scale - L[i]) * (dp[i][j] - dl[i]) * scale : 0.0f;  // dS
            }
        }
        __syncthreads();  // everybody is done with V^T
        store_block_swizzled(sVt, s, ty, tx);
        __syncthreads();
        tile_mma_swizzled(acc, sVt, sK, ty, tx);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qpos = q0 + 4 * ty + i;
        if (qpos >= seq_len) continue;
        *reinterpret_cast<float4 *>(dqr + (tok0 + qpos) * ldq + head * kHeadDim + 4 * tx) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        if (tx == 0) delta[(tok0 + qpos) * heads + head] = dl[i];
    }
}

// Backward, key side: a CTA owns 64 key positions of one (sequence, query head) and walks over the query
// tiles at or after them; the heads of a group leave partial sums (part = head % n_rep) that a second kernel adds:
// dv_j = sum_i p_ij do_i,  dk_j = sum_i ds_ij q_i  (llama.rs:686-712, in the rotated frame).
// P and dS are produced in the (query, key) arrangement and stored row-major, which is already the transposed
// operand form of the two products whose contraction runs over the queries.
// Shared memory: K^T, V^T (once); per query tile Q^T (re-used for P), dO^T (re-used for dS), Q, dO - 96 KiB.
constexpr size_t kAttnDkvSmem = 6 * sizeof(Tile);
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dkdv_kernel(const float *__restrict__ qr, const float *__restrict__ kr, const float *__restrict__ v,
                     const float *__restrict__ d_o, const float *__restrict__ lse, const float *__restrict__ delta,
                     float *__restrict__ dkr, float *__restrict__ dv, size_t part_stride, int seq_len, int heads,
                     int kv_heads) {
    extern __shared__ __align__(16) float attn_smem[];
    Tile &sKt = *reinterpret_cast<Tile *>(attn_smem);
    Tile &sVt = *reinterpret_cast<Tile *>(attn_smem + 1 * kTile * kTile);
    Tile &sQt = *reinterpret_cast<Tile *>(attn_smem + 2 * kTile * kTile);  // Q^T, then P  [query][key]
    Tile &sGt = *reinterpret_cast<Tile *>(attn_smem + 3 * kTile * kTile);  // dO^T, then dS [query][key]
    Tile &sQ = *reinterpret_cast<Tile *>(attn_smem + 4 * kTile * kTile);
    Tile &sG = *reinterpret_cast<Tile *>(attn_smem + 5 * kTile * kTile);
    __shared__ float s_lse[kTile], s_delta[kTile];
    // heavy key tiles (few keys before them, many queries after) first
    const int kb = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int n_rep = heads / kv_heads;
    const int kvh = head / n_rep, rep = head % n_rep;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int k0 = kb * kTile;
    const size_t tok0 = (size_t)seq * seq_len;
    const size_t ldq = (size_t)heads * kHeadDim, ldk = (size_t)kv_heads * kHeadDim;
    const float scale = 1.0f / sqrtf((float)kHeadDim);
    load_tile_transposed(sKt, kr + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
    load_tile_transposed(sVt, v + (tok0 + k0) * ldk + kvh * kHeadDim, ldk, seq_len - k0);
    float dk_acc[4][4], dv_acc[4][4];  // rows = keys 4ty.., columns = dimensions 4tx..
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dk_acc[i][j] = dv_acc[i][j] = 0.0f;
    const int n_qb = (seq_len + kTile - 1) / kTile;
    {
        for (int qb = kb; qb < n_qb; ++qb) {
            const int q0 = qb * kTile;
            __syncthreads();  // the previous tile's P, dS, Q, dO have been consumed (and K^T, V^T are in place)
            load_tile_transposed(sQt, qr + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
            load_tile_transposed(sGt, d_o + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
            load_tile_rowmajor(sQ, qr + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
            load_tile_rowmajor(sG, d_o + (tok0 + q0) * ldq + head * kHeadDim, ldq, seq_len - q0);
            if (threadIdx.x < kTile) {
                const bool ok = q0 + (int)threadIdx.x < seq_len;
                s_lse[threadIdx.x] = ok ? lse[(tok0 + q0 + threadIdx.x) * heads + head] : 0.0f;
                s_delta[threadIdx.x] = ok ? delta[(tok0 + q0 + threadIdx.x) * heads + head] : 0.0f;
            }
            __syncthreads();
            float s[4][4], dp[4][4];  // rows = queries 4ty.., columns = keys 4tx..
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.0f;
            tile_mma(s, sQt, sKt, ty, tx);
            tile_mma(dp, sGt, sVt, ty, tx);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int qi = 4 * ty + i, qpos = q0 + qi;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int kpos = k0 + 4 * tx + j;
                    const bool on = kpos <= qpos && qpos < seq_len;
                    const float p = on ? expf(s[i][j] * scale - s_lse[qi]) : 0.0f;
                    s[i][j] = p;
                    dp[i][j] = on ? p * (dp[i][j] - s_delta[qi]) * scale : 0.0f;  // dS
                }
            }
            __syncthreads();  // everybody is done with Q^T and dO^T
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                *reinterpret_cast<float4 *>(&sQt[4 * ty + i][4 * tx]) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
                *reinterpret_cast<float4 *>(&sGt[4 * ty + i][4 * tx]) = make_float4(dp[i][0], dp[i][1], dp[i][2], dp[i][3]);
            }
            __syncthreads();
            tile_mma(dv_acc, sQt, sG, ty, tx);  // dV[key][d] += sum_q P[q][key] dO[q][d]
            tile_mma(dk_acc, sGt, sQ, ty, tx);  // dK[key][d] += sum_q dS[q][key] Q[q][d]
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int kpos = k0 + 4 * ty + i;
        if (kpos >= seq_len) continue;
        const size_t idx = (size_t)rep * part_stride + (tok0 + kpos) * ldk + kvh * kHeadDim + 4 * tx;
        *reinterpret_cast<float4 *>(dkr + idx) = make_float4(dk_acc[i][0], dk_acc[i][1], dk_acc[i][2], dk_acc[i][3]);
        *reinterpret_cast<float4 *>(dv + idx) = make_float4(dv_acc[i][0], dv_acc[i][1], dv_acc[i][2], dv_acc[i][3]);
    }
}

// out = sum over `parts` partial arrays (stride part_stride), in part order
__global__ void sum_parts_kernel(const float *__restrict__ parts_base, size_t part_stride, int parts, float *__restrict__ out,
                                 size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = parts_base[i];
    for (int p = 1; p < parts; ++p) acc += parts_base[(size_t)p * part_stride + i];
    out[i] = acc;
}

// ---- softmax cross-entropy over the vocabulary (llama.rs:487-514), one CTA per token -----------------------
// row_loss[t] = -(logit[target] - max - log(sum exp));  dlogits = (softmax - onehot) * inv_count, written as
// fp32 (for the exact head) and / or bf16 (operand of the tensor-core head GEMM).
__global__ void __launch_bounds__(256)
softmax_ce_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ targets, size_t vocab, float inv_count,
                  float *__restrict__ row_loss, float *__restrict__ dl_f32, __nv_bfloat16 *__restrict__ dl_bf16) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    __shared__ float s_max, s_sum;
    const size_t t = blockIdx.x;
    const float *row = logits + t * vocab;
    float m = -INFINITY;
    for (size_t j = threadIdx.x; j < vocab; j += blockDim.x) m = fmaxf(m, row[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = red[0];
        for (int i = 1; i < 8; ++i) mm = fmaxf(mm, red[i]);
        s_max = mm;
    }
    __syncthreads();
    const float mx = s_max;
    float sum = 0.0f;
    for (size_t j = threadIdx.x; j < vocab; j += blockDim.x) sum += expf(row[j] - mx);
    sum = warp_sum(sum);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float ss = 0.0f;
        for (int i = 0; i < 8; ++i) ss += red[i];
        s_sum = ss;
        const uint32_t tg = targets[t] < vocab ? targets[t] : 0u;
        row_loss[t] = -(row[tg] - mx - logf(ss));
    }
    __syncthreads();
    const float inv_sum = 1.0f / s_sum;
    const uint32_t tg = targets[t];
    for (size_t j = threadIdx.x; j < vocab; j += blockDim.x) {
        float d = expf(row[j] - mx) * inv_sum * inv_count;
        if (j == tg) d -= inv_count;
        if (dl_f32) dl_f32[t * vocab + j] = d;
        if (dl_bf16) dl_bf16[t * vocab + j] = __float2bfloat16_rn(d);
    }
}

// The same for vocab % 4 == 0, two passes over the row instead of three: pass 1 keeps a running (max, sum) pair
// per thread (the sum is rescaled whenever the maximum moves), pass 2 writes the gradient.  128-bit loads.
constexpr int kCeThreads = 512;
__device__ __forceinline__ float4 load4(const float *p, size_t quad) { return reinterpret_cast<const float4 *>(p)[quad]; }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p, size_t quad) {
    const uint2 u = reinterpret_cast<const uint2 *>(p)[quad];
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// TL = float, or __nv_bfloat16 for logits the training step keeps in bf16.
template <typename TL>
__global__ void __launch_bounds__(kCeThreads)
softmax_ce_vec_kernel(const TL *__restrict__ logits, const uint32_t *__restrict__ targets, size_t vocab, float inv_count,
                      float *__restrict__ row_loss, float *__restrict__ dl_f32, __nv_bfloat16 *__restrict__ dl_bf16) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
    __shared__ float s_max, s_sum;
    const size_t t = blockIdx.x;
    const TL *row = logits + t * vocab;
    const size_t n4 = vocab / 4;
    float m = -INFINITY, sum = 0.0f;
    for (size_t j = threadIdx.x; j < n4; j += kCeThreads) {
        const float4 x = load4(row, j);
        const float mx = fmaxf(fmaxf(m, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
        sum = sum * expf(m - mx) + expf(x.x - mx) + expf(x.y - mx) + expf(x.z - mx) + expf(x.w - mx);
        m = mx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mx = fmaxf(m, om);
        // a thread that saw no element has (-inf, 0): exp(-inf - mx) = 0 unless mx is -inf too, where 0 * nan must not
        // leak - vocab >= 4 * kCeThreads is not required, so guard it
        sum = (m == -INFINITY ? 0.0f : sum * expf(m - mx)) + (om == -INFINITY ? 0.0f : os * expf(om - mx));
        m = mx;
    }
    if ((threadIdx.x & 31) == 0) {
        red_m[threadIdx.x >> 5] = m;
        red_s[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = red_m[0];
        for (int i = 1; i < kCeThreads / 32; ++i) mm = fmaxf(mm, red_m[i]);
        float ss = 0.0f;
        for (int i = 0; i < kCeThreads / 32; ++i) ss += red_m[i] == -INFINITY ? 0.0f : red_s[i] * expf(red_m[i] - mm);
        s_max = mm;
        s_sum = ss;
        const uint32_t tg = targets[t] < vocab ? targets[t] : 0u;
        row_loss[t] = -(as_f32(row[tg]) - mm - logf(ss));
    }
    __syncthreads();
    const float mx = s_max, k = inv_count / s_sum;
    const uint32_t tg = targets[t];
    for (size_t j = threadIdx.x; j < n4; j += kCeThreads) {
        const float4 x = load4(row, j);
        float d[4] = {expf(x.x - mx) * k, expf(x.y - mx) * k, expf(x.z - mx) * k, expf(x.w - mx) * k};
        if (tg / 4 == j) d[tg % 4] -= inv_count;
        if (dl_f32) reinterpret_cast<float4 *>(dl_f32 + t * vocab)[j] = make_float4(d[0], d[1], d[2], d[3]);
        if (dl_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(d[0], d[1]), hi = __floats2bfloat162_rn(d[2], d[3]);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t *>(&lo);
            u.y = *reinterpret_cast<uint32_t *>(&hi);
            reinterpret_cast<uint2 *>(dl_bf16 + t * vocab)[j] = u;
        }
    }
}

inline unsigned blocks_for(size_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }

}  // namespace
}  // namespace qlc

// ---- the model ------------------------------------------------------------------------------------------------
struct LlamaCache {  // per block, what the backward pass needs (llama.rs:471-483; q, k are kept rotated)
    float *x_in = nullptr, *xn_attn = nullptr, *qr = nullptr, *kr = nullptr, *v = nullptr, *attn_out = nullptr,
          *lse = nullptr, *x_mid = nullptr, *xn_mlp = nullptr, *gate = nullptr, *up = nullptr, *act = nullptr;
    __nv_bfloat16 *qr_b = nullptr, *kr_b = nullptr, *v_b = nullptr;  // bf16 copies for the tensor-core attention
    // the bf16 pipeline keeps these instead of their fp32 namesakes
    __nv_bfloat16 *xn_attn_b = nullptr, *attn_out_b = nullptr, *xn_mlp_b = nullptr, *gate_b = nullptr, *up_b = nullptr,
                  *act_b = nullptr;
};
struct LlamaLayer {
    float *attn_norm = nullptr, *mlp_norm = nullptr;
    qlc_layer *proj[QLC_LLAMA_PROJ_COUNT] = {nullptr};
    // gate and up as ONE layer with 2 * intermediate output features (its NF4 payload is the two payloads one after
    // the other), built when that concatenation equals quantising the two matrices separately; the bf16 pipeline
    // then runs one forward GEMM and one input-gradient GEMM (contraction over both) instead of two each
    qlc_layer *gate_up = nullptr;
    // q, k and v as ONE layer (h + 2 kv output features; fp32 block scales, decoded from the three payloads, so no
    // alignment of the double-quantisation groups is needed) whose adapter stacks the projections' adapters: one
    // forward GEMM, one input-gradient GEMM, one pair of LoRA side launches instead of three / two each
    qlc_layer *qkv = nullptr;
    LlamaCache c;
};
struct qlc_llama {
    qlc_ctx *ctx = nullptr;
    // bf16 pipeline: projections that read the same input (q / k / v, gate / up) and input-gradient GEMMs that feed
    // the same sum run side by side, one per lane; a lane is a context of its own (stream, scratch, status word)
    // on the same device, forked from and joined to the model's stream by events
    qlc_ctx *lane[2] = {nullptr, nullptr};
    cudaEvent_t ev_main = nullptr, ev_lane[2] = {nullptr, nullptr};
    qlc_llama_config cfg{};
    size_t kv_dim = 0;
    float *d_embed = nullptr, *d_final_norm = nullptr;
    __nv_bfloat16 *d_embed_bf16 = nullptr;
    std::vector<LlamaLayer> layers;
    // activation storage, sized for `cap_tokens` tokens of `cap_seq`-long sequences
    size_t cap_tokens = 0, cap_seq = 0;
    std::vector<void *> owned;  // every device allocation of the activation storage
    uint32_t *d_ids = nullptr, *d_targets = nullptr;
    float *x_final = nullptr, *hn = nullptr, *logits = nullptr, *dlogits = nullptr, *row_loss = nullptr;
    __nv_bfloat16 *hn_bf16 = nullptr, *dlogits_bf16 = nullptr, *d_attn_b = nullptr;
    // bf16 pipeline: activations between kernels are bf16 wherever the consumer is a tensor-core operand
    bool pipeline = false, cap_tc = false;
    // the training step keeps the logits in bf16 (written by the head GEMM, read twice by the loss kernel); they
    // share the storage of the fp32 logits that qlc_llama_forward returns
    bool want_bf16_logits = false, logits_are_bf16 = false;
    __nv_bfloat16 *dx_b = nullptr, *dx2_b = nullptr, *d_act_b = nullptr, *dg_b = nullptr, *du_b = nullptr, *dq_b = nullptr,
                  *dk_b = nullptr, *dv_b = nullptr, *q_tmp_b = nullptr, *k_tmp_b = nullptr, *tmp_b = nullptr, *dxn_b = nullptr,
                  *qkv_b = nullptr, *dqkv_b = nullptr,  // (T, h + 2 kv): output / upstream gradient of the merged q | k | v layer
                  *dxn2_b = nullptr, *dxn3_b = nullptr;
    float *cos_t = nullptr, *sin_t = nullptr;
    // backward scratch
    float *dx = nullptr, *dx2 = nullptr, *dxn = nullptr, *dxn2 = nullptr, *dxn3 = nullptr, *d_act = nullptr, *dg = nullptr,
          *du = nullptr, *d_attn = nullptr, *dqr = nullptr, *dkr = nullptr, *dq = nullptr, *dk = nullptr, *dv = nullptr,
          *delta = nullptr, *tmp_h = nullptr, *q_tmp = nullptr, *k_tmp = nullptr, *dk_parts = nullptr, *dv_parts = nullptr;
    bool have_cache = false;
};

namespace qlc {
namespace {

size_t proj_out(const qlc_llama *m, int kind) {
    const qlc_llama_config &c = m->cfg;
    switch (kind) {
        case QLC_LLAMA_K: case QLC_LLAMA_V: return m->kv_dim;
        case QLC_LLAMA_GATE: case QLC_LLAMA_UP: return c.intermediate;
        default: return c.hidden;  // q, o, down
    }
}
size_t proj_in(const qlc_llama *m, int kind) { return kind == QLC_LLAMA_DOWN ? m->cfg.intermediate : m->cfg.hidden; }

int dev_alloc(qlc_llama *m, void **p, size_t bytes) {
    QLC_CUDA(cudaMalloc(p, bytes ? bytes : 4));
    m->owned.push_back(*p);
    return QLC_OK;
}
template <class T> int dev_alloc_t(qlc_llama *m, T **p, size_t count) {
    return dev_alloc(m, reinterpret_cast<void **>(p), count * sizeof(T));
}

void free_activations(qlc_llama *m) {
    for (void *p : m->owned) cudaFree(p);
    m->owned.clear();
    m->cap_tokens = m->cap_seq = 0;
    m->have_cache = false;
}

// (Re)allocates the activation storage for n_seq sequences of seq_len tokens and builds the RoPE tables
// exactly as the reference does (llama.rs:795-811: powf, cos, sin in f32 on the host).
// Attention runs on the tensor cores (bf16 operands, fp32 accumulation) whenever the projections do.
bool attn_uses_tc(const qlc_llama *m) {
    return m->ctx->precision == QLC_PRECISION_AUTO || m->ctx->precision == QLC_PRECISION_BF16;
}

// The bf16 pipeline applies when the linears and the attention run on the tensor cores anyway: bf16 mode and
// every projection eligible for the tensor-core path.
bool wants_pipeline(const qlc_llama *m) {
    if (!(m->ctx->precision == QLC_PRECISION_AUTO || m->ctx->precision == QLC_PRECISION_BF16)) return false;
    static const bool off = getenv("QLC_LLAMA_FP32_ACTIVATIONS") != nullptr;  // diagnostics
    if (off || m->cfg.hidden % 64 || m->cfg.intermediate % 64) return false;
    for (const LlamaLayer &L : m->layers)
        for (const qlc_layer *p : L.proj)
            if (!p || !umma_fused_supported(p)) return false;
    return true;
}

int ensure_capacity(qlc_llama *m, size_t n_seq, size_t seq_len) {
    const size_t T = n_seq * seq_len;
    const bool pipe = wants_pipeline(m), tc = attn_uses_tc(m);
    // a change of the attention kernels means a different layout of the row statistics: start from fresh buffers
    if (T <= m->cap_tokens && seq_len == m->cap_seq && pipe == m->pipeline && tc == m->cap_tc) return QLC_OK;
    QLC_CUDA(cudaStreamSynchronize(m->ctx->stream));
    free_activations(m);
    m->pipeline = pipe;
    m->cap_tc = tc;
    const qlc_llama_config &c = m->cfg;
    const size_t h = c.hidden, kv = m->kv_dim, I = c.intermediate, V = c.vocab;
    // row statistics of the attention: the tensor-core kernels pad the position stride (and the fp32 kernels fit)
    const size_t n_stats = n_seq * c.heads * attention_tc_stat_stride(seq_len);
    for (LlamaLayer &L : m->layers) {
        LlamaCache &k = L.c;
        if (pipe) {
            QLC_TRY(dev_alloc_t(m, &k.x_in, T * h));
            QLC_TRY(dev_alloc_t(m, &k.x_mid, T * h));
            QLC_TRY(dev_alloc_t(m, &k.lse, n_stats));
            QLC_TRY(attention_tc_init_stats(m->ctx, k.lse, nullptr, n_seq, seq_len, c.heads));
            __nv_bfloat16 **hb[] = {&k.xn_attn_b, &k.qr_b, &k.attn_out_b, &k.xn_mlp_b};
            for (__nv_bfloat16 **p : hb) QLC_TRY(dev_alloc_t(m, p, T * h));
            QLC_TRY(dev_alloc_t(m, &k.kr_b, T * kv));
            QLC_TRY(dev_alloc_t(m, &k.v_b, T * kv));
            // gate and up share one allocation: two (T, I) matrices, or one (T, 2I) matrix when the block runs
            // the merged gate_up layer
            QLC_TRY(dev_alloc_t(m, &k.gate_b, 2 * T * I));
            k.up_b = k.gate_b + T * I;
            QLC_TRY(dev_alloc_t(m, &k.act_b, T * I));
            continue;
        }
        QLC_TRY(dev_alloc_t(m, &k.x_in, T * h));
        QLC_TRY(dev_alloc_t(m, &k.xn_attn, T * h));
        QLC_TRY(dev_alloc_t(m, &k.qr, T * h));
        QLC_TRY(dev_alloc_t(m, &k.kr, T * kv));
        QLC_TRY(dev_alloc_t(m, &k.v, T * kv));
        QLC_TRY(dev_alloc_t(m, &k.attn_out, T * h));
        QLC_TRY(dev_alloc_t(m, &k.qr_b, T * h));
        QLC_TRY(dev_alloc_t(m, &k.kr_b, T * kv));
        QLC_TRY(dev_alloc_t(m, &k.v_b, T * kv));
        QLC_TRY(dev_alloc_t(m, &k.lse, n_stats));
        QLC_TRY(attention_tc_init_stats(m->ctx, k.lse, nullptr, n_seq, seq_len, c.heads));
        QLC_TRY(dev_alloc_t(m, &k.x_mid, T * h));
        QLC_TRY(dev_alloc_t(m, &k.xn_mlp, T * h));
        QLC_TRY(dev_alloc_t(m, &k.gate, T * I));
        QLC_TRY(dev_alloc_t(m, &k.up, T * I));
        QLC_TRY(dev_alloc_t(m, &k.act, T * I));
    }
    QLC_TRY(dev_alloc_t(m, &m->d_ids, T));
    QLC_TRY(dev_alloc_t(m, &m->d_targets, T));
    QLC_TRY(dev_alloc_t(m, &m->x_final, T * h));
    QLC_TRY(dev_alloc_t(m, &m->hn, T * h));
    QLC_TRY(dev_alloc_t(m, &m->hn_bf16, T * h));
    QLC_TRY(dev_alloc_t(m, &m->logits, T * V));
    QLC_TRY(dev_alloc_t(m, &m->dlogits, T * V));
    QLC_TRY(dev_alloc_t(m, &m->dlogits_bf16, T * V));
    QLC_TRY(dev_alloc_t(m, &m->row_loss, T));
    QLC_TRY(dev_alloc_t(m, &m->d_attn_b, T * h));
    if (pipe) {
        float **hs[] = {&m->dx, &m->dx2, &m->dxn, &m->dqr};
        for (float **p : hs) QLC_TRY(dev_alloc_t(m, p, T * h));
        QLC_TRY(dev_alloc_t(m, &m->dkr, T * kv));
        QLC_TRY(dev_alloc_t(m, &m->k_tmp_b, T * kv));
        QLC_TRY(dev_alloc_t(m, &m->qkv_b, T * (h + 2 * kv)));
        QLC_TRY(dev_alloc_t(m, &m->dqkv_b, T * (h + 2 * kv)));
        __nv_bfloat16 **hb[] = {&m->dx_b, &m->dx2_b, &m->dq_b, &m->q_tmp_b, &m->tmp_b, &m->dxn_b, &m->dxn2_b, &m->dxn3_b};
        for (__nv_bfloat16 **p : hb) QLC_TRY(dev_alloc_t(m, p, T * h));
        QLC_TRY(dev_alloc_t(m, &m->dk_b, T * kv));
        QLC_TRY(dev_alloc_t(m, &m->dv_b, T * kv));
        QLC_TRY(dev_alloc_t(m, &m->dk_parts, (c.heads / c.kv_heads) * T * kv));
        QLC_TRY(dev_alloc_t(m, &m->dv_parts, (c.heads / c.kv_heads) * T * kv));
        QLC_TRY(dev_alloc_t(m, &m->d_act_b, T * I));
        QLC_TRY(dev_alloc_t(m, &m->dg_b, 2 * T * I));  // dg and du: two (T, I) matrices or one (T, 2I) matrix
        m->du_b = m->dg_b + T * I;
    } else {
        float **hs[] = {&m->dx, &m->dx2, &m->dxn, &m->dxn2, &m->dxn3, &m->d_attn, &m->dqr, &m->dq, &m->tmp_h, &m->q_tmp};
        for (float **p : hs) QLC_TRY(dev_alloc_t(m, p, T * h));
        float **ks[] = {&m->dkr, &m->dk, &m->dv, &m->k_tmp};
        for (float **p : ks) QLC_TRY(dev_alloc_t(m, p, T * kv));
        QLC_TRY(dev_alloc_t(m, &m->dk_parts, (c.heads / c.kv_heads) * T * kv));
        QLC_TRY(dev_alloc_t(m, &m->dv_parts, (c.heads / c.kv_heads) * T * kv));
        float **is[] = {&m->d_act, &m->dg, &m->du};
        for (float **p : is) QLC_TRY(dev_alloc_t(m, p, T * I));
    }
    QLC_TRY(dev_alloc_t(m, &m->delta, n_stats));
    QLC_CUDA(cudaMemsetAsync(m->delta, 0, n_stats * 4, m->ctx->stream));
    const size_t half = kHeadDim / 2;
    std::vector<float> cs(seq_len * half), sn(seq_len * half);
    for (size_t pos = 0; pos < seq_len; ++pos)
        for (size_t i = 0; i < half; ++i) {
            const float freq = powf(c.rope_theta, -((float)(2 * i)) / (float)kHeadDim);
            const float ang = (float)pos * freq;
            cs[pos * half + i] = cosf(ang);
            sn[pos * half + i] = sinf(ang);
        }
    QLC_TRY(dev_alloc_t(m, &m->cos_t, seq_len * half));
    QLC_TRY(dev_alloc_t(m, &m->sin_t, seq_len * half));
    QLC_CUDA(cudaMemcpy(m->cos_t, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    QLC_CUDA(cudaMemcpy(m->sin_t, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    m->cap_tokens = T;
    m->cap_seq = seq_len;
    return QLC_OK;
}

#define LK(kernel, grid, block, ...)                                            \
    do {                                                                        \
        QLC_CUDA(launch_pdl(kernel, dim3(grid), dim3(block), 0, st, __VA_ARGS__)); \
        m->ctx->launches += 1;                                                  \
        QLC_CUDA(cudaGetLastError());                                           \
    } while (0)

int lin_fwd(qlc_llama *m, qlc_layer *L, const float *x, size_t T, float *y) {
    return qlc_qlora_forward_dev(m->ctx, L, x, QLC_DTYPE_F32, T, y);
}
// gradients of an adapter go to its own bucket; layers without an adapter get none
int lin_bwd(qlc_llama *m, qlc_layer *L, const float *x, const float *dy, size_t T, float *dx) {
    float *ga = nullptr, *gb = nullptr;
    if (L->r) {
        ga = L->d_grad_bucket;
        gb = L->d_grad_bucket + L->r * L->in_dim;
    }
    return qlc_qlora_backward_dev(m->ctx, L, x, dy, QLC_DTYPE_F32, T, dx, ga, gb);
}

// The tied LM head: logits = hn · E^T, and dH = dlogits · E (llama.rs:324-325, 406).
int head_forward(qlc_llama *m, size_t T, bool hn_bf16_ready = false) {
    const qlc_llama_config &c = m->cfg;
    m->logits_are_bf16 = false;
    if (m->ctx->precision == QLC_PRECISION_FP32_EXACT || c.hidden % 64 || c.vocab % 32)
        return exact_matmul_trans_b(m->ctx, m->hn, m->d_embed, T, c.hidden, c.vocab, m->logits);
    if (!hn_bf16_ready) QLC_TRY(launch_convert_f32_to_bf16(m->ctx, m->hn, m->hn_bf16, T * c.hidden));
    m->logits_are_bf16 = m->want_bf16_logits;
    return umma_gemm_bf16(m->ctx, m->hn_bf16, m->d_embed_bf16, false, m->logits, T, c.vocab, c.hidden, m->logits_are_bf16);
}
int head_backward(qlc_llama *m, size_t T, bool dlogits_is_bf16_ready, float *d_hn) {
    const qlc_llama_config &c = m->cfg;
    if (m->ctx->precision == QLC_PRECISION_FP32_EXACT || c.hidden % 64 || c.vocab % 64)
        return exact_matmul(m->ctx, m->dlogits, m->d_embed, T, c.vocab, c.hidden, d_hn);
    if (!dlogits_is_bf16_ready) QLC_TRY(launch_convert_f32_to_bf16(m->ctx, m->dlogits, m->dlogits_bf16, T * c.vocab));
    return umma_gemm_bf16(m->ctx, m->dlogits_bf16, m->d_embed_bf16, true, d_hn, T, c.hidden, c.vocab);
}
bool head_uses_bf16(const qlc_llama *m) {
    return !(m->ctx->precision == QLC_PRECISION_FP32_EXACT || m->cfg.hidden % 64 || m->cfg.vocab % 64);
}

// ---- the bf16 pipeline ----------------------------------------------------------------------------------------
// Same mathematics as run_forward / run_backward below; every tensor whose consumer is a tensor-core operand is
// produced as bf16 by the kernel before it (normalised activations, attention output, MLP gate / up / product,
// the dY of every linear), so no conversion pass runs between kernels.  The residual stream, the RoPE inputs and
// all reductions stay fp32.
int ensure_lanes(qlc_llama *m) {
    static const bool off = getenv("QLC_LLAMA_NO_LANES") != nullptr;  // diagnostics: everything on one stream
    if (off || m->lane[0]) return QLC_OK;
    qlc_ctx *lanes[2] = {nullptr, nullptr};
    cudaEvent_t evs[3] = {nullptr, nullptr, nullptr};
    int st = QLC_OK;
    for (int i = 0; i < 2 && st == QLC_OK; ++i) st = qlc_ctx_create(m->ctx->device, &lanes[i]);
    for (int i = 0; i < 3 && st == QLC_OK; ++i)
        if (cudaEventCreateWithFlags(&evs[i], cudaEventDisableTiming) != cudaSuccess)
            st = fail(QLC_ERR_GPU, "could not create the events of the model's lanes");
    if (st != QLC_OK) {  // all or nothing: a half-built set of lanes must never be forked to
        for (qlc_ctx *l : lanes) qlc_ctx_destroy(l);
        for (cudaEvent_t e : evs)
            if (e) cudaEventDestroy(e);
        return st;
    }
    m->lane[0] = lanes[0];
    m->lane[1] = lanes[1];
    m->ev_main = evs[0];
    m->ev_lane[0] = evs[1];
    m->ev_lane[1] = evs[2];
    return QLC_OK;
}
// ctx of lane i (0 = the model's own context)
qlc_ctx *lane_ctx(qlc_llama *m, int i) { return (i == 0 || !m->lane[0]) ? m->ctx : m->lane[i - 1]; }
// Lanes 1..n start after everything queued on the model's stream so far.
int lanes_fork(qlc_llama *m, int n) {
    if (!m->lane[0]) return QLC_OK;
    QLC_CUDA(cudaEventRecord(m->ev_main, m->ctx->stream));
    for (int i = 0; i < n; ++i) {
        m->lane[i]->precision = m->ctx->precision;
        QLC_CUDA(cudaStreamWaitEvent(m->lane[i]->stream, m->ev_main, 0));
    }
    return QLC_OK;
}
// The model's stream continues after everything queued on lanes 1..n.
int lanes_join(qlc_llama *m, int n) {
    if (!m->lane[0]) return QLC_OK;
    for (int i = 0; i < n; ++i) {
        QLC_CUDA(cudaEventRecord(m->ev_lane[i], m->lane[i]->stream));
        QLC_CUDA(cudaStreamWaitEvent(m->ctx->stream, m->ev_lane[i], 0));
        m->ctx->launches += m->lane[i]->launches;  // one launch count for the model
        m->lane[i]->launches = 0;
    }
    return QLC_OK;
}
// The merged gate_up layer stands in for gate and up while neither of them has an adapter.
bool uses_gate_up(const LlamaLayer &L) {
    static const bool off = getenv("QLC_LLAMA_NO_GATE_UP") != nullptr;  // diagnostics
    return !off && L.gate_up && L.proj[QLC_LLAMA_GATE] && L.proj[QLC_LLAMA_UP] && L.proj[QLC_LLAMA_GATE]->r == 0 &&
           L.proj[QLC_LLAMA_UP]->r == 0;
}

bool uses_qkv(const LlamaLayer &L) {
    static const bool off = getenv("QLC_LLAMA_NO_QKV") != nullptr;  // diagnostics
    return !off && L.qkv != nullptr;
}

// Rebuilds the adapter operands of every merged q | k | v layer from the projections' current fp32 A / B
// (they change with every optimiser step, and a caller may change them through the projections' handles).
int refresh_qkv_operands(qlc_llama *m) {
    cudaStream_t st = m->ctx->stream;
    static thread_local QkvRefreshBatch batch;
    batch.n = 0;
    auto flush = [&]() -> int {
        if (!batch.n) return QLC_OK;
        LK(qkv_refresh_kernel, dim3(40, (unsigned)batch.n), 256, batch);
        batch.n = 0;
        return QLC_OK;
    };
    for (LlamaLayer &L : m->layers) {
        if (!uses_qkv(L) || !L.qkv->r) continue;
        QkvRefresh &d = batch.d[batch.n++];
        const int kinds[3] = {QLC_LLAMA_Q, QLC_LLAMA_K, QLC_LLAMA_V};
        for (int i = 0; i < 3; ++i) {
            const qlc_layer *P = L.proj[kinds[i]];
            d.a[i] = P->d_a;
            d.b[i] = P->d_b;
            d.r[i] = (uint32_t)P->r;
            d.out[i] = (uint32_t)P->out_dim;
        }
        d.a_pad = L.qkv->d_a_pad;
        d.b_pad = L.qkv->d_b_pad;
        d.bt_pad = L.qkv->d_bt_pad;
        d.r_pad = (uint32_t)L.qkv->r_pad;
        d.in_dim = (uint32_t)L.qkv->in_dim;
        d.out_m = (uint32_t)L.qkv->out_dim;
        if (batch.n == kQkvBatch) QLC_TRY(flush());
    }
    return flush();
}

// After the backward pass: the merged layers' adapter gradients go to the projections' own buckets, where the
// optimiser, the gradient exchange and the getters expect them.
int scatter_qkv_grads(qlc_llama *m) {
    cudaStream_t st = m->ctx->stream;
    static thread_local QkvScatterBatch batch;
    batch.n = 0;
    auto flush = [&]() -> int {
        if (!batch.n) return QLC_OK;
        LK(qkv_scatter_kernel, dim3(8, (unsigned)batch.n), 256, batch);
        batch.n = 0;
        return QLC_OK;
    };
    for (LlamaLayer &L : m->layers) {
        if (!uses_qkv(L) || !L.qkv->r) continue;
        QkvScatter &d = batch.d[batch.n++];
        d.ga_m = L.qkv->d_grad_bucket;
        d.gb_m = L.qkv->d_grad_bucket + L.qkv->r * L.qkv->in_dim;
        const int kinds[3] = {QLC_LLAMA_Q, QLC_LLAMA_K, QLC_LLAMA_V};
        for (int i = 0; i < 3; ++i) {
            qlc_layer *P = L.proj[kinds[i]];
            d.bucket[i] = P->d_grad_bucket;
            d.r[i] = (uint32_t)P->r;
            d.out[i] = (uint32_t)P->out_dim;
        }
        d.r_m = (uint32_t)L.qkv->r;
        d.in_dim = (uint32_t)L.qkv->in_dim;
        if (batch.n == kQkvBatch) QLC_TRY(flush());
    }
    return flush();
}

int pipe_fwd(qlc_llama *m, int lane, qlc_layer *L, const __nv_bfloat16 *x, size_t T, void *y, int y_dtype) {
    return umma_qlora_forward(lane_ctx(m, lane), L, x, T, y, y_dtype, false);
}
int pipe_bwd(qlc_llama *m, int lane, qlc_layer *L, const __nv_bfloat16 *x, const __nv_bfloat16 *dy, size_t T, void *dx,
             int dx_dtype) {
    float *ga = nullptr, *gb = nullptr;
    if (L->r) {
        ga = L->d_grad_bucket;
        gb = L->d_grad_bucket + L->r * L->in_dim;
    }
    return umma_qlora_backward(lane_ctx(m, lane), L, x, dy, T, dx, dx_dtype, ga, gb);
}

int run_forward_pipeline(qlc_llama *m, size_t n_seq, size_t seq_len) {
    const qlc_llama_config &c = m->cfg;
    cudaStream_t st = m->ctx->stream;
    const size_t T = n_seq * seq_len, h = c.hidden, I = c.intermediate;
    const int h2 = (int)(h / 2);
    const unsigned rows_grid = blocks_for(T, 8);
    float2 *const no_f32x2 = nullptr;
    __nv_bfloat162 *const no_bf16x2 = nullptr;
    const bool head_bf16 = head_uses_bf16(m);
    QLC_TRY(ensure_lanes(m));
    QLC_TRY(refresh_qkv_operands(m));
    auto f2 = [](float *p) { return reinterpret_cast<float2 *>(p); };
    auto cf2 = [](const float *p) { return reinterpret_cast<const float2 *>(p); };
    auto b2 = [](__nv_bfloat16 *p) { return reinterpret_cast<__nv_bfloat162 *>(p); };
    auto cb2 = [](const __nv_bfloat16 *p) { return reinterpret_cast<const __nv_bfloat162 *>(p); };
    LK(embed_gather_kernel, (unsigned)T, 128, m->d_ids, m->d_embed, m->layers.empty() ? m->x_final : m->layers[0].c.x_in, T,
       (int)h, (uint32_t)c.vocab);
    if (m->layers.empty())
        LK(pipe_norm_fwd_kernel, rows_grid, 256, cf2(m->x_final), (const __nv_bfloat162 *)nullptr, no_f32x2, cf2(m->d_final_norm),
           c.rms_eps, f2(m->hn), head_bf16 ? b2(m->hn_bf16) : no_bf16x2, T, h2);
    else
        LK(pipe_norm_fwd_kernel, rows_grid, 256, cf2(m->layers[0].c.x_in), (const __nv_bfloat162 *)nullptr, no_f32x2,
           cf2(m->layers[0].attn_norm), c.rms_eps, no_f32x2, b2(m->layers[0].c.xn_attn_b), T, h2);
    for (size_t li = 0; li < m->layers.size(); ++li) {
        LlamaLayer &L = m->layers[li];
        LlamaCache &k = L.c;
        const bool last = li + 1 == m->layers.size();
        if (uses_qkv(L)) {
            QLC_TRY(pipe_fwd(m, 0, L.qkv, k.xn_attn_b, T, m->qkv_b, QLC_DTYPE_BF16));  // (T, h + 2 kv): q | k | v
            LK(rope_qkv_kernel, blocks_for(T * ((c.heads + c.kv_heads) * 4 + c.kv_heads * 8), 256), 256,
               (const __nv_bfloat16 *)m->qkv_b, h + 2 * m->kv_dim, m->cos_t, m->sin_t, k.qr_b, k.kr_b, k.v_b, T, (int)c.heads,
               (int)c.kv_heads, (int)seq_len);
        } else {
            QLC_TRY(lanes_fork(m, 2));
            QLC_TRY(pipe_fwd(m, 0, L.proj[QLC_LLAMA_Q], k.xn_attn_b, T, m->q_tmp_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_fwd(m, 1, L.proj[QLC_LLAMA_K], k.xn_attn_b, T, m->k_tmp_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_fwd(m, 2, L.proj[QLC_LLAMA_V], k.xn_attn_b, T, k.v_b, QLC_DTYPE_BF16));
            QLC_TRY(lanes_join(m, 2));
            LK(rope_qk_kernel<__nv_bfloat16>, blocks_for(T * (c.heads + c.kv_heads) * 4, 256), 256,
               (const __nv_bfloat16 *)m->q_tmp_b, (const __nv_bfloat16 *)m->k_tmp_b, m->cos_t, m->sin_t, k.qr_b, k.kr_b, T,
               (int)c.heads, (int)c.kv_heads, (int)seq_len, 0);
        }
        QLC_TRY(attention_tc_forward(m->ctx, k.qr_b, k.kr_b, k.v_b, nullptr, k.attn_out_b, k.lse, n_seq, seq_len, c.heads,
                                     c.kv_heads));
        QLC_TRY(pipe_fwd(m, 0, L.proj[QLC_LLAMA_O], k.attn_out_b, T, m->tmp_b, QLC_DTYPE_BF16));
        // x_mid = x_in + attention branch, and its normalised copy for the MLP, in one pass
        LK(pipe_norm_fwd_kernel, rows_grid, 256, cf2(k.x_in), cb2(m->tmp_b), f2(k.x_mid), cf2(L.mlp_norm), c.rms_eps, no_f32x2,
           b2(k.xn_mlp_b), T, h2);
        if (uses_gate_up(L)) {
            QLC_TRY(pipe_fwd(m, 0, L.gate_up, k.xn_mlp_b, T, k.gate_b, QLC_DTYPE_BF16));  // (T, 2I): gate | up
            LK(swiglu_fwd_bf16_kernel, blocks_for(T * I / 8, 256), 256, reinterpret_cast<const uint4 *>(k.gate_b),
               reinterpret_cast<const uint4 *>(k.gate_b + I), reinterpret_cast<uint4 *>(k.act_b), T * I / 8, (uint32_t)(I / 8),
               (uint32_t)(2 * I / 8));
        } else {
            QLC_TRY(lanes_fork(m, 1));
            QLC_TRY(pipe_fwd(m, 0, L.proj[QLC_LLAMA_GATE], k.xn_mlp_b, T, k.gate_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_fwd(m, 1, L.proj[QLC_LLAMA_UP], k.xn_mlp_b, T, k.up_b, QLC_DTYPE_BF16));
            QLC_TRY(lanes_join(m, 1));
            LK(swiglu_fwd_bf16_kernel, blocks_for(T * I / 8, 256), 256, reinterpret_cast<const uint4 *>(k.gate_b),
               reinterpret_cast<const uint4 *>(k.up_b), reinterpret_cast<uint4 *>(k.act_b), T * I / 8, (uint32_t)(I / 8),
               (uint32_t)(I / 8));
        }
        QLC_TRY(pipe_fwd(m, 0, L.proj[QLC_LLAMA_DOWN], k.act_b, T, m->tmp_b, QLC_DTYPE_BF16));
        // x_out = x_mid + MLP branch, normalised for the next block's attention (or by the final norm)
        if (last)
            LK(pipe_norm_fwd_kernel, rows_grid, 256, cf2(k.x_mid), cb2(m->tmp_b), f2(m->x_final), cf2(m->d_final_norm), c.rms_eps,
               f2(m->hn), head_bf16 ? b2(m->hn_bf16) : no_bf16x2, T, h2);
        else
            LK(pipe_norm_fwd_kernel, rows_grid, 256, cf2(k.x_mid), cb2(m->tmp_b), f2(m->layers[li + 1].c.x_in),
               cf2(m->layers[li + 1].attn_norm), c.rms_eps, no_f32x2, b2(m->layers[li + 1].c.xn_attn_b), T, h2);
    }
    QLC_TRY(head_forward(m, T, head_bf16));
    m->have_cache = true;
    return QLC_OK;
}

int run_backward_pipeline(qlc_llama *m, size_t n_seq, size_t seq_len, bool dlogits_bf16_ready) {
    const qlc_llama_config &c = m->cfg;
    cudaStream_t st = m->ctx->stream;
    const size_t T = n_seq * seq_len, h = c.hidden, I = c.intermediate;
    const int h2 = (int)(h / 2);
    const unsigned rows_grid = blocks_for(T, 8);
    float *const no_f32 = nullptr;
    const float *const none = nullptr;
    auto f2 = [](float *p) { return reinterpret_cast<float2 *>(p); };
    auto cf2 = [](const float *p) { return reinterpret_cast<const float2 *>(p); };
    auto b2 = [](__nv_bfloat16 *p) { return reinterpret_cast<__nv_bfloat162 *>(p); };
    auto cb2 = [](const __nv_bfloat16 *p) { return reinterpret_cast<const __nv_bfloat162 *>(p); };
    QLC_TRY(head_backward(m, T, dlogits_bf16_ready, m->dxn));
    float *dx = m->dx, *dx_alt = m->dx2;
    __nv_bfloat16 *dx_b = m->dx_b, *dx_alt_b = m->dx2_b;
    LK(rmsnorm_bwd_kernel, rows_grid, 256, m->x_final, m->d_final_norm, m->dxn, c.rms_eps, none, dx, T, (int)h, dx_b, none, none,
       no_f32);
    for (size_t li = m->layers.size(); li-- > 0;) {
        LlamaLayer &L = m->layers[li];
        LlamaCache &k = L.c;
        // MLP branch (llama.rs:554-575)
        QLC_TRY(pipe_bwd(m, 0, L.proj[QLC_LLAMA_DOWN], k.act_b, dx_b, T, m->d_act_b, QLC_DTYPE_BF16));
        if (uses_gate_up(L)) {
            // dg | du as one (T, 2I) matrix: the merged layer's input-gradient GEMM contracts over both
            LK(swiglu_bwd_bf16_kernel, blocks_for(T * I / 8, 256), 256, reinterpret_cast<const uint4 *>(k.gate_b),
               reinterpret_cast<const uint4 *>(k.gate_b + I), reinterpret_cast<const uint4 *>(m->d_act_b),
               reinterpret_cast<uint4 *>(m->dg_b), reinterpret_cast<uint4 *>(m->dg_b + I), T * I / 8, (uint32_t)(I / 8),
               (uint32_t)(2 * I / 8));
            QLC_TRY(pipe_bwd(m, 0, L.gate_up, k.xn_mlp_b, m->dg_b, T, m->dxn_b, QLC_DTYPE_BF16));
            // dx_mid = rmsnorm_backward(x_mid, dxn) + dx   (residual)
            LK(pipe_norm_bwd_kernel, rows_grid, 256, cf2(k.x_mid), cf2(L.mlp_norm), cb2(m->dxn_b), (const __nv_bfloat162 *)nullptr,
               (const __nv_bfloat162 *)nullptr, c.rms_eps, cf2(dx), f2(dx_alt), b2(dx_alt_b), T, h2);
        } else {
            LK(swiglu_bwd_bf16_kernel, blocks_for(T * I / 8, 256), 256, reinterpret_cast<const uint4 *>(k.gate_b),
               reinterpret_cast<const uint4 *>(k.up_b), reinterpret_cast<const uint4 *>(m->d_act_b),
               reinterpret_cast<uint4 *>(m->dg_b), reinterpret_cast<uint4 *>(m->du_b), T * I / 8, (uint32_t)(I / 8),
               (uint32_t)(I / 8));
            QLC_TRY(lanes_fork(m, 1));
            QLC_TRY(pipe_bwd(m, 0, L.proj[QLC_LLAMA_GATE], k.xn_mlp_b, m->dg_b, T, m->dxn_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_bwd(m, 1, L.proj[QLC_LLAMA_UP], k.xn_mlp_b, m->du_b, T, m->dxn2_b, QLC_DTYPE_BF16));
            QLC_TRY(lanes_join(m, 1));
            // dx_mid = rmsnorm_backward(x_mid, dxn + dxn2) + dx   (residual)
            LK(pipe_norm_bwd_kernel, rows_grid, 256, cf2(k.x_mid), cf2(L.mlp_norm), cb2(m->dxn_b), cb2(m->dxn2_b),
               (const __nv_bfloat162 *)nullptr, c.rms_eps, cf2(dx), f2(dx_alt), b2(dx_alt_b), T, h2);
        }
        // attention branch (llama.rs:577-601); dO arrives as bf16 straight from the output projection's dX GEMM
        QLC_TRY(pipe_bwd(m, 0, L.proj[QLC_LLAMA_O], k.attn_out_b, dx_alt_b, T, m->d_attn_b, QLC_DTYPE_BF16));
        QLC_TRY(attention_tc_backward(m->ctx, k.qr_b, k.kr_b, k.v_b, nullptr, nullptr, k.attn_out_b, m->d_attn_b, k.lse, m->delta,
                                      m->dqr, nullptr, nullptr, nullptr, m->dk_parts, m->dv_parts, n_seq, seq_len, c.heads,
                                      c.kv_heads, m->lane[0], m->ev_main, m->ev_lane[0]));
        if (uses_qkv(L)) {
            // dq | dk | dv as one (T, h + 2 kv) matrix: the merged layer's input-gradient GEMM contracts over all three
            const size_t ldm = h + 2 * m->kv_dim;
            LK(attn_bwd_finish_kernel, blocks_for(T * ((c.heads + c.kv_heads) * 4 + c.kv_heads * 8), 256), 256,
               (const float *)m->dqr, (const float *)m->dk_parts, (const float *)m->dv_parts, T * m->kv_dim,
               (int)(c.heads / c.kv_heads), m->cos_t, m->sin_t, m->dqkv_b, m->dqkv_b + h, m->dqkv_b + h + m->kv_dim, T,
               (int)c.heads, (int)c.kv_heads, (int)seq_len, ldm, ldm);
            QLC_TRY(pipe_bwd(m, 0, L.qkv, k.xn_attn_b, m->dqkv_b, T, m->dxn_b, QLC_DTYPE_BF16));
            // dx_in = rmsnorm_backward(x_in, dxn) + dx_mid
            LK(pipe_norm_bwd_kernel, rows_grid, 256, cf2(k.x_in), cf2(L.attn_norm), cb2(m->dxn_b), (const __nv_bfloat162 *)nullptr,
               (const __nv_bfloat162 *)nullptr, c.rms_eps, cf2(dx_alt), f2(dx), b2(dx_b), T, h2);
        } else {
            LK(attn_bwd_finish_kernel, blocks_for(T * ((c.heads + c.kv_heads) * 4 + c.kv_heads * 8), 256), 256,
               (const float *)m->dqr, (const float *)m->dk_parts, (const float *)m->dv_parts, T * m->kv_dim,
               (int)(c.heads / c.kv_heads), m->cos_t, m->sin_t, m->dq_b, m->dk_b, m->dv_b, T, (int)c.heads, (int)c.kv_heads,
               (int)seq_len, h, m->kv_dim);
            QLC_TRY(lanes_fork(m, 2));
            QLC_TRY(pipe_bwd(m, 0, L.proj[QLC_LLAMA_Q], k.xn_attn_b, m->dq_b, T, m->dxn_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_bwd(m, 1, L.proj[QLC_LLAMA_K], k.xn_attn_b, m->dk_b, T, m->dxn2_b, QLC_DTYPE_BF16));
            QLC_TRY(pipe_bwd(m, 2, L.proj[QLC_LLAMA_V], k.xn_attn_b, m->dv_b, T, m->dxn3_b, QLC_DTYPE_BF16));
            QLC_TRY(lanes_join(m, 2));
            // dx_in = rmsnorm_backward(x_in, dxn + dxn2 + dxn3) + dx_mid
            LK(pipe_norm_bwd_kernel, rows_grid, 256, cf2(k.x_in), cf2(L.attn_norm), cb2(m->dxn_b), cb2(m->dxn2_b), cb2(m->dxn3_b),
               c.rms_eps, cf2(dx_alt), f2(dx), b2(dx_b), T, h2);
        }
    }
    return scatter_qkv_grads(m);
}

int run_forward(qlc_llama *m, size_t n_seq, size_t seq_len) {
    if (m->pipeline) return run_forward_pipeline(m, n_seq, seq_len);
    const qlc_llama_config &c = m->cfg;
    cudaStream_t st = m->ctx->stream;
    const size_t T = n_seq * seq_len, h = c.hidden, kv = m->kv_dim, I = c.intermediate;
    const unsigned rows_grid = blocks_for(T, 8);  // 8 warps (rows) per 256-thread CTA
    const dim3 agrid((unsigned)((seq_len + kAttnRows - 1) / kAttnRows), (unsigned)c.heads, (unsigned)n_seq);
    LK(embed_gather_kernel, (unsigned)T, 128, m->d_ids, m->d_embed, m->layers.empty() ? m->x_final : m->layers[0].c.x_in, T,
       (int)h, (uint32_t)c.vocab);
    for (size_t li = 0; li < m->layers.size(); ++li) {
        LlamaLayer &L = m->layers[li];
        LlamaCache &k = L.c;
        float *x_out = li + 1 < m->layers.size() ? m->layers[li + 1].c.x_in : m->x_final;
        LK(rmsnorm_fwd_kernel, rows_grid, 256, k.x_in, L.attn_norm, c.rms_eps, k.xn_attn, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (float *)nullptr);
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_Q], k.xn_attn, T, m->q_tmp));
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_K], k.xn_attn, T, m->k_tmp));
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_V], k.xn_attn, T, k.v));
        const bool tc = attn_uses_tc(m);
        LK(rope_kernel<float>, blocks_for(T * c.heads * 32, 256), 256, m->q_tmp, m->cos_t, m->sin_t, k.qr, T, (int)c.heads,
           (int)seq_len, 0, tc ? k.qr_b : (__nv_bfloat16 *)nullptr);
        LK(rope_kernel<float>, blocks_for(T * c.kv_heads * 32, 256), 256, m->k_tmp, m->cos_t, m->sin_t, k.kr, T, (int)c.kv_heads,
           (int)seq_len, 0, tc ? k.kr_b : (__nv_bfloat16 *)nullptr);
        if (tc) {
            QLC_TRY(launch_convert_f32_to_bf16(m->ctx, k.v, k.v_b, T * kv));
            QLC_TRY(attention_tc_forward(m->ctx, k.qr_b, k.kr_b, k.v_b, k.attn_out, nullptr, k.lse, n_seq, seq_len, c.heads,
                                         c.kv_heads));
        } else {
            attn_fwd_kernel<<<agrid, kAttnThreads, 3 * sizeof(Tile), st>>>(k.qr, k.kr, k.v, k.attn_out, k.lse, (int)seq_len,
                                                                            (int)c.heads, (int)c.kv_heads);
            m->ctx->launches += 1;
            QLC_CUDA(cudaGetLastError());
        }
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_O], k.attn_out, T, m->tmp_h));
        LK(add_kernel, blocks_for(T * h, 256), 256, k.x_in, m->tmp_h, (const float *)nullptr, k.x_mid, T * h);
        LK(rmsnorm_fwd_kernel, rows_grid, 256, k.x_mid, L.mlp_norm, c.rms_eps, k.xn_mlp, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (float *)nullptr);
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_GATE], k.xn_mlp, T, k.gate));
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_UP], k.xn_mlp, T, k.up));
        LK(swiglu_fwd_kernel, blocks_for(T * I, 256), 256, k.gate, k.up, k.act, T * I);
        QLC_TRY(lin_fwd(m, L.proj[QLC_LLAMA_DOWN], k.act, T, m->tmp_h));
        LK(add_kernel, blocks_for(T * h, 256), 256, k.x_mid, m->tmp_h, (const float *)nullptr, x_out, T * h);
    }
    LK(rmsnorm_fwd_kernel, rows_grid, 256, m->x_final, m->d_final_norm, c.rms_eps, m->hn, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (float *)nullptr);
    QLC_TRY(head_forward(m, T));
    (void)kv;
    m->have_cache = true;
    return QLC_OK;
}

// dlogits (fp32 and / or bf16, on the device) -> adapter gradients in the layers' buckets.
int run_backward(qlc_llama *m, size_t n_seq, size_t seq_len, bool dlogits_bf16_ready) {
    if (m->pipeline) return run_backward_pipeline(m, n_seq, seq_len, dlogits_bf16_ready);
    const qlc_llama_config &c = m->cfg;
    cudaStream_t st = m->ctx->stream;
    const size_t T = n_seq * seq_len, h = c.hidden, I = c.intermediate;
    const unsigned rows_grid = blocks_for(T, 8);
    const dim3 agrid((unsigned)((seq_len + kAttnRows - 1) / kAttnRows), (unsigned)c.heads, (unsigned)n_seq);
    QLC_TRY(head_backward(m, T, dlogits_bf16_ready, m->dxn));
    float *dx = m->dx, *dx_alt = m->dx2;
    LK(rmsnorm_bwd_kernel, rows_grid, 256, m->x_final, m->d_final_norm, m->dxn, c.rms_eps, (const float *)nullptr, dx, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (const float *)nullptr, (float *)nullptr);
    for (size_t li = m->layers.size(); li-- > 0;) {
        LlamaLayer &L = m->layers[li];
        LlamaCache &k = L.c;
        // MLP branch (llama.rs:554-575)
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_DOWN], k.act, dx, T, m->d_act));
        LK(swiglu_bwd_kernel, blocks_for(T * I, 256), 256, k.gate, k.up, m->d_act, m->dg, m->du, T * I);
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_GATE], k.xn_mlp, m->dg, T, m->dxn));
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_UP], k.xn_mlp, m->du, T, m->dxn2));
        LK(add_kernel, blocks_for(T * h, 256), 256, m->dxn, m->dxn2, (const float *)nullptr, m->dxn, T * h);
        // dx_mid = rmsnorm_backward(x_mid, dxn) + dx   (residual)
        LK(rmsnorm_bwd_kernel, rows_grid, 256, k.x_mid, L.mlp_norm, m->dxn, c.rms_eps, dx, dx_alt, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (const float *)nullptr, (float *)nullptr);
        // attention branch (llama.rs:577-601)
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_O], k.attn_out, dx_alt, T, m->d_attn));
        if (attn_uses_tc(m)) {
            QLC_TRY(attention_tc_backward(m->ctx, k.qr_b, k.kr_b, k.v_b, k.attn_out, m->d_attn, nullptr, m->d_attn_b, k.lse,
                                          m->delta, m->dqr, m->dkr, m->dv, nullptr, m->dk_parts, m->dv_parts, n_seq, seq_len,
                                          c.heads, c.kv_heads));
        } else {
            QLC_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnDqSmem));
            attn_bwd_dq_kernel<<<agrid, kAttnThreads, kAttnDqSmem, st>>>(k.qr, k.kr, k.v, k.attn_out, m->d_attn, k.lse, m->delta,
                                                                          m->dqr, (int)seq_len, (int)c.heads, (int)c.kv_heads);
            QLC_CUDA(cudaGetLastError());
            QLC_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnDkvSmem));
            attn_bwd_dkdv_kernel<<<agrid, kAttnThreads, kAttnDkvSmem, st>>>(k.qr, k.kr, k.v, m->d_attn, k.lse, m->delta,
                                                                             m->dk_parts, m->dv_parts, T * m->kv_dim, (int)seq_len,
                                                                             (int)c.heads, (int)c.kv_heads);
            m->ctx->launches += 2;
            QLC_CUDA(cudaGetLastError());
            const int n_rep = (int)(c.heads / c.kv_heads);
            LK(sum_parts_kernel, blocks_for(T * m->kv_dim, 256), 256, m->dk_parts, T * m->kv_dim, n_rep, m->dkr, T * m->kv_dim);
            LK(sum_parts_kernel, blocks_for(T * m->kv_dim, 256), 256, m->dv_parts, T * m->kv_dim, n_rep, m->dv, T * m->kv_dim);
        }
        LK(rope_kernel<float>, blocks_for(T * c.heads * 32, 256), 256, m->dqr, m->cos_t, m->sin_t, m->dq, T, (int)c.heads,
           (int)seq_len, 1, (__nv_bfloat16 *)nullptr);
        LK(rope_kernel<float>, blocks_for(T * c.kv_heads * 32, 256), 256, m->dkr, m->cos_t, m->sin_t, m->dk, T, (int)c.kv_heads,
           (int)seq_len, 1, (__nv_bfloat16 *)nullptr);
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_Q], k.xn_attn, m->dq, T, m->dxn));
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_K], k.xn_attn, m->dk, T, m->dxn2));
        QLC_TRY(lin_bwd(m, L.proj[QLC_LLAMA_V], k.xn_attn, m->dv, T, m->dxn3));
        LK(add_kernel, blocks_for(T * h, 256), 256, m->dxn, m->dxn2, m->dxn3, m->dxn, T * h);
        // dx_in = rmsnorm_backward(x_in, dxn) + dx_mid
        LK(rmsnorm_bwd_kernel, rows_grid, 256, k.x_in, L.attn_norm, m->dxn, c.rms_eps, dx_alt, dx, T, (int)h, (__nv_bfloat16 *)nullptr, (const float *)nullptr, (const float *)nullptr, (float *)nullptr);
    }
    return QLC_OK;
}

int check_ids(const qlc_llama *m, const uint32_t *ids, size_t n, const char *what) {
    for (size_t i = 0; i < n; ++i)
        if (ids[i] >= m->cfg.vocab) return fail(QLC_ERR_INVALID_CONFIG, "%s[%zu] = %u is outside the vocabulary (%zu)", what, i, ids[i], m->cfg.vocab);
    return QLC_OK;
}

int upload_ids(qlc_llama *m, const uint32_t *ids, const uint32_t *targets, size_t n_seq, size_t seq_len) {
    if (!m || !ids) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (n_seq == 0 || seq_len == 0) return fail(QLC_ERR_SHAPE_MISMATCH, "empty batch (n_seq %zu, seq_len %zu)", n_seq, seq_len);
    for (const LlamaLayer &L : m->layers)
        for (int k = 0; k < QLC_LLAMA_PROJ_COUNT; ++k)
            if (!L.proj[k]) return fail(QLC_ERR_INVALID_CONFIG, "a layer's weights were never set (qlc_llama_set_layer)");
    const size_t T = n_seq * seq_len;
    QLC_TRY(check_ids(m, ids, T, "ids"));
    if (targets) QLC_TRY(check_ids(m, targets, T, "targets"));
    QLC_CUDA(cudaSetDevice(m->ctx->device));
    QLC_TRY(ensure_capacity(m, n_seq, seq_len));
    QLC_CUDA(cudaMemcpyAsync(m->d_ids, ids, T * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    if (targets) QLC_CUDA(cudaMemcpyAsync(m->d_targets, targets, T * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    return QLC_OK;
}

int sync(qlc_llama *m) {
    // the lanes were joined into the model's stream; their status words still have to be read
    const int st = qlc_ctx_synchronize(m->ctx);
    for (qlc_ctx *l : m->lane)
        if (l) {
            const int sl = qlc_ctx_synchronize(l);
            if (st == QLC_OK && sl != QLC_OK) return sl;
        }
    return st;
}

}  // namespace
}  // namespace qlc

using namespace qlc;

extern "C" {

int qlc_llama_create(qlc_ctx *ctx, const qlc_llama_config *cfg, const float *embed, const float *final_norm,
                     qlc_llama **out) {
    if (!ctx || !cfg || !embed || !final_norm || !out) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (!cfg->hidden || !cfg->heads || !cfg->kv_heads || !cfg->intermediate || !cfg->vocab)
        return fail(QLC_ERR_INVALID_CONFIG, "zero dimension in the model configuration");
    if (cfg->hidden % cfg->heads || cfg->hidden / cfg->heads != (size_t)kHeadDim)
        return fail(QLC_ERR_INVALID_CONFIG, "head dimension must be %d (hidden %zu, heads %zu)", kHeadDim, cfg->hidden, cfg->heads);
    if (cfg->heads % cfg->kv_heads) return fail(QLC_ERR_INVALID_CONFIG, "heads (%zu) must be a multiple of kv_heads (%zu)", cfg->heads, cfg->kv_heads);
    QLC_CUDA(cudaSetDevice(ctx->device));
    qlc_llama *m = new (std::nothrow) qlc_llama;
    if (!m) return fail(QLC_ERR_GPU, "out of host memory");
    m->ctx = ctx;
    m->cfg = *cfg;
    m->kv_dim = cfg->kv_heads * kHeadDim;
    m->layers.resize(cfg->layers);
    ctx->refs += 1;
    const size_t ne = cfg->vocab * cfg->hidden;
    int st = QLC_OK;
    auto chk = [&](cudaError_t e) {
        if (e != cudaSuccess && st == QLC_OK) st = fail(QLC_ERR_GPU, "model set-up: %s", cudaGetErrorString(e));
    };
    chk(cudaMalloc(reinterpret_cast<void **>(&m->d_embed), ne * 4));
    chk(cudaMalloc(reinterpret_cast<void **>(&m->d_embed_bf16), ne * 2 + 16));
    chk(cudaMalloc(reinterpret_cast<void **>(&m->d_final_norm), cfg->hidden * 4));
    if (st == QLC_OK) chk(cudaMemcpyAsync(m->d_embed, embed, ne * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (st == QLC_OK) chk(cudaMemcpyAsync(m->d_final_norm, final_norm, cfg->hidden * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (st == QLC_OK) st = launch_convert_f32_to_bf16(ctx, m->d_embed, m->d_embed_bf16, ne);
    if (st == QLC_OK) st = qlc_ctx_synchronize(ctx);
    if (st != QLC_OK) {
        qlc_llama_destroy(m);
        return st;
    }
    *out = m;
    return QLC_OK;
}

int qlc_llama_destroy(qlc_llama *m) {
    if (!m) return QLC_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (int i = 0; i < 2; ++i) {
        if (m->lane[i]) {
            cudaStreamSynchronize(m->lane[i]->stream);
            qlc_ctx_destroy(m->lane[i]);
        }
        if (m->ev_lane[i]) cudaEventDestroy(m->ev_lane[i]);
    }
    if (m->ev_main) cudaEventDestroy(m->ev_main);
    free_activations(m);
    for (LlamaLayer &L : m->layers) {
        cudaFree(L.attn_norm);
        cudaFree(L.mlp_norm);
        for (qlc_layer *p : L.proj) qlc_layer_destroy(p);
        qlc_layer_destroy(L.gate_up);
        qlc_layer_destroy(L.qkv);
    }
    cudaFree(m->d_embed);
    cudaFree(m->d_embed_bf16);
    cudaFree(m->d_final_norm);
    qlc_ctx *ctx = m->ctx;
    delete m;
    return qlc_ctx_destroy(ctx);
}

// quantize == nullptr: every projection is NF4-quantised; otherwise projection k is quantised iff quantize[k] != 0
// and kept as a raw fp32 matrix (llama.rs:87-93, Proj::Raw) otherwise.
// (Re)builds L.gate_up from the gate and up layers: possible when both are quantised the same way and gate's element
// count is a whole number of quantisation blocks and (double quantisation) of 256-block groups, so that the flat
// blocking of the concatenated (2I, h) matrix (quant.rs:100-118, 283-299) is the two matrices' blockings one after
// the other.  The payload is copied, not re-quantised: the merged layer multiplies by the very same weights.
static int build_gate_up(qlc_llama *m, LlamaLayer &L) {
    qlc_layer_destroy(L.gate_up);
    L.gate_up = nullptr;
    const qlc_layer *g = L.proj[QLC_LLAMA_GATE], *u = L.proj[QLC_LLAMA_UP];
    if (!g || !u || !g->w || !u->w || g->r || u->r) return QLC_OK;
    const qlc_qtensor *qg = g->w, *qu = u->w;
    if (qg->block_size != qu->block_size || qg->dq != qu->dq || qg->n != qu->n || qg->cols != qu->cols) return QLC_OK;
    if (qg->n % qg->block_size || (qg->n & 1) || (qg->dq && qg->nb % 256)) return QLC_OK;
    qlc_qtensor *q = nullptr;
    QLC_TRY(alloc_qtensor(m->ctx, qg->rows + qu->rows, qg->cols, qg->block_size, qg->dq, &q));
    cudaStream_t st = m->ctx->stream;
    int rc = QLC_OK;
    auto copy = [&](void *dst, const void *src, size_t bytes) {
        if (rc == QLC_OK && bytes && cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            rc = fail(QLC_ERR_GPU, "copy of a quantised payload failed");
    };
    copy(q->d_codes, qg->d_codes, qg->n / 2);
    copy(q->d_codes + qg->n / 2, qu->d_codes, qu->n / 2);
    if (qg->dq) {
        copy(q->d_absmax_codes, qg->d_absmax_codes, qg->nb);
        copy(q->d_absmax_codes + qg->nb, qu->d_absmax_codes, qu->nb);
        copy(q->d_absmax2, qg->d_absmax2, qg->nb / 256 * 4);
        copy(q->d_absmax2 + qg->nb / 256, qu->d_absmax2, qu->nb / 256 * 4);
    } else {
        copy(q->d_scales_f32, qg->d_scales_f32, qg->nb * 4);
        copy(q->d_scales_f32 + qg->nb, qu->d_scales_f32, qu->nb * 4);
    }
    if (rc == QLC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(QLC_ERR_GPU, "copy of a quantised payload failed");
    if (rc == QLC_OK) rc = qlc_layer_create(m->ctx, q, nullptr, 0, nullptr, 0, 0, 0.0f, &L.gate_up);
    qlc_qtensor_destroy(q);  // the layer holds its own reference on success
    if (rc == QLC_OK && !umma_fused_supported(L.gate_up)) {
        qlc_layer_destroy(L.gate_up);
        L.gate_up = nullptr;
    }
    return rc;
}

// (Re)builds L.qkv from the q, k and v layers.  The merged (h + 2 kv, h) weight carries fp32 block scales, decoded
// from each projection's payload exactly as dequantisation decodes them (quant.rs:212-221), so it multiplies by the
// very same weights whatever the projections' double-quantisation grouping; each projection must hold a whole
// number of quantisation blocks.  The merged adapter (rank = the sum of the ranks, at most 64) needs one common
// alpha / r; its operands are rebuilt from the projections' A / B before every forward pass.
static int build_qkv(qlc_llama *m, LlamaLayer &L) {
    qlc_layer_destroy(L.qkv);
    L.qkv = nullptr;
    const int kinds[3] = {QLC_LLAMA_Q, QLC_LLAMA_K, QLC_LLAMA_V};
    size_t rows = 0, r_m = 0, n_total = 0, nb_total = 0;
    float scale = 0.0f;
    for (int i = 0; i < 3; ++i) {
        const qlc_layer *P = L.proj[kinds[i]];
        if (!P || !P->w) return QLC_OK;
        const qlc_qtensor *q = P->w;
        if (q->block_size != L.proj[QLC_LLAMA_Q]->w->block_size || q->n % q->block_size || (q->n & 1)) return QLC_OK;
        rows += q->rows;
        n_total += q->n;
        nb_total += q->nb;
        if (P->r) {
            const float sc = P->alpha / (float)P->r;  // lora.rs:64-66
            if (r_m && sc != scale) return QLC_OK;
            scale = sc;
            r_m += P->r;
        }
    }
    if (r_m > 64) return QLC_OK;
    const size_t h = m->cfg.hidden;
    qlc_qtensor *q = nullptr;
    QLC_TRY(alloc_qtensor(m->ctx, rows, h, L.proj[QLC_LLAMA_Q]->w->block_size, false, &q));
    cudaStream_t st = m->ctx->stream;
    int rc = QLC_OK;
    size_t e0 = 0, b0 = 0;
    for (int i = 0; i < 3 && rc == QLC_OK; ++i) {
        const qlc_qtensor *src = L.proj[kinds[i]]->w;
        if (cudaMemcpyAsync(q->d_codes + e0 / 2, src->d_codes, src->n / 2, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            rc = fail(QLC_ERR_GPU, "copy of a quantised payload failed");
        if (rc == QLC_OK) rc = launch_decode_block_scales(m->ctx, src, q->d_scales_f32 + b0);
        e0 += src->n;
        b0 += src->nb;
    }
    if (rc == QLC_OK && r_m) {
        std::vector<float> a0(r_m * h, 0.0f), b0v(rows * r_m, 0.0f);  // placeholders: the operands come from the projections
        rc = qlc_layer_create(m->ctx, q, a0.data(), a0.size(), b0v.data(), b0v.size(), r_m, scale * (float)r_m, &L.qkv);
    } else if (rc == QLC_OK) {
        rc = qlc_layer_create(m->ctx, q, nullptr, 0, nullptr, 0, 0, 0.0f, &L.qkv);
    }
    if (rc == QLC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(QLC_ERR_GPU, "building the merged q | k | v layer failed");
    qlc_qtensor_destroy(q);  // the layer holds its own reference on success
    // the common scale must survive the round trip through alpha, and the fused kernels must take the merged shape
    if (rc == QLC_OK && ((L.qkv->r && L.qkv->alpha / (float)L.qkv->r != scale) || !umma_fused_supported(L.qkv))) {
        qlc_layer_destroy(L.qkv);
        L.qkv = nullptr;
    }
    (void)n_total;
    (void)nb_total;
    return rc;
}

static int set_layer_impl(qlc_llama *m, size_t li, const float *attn_norm, const float *mlp_norm,
                          const float *const *weights, const int *quantize, size_t block_size, int double_quant) {
    if (!m || !attn_norm || !mlp_norm || !weights) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (li >= m->layers.size()) return fail(QLC_ERR_INVALID_CONFIG, "layer %zu of %zu", li, m->layers.size());
    QLC_CUDA(cudaSetDevice(m->ctx->device));
    LlamaLayer &L = m->layers[li];
    const size_t h = m->cfg.hidden;
    if (!L.attn_norm) QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&L.attn_norm), h * 4));
    if (!L.mlp_norm) QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&L.mlp_norm), h * 4));
    QLC_CUDA(cudaMemcpy(L.attn_norm, attn_norm, h * 4, cudaMemcpyHostToDevice));
    QLC_CUDA(cudaMemcpy(L.mlp_norm, mlp_norm, h * 4, cudaMemcpyHostToDevice));
    for (int k = 0; k < QLC_LLAMA_PROJ_COUNT; ++k) {
        if (!weights[k]) return fail(QLC_ERR_INVALID_CONFIG, "null weight matrix %d", k);
        const size_t o = proj_out(m, k), i = proj_in(m, k);
        qlc_layer *nl = nullptr;
        if (!quantize || quantize[k]) {
            QLC_TRY(qlc_layer_create_from_fp32(m->ctx, weights[k], o * i, o, i, block_size, double_quant, nullptr, 0, nullptr,
                                               0, 0, 0.0f, &nl));
        } else {
            float *tmp = nullptr;
            QLC_CUDA(cudaMalloc(reinterpret_cast<void **>(&tmp), (o * i + 4) * 4));
            int st = QLC_OK;
            if (cudaMemcpyAsync(tmp, weights[k], o * i * 4, cudaMemcpyHostToDevice, m->ctx->stream) != cudaSuccess)
                st = fail(QLC_ERR_GPU, "upload of weight matrix %d failed", k);
            if (st == QLC_OK) st = layer_create_raw(m->ctx, tmp, o, i, &nl);
            cudaStreamSynchronize(m->ctx->stream);
            cudaFree(tmp);
            QLC_TRY(st);
        }
        qlc_layer_destroy(L.proj[k]);
        L.proj[k] = nl;
    }
    QLC_TRY(build_gate_up(m, L));
    return build_qkv(m, L);
}

int qlc_llama_set_layer(qlc_llama *m, size_t li, const float *attn_norm, const float *mlp_norm,
                        const float *const *weights, size_t block_size, int double_quant) {
    return set_layer_impl(m, li, attn_norm, mlp_norm, weights, nullptr, block_size, double_quant);
}

int qlc_llama_set_layer_mixed(qlc_llama *m, size_t li, const float *attn_norm, const float *mlp_norm,
                              const float *const *weights, const int *quantize, size_t block_size, int double_quant) {
    if (!quantize) return fail(QLC_ERR_INVALID_CONFIG, "null quantize flags");
    return set_layer_impl(m, li, attn_norm, mlp_norm, weights, quantize, block_size, double_quant);
}

int qlc_llama_attach_adapter(qlc_llama *m, size_t li, int kind, const float *a, const float *b, size_t r, float alpha) {
    if (!m || !a || !b) return fail(QLC_ERR_INVALID_CONFIG, "null argument");
    if (li >= m->layers.size() || kind < 0 || kind >= QLC_LLAMA_PROJ_COUNT)
        return fail(QLC_ERR_INVALID_CONFIG, "no projection %d in layer %zu", kind, li);
    qlc_layer *old = m->layers[li].proj[kind];
    if (!old) return fail(QLC_ERR_INVALID_CONFIG, "set the layer's weights before attaching adapters");
    const size_t o = proj_out(m, kind), i = proj_in(m, kind);
    qlc_layer *nl = nullptr;
    if (old->w) {
        QLC_TRY(qlc_layer_create(m->ctx, qlc_layer_weight(old), a, r * i, b, o * r, r, alpha, &nl));
    } else {
        // A raw projection that becomes an adapter target is quantised now, with the reference's default
        // QuantConfig (block 64, double quantisation), as its loader does for targets (llama.rs:228-249).
        QLC_CUDA(cudaSetDevice(m->ctx->device));
        qlc_qtensor *q = nullptr;
        QLC_TRY(qlc_quantize_nf4_dev(m->ctx, old->d_w_raw, o, i, 64, 1, &q));
        const int st = qlc_layer_create(m->ctx, q, a, r * i, b, o * r, r, alpha, &nl);
        qlc_qtensor_destroy(q);  // the layer holds its own reference on success
        QLC_TRY(st);
    }
    qlc_layer_destroy(old);
    m->layers[li].proj[kind] = nl;
    if (kind == QLC_LLAMA_GATE || kind == QLC_LLAMA_UP) return build_gate_up(m, m->layers[li]);  // (drops the merged layer)
    if (kind == QLC_LLAMA_Q || kind == QLC_LLAMA_K || kind == QLC_LLAMA_V) return build_qkv(m, m->layers[li]);
    return QLC_OK;
}

qlc_layer *qlc_llama_projection(qlc_llama *m, size_t li, int kind) {
    if (!m || li >= m->layers.size() || kind < 0 || kind >= QLC_LLAMA_PROJ_COUNT) return nullptr;
    return m->layers[li].proj[kind];
}

int qlc_llama_forward(qlc_llama *m, const uint32_t *ids, size_t n_seq, size_t seq_len, float *logits) {
    QLC_TRY(upload_ids(m, ids, nullptr, n_seq, seq_len));
    QLC_TRY(run_forward(m, n_seq, seq_len));
    if (logits)
        QLC_CUDA(cudaMemcpyAsync(logits, m->logits, n_seq * seq_len * m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    return sync(m);
}

int qlc_llama_backward(qlc_llama *m, const uint32_t *ids, const float *dlogits, size_t n_seq, size_t seq_len) {
    if (!dlogits) return fail(QLC_ERR_INVALID_CONFIG, "null dlogits");
    QLC_TRY(upload_ids(m, ids, nullptr, n_seq, seq_len));
    QLC_TRY(run_forward(m, n_seq, seq_len));  // forward with recording, as llama.rs:389-400
    QLC_CUDA(cudaMemcpyAsync(m->dlogits, dlogits, n_seq * seq_len * m->cfg.vocab * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    QLC_TRY(run_backward(m, n_seq, seq_len, false));
    return sync(m);
}

// Forward, loss and backward; the loss gradient is (softmax - onehot) / (tokens * ranks): `ranks` > 1 is the
// data-parallel case, where the sum of the ranks' gradients is the gradient of the mean over all their tokens.
static int loss_backward_impl(qlc_llama *m, const uint32_t *ids, const uint32_t *targets, size_t n_seq, size_t seq_len,
                              float *loss, int ranks, bool sync_now) {
    if (!targets) return fail(QLC_ERR_INVALID_CONFIG, "null targets");
    QLC_TRY(upload_ids(m, ids, targets, n_seq, seq_len));
    // On the tensor-core path the head GEMM rounds its operands to bf16 anyway; the loss then also takes the logits
    // as bf16, which halves what the head writes and what the loss kernel reads (twice).
    static const bool f32_logits = getenv("QLC_LLAMA_FP32_LOGITS") != nullptr;  // diagnostics
    m->want_bf16_logits = m->pipeline && head_uses_bf16(m) && m->cfg.vocab % 4 == 0 && !f32_logits;
    const int fwd = run_forward(m, n_seq, seq_len);
    m->want_bf16_logits = false;
    QLC_TRY(fwd);
    const size_t T = n_seq * seq_len;
    cudaStream_t st = m->ctx->stream;
    const bool bf = head_uses_bf16(m);
    const float inv_count = 1.0f / ((float)T * (float)ranks);
    if (m->logits_are_bf16)
        LK(softmax_ce_vec_kernel<__nv_bfloat16>, (unsigned)T, kCeThreads, reinterpret_cast<const __nv_bfloat16 *>(m->logits),
           (const uint32_t *)m->d_targets, m->cfg.vocab, inv_count, m->row_loss, (float *)nullptr, m->dlogits_bf16);
    else if (m->cfg.vocab % 4 == 0)
        LK(softmax_ce_vec_kernel<float>, (unsigned)T, kCeThreads, (const float *)m->logits, (const uint32_t *)m->d_targets,
           m->cfg.vocab, inv_count, m->row_loss, bf ? (float *)nullptr : m->dlogits,
           bf ? m->dlogits_bf16 : (__nv_bfloat16 *)nullptr);
    else
        LK(softmax_ce_kernel, (unsigned)T, 256, m->logits, m->d_targets, m->cfg.vocab, inv_count, m->row_loss,
           bf ? (float *)nullptr : m->dlogits, bf ? m->dlogits_bf16 : (__nv_bfloat16 *)nullptr);
    QLC_TRY(run_backward(m, n_seq, seq_len, bf));
    if (loss) {
        std::vector<float> rl(T);
        QLC_CUDA(cudaMemcpyAsync(rl.data(), m->row_loss, T * 4, cudaMemcpyDeviceToHost, st));
        QLC_TRY(sync(m));
        double s = 0.0;  // mean over all positions (llama.rs:506: per-sequence mean; equal lengths)
        for (float v : rl) s += v;
        *loss = (float)(s / (double)T);
        return QLC_OK;
    }
    return sync_now ? sync(m) : QLC_OK;
}

int qlc_llama_loss_backward(qlc_llama *m, const uint32_t *ids, const uint32_t *targets, size_t n_seq, size_t seq_len,
                            float *loss) {
    return loss_backward_impl(m, ids, targets, n_seq, seq_len, loss, 1, true);
}

static int train_step_impl(qlc_llama *m, qlc_adam *adam, qlc_comm *comm, const uint32_t *ids, const uint32_t *targets,
                           size_t n_seq, size_t seq_len, float *loss) {
    if (!adam) return fail(QLC_ERR_INVALID_CONFIG, "null optimizer");
    if (comm && qlc_comm_context(comm) != m->ctx)
        return fail(QLC_ERR_INVALID_CONFIG, "the communicator must be created on the model's context");
    const int ranks = comm ? qlc_comm_nranks(comm) : 1;
    static const bool host_timing = getenv("QLC_LLAMA_HOST_TIMING") != nullptr;  // diagnostics
    const auto t_begin = std::chrono::steady_clock::now();
    // everything below is ordered on the model's stream: no host synchronisation before the step's end
    QLC_TRY(loss_backward_impl(m, ids, targets, n_seq, seq_len, loss, ranks, false));
    const auto t_bwd = std::chrono::steady_clock::now();
    // optimiser tensor order of the reference's loop: layers reversed, projections in kind order, A then B
    // (qlora-model/examples/train_smollm.rs:42-45, 63-72)
    std::vector<float *> params;
    std::vector<const float *> grads;
    std::vector<size_t> lens;
    std::vector<float *> buckets;
    std::vector<size_t> bucket_lens;
    std::vector<qlc_layer *> updated;
    for (size_t li = m->layers.size(); li-- > 0;)
        for (int k = 0; k < QLC_LLAMA_PROJ_COUNT; ++k) {
            qlc_layer *L = m->layers[li].proj[k];
            if (!L || !L->r) continue;
            const size_t na = L->r * L->in_dim, nb = L->out_dim * L->r;
            params.push_back(L->d_a);
            grads.push_back(L->d_grad_bucket);
            lens.push_back(na);
            params.push_back(L->d_b);
            grads.push_back(L->d_grad_bucket + na);
            lens.push_back(nb);
            buckets.push_back(L->d_grad_bucket);  // A and B gradients of a layer are one contiguous bucket
            bucket_lens.push_back(na + nb);
            updated.push_back(L);
        }
    if (params.empty()) return sync(m);
    if (comm && ranks > 1) QLC_TRY(qlc_comm_allreduce_sum_f32_many(comm, buckets.data(), bucket_lens.data(), buckets.size()));
    QLC_TRY(qlc_adam_step_dev(adam, params.size(), params.data(), grads.data(), lens.data(), nullptr));
    // the bf16 operand copies of all adapters, rebuilt in one launch per 64 adapters
    QLC_TRY(launch_refresh_adapters(m->ctx, updated.data(), updated.size()));
    for (qlc_layer *L : updated) L->shadow_valid = false;
    const auto t_sub = std::chrono::steady_clock::now();
    const int st_sync = sync(m);
    if (host_timing) {
        const auto t_end = std::chrono::steady_clock::now();
        auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
        fprintf(stderr, "[qlc llama] host: forward+backward submitted after %.2f ms, optimiser after %.2f ms, step done after %.2f ms\n",
                ms(t_begin, t_bwd), ms(t_begin, t_sub), ms(t_begin, t_end));
    }
    return st_sync;
}

int qlc_llama_train_step(qlc_llama *m, qlc_adam *adam, const uint32_t *ids, const uint32_t *targets, size_t n_seq,
                         size_t seq_len, float *loss) {
    return train_step_impl(m, adam, nullptr, ids, targets, n_seq, seq_len, loss);
}

int qlc_llama_train_step_dp(qlc_llama *m, qlc_adam *adam, qlc_comm *comm, const uint32_t *ids, const uint32_t *targets,
                            size_t n_seq, size_t seq_len, float *loss) {
    if (!comm) return fail(QLC_ERR_INVALID_CONFIG, "null communicator");
    return train_step_impl(m, adam, comm, ids, targets, n_seq, seq_len, loss);
}

int qlc_llama_adapter_grads(qlc_llama *m, size_t li, int kind, float *grad_a, float *grad_b) {
    qlc_layer *L = qlc_llama_projection(m, li, kind);
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "no projection %d in layer %zu", kind, li);
    if (!L->r) return fail(QLC_ERR_INVALID_CONFIG, "projection %d of layer %zu has no adapter", kind, li);
    const size_t na = L->r * L->in_dim, nb = L->out_dim * L->r;
    QLC_CUDA(cudaSetDevice(m->ctx->device));
    QLC_TRY(sync(m));
    if (grad_a) QLC_CUDA(cudaMemcpy(grad_a, L->d_grad_bucket, na * 4, cudaMemcpyDeviceToHost));
    if (grad_b) QLC_CUDA(cudaMemcpy(grad_b, L->d_grad_bucket + na, nb * 4, cudaMemcpyDeviceToHost));
    return QLC_OK;
}

int qlc_llama_adapter_weights(qlc_llama *m, size_t li, int kind, float *a, float *b) {
    qlc_layer *L = qlc_llama_projection(m, li, kind);
    if (!L) return fail(QLC_ERR_INVALID_CONFIG, "no projection %d in layer %zu", kind, li);
    if (!L->r) return fail(QLC_ERR_INVALID_CONFIG, "projection %d of layer %zu has no adapter", kind, li);
    QLC_CUDA(cudaSetDevice(m->ctx->device));
    QLC_TRY(sync(m));
    if (a) QLC_CUDA(cudaMemcpy(a, L->d_a, L->r * L->in_dim * 4, cudaMemcpyDeviceToHost));
    if (b) QLC_CUDA(cudaMemcpy(b, L->d_b, L->out_dim * L->r * 4, cudaMemcpyDeviceToHost));
    return QLC_OK;
}

}  // extern "C"
