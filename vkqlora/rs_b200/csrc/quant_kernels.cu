// NF4 block-wise quantise / dequantise kernels (bandwidth-bound, bit-exact with the reference).
//
// Reference semantics reproduced here (qlora-core/src/quant.rs):
//   :104-154 quantize  — flat blocks over the row-major buffer, absmax with NaN-ignoring max,
//                        IEEE division w/absmax, nearest codebook entry with first-minimum ties,
//                        element 2i -> low nibble of byte i.
//   :283-299 double_quantize_scales — int8 codes of the block absmax in groups of 256.
//   :212-221 block_scales — (code as i8 as f32) / 127 * absmax2 (two roundings).
//   :157-167 dequantize — one fp32 multiply.
// This translation unit is compiled with -fmad=false and uses the _rn intrinsics so that no
// multiply-add is ever fused and division / sqrt are IEEE-rounded.
#include <type_traits>

#include <cuda_fp16.h>

#include "common.cuh"

namespace qlc {
namespace {

// qlora-core/src/quant.rs:27-44 (f64 literals rounded to f32).
__constant__ float c_nf4_levels[16] = {
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

// Decision thresholds of the reference's 16-way nearest-level scan (quant.rs:263-278),
// expressed on the divided target t = w/absmax: T[i] is the smallest fp32 value for which the
// scan returns a code > i.  The scan's result is monotone in t (rounded distances to a level
// are monotone, and adjacent levels are ~2^20 ulps apart, so no third level can tie), hence
// code(t) = #{ i : t >= T[i] }.  The table was derived by bisection over fp32 bit patterns
// against the scan itself and is re-derived and checked by the test-suite; a NaN target
// compares false everywhere and yields code 0, as in the reference.
__device__ __forceinline__ uint32_t nf4_code_of_target(float t) {
    constexpr uint32_t kT[15] = {0xbf591cd8u, 0xbf1c5270u, 0xbeeb847fu, 0xbeadea76u, 0xbe703cecu,
                                 0xbe0d38bbu, 0xbd3a7870u, 0x3d22fb00u, 0x3df64863u, 0x3e5067e1u,
                                 0x3e9582d5u, 0x3ec753fau, 0x3f006d04u, 0x3f248db0u, 0x3f5c89dau};
    uint32_t c = 0;
#pragma unroll
    for (int i = 0; i < 15; ++i) c += (t >= __uint_as_float(kT[i])) ? 1u : 0u;
    return c;
}

__device__ __forceinline__ uint32_t nf4_code(float w, float absmax) {
    if (absmax == 0.0f) return 7u;  // NF4_ZERO_CODE, quant.rs:47
    return nf4_code_of_target(__fdiv_rn(w, absmax));
}

// Same counting rule as nf4_code_of_target, as a 4-step binary search over the sorted thresholds
// (s_thr: the 15 thresholds in shared memory): code = #{ i : t >= T[i] }.
__device__ __forceinline__ uint32_t nf4_code_bsearch(float t, const float *s_thr) {
    uint32_t c = (t >= __uint_as_float(0x3d22fb00u)) ? 8u : 0u;  // T[7]
    c += (t >= s_thr[c + 3]) ? 4u : 0u;
    c += (t >= s_thr[c + 1]) ? 2u : 0u;
    c += (t >= s_thr[c]) ? 1u : 0u;
    return c;
}
__constant__ uint32_t c_nf4_thresholds[15] = {0xbf591cd8u, 0xbf1c5270u, 0xbeeb847fu, 0xbeadea76u, 0xbe703cecu,
                                              0xbe0d38bbu, 0xbd3a7870u, 0x3d22fb00u, 0x3df64863u, 0x3e5067e1u,
                                              0x3e9582d5u, 0x3ec753fau, 0x3f006d04u, 0x3f248db0u, 0x3f5c89dau};

// int8 code of x relative to amax (quant.rs:291-295; also optim.rs:91):
// clamp(round(x / amax * 127)) with Rust's saturating `as i32` (NaN -> 0).
__device__ __forceinline__ uint8_t i8_code(float x, float amax) {
    if (amax == 0.0f) return 0;
    float r = roundf(__fmul_rn(__fdiv_rn(x, amax), 127.0f));
    int q = (r != r) ? 0 : (int)fminf(fmaxf(r, -127.0f), 127.0f);
    return (uint8_t)(int8_t)q;
}

// Decoded block scale (quant.rs:212-221).
__device__ __forceinline__ float decode_scale(bool dq, const uint8_t *__restrict__ absmax_codes,
                                              const float *__restrict__ absmax2,
                                              const float *__restrict__ scales_f32, size_t blk) {
    if (!dq) return scales_f32[blk];
    float c = (float)(int8_t)absmax_codes[blk];
    return __fmul_rn(__fdiv_rn(c, 127.0f), absmax2[blk / kDoubleQuantBlock]);
}

// ---- the fast path of the code selection ---------------------------------------------------------
// Lane b of a warp holds bin b of a 32-entry table: targets with int(t * kBinScale + 16) == b can only be
// decided by threshold bin_k (every other threshold is more than 1e-3 outside the bin), so the code is
// bin_k + (t >= T[bin_k]).  32 bins of width 1/16 over [-1, 1]; adjacent thresholds are >= 0.08 apart.
constexpr float kBinScale = 15.9999f;
__device__ __forceinline__ void nf4_bin_entry(int lane, const float *s_thr, float &bin_thr, uint32_t &bin_k) {
    bin_k = (uint32_t)(((lane & 16) ? 0xEEEEDDDCCBBA9887ull : 0x6554432221110000ull) >> (4 * (lane & 15))) & 15u;
    bin_thr = s_thr[bin_k];
}

// The eight codes (packed, element j in bits 4j..4j+3) of eight weights of one block with absmax `am`.
// All 32 lanes of the warp must call this together (the bin table is read with shuffles).
// Fast path: classify the approximate target ta = w * (1/absmax), which lies within 3e-7 of the exact
// quotient, against the one decision threshold its bin can reach.  If every ta of the thread stays at
// least 1e-6 away from its threshold, the exact quotient falls on the same side and the codes stand;
// otherwise (about one thread in 10^4) the eight codes are redone with the correctly rounded quotient
// (`redone` reports that, for the self-test's statistics).
__device__ __forceinline__ uint32_t nf4_pack8(const float (&v)[8], float am, float bin_thr, uint32_t bin_k,
                                              const float *s_thr, bool &redone) {
    const bool normal = am > 1e-30f && am < 1e30f;
    float ra;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(ra) : "f"(normal ? am : 1.0f));
    uint32_t packed = 0;
    float nearest = 1.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float ta = __fmul_rn(v[j], ra);
        const int bin = __float2int_rz(__fmaf_rn(ta, kBinScale, 16.0f));  // NaN -> bin 0 -> code 0, as the scan
        const float thr = __shfl_sync(0xffffffffu, bin_thr, bin);
        const uint32_t k = __shfl_sync(0xffffffffu, bin_k, bin);
        const float d = __fsub_rn(ta, thr);
        nearest = fminf(nearest, fabsf(d));
        packed |= (k + (d >= 0.0f ? 1u : 0u)) << (4 * j);
    }
    redone = false;
    if (normal && nearest < 1e-6f) {
        // target = w/absmax through the block's reciprocal: q = RN(w*rd), exact residual, one correction
        // (Markstein) - correctly rounded whenever the quotient is a normal number, and every decision
        // threshold is at |t| >= 0.0398, far above the range where it is not.
        const float rd = __frcp_rn(am);
        packed = 0;
        redone = true;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float q = __fmul_rn(v[j], rd);
            const float t = __fmaf_rn(__fmaf_rn(-q, am, v[j]), rd, q);
            packed |= nf4_code_bsearch(t, s_thr) << (4 * j);
        }
    } else if (!normal) {
        // zero block (code 7), or an absmax at the ends of the exponent range / infinite: IEEE division
        packed = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) packed |= nf4_code(v[j], am) << (4 * j);
    }
    return packed;
}

// ---- quantise, block 64: one CTA per super-block of 256 blocks (16384 elements) ---------------
// 8 consecutive lanes own one 64-element block (8 elements each, two 128-bit loads), the block
// absmax is an 8-lane butterfly, each thread emits one packed 32-bit word of codes.  The 256
// block absmax values stay in shared memory and are double-quantised by the same CTA, so the
// fp32 scales never touch HBM.  Algorithmic traffic: 4 B read + 0.5 B codes + 1/64 B + 4/16384 B
// written per element.
constexpr int kQuantThreads = 256;  // measured: 256 beats 128 at every size of the sweep
// Seven CTAs per SM (36 registers per thread): 148 x 7 = 1036 resident CTAs, so the 1024 super-blocks of a
// 4096 x 4096 weight run as ONE wave instead of a full wave and a 13 % one, and 8192^2 / 16384^2 as 3.95 / 15.8.
template <bool kDQ>
__global__ void __launch_bounds__(kQuantThreads, 7)
quantize_nf4_b64_kernel(const float *__restrict__ w, size_t n, size_t nb, uint8_t *__restrict__ codes,
                        float *__restrict__ scales_f32, uint8_t *__restrict__ absmax_codes,
                        float *__restrict__ absmax2) {
    __shared__ float s_scale[256];
    __shared__ float s_warpmax[kQuantThreads / 32];
    __shared__ float s_thr[16];
    pdl_trigger();
    const int t = threadIdx.x;
    const size_t sb = blockIdx.x;
    const size_t base = sb * 16384;
    if (t < 15) s_thr[t] = __uint_as_float(c_nf4_thresholds[t]);
    __syncthreads();
    pdl_wait();  // nothing above touched memory another kernel writes
    float bin_thr;
    uint32_t bin_k;
    nf4_bin_entry(t & 31, s_thr, bin_thr, bin_k);

#pragma unroll 4
    for (int it = 0; it < 16384 / (8 * kQuantThreads); ++it) {
        const size_t e0 = base + (size_t)it * (8 * kQuantThreads) + (size_t)t * 8;
        float v[8];
        if (e0 + 8 <= n) {
            const float4 lo = __ldcs(reinterpret_cast<const float4 *>(w + e0));
            const float4 hi = __ldcs(reinterpret_cast<const float4 *>(w + e0 + 4));
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
            v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (e0 + j < n) ? w[e0 + j] : 0.0f;
        }
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));  // fmaxf drops NaN like f32::max
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
        bool redone;
        uint32_t packed = nf4_pack8(v, am, bin_thr, bin_k, s_thr, redone);
        if (e0 + 8 > n) {  // ragged end: nibbles past the tensor stay 0 (odd-length padding included)
            const uint32_t valid = (e0 < n) ? (uint32_t)(n - e0) : 0u;
            packed = valid ? (packed & (0xFFFFFFFFu >> (4 * (8 - valid)))) : 0u;
        }
        if (e0 + 8 <= n) {
            *reinterpret_cast<uint32_t *>(codes + e0 / 2) = packed;
        } else if (e0 < n) {
            const size_t nbytes = (n - e0 + 1) / 2;
            for (size_t b = 0; b < nbytes; ++b) codes[e0 / 2 + b] = (uint8_t)(packed >> (8 * b));
        }
        if ((t & 7) == 0) s_scale[it * (kQuantThreads / 8) + (t >> 3)] = am;
    }
    __syncthreads();

    // double quantisation of this super-block's 256 block scales (quant.rs:283-299)
    constexpr int kPer = 256 / kQuantThreads;
    float sc[kPer];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const size_t blk = sb * 256 + i * kQuantThreads + t;
        sc[i] = (blk < nb) ? s_scale[i * kQuantThreads + t] : 0.0f;
        if (!kDQ && blk < nb) scales_f32[blk] = sc[i];
        m = fmaxf(m, fabsf(sc[i]));
    }
    if (!kDQ) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((t & 31) == 0) s_warpmax[t >> 5] = m;
    __syncthreads();
    float amax = s_warpmax[0];
#pragma unroll
    for (int i = 1; i < kQuantThreads / 32; ++i) amax = fmaxf(amax, s_warpmax[i]);
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const size_t blk = sb * 256 + i * kQuantThreads + t;
        if (blk < nb) absmax_codes[blk] = i8_code(sc[i], amax);
    }
    if (t == 0) absmax2[sb] = amax;
}

// ---- quantise, any block size (slow, correct): three small passes -------------------------------
__global__ void block_absmax_kernel(const float *__restrict__ w, size_t n, size_t block_size, size_t nb,
                                    float *__restrict__ scales) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const size_t s = b * block_size;
    const size_t e = (s + block_size < n) ? s + block_size : n;
    float am = 0.0f;
    for (size_t i = s; i < e; ++i) am = fmaxf(am, fabsf(w[i]));
    scales[b] = am;
}

__global__ void pack_codes_kernel(const float *__restrict__ w, size_t n, size_t block_size,
                                  const float *__restrict__ scales, uint8_t *__restrict__ codes) {
    const size_t byte = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = byte * 2;
    if (e0 >= n) return;
    uint32_t c = nf4_code(w[e0], scales[e0 / block_size]);
    if (e0 + 1 < n) c |= nf4_code(w[e0 + 1], scales[(e0 + 1) / block_size]) << 4;
    codes[byte] = (uint8_t)c;
}

__global__ void __launch_bounds__(256)
double_quant_kernel(const float *__restrict__ scales, size_t nb, uint8_t *__restrict__ absmax_codes,
                    float *__restrict__ absmax2) {
    __shared__ float s_warpmax[8];
    const int t = threadIdx.x;
    const size_t blk = (size_t)blockIdx.x * 256 + t;
    const float s = (blk < nb) ? scales[blk] : 0.0f;
    float m = fabsf(s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((t & 31) == 0) s_warpmax[t >> 5] = m;
    __syncthreads();
    float amax = s_warpmax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_warpmax[i]);
    if (blk < nb) absmax_codes[blk] = i8_code(s, amax);
    if (t == 0) absmax2[blockIdx.x] = amax;
}

// ---- dequantise ---------------------------------------------------------------------------------
template <typename T> struct OutVec;
template <> struct OutVec<float> {
    static __device__ __forceinline__ void store8(float *p, const float *v) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4 *>(p) + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
    static __device__ __forceinline__ void store1(float *p, float v) { *p = v; }
};
template <> struct OutVec<__nv_bfloat16> {
    static __device__ __forceinline__ void store8(__nv_bfloat16 *p, const float *v) {
        uint4 o;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t *>(&t);
        t = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t *>(&t);
        t = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t *>(&t);
        t = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t *>(&t);
        __stcs(reinterpret_cast<uint4 *>(p), o);
    }
    static __device__ __forceinline__ void store1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

// One thread per 8 elements (one 32-bit word of codes); requires block_size % 8 == 0 so the 8
// elements share one scale.  Algorithmic traffic per element: 0.5 B codes + 1/64 B absmax code
// (+4/16384 B) read, 4 B (fp32) or 2 B (bf16) written.
template <typename OutT>
__global__ void __launch_bounds__(256)
dequant_words_kernel(const uint8_t *__restrict__ codes, bool dq, const uint8_t *__restrict__ absmax_codes,
                     const float *__restrict__ absmax2, const float *__restrict__ scales_f32, size_t n,
                     size_t block_size, OutT *__restrict__ out, size_t word0) {
    __shared__ float s_lut[16];
    if (threadIdx.x < 16) s_lut[threadIdx.x] = c_nf4_levels[threadIdx.x];
    __syncthreads();
    const size_t word = word0 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = word * 8;
    if (e0 >= n) return;
    // The code buffer is allocated padded to 16 bytes, so a whole-word read is always in bounds.
    const uint32_t cw = __ldcs(reinterpret_cast<const uint32_t *>(codes) + word);
    const float scale = decode_scale(dq, absmax_codes, absmax2, scales_f32, e0 / block_size);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(s_lut[(cw >> (4 * j)) & 15u], scale);
    if (e0 + 8 <= n) {
        OutVec<OutT>::store8(out + e0, v);
    } else {
        for (size_t j = 0; e0 + j < n; ++j) OutVec<OutT>::store1(out + e0 + j, v[j]);
    }
}

// ---- dequantise, block 64, streaming kernels ------------------------------------------------------
// Every thread issues all of its loads first (kU packed words, their absmax codes and second-level
// absmax), then decodes.  Consecutive lanes write consecutive 16-byte pieces, so each store instruction
// of a warp covers 512 contiguous bytes.  The exact quotients (i8 as f32)/127 come from a 256-entry
// table computed once per CTA with IEEE division (quant.rs:212-221).
// kU = 8 for large tensors; 4 when that leaves fewer than two waves of CTAs (4096 x 4096: the last wave of the
// larger CTAs was mostly idle).

__device__ __forceinline__ float scale_from(const float *s_q127, bool dq, uint32_t raw, float a2) {
    return dq ? __fmul_rn(s_q127[raw & 255u], a2) : a2;
}

// fp32 output: thread -> one float4 (4 elements = half a packed word) per unrolled step.
template <int kDeqU>
__global__ void __launch_bounds__(256)
dequant_b64_f32_kernel(const uint32_t *__restrict__ codes, bool dq, const uint8_t *__restrict__ absmax_codes,
                       const float *__restrict__ absmax2, const float *__restrict__ scales_f32, size_t n_quads,
                       float4 *__restrict__ out) {
    pdl_trigger();
    __shared__ float s_lut[16];
    __shared__ float s_q127[256];
    if (threadIdx.x < 16) s_lut[threadIdx.x] = c_nf4_levels[threadIdx.x];
    s_q127[threadIdx.x] = __fdiv_rn((float)(int8_t)(uint8_t)threadIdx.x, 127.0f);
    __syncthreads();
    pdl_wait();  // the tables above depend on nothing another kernel writes
    const size_t q0 = (size_t)blockIdx.x * (256 * kDeqU) + threadIdx.x;
    uint32_t w[kDeqU], raw[kDeqU];
    float a2[kDeqU];
#pragma unroll
    for (int i = 0; i < kDeqU; ++i) {
        const size_t q = q0 + (size_t)i * 256;  // float4 index: elements 4q..4q+3, word q/2, block q/16
        if (q < n_quads) {
            w[i] = __ldcs(codes + (q >> 1));
            const size_t blk = q >> 4;
            if (dq) {
                raw[i] = __ldg(absmax_codes + blk);
                a2[i] = __ldg(absmax2 + (blk >> 8));
            } else {
                raw[i] = 0;
                a2[i] = __ldg(scales_f32 + blk);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kDeqU; ++i) {
        const size_t q = q0 + (size_t)i * 256;
        if (q < n_quads) {
            const float sc = scale_from(s_q127, dq, raw[i], a2[i]);
            const uint32_t h = w[i] >> ((q & 1) * 16);
            float4 o;
            o.x = __fmul_rn(s_lut[h & 15u], sc);
            o.y = __fmul_rn(s_lut[(h >> 4) & 15u], sc);
            o.z = __fmul_rn(s_lut[(h >> 8) & 15u], sc);
            o.w = __fmul_rn(s_lut[(h >> 12) & 15u], sc);
            __stcs(out + q, o);
        }
    }
}

// bf16 output: thread -> one packed word (8 elements -> 16 bytes) per unrolled step.
template <int kDeqU>
__global__ void __launch_bounds__(256)
dequant_b64_bf16_kernel(const uint32_t *__restrict__ codes, bool dq, const uint8_t *__restrict__ absmax_codes,
                        const float *__restrict__ absmax2, const float *__restrict__ scales_f32, size_t n_words,
                        uint4 *__restrict__ out) {
    pdl_trigger();
    __shared__ float s_lut[16];
    __shared__ float s_q127[256];
    if (threadIdx.x < 16) s_lut[threadIdx.x] = c_nf4_levels[threadIdx.x];
    s_q127[threadIdx.x] = __fdiv_rn((float)(int8_t)(uint8_t)threadIdx.x, 127.0f);
    __syncthreads();
    pdl_wait();  // the tables above depend on nothing another kernel writes
    const size_t g0 = (size_t)blockIdx.x * (256 * kDeqU) + threadIdx.x;
    uint32_t w[kDeqU], raw[kDeqU];
    float a2[kDeqU];
#pragma unroll
    for (int i = 0; i < kDeqU; ++i) {
        const size_t g = g0 + (size_t)i * 256;  // word index: elements 8g..8g+7, block g/8
        if (g < n_words) {
            w[i] = __ldcs(codes + g);
            const size_t blk = g >> 3;
            if (dq) {
                raw[i] = __ldg(absmax_codes + blk);
                a2[i] = __ldg(absmax2 + (blk >> 8));
            } else {
                raw[i] = 0;
                a2[i] = __ldg(scales_f32 + blk);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kDeqU; ++i) {
        const size_t g = g0 + (size_t)i * 256;
        if (g < n_words) {
            const float sc = scale_from(s_q127, dq, raw[i], a2[i]);
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 t = __floats2bfloat162_rn(__fmul_rn(s_lut[(w[i] >> (8 * j)) & 15u], sc),
                                                               __fmul_rn(s_lut[(w[i] >> (8 * j + 4)) & 15u], sc));
                o[j] = *reinterpret_cast<const uint32_t *>(&t);
            }
            __stcs(out + g, make_uint4(o[0], o[1], o[2], o[3]));
        }
    }
}

// Any block size: one thread per element.
template <typename OutT>
__global__ void dequant_elems_kernel(const uint8_t *__restrict__ codes, bool dq,
                                     const uint8_t *__restrict__ absmax_codes, const float *__restrict__ absmax2,
                                     const float *__restrict__ scales_f32, size_t n, size_t block_size,
                                     OutT *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t byte = codes[i / 2];
    const uint32_t c = (i & 1) ? (byte >> 4) : (byte & 15u);
    const float scale = decode_scale(dq, absmax_codes, absmax2, scales_f32, i / block_size);
    OutVec<OutT>::store1(out + i, __fmul_rn(c_nf4_levels[c], scale));
}

__global__ void decode_scales_kernel(bool dq, const uint8_t *__restrict__ absmax_codes,
                                     const float *__restrict__ absmax2, const float *__restrict__ scales_f32,
                                     size_t nb, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nb) out[i] = decode_scale(dq, absmax_codes, absmax2, scales_f32, i);
}

// ---- small conversion helpers -----------------------------------------------------------------
__global__ void f32_to_bf16_kernel(const float *__restrict__ in, __nv_bfloat16 *__restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i + 8 <= n && ((reinterpret_cast<uintptr_t>(in + i) | reinterpret_cast<uintptr_t>(out + i)) & 15) == 0) {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(in + i));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(in + i) + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        OutVec<__nv_bfloat16>::store8(out + i, v);
    } else {
        for (size_t j = i; j < n && j < i + 8; ++j) out[j] = __float2bfloat16_rn(in[j]);
    }
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16 *__restrict__ in, float *__restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}

__global__ void pad_to_bf16_kernel(const float *__restrict__ in, size_t rows, size_t cols,
                                   __nv_bfloat16 *__restrict__ out, size_t rows_pad, size_t cols_pad) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows_pad * cols_pad) return;
    const size_t r = i / cols_pad, c = i % cols_pad;
    out[i] = __float2bfloat16_rn((r < rows && c < cols) ? in[r * cols + c] : 0.0f);
}

// out (cols_pad, rows_pad) = in(rows, cols)^T
__global__ void pad_transpose_to_bf16_kernel(const float *__restrict__ in, size_t rows, size_t cols,
                                             __nv_bfloat16 *__restrict__ out, size_t cols_pad, size_t rows_pad) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows_pad * cols_pad) return;
    const size_t c = i / rows_pad, r = i % rows_pad;  // out[c][r]
    out[i] = __float2bfloat16_rn((r < rows && c < cols) ? in[r * cols + c] : 0.0f);
}

// The three padded bf16 operand copies of up to kRefreshBatch adapters in one launch (blockIdx.y = adapter):
// a_pad (r_pad, in) = A with zero rows below r; b_pad (out, r_pad) = B with zero columns right of r;
// bt_pad (r_pad, out) = B^T with zero rows below r.
constexpr int kRefreshBatch = 64;
struct AdapterRefresh {
    const float *a, *b;
    __nv_bfloat16 *a_pad, *b_pad, *bt_pad;
    uint32_t r, r_pad, in_dim, out_dim;
};
struct RefreshBatch {
    int n;
    AdapterRefresh d[kRefreshBatch];
};
__global__ void refresh_adapters_kernel(const RefreshBatch batch) {
    pdl_trigger();
    pdl_wait();
    const AdapterRefresh &d = batch.d[blockIdx.y];
    const size_t na = (size_t)d.r_pad * d.in_dim, nb = (size_t)d.out_dim * d.r_pad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < na + 2 * nb; i += (size_t)gridDim.x * blockDim.x) {
        if (i < na) {
            const size_t r = i / d.in_dim, c = i % d.in_dim;
            d.a_pad[i] = __float2bfloat16_rn(r < d.r ? d.a[r * d.in_dim + c] : 0.0f);
        } else if (i < na + nb) {
            const size_t j = i - na, r = j / d.r_pad, c = j % d.r_pad;
            d.b_pad[j] = __float2bfloat16_rn(c < d.r ? d.b[r * d.r + c] : 0.0f);
        } else {
            const size_t j = i - na - nb, c = j / d.out_dim, r = j % d.out_dim;  // bt_pad[c][r] = B[r][c]
            d.bt_pad[j] = __float2bfloat16_rn(c < d.r ? d.b[r * d.r + c] : 0.0f);
        }
    }
}

// ---- self-tests of the code selection (exhaustive parity sweeps; see the C ABI header) -------------
// Codes of `count` consecutive fp32 bit patterns read as divided targets, two per output byte.
__global__ void selftest_codes_of_targets_kernel(uint32_t first_bits, size_t count, uint8_t *__restrict__ out) {
    for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; 2 * b < count; b += (size_t)gridDim.x * blockDim.x) {
        const uint32_t lo = nf4_code_of_target(__uint_as_float(first_bits + (uint32_t)(2 * b)));
        const uint32_t hi = (2 * b + 1 < count) ? nf4_code_of_target(__uint_as_float(first_bits + (uint32_t)(2 * b + 1))) : 0u;
        out[b] = (uint8_t)(lo | (hi << 4));
    }
}

// Every weight bit pattern in [first_bits, first_bits + count) against one block absmax: the quantise kernel's
// own code selection (nf4_pack8: approximate quotient, 32-bin table, exact redo in the guard band) must give
// the code of the IEEE quotient (nf4_code).  out[0] = weights whose codes differ, out[1] = threads that took
// the exact redo, out[2] = the first differing bit pattern (if any).
__global__ void __launch_bounds__(256)
selftest_fast_path_kernel(float absmax, uint32_t first_bits, unsigned long long count, unsigned long long *out) {
    __shared__ float s_thr[16];
    if (threadIdx.x < 15) s_thr[threadIdx.x] = __uint_as_float(c_nf4_thresholds[threadIdx.x]);
    __syncthreads();
    float bin_thr;
    uint32_t bin_k;
    nf4_bin_entry(threadIdx.x & 31, s_thr, bin_thr, bin_k);
    unsigned long long bad = 0, redo = 0, first_bad = ~0ull;
    const unsigned long long groups = (count + 7) / 8, stride = (unsigned long long)gridDim.x * blockDim.x;
    // whole warps iterate together (the table lives in the lanes); trailing groups are computed and discarded
    const unsigned long long rounds = (groups + stride - 1) / stride;
    for (unsigned long long r = 0; r < rounds; ++r) {
        const unsigned long long g = r * stride + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned long long i = g * 8 + j;
            v[j] = i < count ? __uint_as_float(first_bits + (uint32_t)i) : 0.0f;
        }
        bool redone;
        const uint32_t fast = nf4_pack8(v, absmax, bin_thr, bin_k, s_thr, redone);
        if (g < groups) {
            redo += redone ? 1u : 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const unsigned long long i = g * 8 + j;
                if (i < count && ((fast >> (4 * j)) & 15u) != nf4_code(v[j], absmax)) {
                    bad += 1;
                    if (first_bad == ~0ull) first_bad = first_bits + (uint32_t)i;
                }
            }
        }
    }
    if (bad) {
        atomicAdd(out, bad);
        atomicMin(out + 2, first_bad);
    }
    if (redo) atomicAdd(out + 1, redo);
}

inline unsigned grid_for(size_t work, unsigned per_block) { return (unsigned)((work + per_block - 1) / per_block); }

}  // namespace

int launch_quantize_nf4(qlc_ctx *ctx, const float *d_w, qlc_qtensor *q) {
    const size_t n = q->n, nb = q->nb;
    if (n == 0) return QLC_OK;
    const bool aligned = (reinterpret_cast<uintptr_t>(d_w) & 15) == 0;
    if (q->block_size == 64 && aligned) {
        const unsigned grid = (unsigned)ceil_div(nb, 256);
        // launched so that its CTAs may take SMs while the kernel before it in the stream drains (pdl_wait in the
        // kernel orders its memory accesses behind that kernel's completion)
        if (q->dq)
            QLC_CUDA(launch_pdl(quantize_nf4_b64_kernel<true>, dim3(grid), dim3(kQuantThreads), 0, ctx->stream, d_w, n, nb,
                                q->d_codes, (float *)nullptr, q->d_absmax_codes, q->d_absmax2));
        else
            QLC_CUDA(launch_pdl(quantize_nf4_b64_kernel<false>, dim3(grid), dim3(kQuantThreads), 0, ctx->stream, d_w, n, nb,
                                q->d_codes, q->d_scales_f32, (uint8_t *)nullptr, (float *)nullptr));
        ctx->launches += 1;
    } else {
        float *scales = q->d_scales_f32;
        if (q->dq) {
            void *ws = nullptr;
            QLC_TRY(ctx_workspace(ctx, nb * sizeof(float), &ws));
            scales = static_cast<float *>(ws);
        }
        block_absmax_kernel<<<grid_for(nb, 128), 128, 0, ctx->stream>>>(d_w, n, q->block_size, nb, scales);
        pack_codes_kernel<<<grid_for((n + 1) / 2, 256), 256, 0, ctx->stream>>>(d_w, n, q->block_size, scales,
                                                                                q->d_codes);
        ctx->launches += 2;
        if (q->dq) {
            double_quant_kernel<<<(unsigned)ceil_div(nb, 256), 256, 0, ctx->stream>>>(scales, nb, q->d_absmax_codes,
                                                                                      q->d_absmax2);
            ctx->launches += 1;
        }
    }
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

template <typename OutT>
static int launch_dequantize_t(qlc_ctx *ctx, const qlc_qtensor *q, OutT *d_out) {
    const size_t n = q->n;
    if (n == 0) return QLC_OK;
    const bool out_aligned = (reinterpret_cast<uintptr_t>(d_out) & 31) == 0;
    size_t word0 = 0;  // first packed word the generic kernel still has to do
    if (q->block_size == 64 && out_aligned) {
        // whole CTAs of the streaming kernel, the remainder goes to the generic word kernel
        constexpr bool kF32 = std::is_same<OutT, float>::value;
        constexpr size_t kElemsPerStep = kF32 ? 256 * 4 : 256 * 8;  // one unrolled step of a CTA
        // CTAs of 8 steps, or of 4 when 8 would leave fewer than ~3 waves of resident CTAs (about 6 per SM)
        const size_t small_limit = (size_t)ctx->sm_count * 6 * 3;
        const int u = (n / (8 * kElemsPerStep) < small_limit) ? 4 : 8;
        const size_t ctas = n / (u * kElemsPerStep);
        if (ctas > 0) {
            const uint32_t *codes = reinterpret_cast<const uint32_t *>(q->d_codes);
            const size_t units = ctas * u * 256;
            const bool dq = q->dq;
            float4 *of = reinterpret_cast<float4 *>(d_out);
            uint4 *ob = reinterpret_cast<uint4 *>(d_out);
            const dim3 g((unsigned)ctas), b(256);
            cudaError_t e;
            if (kF32 && u == 8)
                e = launch_pdl(dequant_b64_f32_kernel<8>, g, b, 0, ctx->stream, codes, dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, units, of);
            else if (kF32)
                e = launch_pdl(dequant_b64_f32_kernel<4>, g, b, 0, ctx->stream, codes, dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, units, of);
            else if (u == 8)
                e = launch_pdl(dequant_b64_bf16_kernel<8>, g, b, 0, ctx->stream, codes, dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, units, ob);
            else
                e = launch_pdl(dequant_b64_bf16_kernel<4>, g, b, 0, ctx->stream, codes, dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, units, ob);
            QLC_CUDA(e);
            ctx->launches += 1;
            word0 = ctas * u * kElemsPerStep / 8;
        }
    }
    if (word0 * 8 < n) {
        if (q->block_size % 8 == 0 && out_aligned) {
            const size_t words = ceil_div(n, 8) - word0;
            dequant_words_kernel<OutT><<<grid_for(words, 256), 256, 0, ctx->stream>>>(
                q->d_codes, q->dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, n, q->block_size, d_out, word0);
        } else {
            dequant_elems_kernel<OutT><<<grid_for(n, 256), 256, 0, ctx->stream>>>(
                q->d_codes, q->dq, q->d_absmax_codes, q->d_absmax2, q->d_scales_f32, n, q->block_size, d_out);
        }
        ctx->launches += 1;
    }
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_dequantize(qlc_ctx *ctx, const qlc_qtensor *q, void *d_out, int dtype) {
    if (dtype == QLC_DTYPE_F32) return launch_dequantize_t<float>(ctx, q, static_cast<float *>(d_out));
    if (dtype == QLC_DTYPE_BF16) return launch_dequantize_t<__nv_bfloat16>(ctx, q, static_cast<__nv_bfloat16 *>(d_out));
    return fail(QLC_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
}

int launch_decode_block_scales(qlc_ctx *ctx, const qlc_qtensor *q, float *d_out) {
    if (q->nb == 0) return QLC_OK;
    decode_scales_kernel<<<grid_for(q->nb, 256), 256, 0, ctx->stream>>>(q->dq, q->d_absmax_codes, q->d_absmax2,
                                                                        q->d_scales_f32, q->nb, d_out);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_convert_f32_to_bf16(qlc_ctx *ctx, const float *d_in, __nv_bfloat16 *d_out, size_t n) {
    if (n == 0) return QLC_OK;
    f32_to_bf16_kernel<<<grid_for(ceil_div(n, 8), 256), 256, 0, ctx->stream>>>(d_in, d_out, n);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_convert_bf16_to_f32(qlc_ctx *ctx, const __nv_bfloat16 *d_in, float *d_out, size_t n) {
    if (n == 0) return QLC_OK;
    bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, ctx->stream>>>(d_in, d_out, n);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// fp32 copies rounded to tf32 (round to nearest, ties away: cvt.rna), so that the tensor core's truncation
// of the low 13 mantissa bits is exact.  transposed: out[c][r] = in[r][c].
__global__ void pad_to_tf32_kernel(const float *__restrict__ in, size_t rows, size_t cols, float *__restrict__ out,
                                   size_t out_rows, size_t out_cols, int transposed) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= out_rows * out_cols) return;
    const size_t orow = i / out_cols, ocol = i % out_cols;
    const size_t r = transposed ? ocol : orow, c = transposed ? orow : ocol;
    const float v = (r < rows && c < cols) ? in[r * cols + c] : 0.0f;
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    out[i] = __uint_as_float(u);
}
__global__ void f16_to_f32_kernel(const __half *__restrict__ in, float *__restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half2float(in[i]);
}
int launch_convert_f16_to_f32(qlc_ctx *ctx, const void *d_in, float *d_out, size_t n) {
    if (n == 0) return QLC_OK;
    f16_to_f32_kernel<<<grid_for(n, 256), 256, 0, ctx->stream>>>(static_cast<const __half *>(d_in), d_out, n);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// out[i] = in[i] rounded to tf32 (nearest, ties away), four elements per thread where alignment allows.
__global__ void round_to_tf32_kernel(const float *__restrict__ in, float *__restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= n) {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(in + i));
        uint32_t a, b, c, d;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(a) : "f"(v.x));
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(b) : "f"(v.y));
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(c) : "f"(v.z));
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(d) : "f"(v.w));
        *reinterpret_cast<uint4 *>(out + i) = make_uint4(a, b, c, d);
    } else {
        for (size_t k = i; k < n; ++k) {
            uint32_t a;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(a) : "f"(in[k]));
            out[k] = __uint_as_float(a);
        }
    }
}
int launch_round_to_tf32(qlc_ctx *ctx, const float *d_in, float *d_out, size_t n) {
    if (n == 0) return QLC_OK;
    if ((reinterpret_cast<uintptr_t>(d_in) | reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(QLC_ERR_INVALID_CONFIG, "activation buffers must be 16-byte aligned");
    round_to_tf32_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, ctx->stream>>>(d_in, d_out, n);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_pad_to_tf32(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, float *d_out, size_t out_rows,
                       size_t out_cols, int transposed) {
    const size_t total = out_rows * out_cols;
    if (total == 0) return QLC_OK;
    pad_to_tf32_kernel<<<grid_for(total, 256), 256, 0, ctx->stream>>>(d_in, rows, cols, d_out, out_rows, out_cols,
                                                                       transposed);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_pad_to_bf16(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, __nv_bfloat16 *d_out,
                       size_t rows_pad, size_t cols_pad) {
    const size_t total = rows_pad * cols_pad;
    if (total == 0) return QLC_OK;
    pad_to_bf16_kernel<<<grid_for(total, 256), 256, 0, ctx->stream>>>(d_in, rows, cols, d_out, rows_pad, cols_pad);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int launch_pad_transpose_to_bf16(qlc_ctx *ctx, const float *d_in, size_t rows, size_t cols, __nv_bfloat16 *d_out,
                                 size_t cols_pad, size_t rows_pad) {
    const size_t total = rows_pad * cols_pad;
    if (total == 0) return QLC_OK;
    pad_transpose_to_bf16_kernel<<<grid_for(total, 256), 256, 0, ctx->stream>>>(d_in, rows, cols, d_out, cols_pad,
                                                                                 rows_pad);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// Rebuilds the padded bf16 operand copies of every layer in `layers` that has an adapter, 64 adapters per launch.
int launch_refresh_adapters(qlc_ctx *ctx, qlc_layer *const *layers, size_t n) {
    static thread_local RefreshBatch batch;  // one staging copy per host thread
    batch.n = 0;
    auto flush = [&]() -> int {
        if (!batch.n) return QLC_OK;
        QLC_CUDA(launch_pdl(refresh_adapters_kernel, dim3(16, (unsigned)batch.n), dim3(256), 0, ctx->stream, batch));
        ctx->launches += 1;
        QLC_CUDA(cudaGetLastError());
        batch.n = 0;
        return QLC_OK;
    };
    for (size_t i = 0; i < n; ++i) {
        qlc_layer *L = layers[i];
        if (!L || L->r == 0 || !L->d_a_pad) continue;
        batch.d[batch.n++] = AdapterRefresh{L->d_a, L->d_b, L->d_a_pad, L->d_b_pad, L->d_bt_pad, (uint32_t)L->r,
                                            (uint32_t)L->r_pad, (uint32_t)L->in_dim, (uint32_t)L->out_dim};
        L->pad32_valid = false;  // rebuilt by the next TF32-mode call
        if (batch.n == kRefreshBatch) QLC_TRY(flush());
    }
    return flush();
}

int selftest_codes_of_targets(qlc_ctx *ctx, uint32_t first_bits, size_t count, uint8_t *d_out) {
    if (count == 0) return QLC_OK;
    const unsigned grid = (unsigned)ctx->sm_count * 8u;
    selftest_codes_of_targets_kernel<<<grid, 256, 0, ctx->stream>>>(first_bits, count, d_out);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

int selftest_fast_path(qlc_ctx *ctx, float absmax, uint32_t first_bits, unsigned long long count,
                       unsigned long long *d_out3) {
    if (count == 0) return QLC_OK;
    const unsigned grid = (unsigned)ctx->sm_count * 8u;
    selftest_fast_path_kernel<<<grid, 256, 0, ctx->stream>>>(absmax, first_bits, count, d_out3);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

}  // namespace qlc
