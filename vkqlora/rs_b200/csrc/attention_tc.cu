// Causal grouped-query attention (head dimension 64) on the 5th-generation tensor cores, for the bf16 mode
// of the Llama decoder (llama.cu).  Reference mathematics: qlora-model/src/llama.rs:743-792 (forward) in the
// rotated frame (q, k already carry RoPE).
//
// Forward, one CTA per (128 query positions, head, sequence), two passes over the key tiles so that nothing
// in tensor memory ever has to be rescaled:
//   pass 1  S = Q K^T per 128-key tile (tcgen05.mma, fp32 in TMEM); 128 threads, one query row each, read their
//           row of S and keep its maximum m (one FMNMX per element)
//   pass 2  S again; P = exp((S - m) * scale) is written as bf16 into shared memory in the K-major
//           128-byte-swizzled operand layout while its row sum l accumulates in fp32; O += P V accumulates in
//           TMEM over the tiles and is divided by l on the way out.
// Only the tile on the diagonal applies the causal mask; tiles below it take a path without comparisons.
// Row statistics: lse2 = m * scale * log2(e) + log2(l) and delta = sum_d dO * O live in arrays laid out
// [sequence][head][position], the position stride `stat_stride` rounded up to a multiple of 64 so that a
// 64-position run is one aligned 256-byte bulk copy.  The padding of lse2 holds +infinity (written once by the
// owner of the buffer, attention_tc_init_stats): a padded position then has P = 0 without any comparison.
// Q, K and V tiles arrive by TMA as (rows, 64) bf16 tiles; the same K/V tile shape serves as the K-major B
// operand of Q K^T (N = keys, contraction along the 128-byte rows) and as the MN-major B operand of P V
// (N = the 64 dimensions, contraction along the key rows).
// Warp roles: warp 0 = TMA, warp 1 = MMA issue and TMEM owner, warps 2-5 = the 128 row threads.
// Every wait is bounded; on expiry the kernel records a status, unwinds and frees its TMEM.
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

namespace qlc {
namespace {

// 32 consecutive fp32 values (as register bits) to element offset `at` of an fp32 and / or a bf16 array.
__device__ __forceinline__ void store_row32(float *f, __nv_bfloat16 *b, size_t at, const uint32_t (&v)[32]) {
    if (f) {
#pragma unroll
        for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4 *>(f + at + c) = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]),
                                                                  __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
    }
    if (b) {
#pragma unroll
        for (int c = 0; c < 32; c += 8)
            *reinterpret_cast<uint4 *>(b + at + c) =
                make_uint4(pack_bf16(__uint_as_float(v[c]), __uint_as_float(v[c + 1])),
                           pack_bf16(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])),
                           pack_bf16(__uint_as_float(v[c + 4]), __uint_as_float(v[c + 5])),
                           pack_bf16(__uint_as_float(v[c + 6]), __uint_as_float(v[c + 7])));
    }
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kScale = 0.125f;                                // 1 / sqrt(64)
constexpr float kScaleLog2e = 0.125f * 1.4426950408889634f;     // exp(s * scale) = 2^(s * kScaleLog2e)

constexpr int kQT = 128;                 // query rows per CTA
constexpr int kKT = 128;                 // keys per tile
constexpr uint32_t kTileBytes = 128 * 128;  // a (128 rows, 64 bf16) tile
constexpr uint32_t kStageBytes = 2 * kTileBytes;  // K and V
constexpr uint32_t kPBytes = 2 * kTileBytes;      // P: 128 rows x 128 keys bf16 = two 64-key atoms
constexpr uint32_t kFwdTmemCols = 256;   // S: 128 columns, O: 64 columns
constexpr int kFwdThreads = 6 * 32;
// tiles + 1 KiB of alignment slack; the barriers live in the slack (before the tiles when the dynamic window
// starts at least 128 bytes short of a 1-KiB boundary, after them otherwise), so two CTAs fit on an SM
constexpr uint32_t kFwdTiles = kTileBytes + 2 * kStageBytes + kPBytes;
constexpr size_t kFwdSmem = kFwdTiles + 1024;

__global__ void __launch_bounds__(kFwdThreads)
attn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, float *__restrict__ o, __nv_bfloat16 *__restrict__ o_b,
                   float *__restrict__ lse_out, int stat_stride, int seq_len, int heads, int kv_heads,
                   DeviceStatus *status) {
    pdl_trigger();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base, sKV = base + kTileBytes, sP = sKV + 2 * kStageBytes;
    const uint32_t lead = base - smem_u32(smem_raw);
    uint8_t *ctl = lead >= 128 ? smem_raw : gen + kFwdTiles;  // 128 bytes of barriers, TMEM slot and abort flag
    const uint32_t bars = smem_u32(ctl);
    // barriers: 0 q_full, 1-2 kv_full, 3-4 kv_empty, 5 s_full, 6 s_empty, 7 p_full, 8 p_empty, 9 o_full
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ctl + 96);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid (heads, sequences, query tiles): the last query tiles see the most keys and are launched first
    const int head = blockIdx.x, seq = blockIdx.y, qb = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int kvh = head / (heads / kv_heads);
    const int q0 = qb * kQT;
    const int tok0 = seq * seq_len;
    const int last_q = min(q0 + kQT, seq_len) - 1;   // last valid query position of this CTA
    const int n_kt = last_q / kKT + 1;               // key tiles that hold keys <= last_q
    const int total = 2 * n_kt;                      // pass 1 then pass 2

    if (threadIdx.x == 0) *abort_flag = (status->code != 0) ? 1 : 0;
    __syncthreads();
    if (*abort_flag) return;
    if (threadIdx.x == 0) {
        mbar_init(bar(0), 1);
        mbar_init(bar(1), 1);
        mbar_init(bar(2), 1);
        mbar_init(bar(3), 1);
        mbar_init(bar(4), 1);
        mbar_init(bar(5), 1);
        mbar_init(bar(6), 4);  // one arrival per row warp
        mbar_init(bar(7), 4);
        mbar_init(bar(8), 1);
        mbar_init(bar(9), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kFwdTmemCols);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();  // nothing above reads or writes memory that an earlier kernel produces
    const uint32_t tS = tmem, tO = tmem + 128;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(0), kTileBytes);
            tma_load_2d(sQ, &tmQ, bar(0), head * 64, tok0 + q0);
            for (int it = 0; it < total; ++it) {
                const int s = it & 1, kt = it % n_kt;
                const bool second = it >= n_kt;
                if (!mbar_wait(bar(3 + s), ((it >> 1) & 1) ^ 1, abort_flag, status, 21)) break;
                mbar_arrive_expect_tx(bar(1 + s), second ? kStageBytes : kTileBytes);
                tma_load_2d(sKV + s * kStageBytes, &tmK, bar(1 + s), kvh * 64, tok0 + kt * kKT);
                if (second) tma_load_2d(sKV + s * kStageBytes + kTileBytes, &tmV, bar(1 + s), kvh * 64, tok0 + kt * kKT);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // fp32 accumulate, bf16 operands, M = 128; S: N = 128, both K-major; O: N = 64, B MN-major
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = mbar_wait(bar(0), 0, abort_flag, status, 22);
            for (int it = 0; ok && it < total; ++it) {
                const int s = it & 1;
                const bool second = it >= n_kt;
                if (!mbar_wait(bar(1 + s), (it >> 1) & 1, abort_flag, status, 23)) { ok = false; break; }
                if (!mbar_wait(bar(6), (it & 1) ^ 1, abort_flag, status, 24)) { ok = false; break; }  // S free
                tc_fence_after();
                const uint32_t kbase = sKV + s * kStageBytes;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tS, make_desc(sQ + kk * 32, 16, 1024), make_desc(kbase + kk * 32, 16, 1024), idesc_s, kk > 0);
                umma_commit(bar(5));
                if (!second) {
                    umma_commit(bar(3 + s));  // K consumed once the MMAs are done
                } else {
                    const int j = it - n_kt;
                    if (!mbar_wait(bar(7), j & 1, abort_flag, status, 25)) { ok = false; break; }  // P written
                    tc_fence_after();
                    const uint32_t vbase = kbase + kTileBytes;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        umma_bf16(tO, make_desc(sP + (kk >> 2) * kTileBytes + (kk & 3) * 32, 16, 1024),
                                  make_desc(vbase + kk * 2048, 8192, 1024), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(bar(3 + s));
                    umma_commit(bar(8));  // P may be overwritten
                }
            }
            if (ok) umma_commit(bar(9));
        }
        __syncwarp();
    } else {
        // ---- the 128 row threads ----
        const int quarter = warp & 3;                  // TMEM lanes this warp may access
        const int r = quarter * 32 + lane;             // row of the tile
        const int qpos = q0 + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m = -INFINITY, l = 0.0f, mc = 0.0f;
        bool ok = true;
        for (int it = 0; ok && it < total; ++it) {
            const int kt = it % n_kt;
            const bool second = it >= n_kt;
            const bool diag = (kt + 1) * kKT - 1 > q0;  // the tile holds keys after this CTA's first query
            // every wait of these warps is made warp-uniform: the TMEM loads below need the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait(bar(5), it & 1, abort_flag, status, 26))) { ok = false; break; }
            tc_fence_after();
            if (second) {
                const int j = it - n_kt;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(8), (j & 1) ^ 1, abort_flag, status, 27))) { ok = false; break; }  // P free
            }
            if (it == n_kt) mc = m * kScaleLog2e;
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t v[32];
                tmem_ld32(tS + lane_addr + cc * 32, v);
                tmem_ld_wait();
                const int k_first = kt * kKT + cc * 32;
                if (!second) {
                    if (diag) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) m = fmaxf(m, (k_first + c <= qpos) ? __uint_as_float(v[c]) : -INFINITY);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) m = fmaxf(m, __uint_as_float(v[c]));
                    }
                } else {
                    uint32_t pk[16];
                    if (diag) {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            const float p0 = (k_first + c <= qpos) ? ex2f(fmaf(__uint_as_float(v[c]), kScaleLog2e, -mc)) : 0.0f;
                            const float p1 = (k_first + c + 1 <= qpos) ? ex2f(fmaf(__uint_as_float(v[c + 1]), kScaleLog2e, -mc)) : 0.0f;
                            l += p0 + p1;
                            pk[c >> 1] = pack_bf16(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            const float p0 = ex2f(fmaf(__uint_as_float(v[c]), kScaleLog2e, -mc));
                            const float p1 = ex2f(fmaf(__uint_as_float(v[c + 1]), kScaleLog2e, -mc));
                            l += p0 + p1;
                            pk[c >> 1] = pack_bf16(p0, p1);
                        }
                    }
                    // 32 keys = 64 bytes = four 16-byte chunks of row r in atom cc / 2
                    const uint32_t row_base = sP + (cc >> 1) * kTileBytes + r * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t chunk = (uint32_t)((cc & 1) * 4 + q);
                        sts_v4(row_base + ((chunk ^ (r & 7)) << 4), make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]));
                    }
                }
            }
            tc_fence_before();
            if (second) fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(6));              // S has been read
                if (second) mbar_arrive(bar(7));  // this warp's rows of P are in shared memory
            }
        }
        if (ok && __all_sync(0xffffffffu, mbar_wait(bar(9), 0, abort_flag, status, 28))) {
            tc_fence_after();
            const float inv_l = 1.0f / l;
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32];
                tmem_ld32(tO + lane_addr + cc * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * inv_l);
                if (qpos < seq_len) store_row32(o, o_b, ((size_t)(tok0 + qpos) * heads + head) * 64 + cc * 32, v);
            }
            if (qpos < seq_len) lse_out[((size_t)seq * heads + head) * stat_stride + qpos] = mc + __log2f(l);
        }
        tc_fence_before();
    }
    __syncthreads();
    pause_after_abort(abort_flag);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kFwdTmemCols);
    }
}

// ---- backward ---------------------------------------------------------------------------------------------------
// delta[t, h] = sum_d dO * O (llama.rs:767-773 folds this into the softmax gradient) and the bf16 copy of dO.
// One warp per (token, head).
// Eight consecutive values as fp32.
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
// T = float: fp32 O and dO, writes the bf16 copy of dO; T = __nv_bfloat16: both already bf16, d_o_b unused.
// Eight threads per (token, head) row of 64 values, 8 values each.
template <typename T>
__global__ void attn_prep_kernel(const T *__restrict__ o, const T *__restrict__ d_o, float *__restrict__ delta,
                                 __nv_bfloat16 *__restrict__ d_o_b, size_t rows, int heads, int seq_len, int stat_stride) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t row = i >> 3;
    const int part = (int)(i & 7);
    float s = 0.0f;
    if (row < rows) {
        float a[8], g[8];
        load8(o + row * 64 + part * 8, a);
        load8(d_o + row * 64 + part * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += a[e] * g[e];
        if (d_o_b)
            *reinterpret_cast<uint4 *>(d_o_b + row * 64 + part * 8) =
                make_uint4(pack_bf16(g[0], g[1]), pack_bf16(g[2], g[3]), pack_bf16(g[4], g[5]), pack_bf16(g[6], g[7]));
    }
    // rows * 8 is a multiple of 8 and the block size a multiple of 32: the eight threads of a row share a warp
#pragma unroll
    for (int off = 4; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (row < rows && part == 0) {  // row = token * heads + head
        const size_t tok = row / heads, head = row % heads;
        delta[((tok / seq_len) * heads + head) * stat_stride + tok % seq_len] = s;
    }
}

// Sets the row-statistics arrays to their idle state: lse2 = +infinity (P = 0 at padded positions), delta = 0.
__global__ void attn_init_stats_kernel(float *__restrict__ lse, float *__restrict__ delta, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    lse[i] = INFINITY;
    if (delta) delta[i] = 0.0f;
}

// dK = scale * sum over the group's query heads of the per-head partial; dV = the plain sum.  Parts are added in
// head order, so the result does not depend on which CTA finished first.
__global__ void attn_dkv_finish_kernel(const float *__restrict__ dk_parts, const float *__restrict__ dv_parts,
                                       size_t part_stride, int parts, float *__restrict__ dkr, float *__restrict__ dv,
                                       __nv_bfloat16 *__restrict__ dv_b, size_t n4) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 a = reinterpret_cast<const float4 *>(dk_parts)[i], b = reinterpret_cast<const float4 *>(dv_parts)[i];
    for (int p = 1; p < parts; ++p) {
        const float4 x = reinterpret_cast<const float4 *>(dk_parts + (size_t)p * part_stride)[i];
        const float4 y = reinterpret_cast<const float4 *>(dv_parts + (size_t)p * part_stride)[i];
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
        b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    reinterpret_cast<float4 *>(dkr)[i] = make_float4(a.x * kScale, a.y * kScale, a.z * kScale, a.w * kScale);
    if (dv) reinterpret_cast<float4 *>(dv)[i] = b;
    if (dv_b) reinterpret_cast<uint2 *>(dv_b)[i] = make_uint2(pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
}

constexpr int kBT = 64;                               // the narrow side of a backward tile
constexpr uint32_t kHalfBytes = 64 * 128;             // a (64 rows, 64 bf16) tile
constexpr uint32_t kBwdTmemCols = 256;
constexpr uint32_t kCtlBytes = 128;
// M = 128, N = 64, bf16 operands, fp32 accumulator; B either K-major or MN-major
constexpr uint32_t kIdescN64 = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescN64BMn = kIdescN64 | (1u << 16);

// Writes 32 consecutive bf16 (given as 16 packed pairs) of row r of a (128 rows, 64 columns) K-major operand
// tile: columns 32*half .. 32*half + 31.
__device__ __forceinline__ void store_row_half(uint32_t tile, int r, int half, const uint32_t (&pk)[16]) {
    const uint32_t row_base = tile + r * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t chunk = (uint32_t)(half * 4 + q);
        sts_v4(row_base + ((chunk ^ (r & 7)) << 4), make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]));
    }
}

// dQ, one CTA per (128 query positions, head, sequence), 64-key tiles:
//   S = Q K^T, dP = dO V^T (TMEM) -> dS = P (dP - delta) / sqrt(d) as bf16 in shared memory -> dQ += dS K (TMEM).
constexpr uint32_t kDqTiles = 2 * kTileBytes + 2 * 2 * kHalfBytes + kTileBytes;
constexpr size_t kDqSmem = kDqTiles + kCtlBytes + 1024;

__global__ void __launch_bounds__(kFwdThreads)
attn_tc_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                  const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const float *__restrict__ lse, const float *__restrict__ delta, float *__restrict__ dqr, int stat_stride,
                  int seq_len, int heads, int kv_heads, DeviceStatus *status) {
    pdl_trigger();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmDO);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base, sDO = base + kTileBytes, sKV = sDO + kTileBytes, sDS = sKV + 4 * kHalfBytes;
    uint8_t *ctl = gen + kDqTiles;
    const uint32_t bars = smem_u32(ctl);
    // barriers: 0 q_full, 1-2 kv_full, 3-4 kv_empty, 5 sdp_full, 6 sdp_empty, 7 ds_full, 8 ds_empty, 9 dq_full
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ctl + 96);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.y;
    const int kvh = head / (heads / kv_heads);
    const int q0 = ((int)gridDim.z - 1 - (int)blockIdx.z) * kQT;  // the query tiles with the most keys first
    const int tok0 = seq * seq_len;
    const int last_q = min(q0 + kQT, seq_len) - 1;
    const int n_kt = last_q / kBT + 1;

    if (threadIdx.x == 0) *abort_flag = (status->code != 0) ? 1 : 0;
    __syncthreads();
    if (*abort_flag) return;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 10; ++i) mbar_init(bar(i), (i == 6 || i == 7) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kBwdTmemCols);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();  // nothing above reads or writes memory that an earlier kernel produces
    const uint32_t tS = tmem, tDP = tmem + 64, tDQ = tmem + 128;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(0), 2 * kTileBytes);
            tma_load_2d(sQ, &tmQ, bar(0), head * 64, tok0 + q0);
            tma_load_2d(sDO, &tmDO, bar(0), head * 64, tok0 + q0);
            for (int it = 0; it < n_kt; ++it) {
                const int s = it & 1;
                if (!mbar_wait(bar(3 + s), ((it >> 1) & 1) ^ 1, abort_flag, status, 31)) break;
                mbar_arrive_expect_tx(bar(1 + s), 2 * kHalfBytes);
                tma_load_2d(sKV + s * 2 * kHalfBytes, &tmK, bar(1 + s), kvh * 64, tok0 + it * kBT);
                tma_load_2d(sKV + s * 2 * kHalfBytes + kHalfBytes, &tmV, bar(1 + s), kvh * 64, tok0 + it * kBT);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(bar(0), 0, abort_flag, status, 32);
            for (int it = 0; ok && it < n_kt; ++it) {
                const int s = it & 1;
                if (!mbar_wait(bar(1 + s), (it >> 1) & 1, abort_flag, status, 33)) { ok = false; break; }
                if (!mbar_wait(bar(6), (it & 1) ^ 1, abort_flag, status, 34)) { ok = false; break; }  // S, dP free
                tc_fence_after();
                const uint32_t kb = sKV + s * 2 * kHalfBytes, vb = kb + kHalfBytes;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tS, make_desc(sQ + kk * 32, 16, 1024), make_desc(kb + kk * 32, 16, 1024), kIdescN64, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tDP, make_desc(sDO + kk * 32, 16, 1024), make_desc(vb + kk * 32, 16, 1024), kIdescN64, kk > 0);
                umma_commit(bar(5));
                if (!mbar_wait(bar(7), it & 1, abort_flag, status, 35)) { ok = false; break; }  // dS written
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tDQ, make_desc(sDS + kk * 32, 16, 1024), make_desc(kb + kk * 2048, 8192, 1024), kIdescN64BMn,
                              (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(3 + s));
                umma_commit(bar(8));
            }
            if (ok) umma_commit(bar(9));
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int qpos = q0 + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const bool row_on = qpos < seq_len;
        const size_t stat_at = ((size_t)seq * heads + head) * stat_stride + qpos;
        const float lse_r = row_on ? lse[stat_at] : INFINITY;  // +infinity: P = 0
        const float delta_r = row_on ? delta[stat_at] : 0.0f;
        bool ok = true;
        for (int it = 0; ok && it < n_kt; ++it) {
            const bool diag = (it + 1) * kBT - 1 > q0;  // the tile holds keys after this CTA's first query
            if (!__all_sync(0xffffffffu, mbar_wait(bar(5), it & 1, abort_flag, status, 36))) { ok = false; break; }
            tc_fence_after();
            if (!__all_sync(0xffffffffu, mbar_wait(bar(8), (it & 1) ^ 1, abort_flag, status, 37))) { ok = false; break; }
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32], w[32], pk[16];
                tmem_ld32(tS + lane_addr + cc * 32, v);
                tmem_ld32(tDP + lane_addr + cc * 32, w);
                tmem_ld_wait();
                const int k_first = it * kBT + cc * 32;
                // dS without the 1/sqrt(d) factor, which is applied once to dQ on the way out
                if (diag) {
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float p0 = (k_first + c <= qpos) ? ex2f(fmaf(__uint_as_float(v[c]), kScaleLog2e, -lse_r)) : 0.0f;
                        const float p1 = (k_first + c + 1 <= qpos) ? ex2f(fmaf(__uint_as_float(v[c + 1]), kScaleLog2e, -lse_r)) : 0.0f;
                        pk[c >> 1] = pack_bf16(p0 * (__uint_as_float(w[c]) - delta_r), p1 * (__uint_as_float(w[c + 1]) - delta_r));
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float p0 = ex2f(fmaf(__uint_as_float(v[c]), kScaleLog2e, -lse_r));
                        const float p1 = ex2f(fmaf(__uint_as_float(v[c + 1]), kScaleLog2e, -lse_r));
                        pk[c >> 1] = pack_bf16(p0 * (__uint_as_float(w[c]) - delta_r), p1 * (__uint_as_float(w[c + 1]) - delta_r));
                    }
                }
                store_row_half(sDS, r, cc, pk);
            }
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(6));
                mbar_arrive(bar(7));
            }
        }
        if (ok && __all_sync(0xffffffffu, mbar_wait(bar(9), 0, abort_flag, status, 38))) {
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32];
                tmem_ld32(tDQ + lane_addr + cc * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * kScale);
                if (row_on) store_row32(dqr, nullptr, ((size_t)(tok0 + qpos) * heads + head) * 64 + cc * 32, v);
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    pause_after_abort(abort_flag);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kBwdTmemCols);
    }
}

// dK and dV, one CTA per (128 key positions, query head, sequence).  The CTA walks over the 64-query tiles at or
// after its keys, working on the transposed products so that the key index is the TMEM lane:
//   S^T = K Q^T, dP^T = V dO^T (TMEM)  ->  P^T and dS^T as bf16 in shared memory  ->  dV += P^T dO, dK += dS^T Q,
// both accumulated in TMEM over all query tiles.  lse2 and delta of the 64 queries arrive in shared memory as
// two 256-byte bulk copies next to the Q / dO tiles.  The result is this head's partial of its key/value head's
// gradient (fp32, without the 1/sqrt(d) factor on dK); attn_dkv_finish_kernel adds the group's partials.
constexpr uint32_t kDkvTiles = 2 * kTileBytes + 2 * 2 * kHalfBytes + 2 * kTileBytes;
constexpr uint32_t kStatBytes = 2 * 64 * 4;  // lse2 and delta of one query tile
constexpr size_t kDkvSmem = kDkvTiles + kCtlBytes + 2 * kStatBytes + 1024;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__global__ void __launch_bounds__(kFwdThreads)
attn_tc_dkdv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                    const float *__restrict__ lse, const float *__restrict__ delta, float *__restrict__ dk_parts,
                    float *__restrict__ dv_parts, size_t part_stride, int stat_stride, int seq_len, int heads, int kv_heads,
                    DeviceStatus *status) {
    pdl_trigger();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmDO);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sK = base, sV = base + kTileBytes, sQD = sV + kTileBytes, sPT = sQD + 4 * kHalfBytes,
                   sDST = sPT + kTileBytes;
    uint8_t *ctl = gen + kDkvTiles;
    const uint32_t bars = smem_u32(ctl);
    // barriers: 0 kv_full, 1-2 qdo_full, 3-4 qdo_empty, 5 st_full, 6 st_empty, 7 pds_full, 8 pds_empty, 9 acc_full
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ctl + 96);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const float4 *stats = reinterpret_cast<const float4 *>(ctl + kCtlBytes);  // [stage][lse2 x 64 | delta x 64]
    const uint32_t s_stats = bars + kCtlBytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.y;
    const int n_rep = heads / kv_heads;
    const int kvh = head / n_rep;
    const int k0 = blockIdx.z * kKT;                     // the first key tiles have the most queries: launched first
    const int tok0 = seq * seq_len;
    const int qt_first = k0 / kBT;                       // queries before the first key see none of these keys
    const int total = (seq_len + kBT - 1) / kBT - qt_first;
    const float *lse_row = lse + ((size_t)seq * heads + head) * stat_stride;
    const float *delta_row = delta + ((size_t)seq * heads + head) * stat_stride;

    if (threadIdx.x == 0) *abort_flag = (status->code != 0) ? 1 : 0;
    __syncthreads();
    if (*abort_flag) return;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 10; ++i) mbar_init(bar(i), (i == 6 || i == 7) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kBwdTmemCols);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();  // nothing above reads or writes memory that an earlier kernel produces
    const uint32_t tST = tmem, tDPT = tmem + 64, tDV = tmem + 128, tDK = tmem + 192;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(0), 2 * kTileBytes);
            tma_load_2d(sK, &tmK, bar(0), kvh * 64, tok0 + k0);
            tma_load_2d(sV, &tmV, bar(0), kvh * 64, tok0 + k0);
            for (int it = 0; it < total; ++it) {
                const int s = it & 1;
                const int qt = qt_first + it;
                if (!mbar_wait(bar(3 + s), ((it >> 1) & 1) ^ 1, abort_flag, status, 41)) break;
                mbar_arrive_expect_tx(bar(1 + s), 2 * kHalfBytes + kStatBytes);
                tma_load_2d(sQD + s * 2 * kHalfBytes, &tmQ, bar(1 + s), head * 64, tok0 + qt * kBT);
                tma_load_2d(sQD + s * 2 * kHalfBytes + kHalfBytes, &tmDO, bar(1 + s), head * 64, tok0 + qt * kBT);
                bulk_load(s_stats + s * kStatBytes, lse_row + qt * kBT, 256, bar(1 + s));
                bulk_load(s_stats + s * kStatBytes + 256, delta_row + qt * kBT, 256, bar(1 + s));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(bar(0), 0, abort_flag, status, 42);
            for (int it = 0; ok && it < total; ++it) {
                const int s = it & 1;
                if (!mbar_wait(bar(1 + s), (it >> 1) & 1, abort_flag, status, 43)) { ok = false; break; }
                if (!mbar_wait(bar(6), (it & 1) ^ 1, abort_flag, status, 44)) { ok = false; break; }  // S^T, dP^T free
                tc_fence_after();
                const uint32_t qb = sQD + s * 2 * kHalfBytes, dob = qb + kHalfBytes;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tST, make_desc(sK + kk * 32, 16, 1024), make_desc(qb + kk * 32, 16, 1024), kIdescN64, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tDPT, make_desc(sV + kk * 32, 16, 1024), make_desc(dob + kk * 32, 16, 1024), kIdescN64, kk > 0);
                umma_commit(bar(5));
                if (!mbar_wait(bar(7), it & 1, abort_flag, status, 45)) { ok = false; break; }  // P^T, dS^T written
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tDV, make_desc(sPT + kk * 32, 16, 1024), make_desc(dob + kk * 2048, 8192, 1024), kIdescN64BMn,
                              (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tDK, make_desc(sDST + kk * 32, 16, 1024), make_desc(qb + kk * 2048, 8192, 1024), kIdescN64BMn,
                              (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(3 + s));  // also releases the stage's statistics: the row threads are done with them
                umma_commit(bar(8));
            }
            if (ok) umma_commit(bar(9));
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int kpos = k0 + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        for (int it = 0; ok && it < total; ++it) {
            const int s = it & 1;
            const int q_first = (qt_first + it) * kBT;
            const bool diag = q_first < k0 + kKT - 1;  // the tile holds queries before this CTA's last key
            // the statistics of this stage arrive with its Q / dO tiles
            if (!__all_sync(0xffffffffu, mbar_wait(bar(1 + s), (it >> 1) & 1, abort_flag, status, 49))) { ok = false; break; }
            if (!__all_sync(0xffffffffu, mbar_wait(bar(5), it & 1, abort_flag, status, 46))) { ok = false; break; }
            tc_fence_after();
            if (!__all_sync(0xffffffffu, mbar_wait(bar(8), (it & 1) ^ 1, abort_flag, status, 47))) { ok = false; break; }
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32], w[32], pp[16], pd[16];
                tmem_ld32(tST + lane_addr + cc * 32, v);
                tmem_ld32(tDPT + lane_addr + cc * 32, w);
                tmem_ld_wait();
                const float4 *sl = stats + s * (kStatBytes / 16) + cc * 8;  // lse2 of queries 32cc ..; delta 16 float4 on
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 lq = sl[c >> 2], dq = sl[16 + (c >> 2)];
                    const float lqa[4] = {lq.x, lq.y, lq.z, lq.w}, dqa[4] = {dq.x, dq.y, dq.z, dq.w};
                    float p[4], ds[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        p[e] = ex2f(fmaf(__uint_as_float(v[c + e]), kScaleLog2e, -lqa[e]));
                        if (diag) p[e] = (kpos <= q_first + cc * 32 + c + e) ? p[e] : 0.0f;
                        ds[e] = p[e] * (__uint_as_float(w[c + e]) - dqa[e]);
                    }
                    pp[c >> 1] = pack_bf16(p[0], p[1]);
                    pp[(c >> 1) + 1] = pack_bf16(p[2], p[3]);
                    pd[c >> 1] = pack_bf16(ds[0], ds[1]);
                    pd[(c >> 1) + 1] = pack_bf16(ds[2], ds[3]);
                }
                store_row_half(sPT, r, cc, pp);
                store_row_half(sDST, r, cc, pd);
            }
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(6));
                mbar_arrive(bar(7));
            }
        }
        if (ok && __all_sync(0xffffffffu, mbar_wait(bar(9), 0, abort_flag, status, 48))) {
            tc_fence_after();
            const size_t kv_dim = (size_t)kv_heads * 64;
            const size_t part = (size_t)(head % n_rep) * part_stride;
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t v[32];
                tmem_ld32(tDV + lane_addr + cc * 32, v);  // columns 0-63: dV, 64-127: dK
                tmem_ld_wait();
                if (kpos < seq_len)
                    store_row32((cc < 2 ? dv_parts : dk_parts) + part, nullptr,
                                (size_t)(tok0 + kpos) * kv_dim + kvh * 64 + (cc & 1) * 32, v);
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    pause_after_abort(abort_flag);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kBwdTmemCols);
    }
}

}  // namespace

// Position stride of the row-statistics arrays (lse2, delta) for sequences of seq_len positions.
size_t attention_tc_stat_stride(size_t seq_len) { return (seq_len + 63) / 64 * 64; }

// Puts freshly allocated statistics arrays (n_seq * heads * stride floats each; delta may be null) into the state
// the kernels expect between calls: lse2 = +infinity, delta = 0.  Needed once per allocation, since the kernels
// only ever write the positions below seq_len.
int attention_tc_init_stats(qlc_ctx *ctx, float *lse, float *delta, size_t n_seq, size_t seq_len, size_t heads) {
    const size_t n = n_seq * heads * attention_tc_stat_stride(seq_len);
    if (!n) return QLC_OK;
    QLC_CUDA(launch_pdl(attn_init_stats_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream, lse, delta, n));
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// Forward: bf16 q (tokens, heads*64), k, v (tokens, kv_heads*64) -> the attention output in `o` (fp32) and / or
// `o_b` (bf16), either may be null, and lse2 in the statistics layout.
int attention_tc_forward(qlc_ctx *ctx, const __nv_bfloat16 *qr, const __nv_bfloat16 *kr, const __nv_bfloat16 *v, float *o,
                         __nv_bfloat16 *o_b, float *lse, size_t n_seq, size_t seq_len, size_t heads, size_t kv_heads) {
    const size_t T = n_seq * seq_len;
    alignas(64) CUtensorMap tQ, tK, tV;
    QLC_TRY(make_map_bf16(&tQ, qr, T, heads * 64, 128));
    QLC_TRY(make_map_bf16(&tK, kr, T, kv_heads * 64, 128));
    QLC_TRY(make_map_bf16(&tV, v, T, kv_heads * 64, 128));
    QLC_CUDA(cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem));
    const dim3 grid((unsigned)heads, (unsigned)n_seq, (unsigned)((seq_len + kQT - 1) / kQT));
    QLC_CUDA(launch_pdl(attn_tc_fwd_kernel, grid, dim3(kFwdThreads), kFwdSmem, ctx->stream, tQ, tK, tV, o, o_b, lse,
                        (int)attention_tc_stat_stride(seq_len), (int)seq_len, (int)heads, (int)kv_heads, ctx->d_status));
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// Gradients of the rotated q, k and of v from dO: delta (and the bf16 copy of dO) first, then the dQ kernel, the
// dK/dV kernel and the sum of its per-head partials.  All pointers are device memory; dqr (tokens, heads*64) and
// dkr (tokens, kv_heads*64) are fp32, dV goes to `dv` (fp32) and / or `dv_b` (bf16).  O and dO come either as fp32
// (`o`, `d_o`; `d_o_b` receives the bf16 copy of dO) or, when `o` is null, as bf16 (`o_b`, `d_o_b`).  lse and
// delta are statistics arrays (attention_tc_init_stats); dk_parts and dv_parts are scratch of
// (heads / kv_heads) * tokens * kv_heads * 64 floats each.  With `dq_ctx` (a second context on the same device, and
// two events to fork and join with) the dQ kernel runs on that context's stream beside the dK/dV kernel.  With a
// null `dkr` the per-head partials are left in dk_parts / dv_parts ([head of the group][token][kv_heads * 64],
// dK without the 1/sqrt(64) factor) for the caller to sum.
int attention_tc_backward(qlc_ctx *ctx, const __nv_bfloat16 *qr, const __nv_bfloat16 *kr, const __nv_bfloat16 *v,
                          const float *o, const float *d_o, const __nv_bfloat16 *o_b, __nv_bfloat16 *d_o_b, const float *lse,
                          float *delta, float *dqr, float *dkr, float *dv, __nv_bfloat16 *dv_b, float *dk_parts, float *dv_parts,
                          size_t n_seq, size_t seq_len, size_t heads, size_t kv_heads, qlc_ctx *dq_ctx, cudaEvent_t ev_fork,
                          cudaEvent_t ev_join) {
    const size_t T = n_seq * seq_len;
    const size_t rows = T * heads;
    const int stride = (int)attention_tc_stat_stride(seq_len);
    const dim3 prep_grid((unsigned)((rows * 8 + 255) / 256));
    if (o)
        QLC_CUDA(launch_pdl(attn_prep_kernel<float>, prep_grid, dim3(256), 0, ctx->stream, o, d_o, delta, d_o_b, rows, (int)heads,
                            (int)seq_len, stride));
    else
        QLC_CUDA(launch_pdl(attn_prep_kernel<__nv_bfloat16>, prep_grid, dim3(256), 0, ctx->stream, o_b,
                            (const __nv_bfloat16 *)d_o_b, delta, (__nv_bfloat16 *)nullptr, rows, (int)heads, (int)seq_len, stride));
    QLC_CUDA(cudaGetLastError());
    alignas(64) CUtensorMap tQ128, tDO128, tK64, tV64, tK128, tV128, tQ64, tDO64;
    QLC_TRY(make_map_bf16(&tQ128, qr, T, heads * 64, 128));
    QLC_TRY(make_map_bf16(&tDO128, d_o_b, T, heads * 64, 128));
    QLC_TRY(make_map_bf16(&tK64, kr, T, kv_heads * 64, 64));
    QLC_TRY(make_map_bf16(&tV64, v, T, kv_heads * 64, 64));
    QLC_TRY(make_map_bf16(&tK128, kr, T, kv_heads * 64, 128));
    QLC_TRY(make_map_bf16(&tV128, v, T, kv_heads * 64, 128));
    QLC_TRY(make_map_bf16(&tQ64, qr, T, heads * 64, 64));
    QLC_TRY(make_map_bf16(&tDO64, d_o_b, T, heads * 64, 64));
    QLC_CUDA(cudaFuncSetAttribute(attn_tc_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem));
    QLC_CUDA(cudaFuncSetAttribute(attn_tc_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDkvSmem));
    const dim3 grid((unsigned)heads, (unsigned)n_seq, (unsigned)((seq_len + kQT - 1) / kQT));
    // dQ and dK/dV only share their inputs: with a second context the dQ kernel runs beside the dK/dV kernel
    qlc_ctx *qc = dq_ctx ? dq_ctx : ctx;
    if (dq_ctx) {
        QLC_CUDA(cudaEventRecord(ev_fork, ctx->stream));
        QLC_CUDA(cudaStreamWaitEvent(dq_ctx->stream, ev_fork, 0));
    }
    QLC_CUDA(launch_pdl(attn_tc_dq_kernel, grid, dim3(kFwdThreads), kDqSmem, qc->stream, tQ128, tDO128, tK64, tV64, lse,
                        (const float *)delta, dqr, stride, (int)seq_len, (int)heads, (int)kv_heads, qc->d_status));
    QLC_CUDA(cudaGetLastError());
    if (dq_ctx) QLC_CUDA(cudaEventRecord(ev_join, dq_ctx->stream));
    const size_t part_stride = T * kv_heads * 64;
    QLC_CUDA(launch_pdl(attn_tc_dkdv_kernel, grid, dim3(kFwdThreads), kDkvSmem, ctx->stream, tK128, tV128, tQ64, tDO64, lse,
                        (const float *)delta, dk_parts, dv_parts, part_stride, stride, (int)seq_len, (int)heads, (int)kv_heads,
                        ctx->d_status));
    QLC_CUDA(cudaGetLastError());
    // without dkr the caller sums the per-head partials itself (scaling dK by 1/sqrt(64)), fused with what follows
    if (dkr) {
        QLC_CUDA(launch_pdl(attn_dkv_finish_kernel, dim3((unsigned)((part_stride / 4 + 255) / 256)), dim3(256), 0, ctx->stream,
                            (const float *)dk_parts, (const float *)dv_parts, part_stride, (int)(heads / kv_heads), dkr, dv, dv_b,
                            part_stride / 4));
        QLC_CUDA(cudaGetLastError());
    }
    if (dq_ctx) QLC_CUDA(cudaStreamWaitEvent(ctx->stream, ev_join, 0));
    ctx->launches += 4;
    return QLC_OK;
}

}  // namespace qlc
