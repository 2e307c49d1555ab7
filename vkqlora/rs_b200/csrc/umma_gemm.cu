// Tensor-core path of QloraLinear for sm_100a: tcgen05.mma with TMEM accumulators, TMA-staged
// activation tiles, and the NF4 + double-quant weight tile produced *inside* the kernel.
//
//   forward   Y  = X·deq(Wq)^T + [s·X·A^T]·B^T        (qlora-core/src/qlora.rs:86-107)
//   backward  dX = dY·deq(Wq)  + [s·dY·B]·A            (qlora.rs:135,149,153-156)
//             dB = dY^T·[s·X·A^T]                      (qlora.rs:147)
//             dA = [s·dY·B]^T·X                        (qlora.rs:151)
//
// One kernel template (`umma_gemm_kernel`) covers all six products:
//   * main GEMMs: a CTA owns a 256(rows) x 256(cols) output tile as two 128x256 fp32 accumulators
//     in tensor memory (all 512 columns).  Per 64-deep k-step the activation tile (256x64 bf16)
//     arrives by TMA with the 128-byte swizzle, while sixteen producer warps read the packed
//     nibbles (one 128-bit load per thread) and the 8-bit absmax code of their 64-element
//     quantisation block, decode to bf16 with byte permutes (nf4_decode.cuh) and store the
//     256x64 weight tile straight into the swizzled shared-memory layout the MMA descriptor
//     expects.  The dequantised weight never exists in HBM, and one decoded tile feeds both
//     accumulators.  Forward consumes W K-major ([n][k], quant block along k); backward consumes
//     the same bytes MN-major ([n][k] with k as the output dimension).
//   * the LoRA term is a k-extension: after the last weight k-step the loop runs r_pad/64 more
//     steps whose operands are the small bf16 matrices [s·X·A^T] / B (forward) or [s·dY·B] / A
//     (backward), fetched by TMA, so the rank-r update lands in the same accumulators.
//   * the four skinny products (X·A^T, dY·B, dY^T·T1, Ds^T·X) are the same kernel with both
//     operands from TMA, N = 64, and (for the token-contracted gradients) a split over tokens
//     whose fp32 partials are summed in a fixed order by a small reduce kernel (deterministic).
//
// Warp roles: warp 0 = TMA issue, warp 1 = TMEM owner + MMA issue (one elected thread), the other
// warps are weight-tile producers during the main loop (16 warps, two threads per quantisation block)
// and run the epilogue afterwards (tcgen05.ld, scale, convert, store).  Stages are handed over with mbarriers; every wait is
// bounded: on expiry the kernel raises a status word, unwinds, frees its tensor memory and
// returns, so a logic error can never leave the device spinning.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <map>
#include <new>

#include "common.cuh"
#include "nf4_decode.cuh"
#include "ptx.cuh"

namespace qlc {
namespace {

constexpr int kBM = 128;         // rows per accumulator (UMMA M)
constexpr int kBK = 64;          // contraction elements per stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;       // contraction per tcgen05.mma (bf16)
// Worker warps: with the dequant producer, 16 warps (512 threads, two per 64-element quantisation block)
// build the weight tile of every k-step and then run the epilogue; the TMA-only kernels keep 8 warps,
// which only run the epilogue.
template <bool B_DEQUANT> constexpr int kWorkerWarps = B_DEQUANT ? 16 : 8;
template <bool B_DEQUANT> constexpr int kBlockThreads = 32 * (2 + kWorkerWarps<B_DEQUANT>);
constexpr int kRankPad = 64;     // LoRA rank is zero-padded to a multiple of this
constexpr int kMaxRank = 256;    // ranks the tensor-core path takes (rank-padded products in slices of 64 columns)

__constant__ float c_levels[16] = {
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

struct GemmArgs {
    // weight payload for the in-kernel dequant producer
    const uint8_t *codes;
    const uint8_t *absmax_codes;
    const float *absmax2;
    const float *scales_f32;
    uint32_t blk_shift;  // log2 of the quantisation block size (32, 64, 128 or 256 elements)
    int dq;
    uint32_t w_rows;  // out_dim
    uint32_t w_cols;  // in_dim
    // problem
    uint32_t M;          // output rows
    uint32_t N;          // output columns
    uint32_t k_steps;    // main-loop steps over the whole contraction (contraction / 64)
    uint32_t ext_steps;  // LoRA extension steps appended after the main loop (split 0 only)
    uint32_t splits;     // gridDim.z; the main steps are divided evenly among splits
    uint32_t a_rows;     // output rows per CTA that are real (ACC*128, or 64 for the memory-bound skinny products)
    // output: row-major, `ldo` elements per row; split z writes at out + z * M * ldo
    void *out;
    uint32_t ldo;
    int out_bf16;
    float out_scale;
    uint32_t out_pad_cols;  // bf16 output only: columns [N, out_pad_cols) of each row are written as zeros
    // Two independent products in one launch (TMA-fed kernels only): CTAs with blockIdx.x == 1 work on the
    // second problem, whose operands come through the two `ext` tensor maps.
    int pair;
    uint32_t M2;        // output rows of the second problem
    uint32_t k_steps2;  // its contraction steps
    void *out2;         // its output (same ldo, dtype, scale and padding as the first)
    // Token-split products: when `counters` is set, the last CTA of an output tile to finish adds the split
    // partials (out / out2 hold them) in split order and writes final / final2.
    int *counters;      // one zeroed int per (problem, row tile); the last CTA resets its counter
    float *final1, *final2;
    int transposed1, transposed2;  // final is (cols_used, M) row-major instead of (M, cols_used)
    uint32_t cols_used;
    uint32_t final_ld;  // row pitch of a non-transposed final (0: cols_used), for a column slice of a wider matrix
    int accumulate;     // final += sum instead of final = sum
    // Paired-CTA weight GEMM: work items in launch order.  Items [0, full_items) are whole output tiles;
    // the tiles of the last, partial wave follow, each cut into k_chunks pieces along the contraction so
    // that the wave is short and full.  Pieces leave fp32 partials in split_ws; the last CTA of a tile
    // to finish adds them in chunk order.
    uint32_t row_tiles;   // 512-row tiles of the output
    uint32_t col_tiles;   // 256-column tiles; tile t covers column tile t % col_tiles of row tile t / col_tiles
    int row_fastest;      // diagnostics: the other order (row tile t % row_tiles, column tile t / row_tiles)
    uint32_t full_items;
    uint32_t k_chunks;    // 1: no tile is cut
    float *split_ws;      // [cut tile][chunk][CTA of the pair][2][128][256] fp32
    DeviceStatus *status;
    long long *timing;  // optional per-CTA clock64 stamps (diagnostics; null in normal operation)
};

// ---- PTX wrappers specific to this file (the shared ones are in ptx.cuh) ---------------------------
// Same as umma_bf16 with fp32 operands read as tf32 (8 contraction elements = 32 bytes per instruction).
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// fp32 -> tf32 (10 mantissa bits), round to nearest, ties away from zero.
__device__ __forceinline__ uint32_t tf32_rna(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return u;
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---- the kernel ---------------------------------------------------------------------------------
// Shared-memory tile layouts (all with the 128-byte swizzle: 16-byte chunk c of 128-byte row r is
// stored at chunk c ^ (r & 7); tiles are 1024-byte aligned):
//   K-major operand  (rows = M/N index, 64 contraction elements per row):
//       row r at byte r*128.  Descriptor: SBO = 1024 (8-row groups); +32 bytes per UMMA_K.
//   MN-major operand (rows = contraction index, 64 M/N elements per row, 64-element atoms):
//       atom g (M/N elements 64g..64g+63), contraction row t at byte g*8192 + t*128.
//       Descriptor: LBO = 8192 (next atom), SBO = 1024 (next 8 contraction rows); +2048 per UMMA_K.
// TF32: operands are fp32 in memory and read by the tensor core as tf32.  The byte geometry of a stage
// does not change (128-byte rows, 32 bytes per MMA along the contraction); a k-step then covers 32
// contraction elements, and an MN-major atom 32 elements.
template <int BN, int ACC, bool A_MN, bool B_MN, bool B_DEQUANT, int STAGES, int NI = 1, bool TF32 = false>
__global__ void __launch_bounds__(kBlockThreads<B_DEQUANT>, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmAext, const __grid_constant__ CUtensorMap tmBext,
                 const GemmArgs args) {
    constexpr int kStepElems = TF32 ? 32 : 64;      // contraction elements per k-step (one 128-byte row)
    constexpr int kAtomElems = TF32 ? 32 : 64;      // M/N elements per MN-major atom
    constexpr uint32_t kAtomBytes = kStepElems * 128;  // one MN-major atom of a stage
    constexpr uint32_t kMnStep = TF32 ? 1024 : 2048;    // MN-major operand: bytes per MMA along the contraction
    static_assert(!TF32 || (ACC == 1 && !B_DEQUANT), "tf32: TMA-fed operands, one accumulator");
    constexpr uint32_t kABytes = ACC * kBM * kBK * 2;  // per stage
    constexpr uint32_t kBBytes = BN * kBK * 2;
    constexpr uint32_t kStageBytes = kABytes + kBBytes;
    // NI > 1 (memory-bound skinny products): NI warps issue the MMAs of alternate k-steps into private
    // accumulators that the epilogue adds up in fixed order.  One thread needs several hundred cycles to issue
    // a k-step's four MMAs and their commit, far longer than the tensor core works on them; several issuers
    // overlap that latency, which otherwise caps the rate at which a CTA can consume its TMA stream.
    constexpr uint32_t kTmemCols = ACC * BN * NI < 32 ? 32 : ACC * BN * NI;  // 32..512, power of two
    static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
    static_assert(NI == 1 || (ACC == 1 && !B_DEQUANT && NI <= 4), "several issuers: single tile, TMA-fed operands");
    // Each stage must always be consumed by the same issuer.  A parity wait only tells the current phase from
    // the one before it: an issuer that met a stage for the first time in the stage's second round could find
    // the barrier still in its first phase, take that for "complete", and read a tile that has not landed.
    static_assert(STAGES % NI == 0, "a stage belongs to one issuer");
    static_assert((BN % 64 == 0 || BN == 16 || BN == 32) && BN <= 256, "BN");
    static_assert(BN >= 64 || (ACC == 1 && !B_MN && !B_DEQUANT), "narrow tiles: single accumulator, K-major TMA operand");
    static_assert(!B_DEQUANT || BN == 256, "the producer mapping assumes a 256-column weight tile");

    pdl_trigger();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        prefetch_tmap(&tmAext);
        prefetch_tmap(&tmBext);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + STAGES * kStageBytes;
    // barrier block: full[STAGES], empty[STAGES], tmem_full, then the TMEM base slot and abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * STAGES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + STAGES * kStageBytes + 8 * (2 * STAGES + 1));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // diagnostics: slot k of this CTA's 16 stamps
    long long *const tstamp = args.timing
        ? args.timing + 16 * (size_t)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) : nullptr;
    const bool second = !B_DEQUANT && args.pair && blockIdx.x == 1;  // this CTA works on the second problem
    const uint32_t n0 = (!B_DEQUANT && args.pair) ? 0u : blockIdx.x * BN;  // first output column of this CTA
    const uint32_t m0 = blockIdx.y * args.a_rows;     // first output row
    const uint32_t z = blockIdx.z;
    const uint32_t Mrows = second ? args.M2 : args.M;
    void *const outp = second ? args.out2 : args.out;
    if (m0 >= Mrows) return;  // the two problems of a pair may differ in height (whole CTA leaves)
    const uint32_t steps_per_split = (second ? args.k_steps2 : args.k_steps) / args.splits;
    const uint32_t step_begin = z * steps_per_split;
    const uint32_t main_steps = steps_per_split;
    const uint32_t total_steps = main_steps + (z == 0 ? args.ext_steps : 0u);
    const uint32_t active_issuers = total_steps == 0 ? 1u : (total_steps < (uint32_t)NI ? total_steps : (uint32_t)NI);

    // If an earlier launch on this context already raised a status, do nothing (CTA-uniform test).
    if (threadIdx.x == 0) *abort_flag = (args.status->code != 0) ? 1 : 0;
    __syncthreads();
    if (*abort_flag) return;

    if (tstamp && threadIdx.x == 0) tstamp[0] = clock64();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1 + (B_DEQUANT ? kWorkerWarps<true> : 0));
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, active_issuers);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // everything above touched no memory an earlier kernel writes (the status word is only ever raised)
    if (tstamp && threadIdx.x == 0) tstamp[1] = clock64();

    if (warp == 0) {
        // ---------------- TMA issue ----------------
        if (lane == 0) {
            for (uint32_t it = 0; it < total_steps; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 1)) break;
                const bool ext = it >= main_steps;
                const uint32_t a_dst = smem_base + s * kStageBytes;
                const uint32_t b_dst = a_dst + kABytes;
                const bool b_by_tma = !B_DEQUANT || ext;
                // (a_rows < 128: only the first a_rows rows of the tile are loaded; the rest of the 128-row MMA
                //  operand is stale shared memory whose accumulator rows are never stored)
                const uint32_t a_bytes = (!A_MN || ext) ? args.a_rows * 128u : kABytes;
                mbar_arrive_expect_tx(full_bar(s), a_bytes + (b_by_tma ? kBBytes : 0u));
                const int kc = ext ? (int)((it - main_steps) * kStepElems) : (int)((step_begin + it) * kStepElems);
                const CUtensorMap *ma = (ext || second) ? &tmAext : &tmA;
                const CUtensorMap *mb = (ext || second) ? &tmBext : &tmB;
                if (!A_MN || ext) {
                    // K-major A: (ACC*128) rows x one 128-byte row of contraction elements, boxes of 128 rows
#pragma unroll
                    for (int a = 0; a < ACC; ++a)
                        tma_load_2d(a_dst + a * (kBM * 128), ma, full_bar(s), kc, (int)(m0 + a * kBM));
                } else {
                    // MN-major A: contraction rows x (ACC*128) elements, one box per atom
#pragma unroll
                    for (int g = 0; g < ACC * kBM / kAtomElems; ++g)
                        tma_load_2d(a_dst + g * kAtomBytes, ma, full_bar(s), (int)(m0 + g * kAtomElems), kc);
                }
                if (b_by_tma) {
                    if (!B_MN) {
                        tma_load_2d(b_dst, mb, full_bar(s), kc, (int)n0);
                    } else {
#pragma unroll
                        for (int g = 0; g < BN / kAtomElems; ++g)
                            tma_load_2d(b_dst + g * kAtomBytes, mb, full_bar(s), (int)(n0 + g * kAtomElems), kc);
                    }
                }
            }
        }
        __syncwarp();  // the whole warp reaches the closing barrier together
    } else if (warp <= NI) {
        // ---------------- MMA issue (issuer j = warp - 1 takes k-steps j, j + NI, ...) ----------------
        const uint32_t issuer = (uint32_t)warp - 1u;
        if (lane == 0 && (issuer < active_issuers || total_steps == 0)) {
            constexpr uint32_t kFmt = TF32 ? 2u : 1u;  // operand format: bf16 = 1, tf32 = 2; accumulator fp32 = 1
            constexpr uint32_t idesc_main = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((A_MN ? 1u : 0u) << 15) |
                                            ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                            ((uint32_t)(kBM >> 4) << 24);
            // extension steps always use a K-major A operand
            constexpr uint32_t idesc_ext = idesc_main & ~(1u << 15);
            bool ok = true;
            long long mma_wait = 0;
            for (uint32_t it = issuer; it < total_steps; it += NI) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                const long long tw = tstamp ? clock64() : 0;
                if (!mbar_wait(full_bar(s), ph, abort_flag, args.status, 2)) {
                    ok = false;
                    break;
                }
                if (tstamp) {
                    mma_wait += clock64() - tw;
                    if (it == 0) tstamp[2] = clock64();
                }
                tc_fence_after();
                const bool ext = it >= main_steps;
                const bool a_mn = A_MN && !ext;
                const uint32_t a_src = smem_base + s * kStageBytes;
                const uint32_t b_src = a_src + kABytes;
#pragma unroll
                for (int a = 0; a < ACC; ++a) {
#pragma unroll
                    for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                        // MN-major operands: 16-bit elements use the 16-byte-chunk swizzle whose pattern repeats every
                        // 8 contraction rows (SBO = 8 rows); 32-bit elements must use the 32-byte-chunk swizzle, whose
                        // pattern repeats every 4 rows (SBO = 4 rows).
                        constexpr uint32_t kMnLayout = TF32 ? 1u : 2u, kMnSbo = TF32 ? 512u : 1024u;
                        const uint64_t da = a_mn ? make_desc(a_src + a * 16384 + kk * kMnStep, kAtomBytes, kMnSbo, kMnLayout)
                                                 : make_desc(a_src + a * (kBM * 128) + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_desc(b_src + kk * kMnStep, kAtomBytes, kMnSbo, kMnLayout)
                                                 : make_desc(b_src + kk * 32, 16, 1024);
                        if (TF32)
                            umma_tf32(tmem_base + (a + issuer) * BN, da, db, ext ? idesc_ext : idesc_main,
                                      (it != issuer || kk > 0) ? 1u : 0u);
                        else
                            umma_bf16(tmem_base + (a + issuer) * BN, da, db, ext ? idesc_ext : idesc_main,
                                      (it != issuer || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit(empty_bar(s));
            }
            if (ok) umma_commit(tmem_full_bar);
            if (tstamp && issuer == 0) {
                tstamp[3] = clock64();  // all MMAs issued
                tstamp[4] = mma_wait;   // cycles the MMA thread spent waiting for full stages
            }
        }
        __syncwarp();
    }
    if (warp >= 2) {
        // ---------------- weight-tile producers, then epilogue ----------------
        if (B_DEQUANT) {
            // 512 producer threads build the 256x64 (or 64x256) weight tile of every k-step: two threads per
            // 64-element quantisation block, 32 elements (one 128-bit load of nibbles) each.  The lane ->
            // (row, half) mapping makes every quarter-warp write 4 rows x 2 halves, i.e. 8 different 16-byte
            // slots of the 128-byte swizzle pattern, so the 128-bit stores are bank-conflict free, and the two
            // lanes of a pair read adjacent 16 bytes of the same 32-byte sector.
            const int pt = threadIdx.x - 64;  // 0..511
            const int hf = pt & 1;            // which half of the quantisation block
            uint32_t wrow, wcol, dst_off, r8;
            bool valid;
            if (!B_MN) {
                // forward: tile rows = output features n0..n0+255, block along the contraction
                const int rl = pt >> 1;
                wrow = n0 + rl;
                wcol = 0;  // + k0 per step
                r8 = rl & 7;
                dst_off = rl * 128;
                valid = wrow < args.w_rows;
            } else {
                // backward: tile rows = contraction (out features), 4 atoms of 64 input features
                const int pw = pt >> 5, l = pt & 31;
                const int nl = (pw >> 1) * 8 + ((l >> 1) & 7), q = (pw & 1) * 2 + (l >> 4);
                wrow = nl;  // + step*64
                wcol = n0 + q * 64;
                r8 = nl & 7;
                dst_off = q * 8192 + nl * 128;
                valid = wcol < args.w_cols;
            }
            // Only issues the loads: nothing here may depend on a loaded value, or the thread would sit
            // out a full L2 round trip every k-step.  The scale is decoded when the tile is built.
            auto fetch = [&](uint32_t it, uint4 &c, uint32_t &raw, float &a2) {
                const uint32_t g = step_begin + it;
                const size_t row = B_MN ? (size_t)wrow + (size_t)g * 64 : (size_t)wrow;
                const size_t col = B_MN ? (size_t)wcol : (size_t)g * 64;
                const size_t e = row * args.w_cols + col;  // first element of the quantisation block
                c = ldg_nc_v4(args.codes + (e >> 1) + hf * 16);
                const size_t blk = (e + hf * 32) >> args.blk_shift;  // the thread's 32 elements lie in one block
                if (args.dq) {
                    raw = __ldg(args.absmax_codes + blk);
                    a2 = __ldg(args.absmax2 + (blk >> 8));
                } else {
                    raw = 0;
                    a2 = __ldg(args.scales_f32 + blk);
                }
            };
            uint4 nc = make_uint4(0, 0, 0, 0);
            uint32_t nraw = 0;
            float na2 = 0.0f;
            long long prod_wait = 0;
            if (valid && main_steps > 0) fetch(0, nc, nraw, na2);
            for (uint32_t it = 0; it < total_steps; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                const bool ext = it >= main_steps;
                const uint4 c = nc;
                // (code as i8 as f32) / 127 * absmax2[blk / 256]   (quant.rs:212-221)
                const float scale = args.dq ? __fmul_rn(__fdiv_rn((float)(int8_t)nraw, 127.0f), na2) : na2;
                if (valid && it + 1 < main_steps) fetch(it + 1, nc, nraw, na2);
                const long long tw = tstamp ? clock64() : 0;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 3)) break;
                if (tstamp) prod_wait += clock64() - tw;
                if (!ext) {
                    const uint32_t dst = smem_base + s * kStageBytes + kABytes + dst_off;
                    if (valid) {
                        uint32_t pairs[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            pairs[j] = pack_bf16(__fmul_rn(c_levels[2 * j], scale), __fmul_rn(c_levels[2 * j + 1], scale));
                        const nf4::Tables tb = nf4::make_tables(pairs);
                        const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t o[4];
                            nf4::decode_word(tb, cw[j], o);
                            sts_v4(dst + (((hf * 4 + j) ^ r8) << 4), make_uint4(o[0], o[1], o[2], o[3]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) sts_v4(dst + ((hf * 4 + j) << 4), make_uint4(0, 0, 0, 0));
                    }
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(s));
            }
            if (tstamp && threadIdx.x == 64) {
                tstamp[5] = clock64();  // producer loop done
                tstamp[6] = prod_wait;  // cycles producer warp 0 spent waiting for empty stages
            }
        }

        // epilogue: TMEM -> registers -> global
        if (mbar_wait(tmem_full_bar, 0, abort_flag, args.status, 4)) {
            tc_fence_after();
            if (tstamp && threadIdx.x == 64) tstamp[7] = clock64();  // accumulators complete
            const int quarter = warp & 3;        // TMEM lanes this warp may touch: 32*quarter .. +31
            const int half = (warp - 2) >> 2;    // the warps of a quarter split the columns
            constexpr int kColsPerWarp = BN / (kWorkerWarps<B_DEQUANT> / 4);
            const size_t split_off = (size_t)z * Mrows * args.ldo;
            if constexpr (BN < 64) {
                // Narrow tile (rank-16/32 LoRA products): one warp per lane quarter writes its rows, bf16,
                // followed by zeros up to out_pad_cols so the consumer can read a fixed 64-wide operand.
                const uint32_t lrow = quarter * 32 + lane, row = m0 + lrow;
                if (half == 0) {  // warp-uniform: every lane takes part in the aligned tcgen05.ld
                    const bool ok = row < Mrows && lrow < args.a_rows;
                    __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(outp) + split_off + (size_t)row * args.ldo + n0;
#pragma unroll
                    for (int cc = 0; cc < BN; cc += 16) {
                        uint32_t v[16];
                        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + cc, v);
                        tmem_ld_wait();
                        for (uint32_t ji = 1; ji < active_issuers; ++ji) {  // CTA-uniform trip count
                            uint32_t u[16];
                            tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + ji * BN + cc, u);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                        }
                        if (ok && args.out_bf16) {
#pragma unroll
                            for (int j = 0; j < 16; j += 8) {
                                uint4 pk;
                                pk.x = pack_bf16(__uint_as_float(v[j + 0]) * args.out_scale, __uint_as_float(v[j + 1]) * args.out_scale);
                                pk.y = pack_bf16(__uint_as_float(v[j + 2]) * args.out_scale, __uint_as_float(v[j + 3]) * args.out_scale);
                                pk.z = pack_bf16(__uint_as_float(v[j + 4]) * args.out_scale, __uint_as_float(v[j + 5]) * args.out_scale);
                                pk.w = pack_bf16(__uint_as_float(v[j + 6]) * args.out_scale, __uint_as_float(v[j + 7]) * args.out_scale);
                                *reinterpret_cast<uint4 *>(o + cc + j) = pk;
                            }
                        } else if (ok) {
                            float *of = static_cast<float *>(outp) + split_off + (size_t)row * args.ldo + n0 + cc;
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                float4 f = make_float4(__uint_as_float(v[j + 0]) * args.out_scale, __uint_as_float(v[j + 1]) * args.out_scale,
                                                       __uint_as_float(v[j + 2]) * args.out_scale, __uint_as_float(v[j + 3]) * args.out_scale);
                                if (TF32) {  // a tf32 operand of the kernels that follow: round rather than let them truncate
                                    f.x = __uint_as_float(tf32_rna(f.x));
                                    f.y = __uint_as_float(tf32_rna(f.y));
                                    f.z = __uint_as_float(tf32_rna(f.z));
                                    f.w = __uint_as_float(tf32_rna(f.w));
                                }
                                *reinterpret_cast<float4 *>(of + j) = f;
                            }
                        }
                    }
                    if (ok && args.out_bf16) {
                        for (uint32_t cz = BN; cz < args.out_pad_cols; cz += 8)
                            *reinterpret_cast<uint4 *>(o + cz) = make_uint4(0, 0, 0, 0);
                    } else if (ok) {
                        float *of = static_cast<float *>(outp) + split_off + (size_t)row * args.ldo + n0;
                        for (uint32_t cz = BN; cz < args.out_pad_cols; cz += 4)
                            *reinterpret_cast<float4 *>(of + cz) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                }
            } else
#pragma unroll 1
            for (int a = 0; a < ACC; ++a) {
                const uint32_t row = m0 + a * kBM + quarter * 32 + lane;
#pragma unroll 1
                for (int cc = 0; cc < kColsPerWarp; cc += 32) {
                    const int col = half * kColsPerWarp + cc;
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN + col, v);
                    tmem_ld_wait();
                    if constexpr (NI > 1) {
                        for (uint32_t ji = 1; ji < active_issuers; ++ji) {  // CTA-uniform trip count
                            uint32_t u[32];
                            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ji * BN + col, u);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                        }
                    }
                    const uint32_t gcol = n0 + col;
                    if (row < Mrows && gcol < args.N && a * kBM + quarter * 32 + lane < (int)args.a_rows) {
                        if (args.out_bf16) {
                            __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(outp) + split_off +
                                               (size_t)row * args.ldo + gcol;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 pk;
                                pk.x = pack_bf16(__uint_as_float(v[j + 0]) * args.out_scale, __uint_as_float(v[j + 1]) * args.out_scale);
                                pk.y = pack_bf16(__uint_as_float(v[j + 2]) * args.out_scale, __uint_as_float(v[j + 3]) * args.out_scale);
                                pk.z = pack_bf16(__uint_as_float(v[j + 4]) * args.out_scale, __uint_as_float(v[j + 5]) * args.out_scale);
                                pk.w = pack_bf16(__uint_as_float(v[j + 6]) * args.out_scale, __uint_as_float(v[j + 7]) * args.out_scale);
                                *reinterpret_cast<uint4 *>(o + j) = pk;
                            }
                        } else {
                            float *o = static_cast<float *>(outp) + split_off + (size_t)row * args.ldo + gcol;
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 f;
                                f.x = __uint_as_float(v[j + 0]) * args.out_scale;
                                f.y = __uint_as_float(v[j + 1]) * args.out_scale;
                                f.z = __uint_as_float(v[j + 2]) * args.out_scale;
                                f.w = __uint_as_float(v[j + 3]) * args.out_scale;
                                if (TF32 && args.out_pad_cols) {  // T1p / Dsp: tf32 operands of the kernels that follow
                                    f.x = __uint_as_float(tf32_rna(f.x));
                                    f.y = __uint_as_float(tf32_rna(f.y));
                                    f.z = __uint_as_float(tf32_rna(f.z));
                                    f.w = __uint_as_float(tf32_rna(f.w));
                                }
                                *reinterpret_cast<float4 *>(o + j) = f;
                            }
                        }
                    }
                }
            }
        }
        tc_fence_before();
        if (!B_DEQUANT && args.counters) __threadfence();  // this thread's partial sums are visible device-wide
    }

    __syncthreads();
    pause_after_abort(abort_flag);
    if (tstamp && threadIdx.x == 0) tstamp[8] = clock64();  // epilogue finished
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if constexpr (!B_DEQUANT) {
        if (args.counters) {
            // Token-split partial sums: whichever CTA of this output tile finishes last adds the partials of
            // all splits, always in split order, so the result does not depend on which CTA that is.  Nobody
            // waits for anybody.
            __shared__ int s_last;
            int *counter = args.counters + (second ? gridDim.y : 0u) + blockIdx.y;
            if (threadIdx.x == 0) {
                const int prev = atomicAdd(counter, 1);
                s_last = (prev == (int)gridDim.z - 1) ? 1 : 0;
                if (s_last) *counter = 0;  // ready for the next launch
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                const float *part = static_cast<const float *>(outp);
                float *fin = second ? args.final2 : args.final1;
                const int transposed = second ? args.transposed2 : args.transposed1;
                const uint32_t rows_here = Mrows - m0 < args.a_rows ? Mrows - m0 : args.a_rows;
                const uint32_t cu = args.cols_used;
                for (uint32_t i = threadIdx.x; i < rows_here * cu; i += blockDim.x) {
                    const uint32_t lr = transposed ? i % rows_here : i / cu;
                    const uint32_t c = transposed ? i / rows_here : i % cu;
                    const uint32_t r = m0 + lr;
                    const size_t oi = transposed ? (size_t)c * Mrows + r : (size_t)r * (args.final_ld ? args.final_ld : cu) + c;
                    float v[16];  // at most 16 splits; all loads are issued before the first add
#pragma unroll
                    for (uint32_t zz = 0; zz < 16; ++zz)
                        v[zz] = zz < gridDim.z ? __ldcg(part + ((size_t)zz * Mrows + r) * args.ldo + c) : 0.0f;
                    float acc = args.accumulate ? fin[oi] : 0.0f;
#pragma unroll
                    for (uint32_t zz = 0; zz < 16; ++zz)
                        if (zz < gridDim.z) acc += v[zz];
                    fin[oi] = acc;
                }
            }
        }
    }
}

// ---- the paired-CTA weight GEMM --------------------------------------------------------------------
// Same algorithm as umma_gemm_kernel<256, 2, false, B_MN, true>, but two CTAs of a cluster (a CTA pair on
// one TPC) work as one: tcgen05.mma.cta_group::2 computes a 256-row x 256-column product per instruction,
// each CTA supplying its own 128 activation rows and HALF of the weight tile.  Per CTA and k-step that is
//   * half the nibble decoding (128 quantisation blocks instead of 256), and
//   * half the shared-memory traffic for the weight operand (each half is read once from its home SM
//     and feeds both tensor cores), which is what bounds the single-CTA kernel.
// With 48 KiB per stage there is room for four stages.  Worker warps form two groups that take alternate
// k-steps.  All barriers the MMA thread waits on live in the leader CTA (cluster rank 0): the peer's TMA
// transactions and producer warps signal them remotely; the leader's tcgen05.commit releases the stage in
// both CTAs.  Every wait is bounded as in the single-CTA kernel.
constexpr int kGroupWarps2 = 8;
constexpr int kWorkerWarps2 = 2 * kGroupWarps2;
constexpr int kThreads2 = 32 * (2 + kWorkerWarps2);
constexpr int kStages2 = 4;
constexpr uint32_t kABytes2 = 2 * kBM * kBK * 2;   // two 128x64 activation tiles
constexpr uint32_t kBBytes2 = 128 * kBK * 2;       // this CTA's half of the 256-wide weight tile
constexpr uint32_t kStageBytes2 = kABytes2 + kBBytes2;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
                 "r"(bytes)
                 : "memory");
}
// TMA tile load issued by one CTA of a pair; the completion bytes are reported to `bar`, which may live in
// the peer CTA's shared memory (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma2_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint2 ldg_nc_v2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// Arrives on `cluster_bar` (any CTA of the pair) once all MMAs issued so far by this thread are complete.
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                 : "memory");
}

// TF32: activations and the LoRA operands are fp32 in memory, the producers write fp32 weights rounded to
// tf32, and the tensor core reads everything as tf32: a k-step then covers 32 contraction elements (the same
// bytes), the weight tile's MN-major atoms are 32 elements wide, and the MMA rate is half the bf16 rate.
template <bool B_MN, bool TF32 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
umma_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAext,
                  const __grid_constant__ CUtensorMap tmBext, const __grid_constant__ CUtensorMap tmOut,
                  const GemmArgs args) {
    constexpr int BN = 256;
    constexpr uint32_t kTmemCols = 512;
    constexpr int kStepElems = TF32 ? 32 : 64;         // contraction elements per k-step (one 128-byte row)
    constexpr int kAtomElems = TF32 ? 32 : 64;         // N elements per MN-major atom
    constexpr uint32_t kAtomBytes = kStepElems * 128;  // one MN-major atom of a stage
    constexpr uint32_t kMnStep = TF32 ? 1024 : 2048;   // MN-major operand: bytes per MMA along the contraction

    pdl_trigger();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmAext);
        prefetch_tmap(&tmBext);
        prefetch_tmap(&tmOut);
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages2 * kStageBytes2;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };               // used in the leader CTA only
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages2 + s); };  // one per CTA
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * kStages2);
    const uint32_t pieces_bar = bar_base + 8u * (2 * kStages2 + 1);  // cut tiles: every worker warp stored its partial
    const uint32_t verdict_bar = bar_base + 8u * (2 * kStages2 + 2); // cut tiles: s_last is valid
    uint8_t *tail = smem_gen + kStages2 * kStageBytes2 + 8 * (2 * kStages2 + 3);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 4);
    volatile int *s_last = reinterpret_cast<volatile int *>(tail + 8);
    float *s_q127 = reinterpret_cast<float *>(tail + 16);  // exact (i8 as f32)/127 quotients, 256 entries
    float *s_lev = s_q127 + 256;                           // the 16 NF4 levels (tf32 producers)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    long long *const tstamp = args.timing ? args.timing + 16 * (size_t)blockIdx.x : nullptr;
    // grid: one CTA pair per work item, in launch order (whole tiles first, then the pieces of cut tiles)
    const uint32_t item = blockIdx.x >> 1;
    const bool cut = item >= args.full_items;
    const uint32_t n_chunks = cut ? args.k_chunks : 1u;
    const uint32_t cut_tile = cut ? (item - args.full_items) / n_chunks : 0u;
    const uint32_t chunk = cut ? (item - args.full_items) % n_chunks : 0u;
    const uint32_t tile = cut ? args.full_items + cut_tile : item;
    // Column tile fastest: the pairs resident at one time share a few 512-row slabs of activations (each
    // read from HBM once, then served by L2) and sweep the whole weight payload, which is small enough to
    // stay in L2.
    const uint32_t ct = args.row_fastest ? tile / args.row_tiles : tile % args.col_tiles;
    const uint32_t rt = args.row_fastest ? tile % args.row_tiles : tile / args.col_tiles;
    const uint32_t n0 = ct * BN;                    // first output column of the pair
    const uint32_t nh = n0 + rank * 128;            // first column of this CTA's half of the weight tile
    const uint32_t m0 = (rt * 2 + rank) * (2 * kBM);  // first output row of this CTA
    const uint32_t k_begin = (uint32_t)(((uint64_t)args.k_steps * chunk) / n_chunks);
    const uint32_t main_steps = (uint32_t)(((uint64_t)args.k_steps * (chunk + 1)) / n_chunks) - k_begin;
    const uint32_t total_steps = main_steps + (chunk + 1 == n_chunks ? args.ext_steps : 0u);  // LoRA step: last piece

    if (tstamp && threadIdx.x == 0) {
        tstamp[0] = clock64();
        unsigned long long g;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
        tstamp[12] = (long long)g;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(full_bar(s), 2 + 2 * kGroupWarps2);  // 2 TMA threads + one producer group per CTA
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, 1);
        mbar_init(pieces_bar, kWorkerWarps2);
        mbar_init(verdict_bar, 1);
        *abort_flag = (args.status->code != 0) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (threadIdx.x < 256) s_q127[threadIdx.x] = __fdiv_rn((float)(int8_t)(uint8_t)threadIdx.x, 127.0f);
    if (TF32 && threadIdx.x < 16) s_lev[threadIdx.x] = c_levels[threadIdx.x];
    cluster_sync_all();
    // If an earlier launch already raised a status, the pair does nothing; the decision is the leader's.
    const bool skip = ld_cluster_u32(mapa_u32(smem_u32(const_cast<int *>(abort_flag)), 0)) != 0;
    cluster_sync_all();
    if (skip) return;
    if (threadIdx.x == 0) *abort_flag = 0;

    if (warp == 1) {
        tmem_alloc2(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish2();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // everything above touched no memory an earlier kernel writes (the status word is only ever raised)
    if (tstamp && threadIdx.x == 0) tstamp[1] = clock64();

    if (warp == 0) {
        // ---------------- TMA issue (both CTAs; completion is reported to the leader's barrier) -----------
        if (lane == 0) {
            for (uint32_t it = 0; it < total_steps; ++it) {
                const int s = it % kStages2;
                const uint32_t ph = (it / kStages2) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 11)) break;
                const bool ext = it >= main_steps;
                const uint32_t a_dst = smem_base + s * kStageBytes2;
                const uint32_t b_dst = a_dst + kABytes2;
                const uint32_t lead_full = mapa_u32(full_bar(s), 0);
                mbar_arrive_expect_tx_cluster(lead_full, kABytes2 + (ext ? kBBytes2 : 0u));
                const int kc = ext ? (int)((it - main_steps) * kStepElems) : (int)((k_begin + it) * kStepElems);
                const CUtensorMap *ma = ext ? &tmAext : &tmA;
#pragma unroll
                for (int a = 0; a < 2; ++a)
                    tma_load_2d_pair(a_dst + a * (kBM * 128), ma, lead_full, kc, (int)(m0 + a * kBM));
                if (ext) {
                    if (!B_MN) {
                        tma_load_2d_pair(b_dst, &tmBext, lead_full, kc, (int)nh);  // 128 rows of B_pad
                    } else {
#pragma unroll
                        for (int g = 0; g < 128 / kAtomElems; ++g)
                            tma_load_2d_pair(b_dst + g * kAtomBytes, &tmBext, lead_full, (int)(nh + g * kAtomElems), kc);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issue (leader CTA only) ----------------
        if (leader && lane == 0) {
            constexpr uint32_t kFmt = TF32 ? 2u : 1u;  // operand format: bf16 = 1, tf32 = 2; accumulator fp32 = 1
            constexpr uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((B_MN ? 1u : 0u) << 16) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            bool ok = true;
            long long mma_wait = 0;
            for (uint32_t it = 0; it < total_steps; ++it) {
                const int s = it % kStages2;
                const uint32_t ph = (it / kStages2) & 1u;
                const long long tw = tstamp ? clock64() : 0;
                if (!mbar_wait(full_bar(s), ph, abort_flag, args.status, 12)) {
                    ok = false;
                    break;
                }
                if (tstamp) {
                    mma_wait += clock64() - tw;
                    if (it == 0) tstamp[2] = clock64();
                }
                tc_fence_after();
                const uint32_t a_src = smem_base + s * kStageBytes2;
                const uint32_t b_src = a_src + kABytes2;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
#pragma unroll
                    for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                        const uint64_t da = make_desc(a_src + a * (kBM * 128) + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_desc(b_src + kk * kMnStep, kAtomBytes, TF32 ? 512u : 1024u, TF32 ? 1u : 2u)
                                                 : make_desc(b_src + kk * 32, 16, 1024);
                        if (TF32)
                            umma2_tf32(tmem_base + a * BN, da, db, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                        else
                            umma2_bf16(tmem_base + a * BN, da, db, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma2_commit(mapa_u32(empty_bar(s), 0));
                umma2_commit(mapa_u32(empty_bar(s), 1));
            }
            if (ok) {
                umma2_commit(mapa_u32(tmem_full_bar, 0));
                umma2_commit(mapa_u32(tmem_full_bar, 1));
            }
            if (tstamp) {
                tstamp[3] = clock64();
                tstamp[4] = mma_wait;
            }
        }
        __syncwarp();
    } else {
        // ---------------- weight-tile producers (two groups, alternate k-steps), then epilogue ----------
        const int group = (warp - 2) / kGroupWarps2;
        const int pt = (threadIdx.x - 64) & 255;  // thread inside its group
        long long prod_wait = 0, t_dec = 0, t_fence = 0, t_top = 0;
        if constexpr (TF32) {
            // One k-step covers 32 contraction elements: a thread builds 16 fp32 weights (8 bytes of nibbles,
            // half of a quantisation block's share of the step) = four 16-byte chunks of one 128-byte row.
            const int hf = pt & 1;
            uint32_t r8, dst_off;
            bool valid;
            size_t e0, e_step;  // first weight element of this thread at k-step 0; elements per k-step
            if (!B_MN) {
                // forward: rows = output features nh..nh+127, 32 consecutive input features per k-step
                const int rl = pt >> 1;
                r8 = rl & 7;
                dst_off = rl * 128;
                const size_t row = (size_t)nh + rl;
                valid = row < args.w_rows;
                e0 = row * args.w_cols + hf * 16;
                e_step = 32;
            } else {
                // backward: rows = contraction (32 output features per k-step), four 32-wide atoms of input features
                const int pw = pt >> 5, l = pt & 31;
                const int nl = (pw & 3) * 8 + ((l >> 1) & 7), q = (pw >> 2) * 2 + (l >> 4);
                r8 = nl & 7;
                dst_off = q * 4096 + nl * 128;
                const size_t col = (size_t)nh + q * 32;
                valid = col < args.w_cols;
                e0 = (size_t)nl * args.w_cols + col + hf * 16;
                e_step = (size_t)32 * args.w_cols;
            }
            e0 += (size_t)k_begin * e_step;
            // K-major tile: 16-byte chunks swizzled by the row (chunk ^ row % 8).  MN-major tile of 32-bit elements:
            // 32-byte chunks swizzled by the row (chunk ^ row % 4), each written as two 16-byte halves.
            uint32_t st_off[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                st_off[j] = B_MN ? dst_off + ((((uint32_t)hf * 2 + (j >> 1)) ^ (r8 & 3u)) << 5) + (j & 1) * 16
                                 : dst_off + (((hf * 4 + j) ^ r8) << 4);
            auto fetch = [&](uint32_t it, uint2 &c, uint32_t &raw, float &a2) {
                const size_t e = e0 + (size_t)it * e_step;
                c = ldg_nc_v2(args.codes + (e >> 1));
                const size_t blk = e >> args.blk_shift;  // the thread's 16 elements lie in one block
                if (args.dq) {
                    raw = __ldg(args.absmax_codes + blk);
                    a2 = __ldg(args.absmax2 + (blk >> 8));
                } else {
                    raw = 0;
                    a2 = __ldg(args.scales_f32 + blk);
                }
            };
            uint2 nc = make_uint2(0, 0);
            uint32_t nraw = 0;
            float na2 = 0.0f;
            if (valid && (uint32_t)group < main_steps) fetch(group, nc, nraw, na2);
            for (uint32_t it = group; it < total_steps; it += 2) {
                const int s = it % kStages2;
                const uint32_t ph = (it / kStages2) & 1u;
                const bool ext = it >= main_steps;
                const uint2 c = nc;
                // (code as i8 as f32) / 127 * absmax2[blk / 256]   (quant.rs:212-221)
                const float scale = args.dq ? __fmul_rn(s_q127[nraw & 255u], na2) : na2;
                if (valid && it + 2 < main_steps) fetch(it + 2, nc, nraw, na2);
                const long long tw = tstamp ? clock64() : 0;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 13)) break;
                if (tstamp) prod_wait += clock64() - tw;
                if (!ext) {
                    const uint32_t dst = smem_base + s * kStageBytes2 + kABytes2;
                    const uint32_t cw[2] = {c.x, c.y};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 o = make_uint4(0, 0, 0, 0);
                        if (valid) {
                            const uint32_t w4 = cw[j >> 1] >> (16 * (j & 1));  // four nibbles
                            // level * scale is the exact fp32 dequantised weight (quant.rs:157-167), then tf32
                            o.x = tf32_rna(__fmul_rn(s_lev[w4 & 15u], scale));
                            o.y = tf32_rna(__fmul_rn(s_lev[(w4 >> 4) & 15u], scale));
                            o.z = tf32_rna(__fmul_rn(s_lev[(w4 >> 8) & 15u], scale));
                            o.w = tf32_rna(__fmul_rn(s_lev[(w4 >> 12) & 15u], scale));
                        }
                        sts_v4(dst + st_off[j], o);
                    }
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor cores' async proxy
                }
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(full_bar(s), 0));
            }
        } else {
            const int hf = pt & 1;
            uint32_t r8, dst_off;
            bool valid;
            const uint8_t *code_ptr;   // this thread's 16 bytes of nibbles at k-step 0
            size_t el0;                // its first element (flat index into the weight) at k-step 0
            size_t code_step, el_step;  // increments per k-step
            if (!B_MN) {
                // forward: rows = output features nh..nh+127, quantisation block along the contraction
                const int rl = pt >> 1;
                r8 = rl & 7;
                dst_off = rl * 128;
                const size_t row = (size_t)nh + rl;
                valid = row < args.w_rows;
                const size_t e = row * args.w_cols;
                code_ptr = args.codes + (e >> 1) + hf * 16;
                el0 = e + hf * 32;
                code_step = 32;
                el_step = 64;
            } else {
                // backward: rows = contraction (output features), two 64-wide atoms of input features
                const int pw = pt >> 5, l = pt & 31;
                const int nl = pw * 8 + ((l >> 1) & 7), ql = l >> 4;
                r8 = nl & 7;
                dst_off = ql * 8192 + nl * 128;
                const size_t col = (size_t)nh + ql * 64;
                valid = col < args.w_cols;
                const size_t e = (size_t)nl * args.w_cols + col;
                code_ptr = args.codes + (e >> 1) + hf * 16;
                el0 = e + hf * 32;
                code_step = (size_t)32 * args.w_cols;  // 64 weight rows further down
                el_step = (size_t)64 * args.w_cols;
            }
            code_ptr += (size_t)k_begin * code_step;  // this piece's first k-step
            el0 += (size_t)k_begin * el_step;
            uint32_t st_off[4];
    #pragma unroll
            for (int j = 0; j < 4; ++j) st_off[j] = dst_off + (((hf * 4 + j) ^ r8) << 4);
            // Only issues the loads: nothing here may depend on a loaded value, or the thread would sit out a
            // full L2 round trip every k-step.  The scale is decoded when the tile is built.
            auto fetch = [&](uint32_t it, uint4 &c, uint32_t &raw, float &a2) {
                c = ldg_nc_v4(code_ptr + (size_t)it * code_step);
                const size_t blk = (el0 + (size_t)it * el_step) >> args.blk_shift;  // the thread's 32 elements lie in one block
                if (args.dq) {
                    raw = __ldg(args.absmax_codes + blk);
                    a2 = __ldg(args.absmax2 + (blk >> 8));
                } else {
                    raw = 0;
                    a2 = __ldg(args.scales_f32 + blk);
                }
            };
            uint4 nc = make_uint4(0, 0, 0, 0);
            uint32_t nraw = 0;
            float na2 = 0.0f;
            if (valid && (uint32_t)group < main_steps) fetch(group, nc, nraw, na2);
            for (uint32_t it = group; it < total_steps; it += 2) {
                const int s = it % kStages2;
                const uint32_t ph = (it / kStages2) & 1u;
                const bool ext = it >= main_steps;
                const long long tt = tstamp ? clock64() : 0;
                const uint4 c = nc;
                // (code as i8 as f32) / 127 * absmax2[blk / 256]   (quant.rs:212-221); exact quotients from the table
                const float scale = args.dq ? __fmul_rn(s_q127[nraw & 255u], na2) : na2;
                if (valid && it + 2 < main_steps) fetch(it + 2, nc, nraw, na2);
                const long long tw = tstamp ? clock64() : 0;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 13)) break;
                const long long td = tstamp ? clock64() : 0;
                if (tstamp) {
                    prod_wait += td - tw;
                    t_top += tw - tt;
                }
                if (!ext) {
                    const uint32_t dst = smem_base + s * kStageBytes2 + kABytes2;
                    if (valid) {
                        uint32_t pairs[8];
    #pragma unroll
                        for (int j = 0; j < 8; ++j)
                            pairs[j] = pack_bf16(__fmul_rn(c_levels[2 * j], scale), __fmul_rn(c_levels[2 * j + 1], scale));
                        const nf4::Tables tb = nf4::make_tables(pairs);
                        const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
    #pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t o[4];
                            nf4::decode_word(tb, cw[j], o);
                            sts_v4(dst + st_off[j], make_uint4(o[0], o[1], o[2], o[3]));
                        }
                    } else {
    #pragma unroll
                        for (int j = 0; j < 4; ++j) sts_v4(dst + st_off[j], make_uint4(0, 0, 0, 0));
                    }
                    const long long tf = tstamp ? clock64() : 0;
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor cores' async proxy
                    if (tstamp) {
                        t_dec += tf - td;
                        t_fence += clock64() - tf;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(full_bar(s), 0));
            }
        }
        if (tstamp && threadIdx.x == 64) {
            tstamp[5] = clock64();
            tstamp[6] = prod_wait;
            tstamp[9] = t_dec;
            tstamp[10] = t_fence;
            tstamp[11] = t_top;
        }

        // epilogue: this CTA's two 128x256 accumulators -> registers -> (bf16: shared memory -> TMA store)
        if (mbar_wait(tmem_full_bar, 0, abort_flag, args.status, 14)) {
            tc_fence_after();
            if (tstamp && threadIdx.x == 64) tstamp[7] = clock64();
            const int quarter = warp & 3;
            const int sub = (warp - 2) >> 2;  // 0..3: 64 columns each
            // A piece of a cut tile first leaves its accumulators as an fp32 partial.  The CTA whose partial
            // completes the tile then builds the result from all partials, always adding them in chunk order,
            // so the result does not depend on which piece finished last; the other pieces are done.
            // Each thread later reads back exactly the addresses that the same thread of the other pieces wrote,
            // so a partial is stored thread-interleaved: float4 number g of worker thread t at g * 512 + t
            // (fully coalesced), g = (a * 2 + cc / 32) * 8 + j / 4.
            const size_t piece_floats = (size_t)2 * kBM * BN;
            float *const tile_ws = cut ? args.split_ws + (size_t)cut_tile * n_chunks * 2 * piece_floats : nullptr;
            const uint32_t wt = threadIdx.x - 64;
            bool finish = true;
            if (cut) {
                float4 *mine = reinterpret_cast<float4 *>(tile_ws + ((size_t)chunk * 2 + rank) * piece_floats) + wt;
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
#pragma unroll 1
                    for (int cc = 0; cc < 64; cc += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN + sub * 64 + cc, v);
                        tmem_ld_wait();
                        float4 *o = mine + (size_t)((a * 2 + cc / 32) * 8) * 512;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            __stcg(o + (j / 4) * 512, make_float4(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]),
                                                          __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                    }
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(pieces_bar);
                finish = false;
                if (mbar_wait(pieces_bar, 0, abort_flag, args.status, 15)) {
                    if (threadIdx.x == 64) {
                        int *counter = args.counters + cut_tile * 2 + rank;
                        const int prev = atomicAdd(counter, 1);
                        const int last = (prev == (int)n_chunks - 1) ? 1 : 0;
                        if (last) *counter = 0;  // ready for the next launch
                        *s_last = last;
                        __threadfence();
                        mbar_arrive(verdict_bar);
                    }
                    if (mbar_wait(verdict_bar, 0, abort_flag, args.status, 16)) finish = *s_last != 0;
                }
            }
            // One 32-column group of row (quarter * 32 + lane) of accumulator a.
            auto values = [&](int a, int cc, uint32_t (&v)[32]) {
                if (!cut) {
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN + sub * 64 + cc, v);
                    tmem_ld_wait();
                } else {
                    const float4 *src = reinterpret_cast<const float4 *>(tile_ws + (size_t)rank * piece_floats) + wt +
                                        (size_t)((a * 2 + cc / 32) * 8) * 512;
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                    for (uint32_t ch = 0; ch < n_chunks; ++ch) {
                        const float4 *q = src + (size_t)ch * 2 * (piece_floats / 4);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 f = __ldcg(q + (j / 4) * 512);
                            v[j + 0] = __float_as_uint(__uint_as_float(v[j + 0]) + f.x);
                            v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + f.y);
                            v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + f.z);
                            v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + f.w);
                        }
                    }
                }
            };
            if (finish && cut) __threadfence();  // the other pieces' partials, announced through the counter
            if (finish && args.out_bf16) {
                // All stages are idle now (every MMA has completed), so the pipeline's shared memory is reused:
                // each warp converts its 32 rows x 64 columns to bf16, writes them as a 4 KiB slab in the
                // 128-byte-swizzled layout and hands the slab to the TMA engine, which writes full 128-byte
                // row segments and clips rows/columns beyond the matrix.
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
                    const uint32_t slab = smem_base + (uint32_t)((a * 4 + sub) * 16384 + quarter * 4096);
                    const uint32_t row_off = slab + lane * 128;
                    const uint32_t r8 = lane & 7;
#pragma unroll
                    for (int cc = 0; cc < 64; cc += 32) {
                        uint32_t v[32];
                        values(a, cc, v);
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 pk;
                            pk.x = pack_bf16(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]));
                            pk.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                            pk.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                            pk.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                            const uint32_t chunk16 = (uint32_t)((cc + j) >> 3);
                            sts_v4(row_off + ((chunk16 ^ r8) << 4), pk);
                        }
                    }
                    fence_async_smem();
                    __syncwarp();
                    const uint32_t grow = m0 + a * kBM + quarter * 32, gcol = n0 + sub * 64;
                    if (lane == 0 && grow < args.M && gcol < args.N) tma_store_2d(&tmOut, slab, (int)gcol, (int)grow);
                }
                if (lane == 0) tma_store_commit_and_wait_read();
                __syncwarp();
            } else if (finish) {
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
                    const uint32_t row = m0 + a * kBM + quarter * 32 + lane;
#pragma unroll 1
                    for (int cc = 0; cc < 64; cc += 32) {
                        const int col = sub * 64 + cc;
                        uint32_t v[32];
                        values(a, cc, v);
                        const uint32_t gcol = n0 + col;
                        if (row < args.M && gcol < args.N) {
                            float *o = static_cast<float *>(args.out) + (size_t)row * args.ldo + gcol;
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4 *>(o + j) =
                                    make_float4(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]),
                                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        }
                    }
                }
            }
        }
        tc_fence_before();
    }

    // Neither CTA may leave while its peer can still touch its shared memory or barriers.
    __syncthreads();
    pause_after_abort(abort_flag);
    cluster_sync_all();
    if (tstamp && threadIdx.x == 0) {
        tstamp[8] = clock64();
        unsigned long long g;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
        tstamp[13] = (long long)g;
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}


#include "umma_gemm3.cuh"

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        QLC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p)
            return fail(QLC_ERR_GPU, "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return QLC_OK;
}

// bf16 row-major (rows, cols) matrix; box = 64 columns (128 bytes, swizzled) x box_rows rows.
// Row-major (rows, cols) matrix of bf16 (or fp32 when `f32`), boxes of one 128-byte row segment x box_rows rows.
// swizzle32: 32-byte swizzle chunks, for tiles that the tensor core reads as MN-major 32-bit operands.
// pitch: elements between rows (0: the rows are contiguous, pitch = cols), for column slices of a wider matrix.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool f32 = false,
             bool swizzle32 = false, uint64_t pitch = 0) {
    EncodeTiledFn enc = nullptr;
    QLC_TRY(get_encode_fn(&enc));
    const uint64_t es = f32 ? 4 : 2;
    if (!pitch) pitch = cols;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch * es) % 16)
        return fail(QLC_ERR_GPU, "tensor map: base %p / row pitch %llu bytes must be 16-byte aligned", base,
                    (unsigned long long)(pitch * es));
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch * es};
    const cuuint32_t box[2] = {f32 ? 32u : 64u, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void *>(base), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(QLC_ERR_GPU, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return QLC_OK;
}

template <int BN, int ACC, int STAGES>
constexpr size_t smem_bytes() {
    return (size_t)STAGES * (ACC * kBM * kBK * 2 + BN * kBK * 2) + 8 * (2 * STAGES + 1) + 16 + 1024;
}

// Diagnostics (environment variable QLC_GEMM_TIMING): runs the launch with per-CTA clock64 stamps,
// synchronises and prints where the cycles of an average CTA went.
template <class Launch>
int launch_with_timing(qlc_ctx *ctx, dim3 grid, GemmArgs args, Launch launch) {
    const size_t ctas = (size_t)grid.x * grid.y * grid.z;
    long long *d = nullptr;
    QLC_CUDA(cudaMalloc(&d, ctas * 16 * sizeof(long long)));
    QLC_CUDA(cudaMemsetAsync(d, 0, ctas * 16 * sizeof(long long), ctx->stream));
    args.timing = d;
    launch(args);
    ctx->launches += 1;
    QLC_CUDA(cudaStreamSynchronize(ctx->stream));
    std::vector<long long> h(ctas * 16);
    QLC_CUDA(cudaMemcpy(h.data(), d, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    cudaFree(d);
    double setup = 0, first = 0, loop = 0, mwait = 0, pwait = 0, ploop = 0, drain = 0, epi = 0, total = 0;
    double dec = 0, fen = 0, top = 0;
    for (size_t i = 0; i < ctas; ++i) {
        const long long *t = &h[16 * i];
        setup += t[1] - t[0];
        first += t[2] - t[1];
        loop += t[3] - t[2];
        mwait += t[4];
        ploop += t[5] ? t[5] - t[1] : 0;
        pwait += t[6];
        drain += t[7] - t[3];
        epi += t[8] - t[7];
        total += t[8] - t[0];
        dec += t[9];
        fen += t[10];
        top += t[11];
    }
    if (h[12]) {
        // wall-clock picture (globaltimer, ns): when CTAs started and ended, by launch-order eighths of the grid
        long long g0 = h[12], g1 = 0;
        for (size_t i = 0; i < ctas; ++i) {
            if (h[16 * i + 12] && h[16 * i + 12] < g0) g0 = h[16 * i + 12];
            if (h[16 * i + 13] > g1) g1 = h[16 * i + 13];
        }
        fprintf(stderr, "[qlc timing] kernel span %.1f us; per launch-order eighth: start min/max, end min/max, mean duration (us)\n",
                (g1 - g0) / 1e3);
        for (int e = 0; e < 8; ++e) {
            const size_t lo = ctas * e / 8, hi = ctas * (e + 1) / 8;
            long long s0 = LLONG_MAX, s1 = 0, e0 = LLONG_MAX, e1 = 0;
            double dur = 0;
            for (size_t i = lo; i < hi; ++i) {
                const long long a = h[16 * i + 12] - g0, b = h[16 * i + 13] - g0;
                if (a < s0) s0 = a;
                if (a > s1) s1 = a;
                if (b < e0) e0 = b;
                if (b > e1) e1 = b;
                dur += (double)(b - a);
            }
            fprintf(stderr, "[qlc timing]   CTAs %4zu..%4zu: start %.1f..%.1f  end %.1f..%.1f  mean %.1f\n", lo, hi - 1, s0 / 1e3,
                    s1 / 1e3, e0 / 1e3, e1 / 1e3, dur / 1e3 / (double)(hi - lo));
        }
    }
    const double n = (double)ctas;
    fprintf(stderr,
            "[qlc timing] grid %ux%ux%u steps %u+%u: total %.0f | setup %.0f | first full %.0f | mma loop %.0f "
            "(waiting %.0f) | producer loop %.0f (waiting %.0f, decode %.0f, fence %.0f, top %.0f) | drain %.0f | "
            "epilogue %.0f  [cycles/CTA]\n",
            grid.x, grid.y, grid.z, args.k_steps / args.splits, args.ext_steps, total / n, setup / n, first / n,
            loop / n, mwait / n, ploop / n, pwait / n, dec / n, fen / n, top / n, drain / n, epi / n);
    return QLC_OK;
}

template <int BN, int ACC, bool A_MN, bool B_MN, bool B_DEQUANT, int STAGES, int NI = 1, bool TF32 = false>
int launch_gemm(qlc_ctx *ctx, int prof_slot, const CUtensorMap &tA, const CUtensorMap &tB, const CUtensorMap &tAe,
                const CUtensorMap &tBe, const GemmArgs &args, cudaStream_t stream = nullptr) {
    if (!stream) stream = ctx->stream;
    auto kern = umma_gemm_kernel<BN, ACC, A_MN, B_MN, B_DEQUANT, STAGES, NI, TF32>;
    constexpr size_t smem = smem_bytes<BN, ACC, STAGES>();
    if ((size_t)ctx->umma_smem_optin < smem)
        return fail(QLC_ERR_GPU, "kernel needs %zu bytes of shared memory, device allows %d", smem,
                    ctx->umma_smem_optin);
    QLC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (args.k_steps % args.splits) return fail(QLC_ERR_GPU, "internal: %u steps not divisible by %u splits", args.k_steps, args.splits);
    if (args.a_rows == 0 || args.a_rows > (uint32_t)(ACC * kBM)) return fail(QLC_ERR_GPU, "internal: bad a_rows %u", args.a_rows);
    if (args.pair && (B_DEQUANT || args.N > (uint32_t)BN || args.ext_steps || args.k_steps2 % args.splits))
        return fail(QLC_ERR_GPU, "internal: bad pair launch");
    const uint32_t m_max = args.pair && args.M2 > args.M ? args.M2 : args.M;
    dim3 grid(args.pair ? 2u : (unsigned)ceil_div(args.N, BN), (unsigned)ceil_div(m_max, args.a_rows), args.splits);
    static const bool dump_timing = getenv("QLC_GEMM_TIMING") != nullptr;
    if (dump_timing)
        return launch_with_timing(ctx, grid, args, [&](const GemmArgs &a) {
            kern<<<grid, kBlockThreads<B_DEQUANT>, smem, ctx->stream>>>(tA, tB, tAe, tBe, a);
        });
    prof_begin(ctx, prof_slot, stream);
    QLC_CUDA(launch_pdl(kern, grid, dim3(kBlockThreads<B_DEQUANT>), smem, stream, tA, tB, tAe, tBe, args));
    prof_end(ctx, stream);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// Cutting the tiles of the paired-CTA GEMM's last wave along the contraction: with S pairs resident at a
// time, the `rest` tiles beyond the last full wave are each cut into `chunks` pieces when the pieces still fit
// into one wave; the GPU then ends on a short full wave instead of a long, mostly idle one.
// CTA pairs one launch of the persistent GEMM runs with: every pair of SMs, less the reserved ones.
static uint32_t pair_slots(const qlc_ctx *ctx) {
    const int sms = ctx->sm_count - ctx->reserved_sms;
    return sms >= 2 ? (uint32_t)sms / 2 : 1u;
}
void kcut_plan(const qlc_ctx *ctx, size_t M, size_t N, size_t k_steps, uint32_t *rest, uint32_t *chunks) {
    static const bool no_cut = getenv("QLC_NO_KCUT") != nullptr;  // diagnostics
    const uint32_t tiles = (uint32_t)(ceil_div(M, 4 * kBM) * ceil_div(N, 256));
    const uint32_t slots = pair_slots(ctx);
    *rest = tiles % slots;
    uint32_t c = (*rest && !no_cut) ? slots / *rest : 1u;
    if (c > 4) c = 4;
    // A piece pays its own prologue, partial store and reduction (several microseconds): only worth it when it
    // still carries a main loop of at least 16 k-steps (4 microseconds).
    while (c > 1 && k_steps < 16 * (size_t)c) --c;
    *chunks = c;
}
// Bytes of fp32 partials the cut tiles need (0: nothing is cut).
size_t kcut_bytes(const qlc_ctx *ctx, size_t M, size_t N, size_t k_steps) {
    uint32_t rest = 0, chunks = 1;
    kcut_plan(ctx, M, N, k_steps, &rest, &chunks);
    return chunks > 1 ? (size_t)rest * chunks * 2 * (2 * kBM * 256) * sizeof(float) : 0;
}

template <bool B_MN, bool TF32 = false>
int launch_gemm2(qlc_ctx *ctx, int prof_slot, const CUtensorMap &tA, const CUtensorMap &tAe, const CUtensorMap &tBe,
                 const GemmArgs &args_in, float *split_ws) {
    const GemmArgs &a0 = args_in;
    // bf16 results leave through TMA stores of 32-row x 64-column slabs; fp32 results are stored directly
    CUtensorMap tOut = tA;
    if (a0.out_bf16) QLC_TRY(make_map(&tOut, a0.out, a0.M, a0.N, 32));
    auto kern = umma_gemm2_kernel<B_MN, TF32>;
    constexpr size_t smem = (size_t)kStages2 * kStageBytes2 + 8 * (2 * kStages2 + 3) + 16 + 1024 + 64 + 1024;
    if ((size_t)ctx->umma_smem_optin < smem)
        return fail(QLC_ERR_GPU, "kernel needs %zu bytes of shared memory, device allows %d", smem,
                    ctx->umma_smem_optin);
    QLC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // One CTA pair (cluster 2x1x1) per work item.  A pair covers 512 rows x 256 columns; tiles are numbered
    // row tile fastest.  With S pairs resident at a time, the tiles beyond the last full wave of S are each
    // cut into k_chunks pieces along the contraction when the pieces still fit into one wave: the GPU then
    // ends on a short full wave instead of a long, mostly idle one.
    GemmArgs args = args_in;
    uint32_t rest = 0, chunks = 1;
    if (split_ws) kcut_plan(ctx, args.M, args.N, args.k_steps, &rest, &chunks);
    args.row_tiles = (uint32_t)ceil_div(args.M, 4 * kBM);
    args.col_tiles = (uint32_t)ceil_div(args.N, 256);
    static const bool row_fastest = getenv("QLC_ROW_FASTEST") != nullptr;  // diagnostics
    args.row_fastest = row_fastest ? 1 : 0;
    const uint32_t tiles = args.row_tiles * args.col_tiles;
    args.k_chunks = chunks;
    args.full_items = chunks > 1 ? tiles - rest : tiles;
    const uint32_t items = args.full_items + (chunks > 1 ? rest * chunks : 0u);
    if (chunks > 1) {
        args.split_ws = split_ws;
        QLC_TRY(ctx_tile_counters(ctx, 1, 2 * (size_t)rest, &args.counters));
    }
    dim3 grid(2 * items, 1, 1);
    static const bool dump_timing = getenv("QLC_GEMM_TIMING") != nullptr;
    static const bool one_tile_t = getenv("QLC_GEMM_ONE_TILE_PER_PAIR") != nullptr;
    if (dump_timing && one_tile_t)
        return launch_with_timing(ctx, grid, args, [&](const GemmArgs &a) {
            kern<<<grid, kThreads2, smem, ctx->stream>>>(tA, tAe, tBe, tOut, a);
        });
    if (dump_timing) {
        // the persistent kernel's own sums: per leader CTA, cycles
        auto kern3 = umma_gemm3_kernel<B_MN, TF32, true>;
        QLC_CUDA(cudaFuncSetAttribute(kern3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem3));
        const uint32_t pairs = items < pair_slots(ctx) ? items : pair_slots(ctx);
        const size_t ctas = 2 * (size_t)pairs;
        long long *d = nullptr;
        QLC_CUDA(cudaMalloc(&d, ctas * 16 * sizeof(long long)));
        QLC_CUDA(cudaMemsetAsync(d, 0, ctas * 16 * sizeof(long long), ctx->stream));
        args.timing = d;
        kern3<<<dim3(2 * pairs), kThreads3, kSmem3, ctx->stream>>>(tA, tAe, tBe, tOut, args);
        ctx->launches += 1;
        QLC_CUDA(cudaStreamSynchronize(ctx->stream));
        std::vector<long long> h(ctas * 16);
        QLC_CUDA(cudaMemcpy(h.data(), d, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
        cudaFree(d);
        double tot = 0, issue = 0, wfull = 0, wfirst = 0, wa0 = 0, wa1 = 0, eidle = 0, e0 = 0, e1 = 0, pw = 0, nd = 0;
        for (size_t i = 0; i < ctas; i += 2) {  // leaders
            const long long *t = &h[16 * i];
            tot += t[11] - t[0]; issue += t[1] - t[0]; wfull += t[2]; wfirst += t[3]; wa0 += t[4]; wa1 += t[5];
            eidle += t[6]; e0 += t[7]; e1 += t[8]; nd += t[9]; pw += t[10];
        }
        const double n = (double)pairs;
        fprintf(stderr, "[qlc timing3] %u pairs, %u items (%.2f per pair), %u+%u steps: life %.0f | mma issue span %.0f | mma waits: full %.0f, "
                        "first full of an item %.0f, acc0 %.0f, acc1 %.0f | epilogue: idle %.0f, to acc0 release %.0f, to acc1 release %.0f | "
                        "producer group 0 waiting %.0f  [cycles per pair, sums over its items]\n",
                pairs, items, nd / n, args.k_steps, args.ext_steps, tot / n, issue / n, wfull / n, wfirst / n, wa0 / n, wa1 / n, eidle / n,
                e0 / n, e1 / n, pw / n);
        return QLC_OK;
    }
    // Default: the persistent kernel, one wave of CTA pairs that walk the same item list (QLC_GEMM_ONE_TILE_PER_PAIR
    // selects the one-item-per-pair kernel above, for A/B measurements).
    static const bool one_tile = getenv("QLC_GEMM_ONE_TILE_PER_PAIR") != nullptr;
    if (!one_tile) {
        auto kern3 = umma_gemm3_kernel<B_MN, TF32>;
        if ((size_t)ctx->umma_smem_optin < kSmem3)
            return fail(QLC_ERR_GPU, "kernel needs %zu bytes of shared memory, device allows %d", kSmem3, ctx->umma_smem_optin);
        QLC_CUDA(cudaFuncSetAttribute(kern3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem3));
        const uint32_t pairs = items < pair_slots(ctx) ? items : pair_slots(ctx);
        prof_begin(ctx, prof_slot);
        QLC_CUDA(launch_pdl(kern3, dim3(2 * pairs), dim3(kThreads3), kSmem3, ctx->stream, tA, tAe, tBe, tOut, args));
        prof_end(ctx);
        ctx->launches += 1;
        QLC_CUDA(cudaGetLastError());
        return QLC_OK;
    }
    prof_begin(ctx, prof_slot);
    QLC_CUDA(launch_pdl(kern, grid, dim3(kThreads2), smem, ctx->stream, tA, tAe, tBe, tOut, args));
    prof_end(ctx);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

// Diagnostics: QLC_ONE_CTA=1 routes the weight GEMMs through the single-CTA kernel.
bool use_paired_ctas() {
    static const bool one = getenv("QLC_ONE_CTA") != nullptr;
    return !one;
}

inline size_t a256(size_t b) { return (b + 255) & ~(size_t)255; }

GemmArgs base_args(qlc_ctx *ctx, const qlc_layer *L) {
    GemmArgs a{};
    if (const qlc_qtensor *q = L->w) {  // (a layer with a plain bf16 weight has no NF4 operand to describe)
        a.codes = q->d_codes;
        a.absmax_codes = q->d_absmax_codes;
        a.absmax2 = q->d_absmax2;
        a.scales_f32 = q->d_scales_f32;
        a.blk_shift = 5;
        while (((size_t)1 << a.blk_shift) < q->block_size) ++a.blk_shift;
        a.dq = q->dq ? 1 : 0;
    }
    a.w_rows = (uint32_t)L->out_dim;
    a.w_cols = (uint32_t)L->in_dim;
    a.splits = 1;
    a.a_rows = 128;
    a.out_scale = 1.0f;
    a.status = ctx->d_status;
    return a;
}

// Number of token splits for the token-contracted gradient products: the largest power of two (at most 16)
// that divides the steps and keeps all CTAs resident at once (`slots` = CTAs the GPU holds at a time).
uint32_t pick_splits(uint32_t token_steps, uint32_t tiles, uint32_t slots) {
    uint32_t s = 1;
    while (s * 2 <= 16 && token_steps % (s * 2) == 0 && tiles * s * 2 <= slots) s *= 2;
    return s;
}

}  // namespace

// Plain tensor-core GEMM on bf16 operands, fp32 (or, with c_bf16, bf16) result: C (M, N) = A (M, K) · op(B), K a multiple of 64.
//   b_is_kn == false: B is (N, K) row-major (C = A·B^T);  b_is_kn == true: B is (K, N) row-major (C = A·B).
// Both operands come through TMA (single-CTA kernel, 256x256 tiles).  Used for the tied LM head of the model.
// ext (optional): `ext_steps` further 64-deep steps appended to the contraction, whose A operand comes through
// *tAe (a (M, 64*ext_steps) bf16 matrix, boxes of 128 rows) and whose B operand through *tBe ((N, 64*ext_steps) with
// boxes of 256 rows when !b_is_kn, (64*ext_steps, N) with boxes of 64 rows when b_is_kn): the LoRA term.
static int umma_gemm_bf16_ext(qlc_ctx *ctx, const __nv_bfloat16 *d_a, const __nv_bfloat16 *d_b, bool b_is_kn, void *d_c,
                              size_t M, size_t N, size_t K, bool c_bf16, const CUtensorMap *tAe, const CUtensorMap *tBe,
                              uint32_t ext_steps, int prof_slot) {
    if (M == 0 || N == 0) return QLC_OK;
    if (K == 0 || K % 64 || N % 32 || M >= (1u << 30) || N >= (1u << 30))
        return fail(QLC_ERR_GPU, "tensor-core GEMM needs K a multiple of 64 and N a multiple of 32 (M %zu, N %zu, K %zu)", M, N, K);
    CUtensorMap tA, tB;
    QLC_TRY(make_map(&tA, d_a, M, K, 128));
    GemmArgs a{};
    a.splits = 1;
    a.a_rows = 256;
    a.out_scale = 1.0f;
    a.status = ctx->d_status;
    a.M = (uint32_t)M;
    a.N = (uint32_t)N;
    a.k_steps = (uint32_t)(K / 64);
    a.ext_steps = ext_steps;
    a.out = d_c;
    a.ldo = (uint32_t)N;
    a.out_bf16 = c_bf16 ? 1 : 0;
    if (!b_is_kn) {
        QLC_TRY(make_map(&tB, d_b, N, K, 256));
        return launch_gemm<256, 2, false, false, false, 3>(ctx, prof_slot, tA, tB, ext_steps ? *tAe : tA, ext_steps ? *tBe : tB, a);
    }
    QLC_TRY(make_map(&tB, d_b, K, N, 64));
    return launch_gemm<256, 2, false, true, false, 3>(ctx, prof_slot, tA, tB, ext_steps ? *tAe : tA, ext_steps ? *tBe : tB, a);
}

int umma_gemm_bf16(qlc_ctx *ctx, const __nv_bfloat16 *d_a, const __nv_bfloat16 *d_b, bool b_is_kn, void *d_c, size_t M,
                   size_t N, size_t K, bool c_bf16) {
    if (M == 0 || N == 0) return QLC_OK;
    if (K == 0 || K % 64 || N % 32 || M >= (1u << 30) || N >= (1u << 30))
        return fail(QLC_ERR_GPU, "tensor-core GEMM needs K a multiple of 64 and N a multiple of 32 (M %zu, N %zu, K %zu)", M, N, K);
    CUtensorMap tA, tB;
    QLC_TRY(make_map(&tA, d_a, M, K, 128));
    GemmArgs a{};
    a.splits = 1;
    a.a_rows = 256;
    a.out_scale = 1.0f;
    a.status = ctx->d_status;
    a.M = (uint32_t)M;
    a.N = (uint32_t)N;
    a.k_steps = (uint32_t)(K / 64);
    a.out = d_c;
    a.ldo = (uint32_t)N;
    a.out_bf16 = c_bf16 ? 1 : 0;  // the result as fp32 or rounded to bf16
    // The persistent paired-CTA kernel takes a plain bf16 B operand as well: its LoRA extension steps fetch both
    // operands by TMA, so a GEMM whose whole contraction is "extension" (no weight steps, the producer warps only
    // pass the stage barriers on) runs with the paired MMAs, the one-wave item walk and the overlapped epilogue.
    static const bool plain_one_cta = getenv("QLC_PLAIN_GEMM_ONE_CTA") != nullptr;  // diagnostics
    if (use_paired_ctas() && !plain_one_cta && N % 64 == 0) {
        GemmArgs p{};
        p.splits = 1;
        p.a_rows = 128;
        p.out_scale = 1.0f;
        p.status = ctx->d_status;
        p.M = (uint32_t)M;
        p.N = (uint32_t)N;
        p.w_rows = b_is_kn ? (uint32_t)K : (uint32_t)N;
        p.w_cols = b_is_kn ? (uint32_t)N : (uint32_t)K;
        p.blk_shift = 6;
        p.k_steps = 0;
        p.ext_steps = (uint32_t)(K / 64);
        p.out = d_c;
        p.ldo = (uint32_t)N;
        p.out_bf16 = c_bf16 ? 1 : 0;
        if (!b_is_kn) {
            QLC_TRY(make_map(&tB, d_b, N, K, 128));
            return launch_gemm2<false>(ctx, 0, tA, tA, tB, p, nullptr);
        }
        QLC_TRY(make_map(&tB, d_b, K, N, 64));
        return launch_gemm2<true>(ctx, 0, tA, tA, tB, p, nullptr);
    }
    if (!b_is_kn) {
        QLC_TRY(make_map(&tB, d_b, N, K, 256));
        return launch_gemm<256, 2, false, false, false, 3>(ctx, 0, tA, tB, tA, tB, a);
    }
    QLC_TRY(make_map(&tB, d_b, K, N, 64));
    return launch_gemm<256, 2, false, true, false, 3>(ctx, 0, tA, tB, tA, tB, a);
}

// Tensor map of a row-major bf16 matrix for other translation units (the attention kernels): `map_out` points
// to a CUtensorMap (128 bytes, 64-byte aligned).
int make_map_bf16(void *map_out, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    return make_map(static_cast<CUtensorMap *>(map_out), base, rows, cols, box_rows);
}

bool pdl_enabled() {
    static const bool on = getenv("QLC_NO_PDL") == nullptr;
    return on;
}

// The fused kernels (weight tile dequantised inside the GEMM) take quantisation blocks of 32, 64, 128 or 256
// elements and dimensions that are multiples of 64; a raw projection needs the same dimensions for its TMA-fed GEMMs.
bool umma_fused_supported(const qlc_layer *L) {
    const bool dims_ok = L->in_dim % 64 == 0 && L->out_dim % 64 == 0 && L->in_dim > 0 && L->out_dim > 0 &&
                         L->in_dim < (1u << 30) && L->out_dim < (1u << 30) && L->r <= (size_t)kMaxRank;
    if (!L->w) return dims_ok;
    const qlc_qtensor *q = L->w;
    const bool block_ok = q->block_size == 32 || q->block_size == 64 || q->block_size == 128 || q->block_size == 256;
    return block_ok && dims_ok;
}
// Every other quantised layer (any block size, any dimensions - the reference's GEMMs take any (m, n, k),
// qlora-wgpu/shaders/gemm.wgsl:14-15) reaches the tensor cores through a padded copy: see shadow_layer.
bool umma_supported(const qlc_layer *L) {
    if (umma_fused_supported(L)) return true;
    return L->w != nullptr && L->in_dim > 0 && L->out_dim > 0 && L->in_dim < (1u << 30) - 64 && L->out_dim < (1u << 30) - 64 &&
           L->r <= (size_t)kMaxRank;
}

// Frees what this file attached to a layer: the padded copy (shadow_layer).
void umma_layer_release(qlc_layer *L) {
    qlc_layer *S = L->shadow;
    if (!S) return;
    cudaFree(S->d_w_raw_bf16);
    cudaFree(S->d_a_pad);
    cudaFree(S->d_b_pad);
    cudaFree(S->d_bt_pad);
    cudaFree(S->d_grad_bucket);
    delete S;
    L->shadow = nullptr;
    L->shadow_valid = false;
}

// out (batch, 64) bf16 = s * Src·Low^T, zero beyond the rank: Src is (batch, cols) activations, Low the
// rank-padded (r_pad, cols) bf16 adapter matrix (A_pad for T1 = X·A^T, B^T_pad for Ds = dY·B).
// Memory-bound (reads the activations once).  The MMA is as narrow as the rank allows (N = 16, 32 or 64)
// so that re-reading the adapter tile by every CTA stays small next to the activation stream, 64-row
// tiles double the CTA count so that every SM pulls from HBM, and four warps issue the MMAs.
// Two jobs (the backward pass needs Ds and T1) go out as one launch whose CTAs are small enough for two
// to share an SM.
struct DownJob {
    const void *src;   // (batch, cols) activations: bf16, or fp32 in TF32 mode
    size_t cols;
    const void *low;   // (r_pad, cols) padded adapter matrix of the same type
    void *out;         // (batch, r_pad) of the same type
};
template <bool TF32>
static int lora_down_slice(qlc_ctx *ctx, qlc_layer *L, size_t batch, const DownJob *jobs, int n_jobs);
// Ranks above 64: the padded rank is covered in slices of 64 columns, one launch (or paired launch) per slice;
// slice s reads rows 64s.. of the padded adapter matrix and writes columns 64s.. of the (batch, r_pad) result.
template <bool TF32>
static int lora_down_t(qlc_ctx *ctx, qlc_layer *L, size_t batch, const DownJob *jobs, int n_jobs) {
    const size_t es = TF32 ? 4 : 2;
    for (size_t sl = 0; sl < L->r_pad / kRankPad; ++sl) {
        DownJob j2[2];
        for (int j = 0; j < n_jobs; ++j) {
            j2[j] = jobs[j];
            j2[j].low = static_cast<const char *>(jobs[j].low) + sl * kRankPad * jobs[j].cols * es;
            j2[j].out = static_cast<char *>(jobs[j].out) + sl * kRankPad * es;
        }
        QLC_TRY(lora_down_slice<TF32>(ctx, L, batch, j2, n_jobs));
    }
    return QLC_OK;
}
template <bool TF32>
static int lora_down_slice(qlc_ctx *ctx, qlc_layer *L, size_t batch, const DownJob *jobs, int n_jobs) {
    const uint32_t nn = L->r <= 16 ? 16u : (L->r <= 32 ? 32u : 64u);
    constexpr uint32_t kStep = TF32 ? 32 : 64;
    CUtensorMap tS[2], tL[2];
    for (int j = 0; j < n_jobs; ++j) {
        QLC_TRY(make_map(&tS[j], jobs[j].src, batch, jobs[j].cols, 64, TF32));
        QLC_TRY(make_map(&tL[j], jobs[j].low, kRankPad, jobs[j].cols, nn, TF32));
    }
    if (n_jobs == 1) {
        tS[1] = tS[0];
        tL[1] = tL[0];
    }
    GemmArgs a = base_args(ctx, L);
    a.a_rows = 64;
    a.M = (uint32_t)batch;
    a.N = nn;
    a.k_steps = (uint32_t)(jobs[0].cols / kStep);
    a.out = jobs[0].out;
    a.ldo = (uint32_t)L->r_pad;
    a.out_bf16 = TF32 ? 0 : 1;
    a.out_pad_cols = kRankPad;
    a.out_scale = L->alpha / (float)L->r;  // lora.rs:64-66
    if (n_jobs == 2) {
        a.pair = 1;
        a.M2 = (uint32_t)batch;
        a.k_steps2 = (uint32_t)(jobs[1].cols / kStep);
        a.out2 = jobs[1].out;
        if (nn == 16) return launch_gemm<16, 1, false, false, false, 4, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
        if (nn == 32) return launch_gemm<32, 1, false, false, false, 4, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
        return launch_gemm<64, 1, false, false, false, 4, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
    }
    if (nn == 16) return launch_gemm<16, 1, false, false, false, 8, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
    if (nn == 32) return launch_gemm<32, 1, false, false, false, 8, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
    return launch_gemm<64, 1, false, false, false, 8, 4, TF32>(ctx, 2, tS[0], tL[0], tS[1], tL[1], a);
}
static int lora_down(qlc_ctx *ctx, qlc_layer *L, size_t batch, const DownJob *jobs, int n_jobs, bool tf32 = false) {
    return tf32 ? lora_down_t<true>(ctx, L, batch, jobs, n_jobs) : lora_down_t<false>(ctx, L, batch, jobs, n_jobs);
}
static int lora_down_x(qlc_ctx *ctx, qlc_layer *L, const __nv_bfloat16 *d_x, size_t batch, __nv_bfloat16 *t1p) {
    const DownJob job{d_x, L->in_dim, L->d_a_pad, t1p};  // T1p = s·X·A^T
    return lora_down(ctx, L, batch, &job, 1);
}

// Token-contracted gradients: final (transposed ? (r, wide) : (wide, r)) fp32 = P^T·Q with P (batch, wide) and
// Q (batch, 64) bf16.  The contraction over the token rows is split over CTAs; each split leaves an fp32
// partial and the last CTA of a tile adds them in split order.  One or two jobs per launch (dA and dB).
struct ContractJob {
    const void *p;   // (batch, wide) activations: bf16, or fp32 in TF32 mode
    size_t wide;
    const void *q;   // (batch, r_pad) of the same type
    int transposed;
    float *out;
};
template <bool TF32>
static int token_contract_slice(qlc_ctx *ctx, qlc_layer *L, size_t batch, const ContractJob *jobs, int n_jobs,
                                float *partial, int accumulate, cudaStream_t stream, size_t sl);
// Ranks above 64: one launch per 64-column slice of Q; slice s produces rows 64s.. of a transposed result
// (dA: (r, wide)) or columns 64s.. of a plain one (dB: (wide, r)).
template <bool TF32>
static int token_contract_t(qlc_ctx *ctx, qlc_layer *L, size_t batch, const ContractJob *jobs, int n_jobs,
                            float *partial, int accumulate, cudaStream_t stream) {
    const size_t es = TF32 ? 4 : 2;
    for (size_t sl = 0; sl * kRankPad < L->r; ++sl) {
        ContractJob j2[2];
        for (int j = 0; j < n_jobs; ++j) {
            j2[j] = jobs[j];
            j2[j].q = static_cast<const char *>(jobs[j].q) + sl * kRankPad * es;
            j2[j].out = jobs[j].out + (jobs[j].transposed ? sl * kRankPad * jobs[j].wide : sl * kRankPad);
        }
        QLC_TRY(token_contract_slice<TF32>(ctx, L, batch, j2, n_jobs, partial, accumulate, stream, sl));
    }
    return QLC_OK;
}
template <bool TF32>
static int token_contract_slice(qlc_ctx *ctx, qlc_layer *L, size_t batch, const ContractJob *jobs, int n_jobs,
                                float *partial, int accumulate, cudaStream_t stream, size_t sl) {
    constexpr uint32_t kStep = TF32 ? 32 : 64;
    const size_t batch_pad = (batch + kStep - 1) / kStep * kStep;  // rows past `batch` read as zeros through TMA
    CUtensorMap tP[2], tQ[2];
    uint32_t tiles = 0, tiles_max = 0;
    for (int j = 0; j < n_jobs; ++j) {
        QLC_TRY(make_map(&tP[j], jobs[j].p, batch, jobs[j].wide, kStep, TF32, TF32));
        QLC_TRY(make_map(&tQ[j], jobs[j].q, batch, kRankPad, kStep, TF32, TF32, L->r_pad));
        const uint32_t t = (uint32_t)ceil_div(jobs[j].wide, 128);
        tiles += t;
        if (t > tiles_max) tiles_max = t;
    }
    if (n_jobs == 1) {
        tP[1] = tP[0];
        tQ[1] = tQ[0];
    }
    GemmArgs a = base_args(ctx, L);
    a.M = (uint32_t)jobs[0].wide;
    a.N = kRankPad;
    a.k_steps = (uint32_t)(batch_pad / kStep);
    a.splits = pick_splits(a.k_steps, tiles, 2u * (uint32_t)ctx->sm_count);  // two CTAs fit on an SM
    a.out = partial;
    a.ldo = kRankPad;
    a.out_bf16 = 0;
    a.final1 = jobs[0].out;
    a.transposed1 = jobs[0].transposed;
    a.cols_used = (uint32_t)(L->r - sl * kRankPad < (size_t)kRankPad ? L->r - sl * kRankPad : (size_t)kRankPad);
    a.final_ld = (uint32_t)L->r;
    a.accumulate = accumulate;
    if (n_jobs == 2) {
        a.pair = 1;
        a.M2 = (uint32_t)jobs[1].wide;
        a.k_steps2 = a.k_steps;
        a.out2 = partial + (size_t)a.splits * jobs[0].wide * kRankPad;
        a.final2 = jobs[1].out;
        a.transposed2 = jobs[1].transposed;
    }
    QLC_TRY(ctx_tile_counters(ctx, 0, 2 * (size_t)tiles_max, &a.counters));
    return launch_gemm<64, 1, true, true, false, 4, 4, TF32>(ctx, 3, tP[0], tQ[0], tP[1], tQ[1], a, stream);
}
static int token_contract(qlc_ctx *ctx, qlc_layer *L, size_t batch, const ContractJob *jobs, int n_jobs,
                          float *partial, int accumulate, cudaStream_t stream, bool tf32 = false) {
    return tf32 ? token_contract_t<true>(ctx, L, batch, jobs, n_jobs, partial, accumulate, stream)
                : token_contract_t<false>(ctx, L, batch, jobs, n_jobs, partial, accumulate, stream);
}

// ---- layers the fused kernels do not take (dimensions that are no multiple of 64, other block sizes) ------------
// Such a layer keeps a PADDED COPY of itself: the dequantised weight rounded to bf16 (the value the fused
// producers would build, quant.rs:157-167 then one rounding) in an (out_pad, in_pad) matrix, and its adapter
// matrices padded the same way, both dimensions rounded up to multiples of 64 with zeros.  Calls then pad the
// activations into scratch buffers, run the plain TMA-fed tensor-core GEMMs (with the LoRA term as extension
// steps) and the side products at the padded size, and copy the real rows and columns out.  The zeros add
// nothing to any product.  Cost: 2 bytes per weight of extra device memory for these layers only, and two
// strided copies per call; the fused path of aligned layers is untouched.
static size_t pad64(size_t v) { return (v + 63) / 64 * 64; }

static int shadow_refresh_adapter(qlc_layer *L) {
    qlc_layer *S = L->shadow;
    if (!S || L->r == 0) return QLC_OK;
    QLC_TRY(launch_pad_to_bf16(L->ctx, L->d_a, L->r, L->in_dim, S->d_a_pad, S->r_pad, S->in_dim));
    QLC_TRY(launch_pad_to_bf16(L->ctx, L->d_b, L->out_dim, L->r, S->d_b_pad, S->out_dim, S->r_pad));
    return launch_pad_transpose_to_bf16(L->ctx, L->d_b, L->out_dim, L->r, S->d_bt_pad, S->r_pad, S->out_dim);
}

static int shadow_layer(qlc_ctx *ctx, qlc_layer *L, qlc_layer **out) {
    if (L->shadow) {
        if (!L->shadow_valid) {
            QLC_TRY(shadow_refresh_adapter(L));
            L->shadow_valid = true;
        }
        *out = L->shadow;
        return QLC_OK;
    }
    const size_t in_pad = pad64(L->in_dim), out_pad = pad64(L->out_dim), n = L->out_dim * L->in_dim;
    qlc_layer *S = new (std::nothrow) qlc_layer();
    if (!S) return fail(QLC_ERR_GPU, "out of host memory");
    S->ctx = L->ctx;  // borrowed: the padded copy lives and dies with its layer and takes no reference
    S->in_dim = in_pad;
    S->out_dim = out_pad;
    S->r = L->r;
    S->alpha = L->alpha;
    S->r_pad = L->r_pad;
    int st = QLC_OK;
    auto chk = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == QLC_OK) st = fail(QLC_ERR_GPU, "%s: %s", what, cudaGetErrorString(e));
    };
    float *wide = nullptr;
    chk(cudaMalloc(reinterpret_cast<void **>(&S->d_w_raw_bf16), (out_pad * in_pad + 8) * 2), "cudaMalloc(padded weight)");
    chk(cudaMalloc(reinterpret_cast<void **>(&wide), (n + 4) * 4), "cudaMalloc(dequantised weight)");
    if (L->r) {
        chk(cudaMalloc(reinterpret_cast<void **>(&S->d_a_pad), (S->r_pad * in_pad + 8) * 2), "cudaMalloc(padded A)");
        chk(cudaMalloc(reinterpret_cast<void **>(&S->d_b_pad), (out_pad * S->r_pad + 8) * 2), "cudaMalloc(padded B)");
        chk(cudaMalloc(reinterpret_cast<void **>(&S->d_bt_pad), (out_pad * S->r_pad + 8) * 2), "cudaMalloc(padded B^T)");
        chk(cudaMalloc(reinterpret_cast<void **>(&S->d_grad_bucket), (L->r * in_pad + out_pad * L->r + 4) * 4), "cudaMalloc(padded gradients)");
    }
    if (st == QLC_OK && L->r)
        chk(cudaMemsetAsync(S->d_grad_bucket, 0, (L->r * in_pad + out_pad * L->r) * 4, L->ctx->stream), "cudaMemsetAsync");
    if (st == QLC_OK) st = launch_dequantize(L->ctx, L->w, wide, QLC_DTYPE_F32);
    if (st == QLC_OK) st = launch_pad_to_bf16(L->ctx, wide, L->out_dim, L->in_dim, S->d_w_raw_bf16, out_pad, in_pad);
    L->shadow = S;
    if (st == QLC_OK) st = shadow_refresh_adapter(L);
    cudaStreamSynchronize(L->ctx->stream);
    cudaFree(wide);
    if (st != QLC_OK) {
        umma_layer_release(L);
        return st;
    }
    L->shadow_valid = true;
    (void)ctx;
    *out = S;
    return QLC_OK;
}

// (rows, cols) -> the top-left corner of a zero-filled (rows, cols_pad) scratch matrix, 2-byte elements
static int pad_rows_bf16(qlc_ctx *ctx, const __nv_bfloat16 *src, size_t rows, size_t cols, size_t cols_pad, __nv_bfloat16 **out) {
    __nv_bfloat16 *p = nullptr;
    QLC_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&p), a256(rows * cols_pad * 2), ctx->stream));
    if (cols_pad != cols) QLC_CUDA(cudaMemsetAsync(p, 0, rows * cols_pad * 2, ctx->stream));
    QLC_CUDA(cudaMemcpy2DAsync(p, cols_pad * 2, src, cols * 2, cols * 2, rows, cudaMemcpyDeviceToDevice, ctx->stream));
    *out = p;
    return QLC_OK;
}

static int shadow_forward(qlc_ctx *ctx, qlc_layer *L, const __nv_bfloat16 *d_x, size_t batch, void *d_y, int y_dtype) {
    qlc_layer *S = nullptr;
    QLC_TRY(shadow_layer(ctx, L, &S));
    const size_t es = y_dtype == QLC_DTYPE_BF16 ? 2 : 4;
    __nv_bfloat16 *xp = nullptr;
    void *yp = nullptr;
    QLC_TRY(pad_rows_bf16(ctx, d_x, batch, L->in_dim, S->in_dim, &xp));
    QLC_CUDA(cudaMallocAsync(&yp, a256(batch * S->out_dim * es), ctx->stream));
    int st = umma_qlora_forward(ctx, S, xp, batch, yp, y_dtype, false);
    if (st == QLC_OK && cudaMemcpy2DAsync(d_y, L->out_dim * es, yp, S->out_dim * es, L->out_dim * es, batch,
                                          cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
        st = fail(QLC_ERR_GPU, "copy out of the padded result failed");
    cudaFreeAsync(xp, ctx->stream);
    cudaFreeAsync(yp, ctx->stream);
    return st;
}

static int shadow_backward(qlc_ctx *ctx, qlc_layer *L, const __nv_bfloat16 *d_x, const __nv_bfloat16 *d_dy, size_t batch,
                           void *d_gx, int gx_dtype, float *d_ga, float *d_gb, int accumulate) {
    qlc_layer *S = nullptr;
    QLC_TRY(shadow_layer(ctx, L, &S));
    const size_t es = gx_dtype == QLC_DTYPE_BF16 ? 2 : 4;
    __nv_bfloat16 *xp = nullptr, *dyp = nullptr;
    void *gxp = nullptr;
    QLC_TRY(pad_rows_bf16(ctx, d_x, batch, L->in_dim, S->in_dim, &xp));
    QLC_TRY(pad_rows_bf16(ctx, d_dy, batch, L->out_dim, S->out_dim, &dyp));
    QLC_CUDA(cudaMallocAsync(&gxp, a256(batch * S->in_dim * es), ctx->stream));
    // padded gradients: (r, in_pad) and (out_pad, r)
    float *gap = (L->r && d_ga) ? S->d_grad_bucket : nullptr;
    float *gbp = (L->r && d_gb) ? S->d_grad_bucket + L->r * S->in_dim : nullptr;
    int st = QLC_OK;
    auto copy2d = [&](void *dst, size_t dpitch, const void *src, size_t spitch, size_t width, size_t rows) {
        if (st == QLC_OK && rows && width &&
            cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, rows, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
            st = fail(QLC_ERR_GPU, "copy to or from a padded buffer failed");
    };
    if (accumulate) {  // the running sums go in, so that the padded products add to them
        if (gap) copy2d(gap, S->in_dim * 4, d_ga, L->in_dim * 4, L->in_dim * 4, L->r);
        if (gbp) copy2d(gbp, L->r * 4, d_gb, L->r * 4, L->r * 4, L->out_dim);
    }
    if (st == QLC_OK) st = umma_qlora_backward(ctx, S, xp, dyp, batch, gxp, gx_dtype, gap, gbp, accumulate, false);
    copy2d(d_gx, L->in_dim * es, gxp, S->in_dim * es, L->in_dim * es, batch);
    if (gap) copy2d(d_ga, L->in_dim * 4, gap, S->in_dim * 4, L->in_dim * 4, L->r);
    if (gbp) copy2d(d_gb, L->r * 4, gbp, L->r * 4, L->r * 4, L->out_dim);
    cudaFreeAsync(xp, ctx->stream);
    cudaFreeAsync(dyp, ctx->stream);
    cudaFreeAsync(gxp, ctx->stream);
    return st;
}

// d_x: (batch, in_dim) bf16, or fp32 when tf32.
int umma_qlora_forward(qlc_ctx *ctx, qlc_layer *L, const void *d_x, size_t batch, void *d_y, int y_dtype, bool tf32) {
    if (batch >= (1u << 31) / 2) return fail(QLC_ERR_GPU, "batch too large for the tensor-core path");
    if (L->w && !umma_fused_supported(L)) {
        if (tf32) return fail(QLC_ERR_GPU, "internal: the padded-copy path has no tf32 form");
        return shadow_forward(ctx, L, static_cast<const __nv_bfloat16 *>(d_x), batch, d_y, y_dtype);
    }
    if (!L->w) {  // plain bf16 weight (a raw projection, or the padded copy of a layer): Y = X·W^T (+ LoRA term)
        if (tf32) return fail(QLC_ERR_GPU, "internal: raw projections have no tf32 path");
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(d_x);
        if (L->r == 0)
            return umma_gemm_bf16(ctx, x, L->d_w_raw_bf16, false, d_y, batch, L->out_dim, L->in_dim, y_dtype == QLC_DTYPE_BF16);
        void *ws = nullptr;
        QLC_TRY(ctx_workspace(ctx, a256(batch * L->r_pad * 2), &ws));
        const DownJob job{x, L->in_dim, L->d_a_pad, ws};  // T1p = s·X·A^T
        QLC_TRY(lora_down(ctx, L, batch, &job, 1, false));
        CUtensorMap tT1, tB;
        QLC_TRY(make_map(&tT1, ws, batch, L->r_pad, 128));
        QLC_TRY(make_map(&tB, L->d_b_pad, L->out_dim, L->r_pad, 256));
        return umma_gemm_bf16_ext(ctx, x, L->d_w_raw_bf16, false, d_y, batch, L->out_dim, L->in_dim, y_dtype == QLC_DTYPE_BF16,
                                  &tT1, &tB, (uint32_t)(L->r_pad / 64), 0);
    }
    if (tf32 && !use_paired_ctas()) return fail(QLC_ERR_GPU, "the TF32 mode needs the paired-CTA kernel");
    if (tf32) QLC_TRY(layer_tf32_operands(L));
    const size_t es = tf32 ? 4 : 2, step = tf32 ? 32 : 64;
    void *ws = nullptr;
    const size_t cut_bytes = use_paired_ctas() ? kcut_bytes(ctx, batch, L->out_dim, L->in_dim / step) : 0;
    const size_t rp = L->r_pad ? L->r_pad : (size_t)kRankPad;  // columns of the rank-padded intermediates
    QLC_TRY(ctx_workspace(ctx, a256(batch * rp * es) + cut_bytes, &ws));
    void *t1p = ws;
    float *split_ws = cut_bytes ? reinterpret_cast<float *>(static_cast<char *>(ws) + a256(batch * rp * es)) : nullptr;
    CUtensorMap tX, tT1, tB;
    QLC_TRY(make_map(&tX, d_x, batch, L->in_dim, 128, tf32));
    GemmArgs a = base_args(ctx, L);
    if (L->r > 0) {
        const DownJob job{d_x, L->in_dim, tf32 ? (const void *)L->d_a_pad32 : (const void *)L->d_a_pad, t1p};  // T1p = s·X·A^T
        QLC_TRY(lora_down(ctx, L, batch, &job, 1, tf32));
        QLC_TRY(make_map(&tT1, t1p, batch, rp, 128, tf32));
        QLC_TRY(make_map(&tB, tf32 ? (const void *)L->d_b_pad32 : (const void *)L->d_b_pad, L->out_dim, L->r_pad,
                         use_paired_ctas() ? 128 : 256, tf32));
        a.ext_steps = (uint32_t)(L->r_pad / step);
    } else {
        tT1 = tX;
        tB = tX;
    }
    a.M = (uint32_t)batch;
    a.N = (uint32_t)L->out_dim;
    a.k_steps = (uint32_t)(L->in_dim / step);
    a.out = d_y;
    a.ldo = (uint32_t)L->out_dim;
    a.out_bf16 = (y_dtype == QLC_DTYPE_BF16);
    if (tf32) return launch_gemm2<false, true>(ctx, 0, tX, tT1, tB, a, split_ws);
    if (use_paired_ctas()) return launch_gemm2<false>(ctx, 0, tX, tT1, tB, a, split_ws);
    a.a_rows = 256;
    return launch_gemm<256, 2, false, false, true, 3>(ctx, 0, tX, tX, tT1, tB, a);
}

// ---- forward pass that allocates nothing -----------------------------------------------------------
// The rank-64-padded LoRA intermediate T1p = s*X*A^T, (rows, 64) bf16, is the forward pass's scratch.
// For callers that must not allocate it lives here, in a fixed device array that every GPU which loads
// this library holds from load until exit (1 MiB): room for kNoAllocMaxRows rows.
// In host code `g_forward_scratch` is only a stand-in for the symbol, not a device address: a kernel
// handed it directly would read the wrong memory.  The real address is looked up once per device with
// cudaGetSymbolAddress (while that device is current) and cached below.
constexpr size_t kNoAllocMaxRows = 8192;
static __device__ __align__(256) unsigned char g_forward_scratch[kNoAllocMaxRows * kRankPad * 2];
constexpr int kMaxDevices = 64;
// per device, filled on the first call on that device; atomic because contexts of several host threads may
// make their first call at the same time (they all store the same value)
static std::atomic<void *> g_forward_scratch_addr[kMaxDevices];

int umma_qlora_forward_noalloc(qlc_ctx *ctx, qlc_layer *L, const __nv_bfloat16 *d_x, size_t batch, void *d_y) {
    if (batch > kNoAllocMaxRows)
        return fail(QLC_ERR_INVALID_CONFIG,
                    "qlc_qlora_forward_dev_noalloc handles at most %zu rows per call (its scratch is a fixed "
                    "%zu-byte device array); got %zu rows - split the batch or use qlc_qlora_forward_dev",
                    kNoAllocMaxRows, sizeof(g_forward_scratch), batch);
    if (L->r > (size_t)kRankPad)
        return fail(QLC_ERR_INVALID_CONFIG, "qlc_qlora_forward_dev_noalloc handles LoRA ranks up to %d (its fixed scratch holds %d "
                    "columns per row); got rank %zu - use qlc_qlora_forward_dev", kRankPad, kRankPad, L->r);
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return fail(QLC_ERR_GPU, "device index %d out of range", ctx->device);
    void *scratch = g_forward_scratch_addr[ctx->device].load(std::memory_order_acquire);
    if (!scratch) {
        // one-time set-up for this device (the caller made it current): resolve the symbol's device address
        QLC_CUDA(cudaGetSymbolAddress(&scratch, g_forward_scratch));
        if (!scratch) return fail(QLC_ERR_GPU, "cudaGetSymbolAddress returned a null address");
        g_forward_scratch_addr[ctx->device].store(scratch, std::memory_order_release);
    }
    __nv_bfloat16 *t1p = static_cast<__nv_bfloat16 *>(scratch);
    CUtensorMap tX, tT1, tB;
    QLC_TRY(make_map(&tX, d_x, batch, L->in_dim, 128));
    GemmArgs a = base_args(ctx, L);
    if (L->r > 0) {
        // Rows [0, batch) x 64 of the scratch are fully rewritten here (columns past the rank receive zeros
        // because the padded A rows are zero) and rows >= batch are never read (the tensor map ends at
        // `batch` rows), so nothing left over from an earlier call can leak into this one.
        QLC_TRY(lora_down_x(ctx, L, d_x, batch, t1p));
        QLC_TRY(make_map(&tT1, t1p, batch, kRankPad, 128));
        QLC_TRY(make_map(&tB, L->d_b_pad, L->out_dim, L->r_pad, use_paired_ctas() ? 128 : 256));
        a.ext_steps = (uint32_t)(L->r_pad / 64);
    } else {
        tT1 = tX;
        tB = tX;
    }
    a.M = (uint32_t)batch;
    a.N = (uint32_t)L->out_dim;
    a.k_steps = (uint32_t)(L->in_dim / 64);
    a.out = d_y;
    a.ldo = (uint32_t)L->out_dim;
    a.out_bf16 = 1;
    if (use_paired_ctas()) return launch_gemm2<false>(ctx, 0, tX, tT1, tB, a, nullptr);  // no scratch for cut tiles
    a.a_rows = 256;
    return launch_gemm<256, 2, false, false, true, 3>(ctx, 0, tX, tX, tT1, tB, a);
}

// d_x, d_dy: bf16, or fp32 when tf32.
int umma_qlora_backward(qlc_ctx *ctx, qlc_layer *L, const void *d_x, const void *d_dy, size_t batch, void *d_gx,
                        int gx_dtype, float *d_ga, float *d_gb, int accumulate, bool tf32) {
    if (batch >= (1u << 31) / 2) return fail(QLC_ERR_GPU, "batch too large for the tensor-core path");
    if (L->w && !umma_fused_supported(L)) {
        if (tf32) return fail(QLC_ERR_GPU, "internal: the padded-copy path has no tf32 form");
        return shadow_backward(ctx, L, static_cast<const __nv_bfloat16 *>(d_x), static_cast<const __nv_bfloat16 *>(d_dy), batch,
                               d_gx, gx_dtype, d_ga, d_gb, accumulate);
    }
    if (!L->w) {  // plain bf16 weight: dX = dY·W (+ Ds·A), and the adapter gradients as in the fused path
        if (tf32) return fail(QLC_ERR_GPU, "internal: raw projections have no tf32 path");
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(d_x), *dy = static_cast<const __nv_bfloat16 *>(d_dy);
        if (L->r == 0)
            return umma_gemm_bf16(ctx, dy, L->d_w_raw_bf16, true, d_gx, batch, L->in_dim, L->out_dim, gx_dtype == QLC_DTYPE_BF16);
        const size_t b_small = a256(batch * L->r_pad * 2);
        const size_t b_part = a256((size_t)16 * (L->in_dim + L->out_dim) * kRankPad * 4);
        void *ws = nullptr;
        QLC_TRY(ctx_workspace(ctx, 2 * b_small + b_part, &ws));
        void *t1p = ws, *dsp = static_cast<char *>(ws) + b_small;
        float *partial = reinterpret_cast<float *>(static_cast<char *>(ws) + 2 * b_small);
        const DownJob down[2] = {{dy, L->out_dim, L->d_bt_pad, dsp}, {x, L->in_dim, L->d_a_pad, t1p}};  // Ds, T1
        QLC_TRY(lora_down(ctx, L, batch, down, d_gb ? 2 : 1, false));
        CUtensorMap tDs, tA;
        QLC_TRY(make_map(&tDs, dsp, batch, L->r_pad, 128));
        QLC_TRY(make_map(&tA, L->d_a_pad, L->r_pad, L->in_dim, 64));
        QLC_TRY(umma_gemm_bf16_ext(ctx, dy, L->d_w_raw_bf16, true, d_gx, batch, L->in_dim, L->out_dim, gx_dtype == QLC_DTYPE_BF16,
                                   &tDs, &tA, (uint32_t)(L->r_pad / 64), 1));
        ContractJob jobs[2];
        int n = 0;
        if (d_ga) jobs[n++] = ContractJob{x, L->in_dim, dsp, 1, d_ga};    // dA = Ds^T·X
        if (d_gb) jobs[n++] = ContractJob{dy, L->out_dim, t1p, 0, d_gb};  // dB = dY^T·T1s
        if (n) QLC_TRY(token_contract(ctx, L, batch, jobs, n, partial, accumulate, ctx->stream, false));
        return QLC_OK;
    }
    if (tf32 && !use_paired_ctas()) return fail(QLC_ERR_GPU, "the TF32 mode needs the paired-CTA kernel");
    if (tf32) QLC_TRY(layer_tf32_operands(L));
    const size_t es = tf32 ? 4 : 2, step = tf32 ? 32 : 64;
    const size_t rp = L->r_pad ? L->r_pad : (size_t)kRankPad;  // columns of the rank-padded intermediates
    const size_t b_small = a256(batch * rp * es);
    const size_t b_part = a256((size_t)16 * (L->in_dim + L->out_dim) * kRankPad * 4);
    // The dX GEMM's last wave is only cut when nothing else would fill it (the gradient contractions do).
    static const bool cut_bwd = getenv("QLC_KCUT_BWD") != nullptr;  // diagnostics
    const bool fill = L->r > 0 && (d_ga || d_gb);
    const size_t cut_bytes = (use_paired_ctas() && (!fill || cut_bwd)) ? kcut_bytes(ctx, batch, L->in_dim, L->out_dim / step) : 0;
    void *ws = nullptr;
    QLC_TRY(ctx_workspace(ctx, 2 * b_small + b_part + cut_bytes, &ws));
    float *split_ws = cut_bytes ? reinterpret_cast<float *>(static_cast<char *>(ws) + 2 * b_small + b_part) : nullptr;
    void *t1p = ws;
    void *dsp = static_cast<char *>(ws) + b_small;
    float *partial = reinterpret_cast<float *>(static_cast<char *>(ws) + 2 * b_small);

    static const bool serial = getenv("QLC_SERIAL_GRADS") != nullptr;  // diagnostics: no side stream
    const bool fork = L->r > 0 && (d_ga || d_gb) && !serial;
    const void *a_pad = tf32 ? (const void *)L->d_a_pad32 : (const void *)L->d_a_pad;
    const void *bt_pad = tf32 ? (const void *)L->d_bt_pad32 : (const void *)L->d_bt_pad;
    CUtensorMap tDY, tDs, tA;
    QLC_TRY(make_map(&tDY, d_dy, batch, L->out_dim, 128, tf32));
    GemmArgs a = base_args(ctx, L);
    if (L->r > 0) {
        // Ds = s·dY·B, and T1 = s·X·A^T recomputed as qlora.rs:145 does (only grad_b needs it)
        const DownJob down[2] = {{d_dy, L->out_dim, bt_pad, dsp}, {d_x, L->in_dim, a_pad, t1p}};
        QLC_TRY(lora_down(ctx, L, batch, down, d_gb ? 2 : 1, tf32));
        if (fork) QLC_CUDA(cudaEventRecord(ctx->ev_fork, ctx->stream));
        QLC_TRY(make_map(&tDs, dsp, batch, rp, 128, tf32));
        QLC_TRY(make_map(&tA, a_pad, L->r_pad, L->in_dim, (uint32_t)step, tf32, tf32));
        a.ext_steps = (uint32_t)(L->r_pad / step);
    } else {
        tDs = tDY;
        tA = tDY;
    }
    a.M = (uint32_t)batch;
    a.N = (uint32_t)L->in_dim;
    a.k_steps = (uint32_t)(L->out_dim / step);
    a.out = d_gx;
    a.ldo = (uint32_t)L->in_dim;
    a.out_bf16 = (gx_dtype == QLC_DTYPE_BF16);
    if (tf32)
        QLC_TRY((launch_gemm2<true, true>(ctx, 1, tDY, tDs, tA, a, split_ws)));  // dX
    else if (use_paired_ctas())
        QLC_TRY(launch_gemm2<true>(ctx, 1, tDY, tDs, tA, a, split_ws));  // dX
    else {
        a.a_rows = 256;
        QLC_TRY((launch_gemm<256, 2, false, true, true, 3>(ctx, 1, tDY, tDY, tDs, tA, a)));
    }
    if (L->r > 0) {
        ContractJob jobs[2];
        int n = 0;
        if (d_ga) jobs[n++] = ContractJob{d_x, L->in_dim, dsp, 1, d_ga};    // dA = Ds^T·X
        if (d_gb) jobs[n++] = ContractJob{d_dy, L->out_dim, t1p, 0, d_gb};  // dB = dY^T·T1s
        if (n && fork) {
            // The gradient contractions only need Ds and T1: they run on the low-priority side stream while the
            // dX GEMM is in flight and take the SMs its last, partial wave leaves idle.
            QLC_CUDA(cudaStreamWaitEvent(ctx->side_stream, ctx->ev_fork, 0));
            QLC_TRY(token_contract(ctx, L, batch, jobs, n, partial, accumulate, ctx->side_stream, tf32));
            QLC_CUDA(cudaEventRecord(ctx->ev_join, ctx->side_stream));
            QLC_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
        } else if (n) {
            QLC_TRY(token_contract(ctx, L, batch, jobs, n, partial, accumulate, ctx->stream, tf32));
        }
    }
    return QLC_OK;
}

}  // namespace qlc
