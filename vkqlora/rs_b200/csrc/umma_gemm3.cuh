// The persistent form of the paired-CTA weight GEMM (included by umma_gemm.cu inside its namespace).
//
// Same arithmetic, operands, tile shape and work-item list as umma_gemm2_kernel, but a CTA pair does not end
// with its tile: the grid is one wave of pairs and pair c works through items c, c + pairs, c + 2*pairs, ...
// What that buys:
//   * barrier initialisation, tensor-memory allocation, the scale table and both cluster synchronisations are
//     paid once per pair instead of once per tile;
//   * the epilogue has warps of its own (four, one per TMEM lane quarter), so the TMA warp and the sixteen
//     producer warps run on into the next item while the accumulators of the finished one are read out,
//     converted and stored.  The two accumulators are handed back one at a time (acc_empty[0], then [1]): the
//     first MMAs of the next item start as soon as accumulator 0 has been read, and by then its first four
//     pipeline stages are already built;
//   * results leave through small slabs of shared memory that belong to the epilogue warps (two 4 KiB slabs per
//     warp, TMA stores), so output traffic is spread over the next item's main loop instead of arriving from all
//     SMs at the end of a wave.
// Barrier phases run on across items: every role walks the same sequence of (item, k-step) and keeps its own
// count of stage uses / finished items, from which stage index and parity follow.
// Every wait is bounded as elsewhere; a failed wait unwinds all roles of the CTA.
#pragma once

// Warp roles: warp 0 = TMA, warp 1 = MMA issue and TMEM owner, warps 2-17 = the sixteen producer warps, warps
// 18-21 = the four epilogue warps (their index modulo 4 covers the four TMEM lane quarters).
constexpr int kCtlWarps3 = 2;
constexpr int kProdWarps3 = 2 * kGroupWarps2;  // two producer groups, alternate k-steps
constexpr int kEpiWarps3 = 4;
constexpr int kThreads3 = 32 * (kCtlWarps3 + kProdWarps3 + kEpiWarps3);
constexpr uint32_t kEpiSlabBytes3 = 4096;  // 32 rows x 64 bf16 columns, 128-byte rows
constexpr uint32_t kEpiBytes3 = kEpiWarps3 * 2 * kEpiSlabBytes3;
constexpr int kBars3 = 2 * kStages2 + 5;  // full[4], empty[4], tmem_full, acc_empty[2], pieces, verdict
constexpr size_t kSmem3 = (size_t)kStages2 * kStageBytes2 + kEpiBytes3 + 8 * kBars3 + 16 + 1024 + 64 + 1024;

struct Item3 {
    bool cut;
    uint32_t n_chunks, cut_tile, chunk;
    uint32_t n0, nh, m0;
    uint32_t k_begin, main_steps, total_steps;
};
__device__ __forceinline__ Item3 decode_item3(const GemmArgs &args, uint32_t item, uint32_t rank) {
    Item3 w;
    w.cut = item >= args.full_items;
    w.n_chunks = w.cut ? args.k_chunks : 1u;
    w.cut_tile = w.cut ? (item - args.full_items) / w.n_chunks : 0u;
    w.chunk = w.cut ? (item - args.full_items) % w.n_chunks : 0u;
    const uint32_t tile = w.cut ? args.full_items + w.cut_tile : item;
    const uint32_t ct = args.row_fastest ? tile / args.row_tiles : tile % args.col_tiles;
    const uint32_t rt = args.row_fastest ? tile % args.row_tiles : tile / args.col_tiles;
    w.n0 = ct * 256u;
    w.nh = w.n0 + rank * 128u;
    w.m0 = (rt * 2u + rank) * (2u * kBM);
    w.k_begin = (uint32_t)(((uint64_t)args.k_steps * w.chunk) / w.n_chunks);
    w.main_steps = (uint32_t)(((uint64_t)args.k_steps * (w.chunk + 1)) / w.n_chunks) - w.k_begin;
    w.total_steps = w.main_steps + (w.chunk + 1 == w.n_chunks ? args.ext_steps : 0u);  // LoRA step: last piece
    return w;
}

// TIMING: the diagnostics build (clock64 sums per role).
template <bool B_MN, bool TF32 = false, bool TIMING = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads3, 1)
umma_gemm3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAext,
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
    const uint32_t epi_base = smem_base + kStages2 * kStageBytes2;
    const uint32_t bar_base = epi_base + kEpiBytes3;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };               // used in the leader CTA only
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages2 + s); };  // one per CTA
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * kStages2);           // one per CTA
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages2 + 1 + a); };  // leader CTA only
    const uint32_t pieces_bar = bar_base + 8u * (2 * kStages2 + 3);   // cut tiles: every epilogue warp stored its partial
    const uint32_t verdict_bar = bar_base + 8u * (2 * kStages2 + 4);  // cut tiles: s_last is valid
    uint8_t *tail = smem_gen + kStages2 * kStageBytes2 + kEpiBytes3 + 8 * kBars3;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 4);
    volatile int *s_last = reinterpret_cast<volatile int *>(tail + 8);
    float *s_q127 = reinterpret_cast<float *>(tail + 16);  // exact (i8 as f32)/127 quotients, 256 entries
    float *s_lev = s_q127 + 256;                           // the 16 NF4 levels (tf32 producers)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    // diagnostics (QLC_GEMM_TIMING): 16 clock64 sums / stamps per CTA
    long long *const tstamp = (TIMING && args.timing) ? args.timing + 16 * (size_t)blockIdx.x : nullptr;
    if (tstamp && threadIdx.x == 0) tstamp[0] = clock64();
    const uint32_t items = args.full_items + (args.k_chunks > 1 ? (args.row_tiles * args.col_tiles - args.full_items) * args.k_chunks : 0u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(full_bar(s), 2 + 2 * kGroupWarps2);  // 2 TMA threads + one producer group per CTA
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, 1);
        mbar_init(acc_empty_bar(0), 2 * kEpiWarps3);  // the epilogue warps of both CTAs
        mbar_init(acc_empty_bar(1), 2 * kEpiWarps3);
        mbar_init(pieces_bar, kEpiWarps3);
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

    if (warp < kCtlWarps3) {
      if (warp == 0) {
        // ---------------- TMA issue (both CTAs; completion is reported to the leader's barrier) -----------
        if (lane == 0) {
            uint32_t g = 0;  // stage uses so far
            bool ok = true;
            for (uint32_t item = pair_id; item < items && ok; item += n_pairs) {
                const Item3 w = decode_item3(args, item, rank);
                for (uint32_t it = 0; it < w.total_steps; ++it, ++g) {
                    const int s = g % kStages2;
                    const uint32_t ph = (g / kStages2) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 31)) {
                        ok = false;
                        break;
                    }
                    const bool ext = it >= w.main_steps;
                    const uint32_t a_dst = smem_base + s * kStageBytes2;
                    const uint32_t b_dst = a_dst + kABytes2;
                    const uint32_t lead_full = mapa_u32(full_bar(s), 0);
                    mbar_arrive_expect_tx_cluster(lead_full, kABytes2 + (ext ? kBBytes2 : 0u));
                    const int kc = ext ? (int)((it - w.main_steps) * kStepElems) : (int)((w.k_begin + it) * kStepElems);
                    const CUtensorMap *ma = ext ? &tmAext : &tmA;
#pragma unroll
                    for (int a = 0; a < 2; ++a)
                        tma_load_2d_pair(a_dst + a * (kBM * 128), ma, lead_full, kc, (int)(w.m0 + a * kBM));
                    if (ext) {
                        if (!B_MN) {
                            tma_load_2d_pair(b_dst, &tmBext, lead_full, kc, (int)w.nh);  // 128 rows of B_pad
                        } else {
#pragma unroll
                            for (int gq = 0; gq < 128 / kAtomElems; ++gq)
                                tma_load_2d_pair(b_dst + gq * kAtomBytes, &tmBext, lead_full, (int)(w.nh + gq * kAtomElems), kc);
                        }
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
            uint32_t g = 0, n_done = 0;
            bool ok = true;
            long long t_full = 0, t_first = 0, t_acc[2] = {0, 0};
            // One thread issues every MMA of the pair: whatever it executes between two MMAs is time the tensor
            // cores may sit idle.  The 64-bit operand descriptors are therefore not rebuilt per instruction: their
            // high words (stride, version, swizzle mode) are constants, and the low word is the stage's base value
            // plus a small multiple of the k-slice (the start-address field counts 16-byte units and never carries
            // into the next field).  Barrier addresses in the peer CTA are looked up once.
            const uint64_t da0 = make_desc(smem_base, 16, 1024);
            const uint64_t db0 = B_MN ? make_desc(smem_base + kABytes2, kAtomBytes, TF32 ? 512u : 1024u, TF32 ? 1u : 2u)
                                      : make_desc(smem_base + kABytes2, 16, 1024);
            const uint32_t da_hi = (uint32_t)(da0 >> 32), da_lo0 = (uint32_t)da0;
            const uint32_t db_hi = (uint32_t)(db0 >> 32), db_lo0 = (uint32_t)db0;
            constexpr uint32_t kStage16 = kStageBytes2 >> 4, kAcc16 = (kBM * 128) >> 4;
            constexpr uint32_t kBk16 = B_MN ? (kMnStep >> 4) : 2u;  // B operand: 16-byte units per k-slice
            uint32_t empty_remote[kStages2][2];
#pragma unroll
            for (int st = 0; st < kStages2; ++st) {
                empty_remote[st][0] = mapa_u32(empty_bar(st), 0);
                empty_remote[st][1] = mapa_u32(empty_bar(st), 1);
            }
            const uint32_t tfull_remote[2] = {mapa_u32(tmem_full_bar, 0), mapa_u32(tmem_full_bar, 1)};
            auto desc64 = [](uint32_t lo, uint32_t hi) {
                uint64_t d;
                asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
                return d;
            };
            for (uint32_t item = pair_id; item < items && ok; item += n_pairs, ++n_done) {
                const Item3 w = decode_item3(args, item, rank);
                uint32_t it = 0;
                while (it < w.total_steps && ok) {
                    // the stage index is a compile-time constant inside this block: the four cases are the same
                    // code with different immediates
#pragma unroll
                    for (int st = 0; st < kStages2; ++st) {
                        if ((g & (kStages2 - 1)) != (uint32_t)st || it >= w.total_steps || !ok) continue;
                        const uint32_t ph = (g / kStages2) & 1u;
                        const long long tw = tstamp ? clock64() : 0;
                        if (!mbar_wait(full_bar(st), ph, abort_flag, args.status, 32)) {
                            ok = false;
                            break;
                        }
                        if (tstamp) (it == 0 ? t_first : t_full) += clock64() - tw;  // waiting for a full stage
                        tc_fence_after();
                        const uint32_t a_lo = da_lo0 + st * kStage16, b_lo = db_lo0 + st * kStage16;
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
                            // the first MMA of an item overwrites accumulator a: both CTAs' epilogue warps must have
                            // read the previous item's values out of it
                            if (it == 0) {
                                const long long ta = tstamp ? clock64() : 0;
                                if (!mbar_wait(acc_empty_bar(a), (n_done & 1u) ^ 1u, abort_flag, args.status, 37)) {
                                    ok = false;
                                    break;
                                }
                                if (tstamp) t_acc[a] += clock64() - ta;  // waiting for the epilogue to hand accumulator a back
                                tc_fence_after();
                            }
#pragma unroll
                            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                                const uint64_t da = desc64(a_lo + a * kAcc16 + kk * 2, da_hi);
                                const uint64_t db = desc64(b_lo + kk * kBk16, db_hi);
                                const uint32_t acc = (kk > 0) ? 1u : (it > 0 ? 1u : 0u);
                                if (TF32)
                                    umma2_tf32(tmem_base + a * BN, da, db, idesc, acc);
                                else
                                    umma2_bf16(tmem_base + a * BN, da, db, idesc, acc);
                            }
                        }
                        if (!ok) break;
                        umma2_commit(empty_remote[st][0]);
                        umma2_commit(empty_remote[st][1]);
                        ++it;
                        ++g;
                    }
                }
                if (ok) {
                    umma2_commit(tfull_remote[0]);
                    umma2_commit(tfull_remote[1]);
                }
            }
            if (tstamp) {
                tstamp[1] = clock64();  // all MMAs issued
                tstamp[2] = t_full;
                tstamp[3] = t_first;
                tstamp[4] = t_acc[0];
                tstamp[5] = t_acc[1];
                tstamp[9] = n_done;
            }
        }
        __syncwarp();
      }
    } else if (warp < kCtlWarps3 + kProdWarps3) {
        // ---------------- weight-tile producers (two groups, alternate stage uses) ----------
        const int group = (warp - kCtlWarps3) / kGroupWarps2;
        const int pt = (threadIdx.x - 32 * kCtlWarps3) & 255;  // thread inside its group
        const int hf = pt & 1;
        uint32_t g0 = 0;  // stage uses before the current item
        bool ok = true;
        long long t_pw = 0;
        for (uint32_t item = pair_id; item < items && ok; item += n_pairs) {
            const Item3 w = decode_item3(args, item, rank);
            const uint32_t first = ((g0 & 1u) == (uint32_t)group) ? 0u : 1u;  // this group's first step of the item
            if constexpr (TF32) {
                // One k-step covers 32 contraction elements: a thread builds 16 fp32 weights (8 bytes of nibbles,
                // half of a quantisation block's share of the step) = four 16-byte chunks of one 128-byte row.
                uint32_t r8, dst_off;
                bool valid;
                size_t e0, e_step;  // first weight element of this thread at k-step 0; elements per k-step
                if (!B_MN) {
                    const int rl = pt >> 1;
                    r8 = rl & 7;
                    dst_off = rl * 128;
                    const size_t row = (size_t)w.nh + rl;
                    valid = row < args.w_rows;
                    e0 = row * args.w_cols + hf * 16;
                    e_step = 32;
                } else {
                    const int pw = pt >> 5, l = pt & 31;
                    const int nl = (pw & 3) * 8 + ((l >> 1) & 7), q = (pw >> 2) * 2 + (l >> 4);
                    r8 = nl & 7;
                    dst_off = q * 4096 + nl * 128;
                    const size_t col = (size_t)w.nh + q * 32;
                    valid = col < args.w_cols;
                    e0 = (size_t)nl * args.w_cols + col + hf * 16;
                    e_step = (size_t)32 * args.w_cols;
                }
                e0 += (size_t)w.k_begin * e_step;
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
                if (valid && first < w.main_steps) fetch(first, nc, nraw, na2);
                for (uint32_t it = first; it < w.total_steps; it += 2) {
                    const uint32_t g = g0 + it;
                    const int s = g % kStages2;
                    const uint32_t ph = (g / kStages2) & 1u;
                    const bool ext = it >= w.main_steps;
                    const uint2 c = nc;
                    const float scale = args.dq ? __fmul_rn(s_q127[nraw & 255u], na2) : na2;  // quant.rs:212-221
                    if (valid && it + 2 < w.main_steps) fetch(it + 2, nc, nraw, na2);
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 33)) {
                        ok = false;
                        break;
                    }
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
                uint32_t r8, dst_off;
                bool valid;
                const uint8_t *code_ptr;    // this thread's 16 bytes of nibbles at k-step 0
                size_t el0;                 // its first element (flat index into the weight) at k-step 0
                size_t code_step, el_step;  // increments per k-step
                if (!B_MN) {
                    // forward: rows = output features nh..nh+127, quantisation block along the contraction
                    const int rl = pt >> 1;
                    r8 = rl & 7;
                    dst_off = rl * 128;
                    const size_t row = (size_t)w.nh + rl;
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
                    const size_t col = (size_t)w.nh + ql * 64;
                    valid = col < args.w_cols;
                    const size_t e = (size_t)nl * args.w_cols + col;
                    code_ptr = args.codes + (e >> 1) + hf * 16;
                    el0 = e + hf * 32;
                    code_step = (size_t)32 * args.w_cols;  // 64 weight rows further down
                    el_step = (size_t)64 * args.w_cols;
                }
                code_ptr += (size_t)w.k_begin * code_step;  // this piece's first k-step
                el0 += (size_t)w.k_begin * el_step;
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
                if (valid && first < w.main_steps) fetch(first, nc, nraw, na2);
                for (uint32_t it = first; it < w.total_steps; it += 2) {
                    const uint32_t g = g0 + it;
                    const int s = g % kStages2;
                    const uint32_t ph = (g / kStages2) & 1u;
                    const bool ext = it >= w.main_steps;
                    const uint4 c = nc;
                    // (code as i8 as f32) / 127 * absmax2[blk / 256]   (quant.rs:212-221); exact quotients from the table
                    const float scale = args.dq ? __fmul_rn(s_q127[nraw & 255u], na2) : na2;
                    if (valid && it + 2 < w.main_steps) fetch(it + 2, nc, nraw, na2);
                    const long long tp = tstamp ? clock64() : 0;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, args.status, 33)) {
                        ok = false;
                        break;
                    }
                    if (tstamp) t_pw += clock64() - tp;  // waiting for an empty stage
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
                        fence_async_smem();  // generic-proxy stores -> visible to the tensor cores' async proxy
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_u32(full_bar(s), 0));
                }
            }
            g0 += w.total_steps;
        }
        if (tstamp && pt == 0 && group == 0) tstamp[10] = t_pw;
    } else {
        // ---------------- epilogue warps: accumulators -> registers -> (bf16: shared-memory slab -> TMA store) --------
        const int ew = warp - (kCtlWarps3 + kProdWarps3);  // 0..3
        const int quarter = warp & 3;             // the TMEM lanes this warp may touch: 32 * quarter .. + 31
        const uint32_t et = (uint32_t)ew * 32u + (uint32_t)lane;  // 0..127: this thread among the epilogue threads
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t slabs = epi_base + (uint32_t)ew * 2u * kEpiSlabBytes3;
        const size_t piece_floats = (size_t)2 * kBM * BN;
        uint32_t n_done = 0, cut_seen = 0, slab_flip = 0;
        long long t_idle = 0, t_rel[2] = {0, 0};
        // hands accumulator a back to the MMA thread (every lane's tcgen05.ld of it has completed)
        auto release_acc = [&](int a) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(acc_empty_bar(a), 0));
        };
        bool ok = true;
        for (uint32_t item = pair_id; item < items && ok; item += n_pairs, ++n_done) {
            const Item3 w = decode_item3(args, item, rank);
            const long long te0 = tstamp ? clock64() : 0;
            if (!mbar_wait(tmem_full_bar, n_done & 1u, abort_flag, args.status, 34)) break;
            const long long te1 = tstamp ? clock64() : 0;
            t_idle += te1 - te0;  // epilogue idle, waiting for accumulators
            tc_fence_after();
            // A piece of a cut tile first leaves its accumulators as an fp32 partial.  The CTA whose partial
            // completes the tile then builds the result from all partials, always adding them in chunk order, so
            // the result does not depend on which piece finished last; the other pieces are done.  Each thread
            // later reads back exactly the addresses the same epilogue thread of the other pieces wrote: float4
            // number q of epilogue thread t at q * 128 + t (fully coalesced), q = (a * 8 + cc / 32) * 8 + j / 4.
            float *const tile_ws = w.cut ? args.split_ws + (size_t)w.cut_tile * w.n_chunks * 2 * piece_floats : nullptr;
            bool finish = true;
            if (w.cut) {
                float4 *mine = reinterpret_cast<float4 *>(tile_ws + ((size_t)w.chunk * 2 + rank) * piece_floats) + et;
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
#pragma unroll 1
                    for (int cc = 0; cc < BN; cc += 32) {
                        uint32_t v[32];
                        tmem_ld32(lane_base + a * BN + cc, v);
                        tmem_ld_wait();
                        float4 *o = mine + (size_t)((a * 8 + cc / 32) * 8) * 128;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            __stcg(o + (j / 4) * 128, make_float4(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]),
                                                                  __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                    }
                    release_acc(a);
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(pieces_bar);
                finish = false;
                if (!mbar_wait(pieces_bar, cut_seen & 1u, abort_flag, args.status, 35)) break;
                if (et == 0) {
                    int *counter = args.counters + w.cut_tile * 2 + rank;
                    const int prev = atomicAdd(counter, 1);
                    const int last = (prev == (int)w.n_chunks - 1) ? 1 : 0;
                    if (last) *counter = 0;  // ready for the next launch
                    *s_last = last;
                    __threadfence();
                    mbar_arrive(verdict_bar);
                }
                if (!mbar_wait(verdict_bar, cut_seen & 1u, abort_flag, args.status, 36)) break;
                finish = *s_last != 0;
                ++cut_seen;
                __syncwarp();
                if (finish) __threadfence();  // the other pieces' partials, announced through the counter
            }
            if (!finish) continue;
            // One 32-column group of row (quarter * 32 + lane) of accumulator a: from tensor memory, or (cut tile)
            // the sum of the pieces' partials in chunk order.
            auto values = [&](int a, int cc, uint32_t (&v)[32]) {
                if (!w.cut) {
                    tmem_ld32(lane_base + a * BN + cc, v);
                    tmem_ld_wait();
                } else {
                    const float4 *src = reinterpret_cast<const float4 *>(tile_ws + (size_t)rank * piece_floats) + et +
                                        (size_t)((a * 8 + cc / 32) * 8) * 128;
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                    for (uint32_t ch = 0; ch < w.n_chunks; ++ch) {
                        const float4 *q = src + (size_t)ch * 2 * (piece_floats / 4);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 f = __ldcg(q + (j / 4) * 128);
                            v[j + 0] = __float_as_uint(__uint_as_float(v[j + 0]) + f.x);
                            v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + f.y);
                            v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + f.z);
                            v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + f.w);
                        }
                    }
                }
            };
            if (args.out_bf16) {
                // 32 rows x 64 columns at a time: bf16 into one of the warp's two slabs (128-byte-swizzled rows), then
                // one TMA store, which writes full 128-byte row segments and clips rows / columns past the matrix.
                const uint32_t r8 = lane & 7;
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
#pragma unroll 1
                    for (int sub = 0; sub < 4; ++sub) {
                        const uint32_t slab = slabs + (slab_flip & 1u) * kEpiSlabBytes3;
                        ++slab_flip;
                        // the store that used this slab two stores ago has been read out of shared memory
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                        const uint32_t row_off = slab + lane * 128;
#pragma unroll
                        for (int cc = 0; cc < 64; cc += 32) {
                            uint32_t v[32];
                            values(a, sub * 64 + cc, v);
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
                        const uint32_t grow = w.m0 + a * kBM + quarter * 32, gcol = w.n0 + sub * 64;
                        if (lane == 0) {
                            if (grow < args.M && gcol < args.N) tma_store_2d(&tmOut, slab, (int)gcol, (int)grow);
                            tma_store_commit();  // one group per slab use, also when nothing was stored
                        }
                    }
                    if (!w.cut) release_acc(a);
                    if (tstamp) t_rel[a] += clock64() - te1;  // accumulators complete -> accumulator a handed back
                }
            } else {
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {
                    const uint32_t row = w.m0 + a * kBM + quarter * 32 + lane;
#pragma unroll 1
                    for (int cc = 0; cc < BN; cc += 32) {
                        uint32_t v[32];
                        values(a, cc, v);
                        const uint32_t gcol = w.n0 + cc;
                        if (row < args.M && gcol < args.N) {
                            float *o = static_cast<float *>(args.out) + (size_t)row * args.ldo + gcol;
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4 *>(o + j) =
                                    make_float4(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]),
                                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        }
                    }
                    if (!w.cut) release_acc(a);
                }
            }
        }
        if (tstamp && et == 0) {
            tstamp[6] = t_idle;
            tstamp[7] = t_rel[0];
            tstamp[8] = t_rel[1];
        }
        // the slabs must stay in place until the TMA engine has read the last stores
        if (lane == 0) tma_store_commit_and_wait_read();
        __syncwarp();
        tc_fence_before();
        (void)ok;
    }

    // Neither CTA may leave while its peer can still touch its shared memory or barriers.
    __syncthreads();
    pause_after_abort(abort_flag);
    cluster_sync_all();
    if (tstamp && threadIdx.x == 0) tstamp[11] = clock64();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}
