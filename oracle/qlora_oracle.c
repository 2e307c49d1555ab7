/*
 * CPU ORACLE — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the arithmetic of the reference's `qlora-core`
 * crate (the numerically-defining implementation of the QloraLinear hot path).
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may link or call this file; the CUDA library never does.
 *
 * Parity pin: the reference is Rust and no Rust toolchain exists on the build
 * machine, so the reference itself cannot be executed.  This restatement is
 * pinned instead by (1) every known-answer / property test the reference's own
 * test-suite holds for this path (ported one-for-one in tests/test_oracle_*.py)
 * and (2) a second, independently written numpy restatement that must agree
 * with this one bit-for-bit (oracle/np_oracle.py).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * `-ffp-contract=off` matters: Rust never fuses a*b+c, so neither may we.
 * No -ffast-math, no flush-to-zero.
 *
 * Every function names the reference lines it follows (paths are relative to
 * the reference repository root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* qlora-core/src/quant.rs:27-44 — NF4 codebook; f64 literals rounded to f32. */
static const float ORC_NF4_LEVELS[16] = {
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
/* quant.rs:47 and :50 */
#define ORC_NF4_ZERO_CODE 7
#define ORC_DOUBLE_QUANT_BLOCK 256

const float *orc_nf4_levels(void) { return ORC_NF4_LEVELS; }

/* Rust `f32::max`: returns the non-NaN operand (C fmaxf has the same rule). */
static inline float rs_max(float a, float b) { return fmaxf(a, b); }

/* Rust `x as i32` for f32: saturating, NaN -> 0. */
static inline int32_t rs_f32_as_i32(float x) {
    if (x != x) return 0;
    if (x >= 2147483648.0f) return INT32_MAX;
    if (x <= -2147483648.0f) return INT32_MIN;
    return (int32_t)x;
}

/* malloc(0) may return NULL; never ask for zero bytes. */
static inline size_t nz(size_t v) { return v ? v : 1; }

static inline int32_t clamp_i32(int32_t v, int32_t lo, int32_t hi) {
    return v < lo ? lo : (v > hi ? hi : v);
}

/* quant.rs:263-278 — 16-way scan, strict `<`, first minimum wins. */
uint8_t orc_nearest_nf4_code(float w, float absmax) {
    if (absmax == 0.0f) return ORC_NF4_ZERO_CODE;
    float target = w / absmax;
    uint8_t best = 0;
    float best_dist = INFINITY;
    for (int i = 0; i < 16; ++i) {
        float d = fabsf(ORC_NF4_LEVELS[i] - target);
        if (d < best_dist) {
            best_dist = d;
            best = (uint8_t)i;
        }
    }
    return best;
}

/* Same scan but on an already divided target (used to derive/verify the
 * threshold table the CUDA kernel uses). */
uint8_t orc_nf4_code_of_target(float target) {
    uint8_t best = 0;
    float best_dist = INFINITY;
    for (int i = 0; i < 16; ++i) {
        float d = fabsf(ORC_NF4_LEVELS[i] - target);
        if (d < best_dist) {
            best_dist = d;
            best = (uint8_t)i;
        }
    }
    return best;
}

/* The scan above for `count` consecutive fp32 bit patterns read as targets, two codes per output byte
 * (pattern first_bits + 2i in the low nibble of out[i]); OpenMP over chunks.  Used by the exhaustive sweep
 * that compares the CUDA kernels' code selection with quant.rs:263-278 for every target in [-1, 1]. */
void orc_nf4_codes_of_target_bits(uint32_t first_bits, size_t count, uint8_t *out, int threads) {
    const ptrdiff_t bytes = (ptrdiff_t)((count + 1) / 2);
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (ptrdiff_t b = 0; b < bytes; ++b) {
        uint8_t v = 0;
        for (int h = 0; h < 2; ++h) {
            const size_t i = 2 * (size_t)b + (size_t)h;
            if (i >= count) break;
            const uint32_t bits = first_bits + (uint32_t)i;
            float t;
            memcpy(&t, &bits, 4);
            v |= (uint8_t)(orc_nf4_code_of_target(t) << (4 * h));
        }
        out[b] = v;
    }
}

/* quant.rs:283-299 — int8 double quantisation of the block scales. */
void orc_double_quantize_scales(const float *scales, size_t nb, uint8_t *codes, float *absmax2) {
    size_t nsb = (nb + ORC_DOUBLE_QUANT_BLOCK - 1) / ORC_DOUBLE_QUANT_BLOCK;
    for (size_t sb = 0; sb < nsb; ++sb) {
        size_t s = sb * ORC_DOUBLE_QUANT_BLOCK;
        size_t e = s + ORC_DOUBLE_QUANT_BLOCK < nb ? s + ORC_DOUBLE_QUANT_BLOCK : nb;
        float amax = 0.0f;
        for (size_t i = s; i < e; ++i) amax = rs_max(amax, fabsf(scales[i]));
        absmax2[sb] = amax;
        for (size_t i = s; i < e; ++i) {
            int8_t q;
            if (amax == 0.0f) {
                q = 0;
            } else {
                float v = roundf(scales[i] / amax * 127.0f); /* Rust round: half away from zero */
                q = (int8_t)clamp_i32(rs_f32_as_i32(v), -127, 127);
            }
            codes[i] = (uint8_t)q;
        }
    }
}

/* quant.rs:104-154 — flat blocks over the row-major buffer, short last block.
 * codes: ceil(n/2) bytes (zeroed here). scales_f32: nb floats (always written).
 * If double_quant != 0, absmax_codes (nb) and absmax2 (ceil(nb/256)) are written too. */
void orc_quantize_nf4(const float *w, size_t n, size_t block_size, int double_quant, uint8_t *codes,
                      float *scales_f32, uint8_t *absmax_codes, float *absmax2) {
    size_t nb = (n + block_size - 1) / block_size;
    memset(codes, 0, (n + 1) / 2);
    for (size_t b = 0; b < nb; ++b) {
        size_t s = b * block_size;
        size_t e = s + block_size < n ? s + block_size : n;
        float absmax = 0.0f;
        for (size_t i = s; i < e; ++i) absmax = rs_max(absmax, fabsf(w[i]));
        scales_f32[b] = absmax;
        for (size_t i = s; i < e; ++i) {
            uint8_t code = orc_nearest_nf4_code(w[i], absmax);
            if ((i & 1) == 0)
                codes[i / 2] |= code;
            else
                codes[i / 2] |= (uint8_t)(code << 4);
        }
    }
    if (double_quant) orc_double_quantize_scales(scales_f32, nb, absmax_codes, absmax2);
}

/* quant.rs:212-221 (Int8 arm): (c as i8 as f32) / 127.0 * absmax[i / 256]. */
void orc_block_scales_dq(const uint8_t *absmax_codes, const float *absmax2, size_t nb, float *out) {
    for (size_t i = 0; i < nb; ++i)
        out[i] = (float)(int8_t)absmax_codes[i] / 127.0f * absmax2[i / ORC_DOUBLE_QUANT_BLOCK];
}

/* quant.rs:157-167 — one fp32 multiply per element. */
void orc_dequantize(const uint8_t *codes, const float *scales, size_t n, size_t block_size, float *out) {
    for (size_t idx = 0; idx < n; ++idx) {
        uint8_t byte = codes[idx / 2];
        uint8_t code = (idx & 1) == 0 ? (byte & 0x0F) : (byte >> 4);
        out[idx] = ORC_NF4_LEVELS[code] * scales[idx / block_size];
    }
}

/* lora.rs:129-142 — C = A·B, i-p-j order, accumulate into C.  `threads` > 1
 * splits output rows across OpenMP threads (per-element arithmetic order is
 * unchanged, so results are identical for any thread count). */
void orc_matmul(const float *a, const float *b, size_t m, size_t k, size_t n, float *c, int threads) {
    memset(c, 0, m * n * sizeof(float));
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t p = 0; p < k; ++p) {
            float a_ip = a[i * k + p];
            for (size_t j = 0; j < n; ++j) c[i * n + j] += a_ip * b[p * n + j];
        }
    }
}

/* lora.rs:148-162 — C(k,n) = A(m,k)^T · B(m,n); sequential dot over p. */
void orc_matmul_trans_a(const float *a, const float *b, size_t m, size_t k, size_t n, float *c, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)k; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (size_t p = 0; p < m; ++p) acc += a[p * k + i] * b[p * n + j];
            c[i * n + j] = acc;
        }
    }
}

/* lora.rs:169-183 — C(m,n) = A(m,k) · B(n,k)^T; sequential dot over p. */
void orc_matmul_trans_b(const float *a, const float *b, size_t m, size_t k, size_t n, float *c, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (size_t p = 0; p < k; ++p) acc += a[i * k + p] * b[j * k + p];
            c[i * n + j] = acc;
        }
    }
}

/* lora.rs:64-66 */
float orc_lora_scale(float alpha, size_t r) { return alpha / (float)r; }

/* lora.rs:86-103 — T1 = X·A^T, T2 = T1·B^T, T2 *= s (scale applied last). */
void orc_lora_forward(const float *x, size_t batch, const float *a, const float *b, size_t in_dim,
                      size_t out_dim, size_t r, float alpha, float *out, int threads) {
    float *t1 = (float *)malloc(nz(batch * r) * sizeof(float));
    orc_matmul_trans_b(x, a, batch, in_dim, r, t1, threads);
    orc_matmul_trans_b(t1, b, batch, r, out_dim, out, threads);
    float s = orc_lora_scale(alpha, r);
    for (size_t i = 0; i < batch * out_dim; ++i) out[i] *= s;
    free(t1);
}

/* qlora.rs:86-107 — Y = X·deq(W)^T (+ adapter term added elementwise).
 * w_deq is the dequantised (out_dim, in_dim) weight; r == 0 means no adapter. */
void orc_qlora_forward(const float *x, size_t batch, const float *w_deq, size_t out_dim, size_t in_dim,
                       const float *a, const float *b, size_t r, float alpha, float *y, int threads) {
    orc_matmul_trans_b(x, w_deq, batch, in_dim, out_dim, y, threads);
    if (r > 0) {
        float *d = (float *)malloc(nz(batch * out_dim) * sizeof(float));
        orc_lora_forward(x, batch, a, b, in_dim, out_dim, r, alpha, d, threads);
        for (size_t i = 0; i < batch * out_dim; ++i) y[i] += d[i];
        free(d);
    }
}

/* qlora.rs:116-165 — grad_x = dY·W (+ Ds·A); grad_b = dYs^T·T1; grad_a = Ds^T·X.
 * grad_a / grad_b are only written when r > 0. */
void orc_qlora_backward(const float *x, const float *dy, size_t batch, const float *w_deq, size_t out_dim,
                        size_t in_dim, const float *a, const float *b, size_t r, float alpha, float *grad_x,
                        float *grad_a, float *grad_b, int threads) {
    orc_matmul(dy, w_deq, batch, out_dim, in_dim, grad_x, threads);
    if (r == 0) return;
    float s = orc_lora_scale(alpha, r);
    size_t n_dy = batch * out_dim;
    float *dys = (float *)malloc(nz(n_dy) * sizeof(float));
    for (size_t i = 0; i < n_dy; ++i) dys[i] = dy[i] * s;
    float *t1 = (float *)malloc(nz(batch * r) * sizeof(float));
    orc_matmul_trans_b(x, a, batch, in_dim, r, t1, threads);
    orc_matmul_trans_a(dys, t1, batch, out_dim, r, grad_b, threads);
    float *ds = (float *)malloc(nz(batch * r) * sizeof(float));
    orc_matmul(dys, b, batch, out_dim, r, ds, threads);
    orc_matmul_trans_a(ds, x, batch, r, in_dim, grad_a, threads);
    float *dx_lora = (float *)malloc(nz(batch * in_dim) * sizeof(float));
    orc_matmul(ds, a, batch, r, in_dim, dx_lora, threads);
    for (size_t i = 0; i < batch * in_dim; ++i) grad_x[i] += dx_lora[i];
    free(dys);
    free(t1);
    free(ds);
    free(dx_lora);
}

/* optim.rs:84-94 */
float orc_quantize_block_i8(const float *x, size_t len, uint8_t *codes) {
    float absmax = 0.0f;
    for (size_t i = 0; i < len; ++i) absmax = rs_max(absmax, fabsf(x[i]));
    if (absmax == 0.0f) {
        memset(codes, 0, len);
        return 0.0f;
    }
    for (size_t i = 0; i < len; ++i) {
        float v = roundf(x[i] / absmax * 127.0f);
        codes[i] = (uint8_t)(int8_t)clamp_i32(rs_f32_as_i32(v), -127, 127);
    }
    return absmax;
}

/* optim.rs:96-100 */
void orc_dequant_block_i8(const uint8_t *codes, float absmax, float *out, size_t len) {
    for (size_t i = 0; i < len; ++i) out[i] = (float)(int8_t)codes[i] / 127.0f * absmax;
}

/* optim.rs:206-248 — one tensor's step.  `*step` is the tensor's step counter
 * (incremented here).  Returns the number of blocks streamed. */
size_t orc_adam8bit_step_param(float lr, float beta1, float beta2, float eps, size_t block_size,
                               size_t max_resident_pages, uint64_t *step, size_t numel, uint8_t *m_codes,
                               float *m_scales, uint8_t *v_codes, float *v_scales, float *p, const float *g) {
    size_t num_blocks = (numel + block_size - 1) / block_size;
    *step += 1;
    float t = (float)*step;
    float b1t = 1.0f - powf(beta1, t);
    float b2t = 1.0f - powf(beta2, t);
    size_t window = max_resident_pages < num_blocks ? max_resident_pages : num_blocks;
    if (window < 1) window = 1;
    size_t streamed = 0;
    float *m = (float *)malloc(block_size * sizeof(float));
    float *v = (float *)malloc(block_size * sizeof(float));
    for (size_t block_start = 0; block_start < num_blocks; block_start += window) {
        size_t block_end = block_start + window < num_blocks ? block_start + window : num_blocks;
        for (size_t blk = block_start; blk < block_end; ++blk) {
            size_t s = blk * block_size;
            size_t e = s + block_size < numel ? s + block_size : numel;
            size_t len = e - s;
            orc_dequant_block_i8(m_codes + s, m_scales[blk], m, len);
            orc_dequant_block_i8(v_codes + s, v_scales[blk], v, len);
            for (size_t j = 0; j < len; ++j) {
                float gj = g[s + j];
                m[j] = beta1 * m[j] + (1.0f - beta1) * gj;
                float var = beta2 * v[j] * v[j] + (1.0f - beta2) * gj * gj;
                v[j] = sqrtf(var);
                float mh = m[j] / b1t;
                float vh = var / b2t;
                p[s + j] -= lr * mh / (sqrtf(vh) + eps);
            }
            m_scales[blk] = orc_quantize_block_i8(m, len, m_codes + s);
            v_scales[blk] = orc_quantize_block_i8(v, len, v_codes + s);
            streamed += 1;
        }
    }
    free(m);
    free(v);
    return streamed;
}

/* glibc powf-based bias corrections for step t, exactly as optim.rs:207-210;
 * exported so tests can compare against what the CUDA host code computes. */
void orc_adam_bias_corrections(float beta1, float beta2, uint64_t step, float *b1t, float *b2t) {
    float t = (float)step;
    *b1t = 1.0f - powf(beta1, t);
    *b2t = 1.0f - powf(beta2, t);
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
