/*
 * gt_oracle.c — CPU restatement of the Glacier.Tune frozen-base K-quant projection path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared against and
 * the timed CPU baseline of the benchmark.  Nothing in the shipped library links, loads or calls
 * it; the product path has no CPU fallback.
 *
 * The reference is C# (.NET 10) with three un-vendored NuGet dependencies and cannot be built
 * in an image without a .NET SDK, so every routine here restates the reference algorithm from
 * the cited lines.  Paths are relative to the reference project root.
 *
 * Pinning status:
 *   Q4_K  — pinned by the reference's own known answers: the exhaustive Set/GetScaleMinK4
 *           round trip (tests/Glacier.Tune.Tests/AdversarialQuantizationTests.cs:15-60), the
 *           constant-block fixture (tests/Glacier.Tune.Tests/SyntheticGgufFixture.cs:407-413)
 *           and quantize->dequantize fidelity against the in-repo quantizer
 *           (src/Glacier.Tune/Export/GgufMerger.cs:666-757,
 *            tests/Glacier.Tune.Tests/GgufMergerQuantizationTests.cs:118-191), which fixes the
 *           nibble order.
 *   Q6_K  — the reference holds no test, fixture or CPU source for Q6_K (the only statement of the layout in it is
 *           the CUDA kernel src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:263-332); pinned against the format's own
 *           implementation instead: gguf.quants.dequantize (package gguf 0.19.0) on seeded blocks, bit for bit, with
 *           the generating script and its outputs in tests/golden/ (make_gguf_golden.py, gguf_dequant_golden.npz).
 *           The same fixture pins Q4_K a second time.
 *   LoRA  — pinned by tests/Glacier.Tune.Tests/KernelTests.cs:133-202 (fast path vs naive, 1e-4).
 *   QuantKernels.MatMulBatch / ExtractEmbedding live in Glacier.Inference 1.8.0 (not vendored):
 *           restated here as exact-dequant fp32 GEMM / row dequant, which is what the
 *           reference's CPU-vs-GPU parity test ties them to
 *           (tests/Glacier.Tune.Tests/GradientAndGpuParityTests.cs:174-260).
 *   Layer glue — SwiGLU and RoPE restate in-repo sources (src/Glacier.Tune/Kernels/SwiGluKernel.cs,
 *           RoPEKernel.cs); the reference holds no known answers for them, the tests pin them by
 *           closed forms, finite differences and the rotation's inverse, and by the Qwen2 operators
 *           of the `transformers` package (rotate-half RoPE, SiLU * up; tests/test_oracle_pins_qwen2.py).
 *           RMSNorm lives in Glacier.Tensor 1.1.0 (not vendored): textbook definition, PARITY UNPINNED
 *           against the reference; pinned, forward and backward, to `Qwen2RMSNorm` of transformers
 *           5.5.0 - the definition of the architecture the workload names (same test file).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GT_QK_K 256
#define GT_Q4K_BLOCK_BYTES 144 /* half d; half dmin; u8 scales[12]; u8 qs[128]  (tune_bwd.cu:28-33) */
#define GT_Q6K_BLOCK_BYTES 210 /* u8 ql[128]; u8 qh[64]; i8 scales[16]; half d  (tune_bwd.cu:35-40) */

/* ggml type ids used by the reference's GgufType enum for the types on this path */
#define GT_TYPE_F32 0
#define GT_TYPE_F16 1
#define GT_TYPE_Q4_0 2
#define GT_TYPE_Q8_0 8
#define GT_TYPE_Q4_K 12
#define GT_TYPE_Q6_K 14

#if defined(__GNUC__) && defined(__x86_64__)
#define GT_CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))
#else
#define GT_CLONES
#endif

int gt_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void gt_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* IEEE binary16 -> binary32, exact, subnormals included. */
static inline float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

float gt_oracle_half_to_float(uint16_t h) { return half_bits_to_float(h); }

/* binary32 -> binary16, round to nearest even (matches C# (Half)float). */
uint16_t gt_oracle_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e;
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) out++;
    return out;
}

/* 6-bit scale/min unpack: src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:43-51,
 * src/Glacier.Tune/Export/GgufMerger.cs:781-793. */
void gt_oracle_get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* Inverse packing: src/Glacier.Tune/Export/GgufMerger.cs:765-778. */
void gt_oracle_set_scale_min_k4(int j, uint8_t *scales, uint8_t sc, uint8_t m) {
    if (j < 4) {
        scales[j] = (uint8_t)((scales[j] & 0xC0) | (sc & 0x3F));
        scales[j + 4] = (uint8_t)((scales[j + 4] & 0xC0) | (m & 0x3F));
    } else {
        scales[j + 4] = (uint8_t)((sc & 0x0F) | ((m & 0x0F) << 4));
        scales[j - 4] = (uint8_t)((scales[j - 4] & 0x3F) | ((sc >> 4) << 6));
        scales[j] = (uint8_t)((scales[j] & 0x3F) | ((m >> 4) << 6));
    }
}

/* One Q4_K super-block -> 256 fp32 weights.
 * Element decode: tune_bwd.cu:209-211,234-240:
 *   ib = c>>5; qs_idx = (ib>>1)*32 + (c&31); shift = (ib&1)*4;
 *   w = (f32(d)*sc_ib)*nib - (f32(dmin)*m_ib)                                       */
static void dequant_block_q4k(const uint8_t *blk, float *dst) {
    uint16_t hd, hm;
    memcpy(&hd, blk, 2);
    memcpy(&hm, blk + 2, 2);
    const float d = half_bits_to_float(hd);
    const float dmin = half_bits_to_float(hm);
    const uint8_t *scales = blk + 4;
    const uint8_t *qs = blk + 16;
    for (int ib = 0; ib < 8; ib++) {
        uint8_t sc, m;
        gt_oracle_get_scale_min_k4(ib, scales, &sc, &m);
        const float d_sub = d * (float)sc;
        const float m_sub = dmin * (float)m;
        const uint8_t *q = qs + (ib >> 1) * 32;
        const int shift = (ib & 1) * 4;
        for (int l = 0; l < 32; l++) {
            const float nib = (float)((q[l] >> shift) & 0x0F);
            dst[ib * 32 + l] = d_sub * nib - m_sub;
        }
    }
}

/* One Q6_K super-block -> 256 fp32 weights.  tune_bwd.cu:279-289,311-315. */
static void dequant_block_q6k(const uint8_t *blk, float *dst) {
    const uint8_t *ql = blk;
    const uint8_t *qh = blk + 128;
    const int8_t *scales = (const int8_t *)(blk + 192);
    uint16_t hd;
    memcpy(&hd, blk + 208, 2);
    const float d = half_bits_to_float(hd);
    for (int c = 0; c < 256; c++) {
        const int step = c >> 7, rem = c & 127, quad = rem >> 5, lane = rem & 31;
        const int ql_idx = step * 64 + (quad & 1) * 32 + lane;
        const int ql_shift = quad >= 2 ? 4 : 0;
        const int qh_idx = step * 32 + lane;
        const int qh_shift = quad * 2;
        const int sc_idx = step * 8 + (lane >> 4) + quad * 2;
        const int q = (int)(((ql[ql_idx] >> ql_shift) & 0x0F) | (((qh[qh_idx] >> qh_shift) & 0x03) << 4)) - 32;
        dst[c] = d * (float)scales[sc_idx] * (float)q;
    }
}

int64_t gt_oracle_block_bytes(int type) {
    if (type == GT_TYPE_Q4_K) return GT_Q4K_BLOCK_BYTES;
    if (type == GT_TYPE_Q6_K) return GT_Q6K_BLOCK_BYTES;
    return 0;
}

/* Q4_0 (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:23-26,151-163): 32 weights in 18 bytes, half d then 16 bytes; weight i is
 * d * (nibble - 8) with the low nibble of qs[i] for i < 16 and the high nibble of qs[i - 16] otherwise.
 * Q8_0 (tune_bwd.cu:18-21,375-376): 32 weights in 34 bytes, half d then 32 int8; weight i is d * qs[i].
 * The reference holds no test or fixture for either; both are pinned against gguf.quants.dequantize (tests/golden). */
static void dequant_block_q40(const uint8_t *blk, float *dst) {
    const float d = half_bits_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
    for (int i = 0; i < 32; i++) {
        const int q = (int)((blk[2 + (i & 15)] >> ((i >> 4) << 2)) & 0x0F) - 8;
        dst[i] = d * (float)q;
    }
}
static void dequant_block_q80(const uint8_t *blk, float *dst) {
    const float d = half_bits_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
    for (int i = 0; i < 32; i++) dst[i] = d * (float)(int8_t)blk[2 + i];
}

/* tensor types the row-wise routines accept: F32, F16 (plain rows), the two K-quants, Q4_0 and Q8_0 */
static int type_ok(int type) {
    return type == GT_TYPE_F32 || type == GT_TYPE_F16 || type == GT_TYPE_Q4_0 || type == GT_TYPE_Q8_0 || gt_oracle_block_bytes(type) != 0;
}

/* Dequantize `nblocks` consecutive super-blocks (a flat stream). */
int gt_oracle_dequant_blocks(int type, const uint8_t *blocks, int64_t nblocks, float *dst) {
    const int64_t bb = gt_oracle_block_bytes(type);
    if (bb == 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; b++) {
        if (type == GT_TYPE_Q4_K)
            dequant_block_q4k(blocks + b * bb, dst + b * GT_QK_K);
        else
            dequant_block_q6k(blocks + b * bb, dst + b * GT_QK_K);
    }
    return 0;
}

/* Row dequantize: the role of QuantKernels.ExtractEmbedding(type, W, row, dst, K)
 * (call sites src/Glacier.Tune/Kernels/LoraKernels.BaseBackward.cs:117,125).
 * The weight tensor is the row-major [rows, K] element stream cut into 256-element super-blocks;
 * for K % 256 == 0 that is ordinary row-aligned GGUF, otherwise (K % 32 == 0) a row may start in
 * the middle of a super-block shared with its neighbour. */
static void dequant_row(int type, const uint8_t *w, int64_t row, int K, float *dst) {
    const int64_t bb = gt_oracle_block_bytes(type);
    if (type == GT_TYPE_F32) {
        memcpy(dst, (const float *)w + row * K, (size_t)K * 4);
        return;
    }
    if (type == GT_TYPE_F16) {
        const uint16_t *h = (const uint16_t *)w + row * K;
        for (int k = 0; k < K; k++) dst[k] = half_bits_to_float(h[k]);
        return;
    }
    if (type == GT_TYPE_Q4_0 || type == GT_TYPE_Q8_0) {      /* K % 32 == 0: rows are whole 32-weight blocks */
        const int64_t b32 = type == GT_TYPE_Q4_0 ? 18 : 34;
        const uint8_t *r = w + row * (int64_t)(K / 32) * b32;
        for (int b = 0; b < K / 32; b++) {
            if (type == GT_TYPE_Q4_0) dequant_block_q40(r + b * b32, dst + b * 32);
            else dequant_block_q80(r + b * b32, dst + b * 32);
        }
        return;
    }
    int64_t e0 = row * (int64_t)K;
    int64_t b0 = e0 / GT_QK_K, b1 = (e0 + K - 1) / GT_QK_K;
    float tmp[GT_QK_K];
    for (int64_t b = b0; b <= b1; b++) {
        int64_t lo = b * GT_QK_K, hi = lo + GT_QK_K;
        if (lo >= e0 && hi <= e0 + K) {
            if (type == GT_TYPE_Q4_K)
                dequant_block_q4k(w + b * bb, dst + (lo - e0));
            else
                dequant_block_q6k(w + b * bb, dst + (lo - e0));
        } else {
            if (type == GT_TYPE_Q4_K)
                dequant_block_q4k(w + b * bb, tmp);
            else
                dequant_block_q6k(w + b * bb, tmp);
            int64_t s = lo > e0 ? lo : e0, t = hi < e0 + K ? hi : e0 + K;
            memcpy(dst + (s - e0), tmp + (s - lo), (size_t)(t - s) * 4);
        }
    }
}

int gt_oracle_dequant_rows(int type, const uint8_t *w, int K, int64_t row0, int64_t nrows, float *dst) {
    if (!type_ok(type)) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < nrows; r++) dequant_row(type, w, row0 + r, K, dst + r * (int64_t)K);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * Q4_K quantizer (test infrastructure: builds fixtures the way the reference's tests do).
 * src/Glacier.Tune/Export/GgufMerger.cs:666-757.  MathF.Round is round-half-to-even.
 * ------------------------------------------------------------------------------------------- */
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

void gt_oracle_quantize_row_q4k(const float *src, uint8_t *dst, int n) {
    const int nsb = n / GT_QK_K;
    for (int sb = 0; sb < nsb; sb++) {
        const float *s = src + sb * GT_QK_K;
        uint8_t *blk = dst + (size_t)sb * GT_Q4K_BLOCK_BYTES;
        float sub_scale[8], sub_min[8];
        uint8_t sc[8], m[8], L[256];
        float max_scale = 0.f, max_min = 0.f;
        for (int ib = 0; ib < 8; ib++) {
            const float *b = s + ib * 32;
            float bmin = b[0], bmax = b[0];
            for (int i = 1; i < 32; i++) {
                if (b[i] < bmin) bmin = b[i];
                if (b[i] > bmax) bmax = b[i];
            }
            if (bmin > 0.f) bmin = 0.f;
            sub_scale[ib] = (bmax - bmin) / 15.0f;
            if (sub_scale[ib] > max_scale) max_scale = sub_scale[ib];
            sub_min[ib] = -bmin;
            if (sub_min[ib] > max_min) max_min = sub_min[ib];
        }
        const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        for (int ib = 0; ib < 8; ib++) {
            sc[ib] = (uint8_t)clampi((int)rintf(sub_scale[ib] * inv_scale), 0, 63);
            m[ib] = (uint8_t)clampi((int)rintf(sub_min[ib] * inv_min), 0, 63);
        }
        memset(blk + 4, 0, 12);
        for (int j = 0; j < 8; j++) gt_oracle_set_scale_min_k4(j, blk + 4, sc[j], m[j]);
        uint16_t hd = gt_oracle_float_to_half(max_scale / 63.0f);
        uint16_t hm = gt_oracle_float_to_half(max_min / 63.0f);
        memcpy(blk, &hd, 2);
        memcpy(blk + 2, &hm, 2);
        const float d_super = half_bits_to_float(hd), dmin_super = half_bits_to_float(hm);
        for (int ib = 0; ib < 8; ib++) {
            const float d = d_super * sc[ib], dm = dmin_super * m[ib];
            const float inv_d = d > 0.f ? 1.0f / d : 0.f;
            for (int i = 0; i < 32; i++) {
                int q = inv_d > 0.f ? (int)rintf((s[ib * 32 + i] + dm) * inv_d) : 0;
                L[ib * 32 + i] = (uint8_t)clampi(q, 0, 15);
            }
        }
        uint8_t *qd = blk + 16;
        for (int g = 0; g < 256; g += 64) {
            for (int l = 0; l < 32; l++) qd[l] = (uint8_t)(L[g + l] | (L[g + l + 32] << 4));
            qd += 32;
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * Forward base GEMM: Y[s,o] = sum_k X[s,k] * W[o,k] (+ bias[o]).
 * Role of QuantKernels.MatMulBatch(type, W, X, Y, K, N, T) + the bias loop at
 * src/Glacier.Tune/Model/LoraAdapter.cs:139-152; same contract as the fp32 twin kernel
 * src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:83-128.  fp32 accumulation (timed baseline).
 * ------------------------------------------------------------------------------------------- */
GT_CLONES
static void dot_rows_f32(const float *x, const float *wt, int K, int nr, float *out, int64_t out_stride) {
    for (int r = 0; r < nr; r++) {
        const float *w = wt + (int64_t)r * K;
        float acc = 0.f;
#pragma omp simd reduction(+ : acc)
        for (int k = 0; k < K; k++) acc += x[k] * w[k];
        out[r * out_stride] = acc;
    }
}

int gt_oracle_matmul_batch(int type, const uint8_t *w, const float *x, float *y, int K, int N, int T,
                           const float *bias) {
    if (!type_ok(type)) return -1;
    enum { TILE = 64 };
    float *tile = (float *)aligned_alloc(64, (size_t)TILE * K * sizeof(float));
    if (!tile) return -2;
    for (int o0 = 0; o0 < N; o0 += TILE) {
        const int nr = N - o0 < TILE ? N - o0 : TILE;
#pragma omp parallel for schedule(static)
        for (int r = 0; r < nr; r++) dequant_row(type, w, o0 + r, K, tile + (int64_t)r * K);
#pragma omp parallel for schedule(static)
        for (int s = 0; s < T; s++) dot_rows_f32(x + (int64_t)s * K, tile, K, nr, y + (int64_t)s * N + o0, 1);
    }
    free(tile);
    if (bias) {
#pragma omp parallel for schedule(static)
        for (int s = 0; s < T; s++)
            for (int o = 0; o < N; o++) y[(int64_t)s * N + o] += bias[o];
    }
    return 0;
}

/* Same product accumulated in fp64: the arbiter for tolerance checks (not a reference path). */
int gt_oracle_matmul_batch_f64(int type, const uint8_t *w, const float *x, double *y, int K, int N, int T,
                               const float *bias) {
    if (!type_ok(type)) return -1;
    enum { TILE = 64 };
    float *tile = (float *)aligned_alloc(64, (size_t)TILE * K * sizeof(float));
    if (!tile) return -2;
    for (int o0 = 0; o0 < N; o0 += TILE) {
        const int nr = N - o0 < TILE ? N - o0 : TILE;
#pragma omp parallel for schedule(static)
        for (int r = 0; r < nr; r++) dequant_row(type, w, o0 + r, K, tile + (int64_t)r * K);
#pragma omp parallel for schedule(static)
        for (int s = 0; s < T; s++) {
            const float *xs = x + (int64_t)s * K;
            for (int r = 0; r < nr; r++) {
                const float *wr = tile + (int64_t)r * K;
                double acc = 0.0;
                for (int k = 0; k < K; k++) acc += (double)xs[k] * (double)wr[k];
                y[(int64_t)s * N + o0 + r] = acc + (bias ? (double)bias[o0 + r] : 0.0);
            }
        }
    }
    free(tile);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * LoRA forward delta: low = X*A ; Y[s,:] += (low[s,r]*scaling) * B[r,:], zero coefficients skipped.
 * src/Glacier.Tune/Kernels/LoraKernels.cs:18-122.  A is [K, r] row-major, B is [r, N] row-major
 * (src/Glacier.Tune/Model/LoraAdapter.cs:25-26).
 * ------------------------------------------------------------------------------------------- */
GT_CLONES
static void axpy_f32(float *dst, const float *src, float scale, int n) {
#pragma omp simd
    for (int i = 0; i < n; i++) dst[i] += scale * src[i];
}

static void lora_low(const float *x, const float *a, float *low, int T, int K, int R) {
#pragma omp parallel for schedule(static)
    for (int s = 0; s < T; s++) {
        const float *xs = x + (int64_t)s * K;
        float acc[64];
        for (int r = 0; r < R; r++) acc[r] = 0.f;
        for (int k = 0; k < K; k++) {
            const float xv = xs[k];
            const float *ar = a + (int64_t)k * R;
            for (int r = 0; r < R; r++) acc[r] += xv * ar[r];
        }
        for (int r = 0; r < R; r++) low[(int64_t)s * R + r] = acc[r];
    }
}

/* LoraAdapter.IsZeroDelta: src/Glacier.Tune/Model/LoraAdapter.cs:48-72. */
int gt_oracle_is_zero_delta(const float *b, int64_t n, float scaling) {
    if (scaling == 0.f) return 1;
    for (int64_t i = 0; i < n; i++)
        if (b[i] != 0.f) return 0;
    return 1;
}

int gt_oracle_apply_lora_delta(const float *x, const float *a, const float *b, float *y, int T, int K, int N,
                               int R, float scaling) {
    if (R > 64) return -1;
    float *low = (float *)malloc((size_t)T * R * sizeof(float));
    if (!low) return -2;
    lora_low(x, a, low, T, K, R);
#pragma omp parallel for schedule(static)
    for (int s = 0; s < T; s++) {
        float *ys = y + (int64_t)s * N;
        for (int r = 0; r < R; r++) {
            const float lr = low[(int64_t)s * R + r] * scaling;
            if (lr == 0.f) continue;
            axpy_f32(ys, b + (int64_t)r * N, lr, N);
        }
    }
    free(low);
    return 0;
}

/* LoraAdapter.Forward: base GEMM, then the delta unless the adapter is disabled or B == 0.
 * src/Glacier.Tune/Model/LoraAdapter.cs:128-184. */
int gt_oracle_proj_forward(int type, const uint8_t *w, const float *bias, const float *x, float *y, int K, int N,
                           int T, const float *a, const float *b, int R, float scaling) {
    int rc = gt_oracle_matmul_batch(type, w, x, y, K, N, T, bias);
    if (rc) return rc;
    if (a && b && R > 0 && !gt_oracle_is_zero_delta(b, (int64_t)R * N, scaling))
        rc = gt_oracle_apply_lora_delta(x, a, b, y, T, K, N, R, scaling);
    return rc;
}

/* ---------------------------------------------------------------------------------------------
 * Frozen-base backward: dX[T,K] += dY[T,N] * W[N,K].
 * src/Glacier.Tune/Kernels/LoraKernels.BaseBackward.cs:21-173: 64-row dequant tile, rows whose dY
 * column is all zero are skipped, then (token, 256-column block) slices of AXPYs that skip dY == 0.
 * ------------------------------------------------------------------------------------------- */
int gt_oracle_accumulate_base_backward(int type, const uint8_t *w, const float *dy, float *dx, int T, int K,
                                       int N) {
    if (!w || !dy || !dx || T <= 0 || K <= 0 || N <= 0) return 0;
    if (!type_ok(type)) return -1;
    enum { TILE = 64, COLB = 256 };
    const int col_blocks = (K + COLB - 1) / COLB;
    const int64_t slices = (int64_t)T * col_blocks;
    float *tile = (float *)aligned_alloc(64, (size_t)TILE * K * sizeof(float));
    if (!tile) return -2;
    int active[TILE];
    for (int o0 = 0; o0 < N; o0 += TILE) {
        const int nr = N - o0 < TILE ? N - o0 : TILE;
        int nact = 0;
        for (int r = 0; r < nr; r++) {
            for (int s = 0; s < T; s++)
                if (dy[(int64_t)s * N + o0 + r] != 0.f) {
                    active[nact++] = r;
                    break;
                }
        }
        if (nact == 0) continue;
#pragma omp parallel for schedule(static)
        for (int i = 0; i < nact; i++) dequant_row(type, w, o0 + active[i], K, tile + (int64_t)active[i] * K);
#pragma omp parallel for schedule(static)
        for (int64_t wi = 0; wi < slices; wi++) {
            const int s = (int)(wi / col_blocks);
            const int c0 = (int)(wi % col_blocks) * COLB;
            const int cl = K - c0 < COLB ? K - c0 : COLB;
            float *dxs = dx + (int64_t)s * K + c0;
            const float *dys = dy + (int64_t)s * N + o0;
            for (int i = 0; i < nact; i++) {
                const int r = active[i];
                const float g = dys[r];
                if (g == 0.f) continue;
                axpy_f32(dxs, tile + (int64_t)r * K + c0, g, cl);
            }
        }
    }
    free(tile);
    return 0;
}

/* fp64 arbiter for dX (no accumulate-into semantics: writes the product only). */
int gt_oracle_base_backward_f64(int type, const uint8_t *w, const float *dy, double *dx, int T, int K, int N) {
    if (!type_ok(type)) return -1;
    memset(dx, 0, (size_t)T * K * sizeof(double));
    enum { TILE = 64 };
    float *tile = (float *)aligned_alloc(64, (size_t)TILE * K * sizeof(float));
    if (!tile) return -2;
    for (int o0 = 0; o0 < N; o0 += TILE) {
        const int nr = N - o0 < TILE ? N - o0 : TILE;
#pragma omp parallel for schedule(static)
        for (int r = 0; r < nr; r++) dequant_row(type, w, o0 + r, K, tile + (int64_t)r * K);
#pragma omp parallel for schedule(static)
        for (int s = 0; s < T; s++) {
            double *dxs = dx + (int64_t)s * K;
            for (int r = 0; r < nr; r++) {
                const double g = dy[(int64_t)s * N + o0 + r];
                const float *wr = tile + (int64_t)r * K;
                for (int k = 0; k < K; k++) dxs[k] += g * (double)wr[k];
            }
        }
    }
    free(tile);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * LoRA backward, the five steps of src/Glacier.Tune/Kernels/LoraKernels.cs:125-346:
 *   1 low = X*A                          2 dB[r,:] += sum_s (low[s,r]*scaling) * dY[s,:]
 *   3 dLow = dY*B^T                      4 dA[k,:] += scaling * sum_s X[s,k] * dLow[s,:]
 *   5 dX[s,k] += scaling * <dLow[s,:], A[k,:]>      (only when dX is given)
 * Gradients accumulate (+=).
 * ------------------------------------------------------------------------------------------- */
int gt_oracle_lora_backward(const float *x, const float *dy, const float *a, const float *b, float *ga, float *gb,
                            float *dx, int T, int K, int N, int R, float scaling) {
    if (R > 64) return -1;
    float *low = (float *)malloc((size_t)T * R * sizeof(float));
    float *dlow = (float *)malloc((size_t)T * R * sizeof(float));
    if (!low || !dlow) {
        free(low);
        free(dlow);
        return -2;
    }
    lora_low(x, a, low, T, K, R);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; r++) {
        float *gbr = gb + (int64_t)r * N;
        for (int s = 0; s < T; s++) axpy_f32(gbr, dy + (int64_t)s * N, low[(int64_t)s * R + r] * scaling, N);
    }
#pragma omp parallel for schedule(static)
    for (int s = 0; s < T; s++) {
        const float *dys = dy + (int64_t)s * N;
        for (int r = 0; r < R; r++) {
            const float *br = b + (int64_t)r * N;
            float dot = 0.f;
#pragma omp simd reduction(+ : dot)
            for (int n = 0; n < N; n++) dot += dys[n] * br[n];
            dlow[(int64_t)s * R + r] = dot;
        }
    }
#pragma omp parallel for schedule(static)
    for (int k = 0; k < K; k++) {
        float acc[64];
        for (int r = 0; r < R; r++) acc[r] = 0.f;
        for (int s = 0; s < T; s++) {
            const float wv = x[(int64_t)s * K + k] * scaling;
            const float *dl = dlow + (int64_t)s * R;
            for (int r = 0; r < R; r++) acc[r] += wv * dl[r];
        }
        for (int r = 0; r < R; r++) ga[(int64_t)k * R + r] += acc[r];
    }
    if (dx) {
#pragma omp parallel for schedule(static)
        for (int s = 0; s < T; s++) {
            const float *dl = dlow + (int64_t)s * R;
            float *dxs = dx + (int64_t)s * K;
            for (int k = 0; k < K; k++) {
                const float *ak = a + (int64_t)k * R;
                float dot = 0.f;
                for (int r = 0; r < R; r++) dot += dl[r] * ak[r];
                dxs[k] += dot * scaling;
            }
        }
    }
    free(low);
    free(dlow);
    return 0;
}

/* LoraAdapter.Backward(baseType, W, dY, x, dXInput): base term then adapter term.
 * src/Glacier.Tune/Model/LoraAdapter.cs:190-219. */
int gt_oracle_proj_backward(int type, const uint8_t *w, const float *dy, const float *x, float *dx, int K, int N,
                            int T, const float *a, const float *b, float *ga, float *gb, int R, float scaling) {
    int rc = 0;
    if (dx) rc = gt_oracle_accumulate_base_backward(type, w, dy, dx, T, K, N);
    if (rc) return rc;
    if (a && b && R > 0) rc = gt_oracle_lora_backward(x, dy, a, b, ga, gb, dx, T, K, N, R, scaling);
    return rc;
}

/* Gradient clipping: src/Glacier.Tune/Trainer/LoraTrainer.cs:395-433.  fp64 sum of squares over all
 * gradients; non-finite norm zeroes every gradient and returns 0; norm > max scales by
 * max/(norm+1e-6).  Returns the pre-clip norm. */
double gt_oracle_clip_gradients(float *g, int64_t n, double max_norm) {
    double ss = 0.0;
#pragma omp parallel for reduction(+ : ss) schedule(static)
    for (int64_t i = 0; i < n; i++) ss += (double)g[i] * (double)g[i];
    double norm = sqrt(ss);
    if (isnan(norm) || isinf(norm)) {
        memset(g, 0, (size_t)n * sizeof(float));
        return 0.0;
    }
    if (max_norm > 0.0 && norm > max_norm) {
        const float sc = (float)(max_norm / (norm + 1e-6));
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; i++) g[i] *= sc;
    }
    return norm;
}

/* ---------------------------------------------------------------------------------------------------------
 * Layer glue between the projections (the callers on either side of the path).
 * --------------------------------------------------------------------------------------------------------- */

/* SwiGLU forward: hidden = SiLU(gate) * up, element by element in fp32.
 * src/Glacier.Tune/Kernels/SwiGluKernel.cs:13-31. */
void gt_oracle_swiglu_forward(const float *gate, const float *up, float *hidden, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float g = gate[i], u = up[i];
        const float sig = 1.0f / (1.0f + expf(-g));
        const float silu = g * sig;
        hidden[i] = silu * u;
    }
}

/* SwiGLU backward: dUp = dH * SiLU(g); dGate = dH * u * sig * (1 + g * (1 - sig)).
 * src/Glacier.Tune/Kernels/SwiGluKernel.cs:33-60 (both outputs are assigned, not accumulated). */
void gt_oracle_swiglu_backward(const float *dh, const float *gate, const float *up, float *dgate, float *dup, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float d = dh[i], g = gate[i], u = up[i];
        const float sig = 1.0f / (1.0f + expf(-g));
        const float silu = g * sig;
        dup[i] = d * silu;
        const float dsilu = sig * (1.0f + g * (1.0f - sig));
        dgate[i] = d * u * dsilu;
    }
}

/* RoPE over a sequence, in place: for position pos and pair (i, i + half) of every head,
 *   freq = 1 / pow(base, 2i / ropeDim) (fp32), theta = pos * freq * scale (fp32),
 *   (v0, v1) -> (v0 cos - v1 s, v0 s + v1 cos), s = sin(theta), negated for the inverse (backward) rotation.
 * src/Glacier.Tune/Kernels/RoPEKernel.cs:12-42 (sequence loops) and 44-126 (one position); ropeFreqs == null. */
void gt_oracle_rope(float *q, float *k, int T, int heads_q, int heads_kv, int head_dim, float freq_base, float freq_scale,
                    int rope_dim, int inverse) {
    const int eff = (rope_dim > 0 && rope_dim <= head_dim) ? rope_dim : head_dim;
    const int half = eff / 2;
    if (half <= 0) return;
    const float sign = inverse ? -1.0f : 1.0f;
#pragma omp parallel for schedule(static)
    for (int pos = 0; pos < T; pos++) {
        float *pq = q ? q + (int64_t)pos * heads_q * head_dim : NULL;
        float *pk = k ? k + (int64_t)pos * heads_kv * head_dim : NULL;
        for (int i = 0; i < half; i++) {
            const float base_freq = 1.0f / powf(freq_base, (float)(2 * i) / (float)eff);
            const float theta = (float)pos * base_freq * freq_scale;
            const float c = cosf(theta), s = sinf(theta) * sign;
            for (int h = 0; pq && h < heads_q; h++) {
                float *hd = pq + h * head_dim;
                const float v0 = hd[i], v1 = hd[i + half];
                hd[i] = v0 * c - v1 * s;
                hd[i + half] = v0 * s + v1 * c;
            }
            for (int h = 0; pk && h < heads_kv; h++) {
                float *hd = pk + h * head_dim;
                const float v0 = hd[i], v1 = hd[i + half];
                hd[i] = v0 * c - v1 * s;
                hd[i + half] = v0 * s + v1 * c;
            }
        }
    }
}

/* RMSNorm forward: y[t, :] = x[t, :] * rsqrt(mean(x[t, :]^2) + eps) * w.  The implementation the reference calls
 * (ElementwiseKernels.RMSNorm, Glacier.Tensor 1.1.0, call sites src/Glacier.Tune/Model/TransformerBlock.cs:318,524) is not
 * in the repository: this is the textbook definition, PARITY UNPINNED against the reference and pinned to Qwen2RMSNorm of
 * the transformers package (tests/test_oracle_pins_qwen2.py).  The mean is accumulated in fp64 here so that the oracle
 * is the more accurate side. */
void gt_oracle_rmsnorm_forward(const float *x, const float *w, float *y, int T, int H, float eps) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        const float *xr = x + (int64_t)t * H;
        double ss = 0.0;
        for (int i = 0; i < H; i++) ss += (double)xr[i] * (double)xr[i];
        const float r = (float)(1.0 / sqrt(ss / H + (double)eps));
        for (int i = 0; i < H; i++) y[(int64_t)t * H + i] = xr[i] * r * w[i];
    }
}

/* RMSNorm backward with frozen weight (the reference passes dW = null, TransformerBlock.cs:672,827):
 *   g = dy * w;  dx = r * g - x * r^3 * mean(g * x),  r = rsqrt(mean(x^2) + eps).  Pinning as above (autograd through
 *   Qwen2RMSNorm). */
void gt_oracle_rmsnorm_backward(const float *dy, const float *x, const float *w, float *dx, int T, int H, float eps) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        const float *xr = x + (int64_t)t * H, *gr = dy + (int64_t)t * H;
        double ss = 0.0, gx = 0.0;
        for (int i = 0; i < H; i++) {
            ss += (double)xr[i] * (double)xr[i];
            gx += (double)gr[i] * (double)w[i] * (double)xr[i];
        }
        const double r = 1.0 / sqrt(ss / H + (double)eps);
        const double coef = r * r * r * gx / H;
        for (int i = 0; i < H; i++) dx[(int64_t)t * H + i] = (float)(r * (double)gr[i] * (double)w[i] - (double)xr[i] * coef);
    }
}

/* AdamW step with decoupled weight decay on a flat parameter buffer; `step` counts from 1.
 * The reference takes the optimizer from Glacier.Tensor 1.1.0 (`new AdamW(params, lr, beta1, beta2, eps, weightDecay)`,
 * `.Step()`, src/Glacier.Tune/Trainer/LoraTrainer.cs:56-62,230), whose source is not in the repository: this is the
 * textbook rule (Loshchilov & Hutter), PARITY UNPINNED against the reference, pinned against torch.optim.AdamW by
 * the CPU tests:
 *   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p *= 1 - lr wd;  p -= lr (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps)
 * Moments and parameters are fp32; the two bias corrections are evaluated in fp64 once per step. */
void gt_oracle_adamw_step(float *p, const float *g, float *m, float *v, int64_t n, float lr, float beta1, float beta2,
                          float eps, float weight_decay, int step) {
    const float c1 = (float)(1.0 / (1.0 - pow((double)beta1, (double)step)));
    const float c2 = (float)(1.0 / (1.0 - pow((double)beta2, (double)step)));
    const float decay = 1.0f - lr * weight_decay;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float gi = g[i];
        const float mi = beta1 * m[i] + (1.0f - beta1) * gi;
        const float vi = beta2 * v[i] + (1.0f - beta2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        p[i] = p[i] * decay - lr * (mi * c1) / (sqrtf(vi * c2) + eps);
    }
}


/* ---------------------------------------------------------------------------------------------
 * Streaming cross-entropy over the LM head with its input gradient:
 * FusedCrossEntropyLoss.ComputeLossAndGradients, CPU branch
 * (src/Glacier.Tune/Kernels/FusedCrossEntropyLoss.cs:170-364; the loss-only form :22-168 is the same first pass).
 *   valid tokens: 0 <= label < vocab; loss = mean over them of (logsumexp - target logit)
 *   pass 1, vocabulary tiles of `tile` rows: logits tile by MatMulBatch; running max in fp32, running sum of
 *           exp(logit - max) in fp64, rescaled by exp(old max - new max) when the max moves
 *   pass 2: logits tile again; dLogit = (exp(logit - lse) - [v == target]) / valid; dHidden += dLogit * W tile
 *           (AccumulateBaseBackward)
 * d_hidden (may be NULL: loss only) is [T, H]; rows of ignored tokens are zero.  Returns the loss.
 * ------------------------------------------------------------------------------------------- */
float gt_oracle_cross_entropy(int type, const uint8_t *w, const float *hidden, const int32_t *labels, int T, int H, int V,
                              int tile, float *d_hidden, int32_t *valid_out) {
    if (valid_out) *valid_out = 0;
    if (d_hidden) memset(d_hidden, 0, (size_t)T * H * sizeof(float));
    if (!type_ok(type) || T <= 0) return 0.f;
    int *idx = (int *)malloc((size_t)T * sizeof(int));
    int nv = 0;
    for (int t = 0; t < T; t++)
        if (labels[t] >= 0 && labels[t] < V) idx[nv++] = t;
    if (valid_out) *valid_out = nv;
    if (nv == 0) {
        free(idx);
        return 0.f;
    }
    const float inv_valid = 1.0f / (float)nv;
    if (tile > V) tile = V;
    if (tile < 1) tile = 1;
    const int n_tiles = (V + tile - 1) / tile;
    float *xh = (float *)aligned_alloc(64, (((size_t)nv * H * sizeof(float)) + 63) & ~(size_t)63);
    float *gh = (float *)aligned_alloc(64, (((size_t)nv * H * sizeof(float)) + 63) & ~(size_t)63);
    float *lg = (float *)aligned_alloc(64, (((size_t)nv * tile * sizeof(float)) + 63) & ~(size_t)63);
    float *rmax = (float *)malloc((size_t)nv * sizeof(float));
    double *rsum = (double *)malloc((size_t)nv * sizeof(double));
    float *tlog = (float *)malloc((size_t)nv * sizeof(float));
    double *lse = (double *)malloc((size_t)nv * sizeof(double));
    for (int i = 0; i < nv; i++) {
        memcpy(xh + (size_t)i * H, hidden + (size_t)idx[i] * H, (size_t)H * sizeof(float));
        rmax[i] = -INFINITY;
        rsum[i] = 0.0;
        tlog[i] = 0.f;
    }
    memset(gh, 0, (size_t)nv * H * sizeof(float));
    const int64_t row_bytes = type == GT_TYPE_F32   ? (int64_t)H * 4
                              : type == GT_TYPE_F16 ? (int64_t)H * 2
                              : type == GT_TYPE_Q4_0 ? (int64_t)H / 32 * 18
                              : type == GT_TYPE_Q8_0 ? (int64_t)H / 32 * 34
                                                     : (int64_t)H / GT_QK_K * gt_oracle_block_bytes(type);
    for (int tl = 0; tl < n_tiles; tl++) {
        const int v0 = tl * tile, vc = V - v0 < tile ? V - v0 : tile;
        gt_oracle_matmul_batch(type, w + (int64_t)v0 * row_bytes, xh, lg, H, vc, nv, NULL);
#pragma omp parallel for schedule(static)
        for (int i = 0; i < nv; i++) {
            const float *l = lg + (size_t)i * vc;
            const int y = labels[idx[i]];
            if (y >= v0 && y < v0 + vc) tlog[i] = l[y - v0];
            float tmax = -INFINITY;
            for (int v = 0; v < vc; v++) tmax = l[v] > tmax ? l[v] : tmax;
            const float mnew = rmax[i] > tmax ? rmax[i] : tmax;
            double tsum = 0.0;
            for (int v = 0; v < vc; v++) tsum += (double)expf(l[v] - mnew);
            if (isinf(rmax[i])) rsum[i] = tsum;
            else rsum[i] = rsum[i] * exp((double)rmax[i] - (double)mnew) + tsum;
            rmax[i] = mnew;
        }
    }
    double total = 0.0;
    for (int i = 0; i < nv; i++) {
        lse[i] = (double)rmax[i] + log(rsum[i]);
        total += lse[i] - (double)tlog[i];
    }
    if (d_hidden) {
        for (int tl = 0; tl < n_tiles; tl++) {
            const int v0 = tl * tile, vc = V - v0 < tile ? V - v0 : tile;
            gt_oracle_matmul_batch(type, w + (int64_t)v0 * row_bytes, xh, lg, H, vc, nv, NULL);
#pragma omp parallel for schedule(static)
            for (int i = 0; i < nv; i++) {
                float *l = lg + (size_t)i * vc;
                const int y = labels[idx[i]];
                for (int v = 0; v < vc; v++) {
                    if (v0 + v == y) l[v] = (float)(exp((double)l[v] - lse[i]) - 1.0) * inv_valid;
                    else l[v] = expf((float)((double)l[v] - lse[i])) * inv_valid;
                }
            }
            gt_oracle_accumulate_base_backward(type, w + (int64_t)v0 * row_bytes, lg, gh, nv, H, vc);
        }
        for (int i = 0; i < nv; i++) memcpy(d_hidden + (size_t)idx[i] * H, gh + (size_t)i * H, (size_t)H * sizeof(float));
    }
    free(idx); free(xh); free(gh); free(lg); free(rmax); free(rsum); free(tlog); free(lse);
    return (float)(total * (double)inv_valid);
}

/* ---------------------------------------------------------------------------------------------
 * Causal multi-head attention with grouped KV heads, forward and backward:
 * CausalAttentionKernel.Forward / Backward (src/Glacier.Tune/Kernels/CausalAttentionKernel.cs:17-213).
 * q, out, d_out, dq: [T, heads_q, head_dim]; k, v, dk, dv: [T, heads_kv, head_dim]; probs: [heads_q, T, T] (the
 * reference's storage of the softmax rows; upper triangle zero).  scale = 1 / sqrt(head_dim); head h reads KV
 * head h / (heads_q / heads_kv).  The backward overwrites dq, dk, dv.
 * ------------------------------------------------------------------------------------------- */
void gt_oracle_attention_forward(const float *q, const float *k, const float *v, float *out, float *probs, int T, int HQ, int HK, int D) {
    const int ratio = HQ / HK;
    const float scale = 1.0f / sqrtf((float)D);
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < HQ; h++) {
        const int kh = h / ratio;
        float *ph = probs + (size_t)h * T * T;
        for (int i = 0; i < T; i++) {
            const float *qv = q + ((size_t)i * HQ + h) * D;
            float *pr = ph + (size_t)i * T;
            float mx = -INFINITY;
            for (int j = 0; j <= i; j++) {
                const float *kv = k + ((size_t)j * HK + kh) * D;
                float sc = 0.f;
                for (int d = 0; d < D; d++) sc += qv[d] * kv[d];
                sc *= scale;
                pr[j] = sc;
                if (sc > mx) mx = sc;
            }
            for (int j = i + 1; j < T; j++) pr[j] = 0.f;
            float se = 0.f;
            for (int j = 0; j <= i; j++) {
                const float e = expf(pr[j] - mx);
                pr[j] = e;
                se += e;
            }
            const float inv = se > 0.f ? 1.0f / se : 0.f;
            for (int j = 0; j <= i; j++) pr[j] *= inv;
            float *ov = out + ((size_t)i * HQ + h) * D;
            for (int d = 0; d < D; d++) ov[d] = 0.f;
            for (int j = 0; j <= i; j++) {
                const float p = pr[j];
                const float *vv = v + ((size_t)j * HK + kh) * D;
                for (int d = 0; d < D; d++) ov[d] += p * vv[d];
            }
        }
    }
}

void gt_oracle_attention_backward(const float *d_out, const float *q, const float *k, const float *v, const float *probs, float *dq,
                                  float *dk, float *dv, int T, int HQ, int HK, int D) {
    const int ratio = HQ / HK;
    const float scale = 1.0f / sqrtf((float)D);
    memset(dq, 0, (size_t)T * HQ * D * sizeof(float));
    memset(dk, 0, (size_t)T * HK * D * sizeof(float));
    memset(dv, 0, (size_t)T * HK * D * sizeof(float));
    float *wk = (float *)calloc((size_t)HQ * T * D, sizeof(float));
    float *wv = (float *)calloc((size_t)HQ * T * D, sizeof(float));
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < HQ; h++) {
        const int kh = h / ratio;
        const float *ph = probs + (size_t)h * T * T;
        float *hk = wk + (size_t)h * T * D, *hv = wv + (size_t)h * T * D;
        float *dp = (float *)malloc((size_t)T * sizeof(float));
        float *ds = (float *)malloc((size_t)T * sizeof(float));
        for (int i = 0; i < T; i++) {
            const float *dov = d_out + ((size_t)i * HQ + h) * D;
            const float *pr = ph + (size_t)i * T;
            float dot = 0.f;
            for (int j = 0; j <= i; j++) {
                const float *vv = v + ((size_t)j * HK + kh) * D;
                float x = 0.f;
                for (int d = 0; d < D; d++) x += dov[d] * vv[d];
                dp[j] = x;
                dot += pr[j] * x;
            }
            for (int j = 0; j <= i; j++) ds[j] = pr[j] * (dp[j] - dot) * scale;
            float *dqv = dq + ((size_t)i * HQ + h) * D;
            const float *qv = q + ((size_t)i * HQ + h) * D;
            for (int j = 0; j <= i; j++) {
                const float s = ds[j], p = pr[j];
                const float *kv = k + ((size_t)j * HK + kh) * D;
                float *a = hk + (size_t)j * D, *b = hv + (size_t)j * D;
                for (int d = 0; d < D; d++) {
                    dqv[d] += s * kv[d];
                    a[d] += s * qv[d];
                    b[d] += p * dov[d];
                }
            }
        }
        free(dp);
        free(ds);
    }
#pragma omp parallel for schedule(static)
    for (int kh = 0; kh < HK; kh++)
        for (int j = 0; j < T; j++) {
            float *a = dk + ((size_t)j * HK + kh) * D, *b = dv + ((size_t)j * HK + kh) * D;
            for (int h = kh * ratio; h < (kh + 1) * ratio; h++) {
                const float *sa = wk + ((size_t)h * T + j) * D, *sb = wv + ((size_t)h * T + j) * D;
                for (int d = 0; d < D; d++) {
                    a[d] += sa[d];
                    b[d] += sb[d];
                }
            }
        }
    free(wk);
    free(wv);
}
