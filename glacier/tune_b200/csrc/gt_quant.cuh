// GGUF K-quant block formats as they sit in HBM, and their decoders.
//
// Q4_K keeps the GGUF layout (144 B, 16-byte aligned fields):
//     [0,2) half d   [2,4) half dmin   [4,16) u8 scales[12]   [16,144) u8 qs[128]
// Q6_K is re-laid out at upload so that every field starts on a 16-byte boundary (TMA needs it; the GGUF
// block is 210 B).  Device block, 224 B:
//     [0,16) i8 scales[16]   [16,18) half d   [18,32) pad   [32,160) u8 ql[128]   [160,224) u8 qh[64]
// Decoded values are identical to the reference decode
// (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:43-51,209-211,234-240,279-289,311-315): every product is exact in
// fp32 and Q4_K's final subtraction rounds once, fused or not.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace gt {

constexpr int kTypeF32 = 0;
constexpr int kTypeF16 = 1;       // plain fp16 rows (embedding and LM-head tensors)
constexpr int kTypeQ40 = 2;       // 32 weights in 18 bytes: half d; u8 qs[16]   (exact CUDA-core kernels only)
constexpr int kTypeQ80 = 8;       // 32 weights in 34 bytes: half d; i8 qs[32]   (exact CUDA-core kernels only)
constexpr int kTypeQ4K = 12;
constexpr int kTypeQ6K = 14;
constexpr int kQ4KBlockBytes = 144;
constexpr int kQ6KGgufBlockBytes = 210;
constexpr int kQ6KDevBlockBytes = 224;
constexpr int kQ40BlockBytes = 18;
constexpr int kQ80BlockBytes = 34;

__host__ __device__ constexpr int dev_block_bytes(int qt) {
    return qt == kTypeQ4K ? kQ4KBlockBytes : (qt == kTypeQ6K ? kQ6KDevBlockBytes : 0);
}

__device__ __forceinline__ float half_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// 6-bit (scale, min) pair j of a Q4_K block; s points at the 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t *s, int &sc, int &m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}
// Same, from the three 32-bit words holding scales[0..11].
__device__ __forceinline__ void q4k_scale_min_w(int j, uint32_t w0, uint32_t w1, uint32_t w2, int &sc, int &m) {
    auto byte_of = [&](int i) -> uint32_t {
        const uint32_t w = i < 4 ? w0 : (i < 8 ? w1 : w2);
        return (w >> (8 * (i & 3))) & 0xFFu;
    };
    if (j < 4) {
        sc = byte_of(j) & 63;
        m = byte_of(j + 4) & 63;
    } else {
        sc = (byte_of(j + 4) & 0x0F) | ((byte_of(j - 4) >> 6) << 4);
        m = (byte_of(j + 4) >> 4) | ((byte_of(j) >> 6) << 4);
    }
}

// Exact fp32 value of element c (0..255) of one block.
__device__ __forceinline__ float q4k_decode_elem(const uint8_t *blk, int c) {
    const float d = half_bits_to_f32(*(const uint16_t *)blk);
    const float dmin = half_bits_to_f32(*(const uint16_t *)(blk + 2));
    const int ib = c >> 5;
    int sc, m;
    q4k_scale_min(ib, blk + 4, sc, m);
    const int q = (blk[16 + (ib >> 1) * 32 + (c & 31)] >> ((ib & 1) * 4)) & 0x0F;
    const float d_sub = d * (float)sc;
    const float m_sub = dmin * (float)m;
    return d_sub * (float)q - m_sub;
}
__device__ __forceinline__ float q6k_dev_decode_elem(const uint8_t *blk, int c) {
    const int step = c >> 7, rem = c & 127, quad = rem >> 5, lane = rem & 31;
    const int ql = blk[32 + step * 64 + (quad & 1) * 32 + lane];
    const int qh = blk[160 + step * 32 + lane];
    const int q = (int)(((ql >> (quad >= 2 ? 4 : 0)) & 0x0F) | (((qh >> (quad * 2)) & 0x03) << 4)) - 32;
    const float d = half_bits_to_f32(*(const uint16_t *)(blk + 16));
    const int sc = (int)(int8_t)blk[step * 8 + (lane >> 4) + quad * 2];
    return d * (float)sc * (float)q;
}
// Q4_0 (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:23-26,151-163): weight i of a block = d * (nibble - 8), nibble = low half
// of qs[i] for i < 16, high half of qs[i - 16] otherwise.  Q8_0 (tune_bwd.cu:18-21,375-376): d * qs[i].  Blocks are 18 /
// 34 bytes, so the fp16 scale sits at an even address only: it is read as two bytes.
__device__ __forceinline__ float q40_decode_elem(const uint8_t *blk, int c) {
    const float d = half_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
    const int q = (int)((blk[2 + (c & 15)] >> ((c >> 4) << 2)) & 0x0F) - 8;
    return d * (float)q;
}
__device__ __forceinline__ float q80_decode_elem(const uint8_t *blk, int c) {
    const float d = half_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
    return d * (float)(int8_t)blk[2 + c];
}
// Element e of the flat row-major element stream of a tensor (block = e / 256 for the K-quants, e / 32 for Q4_0 / Q8_0).
template <int QT>
__device__ __forceinline__ float decode_flat(const uint8_t *w, int64_t e) {
    if constexpr (QT == kTypeF32) {
        return ((const float *)w)[e];
    } else if constexpr (QT == kTypeF16) {
        return __half2float(((const __half *)w)[e]);
    } else if constexpr (QT == kTypeQ40) {
        return q40_decode_elem(w + (e >> 5) * kQ40BlockBytes, (int)(e & 31));
    } else if constexpr (QT == kTypeQ80) {
        return q80_decode_elem(w + (e >> 5) * kQ80BlockBytes, (int)(e & 31));
    } else if constexpr (QT == kTypeQ4K) {
        return q4k_decode_elem(w + (e >> 8) * kQ4KBlockBytes, (int)(e & 255));
    } else {
        return q6k_dev_decode_elem(w + (e >> 8) * kQ6KDevBlockBytes, (int)(e & 255));
    }
}

// ------------------------------------------------------------------------------------------------
// 32-element group decoders used by the tensor-core kernels.  A "half block" is 128 consecutive weights of
// one super-block (half = 0/1); it is staged in shared memory as three row-major regions
//     hdr  : kHdrBytes per row   (Q4_K: d, dmin, scales[12];  Q6_K: scales[16], d, pad)
//     q0   : 64 B per row        (Q4_K: qs[64*half ..];       Q6_K: ql[64*half ..])
//     q1   : 32 B per row        (Q6_K only: qh[32*half ..])
// Group grp (0..3) is weights [32*grp, 32*grp+32) of the half block.
// ------------------------------------------------------------------------------------------------
template <int QT>
struct QuantStage;
template <>
struct QuantStage<kTypeQ4K> {
    static constexpr int kHdrBytes = 16, kQ0Bytes = 64, kQ1Bytes = 0;
    static constexpr int kBlockBytes = kQ4KBlockBytes;
    __host__ __device__ static constexpr int hdr_x(int /*half*/) { return 0; }
    __host__ __device__ static constexpr int q0_x(int half) { return 16 + 64 * half; }
    __host__ __device__ static constexpr int q1_x(int /*half*/) { return 0; }
};
template <>
struct QuantStage<kTypeQ6K> {
    static constexpr int kHdrBytes = 32, kQ0Bytes = 64, kQ1Bytes = 32;
    static constexpr int kBlockBytes = kQ6KDevBlockBytes;
    __host__ __device__ static constexpr int hdr_x(int /*half*/) { return 0; }
    __host__ __device__ static constexpr int q0_x(int half) { return 32 + 64 * half; }
    __host__ __device__ static constexpr int q1_x(int half) { return 160 + 32 * half; }
};

// fp16 rows need no staging area and no decoder: TMA writes them straight into the operand stage.  The constants only
// keep the kernel's (unused) packed-block ring well-formed.
template <>
struct QuantStage<kTypeF16> {
    static constexpr int kHdrBytes = 16, kQ0Bytes = 64, kQ1Bytes = 0;
    static constexpr int kBlockBytes = 512;
    __host__ __device__ static constexpr int hdr_x(int) { return 0; }
    __host__ __device__ static constexpr int q0_x(int) { return 0; }
    __host__ __device__ static constexpr int q1_x(int) { return 0; }
};

template <typename T16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// byte i (0..3) of v as an exact fp32 integer plus 2^23
__device__ __forceinline__ float byte_to_magic(uint32_t v, int i) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540u + (uint32_t)i));
}

// (no "memory" clobber: the compiler may keep packed-block loads and header arithmetic in registers across these
// stores, e.g. between the two 32-weight runs a thread decodes from one row; volatile keeps them in program order
// ahead of the proxy fence, which does clobber memory)
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d));
}

__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_splat(float v) {
    __nv_bfloat162 t = __float2bfloat162_rn(v);
    return *reinterpret_cast<uint32_t *>(&t);
}

// Decode group `grp` of half block `half` of one weight row and write its 32 values as four 16-byte chunks of
// a 128-byte-swizzled operand row: chunk (chunk0 + i) lands at dst_row + (((chunk0 + i) ^ swz) << 4),
// swz = (row index within the 1024-byte atom) & 7.
//
// The raw q0 / q1 regions were written by TMA with 64-byte / 32-byte swizzle (conflict-free reads when the
// lanes of a warp walk consecutive rows): 16-byte chunk c of a q0 row sits at (c ^ rsw0) << 4, of a q1 row at
// (c ^ rsw1) << 4, with rsw0 = (row >> 1) & 3 and rsw1 = (row >> 2) & 1.
//
// T16 = __half : every weight is evaluated exactly in fp32 (the reference formula) and rounded once.
// T16 = bf16   : packed bf16x2 arithmetic.  A 4-bit quant q is placed in a bf16 mantissa as v = 1 + q/16
//                (exact), then w = (16a) * v - (16a + b) in one fused multiply-add; a 6-bit quant as
//                v = 1 + q/64, then w = (64a) * (v - 1.5) with an exact subtraction.  The per-sub-block
//                constants are rounded to bf16, which adds an error of the size of the bf16 rounding of w itself.
template <int QT, typename T16>
__device__ __forceinline__ void dequant32_to_swizzled_row(const uint8_t *hdr_row, const uint8_t *q0_row,
                                                          const uint8_t *q1_row, int rsw0, int rsw1, int half, int grp,
                                                          uint32_t dst_row, int swz, int chunk0) {
    constexpr bool kFast = std::is_same<T16, __nv_bfloat16>::value;
    if constexpr (QT == kTypeF16) {
        // never called: fp16 tiles are written by TMA
    } else if constexpr (QT == kTypeQ4K) {
        const uint4 h = *reinterpret_cast<const uint4 *>(hdr_row);
        const float d = half_bits_to_f32(h.x & 0xFFFFu);
        const float dmin = half_bits_to_f32(h.x >> 16);
        int sc, m;
        q4k_scale_min_w(4 * half + grp, h.y, h.z, h.w, sc, m);
        const float a = d * (float)sc;
        const float b = dmin * (float)m;
        const int c0 = (grp >> 1) * 2;
        const uint4 qa = *reinterpret_cast<const uint4 *>(q0_row + ((c0 ^ rsw0) << 4));
        const uint4 qb = *reinterpret_cast<const uint4 *>(q0_row + (((c0 + 1) ^ rsw0) << 4));
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        if constexpr (kFast) {
            const uint32_t a16 = bf16x2_splat(16.f * a);
            const uint32_t c16 = bf16x2_splat(-(16.f * a + b));
            const int rot = (grp & 1) ? 31 : 3;     // nibble -> bits 3..6 of its byte: rotl 3 (low) / rotr 1 (high)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const uint32_t t = (__funnelshift_l(w[2 * i + k], w[2 * i + k], rot) & 0x78787878u) | 0x80808080u;
                    o[2 * k] = bf16x2_fma(__byte_perm(t, 0x3F3F3F3Fu, 0x4140u), a16, c16);
                    o[2 * k + 1] = bf16x2_fma(__byte_perm(t, 0x3F3F3F3Fu, 0x4342u), a16, c16);
                }
                st_shared_v4(dst_row + (uint32_t)(((chunk0 + i) ^ swz) << 4), o[0], o[1], o[2], o[3]);
            }
        } else {
            const float nb = -b;
            const int sh = (grp & 1) * 4;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const uint32_t v = (w[2 * i + k] >> sh) & 0x0F0F0F0Fu;
                    const float f0 = fmaf(a, byte_to_magic(v, 0) - 8388608.f, nb);
                    const float f1 = fmaf(a, byte_to_magic(v, 1) - 8388608.f, nb);
                    const float f2 = fmaf(a, byte_to_magic(v, 2) - 8388608.f, nb);
                    const float f3 = fmaf(a, byte_to_magic(v, 3) - 8388608.f, nb);
                    o[2 * k] = pack2<T16>(f0, f1);
                    o[2 * k + 1] = pack2<T16>(f2, f3);
                }
                st_shared_v4(dst_row + (uint32_t)(((chunk0 + i) ^ swz) << 4), o[0], o[1], o[2], o[3]);
            }
        }
    } else {
        const uint32_t scw = *reinterpret_cast<const uint32_t *>(hdr_row + 8 * half + (grp & 2) * 2);
        // bytes of scw: scales[8*half + 4*(grp>>1) + 0..3]; this group uses 2*(grp&1) and 2*(grp&1)+1
        const int s0 = (int)(int8_t)((scw >> (16 * (grp & 1))) & 0xFF);
        const int s1 = (int)(int8_t)((scw >> (16 * (grp & 1) + 8)) & 0xFF);
        const float d = half_bits_to_f32(*reinterpret_cast<const uint16_t *>(hdr_row + 16));
        const float a0 = d * (float)s0, a1 = d * (float)s1;
        const int c0 = (grp & 1) * 2;
        const uint4 la = *reinterpret_cast<const uint4 *>(q0_row + ((c0 ^ rsw0) << 4));
        const uint4 lb = *reinterpret_cast<const uint4 *>(q0_row + (((c0 + 1) ^ rsw0) << 4));
        const uint4 ha = *reinterpret_cast<const uint4 *>(q1_row + ((0 ^ rsw1) << 4));
        const uint4 hb = *reinterpret_cast<const uint4 *>(q1_row + ((1 ^ rsw1) << 4));
        const uint32_t lw[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
        const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        if constexpr (kFast) {
            const uint32_t m0 = bf16x2_splat(64.f * a0), m1 = bf16x2_splat(64.f * a1);
            const uint32_t k15 = 0x3FC03FC0u;                        // bf16x2 (1.5, 1.5)
            const int lrot = (grp >> 1) ? 29 : 1;                    // low nibble  -> bits 1..4: rotl 1 / rotr 3
            const int hrot = (5 - 2 * grp) & 31;                     // 2 high bits -> bits 5..6
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t mm = i < 2 ? m0 : m1;
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const uint32_t l = lw[2 * i + k], hh = hw[2 * i + k];
                    const uint32_t t = (__funnelshift_l(l, l, lrot) & 0x1E1E1E1Eu) | (__funnelshift_l(hh, hh, hrot) & 0x60606060u) |
                                       0x80808080u;
                    o[2 * k] = bf16x2_mul(bf16x2_sub(__byte_perm(t, 0x3F3F3F3Fu, 0x4140u), k15), mm);
                    o[2 * k + 1] = bf16x2_mul(bf16x2_sub(__byte_perm(t, 0x3F3F3F3Fu, 0x4342u), k15), mm);
                }
                st_shared_v4(dst_row + (uint32_t)(((chunk0 + i) ^ swz) << 4), o[0], o[1], o[2], o[3]);
            }
        } else {
            const int lsh = (grp >> 1) * 4, hsh = grp * 2;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float a = i < 2 ? a0 : a1;
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const uint32_t v = ((lw[2 * i + k] >> lsh) & 0x0F0F0F0Fu) | (((hw[2 * i + k] >> hsh) & 0x03030303u) << 4);
                    const float f0 = a * (byte_to_magic(v, 0) - 8388640.f);
                    const float f1 = a * (byte_to_magic(v, 1) - 8388640.f);
                    const float f2 = a * (byte_to_magic(v, 2) - 8388640.f);
                    const float f3 = a * (byte_to_magic(v, 3) - 8388640.f);
                    o[2 * k] = pack2<T16>(f0, f1);
                    o[2 * k + 1] = pack2<T16>(f2, f3);
                }
                st_shared_v4(dst_row + (uint32_t)(((chunk0 + i) ^ swz) << 4), o[0], o[1], o[2], o[3]);
            }
        }
    }
}

}  // namespace gt
