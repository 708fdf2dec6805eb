// Weight-streaming forward projection for few tokens (T <= 32):  Y[T, N] = X[T, K] * W[N, K]^T (+ bias).
//
// With a handful of tokens every weight is used a handful of times, so the projection is bound by how fast the
// packed K-quant bytes leave HBM, not by the tensor pipe, and the CTA-wide tcgen05 kernel (one MMA per ~200 clocks
// whatever its size) cannot keep up.  Here each WARP streams 16 weight rows through its own shared-memory ring and
// multiplies them on warp-level m16n8k16 MMAs (weights = A operand, tokens = B operand):
//
//   * the quantized integers go into the MMA as they are: a nibble q is dropped into a bf16 bit pattern 0x4300 | q
//     (= 128 + q, exact), one LOP3 per pair of weights, no arithmetic per weight;
//   * scale and offset are applied per 32-weight sub-block AFTER the MMAs, on the fp32 partial sums:
//       sum_k (a*q_k - b) * x_k  =  a * P - (128*a + b) * S,   P = sum_k (128 + q_k) * x_k,  S = sum_k x_k
//     with a = d*sc, b = dmin*m of that row and sub-block (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:209-211 is the
//     same value evaluated element by element) - so the weights enter exactly, only X is rounded to bf16;
//   * the contraction index is permuted inside each 64-weight group so that the bytes a thread loads (8 consecutive
//     bytes of qs) are the A fragments of four MMAs without any shuffle; X is staged once per CTA in shared memory
//     in the matching order, together with S.
//
// Grid: (CTAs per K split, K splits), one CTA of 16 warps per SM.  The packed rows travel global -> shared memory as
// tiled TMA copies into a per-warp ring (two chunks of 16 rows x 288 bytes in flight per warp, one copy per chunk);
// partial sums leave through fp32 atomics into a Y pre-filled with the bias.
// Replaces gemm_q4_k_batch of the reference at small batch (launched at src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:83-129).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "gt_internal.h"
#include "gt_ptx.cuh"
#include "gt_quant.cuh"

namespace gt {

namespace {

constexpr int kSWarps = 16;
constexpr int kSThreads = 32 * kSWarps;
constexpr int kScaleScratch = 16 * 8 * 8;    // per warp: [16 rows][8 sub-blocks] (a, c) pairs

__device__ __forceinline__ void mma_bf16_s(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D = A * B (accumulator input is the zero register: no moves to clear D)
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack_bf16_s(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
// shared-memory loads through 32-bit addresses (no 64-bit pointer arithmetic in the inner loop)
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(a));
    return r;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(a));
    return r;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 r;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(a));
    return r;
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
    float2 r;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(r.x), "=f"(r.y) : "r"(a));
    return r;
}

struct StreamParams {
    CUtensorMap tm_rows;   // packed rows as 32-bit words, boxes of 16 rows x 288 bytes
    const float *X;        // [T, K] fp32
    float *Y;              // [T, N], pre-filled with the bias (or zero): every partial sum is added atomically
    int *status;           // engine status word for bounded waits
    long long *trace;      // optional timeline of warp 0 of CTA (0,0): SM clock stamps, or null
    int T, N, K;
    int blocks_per_row;    // K / 256
    int blocks_per_cta;    // 256-weight blocks per K split (blockIdx.y)
    int tok_stride;        // bytes between tokens in the staged X
};

constexpr int kRingStages = 2;                 // per warp
constexpr int kChunkBlocks = 2;                // 256-weight blocks per ring stage and row
constexpr int kRowStride = kChunkBlocks * kQ4KBlockBytes;    // 288 B: consecutive rows start 8 banks apart
constexpr int kStageBytes = 16 * kRowStride;   // 16 rows
constexpr int kWarpRing = kRingStages * kStageBytes;

// Shared memory: staged X  [TP tokens][blocks_per_cta * 4 groups][4 quarter-warps t4][8 words], token rows padded by
// 16 bytes so that the 128-bit reads of a quarter warp (two tokens x four t4) hit eight different bank groups;
// S [blocks_per_cta * 8 sub-blocks][TP]; per warp: scale scratch, a ring of packed weight rows, its barriers.
//
// Work of one K split = (16-row tile, chunk of two blocks) items in row-major order, cut into equal contiguous runs
// over the warps of the split's CTAs; a warp walks its run with kRingStages chunks in flight (one tiled copy per
// chunk, issued by lane 0) and adds a tile's partial sums into Y whenever it leaves the tile.
template <int NT>
__global__ void __launch_bounds__(kSThreads, 1) k_stream_fwd_q4k(const __grid_constant__ StreamParams p) {
    constexpr int TP = 8 * NT;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int kb0 = blockIdx.y * p.blocks_per_cta;
    const int nb = min(p.blocks_per_cta, p.blocks_per_row - kb0);
    uint8_t *Xs = smem;
    float *Ss = reinterpret_cast<float *>(smem + (size_t)TP * p.tok_stride);
    uint8_t *wbase = reinterpret_cast<uint8_t *>(Ss + p.blocks_per_cta * 8 * TP) + warp * (kScaleScratch + kWarpRing + 128);
    uint8_t *Sc = wbase;
    uint8_t *ring = wbase + kScaleScratch;
    const uint32_t ring_u = smem_u32(ring);
    const uint32_t bar0 = smem_u32(wbase + kScaleScratch + kWarpRing);
    if (tid == 0) abort_flag = 0;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0;
    int trace_n = 0;
    auto stamp = [&]() {
        if (tracing && trace_n < 128) p.trace[trace_n++] = clock64();
    };
    stamp();
    if (lane == 0) {
        for (int i = 0; i < kRingStages; i++) mbar_init(bar0 + 8 * i, 1);
        fence_mbar_init();
        if (warp == 0) tma_prefetch_desc(&p.tm_rows);
    }
    pdl_wait();
    pdl_trigger();
    __syncthreads();

    // ---- this warp's run of items
    const int n_tiles = (p.N + 15) >> 4;
    const int n_chunks = (nb + kChunkBlocks - 1) / kChunkBlocks;
    const int64_t n_items = (int64_t)n_tiles * n_chunks;
    const int n_warps = gridDim.x * kSWarps, wid = blockIdx.x * kSWarps + warp;
    const int i0 = (int)(n_items * wid / n_warps), i1 = (int)(n_items * (wid + 1) / n_warps);
    // (tile, chunk, ring stage) of the next item to issue / to consume, advanced without divisions
    int is_tile = i0 / n_chunks, is_c = i0 % n_chunks, is_st = 0;
    auto issue = [&]() {
        const int tile = is_tile, c = is_c, st = is_st;
        if (++is_c == n_chunks) {
            is_c = 0;
            is_tile++;
        }
        if (++is_st == kRingStages) is_st = 0;
        // one tiled copy per item: 16 rows x two blocks (the box is always transferred whole: rows past N and bytes
        // past the row end arrive as zeros, a second block that belongs to the next K split is simply not used)
        if (lane == 0) {
            const uint32_t bar = bar0 + 8 * st;
            mbar_arrive_expect_tx(bar, (uint32_t)kStageBytes);
            tma_load_2d(ring_u + st * kStageBytes, &p.tm_rows, (kb0 + c * kChunkBlocks) * (kQ4KBlockBytes / 4), tile * 16, bar);
        }
    };
    stamp();
    for (int i = i0; i < i1 && i < i0 + kRingStages; i++) issue();      // in flight while X is staged
    stamp();

    // ---- stage X: one (token, 32-weight sub-block) item per thread and step
    // Consecutive lanes take consecutive float4 of a token row (coalesced); a sub-block of 32 values is 8 lanes.
    // Sub-block sb = 2*group + h: weight e of it sits in byte e of the group's 32 quant bytes (low nibble for h = 0,
    // high for h = 1); MMA thread t4 = e / 8 holds bytes 8*t4 .. 8*t4+7 and wants words (e0,e2) (e1,e3) (e4,e6) (e5,e7).
    const int nf4 = nb * 64;      // float4 per token in this K split
    constexpr int kStageMax = 12;  // float4 per thread: TP * blocks_per_cta * 64 / kSThreads, bounded by the 48 KB of staged X
    float4 xv[kStageMax];
#pragma unroll
    for (int i = 0; i < kStageMax; i++) {      // every load is in flight before the first one is used
        const int item = tid + i * kSThreads;
        const int t = item / nf4, f = item - t * nf4;
        xv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (item < TP * nf4 && t < p.T) xv[i] = __ldg(reinterpret_cast<const float4 *>(p.X + (int64_t)t * p.K + (int64_t)kb0 * 256) + f);
    }
#pragma unroll
    for (int i = 0; i < kStageMax; i++) {
        const int item = tid + i * kSThreads;
        if (item < TP * nf4) {      // uniform over the CTA: TP * nf4 is a multiple of kSThreads
            const int t = item / nf4, f = item - t * nf4;
            const int sb = f >> 3, q = (f >> 1) & 3, hf = f & 1;
            const float4 v = xv[i];
            const uint2 w2 = make_uint2(pack_bf16_s(v.x, v.z), pack_bf16_s(v.y, v.w));
            *reinterpret_cast<uint2 *>(Xs + (size_t)t * p.tok_stride + (sb >> 1) * 128 + q * 32 + (sb & 1) * 16 + hf * 8) = w2;
            // S sums the ROUNDED values, the ones the MMAs see
            float s = __uint_as_float(w2.x << 16) + __uint_as_float(w2.x & 0xFFFF0000u) + __uint_as_float(w2.y << 16) +
                      __uint_as_float(w2.y & 0xFFFF0000u);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if ((f & 7) == 0) Ss[sb * TP + t] = s;
        }
    }
    __syncthreads();

    stamp();
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    constexpr uint32_t kMask = 0x000F000Fu, kBias = 0x43004300u;      // bf16 (128 + q) in both halves
    // D fragment: rows g / g + 8 of the tile, tokens 2*t4, 2*t4 + 1 of each n-tile
    auto flush_tile = [&](int tile) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = tile * 16 + g + ((i & 2) ? 8 : 0), t = nt * 8 + 2 * t4 + (i & 1);
                if (row < p.N && t < p.T) atomicAdd(p.Y + (int64_t)t * p.N + row, acc[nt][i]);
                acc[nt][i] = 0.f;
            }
        }
    };

    // per-thread shared-memory bases: staged X of token g (+ 32 bytes per t4), S of tokens 2*t4, scale scratch
    const uint32_t xs_u = smem_u32(Xs) + g * p.tok_stride + t4 * 32, ss_u = smem_u32(Ss) + 2 * t4 * 4, sc_u = smem_u32(Sc);
    bool ok = true;
    int tile = i0 / n_chunks, c = i0 % n_chunks, st = 0;
    uint32_t phase = 0;
    for (int i = i0; i < i1; i++) {
        const int nblk = min(kChunkBlocks, nb - c * kChunkBlocks);
        ok = mbar_wait_bounded(bar0 + 8 * st, phase, &abort_flag, p.status, 501);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        stamp();
        const uint32_t stage = ring_u + st * kStageBytes;
        for (int bl = 0; bl < nblk; bl++) {
            const int b = c * kChunkBlocks + bl;       // block index inside the K split: position in the staged X
            // scale duty: lane (row = lane & 15, half = lane >> 4) turns four (sc, m) pairs of its row into (a, c)
            {
                const uint4 hdr = lds128(stage + (lane & 15) * kRowStride + bl * kQ4KBlockBytes);
                const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
                const float d = __low2float(dm), dmin = __high2float(dm);
                const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
                const bool hi = lane >= 16;
                const uint32_t sc4 = hi ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
                const uint32_t m4 = hi ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
                float4 o0, o1;
                o0.x = d * (float)(sc4 & 255u);          o0.y = fmaf(128.f, o0.x, dmin * (float)(m4 & 255u));
                o0.z = d * (float)((sc4 >> 8) & 255u);   o0.w = fmaf(128.f, o0.z, dmin * (float)((m4 >> 8) & 255u));
                o1.x = d * (float)((sc4 >> 16) & 255u);  o1.y = fmaf(128.f, o1.x, dmin * (float)((m4 >> 16) & 255u));
                o1.z = d * (float)(sc4 >> 24);           o1.w = fmaf(128.f, o1.z, dmin * (float)(m4 >> 24));
                __syncwarp();      // the previous block's scales have been read
                float4 *dst = reinterpret_cast<float4 *>(Sc + ((lane & 15) * 8 + (hi ? 4 : 0)) * 8);
                dst[0] = o0;
                dst[1] = o1;
                __syncwarp();
            }
            const uint32_t qa = stage + g * kRowStride + bl * kQ4KBlockBytes + 16 + t4 * 8, qb = qa + 8 * kRowStride;
            const uint32_t xb = xs_u + b * 512, sb_u = ss_u + b * 8 * TP * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 ca = lds64(qa + j * 32), cb = lds64(qb + j * 32);
                // (a, c) of sub-blocks 2j, 2j+1 for rows g and g + 8
                const float4 sa = lds128f(sc_u + (g * 8 + 2 * j) * 8), sb8 = lds128f(sc_u + ((g + 8) * 8 + 2 * j) * 8);
                // A fragments of the four MMAs: m = 0,1 low nibbles of bytes 0-3 / 4-7, m = 2,3 the high nibbles
                uint32_t A[4][4];
#pragma unroll
                for (int hw = 0; hw < 2; hw++) {
                    const uint32_t va = hw ? ca.y : ca.x, vb = hw ? cb.y : cb.x;
                    A[hw][0] = (va & kMask) | kBias;            A[hw][1] = (vb & kMask) | kBias;
                    A[hw][2] = ((va >> 8) & kMask) | kBias;     A[hw][3] = ((vb >> 8) & kMask) | kBias;
                    A[2 + hw][0] = ((va >> 4) & kMask) | kBias;  A[2 + hw][1] = ((vb >> 4) & kMask) | kBias;
                    A[2 + hw][2] = ((va >> 12) & kMask) | kBias; A[2 + hw][3] = ((vb >> 12) & kMask) | kBias;
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint32_t xs = xb + nt * 8 * p.tok_stride + j * 128;
                    const uint4 x0 = lds128(xs), x1 = lds128(xs + 16);
                    float P0[4], P1[4];
                    mma_bf16_z(P0, A[0][0], A[0][1], A[0][2], A[0][3], x0.x, x0.y);
                    mma_bf16_z(P1, A[2][0], A[2][1], A[2][2], A[2][3], x1.x, x1.y);
                    mma_bf16_s(P0, A[1][0], A[1][1], A[1][2], A[1][3], x0.z, x0.w);
                    mma_bf16_s(P1, A[3][0], A[3][1], A[3][2], A[3][3], x1.z, x1.w);
                    const float2 S0 = lds64f(sb_u + ((2 * j) * TP + nt * 8) * 4), S1 = lds64f(sb_u + ((2 * j + 1) * TP + nt * 8) * 4);
                    acc[nt][0] += sa.x * P0[0] - sa.y * S0.x + sa.z * P1[0] - sa.w * S1.x;
                    acc[nt][1] += sa.x * P0[1] - sa.y * S0.y + sa.z * P1[1] - sa.w * S1.y;
                    acc[nt][2] += sb8.x * P0[2] - sb8.y * S0.x + sb8.z * P1[2] - sb8.w * S1.x;
                    acc[nt][3] += sb8.x * P0[3] - sb8.y * S0.y + sb8.z * P1[3] - sb8.w * S1.y;
                }
            }
        }
        __syncwarp();      // every lane has read the stage: it can be refilled
        if (i + kRingStages < i1) issue();
        if (c == n_chunks - 1 || i + 1 == i1) flush_tile(tile);
        if (++c == n_chunks) {
            c = 0;
            tile++;
        }
        if (++st == kRingStages) {
            st = 0;
            phase ^= 1u;
        }
    }
    stamp();
    if (!ok) {
        // a wait gave up (status word written): let copies that were already issued land before the ring is released
        for (int k = 0; k < 64; k++) __nanosleep(2000);
    }
}

template <int NT>
cudaError_t launch_nt(const StreamParams &p, dim3 grid, size_t smem, cudaStream_t s) {
    static PerDeviceOnce configured;
    cudaError_t ce = per_device_once(configured, [] { return cudaFuncSetAttribute(k_stream_fwd_q4k<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024); });
    if (ce != cudaSuccess) return ce;
    return launch_k(k_stream_fwd_q4k<NT>, grid, dim3(kSThreads), smem, s, p);
}

}  // namespace

int stream_max_tokens() {
    static const int v = [] {
        const char *e = getenv("GT_STREAM_MAX_T");
        const int n = e ? atoi(e) : 8;      // from 9 tokens on the tensor-core few-token kernel is faster
        return n < 0 ? 0 : (n > 32 ? 32 : n);
    }();
    return v;
}

bool stream_fwd_ok(const WeightDev *w, int T) {
    return w->qtype == kTypeQ4K && w->tma_ok && w->row_bytes > 0 && T >= 1 && T <= stream_max_tokens() && (w->K % 256) == 0;
}

namespace {
int pad_tokens(int T) { return T <= 8 ? 8 : (T <= 16 ? 16 : 32); }
// K splits: the staged X of a split (TP tokens x blocks x 512 B) stays below 48 KB
int stream_splits(const WeightDev *w, int T) {
    const int bpr = w->K / 256;
    const int max_blocks = (48 * 1024) / (pad_tokens(T) * 512);
    const int splits = (bpr + max_blocks - 1) / max_blocks;
    const int per = (bpr + splits - 1) / splits;
    return (bpr + per - 1) / per;
}
}  // namespace

// Y must hold the bias rows (or zero) when this is launched: every partial sum is added atomically.
cudaError_t launch_stream_fwd(const WeightDev *w, const float *X, float *Y_prefilled, int T, int sm_count, int *status, void *trace,
                              cudaStream_t s) {
    StreamParams p{};
    p.tm_rows = w->tm_rows;
    p.X = X;
    p.Y = Y_prefilled;
    p.status = status;
    p.trace = (long long *)trace;
    p.T = T;
    p.N = w->N;
    p.K = w->K;
    p.blocks_per_row = w->K / 256;
    const int splits = stream_splits(w, T);
    p.blocks_per_cta = (p.blocks_per_row + splits - 1) / splits;
    const int TP = pad_tokens(T);
    p.tok_stride = p.blocks_per_cta * 512 + 16;
    const size_t smem = (size_t)TP * p.tok_stride + (size_t)p.blocks_per_cta * 8 * TP * sizeof(float) +
                        (size_t)kSWarps * (kScaleScratch + kWarpRing + 128);
    // one CTA per SM, spread over the K splits; never more warps than 16-row tiles x chunks
    int per_split = sm_count / splits;
    const int64_t items = (int64_t)((w->N + 15) / 16) * ((p.blocks_per_cta + kChunkBlocks - 1) / kChunkBlocks);
    const int64_t max_ctas = (items + kSWarps - 1) / kSWarps;
    if (per_split > max_ctas) per_split = (int)max_ctas;
    if (per_split < 1) per_split = 1;
    const dim3 grid(per_split, splits);
    if (TP == 8) return launch_nt<1>(p, grid, smem, s);
    if (TP == 16) return launch_nt<2>(p, grid, smem, s);
    return launch_nt<4>(p, grid, smem, s);
}

}  // namespace gt
