// Rank-r LoRA products for the bf16 math mode, one pass over each activation tensor:
//   k_lora_xa_tc   low[T,R]  += X[T,K] * A[K,R]                       (+ bf16 copy of X for the base GEMM)
//   k_lora_dy_tc   dLow[T,R] += dY[T,N] * B[R,N]^T ; dB[R,N] += s * low^T * dY   (+ bf16 copy of dY)
//   k_lora_da_tc   dA[K,R]   += s * X[T,K]^T * dLow[T,R]
// They replace the host loops of src/Glacier.Tune/Kernels/LoraKernels.cs:35-54,191-291.  A [64 tokens x 128 columns]
// tile of the fp32 activation tensor is rounded to bf16 once, on its way into shared memory - the same rounding
// that produces the 16-bit copy the base GEMM reads, which is written from the same registers - and every product
// that needs the tile runs on warp-level m16n8k16 bf16 MMAs with fp32 accumulation, fragments fetched with
// ldmatrix (transposed where the contraction runs over tokens).  Partial sums leave the block through fp32
// atomics.  The exact-fp32 CUDA-core versions in gt_fp32_kernels.cu serve the validation modes.
//
// A launch handles up to three 16-rank chunks: the adapters of projections that share their input (q, k, v; gate, up)
// go through one pass over X, and the dY passes of a group's members are one launch (blockIdx.z picks the member).
//
// These kernels should be bound by the HBM read of X / dY: the tile in shared memory is read once from global
// memory and reused by every product that needs it; the instruction count per element is what has to stay small
// (an earlier TF32 m16n8k8 version spent 27 thread instructions per element, mostly scalar fragment loads, and ran
// at a quarter of the HBM rate).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "gt_internal.h"
#include "gt_ptx.cuh"

namespace gt {

namespace {

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four 8x8 b16 matrices; lanes 8i..8i+7 give the row addresses of matrix i
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

constexpr int TT = 64;        // tokens per tile
constexpr int TC = 128;       // columns (of K or N) per tile
constexpr int GSB = 2 * TC + 16;   // smem row stride of the bf16 activation tile in bytes: 8 consecutive rows, 16 B each,
                                   // land in 8 different 4-bank groups (what ldmatrix reads at once)
constexpr int RSB = 48;       // smem row stride of a 16-wide bf16 rank tile in bytes (same property)
constexpr int NI = (TT * TC / 4) / 256;     // float4 loads per thread and tile
constexpr int kMaxChunks = 3;               // 16-rank chunks (of one or several adapters) served by one launch

// ldmatrix lane -> row address of its 8x8 matrix.  `base` = tile address, rows `stride` bytes apart.
//   A operand, stored [m][k]  (non-transposed load): matrices (m0-7,k0-7) (m8-15,k0-7) (m0-7,k8-15) (m8-15,k8-15)
//   A operand, stored [k][m]  (transposed load)    : matrices (k0-7,m0-7) (k0-7,m8-15) (k8-15,m0-7) (k8-15,m8-15)
//   B operand x2 n-tiles, stored [n][k] (non-transposed): (n0-7,k0-7) (n0-7,k8-15) (n8-15,k0-7) (n8-15,k8-15)
//   B operand x2 n-tiles, stored [k][n] (transposed)    : (k0-7,n0-7) (k8-15,n0-7) (k0-7,n8-15) (k8-15,n8-15)
// In every case registers {0,1,2,3} of the result are {a0,a1,a2,a3} resp. {b0,b1 of n-tile 0, b0,b1 of n-tile 1}.
__device__ __forceinline__ uint32_t lm_a_mk(uint32_t base, int stride, int m0, int k0, int lane) {
    return base + (uint32_t)((m0 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + (k0 + (lane >> 4) * 8) * 2);
}
__device__ __forceinline__ uint32_t lm_a_km(uint32_t base, int stride, int m0, int k0, int lane) {
    return base + (uint32_t)((k0 + (lane & 7) + (lane >> 4) * 8) * stride + (m0 + ((lane >> 3) & 1) * 8) * 2);
}
__device__ __forceinline__ uint32_t lm_b_nk(uint32_t base, int stride, int n0, int k0, int lane) {
    return base + (uint32_t)((n0 + (lane & 7) + (lane >> 4) * 8) * stride + (k0 + ((lane >> 3) & 1) * 8) * 2);
}
__device__ __forceinline__ uint32_t lm_b_kn(uint32_t base, int stride, int n0, int k0, int lane) {
    return base + (uint32_t)((k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + (n0 + (lane >> 4) * 8) * 2);
}

// Row fills that ride along with a pass (the split-K GEMM that follows sums into its output, so the output starts as
// the bias rows or as zero): dst[T, N] = bias[N] (or 0).  The blocks of the launch share each fill evenly.
struct FillList {
    int n;
    struct Job {
        float *dst;
        const float *bias;
        int N;
        int64_t total;      // T * N
    } f[kMaxChunks];
};
__device__ __forceinline__ void do_fills(const FillList &fl, int lb, int nb, int tid) {
    for (int j = 0; j < fl.n; j++) {
        const FillList::Job f = fl.f[j];
        if ((f.N & 3) == 0) {
            const int n4 = f.N >> 2;
            const int64_t total4 = f.total >> 2;
            float4 *d4 = reinterpret_cast<float4 *>(f.dst);
            const float4 *b4 = reinterpret_cast<const float4 *>(f.bias);
            for (int64_t i = (int64_t)lb * 256 + tid; i < total4; i += (int64_t)nb * 256)
                d4[i] = f.bias ? __ldg(&b4[i % n4]) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int64_t i = (int64_t)lb * 256 + tid; i < f.total; i += (int64_t)nb * 256) f.dst[i] = f.bias ? f.bias[i % f.N] : 0.f;
        }
    }
}

// A [TT x TC] fp32 tile of src[T, ncols] (rows t0.. below t_end, columns c0..) moves in two steps so that a block can
// have the next tile's loads in flight while it computes on the current one:
//   tile_load   global -> registers (float4 per thread when the tile is interior and aligned); a warp reads one row
//   tile_store  registers -> bf16 in shared memory, and optionally the same bf16 values to dst16 in global memory
__device__ __forceinline__ void tile_load(const float *__restrict__ src, int ncols, int t0, int t_end, int c0, float4 (&v)[NI], int tid) {
    const bool vec = (ncols & 3) == 0 && c0 + TC <= ncols;
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 4), c = (idx % (TC / 4)) * 4;
        const int t = t0 + r;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < t_end) {
            const float *p = src + (int64_t)t * ncols + c0 + c;
            if (vec) {
                v[i] = __ldg(reinterpret_cast<const float4 *>(p));
            } else {
                if (c0 + c < ncols) v[i].x = p[0];
                if (c0 + c + 1 < ncols) v[i].y = p[1];
                if (c0 + c + 2 < ncols) v[i].z = p[2];
                if (c0 + c + 3 < ncols) v[i].w = p[3];
            }
        }
    }
}
__device__ __forceinline__ void tile_store(const float4 (&v)[NI], int t0, int t_end, int c0, uint8_t *tile,
                                           uint16_t *__restrict__ dst16, int ld16, int tid) {
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 4), c = (idx % (TC / 4)) * 4;
        const int t = t0 + r;
        const uint2 pk = make_uint2(pack_bf16(v[i].x, v[i].y), pack_bf16(v[i].z, v[i].w));
        if (dst16 && t < t_end) {
            uint16_t *q = dst16 + (int64_t)t * ld16 + c0 + c;
            if (c0 + c + 3 < ld16 && (ld16 & 3) == 0) {
                *reinterpret_cast<uint2 *>(q) = pk;
            } else {
                const uint16_t e[4] = {(uint16_t)(pk.x & 0xFFFFu), (uint16_t)(pk.x >> 16), (uint16_t)(pk.y & 0xFFFFu), (uint16_t)(pk.y >> 16)};
                for (int j = 0; j < 4; j++)
                    if (c0 + c + j < ld16) q[j] = e[j];
            }
        }
        *reinterpret_cast<uint2 *>(tile + r * GSB + c * 2) = pk;
    }
}
// A [rows x 16] slab of a row-major fp32 matrix with `ld` columns (rows row0.., columns r0..r0+15; zero outside
// row_end / rc) -> bf16 rank tile in shared memory, rows RSB bytes apart.  256 threads.
__device__ __forceinline__ void rank_tile_store(const float *__restrict__ src, int ld, int row0, int row_end, int r0, int rc, int rows,
                                                uint8_t *tile, int tid) {
    for (int i = tid; i < rows * 8; i += 256) {
        const int rr = i >> 3, c = (i & 7) * 2;
        float a = 0.f, b = 0.f;
        if (row0 + rr < row_end) {
            const float *p = src + (int64_t)(row0 + rr) * ld + r0 + c;
            if (c < rc) a = __ldg(p);
            if (c + 1 < rc) b = __ldg(p + 1);
        }
        *reinterpret_cast<uint32_t *>(tile + rr * RSB + c * 2) = pack_bf16(a, b);
    }
}
// fp32 accumulator fragment of a 16 x 8 tile (rows m0 + g / + 8, columns n0 + 2*t4 / + 1) added into dst[rows, ld]
__device__ __forceinline__ void frag_atomic_add(float *dst, int64_t ld, const float (&d)[4], int row_a, int row_end, int col, int col_end,
                                                float scale) {
    const int row_b = row_a + 8;
    if (row_a < row_end) {
        if (col < col_end) atomicAdd(&dst[(int64_t)row_a * ld + col], d[0] * scale);
        if (col + 1 < col_end) atomicAdd(&dst[(int64_t)row_a * ld + col + 1], d[1] * scale);
    }
    if (row_b < row_end) {
        if (col < col_end) atomicAdd(&dst[(int64_t)row_b * ld + col], d[2] * scale);
        if (col + 1 < col_end) atomicAdd(&dst[(int64_t)row_b * ld + col + 1], d[3] * scale);
    }
}

// ------------------------------------------------------------------------------------------------
// low_j[T, R_j] += X[T, K] * A_j[K, R_j] over the block's K slice (grid.y slices of 128) for up to kMaxChunks
// 16-rank chunks that share X (the adapters of q, k, v or of gate, up): X is read and rounded once, fp32 atomics
// into each low_j (pre-zeroed).  8 warps = 4 token m-tiles x 2 halves of the slice's 8 k-steps; each warp covers
// both 8-wide rank n-tiles of every chunk.
// ------------------------------------------------------------------------------------------------
struct XaChunk {
    const float *A;
    float *low;
    int R, r0;
};
struct XaParams {
    const float *X;
    uint16_t *x16;
    int ldx16, T, K, n;
    XaChunk c[kMaxChunks];
    FillList fills;
};
constexpr int kXsBytes = TT * GSB;            // activation tile
constexpr int kAsBytes = TC * RSB;            // per chunk, k_lora_xa_tc: A[k0.., r0..] as [128][16]
constexpr int kLsBytes = TT * RSB;            // per chunk, k_lora_da_tc / k_lora_dy_tc: [64 tokens][16]

__global__ void __launch_bounds__(256) k_lora_xa_tc(const XaParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem;
    uint8_t *As = dyn_smem + kXsBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.x * TT, k0 = blockIdx.y * TC;
    const int T = p.T, K = p.K;
    pdl_wait();
    pdl_trigger();
    float4 v[NI];
    tile_load(p.X, K, t0, T, k0, v, tid);
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j < p.n) {
            const XaChunk c = p.c[j];
            rank_tile_store(c.A, c.R, k0, K, c.r0, min(16, c.R - c.r0), TC, As + j * kAsBytes, tid);
        }
    }
    tile_store(v, t0, T, k0, Xs, p.x16, p.ldx16, tid);
    __syncthreads();
    const int m0 = (warp >> 1) * 16, kh = (warp & 1) * 64;
    const uint32_t xs = smem_u32(Xs), as = smem_u32(As);
    uint32_t a[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ks++) ldsm_x4(lm_a_mk(xs, GSB, m0, kh + ks * 16, lane), a[ks]);
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j >= p.n) break;
        float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t b[4];
            ldsm_x4_t(lm_b_kn(as + j * kAsBytes, RSB, 0, kh + ks * 16, lane), b);
            mma_bf16(d[0], a[ks], b[0], b[1]);
            mma_bf16(d[1], a[ks], b[2], b[3]);
        }
        const XaChunk c = p.c[j];
        const int rc = min(16, c.R - c.r0);
#pragma unroll
        for (int i = 0; i < 2; i++)
            frag_atomic_add(c.low + c.r0, c.R, d[i], t0 + m0 + g, T, i * 8 + 2 * t4, rc, 1.f);
    }
    do_fills(p.fills, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y, tid);
}

// ------------------------------------------------------------------------------------------------
// One pass over dY_m per member m = blockIdx.z: the block owns a 128-column strip and a token group, walked in
// 64-token tiles.
//   dLow[t, r] += sum_c dY[t, c] * B[r, c]      8 warps = 4 token m-tiles x 2 halves of the strip's 8 k-steps
//   dB[r, c]   += s * sum_t low[t, r] * dY[t, c] 1 m-tile (ranks) x 16 n-tiles (columns), 2 per warp, 4 k-steps
// ------------------------------------------------------------------------------------------------
struct DyMember {
    const float *dY, *low, *B;
    float *dB, *dLow;
    uint16_t *dy16;
    int ld16, N, R, r0;
    float scaling;
};
struct DyParams {
    int T, tok_per_group, n;
    DyMember m[kMaxChunks];
    FillList fills;
};

__global__ void __launch_bounds__(256, 3) k_lora_dy_tc(const DyParams p) {
    __shared__ __align__(16) uint8_t Gs[TT * GSB];
    __shared__ __align__(16) uint8_t Bs[16 * GSB];      // B[r0.., c0..] as [16][128]
    __shared__ __align__(16) uint8_t Ls[TT * RSB];      // low tile [64][16]
    pdl_wait();
    pdl_trigger();
    const DyMember m = p.m[blockIdx.z];
    const int N = m.N, R = m.R, r0 = m.r0, T = p.T;
    const int c0 = blockIdx.x * TC;
    const int lb = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, nb = gridDim.x * gridDim.y * gridDim.z;
    if (c0 >= N) {      // a member with fewer column strips than the widest one
        do_fills(p.fills, lb, nb, threadIdx.x);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int tg0 = blockIdx.y * p.tok_per_group, tg1 = min(T, tg0 + p.tok_per_group);
    const int rc = min(16, R - r0);
    float4 v[NI];
    tile_load(m.dY, N, tg0, tg1, c0, v, tid);
    for (int i = tid; i < 16 * (TC / 2); i += 256) {
        const int r = i / (TC / 2), c = (i % (TC / 2)) * 2;
        float a = 0.f, b = 0.f;
        if (r < rc) {
            const float *q = m.B + (int64_t)(r0 + r) * N + c0 + c;
            if (c0 + c < N) a = __ldg(q);
            if (c0 + c + 1 < N) b = __ldg(q + 1);
        }
        *reinterpret_cast<uint32_t *>(Bs + r * GSB + c * 2) = pack_bf16(a, b);
    }
    const uint32_t gs = smem_u32(Gs), bs = smem_u32(Bs), ls = smem_u32(Ls);
    float accB[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int m0 = (warp >> 1) * 16, kh = (warp & 1) * 64;    // dLow: token m-tile, half of the strip's columns
    const int cb = warp * 16;                                 // dB: this warp's two 8-column n-tiles
    uint16_t *dy16 = r0 == 0 ? m.dy16 : nullptr;
    for (int ts = tg0; ts < tg1; ts += TT) {
        __syncthreads();
        tile_store(v, ts, tg1, c0, Gs, dy16, m.ld16, tid);
        if (ts + TT < tg1) tile_load(m.dY, N, ts + TT, tg1, c0, v, tid);     // next tile's loads fly during the MMAs below
        rank_tile_store(m.low, R, ts, tg1, r0, rc, TT, Ls, tid);
        __syncthreads();
        {
            float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                uint32_t a[4], b[4];
                ldsm_x4(lm_a_mk(gs, GSB, m0, kh + ks * 16, lane), a);
                ldsm_x4(lm_b_nk(bs, GSB, 0, kh + ks * 16, lane), b);
                mma_bf16(d[0], a, b[0], b[1]);
                mma_bf16(d[1], a, b[2], b[3]);
            }
#pragma unroll
            for (int i = 0; i < 2; i++) frag_atomic_add(m.dLow + r0, R, d[i], ts + m0 + g, tg1, i * 8 + 2 * t4, rc, 1.f);
        }
#pragma unroll
        for (int ks = 0; ks < TT / 16; ks++) {
            uint32_t a[4], b[4];
            ldsm_x4_t(lm_a_km(ls, RSB, 0, ks * 16, lane), a);        // low^T: m = rank, k = token
            ldsm_x4_t(lm_b_kn(gs, GSB, cb, ks * 16, lane), b);       // dY: k = token, n = column
            mma_bf16(accB[0], a, b[0], b[1]);
            mma_bf16(accB[1], a, b[2], b[3]);
        }
    }
    // accB rows = ranks, columns = strip columns
#pragma unroll
    for (int i = 0; i < 2; i++) frag_atomic_add(m.dB + (int64_t)r0 * N, N, accB[i], g, rc, c0 + cb + i * 8 + 2 * t4, N, m.scaling);
    do_fills(p.fills, lb, nb, tid);
}

// ------------------------------------------------------------------------------------------------
// dA_j[k, r] += s_j * sum_t X[t, k] * dLow_j[t, r] for up to kMaxChunks 16-rank chunks that share X: the block owns
// a 128-column strip of X and a token group.  8 warps = 8 m-tiles of 16 columns; each covers both rank n-tiles of
// every chunk over the 4 token k-steps of a tile.
// ------------------------------------------------------------------------------------------------
struct DaChunk {
    const float *dLow;
    float *dA;
    float scaling;
    int R, r0;
};
struct DaParams {
    const float *X;
    int T, K, n, tok_per_group;
    DaChunk c[kMaxChunks];
};

__global__ void __launch_bounds__(256, 3) k_lora_da_tc(const DaParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem;
    uint8_t *Ls = dyn_smem + kXsBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int T = p.T, K = p.K;
    const int k0 = blockIdx.x * TC;
    const int tg0 = blockIdx.y * p.tok_per_group, tg1 = min(T, tg0 + p.tok_per_group);
    const int m0 = warp * 16;
    pdl_wait();
    pdl_trigger();
    float acc[kMaxChunks][2][4];
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++)
#pragma unroll
        for (int i = 0; i < 2; i++) acc[j][i][0] = acc[j][i][1] = acc[j][i][2] = acc[j][i][3] = 0.f;
    const uint32_t xs = smem_u32(Xs), ls = smem_u32(Ls);
    float4 v[NI];
    tile_load(p.X, K, tg0, tg1, k0, v, tid);
    for (int ts = tg0; ts < tg1; ts += TT) {
        __syncthreads();
        tile_store(v, ts, tg1, k0, Xs, nullptr, 0, tid);
        if (ts + TT < tg1) tile_load(p.X, K, ts + TT, tg1, k0, v, tid);      // next tile's loads fly during the MMAs below
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const DaChunk c = p.c[j];
                rank_tile_store(c.dLow, c.R, ts, tg1, c.r0, min(16, c.R - c.r0), TT, Ls + j * kLsBytes, tid);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < TT / 16; ks++) {
            uint32_t a[4];
            ldsm_x4_t(lm_a_km(xs, GSB, m0, ks * 16, lane), a);       // X^T: m = column of X, k = token
#pragma unroll
            for (int j = 0; j < kMaxChunks; j++) {
                if (j < p.n) {
                    uint32_t b[4];
                    ldsm_x4_t(lm_b_kn(ls + j * kLsBytes, RSB, 0, ks * 16, lane), b);
                    mma_bf16(acc[j][0], a, b[0], b[1]);
                    mma_bf16(acc[j][1], a, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j >= p.n) break;
        const DaChunk c = p.c[j];
        const int rc = min(16, c.R - c.r0);
#pragma unroll
        for (int i = 0; i < 2; i++) frag_atomic_add(c.dA + c.r0, c.R, acc[j][i], k0 + m0 + g, K, i * 8 + 2 * t4, rc, c.scaling);
    }
}

// token groups so that (column strips x groups) covers the SMs about twice; groups are whole 64-token tiles
void pick_groups(int strips, int T, int &groups, int &tpg) {
    static const int waves = [] {
        const char *v = getenv("GT_LORA_WAVES");
        return v ? atoi(v) : 2;
    }();
    groups = (waves * 148 + strips - 1) / (strips > 0 ? strips : 1);
    const int max_groups = (T + TT - 1) / TT;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1) groups = 1;
    tpg = (T + groups - 1) / groups;
    tpg = (tpg + TT - 1) / TT * TT;
    groups = (T + tpg - 1) / tpg;
}

cudaError_t allow_dyn_smem() {
    static cudaError_t done = [] {
        cudaError_t e = cudaFuncSetAttribute(k_lora_xa_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kXsBytes + kMaxChunks * kAsBytes));
        if (e != cudaSuccess) return e;
        return cudaFuncSetAttribute(k_lora_da_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kXsBytes + kMaxChunks * kLsBytes));
    }();
    return done;
}

}  // namespace

static void set_fills(FillList &fl, const RowFill *fills, int n_fills, int T) {
    fl.n = 0;
    for (int j = 0; j < n_fills && fl.n < kMaxChunks; j++)
        fl.f[fl.n++] = FillList::Job{fills[j].dst, fills[j].bias, fills[j].N, (int64_t)T * fills[j].N};
}

cudaError_t launch_lora_xa_group(const float *X, const LoraXaJob *jobs, int n, void *x16, int ldx16, int fp16, int T, int K,
                                 const RowFill *fills, int n_fills, cudaStream_t s) {
    if (T <= 0 || K <= 0 || n <= 0) return cudaSuccess;
    cudaError_t e = allow_dyn_smem();
    if (e != cudaSuccess) return e;
    dim3 grid((T + TT - 1) / TT, (K + TC - 1) / TC);
    XaParams p{};
    p.X = X;
    p.x16 = (uint16_t *)x16;      // written by the first launch only
    p.ldx16 = ldx16;
    (void)fp16;      // bf16 math mode only: the shared-memory tile and the 16-bit copy are the same bf16 values
    p.T = T;
    p.K = K;
    set_fills(p.fills, fills, n_fills, T);      // carried by the first launch
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_xa_tc, grid, dim3(256), kXsBytes + p.n * kAsBytes, s, p);
        p.n = 0;
        p.x16 = nullptr;
        p.fills.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = XaChunk{jobs[j].A, jobs[j].low_zeroed, jobs[j].R, r0};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

cudaError_t launch_lora_dy_group(const LoraDyJob *jobs, int n, int fp16, int T, const RowFill *fills, int n_fills, cudaStream_t s) {
    if (T <= 0 || n <= 0) return cudaSuccess;
    int strips_sum = 0, strips_max = 0;
    for (int j = 0; j < n; j++) {
        const int st = (jobs[j].N + TC - 1) / TC;
        strips_sum += st;
        strips_max = st > strips_max ? st : strips_max;
    }
    int groups, tpg;
    pick_groups(strips_sum, T, groups, tpg);
    DyParams p{};
    p.T = T;
    (void)fp16;
    p.tok_per_group = tpg;
    set_fills(p.fills, fills, n_fills, T);      // carried by the first launch
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_dy_tc, dim3(strips_max, groups, p.n), dim3(256), 0, s, p);
        p.n = 0;
        p.fills.n = 0;
        return le;
    };
    cudaError_t e;
    // rank chunk 0 of every member first (it also writes the 16-bit copy of dY), then the higher chunks
    for (int r0 = 0;; r0 += 16) {
        bool any = false;
        for (int j = 0; j < n; j++) {
            const LoraDyJob &b = jobs[j];
            if (r0 >= b.R || b.N <= 0) continue;
            any = true;
            DyMember m{};
            m.dY = b.dY; m.low = b.low; m.B = b.B; m.dB = b.dB; m.dLow = b.dLow_zeroed; m.dy16 = (uint16_t *)b.dy16;
            m.ld16 = b.ld16; m.N = b.N; m.R = b.R; m.r0 = r0; m.scaling = b.scaling;
            p.m[p.n++] = m;
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
        if (!any) break;
    }
    return flush();
}

cudaError_t launch_lora_da_group(const float *X, const LoraDaJob *jobs, int n, int T, int K, cudaStream_t s) {
    if (T <= 0 || K <= 0 || n <= 0) return cudaSuccess;
    cudaError_t e = allow_dyn_smem();
    if (e != cudaSuccess) return e;
    const int strips = (K + TC - 1) / TC;
    int groups, tpg;
    pick_groups(strips, T, groups, tpg);
    DaParams p{};
    p.X = X;
    p.T = T;
    p.K = K;
    p.tok_per_group = tpg;
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_da_tc, dim3(strips, groups), dim3(256), kXsBytes + p.n * kLsBytes, s, p);
        p.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = DaChunk{jobs[j].dLow, jobs[j].dA, jobs[j].scaling, jobs[j].R, r0};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

cudaError_t launch_lora_xa_tc(const float *X, const float *A, float *low_zeroed, void *x16, int ldx16, int fp16, int T, int K,
                              int R, cudaStream_t s) {
    if (R <= 0) return cudaSuccess;
    const LoraXaJob job{A, low_zeroed, R};
    return launch_lora_xa_group(X, &job, 1, x16, ldx16, fp16, T, K, nullptr, 0, s);
}

cudaError_t launch_lora_dy_tc(const float *dY, const float *low, const float *B, float *dB, float *dLow_zeroed, void *dy16,
                              int ld16, int fp16, float scaling, int T, int N, int R, cudaStream_t s) {
    if (N <= 0 || R <= 0) return cudaSuccess;
    const LoraDyJob job{dY, low, B, dB, dLow_zeroed, dy16, ld16, scaling, N, R};
    return launch_lora_dy_group(&job, 1, fp16, T, nullptr, 0, s);
}

cudaError_t launch_lora_da_tc(const float *X, const float *dLow, float *dA, float scaling, int T, int K, int R, cudaStream_t s) {
    if (R <= 0) return cudaSuccess;
    const LoraDaJob job{dLow, dA, scaling, R};
    return launch_lora_da_group(X, &job, 1, T, K, s);
}

}  // namespace gt
