// Rank-r LoRA products for the bf16 math mode, one pass over each activation tensor:
//   k_lora_xa_tc   low[T,R]  += X[T,K] * A[K,R]                       (+ 16-bit copy of X for the base GEMM)
//   k_lora_dy_tc   dLow[T,R] += dY[T,N] * B[R,N]^T ; dB[R,N] += s * low^T * dY   (+ 16-bit copy of dY)
//   k_lora_da_tc   dA[K,R]   += s * X[T,K]^T * dLow[T,R]
// They replace the host loops of src/Glacier.Tune/Kernels/LoraKernels.cs:35-54,191-291.  Operands are rounded to
// TF32 (10-bit mantissa, round to nearest) when they are staged in shared memory, products accumulate in fp32 in
// warp-level m16n8k8 MMAs, and partial sums leave the block through fp32 atomics; the exact-fp32 CUDA-core versions
// in gt_fp32_kernels.cu serve the validation modes.  A launch handles up to three 16-rank chunks: the adapters of
// projections that share their input (q, k, v; gate, up) go through one pass over X, and the dY passes of a group's
// members are one launch (blockIdx.z picks the member).
//
// These kernels are bound by the HBM read of X / dY, not by arithmetic: the tile in shared memory is read once
// from global memory and reused by every product that needs it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gt_internal.h"
#include "gt_ptx.cuh"

namespace gt {

namespace {

__device__ __forceinline__ uint32_t to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int fp16) {
    if (fp16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

constexpr int TT = 64;     // tokens per tile
constexpr int TC = 128;    // columns (of K or N) per tile
constexpr int GS = TC + 4; // smem row stride of the activation tile (words): rows 4 banks apart
constexpr int RS = 24;     // smem row stride of the 16-wide rank tiles (words)

constexpr int NI = (TT * TC / 4) / 256;     // float4 loads per thread and tile
constexpr int kMaxChunks = 3;               // 16-rank chunks (of one or several adapters) served by one launch

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
//   tile_load   global -> registers (float4 per thread when the tile is interior and aligned)
//   tile_store  registers -> shared memory as TF32, and optionally the 16-bit rounding to dst16 in global memory
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
__device__ __forceinline__ void tile_store(const float4 (&v)[NI], int t0, int t_end, int c0, uint32_t (*tile)[GS],
                                           uint16_t *__restrict__ dst16, int ld16, int fp16, int tid) {
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 4), c = (idx % (TC / 4)) * 4;
        const int t = t0 + r;
        if (dst16 && t < t_end) {
            uint16_t *q = dst16 + (int64_t)t * ld16 + c0 + c;
            if (c0 + c + 3 < ld16 && (ld16 & 3) == 0) {
                *reinterpret_cast<uint2 *>(q) = make_uint2(pack16(v[i].x, v[i].y, fp16), pack16(v[i].z, v[i].w, fp16));
            } else {
                const float e[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                for (int j = 0; j < 4; j++)
                    if (c0 + c + j < ld16) q[j] = (uint16_t)(pack16(e[j], 0.f, fp16) & 0xFFFFu);
            }
        }
        *reinterpret_cast<uint4 *>(&tile[r][c]) = make_uint4(to_tf32(v[i].x), to_tf32(v[i].y), to_tf32(v[i].z), to_tf32(v[i].w));
    }
}

// ------------------------------------------------------------------------------------------------
// low_j[T, R_j] += X[T, K] * A_j[K, R_j] over the block's K slice (grid.y slices of 128) for up to kMaxChunks
// 16-rank chunks that share X (the adapters of q, k, v or of gate, up): X is read and rounded once, fp32 atomics
// into each low_j (pre-zeroed).  8 warps = 4 token m-tiles x 2 rank n-tiles per chunk, 16 k-steps each.
// ------------------------------------------------------------------------------------------------
struct XaChunk {
    const float *A;
    float *low;
    int R, r0;
};
struct XaParams {
    const float *X;
    uint16_t *x16;
    int ldx16, fp16, T, K, n;
    XaChunk c[kMaxChunks];
    FillList fills;
};

__global__ void __launch_bounds__(256) k_lora_xa_tc(const XaParams p) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    uint32_t (*Xs)[GS] = reinterpret_cast<uint32_t (*)[GS]>(dyn_smem);
    uint32_t (*As)[TC][RS] = reinterpret_cast<uint32_t (*)[TC][RS]>(dyn_smem + TT * GS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.x * TT, k0 = blockIdx.y * TC;
    const int T = p.T, K = p.K;
    pdl_wait();
    pdl_trigger();
    float4 v[NI];
    tile_load(p.X, K, t0, T, k0, v, tid);
    float av[kMaxChunks][8];       // this thread's 8 elements of each chunk's [128 x 16] tile of A, in flight with X
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j < p.n) {
            const XaChunk c = p.c[j];
            const int rc = min(16, c.R - c.r0);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int idx = tid + i * 256, k = idx >> 4, r = idx & 15;
                av[j][i] = (k0 + k < K && r < rc) ? __ldg(&c.A[(int64_t)(k0 + k) * c.R + c.r0 + r]) : 0.f;
            }
        }
    }
    tile_store(v, t0, T, k0, Xs, p.x16, p.ldx16, p.fp16, tid);
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j < p.n) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int idx = tid + i * 256;
                As[j][idx >> 4][idx & 15] = to_tf32(av[j][i]);
            }
        }
    }
    __syncthreads();
    const int m0 = (warp >> 1) * 16, n0 = (warp & 1) * 8;
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j >= p.n) break;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < TC / 8; ks++) {
            const int kk = ks * 8;
            mma_tf32(d, Xs[m0 + g][kk + t4], Xs[m0 + g + 8][kk + t4], Xs[m0 + g][kk + t4 + 4], Xs[m0 + g + 8][kk + t4 + 4],
                     As[j][kk + t4][n0 + g], As[j][kk + t4 + 4][n0 + g]);
        }
        const XaChunk c = p.c[j];
        const int rc = min(16, c.R - c.r0);
        const int ta = t0 + m0 + g, tb = ta + 8, ra = n0 + 2 * t4;
        if (ta < T) {
            if (ra < rc) atomicAdd(&c.low[(int64_t)ta * c.R + c.r0 + ra], d[0]);
            if (ra + 1 < rc) atomicAdd(&c.low[(int64_t)ta * c.R + c.r0 + ra + 1], d[1]);
        }
        if (tb < T) {
            if (ra < rc) atomicAdd(&c.low[(int64_t)tb * c.R + c.r0 + ra], d[2]);
            if (ra + 1 < rc) atomicAdd(&c.low[(int64_t)tb * c.R + c.r0 + ra + 1], d[3]);
        }
    }
    do_fills(p.fills, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y, tid);
}

// ------------------------------------------------------------------------------------------------
// One pass over dY_m per member m = blockIdx.z: the block owns a 128-column strip and a token group, walked in
// 64-token tiles.
//   dLow[t, r] += sum_c dY[t, c] * B[r, c]      4 m-tiles (tokens) x 2 n-tiles (ranks) over 8 warps, 16 k-steps
//   dB[r, c]   += s * sum_t low[t, r] * dY[t, c] 1 m-tile (ranks) x 16 n-tiles (columns), 2 per warp, 8 k-steps
// ------------------------------------------------------------------------------------------------
struct DyMember {
    const float *dY, *low, *B;
    float *dB, *dLow;
    uint16_t *dy16;
    int ld16, N, R, r0;
    float scaling;
};
struct DyParams {
    int T, fp16, tok_per_group, n;
    DyMember m[kMaxChunks];
    FillList fills;
};

__global__ void __launch_bounds__(256) k_lora_dy_tc(const DyParams p) {
    __shared__ __align__(16) uint32_t Gs[TT][GS];
    __shared__ uint32_t Bs[16][GS];
    __shared__ uint32_t Ls[TT][RS];
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
    for (int i = tid; i < 16 * TC; i += 256) {
        const int r = i / TC, c = i % TC;
        Bs[r][c] = (r < rc && c0 + c < N) ? to_tf32(__ldg(&m.B[(int64_t)(r0 + r) * N + c0 + c])) : 0u;
    }
    float accB[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int m0 = (warp >> 1) * 16, n0 = (warp & 1) * 8;      // dLow tiles
    const int cb = warp * 16;                                  // dB: this warp's two 8-column n-tiles
    uint16_t *dy16 = r0 == 0 ? m.dy16 : nullptr;
    for (int ts = tg0; ts < tg1; ts += TT) {
        __syncthreads();
        tile_store(v, ts, tg1, c0, Gs, dy16, m.ld16, p.fp16, tid);
        if (ts + TT < tg1) tile_load(m.dY, N, ts + TT, tg1, c0, v, tid);     // next tile's loads fly during the MMAs below
        for (int i = tid; i < TT * 16; i += 256) {
            const int tt = i >> 4, r = i & 15;
            Ls[tt][r] = (ts + tt < tg1 && r < rc) ? to_tf32(m.low[(int64_t)(ts + tt) * R + r0 + r]) : 0u;
        }
        __syncthreads();
        {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < TC / 8; ks++) {
                const int kk = ks * 8;
                mma_tf32(d, Gs[m0 + g][kk + t4], Gs[m0 + g + 8][kk + t4], Gs[m0 + g][kk + t4 + 4], Gs[m0 + g + 8][kk + t4 + 4],
                         Bs[n0 + g][kk + t4], Bs[n0 + g][kk + t4 + 4]);
            }
            const int ta = ts + m0 + g, tb = ta + 8, ra = n0 + 2 * t4;
            if (ta < tg1) {
                if (ra < rc) atomicAdd(&m.dLow[(int64_t)ta * R + r0 + ra], d[0]);
                if (ra + 1 < rc) atomicAdd(&m.dLow[(int64_t)ta * R + r0 + ra + 1], d[1]);
            }
            if (tb < tg1) {
                if (ra < rc) atomicAdd(&m.dLow[(int64_t)tb * R + r0 + ra], d[2]);
                if (ra + 1 < rc) atomicAdd(&m.dLow[(int64_t)tb * R + r0 + ra + 1], d[3]);
            }
        }
#pragma unroll
        for (int ks = 0; ks < TT / 8; ks++) {
            const int kk = ks * 8;      // token index inside the tile
            const uint32_t a0 = Ls[kk + t4][g], a1 = Ls[kk + t4][g + 8], a2 = Ls[kk + t4 + 4][g], a3 = Ls[kk + t4 + 4][g + 8];
#pragma unroll
            for (int j = 0; j < 2; j++)
                mma_tf32(accB[j], a0, a1, a2, a3, Gs[kk + t4][cb + j * 8 + g], Gs[kk + t4 + 4][cb + j * 8 + g]);
        }
    }
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int c = c0 + cb + j * 8 + 2 * t4;
        const int ra = g, rb = g + 8;
        if (c < N) {
            if (ra < rc) atomicAdd(&m.dB[(int64_t)(r0 + ra) * N + c], accB[j][0] * m.scaling);
            if (rb < rc) atomicAdd(&m.dB[(int64_t)(r0 + rb) * N + c], accB[j][2] * m.scaling);
        }
        if (c + 1 < N) {
            if (ra < rc) atomicAdd(&m.dB[(int64_t)(r0 + ra) * N + c + 1], accB[j][1] * m.scaling);
            if (rb < rc) atomicAdd(&m.dB[(int64_t)(r0 + rb) * N + c + 1], accB[j][3] * m.scaling);
        }
    }
    do_fills(p.fills, lb, nb, tid);
}

// ------------------------------------------------------------------------------------------------
// dA_j[k, r] += s_j * sum_t X[t, k] * dLow_j[t, r] for up to kMaxChunks 16-rank chunks that share X: the block owns
// a 128-column strip of X and a token group.  8 warps = 8 m-tiles of 16 columns; each covers both rank n-tiles of
// every chunk over the 8 token k-steps of a tile.
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
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    uint32_t (*Xs)[GS] = reinterpret_cast<uint32_t (*)[GS]>(dyn_smem);
    uint32_t (*Ls)[TT][RS] = reinterpret_cast<uint32_t (*)[TT][RS]>(dyn_smem + TT * GS);
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
    float4 v[NI];
    tile_load(p.X, K, tg0, tg1, k0, v, tid);
    for (int ts = tg0; ts < tg1; ts += TT) {
        __syncthreads();
        tile_store(v, ts, tg1, k0, Xs, nullptr, 0, 0, tid);
        if (ts + TT < tg1) tile_load(p.X, K, ts + TT, tg1, k0, v, tid);      // next tile's loads fly during the MMAs below
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const DaChunk c = p.c[j];
                const int rc = min(16, c.R - c.r0);
                for (int i = tid; i < TT * 16; i += 256) {
                    const int tt = i >> 4, r = i & 15;
                    Ls[j][tt][r] = (ts + tt < tg1 && r < rc) ? to_tf32(c.dLow[(int64_t)(ts + tt) * c.R + c.r0 + r]) : 0u;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < TT / 8; ks++) {
            const int kk = ks * 8;
            const uint32_t a0 = Xs[kk + t4][m0 + g], a1 = Xs[kk + t4][m0 + g + 8], a2 = Xs[kk + t4 + 4][m0 + g],
                           a3 = Xs[kk + t4 + 4][m0 + g + 8];
#pragma unroll
            for (int j = 0; j < kMaxChunks; j++) {
                if (j < p.n) {
#pragma unroll
                    for (int i = 0; i < 2; i++)
                        mma_tf32(acc[j][i], a0, a1, a2, a3, Ls[j][kk + t4][i * 8 + g], Ls[j][kk + t4 + 4][i * 8 + g]);
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
        for (int i = 0; i < 2; i++) {
            const int ka = k0 + m0 + g, kb = ka + 8, r = i * 8 + 2 * t4;
            if (ka < K) {
                if (r < rc) atomicAdd(&c.dA[(int64_t)ka * c.R + c.r0 + r], acc[j][i][0] * c.scaling);
                if (r + 1 < rc) atomicAdd(&c.dA[(int64_t)ka * c.R + c.r0 + r + 1], acc[j][i][1] * c.scaling);
            }
            if (kb < K) {
                if (r < rc) atomicAdd(&c.dA[(int64_t)kb * c.R + c.r0 + r], acc[j][i][2] * c.scaling);
                if (r + 1 < rc) atomicAdd(&c.dA[(int64_t)kb * c.R + c.r0 + r + 1], acc[j][i][3] * c.scaling);
            }
        }
    }
}

// token groups so that (column strips x groups) covers the SMs about twice; groups are whole 64-token tiles
void pick_groups(int strips, int T, int &groups, int &tpg) {
    groups = (2 * 148 + strips - 1) / (strips > 0 ? strips : 1);
    const int max_groups = (T + TT - 1) / TT;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1) groups = 1;
    tpg = (T + groups - 1) / groups;
    tpg = (tpg + TT - 1) / TT * TT;
    groups = (T + tpg - 1) / tpg;
}

constexpr size_t kXsBytes = (size_t)TT * GS * 4;
constexpr size_t kAsBytes = (size_t)TC * RS * 4;       // per chunk, k_lora_xa_tc
constexpr size_t kLsBytes = (size_t)TT * RS * 4;       // per chunk, k_lora_da_tc

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
    p.fp16 = fp16;
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
    p.fp16 = fp16;
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
