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
// The same tile through a two-slot ring in shared memory filled with 16-byte cp.async copies: a block keeps the loads of
// its next TWO tiles in flight while it works on the current one (with one tile of prefetch in registers the loop ran
// at one round of DRAM latency per tile).  Thread `tid` owns pieces tid + 256 i of a slot, writes them (cp.async) and
// reads them back itself, so a slot needs no barrier; only interior, 16-byte-aligned tiles take this path.
constexpr int kRingSlotBytes = TT * TC * 4;       // 32 KiB: one fp32 tile
constexpr int kRingBytes = 2 * kRingSlotBytes;
__device__ __forceinline__ void tile_issue(const float *__restrict__ src, int ncols, int t0, int t_end, int c0, uint32_t slot, int tid) {
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 4), c = (idx % (TC / 4)) * 4;
        const int t = t0 + r;
        const bool ok = t < t_end;
        const float *p = src + (int64_t)(ok ? t : t0) * ncols + c0 + c;      // rows past the end: zero-filled, nothing read
        const uint32_t nbytes = ok ? 16u : 0u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(slot + (uint32_t)idx * 16u), "l"(p), "r"(nbytes) : "memory");
    }
}
__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ring_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void tile_take(uint32_t slot, float4 (&v)[NI], int tid) {
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const uint32_t a = slot + (uint32_t)(tid + i * 256) * 16u;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[i].x), "=f"(v[i].y), "=f"(v[i].z), "=f"(v[i].w) : "r"(a) : "memory");
    }
}
// every tile of columns [c_begin, c_end) of src[., ncols] is interior and 16-byte aligned
__device__ __forceinline__ bool ring_ok(int enabled, const float *src, int ncols, int c_end) {
    return enabled != 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (ncols & 3) == 0 && c_end <= ncols;
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

// Four consecutive floats src[row, col .. col + 3] of a row-major matrix with `ld` columns; zero at and beyond
// col_end or when the row is not valid.  `vec`: rows are 16-byte aligned and ld is a multiple of 4.
__device__ __forceinline__ float4 ld4(const float *__restrict__ src, int64_t row, int ld, int col, int col_end, bool row_ok, bool vec) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!row_ok || col >= col_end) return r;
    const float *p = src + row * ld + col;
    if (vec && col + 3 < col_end) return __ldg(reinterpret_cast<const float4 *>(p));
    r.x = __ldg(p);
    if (col + 1 < col_end) r.y = __ldg(p + 1);
    if (col + 2 < col_end) r.z = __ldg(p + 2);
    if (col + 3 < col_end) r.w = __ldg(p + 3);
    return r;
}
__device__ __forceinline__ void st_bf16x4(uint8_t *dst, const float4 &v) {
    *reinterpret_cast<uint2 *>(dst) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// ------------------------------------------------------------------------------------------------
// low_j[T, R_j] += X[T, K] * A_j[K, R_j] for up to kMaxChunks 16-rank chunks that share X (the adapters of q, k, v or
// of gate, up).  A block owns one 64-token tile and a run of 128-column strips of X: it walks the strips with the
// next strip's X tile and A tiles in flight in registers, keeps its [64 x 16] partial sums of every chunk in
// registers across the strips, and adds them into low_j (pre-zeroed) once at the end - a low element receives one
// atomic add per block that shares its tokens, not one per strip.  X is read and rounded once; its bf16 copy goes
// to x16.  8 warps = 4 token m-tiles x 2 halves of a strip's 8 k-steps; each warp covers both rank n-tiles.
// ------------------------------------------------------------------------------------------------
struct XaChunk {
    const float *A;
    float *low;
    int R, r0, vec;
};
struct XaParams {
    const float *X;
    uint16_t *x16;
    int ldx16, T, K, n, strips_per_block, ring;
    XaChunk c[kMaxChunks];
    FillList fills;
};
constexpr int kXsBytes = TT * GSB;            // activation tile
constexpr int kAsBytes = TC * RSB;            // per chunk, k_lora_xa_tc: A[k0.., r0..] as [128][16]
constexpr int kLsBytes = TT * RSB;            // per chunk, k_lora_da_tc / k_lora_dy_tc: [64 tokens][16]

__global__ void __launch_bounds__(256, 2) k_lora_xa_tc(const XaParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem + kRingBytes;
    uint8_t *As = Xs + kXsBytes;
    const uint32_t ring = smem_u32(dyn_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int T = p.T, K = p.K;
    const int t0 = blockIdx.x * TT;
    const int n_strips = (K + TC - 1) / TC;
    const int s0 = blockIdx.y * p.strips_per_block, s1 = min(n_strips, s0 + p.strips_per_block);
    const bool use_ring = ring_ok(p.ring, p.X, K, s1 * TC);
    pdl_wait();
    pdl_trigger();
    float4 v[NI], av[kMaxChunks][2];
    // this thread's two float4 of every chunk's [128 x 16] tile of A: rows k0 + (tid + 256 i) / 4, columns 4 (tid % 4)
    auto a_load = [&](int k0) {
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const XaChunk c = p.c[j];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int idx = tid + i * 256, row = k0 + (idx >> 2);
                    av[j][i] = ld4(c.A + c.r0, row, c.R, (idx & 3) * 4, min(16, c.R - c.r0), row < K, c.vec != 0);
                }
            }
        }
    };
    if (use_ring) {
        tile_issue(p.X, K, t0, T, s0 * TC, ring, tid);
        ring_commit();
        if (s0 + 1 < s1) tile_issue(p.X, K, t0, T, (s0 + 1) * TC, ring + kRingSlotBytes, tid);
        ring_commit();
    } else {
        tile_load(p.X, K, t0, T, s0 * TC, v, tid);
    }
    a_load(s0 * TC);
    float d[kMaxChunks][2][4];
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++)
#pragma unroll
        for (int i = 0; i < 2; i++) d[j][i][0] = d[j][i][1] = d[j][i][2] = d[j][i][3] = 0.f;
    const int m0 = (warp >> 1) * 16, kh = (warp & 1) * 64;
    const uint32_t xs = smem_u32(Xs), as = smem_u32(As);
    for (int s = s0; s < s1; s++) {
        const uint32_t slot = ring + (uint32_t)((s - s0) & 1) * kRingSlotBytes;
        if (use_ring) {
            ring_wait_all_but_one();
            tile_take(slot, v, tid);
        }
        __syncthreads();
        tile_store(v, t0, T, s * TC, Xs, p.x16, p.ldx16, tid);
        if (use_ring) {      // the slot's values are in registers and used: refill it with the tile after the next one
            if (s + 2 < s1) tile_issue(p.X, K, t0, T, (s + 2) * TC, slot, tid);
            ring_commit();
        }
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int idx = tid + i * 256;
                    st_bf16x4(As + j * kAsBytes + (idx >> 2) * RSB + (idx & 3) * 8, av[j][i]);
                }
            }
        }
        if (s + 1 < s1) {      // the next strip's loads fly during the MMAs below
            if (!use_ring) tile_load(p.X, K, t0, T, (s + 1) * TC, v, tid);
            a_load((s + 1) * TC);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t a[4];
            ldsm_x4(lm_a_mk(xs, GSB, m0, kh + ks * 16, lane), a);
#pragma unroll
            for (int j = 0; j < kMaxChunks; j++) {
                if (j < p.n) {
                    uint32_t b[4];
                    ldsm_x4_t(lm_b_kn(as + j * kAsBytes, RSB, 0, kh + ks * 16, lane), b);
                    mma_bf16(d[j][0], a, b[0], b[1]);
                    mma_bf16(d[j][1], a, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j >= p.n) break;
        const XaChunk c = p.c[j];
        const int rc = min(16, c.R - c.r0);
#pragma unroll
        for (int i = 0; i < 2; i++) frag_atomic_add(c.low + c.r0, c.R, d[j][i], t0 + m0 + g, T, i * 8 + 2 * t4, rc, 1.f);
    }
    do_fills(p.fills, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y, tid);
}

// ------------------------------------------------------------------------------------------------
// The same product from an input that already exists as bf16: low_j[T, R_j] += X16[T, K] * A_j.  Used where the pass
// that produced X wrote its 16-bit copy itself (the SwiGLU kernel emits bf16(SiLU(gate) * up) for the down projection),
// so this pass reads 2 bytes per element instead of 4 and writes no copy.  Same tiling as k_lora_xa_tc; the tile
// travels global -> registers -> shared memory as 16-byte pieces (8 values), the next strip's pieces in flight during
// the MMAs.  Needs K % 8 == 0 and a 16-byte-aligned X16.
// ------------------------------------------------------------------------------------------------
constexpr int NI16 = (TT * TC / 8) / 256;      // 16-byte pieces per thread and tile
__device__ __forceinline__ void tile_load16(const uint16_t *__restrict__ src, int ld, int K, int t0, int T, int c0, uint4 (&v)[NI16], int tid) {
#pragma unroll
    for (int i = 0; i < NI16; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 8), c = (idx % (TC / 8)) * 8;
        const int t = t0 + r;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (t < T && c0 + c < K) v[i] = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)t * ld + c0 + c));
    }
}
__device__ __forceinline__ void tile_store16(const uint4 (&v)[NI16], uint8_t *tile, int tid) {
#pragma unroll
    for (int i = 0; i < NI16; i++) {
        const int idx = tid + i * 256;
        const int r = idx / (TC / 8), c = (idx % (TC / 8)) * 8;
        *reinterpret_cast<uint4 *>(tile + r * GSB + c * 2) = v[i];
    }
}
struct Xa16Params {
    const uint16_t *X16;
    int ld, T, K, n, strips_per_block;
    XaChunk c[kMaxChunks];
};
__global__ void __launch_bounds__(256, 2) k_lora_xa16_tc(const Xa16Params p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem;
    uint8_t *As = Xs + kXsBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int T = p.T, K = p.K;
    const int t0 = blockIdx.x * TT;
    const int n_strips = (K + TC - 1) / TC;
    const int s0 = blockIdx.y * p.strips_per_block, s1 = min(n_strips, s0 + p.strips_per_block);
    pdl_wait();
    pdl_trigger();
    uint4 v[NI16];
    float4 av[kMaxChunks][2];
    auto a_load = [&](int k0) {
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const XaChunk c = p.c[j];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int idx = tid + i * 256, row = k0 + (idx >> 2);
                    av[j][i] = ld4(c.A + c.r0, row, c.R, (idx & 3) * 4, min(16, c.R - c.r0), row < K, c.vec != 0);
                }
            }
        }
    };
    tile_load16(p.X16, p.ld, K, t0, T, s0 * TC, v, tid);
    a_load(s0 * TC);
    float d[kMaxChunks][2][4];
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++)
#pragma unroll
        for (int i = 0; i < 2; i++) d[j][i][0] = d[j][i][1] = d[j][i][2] = d[j][i][3] = 0.f;
    const int m0 = (warp >> 1) * 16, kh = (warp & 1) * 64;
    const uint32_t xs = smem_u32(Xs), as = smem_u32(As);
    for (int s = s0; s < s1; s++) {
        __syncthreads();
        tile_store16(v, Xs, tid);
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int idx = tid + i * 256;
                    st_bf16x4(As + j * kAsBytes + (idx >> 2) * RSB + (idx & 3) * 8, av[j][i]);
                }
            }
        }
        if (s + 1 < s1) {
            tile_load16(p.X16, p.ld, K, t0, T, (s + 1) * TC, v, tid);
            a_load((s + 1) * TC);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t a[4];
            ldsm_x4(lm_a_mk(xs, GSB, m0, kh + ks * 16, lane), a);
#pragma unroll
            for (int j = 0; j < kMaxChunks; j++) {
                if (j < p.n) {
                    uint32_t b[4];
                    ldsm_x4_t(lm_b_kn(as + j * kAsBytes, RSB, 0, kh + ks * 16, lane), b);
                    mma_bf16(d[j][0], a, b[0], b[1]);
                    mma_bf16(d[j][1], a, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxChunks; j++) {
        if (j >= p.n) break;
        const XaChunk c = p.c[j];
        const int rc = min(16, c.R - c.r0);
#pragma unroll
        for (int i = 0; i < 2; i++) frag_atomic_add(c.low + c.r0, c.R, d[j][i], t0 + m0 + g, T, i * 8 + 2 * t4, rc, 1.f);
    }
}

// ------------------------------------------------------------------------------------------------
// One pass over dY_m per member m = blockIdx.z.  A block owns one 64-token tile and a run of 128-column strips of
// dY: it walks the strips with the next strip's dY tile and B tile in flight in registers.
//   dLow[t, r] += sum_c dY[t, c] * B[r, c]      kept in registers across the strips, one atomic add per element and
//                                               block at the end; 8 warps = 4 token m-tiles x 2 halves of a strip's
//                                               8 k-steps, both rank n-tiles per warp
//   dB[r, c]   += s * sum_t low[t, r] * dY[t, c] per strip: 1 m-tile (ranks) x 16 n-tiles (columns), 2 per warp,
//                                               4 token k-steps; added into dB after every strip (one add per
//                                               element and token tile)
// The low tile of the block's tokens is staged once.  The bf16 copy of dY goes to dy16.
// ------------------------------------------------------------------------------------------------
struct DyMember {
    const float *dY, *low, *B;
    float *dB, *dLow;
    uint16_t *dy16;
    int ld16, N, R, r0, vec_b, vec_low;
    float scaling;
};
struct DyParams {
    int T, strips_per_block, n, ring;
    DyMember m[kMaxChunks];
    FillList fills;
};

// IN16: the members' dY exists as bf16 already (dy16, written by the pass that produced it): the tile is read from there,
// 2 bytes per element, and no copy is written.
constexpr int kDySmemBytes = kRingBytes + TT * GSB + 16 * GSB + TT * RSB;
template <bool IN16>
__global__ void __launch_bounds__(256, 2) k_lora_dy_tc(const DyParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Gs = dyn_smem + kRingBytes;      // dY tile, bf16
    uint8_t *Bs = Gs + TT * GSB;              // B[r0.., c0..] as [16][128]
    uint8_t *Ls = Bs + 16 * GSB;              // low tile [64][16]
    const uint32_t ring = smem_u32(dyn_smem);
    pdl_wait();
    pdl_trigger();
    const DyMember m = p.m[blockIdx.z];
    const int N = m.N, R = m.R, r0 = m.r0, T = p.T;
    const int n_strips = (N + TC - 1) / TC;
    const int s0 = blockIdx.x * p.strips_per_block, s1 = min(n_strips, s0 + p.strips_per_block);
    const int lb = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, nb = gridDim.x * gridDim.y * gridDim.z;
    if (s0 >= n_strips) {      // a member with fewer column strips than the widest one
        do_fills(p.fills, lb, nb, threadIdx.x);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.y * TT;
    const int rc = min(16, R - r0);
    float4 v[NI], bv[2];      // (the fp32 tile's registers are dead code with IN16, and the other way round)
    uint4 v16[NI16];
    // this thread's two float4 of the strip's [16 x 128] tile of B: rank (tid + 256 i) / 32, columns 4 ((tid + 256 i) % 32)
    auto b_load = [&](int c0) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int idx = tid + i * 256, r = idx >> 5;
            bv[i] = ld4(m.B, r0 + r, N, c0 + (idx & 31) * 4, N, r < rc, m.vec_b != 0);
        }
    };
    const bool use_ring = !IN16 && ring_ok(p.ring, m.dY, N, s1 * TC);
    if constexpr (IN16) {
        tile_load16(m.dy16, m.ld16, N, t0, T, s0 * TC, v16, tid);
    } else if (use_ring) {
        tile_issue(m.dY, N, t0, T, s0 * TC, ring, tid);
        ring_commit();
        if (s0 + 1 < s1) tile_issue(m.dY, N, t0, T, (s0 + 1) * TC, ring + kRingSlotBytes, tid);
        ring_commit();
    } else {
        tile_load(m.dY, N, t0, T, s0 * TC, v, tid);
    }
    b_load(s0 * TC);
    {
        const int row = tid >> 2;
        const float4 lv = ld4(m.low + r0, t0 + row, R, (tid & 3) * 4, rc, t0 + row < T, m.vec_low != 0);
        st_bf16x4(Ls + row * RSB + (tid & 3) * 8, lv);
    }
    const uint32_t gs = smem_u32(Gs), bs = smem_u32(Bs), ls = smem_u32(Ls);
    float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int m0 = (warp >> 1) * 16, kh = (warp & 1) * 64;    // dLow: token m-tile, half of the strip's columns
    const int cb = warp * 16;                                 // dB: this warp's two 8-column n-tiles
    uint16_t *dy16 = (!IN16 && r0 == 0) ? m.dy16 : nullptr;
    for (int s = s0; s < s1; s++) {
        const int c0 = s * TC;
        const uint32_t slot = ring + (uint32_t)((s - s0) & 1) * kRingSlotBytes;
        if (use_ring) {
            ring_wait_all_but_one();
            tile_take(slot, v, tid);
        }
        __syncthreads();
        if constexpr (IN16) tile_store16(v16, Gs, tid);
        else tile_store(v, t0, T, c0, Gs, dy16, m.ld16, tid);
        if (use_ring) {
            if (s + 2 < s1) tile_issue(m.dY, N, t0, T, (s + 2) * TC, slot, tid);
            ring_commit();
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int idx = tid + i * 256;
            st_bf16x4(Bs + (idx >> 5) * GSB + (idx & 31) * 8, bv[i]);
        }
        if (s + 1 < s1) {      // the next strip's loads fly during the MMAs below
            if constexpr (IN16) tile_load16(m.dy16, m.ld16, N, t0, T, (s + 1) * TC, v16, tid);
            else if (!use_ring) tile_load(m.dY, N, t0, T, (s + 1) * TC, v, tid);
            b_load((s + 1) * TC);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t a[4], b[4];
            ldsm_x4(lm_a_mk(gs, GSB, m0, kh + ks * 16, lane), a);
            ldsm_x4(lm_b_nk(bs, GSB, 0, kh + ks * 16, lane), b);
            mma_bf16(d[0], a, b[0], b[1]);
            mma_bf16(d[1], a, b[2], b[3]);
        }
        float accB[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < TT / 16; ks++) {
            uint32_t a[4], b[4];
            ldsm_x4_t(lm_a_km(ls, RSB, 0, ks * 16, lane), a);        // low^T: m = rank, k = token
            ldsm_x4_t(lm_b_kn(gs, GSB, cb, ks * 16, lane), b);       // dY: k = token, n = column
            mma_bf16(accB[0], a, b[0], b[1]);
            mma_bf16(accB[1], a, b[2], b[3]);
        }
        // accB rows = ranks, columns = strip columns
#pragma unroll
        for (int i = 0; i < 2; i++)
            frag_atomic_add(m.dB + (int64_t)r0 * N, N, accB[i], g, rc, c0 + cb + i * 8 + 2 * t4, N, m.scaling);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) frag_atomic_add(m.dLow + r0, R, d[i], t0 + m0 + g, T, i * 8 + 2 * t4, rc, 1.f);
    do_fills(p.fills, lb, nb, tid);
}

// ------------------------------------------------------------------------------------------------
// dA_j[k, r] += s_j * sum_t X[t, k] * dLow_j[t, r] for up to kMaxChunks 16-rank chunks that share X: the block owns
// a 128-column strip of X and a token group, walked in 64-token tiles with the next tile of X and of every dLow_j
// in flight in registers.  8 warps = 8 m-tiles of 16 columns; each covers both rank n-tiles of every chunk over the
// 4 token k-steps of a tile and keeps its sums in registers until the end.
// ------------------------------------------------------------------------------------------------
struct DaChunk {
    const float *dLow;
    float *dA;
    float scaling;
    int R, r0, vec;
};
struct DaParams {
    const float *X;
    int T, K, n, tok_per_group, ring;
    DaChunk c[kMaxChunks];
};

__global__ void __launch_bounds__(256, 2) k_lora_da_tc(const DaParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem + kRingBytes;
    uint8_t *Ls = Xs + kXsBytes;
    const uint32_t ring = smem_u32(dyn_smem);
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
    float4 v[NI], lv[kMaxChunks];
    // this thread's float4 of every chunk's [64 x 16] tile of dLow: token ts + tid / 4, ranks 4 (tid % 4)
    auto l_load = [&](int ts) {
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const DaChunk c = p.c[j];
                const int row = ts + (tid >> 2);
                lv[j] = ld4(c.dLow + c.r0, row, c.R, (tid & 3) * 4, min(16, c.R - c.r0), row < tg1, c.vec != 0);
            }
        }
    };
    const bool use_ring = ring_ok(p.ring, p.X, K, k0 + TC);
    if (use_ring) {
        tile_issue(p.X, K, tg0, tg1, k0, ring, tid);
        ring_commit();
        if (tg0 + TT < tg1) tile_issue(p.X, K, tg0 + TT, tg1, k0, ring + kRingSlotBytes, tid);
        ring_commit();
    } else {
        tile_load(p.X, K, tg0, tg1, k0, v, tid);
    }
    l_load(tg0);
    for (int ts = tg0, it = 0; ts < tg1; ts += TT, it++) {
        const uint32_t slot = ring + (uint32_t)(it & 1) * kRingSlotBytes;
        if (use_ring) {
            ring_wait_all_but_one();
            tile_take(slot, v, tid);
        }
        __syncthreads();
        tile_store(v, ts, tg1, k0, Xs, nullptr, 0, tid);
        if (use_ring) {
            if (ts + 2 * TT < tg1) tile_issue(p.X, K, ts + 2 * TT, tg1, k0, slot, tid);
            ring_commit();
        }
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++)
            if (j < p.n) st_bf16x4(Ls + j * kLsBytes + (tid >> 2) * RSB + (tid & 3) * 8, lv[j]);
        if (ts + TT < tg1) {      // the next tile's loads fly during the MMAs below
            if (!use_ring) tile_load(p.X, K, ts + TT, tg1, k0, v, tid);
            l_load(ts + TT);
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

// The same from an X that exists as bf16 (see k_lora_xa16_tc): 2 bytes per element read, no rounding pass.
struct Da16Params {
    const uint16_t *X16;
    int ld, T, K, n, tok_per_group;
    DaChunk c[kMaxChunks];
};
__global__ void __launch_bounds__(256, 2) k_lora_da16_tc(const Da16Params p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *Xs = dyn_smem;
    uint8_t *Ls = Xs + kXsBytes;
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
    uint4 v[NI16];
    float4 lv[kMaxChunks];
    auto l_load = [&](int ts) {
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++) {
            if (j < p.n) {
                const DaChunk c = p.c[j];
                const int row = ts + (tid >> 2);
                lv[j] = ld4(c.dLow + c.r0, row, c.R, (tid & 3) * 4, min(16, c.R - c.r0), row < tg1, c.vec != 0);
            }
        }
    };
    tile_load16(p.X16, p.ld, K, tg0, tg1, k0, v, tid);
    l_load(tg0);
    for (int ts = tg0; ts < tg1; ts += TT) {
        __syncthreads();
        tile_store16(v, Xs, tid);
#pragma unroll
        for (int j = 0; j < kMaxChunks; j++)
            if (j < p.n) st_bf16x4(Ls + j * kLsBytes + (tid >> 2) * RSB + (tid & 3) * 8, lv[j]);
        if (ts + TT < tg1) {      // the next tile's loads fly during the MMAs below
            tile_load16(p.X16, p.ld, K, ts + TT, tg1, k0, v, tid);
            l_load(ts + TT);
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

// Two blocks are resident per SM (registers and the 64 KiB ring): a launch should fit ONE wave of kSlots blocks, or a
// second, nearly empty wave doubles its time (400 blocks of 3 strips on 296 slots ran as 2 x 3 strips; 296 blocks of 4
// strips run as 1 x 4).
constexpr int kSlots = 2 * 148;
// token groups so that (column strips x groups) fills one wave; groups are whole 64-token tiles
void pick_groups(int strips, int T, int &groups, int &tpg) {
    groups = kSlots / (strips > 0 ? strips : 1);
    const int max_groups = (T + TT - 1) / TT;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1) groups = 1;
    tpg = (T + groups - 1) / groups;
    tpg = (tpg + TT - 1) / TT * TT;
    groups = (T + tpg - 1) / tpg;
}
// strips per block for the kernels that walk strips: the smallest run for which every member's chunks x token tiles x
// members fit one wave (`strips_max` = strips of the widest member, `members` = grid.z)
int pick_strip_run(int strips_max, int members, int T) {
    const int tiles = (T + TT - 1) / TT;
    int run = 1;
    while (run < strips_max && ((strips_max + run - 1) / run) * tiles * members > kSlots) run++;
    static const int forced = [] {
        const char *v = getenv("GT_LORA_RUN");
        return v ? atoi(v) : 0;
    }();
    if (forced > 0) run = forced;
    return run < 1 ? 1 : run;
}
// GT_LORA_RING=0 turns the cp.async ring off (one tile of prefetch in registers instead): a measurement knob
int ring_enabled() {
    static const int on = [] {
        const char *v = getenv("GT_LORA_RING");
        return (v && v[0] == '0') ? 0 : 1;
    }();
    return on;
}
inline int is_vec(const void *p, int ld) { return ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld & 3) == 0) ? 1 : 0; }

cudaError_t allow_dyn_smem() {
    static PerDeviceOnce configured;
    return per_device_once(configured, [] {
        cudaError_t e = cudaFuncSetAttribute(k_lora_xa_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kRingBytes + kXsBytes + kMaxChunks * kAsBytes));
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k_lora_dy_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDySmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_lora_dy_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDySmemBytes);
        if (e != cudaSuccess) return e;
        return cudaFuncSetAttribute(k_lora_da_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kRingBytes + kXsBytes + kMaxChunks * kLsBytes));
    });
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
    const int strips = (K + TC - 1) / TC;
    XaParams p{};
    p.X = X;
    p.x16 = (uint16_t *)x16;      // written by the first launch only
    p.ldx16 = ldx16;
    (void)fp16;      // bf16 math mode only: the shared-memory tile and the 16-bit copy are the same bf16 values
    p.T = T;
    p.K = K;
    p.strips_per_block = pick_strip_run(strips, 1, T);
    p.ring = ring_enabled();
    dim3 grid((T + TT - 1) / TT, (strips + p.strips_per_block - 1) / p.strips_per_block);
    set_fills(p.fills, fills, n_fills, T);      // carried by the first launch
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_xa_tc, grid, dim3(256), (size_t)(kRingBytes + kXsBytes + p.n * kAsBytes), s, p);
        p.n = 0;
        p.x16 = nullptr;
        p.fills.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = XaChunk{jobs[j].A, jobs[j].low_zeroed, jobs[j].R, r0, is_vec(jobs[j].A, jobs[j].R)};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

cudaError_t launch_lora_xa16_group(const void *X16, int ld16, const LoraXaJob *jobs, int n, int T, int K, cudaStream_t s) {
    if (T <= 0 || K <= 0 || n <= 0) return cudaSuccess;
    if ((K & 7) != 0 || (ld16 & 7) != 0 || (reinterpret_cast<uintptr_t>(X16) & 15) != 0) return cudaErrorInvalidValue;
    static PerDeviceOnce configured;
    cudaError_t e = per_device_once(configured, [] {
        return cudaFuncSetAttribute(k_lora_xa16_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kXsBytes + kMaxChunks * kAsBytes));
    });
    if (e != cudaSuccess) return e;
    const int strips = (K + TC - 1) / TC;
    Xa16Params p{};
    p.X16 = (const uint16_t *)X16;
    p.ld = ld16;
    p.T = T;
    p.K = K;
    p.strips_per_block = pick_strip_run(strips, 1, T);
    dim3 grid((T + TT - 1) / TT, (strips + p.strips_per_block - 1) / p.strips_per_block);
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_xa16_tc, grid, dim3(256), (size_t)(kXsBytes + p.n * kAsBytes), s, p);
        p.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = XaChunk{jobs[j].A, jobs[j].low_zeroed, jobs[j].R, r0, is_vec(jobs[j].A, jobs[j].R)};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

cudaError_t launch_lora_dy_group(const LoraDyJob *jobs, int n, int fp16, int T, const RowFill *fills, int n_fills, cudaStream_t s) {
    if (T <= 0 || n <= 0) return cudaSuccess;
    (void)fp16;
    cudaError_t ae = allow_dyn_smem();
    if (ae != cudaSuccess) return ae;
    int strips_sum = 0, strips_max = 0;
    for (int j = 0; j < n; j++) {
        const int st = (jobs[j].N + TC - 1) / TC;
        strips_sum += st;
        strips_max = st > strips_max ? st : strips_max;
    }
    // members per launch (grid.z): every 16-rank chunk of every member is one, up to kMaxChunks per launch
    int n_chunks = 0;
    for (int j = 0; j < n; j++) n_chunks += (jobs[j].R + 15) / 16;
    const int n_launch_members = n_chunks < kMaxChunks ? (n_chunks > 0 ? n_chunks : 1) : kMaxChunks;
    (void)strips_sum;
    // all members read fp32 dY, or all read the bf16 copy they were given (16-byte rows: N % 8 == 0)
    const bool in16 = jobs[0].dY == nullptr;
    for (int j = 0; j < n; j++)
        if ((jobs[j].dY == nullptr) != in16 || (in16 && (!jobs[j].dy16 || jobs[j].N % 8 != 0 || jobs[j].ld16 % 8 != 0 ||
                                                         (reinterpret_cast<uintptr_t>(jobs[j].dy16) & 15) != 0)))
            return cudaErrorInvalidValue;
    DyParams p{};
    p.T = T;
    p.strips_per_block = pick_strip_run(strips_max, n_launch_members, T);
    p.ring = ring_enabled();
    const dim3 grid_xy((strips_max + p.strips_per_block - 1) / p.strips_per_block, (T + TT - 1) / TT);
    set_fills(p.fills, fills, n_fills, T);      // carried by the first launch
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = in16 ? launch_k(k_lora_dy_tc<true>, dim3(grid_xy.x, grid_xy.y, p.n), dim3(256), (size_t)kDySmemBytes, s, p)
                              : launch_k(k_lora_dy_tc<false>, dim3(grid_xy.x, grid_xy.y, p.n), dim3(256), (size_t)kDySmemBytes, s, p);
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
            m.vec_b = is_vec(b.B, b.N);
            m.vec_low = is_vec(b.low, b.R);
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
    p.ring = ring_enabled();
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_da_tc, dim3(strips, groups), dim3(256), (size_t)(kRingBytes + kXsBytes + p.n * kLsBytes), s, p);
        p.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = DaChunk{jobs[j].dLow, jobs[j].dA, jobs[j].scaling, jobs[j].R, r0, is_vec(jobs[j].dLow, jobs[j].R)};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

cudaError_t launch_lora_da16_group(const void *X16, int ld16, const LoraDaJob *jobs, int n, int T, int K, cudaStream_t s) {
    if (T <= 0 || K <= 0 || n <= 0) return cudaSuccess;
    if ((K & 7) != 0 || (ld16 & 7) != 0 || (reinterpret_cast<uintptr_t>(X16) & 15) != 0) return cudaErrorInvalidValue;
    static PerDeviceOnce configured;
    cudaError_t e = per_device_once(configured, [] {
        return cudaFuncSetAttribute(k_lora_da16_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kXsBytes + kMaxChunks * kLsBytes));
    });
    if (e != cudaSuccess) return e;
    const int strips = (K + TC - 1) / TC;
    int groups, tpg;
    pick_groups(strips, T, groups, tpg);
    Da16Params p{};
    p.X16 = (const uint16_t *)X16;
    p.ld = ld16;
    p.T = T;
    p.K = K;
    p.tok_per_group = tpg;
    auto flush = [&]() -> cudaError_t {
        if (p.n == 0) return cudaSuccess;
        cudaError_t le = launch_k(k_lora_da16_tc, dim3(strips, groups), dim3(256), (size_t)(kXsBytes + p.n * kLsBytes), s, p);
        p.n = 0;
        return le;
    };
    for (int j = 0; j < n; j++)
        for (int r0 = 0; r0 < jobs[j].R; r0 += 16) {
            p.c[p.n++] = DaChunk{jobs[j].dLow, jobs[j].dA, jobs[j].scaling, jobs[j].R, r0, is_vec(jobs[j].dLow, jobs[j].R)};
            if (p.n == kMaxChunks && (e = flush()) != cudaSuccess) return e;
        }
    return flush();
}

}  // namespace gt
