// Causal multi-head attention with grouped KV heads, forward and backward, without the [heads, T, T] buffers.
//
// Replaces tune_attn_causal_gqa_fwd / tune_attn_causal_gqa_bwd_dq_ds / tune_attn_causal_gqa_bwd_dk_dv
// (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:527-717, launched from src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:433-513
// and GpuLoraEngine.Backward.cs:354-459) and their CPU statement CausalAttentionKernel.Forward / Backward
// (src/Glacier.Tune/Kernels/CausalAttentionKernel.cs:17-213).  The reference stores the softmax rows (attnProbs
// [heads_q, T, T]) in the forward and a dS buffer of the same size in the backward; here the forward keeps one
// log-sum-exp per (head, query) and the backward recomputes the probabilities tile by tile.
//
//   scores = q k^T / sqrt(head_dim), key j visible to query i iff j <= i; head h reads KV head h / (heads_q / heads_kv)
//   out = softmax(scores) v
//   dP = dO v^T;  dS = P * (dP - rowsum(dO * out)) / sqrt(head_dim);  dq = dS k;  dk = dS^T q;  dv = P^T dO
//
// Layouts as the reference: q, out, dO, dq [T, heads_q, head_dim]; k, v, dk, dv [T, heads_kv, head_dim], fp32.
// Tiles of 64 queries x 64 keys; the products run on warp-level m16n8k16 MMAs (bf16 operands in the bf16 math mode,
// fp16 in the validation modes) with fp32 accumulation and fp32 softmax statistics.  Attention is about 3 % of a
// layer's FLOPs at 512 tokens; the CTA-wide tcgen05 path is kept for the projections.
//   k_attn_fwd      grid (query tile pairs, heads_q): online softmax over the key tiles at or left of the diagonal,
//                   four compute warps and four fetch warps per block
//   k_attn_delta    rowsum(dO * out) per (head, query)
//   k_attn_bwd      grid (2 * heads_q, tiles), eight compute + four fetch warps; even blocks: dq of one query tile, summed
//                   over its key tiles in registers; odd blocks: dk, dv of one key tile for ONE query head, summed over the
//                   query tiles in registers, written to a per-query-head workspace
//   k_attn_reduce_kv sums the query heads of each KV group (fixed order: results do not change from run to run)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gt_engine_priv.h"
#include "gt_ptx.cuh"

using gt::launch_k;
using gt::pdl_trigger;
using gt::pdl_wait;

using namespace gt;

namespace {

constexpr int D = 128;              // head_dim served
constexpr int BQ = 64, BK = 64;     // tile sizes
constexpr int SD = (D + 8) * 2;     // smem row stride in bytes of a [rows][128] 16-bit tile (272: conflict-free ldmatrix)
constexpr int SP = (BK + 8) * 2;    // smem row stride in bytes of a [64][64] 16-bit tile (144)

template <typename T16>
__device__ __forceinline__ void mma16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T16>
__device__ __forceinline__ uint32_t pk(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pk<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <>
__device__ __forceinline__ uint32_t pk<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// ldmatrix lane -> row address of its 8x8 matrix (rows `stride` bytes apart); result registers {0,1,2,3} are
// {a0,a1,a2,a3} of an A fragment, or {b0,b1} of n-tile n0 followed by {b0,b1} of n-tile n0 + 8.
__device__ __forceinline__ uint32_t a_mk(uint32_t base, int stride, int m0, int k0, int lane) {       // A stored [m][k]
    return base + (uint32_t)((m0 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + (k0 + (lane >> 4) * 8) * 2);
}
__device__ __forceinline__ uint32_t a_km(uint32_t base, int stride, int m0, int k0, int lane) {       // A stored [k][m] (.trans)
    return base + (uint32_t)((k0 + (lane & 7) + (lane >> 4) * 8) * stride + (m0 + ((lane >> 3) & 1) * 8) * 2);
}
__device__ __forceinline__ uint32_t b_nk(uint32_t base, int stride, int n0, int k0, int lane) {       // B stored [n][k]
    return base + (uint32_t)((n0 + (lane & 7) + (lane >> 4) * 8) * stride + (k0 + ((lane >> 3) & 1) * 8) * 2);
}
__device__ __forceinline__ uint32_t b_kn(uint32_t base, int stride, int n0, int k0, int lane) {       // B stored [k][n] (.trans)
    return base + (uint32_t)((k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + (n0 + (lane >> 4) * 8) * 2);
}

// [64 rows x 128] fp32 tile of src (row t = t0 + r at src + t * ld + col0), scaled, -> 16-bit smem tile; rows at or
// beyond T become zero.  NT threads.
template <typename T16, int NT>
__device__ __forceinline__ void load_tile(const float *__restrict__ src, int64_t ld, int col0, int t0, int T, float scale, uint8_t *dst, int tid) {
#pragma unroll
    for (int i = 0; i < (64 * D / 4) / NT; i++) {
        const int idx = tid + i * NT;
        const int r = idx >> 5, c = (idx & 31) * 4;
        const int t = t0 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < T) v = __ldg(reinterpret_cast<const float4 *>(src + (int64_t)t * ld + col0 + c));
        *reinterpret_cast<uint2 *>(dst + r * SD + c * 2) = make_uint2(pk<T16>(v.x * scale, v.y * scale), pk<T16>(v.z * scale, v.w * scale));
    }
}

// Two tiles at once (key and value tile of one step): all loads are issued before the first is used, one round trip.
template <typename T16, int NT>
__device__ __forceinline__ void load_tile_pair(const float *__restrict__ a, const float *__restrict__ b, int64_t ld, int col0, int t0, int T,
                                               uint8_t *dst_a, uint8_t *dst_b, int tid) {
    constexpr int NI = (64 * D / 4) / NT;
    float4 va[NI], vb[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * NT;
        const int r = idx >> 5, c = (idx & 31) * 4;
        const int t = t0 + r;
        va[i] = vb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < T) {
            va[i] = __ldg(reinterpret_cast<const float4 *>(a + (int64_t)t * ld + col0 + c));
            vb[i] = __ldg(reinterpret_cast<const float4 *>(b + (int64_t)t * ld + col0 + c));
        }
    }
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * NT;
        const int r = idx >> 5, c = (idx & 31) * 4;
        *reinterpret_cast<uint2 *>(dst_a + r * SD + c * 2) = make_uint2(pk<T16>(va[i].x, va[i].y), pk<T16>(va[i].z, va[i].w));
        *reinterpret_cast<uint2 *>(dst_b + r * SD + c * 2) = make_uint2(pk<T16>(vb[i].x, vb[i].y), pk<T16>(vb[i].z, vb[i].w));
    }
}

constexpr float kLog2e = 1.4426950408889634f;
// 2^x on the special-function unit (2 ulp; 2^-inf = 0): the probabilities are rounded to 16 bits right after
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ------------------------------------------------------------------------------------------------ forward
// 8 warps: warps 0-3 compute (16 queries each), warps 4-7 fetch - while the compute warps work on key tile j out of one
// shared-memory buffer, the fetch warps read key / value tile j + 1 from global memory, round it and store it into the
// other buffer, so the load latency hides under the MMAs.  A block takes query tile i and its mirror n - 1 - i one after
// the other: every block then walks n + 1 key tiles, the grid is n / 2 x heads blocks (112 at 512 tokens and 28 heads:
// one wave of the 148 SMs, one block per SM).  (One tile per block, longest first as in the backward kernels, measured
// slower here: 33.3 against 32.8 ms for the 28-layer step.)
// Scores are kept in the base-2 domain: q is scaled by log2(e) / sqrt(head_dim) when it is rounded, probabilities are
// exp2(s - m).  lse2[h, t] = m + log2(sum) is what the backward needs.
constexpr int kFwdSmem = 5 * 64 * SD;      // Q + two (K, V) buffers
template <typename T16>
__global__ void __launch_bounds__(256) k_attn_fwd(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                  float *__restrict__ out, float *__restrict__ lse2, int T, int HQ, int HK) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *Qs = smem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const bool compute = warp < 4;
    const int h = blockIdx.y, kh = h / (HQ / HK);
    const int n_qt = (T + BQ - 1) / BQ;
    const int64_t ldq = (int64_t)HQ * D, ldk = (int64_t)HK * D;
    const uint32_t qs = smem_u32(Qs);
    auto kbuf = [&](int b) { return smem + (1 + 2 * b) * 64 * SD; };
    auto vbuf = [&](int b) { return smem + (2 + 2 * b) * 64 * SD; };
    for (int pass = 0; pass < 2; pass++) {
        const int it = pass == 0 ? (int)blockIdx.x : n_qt - 1 - (int)blockIdx.x;
        if (pass == 1 && it <= (int)blockIdx.x) break;      // odd tile count: the middle tile is done once
        const int q0 = it * BQ;
        __syncthreads();      // the previous pass has finished with every buffer
        load_tile<T16, 256>(q, ldq, h * D, q0, T, kLog2e * rsqrtf((float)D), Qs, tid);
        load_tile<T16, 256>(k, ldk, kh * D, 0, T, 1.f, kbuf(0), tid);
        load_tile<T16, 256>(v, ldk, kh * D, 0, T, 1.f, vbuf(0), tid);
        __syncthreads();
        uint32_t qf[D / 16][4];
        float o[D / 8][4];
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        const int row[2] = {q0 + (warp & 3) * 16 + g, q0 + (warp & 3) * 16 + g + 8};
        if (compute) {
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) ldsm4(a_mk(qs, SD, warp * 16, kk * 16, lane), qf[kk]);
#pragma unroll
            for (int n = 0; n < D / 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        }
        for (int jt = 0; jt <= it; jt++) {
            const int k0 = jt * BK;
            if (!compute) {
                if (jt + 1 <= it) load_tile_pair<T16, 128>(k, v, ldk, kh * D, k0 + BK, T, kbuf((jt + 1) & 1), vbuf((jt + 1) & 1), tid - 128);
            } else {
                const uint32_t ks = smem_u32(kbuf(jt & 1)), vs = smem_u32(vbuf(jt & 1));
                float s[BK / 8][4];
#pragma unroll
                for (int n = 0; n < BK / 8; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
                    for (int n = 0; n < BK / 8; n += 2) {
                        uint32_t b[4];
                        ldsm4(b_nk(ks, SD, n * 8, kk * 16, lane), b);
                        mma16<T16>(s[n], qf[kk], b[0], b[1]);
                        mma16<T16>(s[n + 1], qf[kk], b[2], b[3]);
                    }
                }
                // causal mask: only the diagonal tile has masked entries; keys beyond T only in the last tile
                if (jt == it || k0 + BK > T) {
#pragma unroll
                    for (int n = 0; n < BK / 8; n++) {
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const int key = k0 + n * 8 + 2 * t4 + (c & 1);
                            if (key > row[c >> 1] || key >= T) s[n][c] = -INFINITY;
                        }
                    }
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int n = 0; n < BK / 8; n++) {
                    mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
                    mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
                }
                float corr[2];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    // a finite floor keeps (-inf) - (-inf) out of the exponent (a row sees key 0 from the first tile on,
                    // so its maximum is finite anyway)
                    const float mn = fmaxf(fmaxf(m[r], mx[r]), -3.0e38f);
                    corr[r] = ex2(m[r] - mn);
                    m[r] = mn;
                }
                float ps[2] = {0.f, 0.f};
                uint32_t pf[BK / 16][4];
#pragma unroll
                for (int n = 0; n < BK / 8; n++) {
                    const float p0 = ex2(s[n][0] - m[0]), p1 = ex2(s[n][1] - m[0]);
                    const float p2 = ex2(s[n][2] - m[1]), p3 = ex2(s[n][3] - m[1]);
                    ps[0] += p0 + p1;
                    ps[1] += p2 + p3;
                    pf[n >> 1][(n & 1) * 2] = pk<T16>(p0, p1);
                    pf[n >> 1][(n & 1) * 2 + 1] = pk<T16>(p2, p3);
                }
#pragma unroll
                for (int r = 0; r < 2; r++) l[r] = l[r] * corr[r] + ps[r];
                // the running maxima move in the first tiles and then rarely: rescale the accumulator only when one did
                if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
                    for (int n = 0; n < D / 8; n++) {
                        o[n][0] *= corr[0];
                        o[n][1] *= corr[0];
                        o[n][2] *= corr[1];
                        o[n][3] *= corr[1];
                    }
                }
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++) {
#pragma unroll
                    for (int n = 0; n < D / 8; n += 2) {
                        uint32_t b[4];
                        ldsm4t(b_kn(vs, SD, n * 8, kk * 16, lane), b);
                        mma16<T16>(o[n], pf[kk], b[0], b[1]);
                        mma16<T16>(o[n + 1], pf[kk], b[2], b[3]);
                    }
                }
            }
            __syncthreads();      // tile j + 1 is in place, tile j's buffer is free
        }
        if (compute) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
                l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                if (row[r] >= T) continue;
                const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
                float *dst = out + (int64_t)row[r] * ldq + h * D;
#pragma unroll
                for (int n = 0; n < D / 8; n++)
                    *reinterpret_cast<float2 *>(dst + n * 8 + 2 * t4) = make_float2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
                if (t4 == 0) lse2[(int64_t)h * T + row[r]] = m[r] + log2f(l[r]);
            }
        }
    }
}

// delta[h, t] = sum_d dO[t, h, d] * out[t, h, d]; one warp per (t, h)
__global__ void k_attn_delta(const float *__restrict__ d_out, const float *__restrict__ out, float *__restrict__ delta, int T, int HQ) {
    pdl_wait();
    pdl_trigger();
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= T * HQ) return;
    const int t = w / HQ, h = w % HQ;
    const float4 a = __ldg(reinterpret_cast<const float4 *>(d_out + ((int64_t)t * HQ + h) * D) + lane);
    const float4 b = __ldg(reinterpret_cast<const float4 *>(out + ((int64_t)t * HQ + h) * D) + lane);
    float s = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) delta[(int64_t)h * T + t] = s;
}

// Shared first phase of both backward kernels, 8 compute warps: warp = query m-tile (warp & 3) x key half (warp >> 2).
//   S2 = Qs Ks^T (base-2 scores, Qs pre-scaled), P = exp2(S2 - lse2), dP = dOs Vs^T, dS = P (dP - delta) / sqrt(D)
// P and dS go to shared memory as [query][key] 16-bit tiles (zero where masked).
template <typename T16>
__device__ __forceinline__ void bwd_scores(uint32_t qs, uint32_t ks, uint32_t vs, uint32_t dos, uint8_t *Ps, uint8_t *dSs, const float *lse2h,
                                           const float *deltah, int q0, int k0, int T, int warp, int lane) {
    const int g = lane >> 2, t4 = lane & 3;
    const int m0 = (warp & 3) * 16, nh = (warp >> 2) * 32;
    float s[4][4], dp[4][4];
#pragma unroll
    for (int n = 0; n < 4; n++)
#pragma unroll
        for (int c = 0; c < 4; c++) s[n][c] = dp[n][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
        uint32_t aq[4], ad[4];
        ldsm4(a_mk(qs, SD, m0, kk * 16, lane), aq);
        ldsm4(a_mk(dos, SD, m0, kk * 16, lane), ad);
#pragma unroll
        for (int n = 0; n < 4; n += 2) {
            uint32_t bk[4], bv[4];
            ldsm4(b_nk(ks, SD, nh + n * 8, kk * 16, lane), bk);
            ldsm4(b_nk(vs, SD, nh + n * 8, kk * 16, lane), bv);
            mma16<T16>(s[n], aq, bk[0], bk[1]);
            mma16<T16>(s[n + 1], aq, bk[2], bk[3]);
            mma16<T16>(dp[n], ad, bv[0], bv[1]);
            mma16<T16>(dp[n + 1], ad, bv[2], bv[3]);
        }
    }
    const float scale = rsqrtf((float)D);
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int qi = q0 + m0 + g + 8 * r;
        const bool q_ok = qi < T;
        const float ls = q_ok ? lse2h[qi] : 0.f, dl = q_ok ? deltah[qi] : 0.f;
#pragma unroll
        for (int n = 0; n < 4; n++) {
            float p[2], ds[2];
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int key = k0 + nh + n * 8 + 2 * t4 + c;
                const bool ok = q_ok && key <= qi && key < T;
                p[c] = ok ? ex2(s[n][2 * r + c] - ls) : 0.f;
                ds[c] = ok ? p[c] * (dp[n][2 * r + c] - dl) * scale : 0.f;
            }
            const int off = (m0 + g + 8 * r) * SP + (nh + n * 8 + 2 * t4) * 2;
            *reinterpret_cast<uint32_t *>(Ps + off) = pk<T16>(p[0], p[1]);
            *reinterpret_cast<uint32_t *>(dSs + off) = pk<T16>(ds[0], ds[1]);
        }
    }
}

// Both backward kernels: 8 compute warps + 4 fetch warps (384 threads).  The tiles that change from iteration to
// iteration (key / value tiles in the dq kernel, query / dO tiles in the dk, dv kernel) are double-buffered: the fetch
// warps load, round and store the next pair while the compute warps work on the current one.
constexpr int kBwdSmem = 6 * 64 * SD + 2 * 64 * SP;
__device__ __forceinline__ void compute_warps_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// dq[query tile] = sum over key tiles j <= i of dS K.  Compute warps: query m-tile (warp & 3) x half of head_dim (warp >> 2).
template <typename T16>
__device__ __forceinline__ void attn_bwd_dq_block(const float *__restrict__ d_out, const float *__restrict__ q, const float *__restrict__ k,
                                                  const float *__restrict__ v, const float *__restrict__ lse2, const float *__restrict__ delta,
                                                  float *__restrict__ dq, int T, int HQ, int HK, int h, int it) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *Qs = smem, *dOs = Qs + 64 * SD, *Ps = smem + 6 * 64 * SD, *dSs = Ps + 64 * SP;
    auto kbuf = [&](int b) { return smem + (2 + 2 * b) * 64 * SD; };
    auto vbuf = [&](int b) { return smem + (3 + 2 * b) * 64 * SD; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const bool compute = warp < 8;
    const int kh = h / (HQ / HK);
    const int q0 = it * BQ;
    const int64_t ldq = (int64_t)HQ * D, ldk = (int64_t)HK * D;
    if (compute) {
        load_tile<T16, 256>(q, ldq, h * D, q0, T, kLog2e * rsqrtf((float)D), Qs, tid);
        load_tile<T16, 256>(d_out, ldq, h * D, q0, T, 1.f, dOs, tid);
    } else {
        load_tile<T16, 128>(k, ldk, kh * D, 0, T, 1.f, kbuf(0), tid - 256);
        load_tile<T16, 128>(v, ldk, kh * D, 0, T, 1.f, vbuf(0), tid - 256);
    }
    __syncthreads();
    const uint32_t qs = smem_u32(Qs), dos = smem_u32(dOs), dss = smem_u32(dSs);
    const int m0 = (warp & 3) * 16, dh = ((warp >> 2) & 1) * 64;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    for (int jt = 0; jt <= it; jt++) {
        const int k0 = jt * BK;
        if (!compute) {
            if (jt + 1 <= it) {
                load_tile<T16, 128>(k, ldk, kh * D, k0 + BK, T, 1.f, kbuf((jt + 1) & 1), tid - 256);
                load_tile<T16, 128>(v, ldk, kh * D, k0 + BK, T, 1.f, vbuf((jt + 1) & 1), tid - 256);
            }
        } else {
            const uint32_t ks = smem_u32(kbuf(jt & 1)), vs = smem_u32(vbuf(jt & 1));
            bwd_scores<T16>(qs, ks, vs, dos, Ps, dSs, lse2 + (int64_t)h * T, delta + (int64_t)h * T, q0, k0, T, warp, lane);
            compute_warps_sync();
#pragma unroll
            for (int kk = 0; kk < BK / 16; kk++) {
                uint32_t a[4];
                ldsm4(a_mk(dss, SP, m0, kk * 16, lane), a);
#pragma unroll
                for (int n = 0; n < 8; n += 2) {
                    uint32_t b[4];
                    ldsm4t(b_kn(ks, SD, dh + n * 8, kk * 16, lane), b);
                    mma16<T16>(acc[n], a, b[0], b[1]);
                    mma16<T16>(acc[n + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();      // the next tiles are in place; P / dS and this iteration's buffers are free
    }
    if (!compute) return;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int qi = q0 + m0 + g + 8 * r;
        if (qi >= T) continue;
        float *dst = dq + (int64_t)qi * ldq + h * D + dh;
#pragma unroll
        for (int n = 0; n < 8; n++) *reinterpret_cast<float2 *>(dst + n * 8 + 2 * t4) = make_float2(acc[n][2 * r], acc[n][2 * r + 1]);
    }
}

// dk, dv of one key tile for one query head, summed over the query tiles i >= j, into the per-head workspace
// wk, wv [heads_q, T, head_dim].  Compute warps: key m-tile (warp & 3) x half of head_dim (warp >> 2).
template <typename T16>
__device__ __forceinline__ void attn_bwd_dkv_block(const float *__restrict__ d_out, const float *__restrict__ q, const float *__restrict__ k,
                                                   const float *__restrict__ v, const float *__restrict__ lse2, const float *__restrict__ delta,
                                                   float *__restrict__ wk, float *__restrict__ wv, int T, int HQ, int HK, int h, int jt) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *Ks = smem, *Vs = Ks + 64 * SD, *Ps = smem + 6 * 64 * SD, *dSs = Ps + 64 * SP;
    auto qbuf = [&](int b) { return smem + (2 + 2 * b) * 64 * SD; };
    auto obuf = [&](int b) { return smem + (3 + 2 * b) * 64 * SD; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const bool compute = warp < 8;
    const int kh = h / (HQ / HK);
    const int k0 = jt * BK;
    const int64_t ldq = (int64_t)HQ * D, ldk = (int64_t)HK * D;
    const float qscale = kLog2e * rsqrtf((float)D);
    if (compute) {
        load_tile<T16, 256>(k, ldk, kh * D, k0, T, 1.f, Ks, tid);
        load_tile<T16, 256>(v, ldk, kh * D, k0, T, 1.f, Vs, tid);
    } else {
        load_tile<T16, 128>(q, ldq, h * D, jt * BQ, T, qscale, qbuf(0), tid - 256);
        load_tile<T16, 128>(d_out, ldq, h * D, jt * BQ, T, 1.f, obuf(0), tid - 256);
    }
    __syncthreads();
    const uint32_t ks = smem_u32(Ks), vs = smem_u32(Vs), ps = smem_u32(Ps), dss = smem_u32(dSs);
    const int m0 = (warp & 3) * 16, dh = ((warp >> 2) & 1) * 64;
    float ak[8][4], av[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) ak[n][0] = ak[n][1] = ak[n][2] = ak[n][3] = av[n][0] = av[n][1] = av[n][2] = av[n][3] = 0.f;
    const int n_qt = (T + BQ - 1) / BQ;
    for (int it = jt; it < n_qt; it++) {
        const int q0 = it * BQ, b = (it - jt) & 1;
        if (!compute) {
            if (it + 1 < n_qt) {
                load_tile<T16, 128>(q, ldq, h * D, q0 + BQ, T, qscale, qbuf(b ^ 1), tid - 256);
                load_tile<T16, 128>(d_out, ldq, h * D, q0 + BQ, T, 1.f, obuf(b ^ 1), tid - 256);
            }
        } else {
            const uint32_t qs = smem_u32(qbuf(b)), dos = smem_u32(obuf(b));
            bwd_scores<T16>(qs, ks, vs, dos, Ps, dSs, lse2 + (int64_t)h * T, delta + (int64_t)h * T, q0, k0, T, warp, lane);
            compute_warps_sync();
#pragma unroll
            for (int kk = 0; kk < BQ / 16; kk++) {
                uint32_t ap[4], as[4];
                ldsm4t(a_km(ps, SP, m0, kk * 16, lane), ap);       // P^T: m = key, k = query
                ldsm4t(a_km(dss, SP, m0, kk * 16, lane), as);      // dS^T
#pragma unroll
                for (int n = 0; n < 8; n += 2) {
                    uint32_t bo[4], bq[4];
                    ldsm4t(b_kn(dos, SD, dh + n * 8, kk * 16, lane), bo);
                    ldsm4t(b_kn(qs, SD, dh + n * 8, kk * 16, lane), bq);
                    mma16<T16>(av[n], ap, bo[0], bo[1]);
                    mma16<T16>(av[n + 1], ap, bo[2], bo[3]);
                    mma16<T16>(ak[n], as, bq[0], bq[1]);
                    mma16<T16>(ak[n + 1], as, bq[2], bq[3]);
                }
            }
        }
        __syncthreads();
    }
    if (!compute) return;
    // the query tiles held q * log2(e) / sqrt(D): dk = dS^T q needs the plain q
    const float unscale = 1.0f / qscale;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int ki = k0 + m0 + g + 8 * r;
        if (ki >= T) continue;
        float *dk_ = wk + ((int64_t)h * T + ki) * D + dh, *dv_ = wv + ((int64_t)h * T + ki) * D + dh;
#pragma unroll
        for (int n = 0; n < 8; n++) {
            *reinterpret_cast<float2 *>(dk_ + n * 8 + 2 * t4) = make_float2(ak[n][2 * r] * unscale, ak[n][2 * r + 1] * unscale);
            *reinterpret_cast<float2 *>(dv_ + n * 8 + 2 * t4) = make_float2(av[n][2 * r], av[n][2 * r + 1]);
        }
    }
}

// One launch for both halves of the backward: grid (2 * heads, tiles), even blockIdx.x = the dq block of head x / 2, odd =
// its dk, dv block.  blockIdx.y is the tile's rank by length, longest first (the last query tile sees every key tile,
// key tile 0 is seen by every query tile): blocks are handed out rank by rank, head by head, so the 448 blocks of 1..8
// tile steps pack the 148 SMs with one short tail - each half alone (224 blocks) left a tail of its own, and dealt
// shortest first a half took 13.4 tile times instead of 8.7.
static_assert(BQ == BK, "the dq and dk, dv blocks share one tile grid");
template <typename T16>
__global__ void __launch_bounds__(384) k_attn_bwd(const float *__restrict__ d_out, const float *__restrict__ q, const float *__restrict__ k,
                                                  const float *__restrict__ v, const float *__restrict__ lse2, const float *__restrict__ delta,
                                                  float *__restrict__ dq, float *__restrict__ wk, float *__restrict__ wv, int T, int HQ, int HK) {
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x >> 1, rank = blockIdx.y;
    if (blockIdx.x & 1) attn_bwd_dkv_block<T16>(d_out, q, k, v, lse2, delta, wk, wv, T, HQ, HK, h, rank);
    else attn_bwd_dq_block<T16>(d_out, q, k, v, lse2, delta, dq, T, HQ, HK, h, (int)gridDim.y - 1 - rank);
}

// dk[t, kh, :] = sum over the query heads of group kh of wk[h, t, :] (same for dv), heads in ascending order
__global__ void k_attn_reduce_kv(const float *__restrict__ wk, const float *__restrict__ wv, float *__restrict__ dk, float *__restrict__ dv, int T,
                                 int HQ, int HK) {
    pdl_wait();
    pdl_trigger();
    const int64_t n4 = (int64_t)T * HK * D / 4;
    const int ratio = HQ / HK;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int c4 = (int)(i % (D / 4));
        const int kh = (int)((i / (D / 4)) % HK);
        const int t = (int)(i / ((int64_t)(D / 4) * HK));
        float4 sk = make_float4(0.f, 0.f, 0.f, 0.f), sv = sk;
        for (int h = kh * ratio; h < (kh + 1) * ratio; h++) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(wk + ((int64_t)h * T + t) * D) + c4);
            const float4 b = __ldg(reinterpret_cast<const float4 *>(wv + ((int64_t)h * T + t) * D) + c4);
            sk.x += a.x; sk.y += a.y; sk.z += a.z; sk.w += a.w;
            sv.x += b.x; sv.y += b.y; sv.z += b.z; sv.w += b.w;
        }
        reinterpret_cast<float4 *>(dk)[i] = sk;
        reinterpret_cast<float4 *>(dv)[i] = sv;
    }
}

PerDeviceOnce g_attn_attr;
template <typename T16>
cudaError_t attn_allow_smem() {
    cudaError_t e = cudaFuncSetAttribute(k_attn_fwd<T16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_bwd<T16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    return e;
}

int check_shape(int T, int HQ, int HK, int Dh, const char *who) {
    if (T <= 0 || HQ <= 0 || HK <= 0) return failf(GT_ERR_INVALID, "%s: bad shape T=%d heads_q=%d heads_kv=%d", who, T, HQ, HK);
    if (Dh != D) return failf(GT_ERR_UNSUPPORTED, "%s: head_dim %d is not supported (128 only)", who, Dh);
    if (HQ % HK != 0) return failf(GT_ERR_INVALID, "%s: heads_q %d is not a multiple of heads_kv %d", who, HQ, HK);
    return GT_OK;
}

}  // namespace

namespace gt {

int attention_forward_on_device(gt_engine *e, const float *q, const float *k, const float *v, float *out, float *lse, int T, int HQ, int HK,
                                int Dh) {
    int rc = check_shape(T, HQ, HK, Dh, "attention forward");
    if (rc != GT_OK) return rc;
    GT_CUDA(per_device_once(g_attn_attr, [] {
        cudaError_t a = attn_allow_smem<__nv_bfloat16>();
        return a == cudaSuccess ? attn_allow_smem<__half>() : a;
    }));
    const int n_qt = (T + BQ - 1) / BQ;
    const dim3 grid((n_qt + 1) / 2, HQ);      // a block takes query tile i and its mirror n - 1 - i
    if (e->math_mode == GT_MATH_BF16) GT_LAUNCH(e, launch_k(k_attn_fwd<__nv_bfloat16>, grid, dim3(256), kFwdSmem, e->stream, q, k, v, out, lse, T, HQ, HK));
    else GT_LAUNCH(e, launch_k(k_attn_fwd<__half>, grid, dim3(256), kFwdSmem, e->stream, q, k, v, out, lse, T, HQ, HK));
    return GT_OK;
}

int attention_backward_on_device(gt_engine *e, const float *d_out, const float *q, const float *k, const float *v, const float *out,
                                 const float *lse, float *dq, float *dk, float *dv, int T, int HQ, int HK, int Dh) {
    int rc = check_shape(T, HQ, HK, Dh, "attention backward");
    if (rc != GT_OK) return rc;
    GT_CUDA(per_device_once(g_attn_attr, [] {
        cudaError_t a = attn_allow_smem<__nv_bfloat16>();
        return a == cudaSuccess ? attn_allow_smem<__half>() : a;
    }));
    // scratch: delta [HQ, T] and the per-query-head dk / dv workspace [HQ, T, D] x 2
    const size_t n_delta = (((size_t)HQ * T * sizeof(float)) + 255) & ~(size_t)255;
    const size_t n_w = (size_t)HQ * T * D * sizeof(float);
    GT_CUDA(e->attn.reserve(n_delta + 2 * n_w));
    float *delta = (float *)e->attn.p;
    float *wk = (float *)((char *)e->attn.p + n_delta), *wv = wk + (size_t)HQ * T * D;
    GT_LAUNCH(e, launch_k(k_attn_delta, dim3((T * HQ * 32 + 255) / 256), dim3(256), 0, e->stream, d_out, out, delta, T, HQ));
    const dim3 gb(2 * HQ, (T + BQ - 1) / BQ);
    if (e->math_mode == GT_MATH_BF16)
        GT_LAUNCH(e, launch_k(k_attn_bwd<__nv_bfloat16>, gb, dim3(384), kBwdSmem, e->stream, d_out, q, k, v, lse, delta, dq, wk, wv, T, HQ, HK));
    else
        GT_LAUNCH(e, launch_k(k_attn_bwd<__half>, gb, dim3(384), kBwdSmem, e->stream, d_out, q, k, v, lse, delta, dq, wk, wv, T, HQ, HK));
    const int64_t n4 = (int64_t)T * HK * D / 4;
    GT_LAUNCH(e, launch_k(k_attn_reduce_kv, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, e->stream, (const float *)wk, (const float *)wv, dk, dv, T, HQ, HK));
    return GT_OK;
}

}  // namespace gt

extern "C" {

int gt_attention_forward(gt_engine *e, const float *q, const float *k, const float *v, float *out, float *lse, int32_t T, int32_t heads_q,
                         int32_t heads_kv, int32_t head_dim) {
    if (!e || !q || !k || !v || !out || !lse) return failf(GT_ERR_INVALID, "gt_attention_forward: null argument");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return attention_forward_on_device(e, q, k, v, out, lse, T, heads_q, heads_kv, head_dim);
}

int gt_attention_backward(gt_engine *e, const float *d_out, const float *q, const float *k, const float *v, const float *out, const float *lse,
                          float *dq, float *dk, float *dv, int32_t T, int32_t heads_q, int32_t heads_kv, int32_t head_dim) {
    if (!e || !d_out || !q || !k || !v || !out || !lse || !dq || !dk || !dv) return failf(GT_ERR_INVALID, "gt_attention_backward: null argument");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return attention_backward_on_device(e, d_out, q, k, v, out, lse, dq, dk, dv, T, heads_q, heads_kv, head_dim);
}

int gt_supports_attention(int32_t T, int32_t head_dim) { return (T > 0 && head_dim == D) ? 1 : 0; }

}  // extern "C"
