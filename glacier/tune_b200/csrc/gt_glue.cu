// Layer glue between the projections, on device tensors (asynchronous on the engine stream): SwiGLU, RoPE, RMSNorm and
// the residual add.  All of it is one pass over fp32 activations and bound by HBM bandwidth; the reference runs these
// loops on the host between its GPU calls:
//   SwiGLU   src/Glacier.Tune/Kernels/SwiGluKernel.cs:13-60
//   RoPE     src/Glacier.Tune/Kernels/RoPEKernel.cs:12-126 (pairs (i, i + half), freq = base^(-2i/d), inverse = -sin)
//   RMSNorm  ElementwiseKernels.RMSNorm / RMSNormBackward of Glacier.Tensor 1.1.0 (not in the repository; call sites
//            src/Glacier.Tune/Model/TransformerBlock.cs:318,524,672,827, frozen weight: dW is never asked for)
//   add      TensorOps.Add (residual connections, src/Glacier.Tune/Model/TransformerBlock.cs:675)
//   AdamW    the optimizer step on the adapter matrices (AdamW of Glacier.Tensor 1.1.0, not in the repository; built
//            and stepped in src/Glacier.Tune/Trainer/LoraTrainer.cs:56-62,230): textbook decoupled weight decay
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdio>
#include <mutex>

#include "../../../include/glaciertune_b200.h"
#include "gt_internal.h"
#include "gt_ptx.cuh"

namespace {

using gt::pdl_trigger;
using gt::pdl_wait;

__device__ __forceinline__ float sigmoidf_(float g) { return 1.0f / (1.0f + expf(-g)); }

// vectorized when every pointer is 16-byte aligned; n4 = number of float4, tail handled by the scalar loop
__global__ void __launch_bounds__(256) k_swiglu_fwd(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ hidden,
                                                    int64_t n, int vec) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t n4 = n >> 2;
        for (int64_t i = tid; i < n4; i += nth) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gate) + i), u = __ldg(reinterpret_cast<const float4 *>(up) + i);
            float4 h;
            h.x = g.x * sigmoidf_(g.x) * u.x;
            h.y = g.y * sigmoidf_(g.y) * u.y;
            h.z = g.z * sigmoidf_(g.z) * u.z;
            h.w = g.w * sigmoidf_(g.w) * u.w;
            reinterpret_cast<float4 *>(hidden)[i] = h;
        }
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += nth) {
        const float g = gate[i];
        hidden[i] = g * sigmoidf_(g) * up[i];
    }
}

// The same with a 16-bit copy written in the same pass (and the fp32 tensor only when it is wanted): the down
// projection's tensor-core GEMM reads the 16-bit copy, so SiLU(gate) * up never has to be read back in fp32 to be cast
// (GpuLoraEngine.ForwardFfn fuses the activation into its gate / up kernel, gemm_q4_k_swiglu_batch,
// src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:152-183,282-285; here the gate and up tiles of a token live in different
// CTAs of the GEMM, so the activation is folded into the pass that prepares the down projection's operand instead).
__global__ void __launch_bounds__(256) k_swiglu_fwd16(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ hidden,
                                                      uint16_t *__restrict__ h16, int64_t n4, int fp16) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n4; i += nth) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(gate) + i), u = __ldg(reinterpret_cast<const float4 *>(up) + i);
        float4 h;
        h.x = g.x * sigmoidf_(g.x) * u.x;
        h.y = g.y * sigmoidf_(g.y) * u.y;
        h.z = g.z * sigmoidf_(g.z) * u.z;
        h.w = g.w * sigmoidf_(g.w) * u.w;
        if (hidden) reinterpret_cast<float4 *>(hidden)[i] = h;
        uint2 pk;
        if (fp16) {
            __half2 a = __floats2half2_rn(h.x, h.y), b = __floats2half2_rn(h.z, h.w);
            pk = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(h.x, h.y), b = __floats2bfloat162_rn(h.z, h.w);
            pk = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        }
        reinterpret_cast<uint2 *>(h16)[i] = pk;
    }
}

// AdamW over up to kAdamwSegs flat segments (the A and B of several adapters) in one launch: 16 B of parameter,
// gradient and both moments read and 12 B written per element, nothing else.  c1 = 1/(1-beta1^t), c2 = 1/(1-beta2^t),
// decay = 1-lr*wd.  A segment with a flag pointer raises the flag when it leaves a non-zero parameter behind (the
// adapter's "B may be non-zero" word; it is never lowered here: a B that an update returned to exactly zero would
// only cost the delta's arithmetic, not change a result).
struct AdamwHyper {
    float lr, beta1, beta2, eps, decay, c1, c2;
};
struct AdamwBatch {
    gt::AdamwSeg seg[gt::kAdamwSegs];
    int64_t start[gt::kAdamwSegs + 1];      // prefix sum of the segments' work units: a float4 (vec) or one element
    int n;
};
__device__ __forceinline__ void adamw1(float &p, float g, float &m, float &v, const AdamwHyper &h) {
    m = h.beta1 * m + (1.0f - h.beta1) * g;
    v = h.beta2 * v + (1.0f - h.beta2) * g * g;
    p = p * h.decay - h.lr * (m * h.c1) / (sqrtf(v * h.c2) + h.eps);
}
// One grid-stride loop over the units of ALL segments (not one loop per segment: the segments of an adapter are a
// few hundred KB each, and sixteen dependent rounds of DRAM latency would bound the launch).
__global__ void __launch_bounds__(256) k_adamw(const __grid_constant__ AdamwBatch b, AdamwHyper h) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    const int64_t total = b.start[b.n];
    const int lane = threadIdx.x & 31;
    for (int64_t u = tid; u < total; u += nth) {
        int si = 0;
        while (si + 1 < b.n && u >= b.start[si + 1]) si++;
        const gt::AdamwSeg &s = b.seg[si];
        const int64_t i = u - b.start[si];
        bool nz;
        if (s.vec) {
            float4 p = reinterpret_cast<float4 *>(s.p)[i], m = reinterpret_cast<float4 *>(s.m)[i], v = reinterpret_cast<float4 *>(s.v)[i];
            const float4 g = __ldg(reinterpret_cast<const float4 *>(s.g) + i);
            adamw1(p.x, g.x, m.x, v.x, h);
            adamw1(p.y, g.y, m.y, v.y, h);
            adamw1(p.z, g.z, m.z, v.z, h);
            adamw1(p.w, g.w, m.w, v.w, h);
            nz = p.x != 0.f || p.y != 0.f || p.z != 0.f || p.w != 0.f;
            reinterpret_cast<float4 *>(s.p)[i] = p;
            reinterpret_cast<float4 *>(s.m)[i] = m;
            reinterpret_cast<float4 *>(s.v)[i] = v;
        } else {
            adamw1(s.p[i], s.g[i], s.m[i], s.v[i], h);
            nz = s.p[i] != 0.f;
        }
        // one flag store per warp and segment: the lanes of a warp that are in the same segment vote
        const unsigned peers = __match_any_sync(__activemask(), si);
        const bool any = __any_sync(peers, nz);
        if (any && s.flag != nullptr && lane == __ffs(peers) - 1) *s.flag = 1;
    }
    // the last n % 4 elements of the vectorized segments
    if (blockIdx.x == 0) {
        for (int si = 0; si < b.n; si++) {
            const gt::AdamwSeg &s = b.seg[si];
            const int rem = s.vec ? (int)(s.n & 3) : 0;
            if ((int)threadIdx.x < rem) {
                const int64_t i = (s.n & ~(int64_t)3) + threadIdx.x;
                adamw1(s.p[i], s.g[i], s.m[i], s.v[i], h);
                if (s.flag != nullptr && s.p[i] != 0.f) *s.flag = 1;
            }
        }
    }
}

__device__ __forceinline__ void swiglu_bwd1(float d, float g, float u, float &dg, float &du) {
    const float sig = sigmoidf_(g);
    du = d * (g * sig);
    dg = d * u * (sig * (1.0f + g * (1.0f - sig)));
}
__global__ void __launch_bounds__(256) k_swiglu_bwd(const float *__restrict__ dh, const float *__restrict__ gate, const float *__restrict__ up,
                                                    float *__restrict__ dgate, float *__restrict__ dup, int64_t n, int vec) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t n4 = n >> 2;
        for (int64_t i = tid; i < n4; i += nth) {
            const float4 d = __ldg(reinterpret_cast<const float4 *>(dh) + i), g = __ldg(reinterpret_cast<const float4 *>(gate) + i),
                         u = __ldg(reinterpret_cast<const float4 *>(up) + i);
            float4 a, b;
            swiglu_bwd1(d.x, g.x, u.x, a.x, b.x);
            swiglu_bwd1(d.y, g.y, u.y, a.y, b.y);
            swiglu_bwd1(d.z, g.z, u.z, a.z, b.z);
            swiglu_bwd1(d.w, g.w, u.w, a.w, b.w);
            reinterpret_cast<float4 *>(dgate)[i] = a;
            reinterpret_cast<float4 *>(dup)[i] = b;
        }
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += nth) swiglu_bwd1(dh[i], gate[i], up[i], dgate[i], dup[i]);
}

// The same with the two gradients written as bf16 only: they are the 16-bit operands of the gate,up projections'
// transpose GEMM and of their adapters' products, and nothing else reads them (8 bytes less written and 8 less read
// again per element than through the fp32 pair).
__global__ void __launch_bounds__(256) k_swiglu_bwd16(const float *__restrict__ dh, const float *__restrict__ gate, const float *__restrict__ up,
                                                      uint16_t *__restrict__ dg16, uint16_t *__restrict__ du16, int64_t n4) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n4; i += nth) {
        const float4 d = __ldg(reinterpret_cast<const float4 *>(dh) + i), g = __ldg(reinterpret_cast<const float4 *>(gate) + i),
                     u = __ldg(reinterpret_cast<const float4 *>(up) + i);
        float4 a, b;
        swiglu_bwd1(d.x, g.x, u.x, a.x, b.x);
        swiglu_bwd1(d.y, g.y, u.y, a.y, b.y);
        swiglu_bwd1(d.z, g.z, u.z, a.z, b.z);
        swiglu_bwd1(d.w, g.w, u.w, a.w, b.w);
        const __nv_bfloat162 a0 = __floats2bfloat162_rn(a.x, a.y), a1 = __floats2bfloat162_rn(a.z, a.w);
        const __nv_bfloat162 b0 = __floats2bfloat162_rn(b.x, b.y), b1 = __floats2bfloat162_rn(b.z, b.w);
        reinterpret_cast<uint2 *>(dg16)[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
        reinterpret_cast<uint2 *>(du16)[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&b0), *reinterpret_cast<const uint32_t *>(&b1));
    }
}

__global__ void __launch_bounds__(256) k_add(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int64_t n, int vec) {
    pdl_wait();
    pdl_trigger();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t n4 = n >> 2;
        for (int64_t i = tid; i < n4; i += nth) {
            const float4 x = __ldg(reinterpret_cast<const float4 *>(a) + i), y = __ldg(reinterpret_cast<const float4 *>(b) + i);
            reinterpret_cast<float4 *>(out)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
        }
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += nth) out[i] = a[i] + b[i];
}

// One block per position: the first threads evaluate cos / sin of the position's angles once into shared memory (powf
// and a sincosf of a large angle, repeated per head, cost more than the memory traffic), then all threads walk the
// (head, pair) items of q and k with coalesced accesses.  freq and theta follow the reference's fp32 order.
constexpr int kRopeMaxHalf = 256;
__global__ void __launch_bounds__(256) k_rope(float *__restrict__ q, float *__restrict__ k, int T, int heads_q, int heads_kv, int head_dim,
                                              float freq_base, float freq_scale, int eff, float sign, int vec) {
    __shared__ __align__(16) float cs[kRopeMaxHalf], sn[kRopeMaxHalf];
    pdl_wait();
    pdl_trigger();
    const int half = eff >> 1;
    const int pos = blockIdx.x;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float base_freq = 1.0f / powf(freq_base, (float)(2 * i) / (float)eff);
        const float theta = (float)pos * base_freq * freq_scale;
        float s, c;
        sincosf(theta, &s, &c);
        cs[i] = c;
        sn[i] = s * sign;
    }
    __syncthreads();
    const int hq = q ? heads_q : 0, heads = hq + (k ? heads_kv : 0);
    if (vec) {      // four pairs per thread: 16-byte loads and stores of both halves
        const int hq4 = half >> 2;
        for (int it = threadIdx.x; it < heads * hq4; it += blockDim.x) {
            const int h = it / hq4, i = (it - h * hq4) << 2;
            float *p = h < hq ? q + ((int64_t)pos * heads_q + h) * head_dim + i : k + ((int64_t)pos * heads_kv + (h - hq)) * head_dim + i;
            const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + half);
            const float4 c = *reinterpret_cast<const float4 *>(cs + i), s = *reinterpret_cast<const float4 *>(sn + i);
            *reinterpret_cast<float4 *>(p) = make_float4(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y, a.z * c.z - b.z * s.z, a.w * c.w - b.w * s.w);
            *reinterpret_cast<float4 *>(p + half) = make_float4(a.x * s.x + b.x * c.x, a.y * s.y + b.y * c.y, a.z * s.z + b.z * c.z, a.w * s.w + b.w * c.w);
        }
        return;
    }
    for (int it = threadIdx.x; it < heads * half; it += blockDim.x) {
        const int h = it / half, i = it - h * half;
        float *p = h < hq ? q + ((int64_t)pos * heads_q + h) * head_dim + i : k + ((int64_t)pos * heads_kv + (h - hq)) * head_dim + i;
        const float c = cs[i], s = sn[i];
        const float v0 = p[0], v1 = p[half];
        p[0] = v0 * c - v1 * s;
        p[half] = v0 * s + v1 * c;
    }
}

// block-wide sum of up to two values (256 threads)
__device__ __forceinline__ void block_sum2(float &a, float &b) {
    __shared__ float sa[8], sb[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();      // the arrays may still be read from an earlier call
    if (lane == 0) {
        sa[warp] = a;
        sb[warp] = b;
    }
    __syncthreads();
    a = 0.f;
    b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) {
        a += sa[w];
        b += sb[w];
    }
}

// One block per token row; the row (H <= 16 * 256 floats kept in registers, longer rows re-read) is read once.
constexpr int kRowRegs = 16;
__global__ void __launch_bounds__(256) k_rmsnorm_fwd(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y, int H,
                                                     float eps) {
    pdl_wait();
    pdl_trigger();
    const float *xr = x + (int64_t)blockIdx.x * H;
    float *yr = y + (int64_t)blockIdx.x * H;
    float v[kRowRegs];
    float ss = 0.f, unused = 0.f;
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < H ? xr[i] : 0.f;
        ss += v[j] * v[j];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) ss += xr[i] * xr[i];
    block_sum2(ss, unused);
    const float r = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < H) yr[i] = v[j] * r * w[i];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) yr[i] = xr[i] * r * w[i];
}

// sum = a + b (written out: the residual stream), y = RMSNorm(sum) * w: the residual add and the norm that follows it
// in one pass (TransformerBlock.cs:518-528: x1 = x + o, then norm2X = RMSNorm(x1)).  The sum is formed once in fp32 and
// both outputs use it, so the values equal the two separate kernels'.
__global__ void __launch_bounds__(256) k_add_rmsnorm_fwd(const float *__restrict__ a, const float *__restrict__ b, const float *__restrict__ w,
                                                         float *__restrict__ sum, float *__restrict__ y, int H, float eps) {
    pdl_wait();
    pdl_trigger();
    const float *ar = a + (int64_t)blockIdx.x * H, *br = b + (int64_t)blockIdx.x * H;
    float *sr = sum + (int64_t)blockIdx.x * H, *yr = y + (int64_t)blockIdx.x * H;
    float v[kRowRegs];
    float ss = 0.f, unused = 0.f;
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < H ? ar[i] + br[i] : 0.f;
        if (i < H) sr[i] = v[j];
        ss += v[j] * v[j];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) {
        const float t = ar[i] + br[i];
        sr[i] = t;
        ss += t * t;
    }
    block_sum2(ss, unused);
    const float r = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < H) yr[i] = v[j] * r * w[i];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) yr[i] = sr[i] * r * w[i];
}

// dx = r * g - x * r^3 * mean(g * x), g = dy * w (frozen weight)
// (+ residual when given: the gradient that bypasses the norm on the residual connection, TransformerBlock.cs:675,838)
__global__ void __launch_bounds__(256) k_rmsnorm_bwd(const float *__restrict__ dy, const float *__restrict__ x, const float *__restrict__ w,
                                                     const float *residual, float *dx, int H, float eps) {
    pdl_wait();
    pdl_trigger();
    const float *xr = x + (int64_t)blockIdx.x * H, *gr = dy + (int64_t)blockIdx.x * H;
    const float *rr = residual ? residual + (int64_t)blockIdx.x * H : nullptr;
    float *dr = dx + (int64_t)blockIdx.x * H;
    // (the residual may alias dx: its values are taken before anything is stored)
    float xv[kRowRegs], gv[kRowRegs], rv[kRowRegs];
    float ss = 0.f, gx = 0.f;
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        xv[j] = i < H ? xr[i] : 0.f;
        gv[j] = i < H ? gr[i] * w[i] : 0.f;
        rv[j] = (rr && i < H) ? rr[i] : 0.f;
        ss += xv[j] * xv[j];
        gx += gv[j] * xv[j];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) {
        ss += xr[i] * xr[i];
        gx += gr[i] * w[i] * xr[i];
    }
    block_sum2(ss, gx);
    const float r = rsqrtf(ss / (float)H + eps);
    const float coef = r * r * r * gx / (float)H;
#pragma unroll
    for (int j = 0; j < kRowRegs; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < H) dr[i] = r * gv[j] - xv[j] * coef + rv[j];
    }
    for (int i = threadIdx.x + kRowRegs * 256; i < H; i += 256) dr[i] = r * gr[i] * w[i] - xr[i] * coef + (rr ? rr[i] : 0.f);
}

int aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
unsigned stream_blocks(int64_t n, int sm_count) {
    const int64_t want = (n / 4 + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 8;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}
int cuda_fail(const char *what, cudaError_t e) {
    char msg[200];
    snprintf(msg, sizeof(msg), "%s: %s", what, cudaGetErrorString(e));
    return gt::set_last_error(GT_ERR_CUDA, msg);
}

}  // namespace

namespace gt {
// launchers for callers inside the library (the fused FFN calls): same kernels, caller holds the engine lock
cudaError_t launch_swiglu_fwd(const float *gate, const float *up, float *hidden, int64_t n, int sm_count, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    return launch_k(k_swiglu_fwd, dim3(stream_blocks(n, sm_count)), dim3(256), (size_t)0, s, gate, up, hidden, n,
                    aligned16(gate) && aligned16(up) && aligned16(hidden) ? 1 : 0);
}
cudaError_t launch_swiglu_fwd16(const float *gate, const float *up, float *hidden, void *h16, int64_t n, int fp16, int sm_count, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    if ((n & 3) != 0 || !aligned16(gate) || !aligned16(up) || (hidden && !aligned16(hidden)) || (reinterpret_cast<uintptr_t>(h16) & 7) != 0)
        return cudaErrorInvalidValue;
    return launch_k(k_swiglu_fwd16, dim3(stream_blocks(n, sm_count)), dim3(256), (size_t)0, s, gate, up, hidden, (uint16_t *)h16, n >> 2, fp16);
}
cudaError_t launch_swiglu_bwd(const float *d_hidden, const float *gate, const float *up, float *d_gate, float *d_up, int64_t n, int sm_count,
                              cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    const int vec = aligned16(d_hidden) && aligned16(gate) && aligned16(up) && aligned16(d_gate) && aligned16(d_up) ? 1 : 0;
    return launch_k(k_swiglu_bwd, dim3(stream_blocks(n, sm_count)), dim3(256), (size_t)0, s, d_hidden, gate, up, d_gate, d_up, n, vec);
}
cudaError_t launch_swiglu_bwd16(const float *d_hidden, const float *gate, const float *up, void *d_gate16, void *d_up16, int64_t n, int sm_count,
                                cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    if ((n & 3) != 0 || !aligned16(d_hidden) || !aligned16(gate) || !aligned16(up) || (reinterpret_cast<uintptr_t>(d_gate16) & 7) != 0 ||
        (reinterpret_cast<uintptr_t>(d_up16) & 7) != 0)
        return cudaErrorInvalidValue;
    return launch_k(k_swiglu_bwd16, dim3(stream_blocks(n, sm_count)), dim3(256), (size_t)0, s, d_hidden, gate, up, (uint16_t *)d_gate16,
                    (uint16_t *)d_up16, n >> 2);
}
cudaError_t launch_add(const float *a, const float *b, float *out, int64_t n, int sm_count, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    return launch_k(k_add, dim3(stream_blocks(n, sm_count)), dim3(256), (size_t)0, s, a, b, out, n, aligned16(a) && aligned16(b) && aligned16(out) ? 1 : 0);
}
cudaError_t launch_rope(float *q, float *k, int T, int heads_q, int heads_kv, int head_dim, float freq_base, float freq_scale, int rope_dim,
                        int inverse, cudaStream_t s) {
    const int eff = (rope_dim > 0 && rope_dim <= head_dim) ? rope_dim : head_dim;      // RoPEKernel.cs:55
    if (T <= 0 || eff / 2 <= 0) return cudaSuccess;
    if (eff / 2 > kRopeMaxHalf) return cudaErrorInvalidValue;      // rotary dimensions above 512 are not served
    // 16-byte accesses where every head's halves start on a 16-byte boundary
    const int vec = (eff / 2) % 4 == 0 && head_dim % 4 == 0 && (!q || aligned16(q)) && (!k || aligned16(k)) ? 1 : 0;
    return launch_k(k_rope, dim3((unsigned)T), dim3(256), (size_t)0, s, q, k, T, heads_q, heads_kv, head_dim, freq_base, freq_scale, eff,
                    inverse ? -1.0f : 1.0f, vec);
}
cudaError_t launch_rmsnorm_fwd(const float *x, const float *w, float *y, int T, int H, float eps, cudaStream_t s) {
    return launch_k(k_rmsnorm_fwd, dim3((unsigned)T), dim3(256), (size_t)0, s, x, w, y, H, eps);
}
cudaError_t launch_rmsnorm_bwd(const float *dy, const float *x, const float *w, const float *residual, float *dx, int T, int H, float eps,
                               cudaStream_t s) {
    return launch_k(k_rmsnorm_bwd, dim3((unsigned)T), dim3(256), (size_t)0, s, dy, x, w, residual, dx, H, eps);
}
cudaError_t launch_add_rmsnorm_fwd(const float *a, const float *b, const float *w, float *sum, float *y, int T, int H, float eps, cudaStream_t s) {
    return launch_k(k_add_rmsnorm_fwd, dim3((unsigned)T), dim3(256), (size_t)0, s, a, b, w, sum, y, H, eps);
}
cudaError_t launch_adamw(const AdamwSeg *segs, int n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                         int sm_count, cudaStream_t s) {
    AdamwHyper h;
    h.lr = lr, h.beta1 = beta1, h.beta2 = beta2, h.eps = eps;
    h.decay = 1.0f - lr * weight_decay;
    h.c1 = (float)(1.0 / (1.0 - pow((double)beta1, (double)step)));
    h.c2 = (float)(1.0 / (1.0 - pow((double)beta2, (double)step)));
    for (int i0 = 0; i0 < n; i0 += kAdamwSegs) {
        AdamwBatch b;
        b.n = 0;
        b.start[0] = 0;
        for (int i = i0; i < n && i < i0 + kAdamwSegs; i++) {
            if (segs[i].n <= 0) continue;
            AdamwSeg &g = b.seg[b.n];
            g = segs[i];
            g.vec = aligned16(g.p) && aligned16(g.g) && aligned16(g.m) && aligned16(g.v) ? 1 : 0;
            b.start[b.n + 1] = b.start[b.n] + (g.vec ? g.n >> 2 : g.n);
            b.n++;
        }
        if (b.n == 0) continue;
        for (int i = b.n; i < kAdamwSegs; i++) b.start[i + 1] = b.start[b.n];
        // units are float4 for aligned segments: size the grid for 4 elements per unit
        const int64_t longest = b.start[b.n] * 4;
        const cudaError_t ce = launch_k(k_adamw, dim3(stream_blocks(longest, sm_count)), dim3(256), (size_t)0, s, b, h);
        if (ce != cudaSuccess) return ce;
    }
    return cudaSuccess;
}
}  // namespace gt

extern "C" int gt_swiglu_forward(gt_engine *eng, const float *gate, const float *up, float *hidden, int64_t n) {
    if (!eng || !gate || !up || !hidden) return gt::set_last_error(GT_ERR_INVALID, "gt_swiglu_forward: null argument");
    if (n <= 0) return GT_OK;
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess)
        ce = gt::launch_k(k_swiglu_fwd, dim3(stream_blocks(n, ev.sm_count)), dim3(256), (size_t)0, ev.stream, gate, up, hidden, n,
                          aligned16(gate) && aligned16(up) && aligned16(hidden) ? 1 : 0);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_swiglu_forward", ce);
}

extern "C" int gt_swiglu_backward(gt_engine *eng, const float *d_hidden, const float *gate, const float *up, float *d_gate, float *d_up,
                                  int64_t n) {
    if (!eng || !d_hidden || !gate || !up || !d_gate || !d_up) return gt::set_last_error(GT_ERR_INVALID, "gt_swiglu_backward: null argument");
    if (n <= 0) return GT_OK;
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    const int vec = aligned16(d_hidden) && aligned16(gate) && aligned16(up) && aligned16(d_gate) && aligned16(d_up) ? 1 : 0;
    if (ce == cudaSuccess)
        ce = gt::launch_k(k_swiglu_bwd, dim3(stream_blocks(n, ev.sm_count)), dim3(256), (size_t)0, ev.stream, d_hidden, gate, up, d_gate,
                          d_up, n, vec);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_swiglu_backward", ce);
}

extern "C" int gt_add(gt_engine *eng, const float *a, const float *b, float *out, int64_t n) {
    if (!eng || !a || !b || !out) return gt::set_last_error(GT_ERR_INVALID, "gt_add: null argument");
    if (n <= 0) return GT_OK;
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess)
        ce = gt::launch_k(k_add, dim3(stream_blocks(n, ev.sm_count)), dim3(256), (size_t)0, ev.stream, a, b, out, n,
                          aligned16(a) && aligned16(b) && aligned16(out) ? 1 : 0);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_add", ce);
}

extern "C" int gt_rope(gt_engine *eng, float *q, float *k, int32_t T, int32_t heads_q, int32_t heads_kv, int32_t head_dim, float freq_base,
                       float freq_scale, int32_t rope_dim, int32_t inverse) {
    if (!eng || (!q && !k)) return gt::set_last_error(GT_ERR_INVALID, "gt_rope: null argument");
    if (T <= 0) return GT_OK;
    if (head_dim <= 0 || (q && heads_q <= 0) || (k && heads_kv <= 0) || freq_base <= 0.f)
        return gt::set_last_error(GT_ERR_INVALID, "gt_rope: head counts, head_dim and freq_base must be positive");
    const int eff = (rope_dim > 0 && rope_dim <= head_dim) ? rope_dim : head_dim;      // RoPEKernel.cs:55
    if (eff / 2 <= 0) return GT_OK;
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess)
        ce = gt::launch_rope(q, k, (int)T, (int)heads_q, (int)heads_kv, (int)head_dim, freq_base, freq_scale, (int)rope_dim, (int)inverse, ev.stream);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_rope", ce);
}

extern "C" int gt_rmsnorm_forward(gt_engine *eng, const float *x, const float *w, float *y, int32_t T, int32_t H, float eps) {
    if (!eng || !x || !w || !y) return gt::set_last_error(GT_ERR_INVALID, "gt_rmsnorm_forward: null argument");
    if (T <= 0 || H <= 0) return gt::set_last_error(GT_ERR_INVALID, "gt_rmsnorm_forward: T and H must be positive");
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess) ce = gt::launch_k(k_rmsnorm_fwd, dim3((unsigned)T), dim3(256), (size_t)0, ev.stream, x, w, y, (int)H, eps);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_rmsnorm_forward", ce);
}

extern "C" int gt_rmsnorm_backward(gt_engine *eng, const float *dy, const float *x, const float *w, float *dx, int32_t T, int32_t H, float eps) {
    if (!eng || !dy || !x || !w || !dx) return gt::set_last_error(GT_ERR_INVALID, "gt_rmsnorm_backward: null argument");
    if (T <= 0 || H <= 0) return gt::set_last_error(GT_ERR_INVALID, "gt_rmsnorm_backward: T and H must be positive");
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess) ce = gt::launch_rmsnorm_bwd(dy, x, w, nullptr, dx, (int)T, (int)H, eps, ev.stream);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_rmsnorm_backward", ce);
}

extern "C" int gt_adamw_step(gt_engine *eng, float *p, const float *g, float *m, float *v, int64_t n, float lr, float beta1, float beta2,
                             float eps, float weight_decay, int32_t step) {
    if (!eng || !p || !g || !m || !v) return gt::set_last_error(GT_ERR_INVALID, "gt_adamw_step: null argument");
    if (step < 1) return gt::set_last_error(GT_ERR_INVALID, "gt_adamw_step: step counts from 1");
    if (!(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f))
        return gt::set_last_error(GT_ERR_INVALID, "gt_adamw_step: beta1 and beta2 must lie in [0, 1)");
    if (n <= 0) return GT_OK;
    const gt::EngineView ev = gt::engine_view(eng);
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(ev.mutex));
    cudaError_t ce = cudaSetDevice(ev.device);
    if (ce == cudaSuccess && gt::engine_join_comm(eng) != GT_OK) return GT_ERR_CUDA;      // a pending gradient exchange comes first
    const gt::AdamwSeg seg{p, g, m, v, nullptr, n, 0};
    if (ce == cudaSuccess) ce = gt::launch_adamw(&seg, 1, lr, beta1, beta2, eps, weight_decay, (int)step, ev.sm_count, ev.stream);
    return ce == cudaSuccess ? GT_OK : cuda_fail("gt_adamw_step", ce);
}
