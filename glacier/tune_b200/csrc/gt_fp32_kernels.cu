// CUDA-core kernels: exact dequantization, the fp32 validation GEMMs, and the rank-r LoRA products
// (low = X*A, dB, dLow, dA) with fp32 accumulation.  The tensor-core GEMMs live in gt_umma_gemm.cu.
#include "gt_internal.h"
#include "gt_ptx.cuh"
#include "gt_quant.cuh"

namespace gt {

// ------------------------------------------------------------------------------------------------
// Q6_K upload re-layout: GGUF 210-byte block -> 224-byte device block (see gt_quant.cuh).
// ------------------------------------------------------------------------------------------------
__global__ void k_q6k_repack(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int64_t nblocks) {
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (b >= nblocks) return;
    const int lane = threadIdx.x & 31;
    const uint8_t *s = src + b * kQ6KGgufBlockBytes;
    uint8_t *d = dst + b * kQ6KDevBlockBytes;
    for (int i = lane; i < 224; i += 32) {
        uint8_t v = 0;
        if (i < 16) v = s[192 + i];            // scales
        else if (i < 18) v = s[208 + (i - 16)];  // d
        else if (i < 32) v = 0;
        else if (i < 160) v = s[i - 32];       // ql
        else v = s[128 + (i - 160)];           // qh
        d[i] = v;
    }
}
cudaError_t launch_q6k_repack(const uint8_t *gguf_blocks, uint8_t *dev_blocks, int64_t nblocks, cudaStream_t s) {
    if (nblocks <= 0) return cudaSuccess;
    const int wpb = 8;
    k_q6k_repack<<<(unsigned)((nblocks + wpb - 1) / wpb), wpb * 32, 0, s>>>(gguf_blocks, dev_blocks, nblocks);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Row dequantization to fp32, bit-exact with the reference decode.
// ------------------------------------------------------------------------------------------------
template <int QT>
__global__ void k_dequant_rows(const uint8_t *__restrict__ w, int K, int64_t row0, int64_t nrows, float *__restrict__ out) {
    const int64_t total = nrows * (int64_t)K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        out[i] = decode_flat<QT>(w, row0 * (int64_t)K + i);
    }
}
cudaError_t launch_dequant_rows(int qt, const uint8_t *w, int K, int64_t row0, int64_t nrows, float *out, cudaStream_t s) {
    const int64_t total = nrows * (int64_t)K;
    if (total <= 0) return cudaSuccess;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads > 148 * 16 ? 148 * 16 : (total + threads - 1) / threads);
    if (qt == kTypeQ4K) k_dequant_rows<kTypeQ4K><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    else if (qt == kTypeQ6K) k_dequant_rows<kTypeQ6K><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    else if (qt == kTypeF16) k_dequant_rows<kTypeF16><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    else if (qt == kTypeQ40) k_dequant_rows<kTypeQ40><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    else if (qt == kTypeQ80) k_dequant_rows<kTypeQ80><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    else k_dequant_rows<kTypeF32><<<blocks, threads, 0, s>>>(w, K, row0, nrows, out);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// fp32 validation GEMMs (CUDA cores, exact weights).  64x64 output tile, 16-deep slabs, 4x4 per thread.
// Weights are addressed as a flat element stream so tensors whose rows are not whole super-blocks work too.
// ------------------------------------------------------------------------------------------------
constexpr int FT = 64, FS = 16;

template <int QT>
__global__ void __launch_bounds__(256) k_gemm_fp32_fwd(const uint8_t *__restrict__ w, const float *__restrict__ X,
                                                       float *__restrict__ Y, float *__restrict__ residual,
                                                       const float *__restrict__ bias, int T, int N, int K) {
    __shared__ float Xs[FS][FT + 4];
    __shared__ float Ws[FS][FT + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * FT, t0 = blockIdx.y * FT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += FS) {
        {   // X tile: 64 tokens x 16 k; thread -> token tid/4, 4 consecutive k
            const int t = t0 + (tid >> 2), kk = (tid & 3) * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + kk + j;
                Xs[kk + j][tid >> 2] = (t < T && k < K) ? X[(int64_t)t * K + k] : 0.f;
            }
            const int n = n0 + (tid >> 2);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + kk + j;
                Ws[kk + j][tid >> 2] = (n < N && k < K) ? decode_flat<QT>(w, (int64_t)n * K + k) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < FS; k++) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) xv[i] = Xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (residual) residual[(int64_t)t * N + n] += v;
            if (Y) Y[(int64_t)t * N + n] = v;
        }
    }
}

template <int QT>
__global__ void __launch_bounds__(256) k_gemm_fp32_bwd(const uint8_t *__restrict__ w, const float *__restrict__ dY,
                                                       float *__restrict__ dX, int T, int N, int K) {
    __shared__ float Gs[FS][FT + 4];   // dY tile  [n][token]
    __shared__ float Ws[FS][FT + 4];   // W tile   [n][k]
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int k0 = blockIdx.x * FT, t0 = blockIdx.y * FT;
    float acc[4][4] = {};
    for (int n0 = 0; n0 < N; n0 += FS) {
        {
            const int t = t0 + (tid >> 2), nn = (tid & 3) * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + nn + j;
                Gs[nn + j][tid >> 2] = (t < T && n < N) ? dY[(int64_t)t * N + n] : 0.f;
            }
            const int n = n0 + (tid >> 4), kk = (tid & 15) * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + kk + j;
                Ws[tid >> 4][kk + j] = (n < N && k < K) ? decode_flat<QT>(w, (int64_t)n * K + k) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int n = 0; n < FS; n++) {
            float gv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) gv[i] = Gs[n][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[n][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(gv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + tx * 4 + j;
            if (k < K) dX[(int64_t)t * K + k] += acc[i][j];
        }
    }
}

cudaError_t launch_gemm_fp32_fwd(int qt, const uint8_t *w, const float *X, float *Y, float *residual, const float *bias,
                                 int T, int N, int K, cudaStream_t s) {
    if (T <= 0 || N <= 0) return cudaSuccess;
    dim3 grid((N + FT - 1) / FT, (T + FT - 1) / FT);
    if (qt == kTypeQ4K) k_gemm_fp32_fwd<kTypeQ4K><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    else if (qt == kTypeQ6K) k_gemm_fp32_fwd<kTypeQ6K><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    else if (qt == kTypeF16) k_gemm_fp32_fwd<kTypeF16><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    else if (qt == kTypeQ40) k_gemm_fp32_fwd<kTypeQ40><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    else if (qt == kTypeQ80) k_gemm_fp32_fwd<kTypeQ80><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    else k_gemm_fp32_fwd<kTypeF32><<<grid, 256, 0, s>>>(w, X, Y, residual, bias, T, N, K);
    return cudaGetLastError();
}
cudaError_t launch_gemm_fp32_bwd(int qt, const uint8_t *w, const float *dY, float *dX, int T, int N, int K, cudaStream_t s) {
    if (T <= 0 || K <= 0) return cudaSuccess;
    dim3 grid((K + FT - 1) / FT, (T + FT - 1) / FT);
    if (qt == kTypeQ4K) k_gemm_fp32_bwd<kTypeQ4K><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    else if (qt == kTypeQ6K) k_gemm_fp32_bwd<kTypeQ6K><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    else if (qt == kTypeF16) k_gemm_fp32_bwd<kTypeF16><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    else if (qt == kTypeQ40) k_gemm_fp32_bwd<kTypeQ40><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    else if (qt == kTypeQ80) k_gemm_fp32_bwd<kTypeQ80><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    else k_gemm_fp32_bwd<kTypeF32><<<grid, 256, 0, s>>>(w, dY, dX, T, N, K);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// 16-bit rounding helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint16_t round16(float v, int fp16) {
    if (fp16) return __half_as_ushort(__float2half_rn(v));
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

__global__ void k_cast16(const float *__restrict__ src, uint16_t *__restrict__ dst, int rows, int cols, int ld, int fp16) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = (int64_t)rows * ld;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / ld), c = (int)(i % ld);
        dst[i] = c < cols ? round16(src[(int64_t)r * cols + c], fp16) : (uint16_t)0;
    }
}
cudaError_t launch_cast16(const float *src, void *dst, int rows, int cols, int ld_dst, int fp16, cudaStream_t s) {
    const int64_t total = (int64_t)rows * ld_dst;
    if (total <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
    return launch_k(k_cast16, dim3(blocks), dim3(256), 0, s, src, (uint16_t *)dst, rows, cols, ld_dst, fp16);
}

// ------------------------------------------------------------------------------------------------
// Paired rows: a K-quant tensor whose rows are HALF a whole number of super-blocks (in_features % 256 == 128, the
// 4864 x 896 case: 3.5 blocks per row) is, as a byte stream, also the tensor W2 [out / 2, 2 * in] whose row s is row 2s
// followed by row 2s + 1 - and W2 has whole super-blocks per row, so the TMA / tensor-core kernel can read it.
//   forward   Y[t, 2s + h] = X[t] . W[2s + h]  =  X2[2t + h] . W2[s]   with X2[2t] = [X[t] | 0], X2[2t + 1] = [0 | X[t]]
//   backward  dX[t] = sum_s dY[t, 2s] W2[s, :in] + dY[t, 2s + 1] W2[s, in:]  =  Z[2t, :in] + Z[2t + 1, in:],
//             Z = dY2 W2 with dY2[2t + h, s] = dY[t, 2s + h]
// Half of the MMA work multiplies zeros; what it buys is the tensor path for a shape that otherwise runs on CUDA cores.
// ------------------------------------------------------------------------------------------------
// x2 [2T, 2K] 16-bit from X [T, K] fp32
__global__ void k_pair_expand16(const float *__restrict__ X, uint16_t *__restrict__ x2, int T, int K, int fp16) {
    const int64_t total = (int64_t)2 * T * 2 * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % (2 * K));
        const int64_t r = i / (2 * K);
        const int h = (int)(r & 1);
        const int64_t t = r >> 1;
        const bool live = (c >= K) == (h == 1);
        const float v = live ? X[t * K + (c - h * K)] : 0.f;
        x2[i] = fp16 ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
}
// Y [T, N] (+)= tmp [2T, N / 2] interleaved, + bias
__global__ void k_pair_interleave(const float *__restrict__ tmp, const float *__restrict__ bias, float *__restrict__ Y, int T, int N) {
    const int64_t total = (int64_t)T * N;
    const int half = N >> 1;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int n = (int)(i % N);
        const int64_t t = i / N;
        Y[i] = tmp[(2 * t + (n & 1)) * half + (n >> 1)] + (bias ? bias[n] : 0.f);
    }
}
// dy2 [2T, ld] 16-bit: dy2[2t + h, s] = dY[t, 2s + h]; columns at and beyond N / 2 are zero
__global__ void k_pair_gather16(const float *__restrict__ dY, uint16_t *__restrict__ dy2, int T, int N, int ld, int fp16) {
    const int64_t total = (int64_t)2 * T * ld;
    const int half = N >> 1;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int s = (int)(i % ld);
        const int64_t r = i / ld;
        const float v = s < half ? dY[(r >> 1) * N + 2 * s + (int)(r & 1)] : 0.f;
        dy2[i] = fp16 ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
}
// dX [T, K] (= or +=) Z[2t, :K] + Z[2t + 1, K:]
__global__ void k_pair_fold(const float *__restrict__ Z, float *__restrict__ dX, int T, int K, int assign) {
    const int64_t total = (int64_t)T * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % K);
        const int64_t t = i / K;
        const float v = Z[(2 * t) * 2 * K + k] + Z[(2 * t + 1) * 2 * K + K + k];
        dX[i] = assign ? v : dX[i] + v;
    }
}
static unsigned pair_blocks(int64_t total) { return (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256); }
cudaError_t launch_pair_expand16(const float *X, void *x2, int T, int K, int fp16, cudaStream_t s) {
    k_pair_expand16<<<pair_blocks((int64_t)4 * T * K), 256, 0, s>>>(X, (uint16_t *)x2, T, K, fp16);
    return cudaGetLastError();
}
cudaError_t launch_pair_interleave(const float *tmp, const float *bias, float *Y, int T, int N, cudaStream_t s) {
    k_pair_interleave<<<pair_blocks((int64_t)T * N), 256, 0, s>>>(tmp, bias, Y, T, N);
    return cudaGetLastError();
}
cudaError_t launch_pair_gather16(const float *dY, void *dy2, int T, int N, int ld, int fp16, cudaStream_t s) {
    k_pair_gather16<<<pair_blocks((int64_t)2 * T * ld), 256, 0, s>>>(dY, (uint16_t *)dy2, T, N, ld, fp16);
    return cudaGetLastError();
}
cudaError_t launch_pair_fold(const float *Z, float *dX, int T, int K, int assign, cudaStream_t s) {
    k_pair_fold<<<pair_blocks((int64_t)T * K), 256, 0, s>>>(Z, dX, T, K, assign);
    return cudaGetLastError();
}

__global__ void k_fill_rows(float *__restrict__ Y, const float *__restrict__ bias, int T, int N) {
    pdl_wait();
    pdl_trigger();
    const int64_t total = (int64_t)T * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        Y[i] = bias ? bias[i % N] : 0.f;
}
cudaError_t launch_fill_rows(float *Y, const float *bias, int T, int N, cudaStream_t s) {
    const int64_t total = (int64_t)T * N;
    if (total <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
    return launch_k(k_fill_rows, dim3(blocks), dim3(256), 0, s, Y, bias, T, N);
}

__global__ void k_add_inplace(float *__restrict__ dst, const float *__restrict__ src, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] += src[i];
}
cudaError_t launch_add_inplace(float *dst, const float *src, int64_t n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
    k_add_inplace<<<blocks, 256, 0, s>>>(dst, src, n);
    return cudaGetLastError();
}

__global__ void k_any_nonzero(const float *__restrict__ b, int64_t n, int *flag) {
    int found = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        if (b[i] != 0.f) found = 1;
    if (__syncthreads_or(found) && threadIdx.x == 0) atomicOr(flag, 1);
}
cudaError_t launch_any_nonzero(const float *B, int64_t n, int *flag, cudaStream_t s) {
    cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int), s);
    if (e != cudaSuccess || n <= 0) return e;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 296 ? 296 : (n + 255) / 256);
    k_any_nonzero<<<blocks, 256, 0, s>>>(B, n, flag);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// low[T, R] = X[T, K] * A[K, R]   (src/Glacier.Tune/Kernels/LoraKernels.cs:35-54 on the CPU path)
// Block: 4 tokens x all K, 256 threads stride over K, 16 ranks [r0, r0+16) per launch.
// The same pass can emit the 16-bit copy of X that the tensor-core GEMM reads.
// ------------------------------------------------------------------------------------------------
constexpr int LOW_TOK = 4;
__global__ void __launch_bounds__(256) k_lora_low(const float *__restrict__ X, const float *__restrict__ A,
                                                  float *__restrict__ low, uint16_t *__restrict__ x16, int ldx16, int fp16,
                                                  int T, int K, int R, int r0) {
    __shared__ float red[8][LOW_TOK][16];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.x * LOW_TOK;
    const int rc = min(16, R - r0);
    float acc[LOW_TOK][16];
#pragma unroll
    for (int i = 0; i < LOW_TOK; i++)
#pragma unroll
        for (int r = 0; r < 16; r++) acc[i][r] = 0.f;
    for (int k = tid; k < K; k += 256) {
        float a[16];
        if (rc == 16 && (R & 3) == 0) {
            const float4 *ap = reinterpret_cast<const float4 *>(A + (int64_t)k * R + r0);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 v = ap[q];
                a[4 * q] = v.x; a[4 * q + 1] = v.y; a[4 * q + 2] = v.z; a[4 * q + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int r = 0; r < 16; r++) a[r] = r < rc ? A[(int64_t)k * R + r0 + r] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < LOW_TOK; i++) {
            const int t = t0 + i;
            const float xv = t < T ? X[(int64_t)t * K + k] : 0.f;
            if (x16 && t < T) x16[(int64_t)t * ldx16 + k] = round16(xv, fp16);
#pragma unroll
            for (int r = 0; r < 16; r++) acc[i][r] = fmaf(xv, a[r], acc[i][r]);
        }
    }
#pragma unroll
    for (int i = 0; i < LOW_TOK; i++)
#pragma unroll
        for (int r = 0; r < 16; r++) {
            float v = acc[i][r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp][i][r] = v;
        }
    __syncthreads();
    if (tid < LOW_TOK * 16) {
        const int i = tid >> 4, r = tid & 15;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; wv++) v += red[wv][i][r];
        const int t = t0 + i;
        if (t < T && r < rc) low[(int64_t)t * R + r0 + r] = v;
    }
}
cudaError_t launch_lora_low(const float *X, const float *A, float *low, void *x16, int ldx16, int fp16, int T, int K, int R,
                            cudaStream_t s) {
    if (T <= 0 || R <= 0) return cudaSuccess;
    for (int r0 = 0; r0 < R; r0 += 16) {
        k_lora_low<<<(T + LOW_TOK - 1) / LOW_TOK, 256, 0, s>>>(X, A, low, r0 == 0 ? (uint16_t *)x16 : nullptr, ldx16, fp16,
                                                                T, K, R, r0);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// Y[t, n] += sum_r (low[t, r] * scaling) * B[r, n]   (LoraKernels.cs:57-86); fp32 validation path.
__global__ void k_lora_delta_fp32(const float *__restrict__ low, const float *__restrict__ B, float *__restrict__ Y,
                                  float *__restrict__ residual, int T, int N, int R, float scaling,
                                  const int *__restrict__ nonzero_flag) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (n >= N || t >= T) return;
    if (nonzero_flag && *nonzero_flag == 0) return;   // LoraAdapter.IsZeroDelta: B == 0 skips the delta
    float acc = 0.f;
    for (int r = 0; r < R; r++) acc = fmaf(low[(int64_t)t * R + r] * scaling, B[(int64_t)r * N + n], acc);
    if (Y) Y[(int64_t)t * N + n] += acc;
    if (residual) residual[(int64_t)t * N + n] += acc;
}
cudaError_t launch_lora_delta_fp32(const float *low, const float *B, float *Y, float *residual, int T, int N, int R,
                                   float scaling, const int *nonzero_flag, cudaStream_t s) {
    if (T <= 0 || N <= 0 || R <= 0) return cudaSuccess;
    dim3 grid((N + 255) / 256, T);
    k_lora_delta_fp32<<<grid, 256, 0, s>>>(low, B, Y, residual, T, N, R, scaling, nonzero_flag);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// One pass over dY[T, N] (LoraKernels.cs:191-246 on the CPU path):
//     dB[r, n]  += scaling * sum_t low[t, r] * dY[t, n]
//     dLow[t,r] += sum_n dY[t, n] * B[r, n]            (dLow pre-zeroed by the caller)
//     dy16[t,n]  = round16(dY[t, n])                   (optional operand copy for the tensor-core dX GEMM)
// Block: 128 columns x a token group, walked in 32-token sub-tiles staged in shared memory.
// ------------------------------------------------------------------------------------------------
constexpr int DY_COLS = 128, DY_TOK = 32;
__global__ void __launch_bounds__(256) k_lora_bwd_dy(const float *__restrict__ dY, const float *__restrict__ low,
                                                     const float *__restrict__ B, float *__restrict__ dB,
                                                     float *__restrict__ dLow, uint16_t *__restrict__ dy16, int ld16,
                                                     int fp16, float scaling, int T, int N, int R, int r0, int tok_per_group) {
    __shared__ float Gs[DY_TOK][DY_COLS + 1];
    __shared__ float Bs[16][DY_COLS + 1];
    __shared__ float Ls[DY_TOK][16];
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * DY_COLS;
    const int tg0 = blockIdx.y * tok_per_group, tg1 = min(T, tg0 + tok_per_group);
    const int rc = min(16, R - r0);
    for (int i = tid; i < 16 * DY_COLS; i += 256) {
        const int r = i / DY_COLS, c = i % DY_COLS;
        Bs[r][c] = (r < rc && n0 + c < N) ? B[(int64_t)(r0 + r) * N + n0 + c] : 0.f;
    }
    const int col = tid & 127, hf = tid >> 7;       // phase 1: column, token half
    const int pt = tid >> 3, rg = tid & 7;          // phase 2: token, rank pair
    float accB[16];
#pragma unroll
    for (int r = 0; r < 16; r++) accB[r] = 0.f;
    for (int ts = tg0; ts < tg1; ts += DY_TOK) {
        __syncthreads();
        for (int i = tid; i < DY_TOK * DY_COLS; i += 256) {
            const int tt = i / DY_COLS, c = i % DY_COLS;
            const int t = ts + tt, n = n0 + c;
            float v = 0.f;
            if (t < tg1 && n < N) {
                v = dY[(int64_t)t * N + n];
                if (dy16 && r0 == 0) dy16[(int64_t)t * ld16 + n] = round16(v, fp16);
            }
            Gs[tt][c] = v;
        }
        for (int i = tid; i < DY_TOK * 16; i += 256) {
            const int tt = i >> 4, r = i & 15;
            const int t = ts + tt;
            Ls[tt][r] = (t < tg1 && r < rc) ? low[(int64_t)t * R + r0 + r] : 0.f;
        }
        __syncthreads();
        // phase 1: dB partial, thread = (column, token half)
#pragma unroll 4
        for (int tt = hf * 16; tt < hf * 16 + 16; tt++) {
            const float g = Gs[tt][col];
#pragma unroll
            for (int r = 0; r < 16; r++) accB[r] = fmaf(Ls[tt][r], g, accB[r]);
        }
        // phase 2: dLow partial, thread = (token, rank pair)
        {
            float d0 = 0.f, d1 = 0.f;
#pragma unroll 8
            for (int c = 0; c < DY_COLS; c++) {
                const float g = Gs[pt][c];
                d0 = fmaf(g, Bs[2 * rg][c], d0);
                d1 = fmaf(g, Bs[2 * rg + 1][c], d1);
            }
            const int t = ts + pt;
            if (t < tg1) {
                if (2 * rg < rc) atomicAdd(&dLow[(int64_t)t * R + r0 + 2 * rg], d0);
                if (2 * rg + 1 < rc) atomicAdd(&dLow[(int64_t)t * R + r0 + 2 * rg + 1], d1);
            }
        }
    }
    const int n = n0 + col;
    if (n < N) {
#pragma unroll
        for (int r = 0; r < 16; r++)
            if (r < rc) atomicAdd(&dB[(int64_t)(r0 + r) * N + n], accB[r] * scaling);
    }
}
cudaError_t launch_lora_bwd_dy(const float *dY, const float *low, const float *B, float *dB, float *dLow, void *dy16,
                               int ld16, int fp16, float scaling, int T, int N, int R, cudaStream_t s) {
    if (T <= 0 || N <= 0 || R <= 0) return cudaSuccess;
    const int col_blocks = (N + DY_COLS - 1) / DY_COLS;
    int groups = (2 * 148 + col_blocks - 1) / col_blocks;
    const int max_groups = (T + DY_TOK - 1) / DY_TOK;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1) groups = 1;
    int tpg = (T + groups - 1) / groups;
    tpg = (tpg + DY_TOK - 1) / DY_TOK * DY_TOK;
    groups = (T + tpg - 1) / tpg;
    for (int r0 = 0; r0 < R; r0 += 16) {
        k_lora_bwd_dy<<<dim3(col_blocks, groups), 256, 0, s>>>(dY, low, B, dB, dLow, (uint16_t *)dy16, ld16, fp16, scaling, T,
                                                               N, R, r0, tpg);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// dA[k, r] += scaling * sum_t X[t, k] * dLow[t, r]   (LoraKernels.cs:251-291)
constexpr int DA_COLS = 128;
__global__ void __launch_bounds__(128) k_lora_bwd_x(const float *__restrict__ X, const float *__restrict__ dLow,
                                                    float *__restrict__ dA, float scaling, int T, int K, int R, int r0,
                                                    int tok_per_group) {
    __shared__ float Ls[64][16];
    const int tid = threadIdx.x;
    const int k = blockIdx.x * DA_COLS + tid;
    const int tg0 = blockIdx.y * tok_per_group, tg1 = min(T, tg0 + tok_per_group);
    const int rc = min(16, R - r0);
    float acc[16];
#pragma unroll
    for (int r = 0; r < 16; r++) acc[r] = 0.f;
    for (int ts = tg0; ts < tg1; ts += 64) {
        __syncthreads();
        for (int i = tid; i < 64 * 16; i += 128) {
            const int tt = i >> 4, r = i & 15;
            const int t = ts + tt;
            Ls[tt][r] = (t < tg1 && r < rc) ? dLow[(int64_t)t * R + r0 + r] : 0.f;
        }
        __syncthreads();
        if (k < K) {
            const int tn = min(64, tg1 - ts);
            for (int tt = 0; tt < tn; tt++) {
                const float xv = X[(int64_t)(ts + tt) * K + k];
#pragma unroll
                for (int r = 0; r < 16; r++) acc[r] = fmaf(xv, Ls[tt][r], acc[r]);
            }
        }
    }
    if (k < K) {
#pragma unroll
        for (int r = 0; r < 16; r++)
            if (r < rc) atomicAdd(&dA[(int64_t)k * R + r0 + r], acc[r] * scaling);
    }
}
cudaError_t launch_lora_bwd_x(const float *X, const float *dLow, float *dA, float scaling, int T, int K, int R, cudaStream_t s) {
    if (T <= 0 || K <= 0 || R <= 0) return cudaSuccess;
    const int col_blocks = (K + DA_COLS - 1) / DA_COLS;
    int groups = (4 * 148 + col_blocks - 1) / col_blocks;
    const int max_groups = (T + 63) / 64;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1) groups = 1;
    int tpg = (T + groups - 1) / groups;
    tpg = (tpg + 63) / 64 * 64;
    groups = (T + tpg - 1) / tpg;
    for (int r0 = 0; r0 < R; r0 += 16) {
        k_lora_bwd_x<<<dim3(col_blocks, groups), 128, 0, s>>>(X, dLow, dA, scaling, T, K, R, r0, tpg);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// dX[t, k] += scaling * <dLow[t, :], A[k, :]>   (LoraKernels.cs:296-339); fp32 validation path.
__global__ void k_lora_dx_fp32(const float *__restrict__ dLow, const float *__restrict__ A, float *__restrict__ dX,
                               float scaling, int T, int K, int R) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (k >= K || t >= T) return;
    float acc = 0.f;
    for (int r = 0; r < R; r++) acc = fmaf(dLow[(int64_t)t * R + r], A[(int64_t)k * R + r], acc);
    dX[(int64_t)t * K + k] += acc * scaling;
}
cudaError_t launch_lora_dx_fp32(const float *dLow, const float *A, float *dX, float scaling, int T, int K, int R, cudaStream_t s) {
    if (T <= 0 || K <= 0 || R <= 0) return cudaSuccess;
    dim3 grid((K + 255) / 256, T);
    k_lora_dx_fp32<<<grid, 256, 0, s>>>(dLow, A, dX, scaling, T, K, R);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Gradient scaling + global-norm clip (src/Glacier.Tune/Trainer/LoraTrainer.cs:352-377,395-433):
// g *= pre_scale; norm = sqrt(sum g^2) in fp64; non-finite norm -> all zero; norm > max -> g *= max/(norm+1e-6).
// scratch[0] = sum of squares, scratch[1] = norm reported to the host.
// ------------------------------------------------------------------------------------------------
__global__ void k_scale_sumsq(float *__restrict__ g, int64_t n, float pre_scale, double *scratch) {
    double ss = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = g[i] * pre_scale;
        if (pre_scale != 1.0f) g[i] = v;
        ss += (double)v * (double)v;
    }
    __shared__ double red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
        atomicAdd(&scratch[0], t);
    }
}
__global__ void k_clip_apply(float *__restrict__ g, int64_t n, double max_norm, double *scratch) {
    const double norm = sqrt(scratch[0]);
    // ClipGradients returns at once when maxNorm <= 0 (LoraTrainer.cs:398): the gradients stay as they are, even
    // non-finite ones; only a positive maxNorm zeroes them on a non-finite norm (LoraTrainer.cs:417-424)
    const bool bad = max_norm > 0.0 && (isnan(norm) || isinf(norm));
    if (blockIdx.x == 0 && threadIdx.x == 0) scratch[1] = bad ? 0.0 : norm;
    if (!bad && !(max_norm > 0.0 && norm > max_norm)) return;
    const float sc = bad ? 0.f : (float)(max_norm / (norm + 1e-6));
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        g[i] = bad ? 0.f : g[i] * sc;
}
__global__ void k_scale(float *__restrict__ g, int64_t n, float scale) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) g[i] *= scale;
}
cudaError_t launch_scale(float *g, int64_t n, float scale, cudaStream_t s) {
    if (n <= 0 || scale == 1.0f) return cudaSuccess;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
    k_scale<<<blocks, 256, 0, s>>>(g, n, scale);
    return cudaGetLastError();
}
cudaError_t launch_scale_clip(float *g, int64_t n, float pre_scale, double max_norm, double *scratch, cudaStream_t s) {
    cudaError_t e = cudaMemsetAsync(scratch, 0, 2 * sizeof(double), s);
    if (e != cudaSuccess) return e;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
    k_scale_sumsq<<<blocks ? blocks : 1, 256, 0, s>>>(g, n, pre_scale, scratch);
    k_clip_apply<<<blocks ? blocks : 1, 256, 0, s>>>(g, n, max_norm, scratch);
    return cudaGetLastError();
}

}  // namespace gt
