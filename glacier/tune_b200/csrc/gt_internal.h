// Internal launch interface between the translation units of libglaciertune_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace gt {

// cudaFuncSetAttribute (dynamic shared memory above 48 KB) applies to the CURRENT device only: an engine on a second
// device of the same process needs its own call.  One PerDeviceOnce per kernel (or group of kernels) remembers on
// which devices `fn` has run; thread-safe.
struct PerDeviceOnce {
    std::mutex mu;
    bool done[64] = {};
};
template <typename F>
cudaError_t per_device_once(PerDeviceOnce &st, F &&fn) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return fn();
    std::lock_guard<std::mutex> lk(st.mu);
    if (st.done[dev]) return cudaSuccess;
    e = fn();
    if (e == cudaSuccess) st.done[dev] = true;
    return e;
}

// Device copy of one frozen base tensor.
struct WeightDev {
    int qtype = 0;
    int N = 0, K = 0;             // [out_features, in_features]
    uint8_t *data = nullptr;      // device blocks (Q4_K: GGUF bytes; Q6_K: 224-byte device blocks; F32: floats)
    int64_t nbytes = 0;
    int64_t row_bytes = 0;        // K/256 * block bytes when K % 256 == 0, else 0 (flat super-block stream)
    float *bias = nullptr;        // [N] or null
    bool tma_ok = false;          // row-aligned and tensor maps built
    CUtensorMap tm_hdr, tm_q0, tm_q1;   // 2-D byte maps over [N, row_bytes], boxes of 64 rows (backward raw stages)
    CUtensorMap tm_hdr_f, tm_q0_f, tm_q1_f;   // the same with boxes of 128 rows (forward raw stages: half as many copies)
    CUtensorMap tm_rows;                // Q4_K: 32-bit words over [N, row_bytes / 4], boxes of 16 rows x 288 bytes (two blocks)
    CUtensorMap tm_blk_f, tm_blk_b;     // whole super-blocks: boxes of one block x 256 rows / x 64 rows (few-token kernel)
};

// ---- CUDA-core kernels (gt_fp32_kernels.cu) -------------------------------------------------------------
cudaError_t launch_q6k_repack(const uint8_t *gguf_blocks, uint8_t *dev_blocks, int64_t nblocks, cudaStream_t s);
cudaError_t launch_dequant_rows(int qt, const uint8_t *w, int K, int64_t row0, int64_t nrows, float *out, cudaStream_t s);
cudaError_t launch_gemm_fp32_fwd(int qt, const uint8_t *w, const float *X, float *Y, float *residual, const float *bias,
                                 int T, int N, int K, cudaStream_t s);
cudaError_t launch_gemm_fp32_bwd(int qt, const uint8_t *w, const float *dY, float *dX, int T, int N, int K, cudaStream_t s);

// LoRA (all fp32 arithmetic).  A is [K, R] row-major, B is [R, N] row-major.  Kernels handle ranks
// [r0, r0+16) of R per launch.
// low[T,R] = X*A ; optionally x16[T, ldx16] = round16(X) (r0 == 0 pass only).
cudaError_t launch_lora_low(const float *X, const float *A, float *low, void *x16, int ldx16, int fp16, int T, int K,
                            int R, cudaStream_t s);
// Y[T,N] += scaling * low * B
cudaError_t launch_lora_delta_fp32(const float *low, const float *B, float *Y, float *residual, int T, int N, int R,
                                   float scaling, const int *nonzero_flag, cudaStream_t s);
// One pass over dY: dB += scaling * low^T * dY ; dLow (pre-zeroed) += dY * B^T ; dy16 = round16(dY) (optional).
cudaError_t launch_lora_bwd_dy(const float *dY, const float *low, const float *B, float *dB, float *dLow, void *dy16,
                               int ld16, int fp16, float scaling, int T, int N, int R, cudaStream_t s);
// dA += scaling * X^T * dLow
cudaError_t launch_lora_bwd_x(const float *X, const float *dLow, float *dA, float scaling, int T, int K, int R,
                              cudaStream_t s);
// dX[T,K] += scaling * dLow * A^T
cudaError_t launch_lora_dx_fp32(const float *dLow, const float *A, float *dX, float scaling, int T, int K, int R,
                                cudaStream_t s);
cudaError_t launch_cast16(const float *src, void *dst, int rows, int cols, int ld_dst, int fp16, cudaStream_t s);
// paired-row view of a tensor with in_features % 256 == 128 (see gt_fp32_kernels.cu)
cudaError_t launch_pair_expand16(const float *X, void *x2, int T, int K, int fp16, cudaStream_t s);
cudaError_t launch_pair_interleave(const float *tmp, const float *bias, float *Y, int T, int N, cudaStream_t s);
cudaError_t launch_pair_gather16(const float *dY, void *dy2, int T, int N, int ld, int fp16, cudaStream_t s);
cudaError_t launch_pair_fold(const float *Z, float *dX, int T, int K, int assign, cudaStream_t s);
// Y[t, :] = bias (or 0)
cudaError_t launch_fill_rows(float *Y, const float *bias, int T, int N, cudaStream_t s);
// residual += Y
cudaError_t launch_add_inplace(float *dst, const float *src, int64_t n, cudaStream_t s);
// *flag = any(B != 0)
cudaError_t launch_any_nonzero(const float *B, int64_t n, int *flag, cudaStream_t s);
// scratch: 2 doubles on the device
cudaError_t launch_scale_clip(float *g, int64_t n, float pre_scale, double max_norm, double *scratch, cudaStream_t s);
// g *= scale (no norm, no scratch)
cudaError_t launch_scale(float *g, int64_t n, float scale, cudaStream_t s);

// ---- LoRA products on bf16 warp MMAs for the bf16 math mode (gt_lora_tc.cu); same contracts as the fp32 versions,
// except that `low` / `dLow` must be zero on entry (partial sums arrive by atomics).  Adapters of projections that
// share X go through one pass over it; the dY passes of several members are one launch.  x16 / dy16 (may be null)
// receive the 16-bit copies.
struct LoraXaJob {
    const float *A;
    float *low_zeroed;
    int R;
};
struct LoraDyJob {      // dY == nullptr: dy16 already holds bf16(dY) and is read instead (bf16 mode)
    const float *dY, *low, *B;
    float *dB, *dLow_zeroed;
    void *dy16;
    int ld16;
    float scaling;
    int N, R;
};
struct LoraDaJob {
    const float *dLow;
    float *dA;
    float scaling;
    int R;
};
// dst[T, N] = bias[N] (or zero): up to three such fills ride along with a pass (the output of a split-K GEMM)
struct RowFill {
    float *dst;
    const float *bias;
    int N;
};
cudaError_t launch_lora_xa_group(const float *X, const LoraXaJob *jobs, int n, void *x16, int ldx16, int fp16, int T, int K,
                                 const RowFill *fills, int n_fills, cudaStream_t s);
// the same from an input that already exists as bf16 [T, ld16] (K % 8 == 0, 16-byte aligned): no copy is written
cudaError_t launch_lora_xa16_group(const void *X16, int ld16, const LoraXaJob *jobs, int n, int T, int K, cudaStream_t s);
cudaError_t launch_lora_dy_group(const LoraDyJob *jobs, int n, int fp16, int T, const RowFill *fills, int n_fills, cudaStream_t s);
// dA from an X that exists as bf16 [T, ld16] (K % 8 == 0, 16-byte aligned)
cudaError_t launch_lora_da16_group(const void *X16, int ld16, const LoraDaJob *jobs, int n, int T, int K, cudaStream_t s);
cudaError_t launch_lora_da_group(const float *X, const LoraDaJob *jobs, int n, int T, int K, cudaStream_t s);

// ---- tcgen05 kernels (gt_umma_gemm.cu) ------------------------------------------------------------------
struct UmmaLaunch {
    const WeightDev *w = nullptr;
    int backward = 0;              // 0: out[T,N] = act[T,K] * W^T ; 1: out[T,K] += act[T,N] * W
    int fp16 = 0;                  // operand format: 0 bf16, 1 fp16
    const void *act16 = nullptr;   // 16-bit activations [T, ld_act]
    int ld_act = 0;
    int T = 0;
    float *out = nullptr;          // fp32 [T, ld_out]
    int ld_out = 0;
    const float *bias = nullptr;   // forward only
    int out_prefilled = 0;         // forward: out already holds bias/zero, accumulate with atomics (split-K)
    int out_assign = 0;            // backward, member 0: out is overwritten ("dX ="); honoured with plain stores when
                                   // splits == 1, otherwise the caller must have cleared out
    // fused LoRA rank-update (optional)
    const float *lora_act = nullptr;    // fp32 [T, R]: X*A (forward) or dY*B^T (backward)
    float lora_scale = 1.f;             // alpha / r, applied when the tile is rounded to 16 bits
    const float *lora_w = nullptr;      // forward: B [R, N]; backward: A [K, R]
    int rank = 0;
    const int *lora_flag = nullptr;     // device int: 0 -> skip the update
    int splits = 1;
    int *status = nullptr;              // device int[4]
    void *trace = nullptr;              // optional device int64[12*128] timeline buffer
    // a window of the weight's rows [row_base, row_base + rows) instead of all of them (rows == 0: the whole tensor):
    // the vocabulary tiles of the LM head.  `out` / `act16` then belong to the window (column 0 = row row_base).
    int row_base = 0, rows = 0;
};
int umma_pick_splits(const WeightDev *w, int backward, int T, int sm_count);
// Returns cudaSuccess or an error; `err` receives a description on failure of a non-CUDA kind.
cudaError_t launch_umma_gemm(const UmmaLaunch &L, cudaStream_t s, const char **err);
// The few-token kernel (gt_umma_few.cu): up to 128 tokens, one member per launch, no fused adapter term.
bool umma_few_ok(const UmmaLaunch &L);
// launch_umma_group will serve these members with the few-token kernel; their adapter terms then follow on kernels that
// update the output with plain read-modify-writes, so such a launch must not run beside another one into the same output
bool umma_group_few(const UmmaLaunch *m, int n);
void umma_few_shape(const UmmaLaunch &L, int *tiles, int *units);
cudaError_t launch_umma_few(const UmmaLaunch &L, cudaStream_t s, const char **err);
bool tmap_encode_2d(CUtensorMap *tm, CUtensorMapDataType dt, const void *base, uint64_t d0, uint64_t d1, uint64_t stride1_bytes,
                    uint32_t b0, uint32_t b1, CUtensorMapSwizzle swz);
// Up to three projections in one launch (see gt_umma_gemm.cu); umma_group_ok tells whether they qualify.
bool umma_group_ok(const UmmaLaunch *m, int n);
int umma_group_splits(const UmmaLaunch *m, int n, int sm_count);
// dual forward (gate | up, SwiGLU product in the epilogue): see umma_dual_ok
struct UmmaDual {
    void *h16 = nullptr;      // 16-bit [T, ld_h16] in the launch's operand format, or null
    int ld_h16 = 0;
};
bool umma_dual_ok(const UmmaLaunch *m, int sm_count);
cudaError_t launch_umma_group(const UmmaLaunch *m, int n, cudaStream_t s, const char **err, const UmmaDual *dual = nullptr);
cudaError_t umma_init_weight_maps(WeightDev *w, const char **err);
bool umma_available();
cudaError_t launch_bounded_wait_selftest(int *status, long long limit_cycles, cudaStream_t s);


// ---- views of the opaque C-ABI handles for translation units outside gt_engine.cu ---------------------------
struct EngineView {
    int device;
    int math_mode;
    int sm_count;
    cudaStream_t stream;
    int *status;       // device int[4], bounded-wait codes of the tensor-core kernels
    void *mutex;       // std::mutex * serialising calls on the engine
};
// ---- weight-streaming forward projection for few tokens (gt_stream_gemm.cu): warp-level MMAs on the quantized
// integers, scales applied per sub-block on the partial sums.  Q4_K, whole 256-wide rows, T <= stream_max_tokens().
int stream_max_tokens();
bool stream_fwd_ok(const WeightDev *w, int T);
cudaError_t launch_stream_fwd(const WeightDev *w, const float *X, float *Y_prefilled, int T, int sm_count, int *status, void *trace,
                              cudaStream_t s);

// ---- layer glue launchers used inside the library (gt_glue.cu)
cudaError_t launch_swiglu_fwd(const float *gate, const float *up, float *hidden, int64_t n, int sm_count, cudaStream_t s);
// hidden = SiLU(gate) * up written as fp32 (hidden, may be null) and as 16-bit (h16: bf16, or fp16 when fp16 != 0) in one
// pass; n % 4 == 0 and 16-byte-aligned pointers
cudaError_t launch_swiglu_fwd16(const float *gate, const float *up, float *hidden_or_null, void *h16, int64_t n, int fp16, int sm_count,
                                cudaStream_t s);
// dGate, dUp as bf16 only (the operands of the gate,up transpose GEMM); n % 4 == 0, 16-byte-aligned inputs
cudaError_t launch_swiglu_bwd16(const float *d_hidden, const float *gate, const float *up, void *d_gate16, void *d_up16, int64_t n, int sm_count,
                                cudaStream_t s);
// one flat segment of an AdamW launch: parameters, gradients and both moments, n elements; flag (optional) is set to 1
// when a parameter of the segment is non-zero after the step (vec is filled in by the launcher)
struct AdamwSeg {
    float *p;
    const float *g;
    float *m, *v;
    int *flag;
    int64_t n;
    int vec;
};
constexpr int kAdamwSegs = 32;      // segments per launch (16 adapters)
cudaError_t launch_adamw(const AdamwSeg *segs, int n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                         int sm_count, cudaStream_t s);
cudaError_t launch_swiglu_bwd(const float *d_hidden, const float *gate, const float *up, float *d_gate, float *d_up, int64_t n, int sm_count,
                              cudaStream_t s);

cudaError_t launch_add(const float *a, const float *b, float *out, int64_t n, int sm_count, cudaStream_t s);
cudaError_t launch_rope(float *q, float *k, int T, int heads_q, int heads_kv, int head_dim, float freq_base, float freq_scale, int rope_dim,
                        int inverse, cudaStream_t s);
cudaError_t launch_rmsnorm_fwd(const float *x, const float *w, float *y, int T, int H, float eps, cudaStream_t s);
// dx = RMSNorm backward (+ residual, which may be null and may alias dx)
cudaError_t launch_rmsnorm_bwd(const float *dy, const float *x, const float *w, const float *residual, float *dx, int T, int H, float eps,
                               cudaStream_t s);
// sum = a + b (sum may alias a or b), y = RMSNorm(sum) * w
cudaError_t launch_add_rmsnorm_fwd(const float *a, const float *b, const float *w, float *sum, float *y, int T, int H, float eps, cudaStream_t s);

// ---- launches with programmatic dependent launch (the kernel must call pdl_wait() before touching global memory).
// On by default; environment GT_PDL=0 launches in plain stream order.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace gt
struct gt_engine;
struct gt_weight;
namespace gt {
EngineView engine_view(gt_engine *e);
const WeightDev *weight_view(const gt_weight *w);
int set_last_error(int code, const char *text);     // records the text for gt_last_error(), returns code
int engine_join_comm(gt_engine *e);                 // engine stream waits for gradient exchanges begun on the side stream (lock held)
}  // namespace gt
