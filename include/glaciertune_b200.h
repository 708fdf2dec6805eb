/*
 * glaciertune_b200.h — C ABI of libglaciertune_b200.so
 *
 * A B200 (sm_100a) replacement for the CUDA backend of Glacier.Tune's frozen-base projection path:
 *   forward   Y  = X * W^T (+ bias) + (alpha/r) * (X * A) * B
 *   backward  dX += dY * W + (alpha/r) * (dY * B^T) * A^T ;  dA += ... ;  dB += ...
 * with W a GGUF K-quant tensor (Q4_K, Q6_K) or F32, row-major [out, in], super-blocks along `in`.
 *
 * Conventions
 *   - every function returns 0 on success or a negative gt_status; gt_last_error() gives the text of
 *     the calling thread's last failure.  Nothing throws, nothing calls back.
 *   - plain pointers and integer sizes only.  Activation pointers are HOST pointers unless the call is
 *     given GT_FLAG_DEVICE_PTRS, in which case they are device pointers on the engine's device and the
 *     call only enqueues work on the engine's stream.
 *   - host-pointer calls are complete on return (the reference engine is synchronous:
 *     src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:29-47).
 *   - an engine serialises its calls internally; it may be used from several host threads
 *     (the reference takes one lock per call: src/Glacier.Tune/Gpu/GpuLoraEngine.cs:54).
 *   - LoRA factors use the reference's storage: A is [in, rank] row-major, B is [rank, out] row-major
 *     (src/Glacier.Tune/Model/LoraAdapter.cs:25-26).  All activations and gradients are fp32 row-major.
 *   - there is no CPU fallback: without a usable sm_100 device gt_engine_create fails.
 *
 * "Replaces" comments cite the reference member each entry point stands in for
 * (paths relative to the reference project root).
 */
#ifndef GLACIERTUNE_B200_H
#define GLACIERTUNE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GT_API __attribute__((visibility("default")))
#else
#define GT_API
#endif

typedef struct gt_engine gt_engine;
typedef struct gt_weight gt_weight;
typedef struct gt_adapter gt_adapter;
typedef struct gt_model gt_model;

/* ggml tensor type ids, as in the reference's GgufType */
enum { GT_TYPE_F32 = 0, GT_TYPE_F16 = 1, GT_TYPE_Q4_0 = 2, GT_TYPE_Q8_0 = 8, GT_TYPE_Q4_K = 12, GT_TYPE_Q6_K = 14 };

enum gt_status {
    GT_OK = 0,
    GT_ERR_INVALID = -1,     /* bad argument (null pointer, size mismatch, in % 256 != 0, ...) */
    GT_ERR_UNSUPPORTED = -2, /* tensor type / shape outside what the kernels handle */
    GT_ERR_CUDA = -3,        /* a CUDA call failed; text in gt_last_error() */
    GT_ERR_NO_DEVICE = -4,   /* no sm_100 device */
    GT_ERR_KERNEL = -5,      /* a kernel reported a bounded-wait timeout or a self-check failure */
    GT_ERR_NCCL = -6,
    GT_ERR_OOM = -7
};

/* arithmetic of the base GEMMs */
enum gt_math_mode {
    GT_MATH_BF16 = 0, /* tcgen05 MMA, bf16 operands, fp32 accumulation (default) */
    GT_MATH_FP16 = 1, /* tcgen05 MMA, fp16 operands rounded once from the exact fp32 weight: validation mode */
    GT_MATH_FP32 = 2  /* CUDA-core fp32 FMA on exactly dequantized weights: validation mode */
};

enum gt_direction { GT_DIR_FORWARD = 0, GT_DIR_BACKWARD = 1 };

enum gt_flags {
    GT_FLAG_DEVICE_PTRS = 1, /* activation pointers are device pointers; asynchronous on the engine stream */
    GT_FLAG_NO_LORA = 2,     /* skip the adapter terms even when an adapter is given */
    GT_FLAG_REUSE_LOW = 4,   /* backward: X is the tensor the last forward through this adapter saw, so X*A kept from
                                that call is reused instead of recomputed (the reference recomputes it,
                                src/Glacier.Tune/Kernels/LoraKernels.cs:147-186; the value is the same).  With host
                                buffers the device copy of X staged by that forward is reused as well (X is not
                                uploaded a second time; the adapter holds T x in_features floats for it) */
    GT_FLAG_HOST_ASYNC = 16, /* host buffers only, page-locked: the call returns once its copies and kernels are queued
                                (uploads, kernels and downloads of consecutive calls overlap on separate streams); the
                                outputs are valid, and the inputs may be changed, after gt_sync().  Without the flag a
                                host-buffer call returns with its outputs written, like the reference's */
    GT_FLAG_DX_ASSIGN = 8    /* backward: dX = ... instead of dX += ...: the call clears dX itself, which replaces the
                                zero-filled buffer the reference hands to LoraAdapter.Backward
                                (AutogradScratchWorkspace.Wrap) without a separate fill */
};

typedef struct gt_config {
    int32_t device;       /* CUDA device ordinal                                              */
    int32_t math_mode;    /* gt_math_mode                                                     */
    void *stream;         /* cudaStream_t to run on, or NULL: the engine creates its own      */
    int32_t max_tokens;   /* with max_features: engine scratch (16-bit operand copies, FFN intermediates) and every
                             adapter's per-step scratch are allocated for this many tokens at creation, so that no later
                             projection call up to that size allocates; 0: allocate (and grow) on demand, as the
                             reference does (src/Glacier.Tune/Gpu/GpuLoraEngine.Memory.cs:7-114)        */
    int32_t max_features; /* largest in/out feature count of a projection, a group's outputs counted together
                             (q|k|v, gate|up: 2 x 18944 for the 7B layer); 0: nothing reserved up front      */
} gt_config;

/* Log callback (the reference logs through GlacierDiagnostics, e.g. src/Glacier.Tune/Gpu/GpuLoraEngine.cs:251,320 and
 * the CPU-fallback warning at src/Glacier.Tune/Model/GgufLoraModel.cs:76-80).  The library calls it, from the calling
 * thread, with every error text it records and with informational messages (uploads, reserved scratch); without a
 * callback it is silent.  Process-wide. */
enum gt_log_level { GT_LOG_DEBUG = 0, GT_LOG_INFO = 1, GT_LOG_ERROR = 2 };
typedef void (*gt_log_fn)(int level, const char *message, void *user);
GT_API int gt_set_logger(gt_log_fn fn_or_null, void *user);

GT_API const char *gt_last_error(void);
GT_API const char *gt_version(void);

/* Replaces: new GpuLoraEngine(weights, deviceOrdinal) / Dispose()
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.cs:114-218,335-383).  Weight upload is a separate call. */
GT_API int gt_engine_create(const gt_config *cfg, gt_engine **out);
GT_API int gt_engine_destroy(gt_engine *eng);
GT_API int gt_engine_set_math_mode(gt_engine *eng, int math_mode);
/* Wait for everything queued on the engine's stream; reports bounded-wait timeouts of the kernels. */
GT_API int gt_sync(gt_engine *eng);

/* Replaces: SupportsForwardGemm / SupportsBackwardGemm
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:13-14, GpuLoraEngine.Backward.cs:12-13).  Returns 1 or 0.
 * Q4_K and Q6_K run on the tensor cores; F32, F16, Q4_0 and Q8_0 projections (the reference's other types: gemm_q4_0_batch,
 * gemm_q8_0_bwd, gemm_q4_0_bwd, src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:131-190,335-460) run on the exact fp32 CUDA-core
 * kernels in every math mode (F16 tensors are meant for the embedding and the LM head, whose calls below use the tensor
 * cores). */
GT_API int gt_supports(int ggml_type, int direction);

/* Replaces: UploadBaseWeights (src/Glacier.Tune/Gpu/GpuLoraEngine.cs:240-321) for one tensor, and the
 * Get{Q,K,V,AttnOut,Gate,Up,Down}/Get*Bias handles (GpuLoraEngine.cs:323-333).
 * host_bytes is the GGUF tensor data ([out, in] row-major, nbytes = out*in/256 * block size, or out*in*4
 * for F32).  The bytes are copied; Q6_K is re-laid out on the device in 16-byte-aligned blocks with
 * identical dequantized values.  bias may be NULL. */
GT_API int gt_weight_upload(gt_engine *eng, int ggml_type, const void *host_bytes, int64_t nbytes,
                            int32_t out_features, int32_t in_features, const float *bias_or_null,
                            gt_weight **out);
GT_API int gt_weight_free(gt_weight *w);

/* Replaces: the role of QuantKernels.ExtractEmbedding(type, W, row, dst, K) on the uploaded copy
 * (call sites src/Glacier.Tune/Kernels/LoraKernels.BaseBackward.cs:117,125): dequantize rows
 * [row0, row0+nrows) to fp32, bit-exact with the reference decode
 * (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:209-211,234-240,279-289,311-315).  `out` follows `flags`. */
GT_API int gt_dequant_rows(gt_engine *eng, const gt_weight *w, int64_t row0, int64_t nrows, float *out,
                           int32_t flags);

/* Replaces: the LoraAdapter state that the reference keeps on the host
 * (src/Glacier.Tune/Model/LoraAdapter.cs:88-125): A, B and their gradient accumulators, on the device. */
GT_API int gt_adapter_create(gt_engine *eng, int32_t in_features, int32_t out_features, int32_t rank, float alpha,
                             gt_adapter **out);
GT_API int gt_adapter_free(gt_adapter *ad);
GT_API int gt_adapter_upload(gt_adapter *ad, const float *A_in_by_rank, const float *B_rank_by_out);
GT_API int gt_adapter_download(gt_adapter *ad, float *A_in_by_rank, float *B_rank_by_out);
GT_API int gt_adapter_grads_download(gt_adapter *ad, float *dA_in_by_rank, float *dB_rank_by_out);
GT_API int gt_adapter_grads_zero(gt_adapter *ad);
/* Replaces: LoraAdapter.UpdateAlpha (src/Glacier.Tune/Model/LoraAdapter.cs:74-77). */
GT_API int gt_adapter_set_alpha(gt_adapter *ad, float alpha);
/* Device addresses of A, B, dA, dB (fp32) for a resident optimizer or a gradient all-reduce (any of the four may be
 * NULL).  Asking for B raises the adapter's "B may be non-zero" flag, because the library can no longer know when B
 * leaves its all-zero initial state (LoraAdapter.IsZeroDelta, src/Glacier.Tune/Model/LoraAdapter.cs:48-72): from then
 * on every forward evaluates the adapter term.  A caller that writes A or B through these pointers calls
 * gt_adapter_params_changed afterwards. */
GT_API int gt_adapter_device_ptrs(gt_adapter *ad, float **A, float **B, float **dA, float **dB);
/* Replaces: the scan of B inside LoraAdapter.IsZeroDelta (src/Glacier.Tune/Model/LoraAdapter.cs:48-72), which the
 * reference repeats on the host at every forward; here the answer is cached in a device flag.  This call tells the
 * library that A or B changed behind its back (written through the device pointers): the flag is recomputed from the
 * values on the engine stream and X*A kept from an earlier forward is dropped.  Not needed after gt_adapter_upload or
 * the library's own AdamW steps. */
GT_API int gt_adapter_params_changed(gt_adapter *ad);
/* Point the adapter's gradient accumulators into a caller-owned device buffer (one flat allocation per
 * model in the reference's parameter order, src/Glacier.Tune/Model/TransformerBlock.cs:167-174). */
GT_API int gt_adapter_bind_grads(gt_adapter *ad, float *dA_dev, float *dB_dev);

/* Replaces: LoraAdapter.Forward -> GpuLoraEngine.ForwardProjection + LoraKernels.ApplyLoraDelta
 * (src/Glacier.Tune/Model/LoraAdapter.cs:128-184, src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:16-48,
 *  src/Glacier.Tune/Kernels/LoraKernels.cs:18-122).
 * Y[T,out] = X[T,in] * W^T + bias + scaling*(X*A)*B.  The adapter term is skipped when adapter is NULL,
 * GT_FLAG_NO_LORA is set, or B is entirely zero (LoraAdapter.IsZeroDelta, LoraAdapter.cs:48-72). */
GT_API int gt_proj_forward(gt_engine *eng, const gt_weight *w, gt_adapter *adapter_or_null, const float *X, float *Y,
                           int32_t T, int32_t flags);

/* Replaces: LoraAdapter.Backward -> GpuLoraEngine.BackwardProjection + LoraKernels.Backward
 * (src/Glacier.Tune/Model/LoraAdapter.cs:190-260, src/Glacier.Tune/Gpu/GpuLoraEngine.Backward.cs:58-92,
 *  src/Glacier.Tune/Kernels/LoraKernels.cs:125-346).
 * dX (may be NULL) is ACCUMULATED into: dX += dY*W + scaling*(dY*B^T)*A^T; the reference hands in a
 * zero-filled buffer (src/Glacier.Tune/Model/AutogradScratchWorkspace.cs:138-145).  The adapter's dA and dB
 * accumulate across calls until gt_adapter_grads_zero. */
GT_API int gt_proj_backward(gt_engine *eng, const gt_weight *w, gt_adapter *adapter_or_null, const float *dY,
                            const float *X, float *dX_accum_or_null, int32_t T, int32_t flags);

/* No counterpart in the reference.  Largest token count for which gt_proj_forward runs the few-token weight-streaming
 * kernel on Q4_K weights instead of the CTA-wide tensor-core kernel (0 = never; environment GT_STREAM_MAX_T, 0..32,
 * read once per process). */
GT_API int gt_stream_max_tokens(void);

/* Replaces: GpuLoraEngine.ForwardQKV and the gate/up half of ForwardFfn
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:205-245,247-364): n (1..3) projections of the SAME input X,
 * Y[j] = X * W_j^T + bias_j + scaling_j*(X*A_j)*B_j.  With device pointers and members of one quantization type the
 * group costs one pass over X and one GEMM launch; otherwise it runs as n gt_proj_forward calls. */
GT_API int gt_proj_forward_group(gt_engine *eng, int32_t n, const gt_weight *const *weights, gt_adapter *const *adapters_or_null,
                                 const float *X, float *const *Y, int32_t T, int32_t flags);
/* Replaces: the q|k|v and gate|up LoraAdapter.Backward calls of a block plus the sum of their input gradients
 * (src/Glacier.Tune/Model/TransformerBlock.cs:660-663,812-816): dX += sum_j (dY[j] * W_j + adapter term j) into ONE
 * buffer (dX may be NULL: gradients of the adapters only); dA_j, dB_j accumulate. */
GT_API int gt_proj_backward_group(gt_engine *eng, int32_t n, const gt_weight *const *weights, gt_adapter *const *adapters_or_null,
                                  const float *const *dY, const float *X, float *dX_accum_or_null, int32_t T, int32_t flags);

/* Replaces: GpuLoraEngine.ForwardFfn(layer, norm2X, outGate?, outUp?, outHidden?, outDown, gateLora, upLora, downLora, seqLen)
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:247-364): gate and up projections of X as one group, hidden =
 * SiLU(gate) * up, out_down = down projection of hidden, the adapters' terms included.  adapters = {gate, up, down}
 * (the array or any entry may be NULL).  out_gate / out_up / out_hidden may be NULL: the tensors then live in engine
 * scratch only.  With host buffers X goes up once and only the outputs that were asked for come back. */
GT_API int gt_ffn_forward(gt_engine *eng, const gt_weight *w_gate, const gt_weight *w_up, const gt_weight *w_down,
                          gt_adapter *const *adapters_or_null, const float *X, float *out_gate_or_null, float *out_up_or_null,
                          float *out_hidden_or_null, float *out_down, int32_t T, int32_t flags);
/* Replaces: the FFN half of TransformerBlock.Backward (src/Glacier.Tune/Model/TransformerBlock.cs:625-666): down.Backward,
 * SwiGluKernel.Backward, gate.Backward and up.Backward into one input gradient.  Device tensors only
 * (GT_FLAG_DEVICE_PTRS): gate, up, hidden are the tensors the forward produced; dX is accumulated into, or written with
 * GT_FLAG_DX_ASSIGN; adapter gradients accumulate. */
GT_API int gt_ffn_backward(gt_engine *eng, const gt_weight *w_gate, const gt_weight *w_up, const gt_weight *w_down,
                           gt_adapter *const *adapters_or_null, const float *dY, const float *X, const float *gate, const float *up,
                           const float *hidden, float *dX, int32_t T, int32_t flags);

/* ---- layer glue on device tensors (asynchronous on the engine stream): what sits between the projections ---- */
/* Replaces: SwiGluKernel.Forward (src/Glacier.Tune/Kernels/SwiGluKernel.cs:13-31): hidden = SiLU(gate) * up, n elements. */
GT_API int gt_swiglu_forward(gt_engine *eng, const float *gate, const float *up, float *hidden, int64_t n);
/* Replaces: SwiGluKernel.Backward (SwiGluKernel.cs:33-60): dUp = dH * SiLU(g), dGate = dH * u * sig * (1 + g (1 - sig));
 * both outputs are assigned. */
GT_API int gt_swiglu_backward(gt_engine *eng, const float *d_hidden, const float *gate, const float *up, float *d_gate, float *d_up,
                              int64_t n);
/* Replaces: RoPEKernel.ForwardSequence / BackwardSequence (src/Glacier.Tune/Kernels/RoPEKernel.cs:12-126) without the
 * ropeFreqs table: q [T, heads_q * head_dim] and k [T, heads_kv * head_dim] rotated in place (either may be NULL),
 * pairs (i, i + rope_dim/2), rope_dim <= 0 means head_dim; inverse != 0 is the backward rotation. */
GT_API int gt_rope(gt_engine *eng, float *q_or_null, float *k_or_null, int32_t T, int32_t heads_q, int32_t heads_kv, int32_t head_dim,
                   float freq_base, float freq_scale, int32_t rope_dim, int32_t inverse);
/* Replaces: ElementwiseKernels.RMSNorm / RMSNormBackward of Glacier.Tensor as called at
 * src/Glacier.Tune/Model/TransformerBlock.cs:318,524,672,827 (frozen weight, dW never computed):
 * y = x * rsqrt(mean(x^2) + eps) * w;  dx = r * (dy * w) - x * r^3 * mean(dy * w * x). */
GT_API int gt_rmsnorm_forward(gt_engine *eng, const float *x, const float *w, float *y, int32_t T, int32_t H, float eps);
GT_API int gt_rmsnorm_backward(gt_engine *eng, const float *dy, const float *x, const float *w, float *dx, int32_t T, int32_t H, float eps);
/* Replaces: TensorOps.Add for the residual connections (TransformerBlock.cs:675): out = a + b (out may alias a or b). */
GT_API int gt_add(gt_engine *eng, const float *a, const float *b, float *out, int64_t n);

/* ---- causal attention with grouped KV heads (device tensors, asynchronous on the engine stream) ------------------ */
/* Replaces: GpuLoraEngine.SupportsAttention(seqLen, headDim) (src/Glacier.Tune/Gpu/GpuLoraEngine.cs:111).  1 or 0. */
GT_API int gt_supports_attention(int32_t T, int32_t head_dim);
/* Replaces: GpuLoraEngine.ForwardAttention (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:433-513, kernel
 * tune_attn_causal_gqa_fwd, src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:527-596) and CausalAttentionKernel.Forward
 * (src/Glacier.Tune/Kernels/CausalAttentionKernel.cs:17-78): out = softmax(q k^T / sqrt(head_dim), causal) v with
 * head h reading KV head h / (heads_q / heads_kv).  q, out: [T, heads_q, head_dim]; k, v: [T, heads_kv, head_dim],
 * fp32, 16-byte aligned; head_dim 128.  Instead of the reference's attnProbs [heads_q, T, T] the call keeps
 * lse [heads_q, T] (base-2 log-sum-exp of the scaled scores) for the backward.  RoPE is not applied here: call
 * gt_rope on q and k first (the reference engine rotates inside ForwardAttention). */
GT_API int gt_attention_forward(gt_engine *eng, const float *q, const float *k, const float *v, float *out, float *lse, int32_t T,
                                int32_t heads_q, int32_t heads_kv, int32_t head_dim);
/* Replaces: GpuLoraEngine.BackwardAttention (src/Glacier.Tune/Gpu/GpuLoraEngine.Backward.cs:354-459, kernels
 * tune_attn_causal_gqa_bwd_dq_ds / _bwd_dk_dv, tune_bwd.cu:598-717) and CausalAttentionKernel.Backward
 * (CausalAttentionKernel.cs:80-213): dq, dk, dv are overwritten (the reference clears them first).  q, k, v, out and
 * lse are the forward's tensors (q and k rotated); the probabilities are recomputed tile by tile, no [heads_q, T, T]
 * buffer exists.  The gradients are those of the rotated q and k: apply gt_rope(..., inverse = 1) to dq and dk next. */
GT_API int gt_attention_backward(gt_engine *eng, const float *d_out, const float *q, const float *k, const float *v, const float *out,
                                 const float *lse, float *dq, float *dk, float *dv, int32_t T, int32_t heads_q, int32_t heads_kv,
                                 int32_t head_dim);

/* ---- LM head: streaming cross-entropy, logits, embedding lookup -------------------------------------------------- */
/* Replaces: FusedCrossEntropyLoss.ComputeLossAndGradients / ComputeLoss
 * (src/Glacier.Tune/Kernels/FusedCrossEntropyLoss.cs:22-168,170-364) with the engine calls they drive,
 * GpuLoraEngine.ComputeTiledLmHeadLoss / ComputeTiledLmHeadLossAndGradients
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Backward.cs:98-352): the loss of the LM head over `hidden` [T, in] against
 * `labels` [T] (int32; a label outside [0, vocab) is ignored, as -100 is), mean over the valid tokens, and - when
 * d_hidden is not NULL - its gradient with respect to hidden, [T, in] (zero rows for ignored tokens).  The vocabulary
 * is walked in tiles with an online log-sum-exp on the device; the [T, vocab] logits are never formed and nothing
 * visits the host.  lm_head is an F16 tensor [vocab, in] (in % 128 == 0); the GEMMs run with fp16 operands and fp32
 * accumulation in every math mode.  valid_out (may be NULL) receives the number of valid tokens.
 * With GT_FLAG_DEVICE_PTRS hidden, labels, loss_out (one float), valid_out (one int32) and d_hidden are device
 * pointers and the call only queues work; otherwise all five are host pointers and the call is complete on return. */
GT_API int gt_lm_head_loss(gt_engine *eng, const gt_weight *lm_head, const float *hidden, const int32_t *labels, int32_t T,
                           float *loss_out, int32_t *valid_out_or_null, float *d_hidden_or_null, int32_t flags);
/* Replaces: GpuLoraEngine.ComputeLmHeadLogits (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:50-81): the full
 * logits[T, vocab] = hidden * W^T for evaluation.  Device tensors (GT_FLAG_DEVICE_PTRS), vocab % 4 == 0. */
GT_API int gt_lm_head_logits(gt_engine *eng, const gt_weight *lm_head, const float *hidden, float *logits, int32_t T, int32_t flags);
/* Replaces: the embedding loop of GgufLoraModel.ForwardLossAndBackward, QuantKernels.ExtractEmbedding per token
 * (src/Glacier.Tune/Model/GgufLoraModel.cs:456-462): out[t, :] = fp32 row tokens[t] of the embedding tensor (any
 * uploaded type).  A token outside [0, vocab) is an error on the host-pointer path (the reference throws,
 * GgufLoraModel.cs:443-452) and yields a zero row on the device-pointer path. */
GT_API int gt_embedding_forward(gt_engine *eng, const gt_weight *embedding, const int32_t *tokens, int32_t T, float *out, int32_t flags);

/* Replaces: GpuLoraEngine.LaunchGemmBatch(type, dY, dX, dW, kCols, mRows, batch, dBias, dResidual)
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:83-129): device pointers, asynchronous.
 * Y (may be NULL) = X*W^T + bias; residual (may be NULL) += X*W^T + bias, as the reference kernels do
 * (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:118-124). */
GT_API int gt_launch_gemm_batch(gt_engine *eng, const gt_weight *w, float *dY_out, const float *dX_in, int32_t batch,
                                float *d_residual_or_null);
/* Replaces: GpuLoraEngine.LaunchGemmBwd(type, dDX, dDY, dW, kCols, mRows, batch)
 * (src/Glacier.Tune/Gpu/GpuLoraEngine.Backward.cs:15-56): dDX[batch,in] += dDY[batch,out] * W. */
GT_API int gt_launch_gemm_bwd(gt_engine *eng, const gt_weight *w, float *dDX_accum, const float *dDY, int32_t batch);

/* No counterpart in the reference (its engine allocates and grows device scratch on demand,
 * src/Glacier.Tune/Gpu/GpuLoraEngine.Memory.cs:7-114).  Same result as gt_launch_gemm_bwd - dDX[batch,in] +=
 * dDY[batch,out] * W on device pointers, asynchronous on the engine stream - for hosts that may not allocate
 * device memory when they call: inside a stream capture, in a loop that cannot afford cudaMalloc's device-wide
 * synchronisation, or after all memory has been handed to a pool.  The 16-bit copy of dDY that the tensor-core
 * kernel reads lives in a fixed 4 MiB array inside the library image (held by every GPU that loads the library)
 * instead of the engine's grow-only buffer, and the call performs no allocation of any kind.
 *   - batch * round_up(out, 8) must be <= 2,097,152 elements, else GT_ERR_UNSUPPORTED and nothing is launched;
 *   - tensor-core math modes and K-quant weights with in % 256 == 0 only (GT_ERR_UNSUPPORTED otherwise);
 *   - the first call on a device looks up the array's device address: make that call before any stream capture;
 *   - all calls share the array (it keeps the previous call's contents; every element read is rewritten first, so
 *     nothing needs clearing); calls whose GPU work overlaps on one device race on it - serialise them. */
GT_API int gt_launch_gemm_bwd_static(gt_engine *eng, const gt_weight *w, float *dDX_accum, const float *dDY, int32_t batch);

/* Replaces: LoraTrainer.ScaleAccumulatedGradients / ClipGradients
 * (src/Glacier.Tune/Trainer/LoraTrainer.cs:352-377,395-433) on a flat device gradient buffer:
 * g *= pre_scale; norm = sqrt(sum g^2) in fp64; non-finite -> g = 0, *norm_out = 0; norm > max_norm ->
 * g *= max_norm/(norm+1e-6).  norm_out is a host pointer; the call is complete on return. */
GT_API int gt_grads_scale_clip(gt_engine *eng, float *g_dev, int64_t n, float pre_scale, double max_norm,
                               double *norm_out);

/* Replaces: the optimizer step of the trainer - `new AdamW(params, lr, beta1, beta2, eps, weightDecay)`, `.Step()`
 * (src/Glacier.Tune/Trainer/LoraTrainer.cs:56-62,230; AdamW itself is in Glacier.Tensor 1.1.0, not in the
 * repository: textbook decoupled weight decay, parity unpinned against the reference, pinned against
 * torch.optim.AdamW by the tests).  `step` counts from 1 and selects the bias corrections:
 *   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p *= 1 - lr wd;  p -= lr (m/(1-b1^t)) / (sqrt(v/(1-b2^t)) + eps)
 * gt_adamw_step works on flat device buffers (p, m, v updated in place; m and v start as zeros).
 * gt_adapter_adamw_step updates an adapter's A and B from its gradient accumulators (wherever they are bound) in one
 * launch and keeps both moments inside the adapter (zero before its first step); the learning-rate schedule stays
 * with the caller.  gt_adapters_adamw_step does the same for n adapters of one engine, sixteen adapters per launch
 * (the 196 adapters of a 28-layer model: 13 launches).  All three are asynchronous on the engine stream. */
GT_API int gt_adamw_step(gt_engine *eng, float *p_dev, const float *g_dev, float *m_dev, float *v_dev, int64_t n, float lr, float beta1,
                         float beta2, float eps, float weight_decay, int32_t step);
GT_API int gt_adapter_adamw_step(gt_adapter *ad, float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step);
GT_API int gt_adapters_adamw_step(gt_engine *eng, int32_t n, gt_adapter *const *adapters, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, int32_t step);

/* ---- the training step of a whole model, device resident -------------------------------------------------------- */
typedef struct gt_model_config {
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;
    float rms_eps;        /* RMSNorm epsilon (ModelWeights.RmsNormEps)                                           */
    float rope_theta;     /* RoPE frequency base (rope_freq_base)                                                 */
    int32_t max_tokens;   /* longest sequence a step may carry; every activation buffer is allocated for it       */
    int32_t checkpoint;   /* != 0: activation checkpointing - keep only the block inputs, recompute in the backward */
    int32_t no_graph;     /* != 0: gt_model_forward_backward always launches its kernels one by one (see there)    */
    int32_t reserved[3];
} gt_model_config;

/* Replaces: the construction of GgufLoraModel's layer list (src/Glacier.Tune/Model/GgufLoraModel.cs:60-130) for the
 * step driver below.  Allocates every activation buffer of a step once (nothing is allocated per step).  The weights
 * and adapters are the caller's handles; the model only refers to them. */
GT_API int gt_model_create(gt_engine *eng, const gt_model_config *cfg, gt_model **out);
GT_API int gt_model_destroy(gt_model *m);
/* weights / adapters: seven entries in the reference's order q, k, v, o, gate, up, down
 * (src/Glacier.Tune/Model/TransformerBlock.cs:149-165); adapter entries (or the array) may be NULL.  attn_norm and
 * ffn_norm are host arrays [hidden] (ModelWeights.AttnNormWeight / FfnNormWeight).  q/k/v biases ride in their weights. */
GT_API int gt_model_set_block(gt_model *m, int32_t layer, const gt_weight *const *weights, gt_adapter *const *adapters_or_null,
                              const float *attn_norm, const float *ffn_norm);
/* embedding [vocab, hidden] (any uploaded type), out_norm host [hidden], lm_head F16 [vocab, hidden]. */
GT_API int gt_model_set_head(gt_model *m, const gt_weight *embedding, const float *out_norm, const gt_weight *lm_head);
/* Binds the gradient accumulators of every adapter into ONE flat device buffer in the reference's parameter order
 * (layer -> q, k, v, o, gate, up, down -> A, B; TransformerBlock.cs:167-174) - what the data-parallel all-reduce, the
 * clip and the optimizer step run over.  Call after every block is set; returns the buffer and its length. */
GT_API int gt_model_bind_grads(gt_model *m, float **grads_dev_or_null, int64_t *count_or_null);
/* Replaces: GgufLoraModel.ComputeLoss (src/Glacier.Tune/Model/GgufLoraModel.cs:370-426): forward only, mean
 * cross-entropy over the valid labels.  tokens, labels: int32 [T]. */
GT_API int gt_model_loss(gt_model *m, const int32_t *tokens, const int32_t *labels, int32_t T, float *loss_out, int32_t *valid_out_or_null,
                         int32_t flags);
/* Replaces: GgufLoraModel.ForwardLossAndBackward(inputTokens, targetTokens, checkpointActivations)
 * (src/Glacier.Tune/Model/GgufLoraModel.cs:428-557) with TransformerBlock.Forward / Backward
 * (src/Glacier.Tune/Model/TransformerBlock.cs:307-595,625-840): embedding, the blocks, final RMSNorm, streaming
 * cross-entropy, and the reverse pass; the adapters' gradients ACCUMULATE.  With a data-parallel communicator on the
 * engine (gt_dp_init) and a bound gradient buffer, each block's gradients are all-reduced (averaged over the ranks) on
 * the side stream as soon as its backward is queued, last block first.
 * Host pointers (default): tokens / labels are host arrays and the call returns the loss (complete on return; an input
 * token outside the vocabulary is GT_ERR_INVALID as the reference throws).  GT_FLAG_DEVICE_PTRS: tokens, labels and
 * loss_out (one float, may be NULL) are device pointers and the call only queues work.
 * The device work of a step is the same every time, so from the third call with one token count on it is replayed from a
 * CUDA graph captured during the second (one launch on the host instead of ~1400, no launch gaps between the short
 * kernels); the graph is dropped when a buffer it points at moves (a scratch buffer grows, gt_model_set_*,
 * gt_model_bind_grads, gt_dp_init / gt_dp_finalize, another math mode) and is not used while gt_profile_enable or
 * gt_debug_set_trace is on, with gt_model_config.no_graph, or with GT_STEP_GRAPH=0 in the environment. */
GT_API int gt_model_forward_backward(gt_model *m, const int32_t *tokens, const int32_t *labels, int32_t T, float *loss_out, int32_t flags);
/* State of the captured step (no counterpart in the reference, whose step is a host loop): whether a graph stands ready
 * for the next call, how many calls have been replays so far, and how many kernels one replay launches.  Any pointer
 * may be NULL. */
GT_API int gt_model_step_info(gt_model *m, int32_t *graph_ready, int64_t *replays, int64_t *kernels_per_replay);
/* Replaces: the tail of a training step in LoraTrainer (src/Glacier.Tune/Trainer/LoraTrainer.cs:217-231):
 * ScaleAccumulatedGradients(grad_scale) -> ClipGradients(max_norm; <= 0: no clipping) -> AdamW step on every adapter
 * -> ZeroGrad, all on the device over the flat gradient buffer, after every pending gradient exchange.  `step` counts
 * from 1.  norm_out (may be NULL) receives the pre-clip global norm and makes the call synchronous; without it the
 * call only queues work. */
GT_API int gt_model_optimizer_step(gt_model *m, float lr, float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                                   double max_norm, int32_t step, double *norm_out_or_null);

/* Profiling (the reference only has Stopwatch breakdowns at Debug level,
 * src/Glacier.Tune/Model/TransformerBlock.cs:311-312,582-586).  While enabled, every tensor-core GEMM launch is
 * bracketed by CUDA events on the engine stream.  gt_profile_read synchronises and returns the summed GEMM time,
 * the number of GEMM launches, their base-term FLOPs (2*T*out*in each) and the number of kernels launched by
 * the projection calls since the last reset. */
GT_API int gt_profile_enable(gt_engine *eng, int on);
GT_API int gt_profile_read(gt_engine *eng, double *gemm_ms, int64_t *gemm_launches, double *gemm_flops,
                           int64_t *kernel_launches, int reset);

/* Failure-path self-test (no counterpart in the reference): launches a one-block kernel whose only wait can never
 * be satisfied, with a limit of `limit_cycles` SM clocks.  The wait gives up, records code 999 and the kernel
 * returns; the call then reports GT_ERR_KERNEL the way a timed-out GEMM would.  The device is not faulted or hung. */
GT_API int gt_debug_wait_selftest(gt_engine *eng, int64_t limit_cycles);

/* Kernel timeline for tuning: while dev_buf (device, 12*128 int64, or NULL to stop) is set, the first CTA of every
 * tensor-core GEMM launch writes SM-clock stamps of its pipeline events into it (rows: 0 weight-block loads issued,
 * 1 activation loads issued, 2-4 / 5-7 dequant group 0 / 1 (blocks arrived, slot free, tile published), 8 MMA
 * operands ready, 9 MMAs issued, 11 start / accumulator ready / end).  No counterpart in the reference. */
GT_API int gt_debug_set_trace(gt_engine *eng, void *dev_buf);

/* Data parallel step driver (no counterpart in the reference, which is single-GPU: one GpuContext,
 * src/Glacier.Tune/Gpu/GpuLoraEngine.cs:114-130).  One process per GPU; each holds a replica of the frozen
 * base and the adapters and processes its own sequences; the flat fp32 LoRA-gradient buffer is summed with
 * one NCCL all-reduce on the engine stream, then scaled (1/world reproduces the reference's gradient-accumulation
 * averaging, src/Glacier.Tune/Trainer/LoraTrainer.cs:217-220).  Rank 0 creates the 128-byte id and hands it
 * to the other ranks out of band. */
GT_API int gt_dp_unique_id(void *out_id, int32_t nbytes);
GT_API int gt_dp_init(gt_engine *eng, int32_t world, int32_t rank, const void *unique_id, int32_t nbytes);
GT_API int gt_dp_allreduce(gt_engine *eng, float *g_dev, int64_t count, float scale);
/* Overlapped form for per-bucket exchange (a layer's or a projection group's gradients as soon as its backward has
 * produced them): _begin queues the all-reduce of one slice on a side stream that starts after the work queued on the
 * engine stream so far, so that the backward kernels queued afterwards run beside it; _end makes the engine stream wait
 * for every slice begun (gt_sync and gt_dp_allreduce do so too).  Every rank must begin the same slices in the same
 * order.  Works inside a stream capture of the engine stream when _end is called before the capture ends. */
GT_API int gt_dp_allreduce_begin(gt_engine *eng, float *g_dev, int64_t count, float scale);
GT_API int gt_dp_allreduce_end(gt_engine *eng);
GT_API int gt_dp_finalize(gt_engine *eng);

#ifdef __cplusplus
}
#endif
#endif /* GLACIERTUNE_B200_H */
