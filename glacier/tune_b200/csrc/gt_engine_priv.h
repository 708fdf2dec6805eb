// Private definitions shared by the translation units that implement the C ABI (gt_engine.cu, gt_lmhead.cu,
// gt_attention.cu, gt_model.cu): the opaque handle types, the grow-only scratch buffer, error helpers, and the
// device-pointer forms of the projection calls (engine lock held by the caller).
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>

#include "../../../include/glaciertune_b200.h"
#include "gt_internal.h"
#include "gt_quant.cuh"

namespace gt {
// records the text for gt_last_error() (per thread), passes it to the logger, and returns `code`
int failf(int code, const char *fmt, ...);
// message to the callback installed with gt_set_logger (nothing when none is installed)
void logf(int level, const char *fmt, ...);
}  // namespace gt

#define GT_CUDA(call)                                                                                        \
    do {                                                                                                     \
        cudaError_t _e = (call);                                                                             \
        if (_e != cudaSuccess) return gt::failf(GT_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_e)); \
    } while (0)

#define GT_LAUNCH(eng, call)         \
    do {                             \
        GT_CUDA(call);               \
        (eng)->kernel_launches += 1; \
    } while (0)

namespace gt {
// grow-only device buffer (the reference engine grows its scratch x2 on demand and never shrinks:
// src/Glacier.Tune/Gpu/GpuLoraEngine.Memory.cs:7-114)
// Counts every event that moves a device buffer the library's kernels are pointed at (a scratch buffer that grew, an
// adapter whose gradient accumulators were rebound): a captured CUDA graph of a step is only replayed while the
// count it was captured under still stands.
inline std::atomic<uint64_t> &layout_generation() {
    static std::atomic<uint64_t> g{0};
    return g;
}
struct Scratch {
    void *p = nullptr;
    size_t cap = 0;
    cudaError_t reserve(size_t bytes) {
        if (bytes <= cap) return cudaSuccess;
        layout_generation().fetch_add(1);
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        size_t want = bytes + bytes / 4;
        cudaError_t e = cudaMalloc(&p, want);
        if (e == cudaSuccess) cap = want;
        return e;
    }
    void release() {
        if (p) layout_generation().fetch_add(1);
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
    }
};
}  // namespace gt
using gt::Scratch;

constexpr int kHostSlots = 8;
constexpr int kSlotIn = 4, kSlotOut = 4;      // forward: X -> Y_j; backward: dY_j, X -> dX; FFN: X -> Y, gate, up, hidden
struct HostSlot {
    Scratch in[kSlotIn], out[kSlotOut];
    cudaEvent_t h2d_done = nullptr, compute_done = nullptr, d2h_done = nullptr;
    bool used = false;
};

struct gt_engine {
    int device = 0;
    int max_tokens = 0;          // gt_config.max_tokens: adapters reserve their per-step scratch for it at creation
    int math_mode = GT_MATH_BF16;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    std::mutex mu;
    int *status = nullptr;       // device int[4]; [0] = first bounded-wait timeout code
    double *clip = nullptr;      // device double[2]
    Scratch x16, dy16, dlow, ytmp, pair_tmp;
    Scratch ce, ce_host;         // LM-head cross-entropy: logits / probability tiles and per-token state; host staging
    Scratch attn;                // attention: log-sum-exp rows and the dO.O row sums
    Scratch ffn[3];              // gate, up, hidden (forward) / dHidden, dGate, dUp (backward) of the fused FFN calls
    // Host-buffer calls: a ring of staging slots and two copy streams, so that the upload of one call, the kernels
    // of the previous one and the download of the one before run at the same time (GT_FLAG_HOST_ASYNC), and a
    // synchronous call still overlaps its own download with nothing in its way.
    HostSlot slots[kHostSlots];
    int slot_next = 0;
    cudaStream_t s_h2d = nullptr, s_d2h = nullptr;
    // overlapped gradient exchange: collectives queued on a side stream between a fork and a join of the engine stream
    cudaStream_t s_comm = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // dA = s * X^T * dLow needs only the pass over dY, not the dX GEMM that follows it: it runs on a side stream beside
    // that GEMM (fork after the dY pass, join after the GEMM launch), so its launch gap and tail hide under the GEMM
    cudaStream_t s_aux = nullptr;
    cudaEvent_t ev_aux_fork = nullptr, ev_aux_join = nullptr;
    bool aux_pending = false;
    bool comm_pending = false;
    ncclComm_t comm = nullptr;    // data-parallel communicator (gt_dp_init)
    int dp_world = 1, dp_rank = 0;
    // profiling: CUDA-event pairs around every tensor-core GEMM launch, and a count of kernel launches
    bool profile = false;
    std::vector<cudaEvent_t> ev_pool;
    size_t ev_used = 0;
    double gemm_flops = 0.0;
    int64_t gemm_launches = 0, kernel_launches = 0;
    void *trace = nullptr;       // device timeline buffer handed to the next GEMM launches (gt_debug_set_trace)
    std::vector<gt_model *> models;      // models that may hold a captured step of this engine (see gt_model.cu)
};

struct gt_weight {
    gt_engine *eng = nullptr;
    gt::WeightDev dev;
    // K-quant tensor with in_features % 256 == 128 and an even row count: the same bytes seen as [N / 2, 2 K], whole
    // super-blocks per row, with tensor maps (shares dev.data; owns nothing)
    gt::WeightDev paired;
    bool has_paired = false;
};

struct gt_adapter {
    gt_engine *eng = nullptr;
    int in = 0, out = 0, rank = 0;
    float alpha = 0.f, scaling = 0.f;
    float *A = nullptr, *B = nullptr, *dA = nullptr, *dB = nullptr;
    bool own_grads = true;
    int *b_nonzero = nullptr;    // device flag: any(B != 0), refreshed whenever B is uploaded
    Scratch low;                 // low = X*A of the last forward / backward through this adapter, then dLow = dY*B^T;
                                 // [low_T, rank] fp32 each
    int low_T = 0;
    bool dlow_clean = false;     // dLow is still all zero (cleared together with low, not yet summed into)
    Scratch xkeep;               // host-buffer calls: device copy of the X of the last forward, for a backward that
    int xkeep_T = 0;             // reuses it (GT_FLAG_REUSE_LOW) instead of uploading X again
    Scratch moments;             // AdamW state [mA | vA | mB | vB], allocated and zeroed by the first optimizer step
};


namespace gt {
constexpr int kMaxGroup = 3;
int check_status(gt_engine *e);
bool tensor_path(const gt_engine *e, const gt_weight *w);
// launch (bracketed by events while profiling) on the engine stream, or on `on` when given
cudaError_t timed_umma_group(gt_engine *e, const UmmaLaunch *m, int n, const char **msg, cudaStream_t on = nullptr,
                             const UmmaDual *dual = nullptr);
bool side_da_enabled();
// device-pointer forms of the projection calls; the caller holds the engine lock and has made the device current
// (x16_ready / X16: the input as bf16 [T, K] where the caller has it - bf16 mode, tensor path; the fp32 X may then be null)
int forward_group_device(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *Xd, float *const *Yd,
                         int T, int flags, const void *x16_ready = nullptr, void *dual_h16 = nullptr);
int backward_group_device(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *const *dYd,
                          const float *Xd, float *dXd, int T, int flags, const void *X16 = nullptr, bool dy16_ready = false);
// SiLU(gate) * up can be kept as bf16 only (hidden16: [T, ffn] bf16, hidden_d null) when ffn_hidden16_ok(): the SwiGLU pass
// then writes the down projection's 16-bit operand itself and the adapter products of the down projection read that copy.
bool ffn_hidden16_ok(const gt_engine *e, const gt_weight *const *w, int T);
int ffn_forward_device(gt_engine *e, const gt_weight *const *w, gt_adapter *const *ad, const float *Xd, float *gate_d, float *up_d,
                       float *hidden_d, float *Yd, int T, int flags, void *hidden16 = nullptr);
int ffn_backward_device(gt_engine *e, const gt_weight *const *w, gt_adapter *const *ad, const float *dYd, const float *Xd,
                        const float *gate_d, const float *up_d, const float *hidden_d, float *dXd, int T, int flags,
                        const void *hidden16 = nullptr);
int join_comm(gt_engine *e);
int allreduce_begin_locked(gt_engine *e, float *g_dev, int64_t count, float scale);
// forget the captured step of every model of this engine (before the communicator its collectives belong to goes away)
void drop_step_graphs(gt_engine *e);
// LM head and embedding on device tensors (gt_lmhead.cu); loss_dev / valid_dev are device scalars (may be null)
int lm_head_loss_on_device(gt_engine *e, const gt_weight *w, const float *hidden, const int *labels, int T, float *loss_dev, int *valid_dev,
                           float *d_hidden);
int embedding_on_device(gt_engine *e, const gt_weight *w, const int *tokens, int T, float *out, int *bad_dev);
// causal GQA attention on device tensors (gt_attention.cu); lse: [heads_q, T] fp32 kept for the backward
int attention_forward_on_device(gt_engine *e, const float *q, const float *k, const float *v, float *out, float *lse, int T, int heads_q,
                                int heads_kv, int head_dim);
int attention_backward_on_device(gt_engine *e, const float *d_out, const float *q, const float *k, const float *v, const float *out,
                                 const float *lse, float *dq, float *dk, float *dv, int T, int heads_q, int heads_kv, int head_dim);
}  // namespace gt
