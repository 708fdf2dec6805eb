// LM head on the device: streaming cross-entropy with its input gradient, full logits, and the embedding lookup.
//
// Replaces the host loops of FusedCrossEntropyLoss.ComputeLoss / ComputeLossAndGradients
// (src/Glacier.Tune/Kernels/FusedCrossEntropyLoss.cs:22-168,170-364) and the engine calls they drive,
// GpuLoraEngine.ComputeTiledLmHeadLoss / ComputeTiledLmHeadLossAndGradients / ComputeLmHeadLogits
// (src/Glacier.Tune/Gpu/GpuLoraEngine.Backward.cs:98-352, GpuLoraEngine.Forward.cs:50-81), which compute the tile
// GEMMs on the GPU and bring every logits tile back to the host for max / sum-exp / softmax.
//
// The vocabulary is walked in tiles of about one wave of 128-row CTAs; the [T, vocab] logits never exist.  Per tile:
//   1. logits[T, Vt] = hidden16 * W16[v0 .. v0+Vt)^T        tcgen05 GEMM, fp16 operands, fp32 accumulation
//   2. k_ce_tile (one block per token): running max m and sum s (online log-sum-exp, s in fp64 as the reference),
//      the target's logit, P16 = exp(logits - m_new) in fp16, and - when the maximum moved - the token's row of the
//      gradient accumulator is rescaled by exp(m_old - m_new)
//   3. acc[T, H] += P16 * W16[v0 .. v0+Vt)                  the transpose GEMM of the same kernel
// and at the end  loss = mean over valid tokens of (m + log s - target logit),
//                 dHidden = (acc / s - W[target]) / valid    (zero rows for ignored tokens).
// acc / s = sum_v softmax_v W_v, so this equals the reference's two-pass form (log-sum-exp first, then
// softmax - onehot through AccumulateBaseBackward) without the second logits GEMM.
#include <cuda_fp16.h>

#include "gt_engine_priv.h"

using namespace gt;

namespace {

constexpr int kCeThreads = 256;

__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < kCeThreads / 32; i++) r = fmaxf(r, red[i]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < kCeThreads / 32; i++) r += red[i];
    __syncthreads();
    return r;
}

// per-token state of the online log-sum-exp
struct CeState {
    float *m;        // running maximum
    double *s;       // running sum of exp(logit - m)
    float *tl;       // logit of the target
    int *valid;      // [0] = number of tokens with a label in [0, vocab)
    double *loss;    // [0] = sum over valid tokens of (lse - target logit)
};

__global__ void k_ce_init(CeState st, const int *__restrict__ labels, int T, int vocab) {
    int cnt = 0;
    for (int t = threadIdx.x; t < T; t += blockDim.x) {
        st.m[t] = -INFINITY;
        st.s[t] = 0.0;
        st.tl[t] = 0.f;
        const int y = labels[t];
        cnt += (y >= 0 && y < vocab) ? 1 : 0;
    }
    __shared__ int red[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += red[i];
        st.valid[0] = tot;
        st.loss[0] = 0.0;
    }
}

// One block per token.  logits: [T, ld] fp32, columns [0, n_valid) of this tile are vocabulary ids v0 + column.
__global__ void __launch_bounds__(kCeThreads) k_ce_tile(CeState st, const float *__restrict__ logits, int ld, int n_valid, int v0,
                                                        const int *__restrict__ labels, __half *__restrict__ P16, int ldp,
                                                        float *__restrict__ acc, int H) {
    __shared__ float red[kCeThreads / 32];
    const int t = blockIdx.x;
    const float *row = logits + (int64_t)t * ld;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < n_valid; c += kCeThreads) mx = fmaxf(mx, row[c]);
    mx = block_max(mx, red);
    const float m_old = st.m[t];
    const float m_new = fmaxf(m_old, mx);
    float sum = 0.f;
    __half *prow = P16 ? P16 + (int64_t)t * ldp : nullptr;
    for (int c = threadIdx.x; c < ldp; c += kCeThreads) {
        float p = 0.f;
        if (c < n_valid) {
            p = __expf(row[c] - m_new);
            sum += p;
        }
        if (prow) prow[c] = __float2half_rn(p);
    }
    sum = block_sum(sum, red);
    const float factor = m_old == -INFINITY ? 0.f : __expf(m_old - m_new);
    if (threadIdx.x == 0) {
        st.m[t] = m_new;
        st.s[t] = st.s[t] * (double)factor + (double)sum;
        const int y = labels[t];
        if (y >= v0 && y < v0 + n_valid) st.tl[t] = row[y - v0];
    }
    // the accumulator holds sum_v exp(l_v - m_old) W_v: bring it to the new maximum
    if (acc && factor != 1.f && m_old != -INFINITY) {
        float *a = acc + (int64_t)t * H;
        for (int c = threadIdx.x; c < H; c += kCeThreads) a[c] *= factor;
    }
}

// dH[t, :] = (acc[t, :] / s - W[target, :]) / valid for valid tokens, 0 otherwise (in place: dH is the accumulator);
// loss sum and the per-token terms.
__global__ void __launch_bounds__(kCeThreads) k_ce_finalize(CeState st, const int *__restrict__ labels, int vocab, const __half *__restrict__ W,
                                                            float *__restrict__ dH, int H) {
    const int t = blockIdx.x;
    const int y = labels[t];
    const bool ok = y >= 0 && y < vocab;
    const int nv = st.valid[0];
    if (threadIdx.x == 0 && ok) {
        const double lse = (double)st.m[t] + log(st.s[t]);
        atomicAdd(st.loss, lse - (double)st.tl[t]);
    }
    if (!dH) return;
    float *a = dH + (int64_t)t * H;
    if (!ok || nv <= 0) {
        for (int c = threadIdx.x; c < H; c += kCeThreads) a[c] = 0.f;
        return;
    }
    const float inv_s = (float)(1.0 / st.s[t]);
    const float inv_valid = 1.0f / (float)nv;
    const __half *wr = W + (int64_t)y * H;
    for (int c = threadIdx.x; c < H; c += kCeThreads) a[c] = (a[c] * inv_s - __half2float(wr[c])) * inv_valid;
}

__global__ void k_ce_loss_out(CeState st, float *loss_out, int *valid_out) {
    const int nv = st.valid[0];
    if (loss_out) *loss_out = nv > 0 ? (float)(st.loss[0] / (double)nv) : 0.f;
    if (valid_out) *valid_out = nv;
}

// Embedding rows: out[t, :] = decode(W[token[t], :]) (QuantKernels.ExtractEmbedding per token,
// src/Glacier.Tune/Model/GgufLoraModel.cs:456-462); a token outside [0, vocab) gives a zero row and raises bad[0].
template <int QT>
__global__ void k_embed_rows(const uint8_t *__restrict__ w, int K, int vocab, const int *__restrict__ tokens, float *__restrict__ out, int *bad) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float *o = out + (int64_t)t * K;
    if (tok < 0 || tok >= vocab) {
        for (int c = threadIdx.x; c < K; c += blockDim.x) o[c] = 0.f;
        if (threadIdx.x == 0 && bad) atomicAdd(bad, 1);
        return;
    }
    const int64_t base = (int64_t)tok * K;
    for (int c = threadIdx.x; c < K; c += blockDim.x) o[c] = decode_flat<QT>(w, base + c);
}

// vocabulary tile: about one wave of 128-row CTAs, an even number of them (CTA pairs), the tiles nearly equal
int vocab_tile_rows(int vocab, int sm_count) {
    const int tiles_total = (vocab + 127) / 128;
    const int waves = (tiles_total + sm_count - 1) / sm_count;
    int per = (tiles_total + waves - 1) / waves;
    per = (per + 1) & ~1;
    return per * 128;
}

struct CeBuffers {
    float *logits;
    __half *p16, *h16;
    CeState st;
    int vt;
};

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

int ce_reserve(gt_engine *e, int T, int H, int vocab, bool want_grad, CeBuffers *b) {
    const int vt = vocab_tile_rows(vocab, e->sm_count);
    const size_t n_logits = align256((size_t)T * vt * sizeof(float));
    const size_t n_p16 = want_grad ? align256((size_t)T * vt * sizeof(__half)) : 0;
    const size_t n_h16 = align256((size_t)T * H * sizeof(__half));
    const size_t n_m = align256((size_t)T * sizeof(float)), n_s = align256((size_t)T * sizeof(double));
    const size_t total = n_logits + n_p16 + n_h16 + 2 * n_m + n_s + 256;
    GT_CUDA(e->ce.reserve(total));
    char *p = (char *)e->ce.p;
    b->logits = (float *)p; p += n_logits;
    b->p16 = want_grad ? (__half *)p : nullptr; p += n_p16;
    b->h16 = (__half *)p; p += n_h16;
    b->st.m = (float *)p; p += n_m;
    b->st.tl = (float *)p; p += n_m;
    b->st.s = (double *)p; p += n_s;
    b->st.loss = (double *)p;
    b->st.valid = (int *)(p + 16);
    b->vt = vt;
    return GT_OK;
}

UmmaLaunch head_launch(gt_engine *e, const WeightDev *w, bool backward, const void *act16, int ld_act, int T, float *out, int ld_out,
                       int v0, int rows) {
    UmmaLaunch L;
    L.w = w;
    L.backward = backward ? 1 : 0;
    L.fp16 = 1;
    L.act16 = act16;
    L.ld_act = ld_act;
    L.T = T;
    L.out = out;
    L.ld_out = ld_out;
    L.row_base = v0;
    L.rows = rows;
    L.status = e->status;
    L.trace = e->trace;
    L.splits = umma_group_splits(&L, 1, e->sm_count);
    return L;
}

int check_head(const gt_engine *e, const gt_weight *w, const char *who) {
    if (!e || !w) return failf(GT_ERR_INVALID, "%s: null argument", who);
    if (w->dev.qtype != kTypeF16 || !w->dev.tma_ok)
        return failf(GT_ERR_UNSUPPORTED, "%s: the LM head must be an F16 tensor with in_features %% 128 == 0 (got type %d, [%d, %d])", who,
                     w->dev.qtype, w->dev.N, w->dev.K);
    return GT_OK;
}

// device tensors; lock held
int lm_head_loss_device(gt_engine *e, const gt_weight *w, const float *hidden, const int *labels, int T, float *loss_dev, int *valid_dev,
                        float *d_hidden) {
    const WeightDev &wd = w->dev;
    const int V = wd.N, H = wd.K;
    CeBuffers b;
    int rc = ce_reserve(e, T, H, V, d_hidden != nullptr, &b);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_cast16(hidden, b.h16, T, H, H, 1, e->stream));
    k_ce_init<<<1, 256, 0, e->stream>>>(b.st, labels, T, V);
    GT_LAUNCH(e, cudaGetLastError());
    if (d_hidden) GT_CUDA(cudaMemsetAsync(d_hidden, 0, (size_t)T * H * sizeof(float), e->stream));
    for (int v0 = 0; v0 < V; v0 += b.vt) {
        const int rows = V - v0 < b.vt ? V - v0 : b.vt;
        const char *msg = nullptr;
        UmmaLaunch f = head_launch(e, &wd, false, b.h16, H, T, b.logits, b.vt, v0, rows);
        cudaError_t ce = timed_umma_group(e, &f, 1, &msg);
        if (ce != cudaSuccess) return failf(GT_ERR_CUDA, "LM-head logits GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
        k_ce_tile<<<T, kCeThreads, 0, e->stream>>>(b.st, b.logits, b.vt, rows, v0, labels, b.p16, b.vt, d_hidden, H);
        GT_LAUNCH(e, cudaGetLastError());
        if (d_hidden) {
            UmmaLaunch g = head_launch(e, &wd, true, b.p16, b.vt, T, d_hidden, H, v0, rows);
            ce = timed_umma_group(e, &g, 1, &msg);
            if (ce != cudaSuccess) return failf(GT_ERR_CUDA, "LM-head gradient GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
        }
    }
    k_ce_finalize<<<T, kCeThreads, 0, e->stream>>>(b.st, labels, V, (const __half *)wd.data, d_hidden, H);
    GT_LAUNCH(e, cudaGetLastError());
    k_ce_loss_out<<<1, 1, 0, e->stream>>>(b.st, loss_dev, valid_dev);
    GT_LAUNCH(e, cudaGetLastError());
    return GT_OK;
}

}  // namespace

namespace gt {
int lm_head_loss_on_device(gt_engine *e, const gt_weight *w, const float *hidden, const int *labels, int T, float *loss_dev, int *valid_dev,
                           float *d_hidden) {
    return lm_head_loss_device(e, w, hidden, labels, T, loss_dev, valid_dev, d_hidden);
}

int embedding_on_device(gt_engine *e, const gt_weight *w, const int *tokens, int T, float *out, int *bad_dev) {
    const WeightDev &wd = w->dev;
    switch (wd.qtype) {
        case kTypeF16: k_embed_rows<kTypeF16><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        case kTypeF32: k_embed_rows<kTypeF32><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        case kTypeQ40: k_embed_rows<kTypeQ40><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        case kTypeQ80: k_embed_rows<kTypeQ80><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        case kTypeQ4K: k_embed_rows<kTypeQ4K><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        case kTypeQ6K: k_embed_rows<kTypeQ6K><<<T, 256, 0, e->stream>>>(wd.data, wd.K, wd.N, tokens, out, bad_dev); break;
        default: return failf(GT_ERR_UNSUPPORTED, "embedding type %d is not supported", wd.qtype);
    }
    GT_LAUNCH(e, cudaGetLastError());
    return GT_OK;
}
}  // namespace gt

extern "C" {

int gt_lm_head_loss(gt_engine *e, const gt_weight *w, const float *hidden, const int32_t *labels, int32_t T, float *loss_out,
                    int32_t *valid_out, float *d_hidden, int32_t flags) {
    int rc = check_head(e, w, "gt_lm_head_loss");
    if (rc != GT_OK) return rc;
    if (!hidden || !labels || !loss_out) return failf(GT_ERR_INVALID, "gt_lm_head_loss: null argument");
    if (T <= 0) return failf(GT_ERR_INVALID, "T must be positive (got %d)", T);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (flags & GT_FLAG_DEVICE_PTRS) return lm_head_loss_device(e, w, hidden, labels, T, loss_out, valid_out, d_hidden);
    // host buffers: stage hidden and labels, bring the loss (and the gradient) back; complete on return
    const int H = w->dev.K;
    const size_t bh = (size_t)T * H * sizeof(float), bl = align256((size_t)T * sizeof(int));
    GT_CUDA(e->ce_host.reserve(2 * align256(bh) + bl + 256));
    char *p = (char *)e->ce_host.p;
    float *hid_d = (float *)p;
    float *dh_d = (float *)(p + align256(bh));
    int *lab_d = (int *)(p + 2 * align256(bh));
    float *loss_d = (float *)(p + 2 * align256(bh) + bl);
    int *valid_d = (int *)(loss_d + 1);
    GT_CUDA(cudaMemcpyAsync(hid_d, hidden, bh, cudaMemcpyHostToDevice, e->stream));
    GT_CUDA(cudaMemcpyAsync(lab_d, labels, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    rc = lm_head_loss_device(e, w, hid_d, lab_d, T, loss_d, valid_d, d_hidden ? dh_d : nullptr);
    if (rc != GT_OK) return rc;
    float hl = 0.f;
    int hv = 0;
    GT_CUDA(cudaMemcpyAsync(&hl, loss_d, sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaMemcpyAsync(&hv, valid_d, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    if (d_hidden) GT_CUDA(cudaMemcpyAsync(d_hidden, dh_d, bh, cudaMemcpyDeviceToHost, e->stream));
    rc = check_status(e);
    *loss_out = hl;
    if (valid_out) *valid_out = hv;
    return rc;
}

int gt_lm_head_logits(gt_engine *e, const gt_weight *w, const float *hidden, float *logits, int32_t T, int32_t flags) {
    int rc = check_head(e, w, "gt_lm_head_logits");
    if (rc != GT_OK) return rc;
    if (!hidden || !logits) return failf(GT_ERR_INVALID, "gt_lm_head_logits: null argument");
    if (T <= 0) return failf(GT_ERR_INVALID, "T must be positive (got %d)", T);
    if (!(flags & GT_FLAG_DEVICE_PTRS)) return failf(GT_ERR_UNSUPPORTED, "gt_lm_head_logits takes device tensors (GT_FLAG_DEVICE_PTRS)");
    const WeightDev &wd = w->dev;
    const int V = wd.N, H = wd.K;
    if (V % 4 != 0) return failf(GT_ERR_UNSUPPORTED, "gt_lm_head_logits: vocabulary size must be a multiple of 4");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    CeBuffers b;
    rc = ce_reserve(e, T, H, V, false, &b);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_cast16(hidden, b.h16, T, H, H, 1, e->stream));
    for (int v0 = 0; v0 < V; v0 += b.vt) {
        const int rows = V - v0 < b.vt ? V - v0 : b.vt;
        const char *msg = nullptr;
        UmmaLaunch f = head_launch(e, &wd, false, b.h16, H, T, logits + v0, V, v0, rows);
        cudaError_t ce = timed_umma_group(e, &f, 1, &msg);
        if (ce != cudaSuccess) return failf(GT_ERR_CUDA, "LM-head logits GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
    }
    return GT_OK;
}

int gt_embedding_forward(gt_engine *e, const gt_weight *w, const int32_t *tokens, int32_t T, float *out, int32_t flags) {
    if (!e || !w || !tokens || !out) return failf(GT_ERR_INVALID, "gt_embedding_forward: null argument");
    if (T <= 0) return failf(GT_ERR_INVALID, "T must be positive (got %d)", T);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (flags & GT_FLAG_DEVICE_PTRS) return embedding_on_device(e, w, tokens, T, out, nullptr);
    const int K = w->dev.K;
    const size_t bo = (size_t)T * K * sizeof(float);
    GT_CUDA(e->ce_host.reserve(align256(bo) + align256((size_t)T * sizeof(int)) + 256));
    float *out_d = (float *)e->ce_host.p;
    int *tok_d = (int *)((char *)e->ce_host.p + align256(bo));
    int *bad_d = tok_d + ((T + 63) & ~63);
    GT_CUDA(cudaMemcpyAsync(tok_d, tokens, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    GT_CUDA(cudaMemsetAsync(bad_d, 0, sizeof(int), e->stream));
    int rc = embedding_on_device(e, w, tok_d, T, out_d, bad_d);
    if (rc != GT_OK) return rc;
    int bad = 0;
    GT_CUDA(cudaMemcpyAsync(out, out_d, bo, cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaMemcpyAsync(&bad, bad_d, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    // the reference throws ArgumentOutOfRangeException for such a token (GgufLoraModel.cs:443-452)
    if (bad) return failf(GT_ERR_INVALID, "gt_embedding_forward: %d token id(s) outside the vocabulary [0, %d)", bad, w->dev.N);
    return GT_OK;
}

}  // extern "C"
