// C ABI of libglaciertune_b200.so (declared in include/glaciertune_b200.h): engine, weight upload,
// adapters, projection forward / backward.  Host-side orchestration only; kernels are in
// gt_fp32_kernels.cu (CUDA cores) and gt_umma_gemm.cu (tcgen05).
#include <cuda_runtime.h>

#include <cstdlib>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "gt_engine_priv.h"

using namespace gt;

namespace gt {
namespace {
thread_local char g_err[512] = "";
std::mutex g_log_mu;
gt_log_fn g_log_fn = nullptr;
void *g_log_user = nullptr;
}  // namespace
void logf(int level, const char *fmt, ...) {
    gt_log_fn fn;
    void *user;
    {
        std::lock_guard<std::mutex> lk(g_log_mu);
        fn = g_log_fn;
        user = g_log_user;
    }
    if (!fn) return;
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    fn(level, buf, user);
}
int failf(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    logf(GT_LOG_ERROR, "%s", g_err);
    return code;
}
}  // namespace gt
#define fail gt::failf

namespace gt {

int check_status(gt_engine *e) {
    int h[4] = {0, 0, 0, 0};
    GT_CUDA(cudaMemcpyAsync(h, e->status, sizeof(h), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    if (h[0] != 0) {
        cudaMemsetAsync(e->status, 0, 4 * sizeof(int), e->stream);
        return fail(GT_ERR_KERNEL, "tensor-core GEMM gave up on a bounded wait (code %d: role %d, barrier %d)", h[0],
                    h[0] / 100, h[0] % 100);
    }
    return GT_OK;
}

bool tensor_path(const gt_engine *e, const gt_weight *w) {
    return e->math_mode != GT_MATH_FP32 && w->dev.tma_ok && (w->dev.qtype == kTypeQ4K || w->dev.qtype == kTypeQ6K);
}

int round8(int n) { return (n + 7) & ~7; }

cudaEvent_t next_event(gt_engine *e) {
    if (e->ev_used == e->ev_pool.size()) {
        cudaEvent_t ev = nullptr;
        if (cudaEventCreate(&ev) != cudaSuccess) return nullptr;
        e->ev_pool.push_back(ev);
    }
    return e->ev_pool[e->ev_used++];
}

// launch the tensor-core GEMM (one launch for all members), bracketed by events when profiling is on
cudaError_t timed_umma_group(gt_engine *e, const UmmaLaunch *m, int n, const char **msg, cudaStream_t on, const UmmaDual *dual) {
    cudaStream_t st = on ? on : e->stream;
    cudaEvent_t a = nullptr, b = nullptr;
    if (e->profile) {
        a = next_event(e);
        b = next_event(e);
        if (a) cudaEventRecord(a, e->stream);
    }
    cudaError_t ce = launch_umma_group(m, n, st, msg, dual);
    if (ce != cudaSuccess) cudaGetLastError();      // a refused launch must not linger as the thread's "last error"
    if (e->profile && b) cudaEventRecord(b, e->stream);
    e->gemm_launches += 1;
    e->kernel_launches += 1;
    for (int j = 0; j < n; j++) e->gemm_flops += 2.0 * (double)m[j].T * (double)(m[j].rows > 0 ? m[j].rows : m[j].w->N) * (double)m[j].w->K;
    return ce;
}


// Members of one quantization type form one GEMM launch; a Q4_K_M mix (q, k in Q4_K, v in Q6_K) takes two.
// order[] lists the member indices type by type, count[] the size of each run.
int partition_by_type(int n, const gt_weight *const *w, int *order, int *count) {
    int runs = 0, pos = 0;
    bool taken[kMaxGroup] = {false, false, false};
    for (int j = 0; j < n; j++) {
        if (taken[j]) continue;
        count[runs] = 0;
        for (int i = j; i < n; i++) {
            if (!taken[i] && w[i]->dev.qtype == w[j]->dev.qtype) {
                taken[i] = true;
                order[pos++] = i;
                count[runs]++;
            }
        }
        runs++;
    }
    return runs;
}

// The adapter's scratch holds low = X*A and dLow = dY*B^T of the current step side by side, [T, rank] fp32 each.
size_t low_bytes(const gt_adapter *a, int T) { return ((size_t)T * a->rank * sizeof(float) + 255) & ~(size_t)255; }
float *low_of(const gt_adapter *a) { return (float *)a->low.p; }
float *dlow_of(const gt_adapter *a, int T) { return (float *)((char *)a->low.p + low_bytes(a, T)); }

// low_j = X * A_j for every listed adapter (they share X), and optionally the 16-bit copy of X.  One memset per
// adapter clears low (the warp-MMA kernel sums into it) and dLow of the same step; one kernel pass reads X.
int compute_low(gt_engine *e, gt_adapter *const *ads, int n, const float *Xd, void *x16, int fp16, int T, int K,
                const RowFill *fills = nullptr, int n_fills = 0) {
    LoraXaJob jobs[kMaxGroup];
    for (int j = 0; j < n; j++) {
        gt_adapter *a = ads[j];
        GT_CUDA(a->low.reserve(2 * low_bytes(a, T)));
        GT_CUDA(cudaMemsetAsync(a->low.p, 0, 2 * low_bytes(a, T), e->stream));
        a->low_T = T;
        a->dlow_clean = true;
        jobs[j] = LoraXaJob{a->A, low_of(a), a->rank};
    }
    if (e->math_mode == GT_MATH_BF16) {
        GT_LAUNCH(e, launch_lora_xa_group(Xd, jobs, n, x16, K, fp16, T, K, fills, n_fills, e->stream));      // fills ride along
    } else {
        for (int j = 0; j < n_fills; j++) GT_LAUNCH(e, launch_fill_rows(fills[j].dst, fills[j].bias, T, fills[j].N, e->stream));
        for (int j = 0; j < n; j++)
            GT_LAUNCH(e, launch_lora_low(Xd, jobs[j].A, jobs[j].low_zeroed, j == 0 ? x16 : nullptr, K, fp16, T, K, jobs[j].R, e->stream));
    }
    return GT_OK;
}

// The same from an X that already exists as bf16 [T, K] (bf16 mode only): low_j = X16 * A_j, no copy is written.
int compute_low16(gt_engine *e, gt_adapter *const *ads, int n, const void *X16, int T, int K, const RowFill *fills = nullptr,
                  int n_fills = 0) {
    LoraXaJob jobs[kMaxGroup];
    for (int j = 0; j < n; j++) {
        gt_adapter *a = ads[j];
        GT_CUDA(a->low.reserve(2 * low_bytes(a, T)));
        GT_CUDA(cudaMemsetAsync(a->low.p, 0, 2 * low_bytes(a, T), e->stream));
        a->low_T = T;
        a->dlow_clean = true;
        jobs[j] = LoraXaJob{a->A, low_of(a), a->rank};
    }
    for (int j = 0; j < n_fills; j++) GT_LAUNCH(e, launch_fill_rows(fills[j].dst, fills[j].bias, T, fills[j].N, e->stream));
    if (n) GT_LAUNCH(e, launch_lora_xa16_group(X16, K, jobs, n, T, K, e->stream));
    return GT_OK;
}

int forward_device(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *Xd, float *Yd, int T, bool use_lora);
int backward_device(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *dYd, const float *Xd, float *dXd, int T,
                    bool use_lora, bool reuse_low, bool assign);

bool group_tensor_ok(const gt_engine *e, int n, const gt_weight *const *w) {
    if (n < 1 || n > kMaxGroup) return false;
    for (int j = 0; j < n; j++)
        if (!tensor_path(e, w[j]) || w[j]->dev.K != w[0]->dev.K) return false;      // quantization types may differ (Q4_K_M mixes)
    return true;
}

// Y_j = X * W_j^T (+ bias_j) (+ lora_j) for 1..3 projections that read the same X.  Tensor-core path: one pass over X
// (16-bit copy + every adapter's X*A), one GEMM launch.  Anything else runs member by member.
// x16_ready (bf16 mode, members on the tensor path): the input already exists as bf16 [T, K] - nothing is cast, the
// adapters' X*A reads that copy, Xd may be null.
// dual_h16 (two members that ffn_dual_ok() accepted): the launch is the dual forward - it also writes
// SiLU(Y_0) * Y_1 as 16-bit values to dual_h16 [T, out], and either Y_j may be null.
int forward_group_device(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *Xd, float *const *Yd,
                         int T, int flags, const void *x16_ready, void *dual_h16) {
    bool lora[kMaxGroup];
    for (int j = 0; j < n; j++) {
        lora[j] = ad && ad[j] && !(flags & GT_FLAG_NO_LORA) && ad[j]->rank > 0 && ad[j]->scaling != 0.f;
        if (ad && ad[j] && !lora[j]) ad[j]->low_T = 0;      // nothing kept for a later backward to reuse
        if (ad && ad[j]) ad[j]->xkeep_T = 0;                // a kept copy of an earlier X is stale now (the host path renews it)
    }
    if (dual_h16 && (n != 2 || !group_tensor_ok(e, n, w) || T <= 128))
        return fail(GT_ERR_INVALID, "forward_group_device: the dual forward was asked for a group it does not serve");
    if (!group_tensor_ok(e, n, w)) {
        for (int j = 0; j < n; j++) {
            int rc = forward_device(e, w[j], ad ? ad[j] : nullptr, Xd, Yd[j], T, lora[j]);
            if (rc != GT_OK) return rc;
        }
        return GT_OK;
    }
    const int K = w[0]->dev.K;
    const int fp16 = e->math_mode == GT_MATH_FP16;
    // Few tokens: the projection is bound by streaming the packed weights, which the warp-level kernel does several
    // times faster than the CTA-wide tensor-core kernel; the adapter term is added by the exact rank-r kernel.
    bool stream = !x16_ready && e->math_mode == GT_MATH_BF16 && (reinterpret_cast<uintptr_t>(Xd) & 15) == 0;
    for (int j = 0; j < n && stream; j++) stream = stream_fwd_ok(&w[j]->dev, T);
    if (stream) {
        gt_adapter *with[kMaxGroup];
        int n_with = 0;
        for (int j = 0; j < n; j++)
            if (lora[j]) with[n_with++] = ad[j];
        if (n_with) {
            int rc = compute_low(e, with, n_with, Xd, nullptr, 0, T, K);
            if (rc != GT_OK) return rc;
        }
        for (int j = 0; j < n; j++) {
            const WeightDev &wd = w[j]->dev;
            GT_LAUNCH(e, launch_fill_rows(Yd[j], wd.bias, T, wd.N, e->stream));      // the kernel adds into Y
            cudaEvent_t ea = nullptr, eb = nullptr;
            if (e->profile) {
                ea = next_event(e);
                eb = next_event(e);
                if (ea) cudaEventRecord(ea, e->stream);
            }
            cudaError_t ce = launch_stream_fwd(&wd, Xd, Yd[j], T, e->sm_count, e->status, e->trace, e->stream);
            if (e->profile && eb) cudaEventRecord(eb, e->stream);
            e->gemm_launches += 1;
            e->kernel_launches += 1;
            e->gemm_flops += 2.0 * (double)T * (double)wd.N * (double)K;
            if (ce != cudaSuccess) return fail(GT_ERR_CUDA, "streaming forward launch failed: %s", cudaGetErrorString(ce));
            if (lora[j])
                GT_LAUNCH(e, launch_lora_delta_fp32(low_of(ad[j]), ad[j]->B, Yd[j], nullptr, T, wd.N, ad[j]->rank, ad[j]->scaling,
                                                    ad[j]->b_nonzero, e->stream));
        }
        return GT_OK;
    }
    if (!x16_ready) GT_CUDA(e->x16.reserve((size_t)T * K * 2));
    const void *act16 = x16_ready ? x16_ready : e->x16.p;
    UmmaLaunch m[kMaxGroup];
    for (int j = 0; j < n; j++) {
        const WeightDev &wd = w[j]->dev;
        m[j].w = &wd;
        m[j].backward = 0;
        m[j].fp16 = fp16;
        m[j].act16 = act16;
        m[j].ld_act = K;
        m[j].T = T;
        m[j].out = Yd[j];
        m[j].ld_out = wd.N;
        m[j].bias = wd.bias;
        if (lora[j]) {
            m[j].lora_scale = ad[j]->scaling;
            m[j].lora_w = ad[j]->B;
            m[j].rank = ad[j]->rank;
            m[j].lora_flag = ad[j]->b_nonzero;
        }
        m[j].status = e->status;
        m[j].trace = e->trace;
    }
    // one launch per quantization type; split-K sums into the outputs: they start as the bias rows, written by the
    // pass over X below
    int order[kMaxGroup], count[kMaxGroup];
    const int runs = partition_by_type(n, w, order, count);
    UmmaLaunch run_m[kMaxGroup];      // members in launch order
    RowFill fills[kMaxGroup];
    int n_fills = 0;
    for (int r = 0, pos = 0; r < runs; pos += count[r], r++) {
        for (int i = 0; i < count[r]; i++) run_m[pos + i] = m[order[pos + i]];
        const int splits = dual_h16 ? 1 : umma_group_splits(run_m + pos, count[r], e->sm_count);
        for (int i = 0; i < count[r]; i++) {
            const int j = order[pos + i];
            m[j].splits = splits;
            if (splits > 1) {
                fills[n_fills++] = RowFill{Yd[j], w[j]->dev.bias, w[j]->dev.N};
                m[j].out_prefilled = 1;
            }
        }
    }
    gt_adapter *with[kMaxGroup];
    int n_with = 0;
    for (int j = 0; j < n; j++)
        if (lora[j]) with[n_with++] = ad[j];
    if (x16_ready) {
        int rc = compute_low16(e, with, n_with, x16_ready, T, K, fills, n_fills);
        if (rc != GT_OK) return rc;
        for (int j = 0; j < n; j++)
            if (lora[j]) m[j].lora_act = low_of(ad[j]);
    } else if (n_with) {
        int rc = compute_low(e, with, n_with, Xd, e->x16.p, fp16, T, K, fills, n_fills);
        if (rc != GT_OK) return rc;
        for (int j = 0; j < n; j++)
            if (lora[j]) m[j].lora_act = low_of(ad[j]);       // the adapter's scratch is allocated by now
    } else {
        GT_LAUNCH(e, launch_cast16(Xd, e->x16.p, T, K, K, fp16, e->stream));
        for (int j = 0; j < n_fills; j++) GT_LAUNCH(e, launch_fill_rows(fills[j].dst, fills[j].bias, T, fills[j].N, e->stream));
    }
    // A Q4_K_M mix gives two launches (q, k in Q4_K | v in Q6_K) that read the same X and write different outputs: the
    // second one runs on the side stream beside the first (neither fills the GPU by itself)
    const bool side = runs > 1 && e->s_aux && !e->profile && side_da_enabled();
    if (side) {
        GT_CUDA(cudaEventRecord(e->ev_aux_fork, e->stream));
        GT_CUDA(cudaStreamWaitEvent(e->s_aux, e->ev_aux_fork, 0));
    }
    UmmaDual dual;
    if (dual_h16) {
        dual.h16 = dual_h16;
        dual.ld_h16 = w[0]->dev.N;
        if (runs != 1) return fail(GT_ERR_INVALID, "forward_group_device: the dual forward needs one quantization type");
    }
    for (int r = 0, pos = 0; r < runs; pos += count[r], r++) {
        for (int i = 0; i < count[r]; i++) run_m[pos + i] = m[order[pos + i]];
        const char *msg = nullptr;
        cudaError_t ce = timed_umma_group(e, run_m + pos, count[r], &msg, (side && r > 0) ? e->s_aux : nullptr, dual_h16 ? &dual : nullptr);
        if (ce != cudaSuccess) return fail(GT_ERR_CUDA, "forward GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
    }
    if (side) {
        GT_CUDA(cudaEventRecord(e->ev_aux_join, e->s_aux));
        GT_CUDA(cudaStreamWaitEvent(e->stream, e->ev_aux_join, 0));
    }
    return GT_OK;
}

// out[T, N] = act * W^T (+bias) (+ lora) on the engine stream, device pointers.
// the base product of a paired-row tensor on the tensor path (see the paired-row kernels in gt_fp32_kernels.cu)
bool paired_path(const gt_engine *e, const gt_weight *w) { return e->math_mode != GT_MATH_FP32 && w->has_paired; }

int paired_forward_base(gt_engine *e, const gt_weight *w, const float *Xd, float *Yd, int T) {
    const WeightDev &wd = w->dev, &pv = w->paired;
    const int fp16 = e->math_mode == GT_MATH_FP16;
    GT_CUDA(e->x16.reserve((size_t)2 * T * pv.K * 2));
    GT_CUDA(e->pair_tmp.reserve((size_t)2 * T * pv.N * sizeof(float)));
    GT_LAUNCH(e, launch_pair_expand16(Xd, e->x16.p, T, wd.K, fp16, e->stream));
    UmmaLaunch L;
    L.w = &pv;
    L.fp16 = fp16;
    L.act16 = e->x16.p;
    L.ld_act = pv.K;
    L.T = 2 * T;
    L.out = (float *)e->pair_tmp.p;
    L.ld_out = pv.N;
    L.status = e->status;
    L.trace = e->trace;
    L.splits = umma_group_splits(&L, 1, e->sm_count);
    if (L.splits > 1) {
        GT_LAUNCH(e, launch_fill_rows(L.out, nullptr, 2 * T, pv.N, e->stream));
        L.out_prefilled = 1;
    }
    const char *msg = nullptr;
    cudaError_t ce = timed_umma_group(e, &L, 1, &msg);
    if (ce != cudaSuccess) return fail(GT_ERR_CUDA, "forward GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
    GT_LAUNCH(e, launch_pair_interleave(L.out, wd.bias, Yd, T, wd.N, e->stream));
    return GT_OK;
}

int paired_backward_base(gt_engine *e, const gt_weight *w, const float *dYd, float *dXd, int T, bool assign) {
    const WeightDev &wd = w->dev, &pv = w->paired;
    const int fp16 = e->math_mode == GT_MATH_FP16;
    const int ld16 = round8(pv.N);
    GT_CUDA(e->dy16.reserve((size_t)2 * T * ld16 * 2));
    GT_CUDA(e->pair_tmp.reserve((size_t)2 * T * pv.K * sizeof(float)));
    GT_LAUNCH(e, launch_pair_gather16(dYd, e->dy16.p, T, wd.N, ld16, fp16, e->stream));
    UmmaLaunch L;
    L.w = &pv;
    L.backward = 1;
    L.fp16 = fp16;
    L.act16 = e->dy16.p;
    L.ld_act = ld16;
    L.T = 2 * T;
    L.out = (float *)e->pair_tmp.p;
    L.ld_out = pv.K;
    L.status = e->status;
    L.trace = e->trace;
    L.splits = umma_group_splits(&L, 1, e->sm_count);
    if (L.splits == 1) L.out_assign = 1;
    else GT_LAUNCH(e, launch_fill_rows(L.out, nullptr, 2 * T, pv.K, e->stream));
    const char *msg = nullptr;
    cudaError_t ce = timed_umma_group(e, &L, 1, &msg);
    if (ce != cudaSuccess) return fail(GT_ERR_CUDA, "backward GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
    GT_LAUNCH(e, launch_pair_fold(L.out, dXd, T, wd.K, assign ? 1 : 0, e->stream));
    return GT_OK;
}

int forward_device(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *Xd, float *Yd, int T, bool use_lora) {
    if (tensor_path(e, w)) return forward_group_device(e, 1, &w, &ad, Xd, &Yd, T, use_lora ? 0 : GT_FLAG_NO_LORA);
    const WeightDev &wd = w->dev;
    const int N = wd.N, K = wd.K;
    if (paired_path(e, w)) {
        int prc = paired_forward_base(e, w, Xd, Yd, T);
        if (prc != GT_OK) return prc;
    } else {
        GT_LAUNCH(e, launch_gemm_fp32_fwd(wd.qtype, wd.data, Xd, Yd, nullptr, wd.bias, T, N, K, e->stream));
    }
    if (use_lora) {
        int rc = compute_low(e, &ad, 1, Xd, nullptr, 0, T, K);
        if (rc != GT_OK) return rc;
        GT_LAUNCH(e, launch_lora_delta_fp32(low_of(ad), ad->B, Yd, nullptr, T, N, ad->rank, ad->scaling, ad->b_nonzero, e->stream));
    } else if (ad) {
        ad->low_T = 0;
    }
    return GT_OK;
}

// The adapter half of a backward: dB += s*low^T*dY, dLow = dY*B^T, dA += s*X^T*dLow for every member with an adapter
// (one launch per product in the bf16 mode), and the 16-bit copy of each dY where dy16[j] is given.
int aux_init(gt_engine *e) {
    if (e->s_aux) return GT_OK;
    GT_CUDA(cudaStreamCreateWithFlags(&e->s_aux, cudaStreamNonBlocking));
    GT_CUDA(cudaEventCreateWithFlags(&e->ev_aux_fork, cudaEventDisableTiming));
    GT_CUDA(cudaEventCreateWithFlags(&e->ev_aux_join, cudaEventDisableTiming));
    return GT_OK;
}
// the engine stream waits for a dA pass that was put on the side stream
int aux_join(gt_engine *e) {
    if (!e->aux_pending) return GT_OK;
    GT_CUDA(cudaStreamWaitEvent(e->stream, e->ev_aux_join, 0));
    e->aux_pending = false;
    return GT_OK;
}
bool side_da_enabled() {
    static const bool on = [] {
        const char *v = getenv("GT_SIDE_DA");
        return !(v && v[0] == '0');
    }();
    return on;
}

int lora_backward_group(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const bool *lora,
                        const float *const *dYd, const float *Xd, void *const *dy16, const int *ld16, int T, bool reuse_low,
                        float *zero_dx, bool side_da = false, const void *X16 = nullptr) {
    const int K = w[0]->dev.K;
    const int fp16 = e->math_mode == GT_MATH_FP16;
    const bool fast = e->math_mode == GT_MATH_BF16;      // bf16 warp-MMA reductions; exact fp32 otherwise
    gt_adapter *fresh[kMaxGroup];
    int n_fresh = 0;
    for (int j = 0; j < n; j++) {
        if (!lora[j]) continue;
        gt_adapter *a = ad[j];
        if (reuse_low && a->low.p && a->low_T == T) {
            if (!a->dlow_clean) GT_CUDA(cudaMemsetAsync(dlow_of(a, T), 0, low_bytes(a, T), e->stream));
        } else {
            fresh[n_fresh++] = a;
        }
    }
    if (n_fresh) {
        int rc = X16 ? compute_low16(e, fresh, n_fresh, X16, T, K) : compute_low(e, fresh, n_fresh, Xd, nullptr, 0, T, K);
        if (rc != GT_OK) return rc;
    }
    LoraDyJob dy[kMaxGroup];
    LoraDaJob da[kMaxGroup];
    int nl = 0;
    for (int j = 0; j < n; j++) {
        if (!lora[j]) {
            // (a null dY_j: its 16-bit copy is in place already)
            if (dy16[j] && dYd[j]) GT_LAUNCH(e, launch_cast16(dYd[j], dy16[j], T, w[j]->dev.N, ld16[j], fp16, e->stream));
            continue;
        }
        gt_adapter *a = ad[j];
        a->dlow_clean = false;
        dy[nl] = LoraDyJob{dYd[j], low_of(a), a->B, a->dB, dlow_of(a, T), dy16[j], ld16[j], a->scaling, w[j]->dev.N, a->rank};
        da[nl] = LoraDaJob{dlow_of(a, T), a->dA, a->scaling, a->rank};
        nl++;
    }
    // "dX =" instead of "dX +=": the buffer is cleared by the pass over dY (or by a fill of its own)
    const RowFill zero{zero_dx, nullptr, K};
    if (zero_dx && !(fast && nl)) GT_LAUNCH(e, launch_fill_rows(zero_dx, nullptr, T, K, e->stream));
    if (!nl) return GT_OK;
    if (fast) {
        GT_LAUNCH(e, launch_lora_dy_group(dy, nl, fp16, T, zero_dx ? &zero : nullptr, zero_dx ? 1 : 0, e->stream));
        cudaStream_t da_stream = e->stream;
        if (side_da && e->s_aux) {
            GT_CUDA(cudaEventRecord(e->ev_aux_fork, e->stream));
            GT_CUDA(cudaStreamWaitEvent(e->s_aux, e->ev_aux_fork, 0));
            da_stream = e->s_aux;
        }
        if (X16) GT_LAUNCH(e, launch_lora_da16_group(X16, K, da, nl, T, K, da_stream));
        else GT_LAUNCH(e, launch_lora_da_group(Xd, da, nl, T, K, da_stream));
        if (da_stream != e->stream) {
            GT_CUDA(cudaEventRecord(e->ev_aux_join, e->s_aux));
            e->aux_pending = true;
        }
    } else {
        for (int j = 0; j < nl; j++) {
            GT_LAUNCH(e, launch_lora_bwd_dy(dy[j].dY, dy[j].low, dy[j].B, dy[j].dB, dy[j].dLow_zeroed, dy[j].dy16, dy[j].ld16, fp16,
                                            dy[j].scaling, T, dy[j].N, dy[j].R, e->stream));
            GT_LAUNCH(e, launch_lora_bwd_x(Xd, da[j].dLow, da[j].dA, da[j].scaling, T, K, da[j].R, e->stream));
        }
    }
    return GT_OK;
}

// dX += sum_j dY_j * W_j (+ lora terms); dA_j, dB_j accumulate.  Tensor-core path: one GEMM launch for the group.
// X16 (bf16 mode, members on the tensor path): the forward input as bf16 [T, K] instead of the fp32 Xd (which may be null).
// where the 16-bit copies of a group's dY_j live inside the engine's dy16 scratch
static size_t dy16_layout(int n, const gt_weight *const *w, int T, size_t *off, int *ld) {
    size_t total = 0;
    for (int j = 0; j < n; j++) {
        ld[j] = round8(w[j]->dev.N);
        off[j] = total;
        total += ((size_t)T * ld[j] * 2 + 255) & ~(size_t)255;
    }
    return total;
}

int backward_group_device(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *const *dYd,
                          const float *Xd, float *dXd, int T, int flags, const void *X16, bool dy16_ready) {
    bool lora[kMaxGroup];
    for (int j = 0; j < n; j++) lora[j] = ad && ad[j] && !(flags & GT_FLAG_NO_LORA) && ad[j]->rank > 0;
    const bool reuse_low = (flags & GT_FLAG_REUSE_LOW) != 0;
    const bool assign = (flags & GT_FLAG_DX_ASSIGN) != 0 && dXd;
    if (!group_tensor_ok(e, n, w) || !dXd) {
        if (dy16_ready) return fail(GT_ERR_INVALID, "backward_group_device: 16-bit gradients need the tensor path");
        for (int j = 0; j < n; j++) {
            int rc = backward_device(e, w[j], ad ? ad[j] : nullptr, dYd[j], Xd, dXd, T, lora[j], reuse_low, assign && j == 0);
            if (rc != GT_OK) return rc;
        }
        return GT_OK;
    }
    const int K = w[0]->dev.K;
    const int fp16 = e->math_mode == GT_MATH_FP16;
    size_t dy_off[kMaxGroup];
    int ld16[kMaxGroup];
    void *dy16[kMaxGroup];
    const size_t dy_total = dy16_layout(n, w, T, dy_off, ld16);
    if (dy16_ready && (e->dy16.cap < dy_total || e->math_mode != GT_MATH_BF16 || !group_tensor_ok(e, n, w) || !dXd))
        return fail(GT_ERR_INVALID, "backward_group_device: the 16-bit gradients are not where this call reads them");
    GT_CUDA(e->dy16.reserve(dy_total));
    for (int j = 0; j < n; j++) dy16[j] = (char *)e->dy16.p + dy_off[j];
    UmmaLaunch m[kMaxGroup];
    for (int j = 0; j < n; j++) {
        const WeightDev &wd = w[j]->dev;
        m[j].w = &wd;
        m[j].backward = 1;
        m[j].fp16 = fp16;
        m[j].act16 = dy16[j];
        m[j].ld_act = ld16[j];
        m[j].T = T;
        m[j].out = dXd;
        m[j].ld_out = K;
        m[j].status = e->status;
        m[j].trace = e->trace;
    }
    // one launch per quantization type, all summing into the same dX.  "dX =": when the first launch has one CTA per
    // output tile (no split-K) it writes dX with plain stores and nothing has to clear the buffer first; otherwise the
    // pass over dY (or a fill of its own) clears it and every launch adds.
    int order[kMaxGroup], count[kMaxGroup], run_splits[kMaxGroup];
    const int runs = partition_by_type(n, w, order, count);
    UmmaLaunch run_m[kMaxGroup];
    for (int r = 0, pos = 0; r < runs; pos += count[r], r++) {
        for (int i = 0; i < count[r]; i++) run_m[pos + i] = m[order[pos + i]];
        run_splits[r] = umma_group_splits(run_m + pos, count[r], e->sm_count);
    }
    const bool store_first = assign && run_splits[0] == 1;
    int rc = lora_backward_group(e, n, w, ad, lora, dYd, Xd, dy16, ld16, T, reuse_low, (assign && !store_first) ? dXd : nullptr,
                                 side_da_enabled() && !e->profile,       // profiling times each GEMM alone on the device
                                 e->math_mode == GT_MATH_BF16 ? X16 : nullptr);
    if (rc != GT_OK) return rc;
    for (int j = 0; j < n; j++) {
        if (lora[j]) {
            m[j].lora_act = dlow_of(ad[j], T);      // the adapter's scratch is allocated by now
            m[j].lora_scale = ad[j]->scaling;
            m[j].lora_w = ad[j]->A;
            m[j].rank = ad[j]->rank;
        }
    }
    // A run served by the few-token kernel adds its adapter terms to dX with plain read-modify-writes: then no run of
    // this call may work on the side stream (the runs' types differ, so some may be few-token launches and some not)
    bool any_few = false;
    for (int r = 0, pos = 0; r < runs; pos += count[r], r++) {
        for (int i = 0; i < count[r]; i++) run_m[pos + i] = m[order[pos + i]];
        any_few = any_few || umma_group_few(run_m + pos, count[r]);
    }
    for (int r = 0, pos = 0; r < runs; pos += count[r], r++) {
        for (int i = 0; i < count[r]; i++) {
            run_m[pos + i] = m[order[pos + i]];
            run_m[pos + i].splits = run_splits[r];
        }
        run_m[pos].out_assign = (r == 0 && store_first) ? 1 : 0;
        // launches of the other quantization types add into the same dX with atomics: beside the first one on the side
        // stream (behind the dA pass there), unless the first one writes dX with plain stores
        const bool side = r > 0 && !store_first && e->s_aux && !e->profile && side_da_enabled() && !any_few;
        if (side && !e->aux_pending) {      // no dA pass was forked: fork now (the pass over dY is complete by stream order)
            GT_CUDA(cudaEventRecord(e->ev_aux_fork, e->stream));
            GT_CUDA(cudaStreamWaitEvent(e->s_aux, e->ev_aux_fork, 0));
        }
        const char *msg = nullptr;
        cudaError_t ce = timed_umma_group(e, run_m + pos, count[r], &msg, side ? e->s_aux : nullptr);
        if (ce != cudaSuccess) return fail(GT_ERR_CUDA, "backward GEMM launch failed: %s", msg ? msg : cudaGetErrorString(ce));
        if (side) {
            GT_CUDA(cudaEventRecord(e->ev_aux_join, e->s_aux));
            e->aux_pending = true;
        }
    }
    return aux_join(e);      // the dA pass and the side launches are part of this call
}

// dX += dY*W (+ lora term); dA, dB accumulate.  Device pointers.
int backward_device(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *dYd, const float *Xd, float *dXd, int T,
                    bool use_lora, bool reuse_low, bool assign) {
    if (tensor_path(e, w) && dXd) {
        const int flags = (use_lora ? 0 : GT_FLAG_NO_LORA) | (reuse_low ? GT_FLAG_REUSE_LOW : 0) | (assign ? GT_FLAG_DX_ASSIGN : 0);
        return backward_group_device(e, 1, &w, &ad, &dYd, Xd, dXd, T, flags);
    }
    // exact fp32 kernels (validation mode, weights outside the tensor-core layout) or adapter gradients only
    const WeightDev &wd = w->dev;
    const int N = wd.N, K = wd.K;
    const bool paired = paired_path(e, w) && dXd;
    if (paired) {      // the base product writes (or adds into) dX itself
        int prc = paired_backward_base(e, w, dYd, dXd, T, assign);
        if (prc != GT_OK) return prc;
    } else if (assign && dXd) {
        GT_LAUNCH(e, launch_fill_rows(dXd, nullptr, T, K, e->stream));
    }
    if (use_lora) {
        const bool lora = true;
        void *no16 = nullptr;
        const int ld16 = round8(N);
        int rc = lora_backward_group(e, 1, &w, &ad, &lora, &dYd, Xd, &no16, &ld16, T, reuse_low, nullptr);
        if (rc != GT_OK) return rc;
        if (dXd) GT_LAUNCH(e, launch_lora_dx_fp32(dlow_of(ad, T), ad->A, dXd, ad->scaling, T, K, ad->rank, e->stream));
    }
    if (dXd && !paired) GT_LAUNCH(e, launch_gemm_fp32_bwd(wd.qtype, wd.data, dYd, dXd, T, N, K, e->stream));
    return GT_OK;
}


// FFN block on device tensors: gate, up = projections of X (one group); hidden = SiLU(gate) * up; Y = down(hidden).
// w / ad = {gate, up, down}.  gate_d / up_d / hidden_d may be null (engine scratch is used).
// The SwiGLU pass can write the down projection's 16-bit operand itself: bf16 mode, down on the tensor path, more tokens
// than the few-token kernels take (they stage fp32 activations themselves), ffn a multiple of 8.
bool ffn_hidden16_ok(const gt_engine *e, const gt_weight *const *w, int T) {
    static const bool on = !(getenv("GT_SWIGLU_FOLD") && atoi(getenv("GT_SWIGLU_FOLD")) == 0);
    const gt_weight *down = w[2];
    return on && e->math_mode == GT_MATH_BF16 && tensor_path(e, down) && T > 64 && (down->dev.K % 8) == 0;
}

// The SwiGLU backward can write dGate, dUp as the bf16 operands of the gate,up transpose GEMM directly (no fp32 pair, no
// cast pass): bf16 mode, both on the tensor path with the same row length, a multiple of 8 (their 16-bit rows are then
// dense), more tokens than any few-token kernel takes.
bool ffn_dy16_ok(const gt_engine *e, const gt_weight *const *w, int T) {
    static const bool on = !(getenv("GT_SWIGLU_FOLD") && atoi(getenv("GT_SWIGLU_FOLD")) == 0);
    return on && e->math_mode == GT_MATH_BF16 && group_tensor_ok(e, 2, w) && T > 128 && w[0]->dev.N == w[1]->dev.N && (w[0]->dev.N % 8) == 0;
}

// gate | up in ONE launch whose epilogue forms SiLU(gate) * up (the reference's gemm_q4_k_swiglu_batch,
// GpuLoraEngine.Forward.cs:152-183,282-285): both of one quantization type on the tensor path, enough 64-feature tiles to
// fill the GPU without split-K, adapter ranks up to 32.  GT_FFN_DUAL=0 keeps the separate SwiGLU pass.
bool ffn_dual_ok(const gt_engine *e, const gt_weight *const *w, gt_adapter *const *ad, int T, int flags) {
    static const bool on = !(getenv("GT_FFN_DUAL") && atoi(getenv("GT_FFN_DUAL")) == 0);
    if (!on || !ffn_hidden16_ok(e, w, T) || !group_tensor_ok(e, 2, w) || w[0]->dev.qtype != w[1]->dev.qtype || T <= 128) return false;
    UmmaLaunch m[2];
    for (int j = 0; j < 2; j++) {
        m[j].w = &w[j]->dev;
        m[j].T = T;
        m[j].fp16 = e->math_mode == GT_MATH_FP16;
        m[j].rank = (ad && ad[j] && !(flags & GT_FLAG_NO_LORA)) ? ad[j]->rank : 0;
    }
    return umma_dual_ok(m, e->sm_count);
}

int ffn_forward_device(gt_engine *e, const gt_weight *const *w, gt_adapter *const *ad, const float *Xd, float *gate_d, float *up_d,
                       float *hidden_d, float *Yd, int T, int flags, void *hidden16) {
    const int F = w[0]->dev.N;
    const size_t bf = (size_t)T * F * sizeof(float);
    const bool fold = ffn_hidden16_ok(e, w, T);
    if (hidden16 && !fold) return fail(GT_ERR_INVALID, "ffn_forward_device: a 16-bit hidden tensor needs ffn_hidden16_ok()");
    if (hidden16 && !hidden_d && ffn_dual_ok(e, w, ad, T, flags)) {
        // The caller keeps the product as bf16 only, in a buffer of its own: the gate | up launch writes it from its epilogue.
        // gate and up themselves are written where the caller gave a place for them (a backward needs them; a forward
        // pass whose state is recomputed later does not).
        float *gu[2] = {gate_d, up_d};
        int rc = forward_group_device(e, 2, w, ad, Xd, gu, T, flags, nullptr, hidden16);
        if (rc != GT_OK || !Yd) return rc;
        float *yd = Yd;
        return forward_group_device(e, 1, w + 2, ad ? ad + 2 : nullptr, nullptr, &yd, T, flags, hidden16);
    }
    float *bufs[3] = {gate_d, up_d, hidden_d};
    for (int i = 0; i < 3; i++) {
        if (!bufs[i] && !(i == 2 && fold)) {      // folded: the fp32 product is written only where the caller wants it
            GT_CUDA(e->ffn[i].reserve(bf));
            bufs[i] = (float *)e->ffn[i].p;
        }
    }
    float *gu[2] = {bufs[0], bufs[1]};
    int rc = forward_group_device(e, 2, w, ad, Xd, gu, T, flags);
    if (rc != GT_OK) return rc;
    float *yd = Yd;
    if (!Yd) {
        // activation only (the recomputed forward of a checkpointed block: the down projection's output is the stored
        // input of the next block, nobody reads it again); X*A of the down adapter, kept from the first forward, stays valid
        if (fold) {
            if (!hidden16) return GT_OK;      // nowhere to keep the product
            GT_LAUNCH(e, launch_swiglu_fwd16(bufs[0], bufs[1], bufs[2], hidden16, (int64_t)T * F, 0, e->sm_count, e->stream));
        } else {
            GT_LAUNCH(e, launch_swiglu_fwd(bufs[0], bufs[1], bufs[2], (int64_t)T * F, e->sm_count, e->stream));
        }
        return GT_OK;
    }
    if (fold) {
        // SiLU(gate) * up goes out as the bf16 operand of the down projection (and as fp32 only if asked for): the separate
        // pass that would read the fp32 product back to round it does not run
        void *h16 = hidden16;
        if (!h16) {
            GT_CUDA(e->x16.reserve((size_t)T * F * 2));
            h16 = e->x16.p;
        }
        GT_LAUNCH(e, launch_swiglu_fwd16(bufs[0], bufs[1], bufs[2], h16, (int64_t)T * F, 0, e->sm_count, e->stream));
        return forward_group_device(e, 1, w + 2, ad ? ad + 2 : nullptr, bufs[2], &yd, T, flags, h16);
    }
    GT_LAUNCH(e, launch_swiglu_fwd(bufs[0], bufs[1], bufs[2], (int64_t)T * F, e->sm_count, e->stream));
    return forward_group_device(e, 1, w + 2, ad ? ad + 2 : nullptr, bufs[2], &yd, T, flags);
}

// The matching backward: dHidden = dY * W_down (+ adapter), (dGate, dUp) = SwiGLU'(dHidden, gate, up),
// dX (+)= dGate * W_gate + dUp * W_up (+ adapters); adapter gradients accumulate.  Device tensors.
int ffn_backward_device(gt_engine *e, const gt_weight *const *w, gt_adapter *const *ad, const float *dYd, const float *Xd,
                        const float *gate_d, const float *up_d, const float *hidden_d, float *dXd, int T, int flags,
                        const void *hidden16) {
    const int F = w[0]->dev.N;
    const size_t bf = (size_t)T * F * sizeof(float);
    if (hidden16 && !ffn_hidden16_ok(e, w, T))
        return fail(GT_ERR_INVALID, "ffn_backward_device: a 16-bit hidden tensor needs ffn_hidden16_ok()");
    for (int i = 0; i < 3; i++) GT_CUDA(e->ffn[i].reserve(bf));
    float *dh = (float *)e->ffn[0].p, *dg = (float *)e->ffn[1].p, *du = (float *)e->ffn[2].p;
    if (gate_d == dh || gate_d == dg || gate_d == du || up_d == dh || up_d == dg || up_d == du ||
        (hidden_d && (hidden_d == dh || hidden_d == dg || hidden_d == du)))
        return fail(GT_ERR_INVALID, "gt_ffn_backward: gate, up and hidden must be the caller's buffers (the forward call was given NULL)");
    const float *dy1 = dYd;
    int rc = backward_group_device(e, 1, w + 2, ad ? ad + 2 : nullptr, &dy1, hidden_d, dh, T,
                                   (flags & ~GT_FLAG_DX_ASSIGN) | GT_FLAG_DX_ASSIGN, hidden16);      // dHidden is written, not added to
    if (rc != GT_OK) return rc;
    if (ffn_dy16_ok(e, w, T) && dXd) {
        // dGate, dUp as bf16 only, written where the group's transpose GEMM and adapter passes read their 16-bit dY
        size_t off[2];
        int ld[2];
        GT_CUDA(e->dy16.reserve(dy16_layout(2, w, T, off, ld)));
        GT_LAUNCH(e, launch_swiglu_bwd16(dh, gate_d, up_d, (char *)e->dy16.p + off[0], (char *)e->dy16.p + off[1], (int64_t)T * F, e->sm_count,
                                         e->stream));
        const float *none[2] = {nullptr, nullptr};
        return backward_group_device(e, 2, w, ad, none, Xd, dXd, T, flags, nullptr, true);
    }
    GT_LAUNCH(e, launch_swiglu_bwd(dh, gate_d, up_d, dg, du, (int64_t)T * F, e->sm_count, e->stream));
    const float *dgu[2] = {dg, du};
    return backward_group_device(e, 2, w, ad, dgu, Xd, dXd, T, flags);
}

// the engine stream waits for the collectives begun on the side stream (gt_dp_allreduce_begin)
int join_comm(gt_engine *e) {
    if (!e->comm_pending) return GT_OK;
    GT_CUDA(cudaStreamWaitEvent(e->stream, e->ev_join, 0));
    e->comm_pending = false;
    return GT_OK;
}

// ---- host-buffer calls -------------------------------------------------------------------------------------------
int host_pipeline_init(gt_engine *e) {
    if (e->s_h2d) return GT_OK;
    GT_CUDA(cudaStreamCreateWithFlags(&e->s_h2d, cudaStreamNonBlocking));
    GT_CUDA(cudaStreamCreateWithFlags(&e->s_d2h, cudaStreamNonBlocking));
    for (HostSlot &sl : e->slots) {
        GT_CUDA(cudaEventCreateWithFlags(&sl.h2d_done, cudaEventDisableTiming));
        GT_CUDA(cudaEventCreateWithFlags(&sl.compute_done, cudaEventDisableTiming));
        GT_CUDA(cudaEventCreateWithFlags(&sl.d2h_done, cudaEventDisableTiming));
    }
    return GT_OK;
}

HostSlot &next_slot(gt_engine *e) {
    HostSlot &sl = e->slots[e->slot_next];
    e->slot_next = (e->slot_next + 1) % kHostSlots;
    return sl;
}

// A synchronous call returns with its outputs in the host buffers; an asynchronous one (pinned buffers) returns
// once everything is queued, and gt_sync() completes it.
int finish_host_call(gt_engine *e, int flags) {
    if (flags & GT_FLAG_HOST_ASYNC) return GT_OK;
    int rc = check_status(e);
    GT_CUDA(cudaStreamSynchronize(e->s_d2h));
    return rc;
}

int forward_host(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *X, float *const *Y, int T,
                 int flags) {
    int rc = host_pipeline_init(e);
    if (rc != GT_OK) return rc;
    HostSlot &sl = next_slot(e);
    const size_t bx = (size_t)T * w[0]->dev.K * sizeof(float);
    GT_CUDA(sl.in[0].reserve(bx));
    float *Yd[kMaxGroup];
    for (int j = 0; j < n; j++) {
        GT_CUDA(sl.out[j].reserve((size_t)T * w[j]->dev.N * sizeof(float)));
        Yd[j] = (float *)sl.out[j].p;
    }
    if (sl.used) GT_CUDA(cudaStreamWaitEvent(e->s_h2d, sl.compute_done, 0));      // the slot's last call has read its inputs
    GT_CUDA(cudaMemcpyAsync(sl.in[0].p, X, bx, cudaMemcpyHostToDevice, e->s_h2d));
    GT_CUDA(cudaEventRecord(sl.h2d_done, e->s_h2d));
    GT_CUDA(cudaStreamWaitEvent(e->stream, sl.h2d_done, 0));
    if (sl.used) GT_CUDA(cudaStreamWaitEvent(e->stream, sl.d2h_done, 0));         // ... and its outputs have left
    rc = forward_group_device(e, n, w, ad, (const float *)sl.in[0].p, Yd, T, flags);
    if (rc != GT_OK) return rc;
    // the first adapted member keeps the staged X on the device: a backward that promises the same X
    // (GT_FLAG_REUSE_LOW) reads it from there instead of uploading it again
    for (int j = 0; j < n; j++) {
        if (ad && ad[j] && !(flags & GT_FLAG_NO_LORA) && ad[j]->rank > 0) {
            GT_CUDA(ad[j]->xkeep.reserve(bx));
            GT_CUDA(cudaMemcpyAsync(ad[j]->xkeep.p, sl.in[0].p, bx, cudaMemcpyDeviceToDevice, e->stream));
            ad[j]->xkeep_T = T;
            break;
        }
    }
    GT_CUDA(cudaEventRecord(sl.compute_done, e->stream));
    GT_CUDA(cudaStreamWaitEvent(e->s_d2h, sl.compute_done, 0));
    for (int j = 0; j < n; j++)
        GT_CUDA(cudaMemcpyAsync(Y[j], Yd[j], (size_t)T * w[j]->dev.N * sizeof(float), cudaMemcpyDeviceToHost, e->s_d2h));
    GT_CUDA(cudaEventRecord(sl.d2h_done, e->s_d2h));
    sl.used = true;
    return finish_host_call(e, flags);
}

int backward_host(gt_engine *e, int n, const gt_weight *const *w, gt_adapter *const *ad, const float *const *dY, const float *X,
                  float *dX, int T, int flags) {
    int rc = host_pipeline_init(e);
    if (rc != GT_OK) return rc;
    HostSlot &sl = next_slot(e);
    const size_t bx = (size_t)T * w[0]->dev.K * sizeof(float);
    const bool assign = (flags & GT_FLAG_DX_ASSIGN) != 0;
    bool need_x = false;
    const float *x_kept = nullptr;
    for (int j = 0; j < n; j++) {
        if (ad && ad[j] && !(flags & GT_FLAG_NO_LORA) && ad[j]->rank > 0) {
            if (!need_x && (flags & GT_FLAG_REUSE_LOW) && ad[j]->xkeep.p && ad[j]->xkeep_T == T) x_kept = (const float *)ad[j]->xkeep.p;
            need_x = true;
        }
    }
    if (x_kept) need_x = false;      // X of the forward is still on the device
    const float *dYd[kMaxGroup];
    for (int j = 0; j < n; j++) {
        GT_CUDA(sl.in[j].reserve((size_t)T * w[j]->dev.N * sizeof(float)));
        dYd[j] = (const float *)sl.in[j].p;
    }
    if (need_x) GT_CUDA(sl.in[kSlotIn - 1].reserve(bx));
    if (dX) GT_CUDA(sl.out[0].reserve(bx));
    if (sl.used) {
        GT_CUDA(cudaStreamWaitEvent(e->s_h2d, sl.compute_done, 0));
        if (dX && !assign) GT_CUDA(cudaStreamWaitEvent(e->s_h2d, sl.d2h_done, 0));
    }
    for (int j = 0; j < n; j++)
        GT_CUDA(cudaMemcpyAsync(sl.in[j].p, dY[j], (size_t)T * w[j]->dev.N * sizeof(float), cudaMemcpyHostToDevice, e->s_h2d));
    if (need_x) GT_CUDA(cudaMemcpyAsync(sl.in[kSlotIn - 1].p, X, bx, cudaMemcpyHostToDevice, e->s_h2d));
    // "dX +=": the reference uploads dX too and the kernel accumulates into it (GpuLoraEngine.Backward.cs:85-89)
    if (dX && !assign) GT_CUDA(cudaMemcpyAsync(sl.out[0].p, dX, bx, cudaMemcpyHostToDevice, e->s_h2d));
    GT_CUDA(cudaEventRecord(sl.h2d_done, e->s_h2d));
    GT_CUDA(cudaStreamWaitEvent(e->stream, sl.h2d_done, 0));
    if (sl.used) GT_CUDA(cudaStreamWaitEvent(e->stream, sl.d2h_done, 0));
    rc = backward_group_device(e, n, w, ad, dYd, x_kept ? x_kept : (need_x ? (const float *)sl.in[kSlotIn - 1].p : nullptr),
                               dX ? (float *)sl.out[0].p : nullptr, T, flags);
    if (rc != GT_OK) return rc;
    GT_CUDA(cudaEventRecord(sl.compute_done, e->stream));
    GT_CUDA(cudaStreamWaitEvent(e->s_d2h, sl.compute_done, 0));
    if (dX) GT_CUDA(cudaMemcpyAsync(dX, sl.out[0].p, bx, cudaMemcpyDeviceToHost, e->s_d2h));
    GT_CUDA(cudaEventRecord(sl.d2h_done, e->s_d2h));
    sl.used = true;
    return finish_host_call(e, flags);
}

}  // namespace

namespace gt {
bool pdl_enabled() {
    static const bool on = [] {
        // on unless GT_PDL=0.  Nothing on the seven projections alone (a GEMM CTA holds the whole shared memory, so a
        // dependent CTA cannot become resident early), 2 ms of the 28-layer training step, whose ~1000 short kernels
        // between the GEMMs otherwise pay a launch gap each.
        const char *v = getenv("GT_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}
EngineView engine_view(gt_engine *e) { return EngineView{e->device, e->math_mode, e->sm_count, e->stream, e->status, &e->mu}; }
const WeightDev *weight_view(const gt_weight *w) { return &w->dev; }
int set_last_error(int code, const char *text) { return fail(code, "%s", text); }
int engine_join_comm(gt_engine *e) { return join_comm(e); }
}  // namespace gt

extern "C" {

const char *gt_last_error(void) { return g_err; }

int gt_set_logger(gt_log_fn fn, void *user) {
    std::lock_guard<std::mutex> lk(g_log_mu);
    g_log_fn = fn;
    g_log_user = user;
    return GT_OK;
}
const char *gt_version(void) { return "glaciertune_b200 0.1 (sm_100a)"; }

int gt_supports(int ggml_type, int direction) {
    if (direction != GT_DIR_FORWARD && direction != GT_DIR_BACKWARD) return 0;
    // Q4_0 and Q8_0 (the reference's other Supports*Gemm types) run on the exact CUDA-core kernels in every math mode
    return (ggml_type == GT_TYPE_Q4_K || ggml_type == GT_TYPE_Q6_K || ggml_type == GT_TYPE_F32 || ggml_type == GT_TYPE_F16 ||
            ggml_type == GT_TYPE_Q4_0 || ggml_type == GT_TYPE_Q8_0) ? 1 : 0;
}

int gt_engine_create(const gt_config *cfg, gt_engine **out) {
    if (!out) return fail(GT_ERR_INVALID, "gt_engine_create: out is null");
    *out = nullptr;
    const int dev = cfg ? cfg->device : 0;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return fail(GT_ERR_NO_DEVICE, "no CUDA device is visible; this library has no CPU path");
    }
    if (dev < 0 || dev >= count) return fail(GT_ERR_INVALID, "device ordinal %d out of range (%d devices)", dev, count);
    cudaDeviceProp prop;
    GT_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) return fail(GT_ERR_NO_DEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only", dev, prop.major, prop.minor);
    GT_CUDA(cudaSetDevice(dev));
    if (!umma_available()) return fail(GT_ERR_CUDA, "the CUDA driver does not export cuTensorMapEncodeTiled");
    gt_engine *e = new (std::nothrow) gt_engine();
    if (!e) return fail(GT_ERR_OOM, "out of host memory");
    e->device = dev;
    e->sm_count = prop.multiProcessorCount;
    e->math_mode = cfg ? cfg->math_mode : GT_MATH_BF16;
    if (e->math_mode < GT_MATH_BF16 || e->math_mode > GT_MATH_FP32) {
        delete e;
        return fail(GT_ERR_INVALID, "unknown math mode %d", cfg->math_mode);
    }
    if (cfg && cfg->stream) {
        e->stream = (cudaStream_t)cfg->stream;
    } else {
        cudaError_t ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
        if (ce != cudaSuccess) {
            delete e;
            return fail(GT_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(ce));
        }
        e->own_stream = true;
    }
    cudaError_t ce = cudaMalloc((void **)&e->status, 4 * sizeof(int));
    if (ce == cudaSuccess) ce = cudaMalloc((void **)&e->clip, 2 * sizeof(double));
    if (ce == cudaSuccess && aux_init(e) != GT_OK) ce = cudaErrorUnknown;      // side stream of the dA passes
    // scratch sized up front, so that no projection call of up to max_tokens tokens on tensors of up to max_features
    // input / output features allocates (a group's outputs together count as one tensor: q | k | v, gate | up)
    e->max_tokens = (cfg && cfg->max_tokens > 0) ? cfg->max_tokens : 0;
    if (ce == cudaSuccess && cfg && cfg->max_tokens > 0 && cfg->max_features > 0) {
        const size_t T = (size_t)cfg->max_tokens, F = (size_t)cfg->max_features;
        ce = e->x16.reserve(T * F * 2);
        if (ce == cudaSuccess) ce = e->dy16.reserve(T * (F + 64) * 2 + 3 * 256);
        for (int i = 0; i < 3 && ce == cudaSuccess; i++) ce = e->ffn[i].reserve(T * F * sizeof(float));
        if (ce == cudaSuccess) logf(GT_LOG_INFO, "engine on device %d: scratch reserved for %zu tokens x %zu features (%.1f MB)", dev, T, F,
                                    (double)(e->x16.cap + e->dy16.cap + 3 * e->ffn[0].cap) / 1e6);
    }
    if (ce == cudaSuccess) ce = cudaMemset(e->status, 0, 4 * sizeof(int));
    if (ce != cudaSuccess) {
        gt_engine_destroy(e);
        return fail(GT_ERR_CUDA, "engine allocation failed: %s", cudaGetErrorString(ce));
    }
    *out = e;
    return GT_OK;
}

int gt_engine_destroy(gt_engine *e) {
    if (!e) return GT_OK;
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    if (e->s_h2d) cudaStreamSynchronize(e->s_h2d);
    if (e->s_d2h) cudaStreamSynchronize(e->s_d2h);
    Scratch *all[] = {&e->x16, &e->dy16, &e->dlow, &e->ytmp, &e->pair_tmp, &e->ffn[0], &e->ffn[1], &e->ffn[2], &e->ce, &e->ce_host, &e->attn};
    for (Scratch *s : all) s->release();
    for (HostSlot &sl : e->slots) {
        for (Scratch &b : sl.in) b.release();
        for (Scratch &b : sl.out) b.release();
        if (sl.h2d_done) cudaEventDestroy(sl.h2d_done);
        if (sl.compute_done) cudaEventDestroy(sl.compute_done);
        if (sl.d2h_done) cudaEventDestroy(sl.d2h_done);
    }
    if (e->s_comm) {
        cudaStreamSynchronize(e->s_comm);
        cudaStreamDestroy(e->s_comm);
    }
    if (e->s_aux) {
        cudaStreamSynchronize(e->s_aux);
        cudaStreamDestroy(e->s_aux);
    }
    if (e->ev_aux_fork) cudaEventDestroy(e->ev_aux_fork);
    if (e->ev_aux_join) cudaEventDestroy(e->ev_aux_join);
    if (e->ev_fork) cudaEventDestroy(e->ev_fork);
    if (e->ev_join) cudaEventDestroy(e->ev_join);
    if (e->s_h2d) cudaStreamDestroy(e->s_h2d);
    if (e->s_d2h) cudaStreamDestroy(e->s_d2h);
    if (e->status) cudaFree(e->status);
    if (e->clip) cudaFree(e->clip);
    for (cudaEvent_t ev : e->ev_pool) cudaEventDestroy(ev);
    if (e->own_stream && e->stream) cudaStreamDestroy(e->stream);
    delete e;
    return GT_OK;
}

int gt_engine_set_math_mode(gt_engine *e, int math_mode) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    if (math_mode < GT_MATH_BF16 || math_mode > GT_MATH_FP32) return fail(GT_ERR_INVALID, "unknown math mode %d", math_mode);
    std::lock_guard<std::mutex> lk(e->mu);
    e->math_mode = math_mode;
    return GT_OK;
}

int gt_sync(gt_engine *e) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    int rc = join_comm(e);                                     // collectives begun on the side stream
    if (rc != GT_OK) return rc;
    rc = check_status(e);                                      // drains the engine stream
    if (e->s_d2h) GT_CUDA(cudaStreamSynchronize(e->s_d2h));      // and the downloads of asynchronous host-buffer calls
    return rc;
}

int gt_debug_wait_selftest(gt_engine *e, int64_t limit_cycles) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    if (limit_cycles <= 0 || limit_cycles > 2000000000ll) return fail(GT_ERR_INVALID, "limit must be in (0, 2e9] cycles");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    GT_CUDA(launch_bounded_wait_selftest(e->status, limit_cycles, e->stream));
    return check_status(e);       // expected: GT_ERR_KERNEL carrying code 999
}

int gt_debug_set_trace(gt_engine *e, void *dev_buf) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    e->trace = dev_buf;
    return GT_OK;
}

int gt_profile_enable(gt_engine *e, int on) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    e->profile = on != 0;
    return GT_OK;
}

int gt_profile_read(gt_engine *e, double *gemm_ms, int64_t *gemm_launches, double *gemm_flops, int64_t *kernel_launches,
                    int reset) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    double ms = 0.0;
    for (size_t i = 0; i + 1 < e->ev_used; i += 2) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, e->ev_pool[i], e->ev_pool[i + 1]) == cudaSuccess) ms += t;
    }
    cudaGetLastError();
    if (gemm_ms) *gemm_ms = ms;
    if (gemm_launches) *gemm_launches = e->gemm_launches;
    if (gemm_flops) *gemm_flops = e->gemm_flops;
    if (kernel_launches) *kernel_launches = e->kernel_launches;
    if (reset) {
        e->ev_used = 0;
        e->gemm_launches = 0;
        e->kernel_launches = 0;
        e->gemm_flops = 0.0;
    }
    return GT_OK;
}

int gt_weight_upload(gt_engine *e, int ggml_type, const void *host_bytes, int64_t nbytes, int32_t out_features,
                     int32_t in_features, const float *bias, gt_weight **out) {
    if (!e || !host_bytes || !out) return fail(GT_ERR_INVALID, "gt_weight_upload: null argument");
    *out = nullptr;
    if (!gt_supports(ggml_type, GT_DIR_FORWARD)) return fail(GT_ERR_UNSUPPORTED, "ggml type %d is not supported", ggml_type);
    if (out_features <= 0 || in_features <= 0) return fail(GT_ERR_INVALID, "bad shape [%d, %d]", out_features, in_features);
    const int64_t nelem = (int64_t)out_features * in_features;
    int64_t expect;
    if (ggml_type == GT_TYPE_F32) {
        expect = nelem * 4;
    } else if (ggml_type == GT_TYPE_F16) {
        expect = nelem * 2;
    } else if (ggml_type == GT_TYPE_Q4_0 || ggml_type == GT_TYPE_Q8_0) {
        if (in_features % 32 != 0)
            return fail(GT_ERR_INVALID, "tensor [%d, %d] is not a whole number of 32-weight blocks per row", out_features, in_features);
        expect = nelem / 32 * (ggml_type == GT_TYPE_Q4_0 ? kQ40BlockBytes : kQ80BlockBytes);
    } else {
        if (nelem % 256 != 0 || in_features % 32 != 0)
            return fail(GT_ERR_INVALID, "K-quant tensor [%d, %d] is not a whole number of 256-weight super-blocks", out_features,
                        in_features);
        expect = nelem / 256 * (ggml_type == GT_TYPE_Q4_K ? kQ4KBlockBytes : kQ6KGgufBlockBytes);
    }
    if (nbytes != expect) return fail(GT_ERR_INVALID, "tensor byte size %lld does not match shape (expected %lld)", (long long)nbytes, (long long)expect);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    gt_weight *w = new (std::nothrow) gt_weight();
    if (!w) return fail(GT_ERR_OOM, "out of host memory");
    w->eng = e;
    WeightDev &d = w->dev;
    d.qtype = ggml_type;
    d.N = out_features;
    d.K = in_features;
    cudaError_t ce = cudaSuccess;
    if (ggml_type == GT_TYPE_Q6_K) {
        const int64_t nb = nelem / 256;
        d.nbytes = nb * kQ6KDevBlockBytes;
        void *tmp = nullptr;
        ce = cudaMalloc((void **)&d.data, d.nbytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&tmp, nbytes);
        if (ce == cudaSuccess) ce = cudaMemcpyAsync(tmp, host_bytes, nbytes, cudaMemcpyHostToDevice, e->stream);
        if (ce == cudaSuccess) ce = launch_q6k_repack((const uint8_t *)tmp, d.data, nb, e->stream);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
        if (tmp) cudaFree(tmp);
    } else {
        d.nbytes = nbytes;
        ce = cudaMalloc((void **)&d.data, d.nbytes);
        if (ce == cudaSuccess) ce = cudaMemcpyAsync(d.data, host_bytes, nbytes, cudaMemcpyHostToDevice, e->stream);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    }
    if (ce == cudaSuccess && bias) {
        ce = cudaMalloc((void **)&d.bias, (size_t)out_features * sizeof(float));
        if (ce == cudaSuccess) ce = cudaMemcpy(d.bias, bias, (size_t)out_features * sizeof(float), cudaMemcpyHostToDevice);
    }
    if (ce != cudaSuccess) {
        gt_weight_free(w);
        return fail(ce == cudaErrorMemoryAllocation ? GT_ERR_OOM : GT_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(ce));
    }
    if (ggml_type == GT_TYPE_F16) d.row_bytes = (int64_t)in_features * 2;
    else if ((ggml_type == GT_TYPE_Q4_K || ggml_type == GT_TYPE_Q6_K) && in_features % 256 == 0)
        d.row_bytes = (int64_t)(in_features / 256) * dev_block_bytes(ggml_type);
    const char *msg = nullptr;
    if (umma_init_weight_maps(&d, &msg) != cudaSuccess) {
        gt_weight_free(w);
        return fail(GT_ERR_CUDA, "%s", msg ? msg : "tensor map creation failed");
    }
    if (!d.tma_ok && (ggml_type == GT_TYPE_Q4_K || ggml_type == GT_TYPE_Q6_K) && in_features % 256 == 128 && out_features % 2 == 0) {
        WeightDev &v = w->paired;
        v = d;
        v.bias = nullptr;
        v.N = out_features / 2;
        v.K = 2 * in_features;
        v.row_bytes = (int64_t)(v.K / 256) * dev_block_bytes(ggml_type);
        const char *pm = nullptr;
        w->has_paired = umma_init_weight_maps(&v, &pm) == cudaSuccess && v.tma_ok;
    }
    logf(GT_LOG_DEBUG, "weight [%d, %d] type %d uploaded: %.2f MB on device %d%s", out_features, in_features, ggml_type, (double)d.nbytes / 1e6,
         e->device, d.tma_ok ? "" : (w->has_paired ? " (tensor path through the paired-row view)" : " (CUDA-core path only)"));
    *out = w;
    return GT_OK;
}

int gt_weight_free(gt_weight *w) {
    if (!w) return GT_OK;
    if (w->eng) cudaSetDevice(w->eng->device);
    if (w->dev.data) cudaFree(w->dev.data);
    if (w->dev.bias) cudaFree(w->dev.bias);
    delete w;
    return GT_OK;
}

int gt_dequant_rows(gt_engine *e, const gt_weight *w, int64_t row0, int64_t nrows, float *out, int32_t flags) {
    if (!e || !w || !out) return fail(GT_ERR_INVALID, "gt_dequant_rows: null argument");
    if (row0 < 0 || nrows < 0 || row0 + nrows > w->dev.N) return fail(GT_ERR_INVALID, "rows [%lld, %lld) outside [0, %d)", (long long)row0, (long long)(row0 + nrows), w->dev.N);
    if (nrows == 0) return GT_OK;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    const size_t bytes = (size_t)nrows * w->dev.K * sizeof(float);
    float *dst = out;
    if (!(flags & GT_FLAG_DEVICE_PTRS)) {
        GT_CUDA(e->ytmp.reserve(bytes));
        dst = (float *)e->ytmp.p;
    }
    GT_CUDA(launch_dequant_rows(w->dev.qtype, w->dev.data, w->dev.K, row0, nrows, dst, e->stream));
    if (!(flags & GT_FLAG_DEVICE_PTRS)) {
        GT_CUDA(cudaMemcpyAsync(out, dst, bytes, cudaMemcpyDeviceToHost, e->stream));
        GT_CUDA(cudaStreamSynchronize(e->stream));
    }
    return GT_OK;
}

int gt_adapter_create(gt_engine *e, int32_t in_features, int32_t out_features, int32_t rank, float alpha, gt_adapter **out) {
    if (!e || !out) return fail(GT_ERR_INVALID, "gt_adapter_create: null argument");
    *out = nullptr;
    if (in_features <= 0 || out_features <= 0 || rank <= 0) return fail(GT_ERR_INVALID, "bad adapter shape in=%d out=%d rank=%d", in_features, out_features, rank);
    if (rank > 64) return fail(GT_ERR_UNSUPPORTED, "rank %d > 64 is not supported", rank);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    gt_adapter *a = new (std::nothrow) gt_adapter();
    if (!a) return fail(GT_ERR_OOM, "out of host memory");
    a->eng = e;
    a->in = in_features;
    a->out = out_features;
    a->rank = rank;
    a->alpha = alpha;
    a->scaling = alpha / (float)rank;   // LoraAdapter.cs:99
    const size_t na = (size_t)in_features * rank * sizeof(float), nb = (size_t)rank * out_features * sizeof(float);
    cudaError_t ce = cudaMalloc((void **)&a->A, na);
    if (ce == cudaSuccess) ce = cudaMalloc((void **)&a->B, nb);
    if (ce == cudaSuccess) ce = cudaMalloc((void **)&a->dA, na);
    if (ce == cudaSuccess) ce = cudaMalloc((void **)&a->dB, nb);
    if (ce == cudaSuccess) ce = cudaMalloc((void **)&a->b_nonzero, sizeof(int));
    if (ce == cudaSuccess) ce = cudaMemsetAsync(a->A, 0, na, e->stream);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(a->B, 0, nb, e->stream);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(a->dA, 0, na, e->stream);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(a->dB, 0, nb, e->stream);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(a->b_nonzero, 0, sizeof(int), e->stream);
    if (ce == cudaSuccess && e->max_tokens > 0) ce = a->low.reserve(2 * low_bytes(a, e->max_tokens));      // X*A | dY*B^T of a step
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    if (ce != cudaSuccess) {
        gt_adapter_free(a);
        return fail(GT_ERR_CUDA, "adapter allocation failed: %s", cudaGetErrorString(ce));
    }
    *out = a;
    return GT_OK;
}

int gt_adapter_free(gt_adapter *a) {
    if (!a) return GT_OK;
    if (a->eng) cudaSetDevice(a->eng->device);
    if (a->A) cudaFree(a->A);
    if (a->B) cudaFree(a->B);
    if (a->own_grads) {
        if (a->dA) cudaFree(a->dA);
        if (a->dB) cudaFree(a->dB);
    }
    if (a->b_nonzero) cudaFree(a->b_nonzero);
    a->low.release();
    a->xkeep.release();
    a->moments.release();
    delete a;
    return GT_OK;
}

int gt_adapter_upload(gt_adapter *a, const float *A, const float *B) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    gt_engine *e = a->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (A) GT_CUDA(cudaMemcpyAsync(a->A, A, (size_t)a->in * a->rank * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    if (B) {
        GT_CUDA(cudaMemcpyAsync(a->B, B, (size_t)a->rank * a->out * sizeof(float), cudaMemcpyHostToDevice, e->stream));
        GT_CUDA(launch_any_nonzero(a->B, (int64_t)a->rank * a->out, a->b_nonzero, e->stream));
    }
    GT_CUDA(cudaStreamSynchronize(e->stream));
    return GT_OK;
}

int gt_adapter_download(gt_adapter *a, float *A, float *B) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    gt_engine *e = a->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (A) GT_CUDA(cudaMemcpyAsync(A, a->A, (size_t)a->in * a->rank * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    if (B) GT_CUDA(cudaMemcpyAsync(B, a->B, (size_t)a->rank * a->out * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    return GT_OK;
}

int gt_adapter_grads_download(gt_adapter *a, float *dA, float *dB) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    gt_engine *e = a->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (dA) GT_CUDA(cudaMemcpyAsync(dA, a->dA, (size_t)a->in * a->rank * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    if (dB) GT_CUDA(cudaMemcpyAsync(dB, a->dB, (size_t)a->rank * a->out * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    return GT_OK;
}

int gt_adapter_grads_zero(gt_adapter *a) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    gt_engine *e = a->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    GT_CUDA(cudaMemsetAsync(a->dA, 0, (size_t)a->in * a->rank * sizeof(float), e->stream));
    GT_CUDA(cudaMemsetAsync(a->dB, 0, (size_t)a->rank * a->out * sizeof(float), e->stream));
    return GT_OK;
}

int gt_adapters_adamw_step(gt_engine *e, int32_t n, gt_adapter *const *ads, float lr, float beta1, float beta2, float eps,
                           float weight_decay, int32_t step) {
    if (!e || (n > 0 && !ads)) return fail(GT_ERR_INVALID, "gt_adapters_adamw_step: null argument");
    if (step < 1) return fail(GT_ERR_INVALID, "gt_adapters_adamw_step: step counts from 1 (got %d)", step);
    if (!(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f))
        return fail(GT_ERR_INVALID, "gt_adapters_adamw_step: beta1 and beta2 must lie in [0, 1)");
    for (int i = 0; i < n; i++) {
        if (!ads[i]) return fail(GT_ERR_INVALID, "gt_adapters_adamw_step: adapter %d is null", i);
        if (ads[i]->eng != e) return fail(GT_ERR_INVALID, "gt_adapters_adamw_step: adapter %d belongs to another engine", i);
    }
    if (n <= 0) return GT_OK;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    int jrc = join_comm(e);      // the update reads gradients that a pending exchange may still be writing
    if (jrc != GT_OK) return jrc;
    std::vector<gt::AdamwSeg> segs;
    segs.reserve((size_t)2 * n);
    for (int i = 0; i < n; i++) {
        gt_adapter *a = ads[i];
        const int64_t na = (int64_t)a->in * a->rank, nb = (int64_t)a->rank * a->out;
        const int64_t na_pad = (na + 3) & ~(int64_t)3, nb_pad = (nb + 3) & ~(int64_t)3;      // keeps every segment 16-byte aligned
        if (!a->moments.p) {
            const size_t bytes = (size_t)(2 * na_pad + 2 * nb_pad) * sizeof(float);
            GT_CUDA(a->moments.reserve(bytes));
            GT_CUDA(cudaMemsetAsync(a->moments.p, 0, bytes, e->stream));
        }
        float *mA = static_cast<float *>(a->moments.p), *vA = mA + na_pad, *mB = vA + na_pad, *vB = mB + nb_pad;
        segs.push_back(gt::AdamwSeg{a->A, a->dA, mA, vA, nullptr, na, 0});
        segs.push_back(gt::AdamwSeg{a->B, a->dB, mB, vB, a->b_nonzero, nb, 0});     // B may leave zero: raise the delta's flag
    }
    GT_CUDA(gt::launch_adamw(segs.data(), (int)segs.size(), lr, beta1, beta2, eps, weight_decay, (int)step, e->sm_count, e->stream));
    return GT_OK;
}

int gt_adapter_adamw_step(gt_adapter *a, float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    return gt_adapters_adamw_step(a->eng, 1, &a, lr, beta1, beta2, eps, weight_decay, step);
}

int gt_adapter_set_alpha(gt_adapter *a, float alpha) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    std::lock_guard<std::mutex> lk(a->eng->mu);
    a->alpha = alpha;
    a->scaling = a->rank > 0 ? alpha / (float)a->rank : 0.f;
    return GT_OK;
}

int gt_adapter_device_ptrs(gt_adapter *a, float **A, float **B, float **dA, float **dB) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    if (A) *A = a->A;
    if (dA) *dA = a->dA;
    if (dB) *dB = a->dB;
    if (B) {
        // The caller may now write B behind the library's back (a resident optimizer): the "B is all zero" flag that
        // lets the forward skip the adapter term can no longer be trusted, so it is raised (a stale 1 costs arithmetic,
        // never correctness).  gt_adapter_params_changed() recomputes it from the values.
        gt_engine *e = a->eng;
        std::lock_guard<std::mutex> lk(e->mu);
        GT_CUDA(cudaSetDevice(e->device));
        GT_CUDA(cudaMemsetAsync(a->b_nonzero, 1, sizeof(int), e->stream));      // 0x01010101: non-zero
        *B = a->B;
    }
    return GT_OK;
}

int gt_adapter_params_changed(gt_adapter *a) {
    if (!a) return fail(GT_ERR_INVALID, "adapter is null");
    gt_engine *e = a->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    GT_CUDA(launch_any_nonzero(a->B, (int64_t)a->rank * a->out, a->b_nonzero, e->stream));
    a->low_T = 0;        // X*A kept from an earlier forward was computed with the old A
    a->xkeep_T = 0;
    return GT_OK;
}

int gt_adapter_bind_grads(gt_adapter *a, float *dA_dev, float *dB_dev) {
    if (!a || !dA_dev || !dB_dev) return fail(GT_ERR_INVALID, "gt_adapter_bind_grads: null argument");
    std::lock_guard<std::mutex> lk(a->eng->mu);
    cudaSetDevice(a->eng->device);
    if (a->own_grads) {
        cudaStreamSynchronize(a->eng->stream);
        if (a->dA) cudaFree(a->dA);
        if (a->dB) cudaFree(a->dB);
    }
    a->own_grads = false;
    gt::layout_generation().fetch_add(1);
    a->dA = dA_dev;
    a->dB = dB_dev;
    return GT_OK;
}

int gt_proj_forward(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *X, float *Y, int32_t T, int32_t flags) {
    if (!e || !w || !X || !Y) return fail(GT_ERR_INVALID, "gt_proj_forward: null argument");
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    if (ad && (ad->in != w->dev.K || ad->out != w->dev.N)) return fail(GT_ERR_INVALID, "adapter [%d -> %d] does not match weight [%d -> %d]", ad->in, ad->out, w->dev.K, w->dev.N);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    // LoraAdapter.Forward: the delta is skipped when the adapter is disabled, scaling == 0, or B == 0
    // (B == 0 is decided on the device from the flag written at upload).
    if (flags & GT_FLAG_DEVICE_PTRS) {
        const bool use_lora = ad && !(flags & GT_FLAG_NO_LORA) && ad->rank > 0 && ad->scaling != 0.f;
        return forward_device(e, w, ad, X, Y, T, use_lora);
    }
    return forward_host(e, 1, &w, &ad, X, &Y, T, flags);
}

int gt_proj_backward(gt_engine *e, const gt_weight *w, gt_adapter *ad, const float *dY, const float *X, float *dX, int32_t T,
                     int32_t flags) {
    if (!e || !w || !dY) return fail(GT_ERR_INVALID, "gt_proj_backward: null argument");
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    if (ad && (ad->in != w->dev.K || ad->out != w->dev.N)) return fail(GT_ERR_INVALID, "adapter [%d -> %d] does not match weight [%d -> %d]", ad->in, ad->out, w->dev.K, w->dev.N);
    const bool use_lora = ad && !(flags & GT_FLAG_NO_LORA) && ad->rank > 0;
    if (use_lora && !X) return fail(GT_ERR_INVALID, "gt_proj_backward: X is required for the adapter gradients");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    const bool assign = (flags & GT_FLAG_DX_ASSIGN) != 0;
    if (flags & GT_FLAG_DEVICE_PTRS) return backward_device(e, w, ad, dY, X, dX, T, use_lora, (flags & GT_FLAG_REUSE_LOW) != 0, assign);
    return backward_host(e, 1, &w, &ad, &dY, X, dX, T, flags);
}

int gt_stream_max_tokens(void) { return stream_max_tokens(); }

namespace {
int check_ffn(const gt_weight *wg, const gt_weight *wu, const gt_weight *wd, gt_adapter *const *ad, const char *who) {
    if (!wg || !wu || !wd) return fail(GT_ERR_INVALID, "%s: null weight", who);
    if (wg->dev.N != wu->dev.N || wg->dev.K != wu->dev.K)
        return fail(GT_ERR_INVALID, "%s: gate [%d x %d] and up [%d x %d] differ in shape", who, wg->dev.N, wg->dev.K, wu->dev.N, wu->dev.K);
    if (wd->dev.K != wg->dev.N || wd->dev.N != wg->dev.K)
        return fail(GT_ERR_INVALID, "%s: down is [%d x %d], expected [%d x %d]", who, wd->dev.N, wd->dev.K, wg->dev.K, wg->dev.N);
    const gt_weight *w[3] = {wg, wu, wd};
    for (int j = 0; ad && j < 3; j++)
        if (ad[j] && (ad[j]->in != w[j]->dev.K || ad[j]->out != w[j]->dev.N)) return fail(GT_ERR_INVALID, "%s: adapter %d does not match its weight", who, j);
    return GT_OK;
}
}  // namespace

int gt_ffn_forward(gt_engine *e, const gt_weight *w_gate, const gt_weight *w_up, const gt_weight *w_down, gt_adapter *const *adapters,
                   const float *X, float *out_gate, float *out_up, float *out_hidden, float *out_down, int32_t T, int32_t flags) {
    if (!e || !X || !out_down) return fail(GT_ERR_INVALID, "gt_ffn_forward: null argument");
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    int rc = check_ffn(w_gate, w_up, w_down, adapters, "gt_ffn_forward");
    if (rc != GT_OK) return rc;
    const gt_weight *w[3] = {w_gate, w_up, w_down};
    gt_adapter *ad[3] = {adapters ? adapters[0] : nullptr, adapters ? adapters[1] : nullptr, adapters ? adapters[2] : nullptr};
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (flags & GT_FLAG_DEVICE_PTRS) return ffn_forward_device(e, w, ad, X, out_gate, out_up, out_hidden, out_down, T, flags);
    // host buffers: X goes up once, the intermediate tensors stay on the device; only the outputs that were asked for
    // come back (the reference moves gate, up and hidden across PCIe up to five times per layer)
    rc = host_pipeline_init(e);
    if (rc != GT_OK) return rc;
    HostSlot &sl = next_slot(e);
    const int H = w_gate->dev.K, F = w_gate->dev.N;
    const size_t bx = (size_t)T * H * sizeof(float), bf = (size_t)T * F * sizeof(float);
    GT_CUDA(sl.in[0].reserve(bx));
    GT_CUDA(sl.out[0].reserve(bx));
    float *host_out[3] = {out_gate, out_up, out_hidden};
    float *dev_out[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < 3; i++) {
        if (host_out[i]) {
            GT_CUDA(sl.out[1 + i].reserve(bf));
            dev_out[i] = (float *)sl.out[1 + i].p;
        }
    }
    if (sl.used) GT_CUDA(cudaStreamWaitEvent(e->s_h2d, sl.compute_done, 0));
    GT_CUDA(cudaMemcpyAsync(sl.in[0].p, X, bx, cudaMemcpyHostToDevice, e->s_h2d));
    GT_CUDA(cudaEventRecord(sl.h2d_done, e->s_h2d));
    GT_CUDA(cudaStreamWaitEvent(e->stream, sl.h2d_done, 0));
    if (sl.used) GT_CUDA(cudaStreamWaitEvent(e->stream, sl.d2h_done, 0));
    rc = ffn_forward_device(e, w, ad, (const float *)sl.in[0].p, dev_out[0], dev_out[1], dev_out[2], (float *)sl.out[0].p, T, flags);
    if (rc != GT_OK) return rc;
    GT_CUDA(cudaEventRecord(sl.compute_done, e->stream));
    GT_CUDA(cudaStreamWaitEvent(e->s_d2h, sl.compute_done, 0));
    GT_CUDA(cudaMemcpyAsync(out_down, sl.out[0].p, bx, cudaMemcpyDeviceToHost, e->s_d2h));
    for (int i = 0; i < 3; i++)
        if (host_out[i]) GT_CUDA(cudaMemcpyAsync(host_out[i], dev_out[i], bf, cudaMemcpyDeviceToHost, e->s_d2h));
    GT_CUDA(cudaEventRecord(sl.d2h_done, e->s_d2h));
    sl.used = true;
    return finish_host_call(e, flags);
}

int gt_ffn_backward(gt_engine *e, const gt_weight *w_gate, const gt_weight *w_up, const gt_weight *w_down, gt_adapter *const *adapters,
                    const float *dY, const float *X, const float *gate, const float *up, const float *hidden, float *dX, int32_t T,
                    int32_t flags) {
    if (!e || !dY || !gate || !up || !dX) return fail(GT_ERR_INVALID, "gt_ffn_backward: null argument");
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    if (!(flags & GT_FLAG_DEVICE_PTRS)) return fail(GT_ERR_UNSUPPORTED, "gt_ffn_backward takes device tensors (GT_FLAG_DEVICE_PTRS)");
    int rc = check_ffn(w_gate, w_up, w_down, adapters, "gt_ffn_backward");
    if (rc != GT_OK) return rc;
    const gt_weight *w[3] = {w_gate, w_up, w_down};
    gt_adapter *ad[3] = {adapters ? adapters[0] : nullptr, adapters ? adapters[1] : nullptr, adapters ? adapters[2] : nullptr};
    const bool lora = !(flags & GT_FLAG_NO_LORA);
    if (lora && ((ad[0] || ad[1]) && !X)) return fail(GT_ERR_INVALID, "gt_ffn_backward: X is required for the gate / up adapter gradients");
    if (lora && ad[2] && !hidden) return fail(GT_ERR_INVALID, "gt_ffn_backward: hidden is required for the down adapter gradients");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return ffn_backward_device(e, w, ad, dY, X, gate, up, hidden, dX, T, flags);
}

int gt_proj_forward_group(gt_engine *e, int32_t n, const gt_weight *const *w, gt_adapter *const *ad, const float *X, float *const *Y,
                          int32_t T, int32_t flags) {
    if (!e || !w || !X || !Y) return fail(GT_ERR_INVALID, "gt_proj_forward_group: null argument");
    if (n < 1 || n > kMaxGroup) return fail(GT_ERR_INVALID, "a group holds 1 to %d projections (got %d)", kMaxGroup, n);
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    for (int j = 0; j < n; j++) {
        if (!w[j] || !Y[j]) return fail(GT_ERR_INVALID, "gt_proj_forward_group: member %d is null", j);
        if (w[j]->dev.K != w[0]->dev.K) return fail(GT_ERR_INVALID, "members of a group share their input: in_features %d vs %d", w[j]->dev.K, w[0]->dev.K);
        if (ad && ad[j] && (ad[j]->in != w[j]->dev.K || ad[j]->out != w[j]->dev.N)) return fail(GT_ERR_INVALID, "adapter %d does not match its weight", j);
    }
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (!(flags & GT_FLAG_DEVICE_PTRS)) return forward_host(e, n, w, ad, X, Y, T, flags);
    return forward_group_device(e, n, w, ad, X, Y, T, flags);
}

int gt_proj_backward_group(gt_engine *e, int32_t n, const gt_weight *const *w, gt_adapter *const *ad, const float *const *dY,
                           const float *X, float *dX, int32_t T, int32_t flags) {
    if (!e || !w || !dY) return fail(GT_ERR_INVALID, "gt_proj_backward_group: null argument");
    if (n < 1 || n > kMaxGroup) return fail(GT_ERR_INVALID, "a group holds 1 to %d projections (got %d)", kMaxGroup, n);
    if (T <= 0) return fail(GT_ERR_INVALID, "T must be positive (got %d)", T);
    for (int j = 0; j < n; j++) {
        if (!w[j] || !dY[j]) return fail(GT_ERR_INVALID, "gt_proj_backward_group: member %d is null", j);
        if (w[j]->dev.K != w[0]->dev.K) return fail(GT_ERR_INVALID, "members of a group share their input: in_features %d vs %d", w[j]->dev.K, w[0]->dev.K);
        if (ad && ad[j] && (ad[j]->in != w[j]->dev.K || ad[j]->out != w[j]->dev.N)) return fail(GT_ERR_INVALID, "adapter %d does not match its weight", j);
        if (ad && ad[j] && !(flags & GT_FLAG_NO_LORA) && !X) return fail(GT_ERR_INVALID, "gt_proj_backward_group: X is required for the adapter gradients");
    }
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (!(flags & GT_FLAG_DEVICE_PTRS)) return backward_host(e, n, w, ad, dY, X, dX, T, flags);
    return backward_group_device(e, n, w, ad, dY, X, dX, T, flags);
}

int gt_launch_gemm_batch(gt_engine *e, const gt_weight *w, float *dY_out, const float *dX_in, int32_t batch, float *d_residual) {
    if (!e || !w || !dX_in) return fail(GT_ERR_INVALID, "gt_launch_gemm_batch: null argument");
    if (batch <= 0) return fail(GT_ERR_INVALID, "batch must be positive (got %d)", batch);
    if (!dY_out && !d_residual) return GT_OK;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    const int N = w->dev.N, K = w->dev.K;
    if (!tensor_path(e, w)) {
        GT_CUDA(launch_gemm_fp32_fwd(w->dev.qtype, w->dev.data, dX_in, dY_out, d_residual, w->dev.bias, batch, N, K, e->stream));
        return GT_OK;
    }
    float *yd = dY_out;
    if (!yd) {
        GT_CUDA(e->ytmp.reserve((size_t)batch * N * sizeof(float)));
        yd = (float *)e->ytmp.p;
    }
    int rc = forward_device(e, w, nullptr, dX_in, yd, batch, false);
    if (rc != GT_OK) return rc;
    if (d_residual) GT_CUDA(launch_add_inplace(d_residual, yd, (int64_t)batch * N, e->stream));
    return GT_OK;
}

int gt_launch_gemm_bwd(gt_engine *e, const gt_weight *w, float *dDX, const float *dDY, int32_t batch) {
    if (!e || !w || !dDX || !dDY) return fail(GT_ERR_INVALID, "gt_launch_gemm_bwd: null argument");
    if (batch <= 0) return fail(GT_ERR_INVALID, "batch must be positive (got %d)", batch);
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return backward_device(e, w, nullptr, dDY, nullptr, dDX, batch, false, false, false);
}

int gt_grads_scale_clip(gt_engine *e, float *g_dev, int64_t n, float pre_scale, double max_norm, double *norm_out) {
    if (!e || !g_dev || n < 0) return fail(GT_ERR_INVALID, "gt_grads_scale_clip: bad argument");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    int jrc = join_comm(e);      // gradient slices still being exchanged on the side stream come first
    if (jrc != GT_OK) return jrc;
    GT_CUDA(launch_scale_clip(g_dev, n, pre_scale, max_norm, e->clip, e->stream));
    double h[2] = {0, 0};
    GT_CUDA(cudaMemcpyAsync(h, e->clip, sizeof(h), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    if (norm_out) *norm_out = max_norm > 0.0 ? h[1] : 0.0;   // ClipGradients returns 0 when maxNorm <= 0
    return GT_OK;
}

// ------------------------------------------------------------------------------------------------
// Data parallel: one process per GPU, every rank holds a replica of the frozen base and of the adapters;
// the flat fp32 LoRA-gradient buffer is summed over NVLink with one NCCL all-reduce per step.
// NCCL is bound at run time (dlopen) so the library loads on hosts without it.
// ------------------------------------------------------------------------------------------------
namespace {
struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
NcclApi &nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) {
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
            api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
            api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy && api.GetErrorString;
        }
    }
    return api;
}
}  // namespace

int gt_dp_unique_id(void *out, int32_t nbytes) {
    if (!out || nbytes < (int32_t)sizeof(ncclUniqueId)) return fail(GT_ERR_INVALID, "unique id buffer must hold %d bytes", (int)sizeof(ncclUniqueId));
    NcclApi &n = nccl_api();
    if (!n.ok) return fail(GT_ERR_NCCL, "libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    ncclResult_t r = n.GetUniqueId(&id);
    if (r != ncclSuccess) return fail(GT_ERR_NCCL, "ncclGetUniqueId: %s", n.GetErrorString(r));
    memcpy(out, &id, sizeof(id));
    return GT_OK;
}

int gt_dp_init(gt_engine *e, int32_t world, int32_t rank, const void *unique_id, int32_t nbytes) {
    if (!e || !unique_id || nbytes < (int32_t)sizeof(ncclUniqueId)) return fail(GT_ERR_INVALID, "gt_dp_init: bad argument");
    if (world < 1 || rank < 0 || rank >= world) return fail(GT_ERR_INVALID, "bad rank %d of world %d", rank, world);
    NcclApi &n = nccl_api();
    if (!n.ok) return fail(GT_ERR_NCCL, "libnccl.so.2 could not be loaded");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    if (e->comm) return fail(GT_ERR_INVALID, "data-parallel group already initialised");
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclResult_t r = n.CommInitRank(&e->comm, world, id, rank);
    if (r != ncclSuccess) {
        e->comm = nullptr;
        return fail(GT_ERR_NCCL, "ncclCommInitRank: %s", n.GetErrorString(r));
    }
    e->dp_world = world;
    e->dp_rank = rank;
    drop_step_graphs(e);
    return GT_OK;
}

namespace {
// all-reduce (+ scale) of g_dev on `st`; scale == 1/world lets the collective average, no extra pass
int allreduce_on(gt_engine *e, float *g_dev, int64_t count, float scale, cudaStream_t st) {
    if (e->comm) {
        NcclApi &n = nccl_api();
        const float inv = 1.0f / (float)e->dp_world;
        const bool avg = scale == inv;
        ncclResult_t r = n.AllReduce(g_dev, g_dev, (size_t)count, ncclFloat, avg ? ncclAvg : ncclSum, e->comm, st);
        if (r != ncclSuccess) return fail(GT_ERR_NCCL, "ncclAllReduce: %s", n.GetErrorString(r));
        if (avg) return GT_OK;
    }
    if (scale != 1.0f) GT_CUDA(launch_scale(g_dev, count, scale, st));      // plain scale: no norm, no shared scratch
    return GT_OK;
}
}  // namespace

int gt_dp_allreduce(gt_engine *e, float *g_dev, int64_t count, float scale) {
    if (!e || !g_dev || count < 0) return fail(GT_ERR_INVALID, "gt_dp_allreduce: bad argument");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    int rc = join_comm(e);      // collectives of one communicator run in issue order
    if (rc != GT_OK) return rc;
    return allreduce_on(e, g_dev, count, scale, e->stream);
}

}  // extern "C"
namespace gt {
// queue the all-reduce of one slice on the side stream, after everything queued on the engine stream so far (lock held)
int allreduce_begin_locked(gt_engine *e, float *g_dev, int64_t count, float scale) {
    if (!e->s_comm) {
        GT_CUDA(cudaStreamCreateWithFlags(&e->s_comm, cudaStreamNonBlocking));
        GT_CUDA(cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming));
        GT_CUDA(cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming));
    }
    // fork: the side stream starts once everything queued on the engine stream so far (the kernels that produced
    // these gradients) has finished; later engine-stream work runs beside the collective
    GT_CUDA(cudaEventRecord(e->ev_fork, e->stream));
    GT_CUDA(cudaStreamWaitEvent(e->s_comm, e->ev_fork, 0));
    int rc = allreduce_on(e, g_dev, count, scale, e->s_comm);
    if (rc != GT_OK) return rc;
    GT_CUDA(cudaEventRecord(e->ev_join, e->s_comm));
    e->comm_pending = true;
    return GT_OK;
}
}  // namespace gt
extern "C" {

int gt_dp_allreduce_begin(gt_engine *e, float *g_dev, int64_t count, float scale) {
    if (!e || !g_dev || count < 0) return fail(GT_ERR_INVALID, "gt_dp_allreduce_begin: bad argument");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return allreduce_begin_locked(e, g_dev, count, scale);
}

int gt_dp_allreduce_end(gt_engine *e) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    return join_comm(e);
}

int gt_dp_finalize(gt_engine *e) {
    if (!e) return fail(GT_ERR_INVALID, "engine is null");
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->comm) {
        cudaSetDevice(e->device);
        cudaStreamSynchronize(e->stream);
        if (e->s_comm) cudaStreamSynchronize(e->s_comm);
        drop_step_graphs(e);
        nccl_api().CommDestroy(e->comm);
        e->comm = nullptr;
    }
    e->dp_world = 1;
    e->dp_rank = 0;
    return GT_OK;
}

}  // extern "C"
