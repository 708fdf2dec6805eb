// The training step of a LoRA-adapted decoder on the device: embedding -> transformer blocks -> final RMSNorm ->
// streaming cross-entropy -> reverse pass -> (all-reduce) -> clip -> AdamW, with nothing on the host between the
// operations.
//
// Replaces the step driver of the reference: GgufLoraModel.ForwardLossAndBackward / ComputeLoss
// (src/Glacier.Tune/Model/GgufLoraModel.cs:370-557), TransformerBlock.Forward / Backward
// (src/Glacier.Tune/Model/TransformerBlock.cs:307-595,625-840) and the trainer's per-step tail
// (src/Glacier.Tune/Trainer/LoraTrainer.cs:217-231: scale the accumulated gradients, clip, optimizer step, zero).
// The reference keeps every activation on the host and crosses PCIe around each projection; here the tensors of a
// step live in one device allocation made at gt_model_create.
//
// Block (pre-norm, as TransformerBlock.Forward):
//   n1 = RMSNorm(x) ; q,k,v = proj(n1) (+bias, +LoRA) ; RoPE(q,k) ; a = causal GQA attention ; x1 = x + proj_o(a)
//   n2 = RMSNorm(x1) ; g,u = proj(n2) ; h = SiLU(g) * u ; out = x1 + proj_down(h)
// Activation checkpointing (GgufLoraModel.cs:505-531): the forward keeps only every block's input; the backward
// recomputes a block's forward into the one set of state buffers right before that block's backward.
// Data parallel: when the engine has a communicator (gt_dp_init), the gradients of a block are all-reduced on the
// side stream as soon as that block's backward is queued - last block first - beside the backward of the blocks
// below it; the optimizer step waits for all of them.
#include <vector>

#include "gt_engine_priv.h"

using namespace gt;

namespace {
enum { kQ = 0, kK, kV, kO, kGate, kUp, kDown, kProj };

struct BlockState {      // what a block's backward needs from its forward
    float *n1, *q, *k, *v, *attn, *lse, *x1, *n2, *gate, *up, *hidden;
};
struct LayerDev {
    const gt_weight *w[kProj] = {};
    gt_adapter *ad[kProj] = {};
    float *norm1 = nullptr, *norm2 = nullptr;      // device, [hidden]
    int64_t g0 = 0, g1 = 0;                        // this layer's slice of the flat gradient buffer
};
}  // namespace

struct gt_model {
    gt_engine *eng = nullptr;
    gt_model_config cfg{};
    std::vector<LayerDev> layers;
    const gt_weight *embedding = nullptr, *lm_head = nullptr;
    float *out_norm = nullptr;
    float *arena = nullptr;            // every activation buffer of a step
    size_t arena_bytes = 0;
    std::vector<float *> x;            // x[l] = input of block l, x[L] = output of the last block; [T, hidden] each
    std::vector<BlockState> st;        // one set (checkpointing) or one per block
    float *tmp_h = nullptr;            // projection output before the residual add
    float *fnorm = nullptr, *dfnorm = nullptr, *dx_a = nullptr, *dx_b = nullptr, *dn = nullptr, *dx1 = nullptr;
    float *dattn = nullptr, *dq = nullptr, *dk = nullptr, *dv = nullptr;
    int *tokens = nullptr, *labels = nullptr, *valid = nullptr, *bad = nullptr;
    float *loss = nullptr;
    float *grads = nullptr;            // flat gradient buffer (reference parameter order), or null until bound
    int64_t n_grads = 0;
    std::vector<gt_adapter *> adapters;      // in parameter order
    // The step's device work (embedding .. last block's backward and gradient exchange) as a CUDA graph: the first call
    // with a given shape runs eagerly (every scratch buffer reaches its size), the second is captured from the same code
    // and launched, later ones replay it while nothing it points at has moved (StepKey).  A replay costs the host one
    // launch instead of ~1400 and leaves no launch gaps between the short kernels.
    struct StepKey {
        int T = 0, world = 0, math = 0;
        uint64_t gen = 0;
        const void *comm = nullptr;
        bool operator==(const StepKey &o) const { return T == o.T && world == o.world && math == o.math && gen == o.gen && comm == o.comm; }
    };
    cudaGraphExec_t step_exec = nullptr;
    int64_t step_replays = 0;
    StepKey step_key, warm_key;
    bool warm = false;
    bool graph_off = false;            // configuration, GT_STEP_GRAPH=0, or a capture that failed
    int64_t step_launches = 0;         // kernels of the captured step (the engine's launch count, per replay)
};

namespace {

size_t a256(size_t n) { return (n + 255) & ~(size_t)255; }

void drop_graph(gt_model *m) {
    if (m->step_exec) cudaGraphExecDestroy(m->step_exec);
    m->step_exec = nullptr;
    m->warm = false;
}

int check_ready(const gt_model *m, const char *who) {
    if (!m) return failf(GT_ERR_INVALID, "%s: model is null", who);
    if (!m->embedding || !m->lm_head || !m->out_norm) return failf(GT_ERR_INVALID, "%s: gt_model_set_head has not been called", who);
    for (size_t l = 0; l < m->layers.size(); l++)
        if (!m->layers[l].w[kQ]) return failf(GT_ERR_INVALID, "%s: block %d has not been set", who, (int)l);
    return GT_OK;
}

// One block forward on the engine stream; s receives the state.  n1_ready: s.n1 already holds RMSNorm(x_in) (the block
// before wrote it together with its output).  next_norm / next_n1 (may be null): the norm weight and destination of
// the norm that follows this block's output - the next block's attention norm or the model's output norm - computed
// in the same pass as the residual add.  x_out == nullptr: the state only (the recomputed forward of a checkpointed block) -
// the down projection and the residual add after it are left out, their result is the stored input of the next block.
// keep_gu = false: nothing will read this pass's gate and up tensors (the block's state is recomputed before its backward),
// so where the FFN can do without them they are not written.
int block_forward(gt_model *m, int l, const float *x_in, float *x_out, BlockState &s, int T, bool n1_ready, const float *next_norm,
                  float *next_n1, bool keep_gu = true) {
    gt_engine *e = m->eng;
    const gt_model_config &c = m->cfg;
    const LayerDev &L = m->layers[l];
    const int H = c.hidden;
    if (!n1_ready) GT_LAUNCH(e, launch_rmsnorm_fwd(x_in, L.norm1, s.n1, T, H, c.rms_eps, e->stream));
    float *qkv[3] = {s.q, s.k, s.v};
    int rc = forward_group_device(e, 3, L.w + kQ, L.ad + kQ, s.n1, qkv, T, 0);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_rope(s.q, s.k, T, c.n_heads, c.n_kv_heads, c.head_dim, c.rope_theta, 1.0f, c.head_dim, 0, e->stream));
    rc = attention_forward_on_device(e, s.q, s.k, s.v, s.attn, s.lse, T, c.n_heads, c.n_kv_heads, c.head_dim);
    if (rc != GT_OK) return rc;
    float *o = m->tmp_h;
    rc = forward_group_device(e, 1, L.w + kO, L.ad + kO, s.attn, &o, T, 0);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_add_rmsnorm_fwd(x_in, o, L.norm2, s.x1, s.n2, T, H, c.rms_eps, e->stream));      // x1 = x + o; n2 = norm(x1)
    const gt_weight *fw[3] = {L.w[kGate], L.w[kUp], L.w[kDown]};
    gt_adapter *fa[3] = {L.ad[kGate], L.ad[kUp], L.ad[kDown]};
    // SiLU(gate) * up is kept as bf16 only where the engine can work from that (the buffer is sized for fp32 either way)
    const bool h16 = ffn_hidden16_ok(e, fw, T);
    const bool drop_gu = !keep_gu && h16 && x_out;      // (without the 16-bit product the SwiGLU pass reads them from the state)
    rc = ffn_forward_device(e, fw, fa, s.n2, drop_gu ? nullptr : s.gate, drop_gu ? nullptr : s.up, h16 ? nullptr : s.hidden,
                            x_out ? m->tmp_h : nullptr, T, 0, h16 ? (void *)s.hidden : nullptr);
    if (rc != GT_OK || !x_out) return rc;
    if (next_norm && next_n1) GT_LAUNCH(e, launch_add_rmsnorm_fwd(s.x1, m->tmp_h, next_norm, x_out, next_n1, T, H, c.rms_eps, e->stream));
    else GT_LAUNCH(e, launch_add(s.x1, m->tmp_h, x_out, (int64_t)T * H, e->sm_count, e->stream));
    return GT_OK;
}

// One block backward: d_out [T, H] -> d_in [T, H] (may not alias d_out); adapter gradients accumulate.
int block_backward(gt_model *m, int l, const float *d_out, const float *x_in, const BlockState &s, float *d_in, int T) {
    gt_engine *e = m->eng;
    const gt_model_config &c = m->cfg;
    const LayerDev &L = m->layers[l];
    const int H = c.hidden;
    const int flags = GT_FLAG_REUSE_LOW | GT_FLAG_DX_ASSIGN;
    const gt_weight *fw[3] = {L.w[kGate], L.w[kUp], L.w[kDown]};
    gt_adapter *fa[3] = {L.ad[kGate], L.ad[kUp], L.ad[kDown]};
    // A. FFN: down, SwiGLU, gate | up -> dNorm2X; RMSNorm2 backward + residual: dX1 = dOut + dNorm(dNorm2X)
    const bool h16 = ffn_hidden16_ok(e, fw, T);
    int rc = ffn_backward_device(e, fw, fa, d_out, s.n2, s.gate, s.up, h16 ? nullptr : s.hidden, m->dn, T, flags,
                                 h16 ? (const void *)s.hidden : nullptr);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_rmsnorm_bwd(m->dn, s.x1, L.norm2, d_out, m->dx1, T, H, c.rms_eps, e->stream));
    // B. attention: o projection, attention, RoPE, q | k | v -> dNorm1X; RMSNorm1 backward + residual
    const float *dy_o = m->dx1;
    rc = backward_group_device(e, 1, L.w + kO, L.ad + kO, &dy_o, s.attn, m->dattn, T, flags);
    if (rc != GT_OK) return rc;
    rc = attention_backward_on_device(e, m->dattn, s.q, s.k, s.v, s.attn, s.lse, m->dq, m->dk, m->dv, T, c.n_heads, c.n_kv_heads, c.head_dim);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_rope(m->dq, m->dk, T, c.n_heads, c.n_kv_heads, c.head_dim, c.rope_theta, 1.0f, c.head_dim, 1, e->stream));
    const float *dqkv[3] = {m->dq, m->dk, m->dv};
    rc = backward_group_device(e, 3, L.w + kQ, L.ad + kQ, dqkv, s.n1, m->dn, T, flags);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_rmsnorm_bwd(m->dn, x_in, L.norm1, m->dx1, d_in, T, H, c.rms_eps, e->stream));
    return GT_OK;
}

int stage_inputs(gt_model *m, const int32_t *tokens, const int32_t *labels, int T, int flags) {
    gt_engine *e = m->eng;
    const cudaMemcpyKind kind = (flags & GT_FLAG_DEVICE_PTRS) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    GT_CUDA(cudaMemcpyAsync(m->tokens, tokens, (size_t)T * sizeof(int), kind, e->stream));
    GT_CUDA(cudaMemcpyAsync(m->labels, labels, (size_t)T * sizeof(int), kind, e->stream));
    GT_CUDA(cudaMemsetAsync(m->bad, 0, sizeof(int), e->stream));
    return GT_OK;
}

int forward_all(gt_model *m, int T, bool keep_states) {
    gt_engine *e = m->eng;
    int rc = embedding_on_device(e, m->embedding, m->tokens, T, m->x[0], m->bad);
    if (rc != GT_OK) return rc;
    const int L = (int)m->layers.size();
    for (int l = 0; l < L; l++) {
        BlockState &s = m->st[keep_states ? l : 0];
        // the norm that follows this block's output rides on its last residual add: the next block's attention norm
        // (into that block's state; with one shared state set its n1 has been consumed by then) or the output norm
        const float *next_w = l + 1 < L ? m->layers[l + 1].norm1 : m->out_norm;
        float *next_n1 = l + 1 < L ? m->st[keep_states ? l + 1 : 0].n1 : m->fnorm;
        // with one shared state set only the last block's state survives until its backward
        rc = block_forward(m, l, m->x[l], m->x[l + 1], s, T, l > 0, next_w, next_n1, keep_states || l == L - 1);
        if (rc != GT_OK) return rc;
    }
    return GT_OK;
}

int finish_loss(gt_model *m, float *loss_out, int32_t *valid_out, int flags) {
    gt_engine *e = m->eng;
    if (flags & GT_FLAG_DEVICE_PTRS) {
        if (loss_out) GT_CUDA(cudaMemcpyAsync(loss_out, m->loss, sizeof(float), cudaMemcpyDeviceToDevice, e->stream));
        if (valid_out) GT_CUDA(cudaMemcpyAsync(valid_out, m->valid, sizeof(int), cudaMemcpyDeviceToDevice, e->stream));
        return GT_OK;
    }
    float hl = 0.f;
    int hv = 0, hb = 0;
    GT_CUDA(cudaMemcpyAsync(&hl, m->loss, sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaMemcpyAsync(&hv, m->valid, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    GT_CUDA(cudaMemcpyAsync(&hb, m->bad, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    int rc = check_status(e);
    if (rc != GT_OK) return rc;
    if (hb) return failf(GT_ERR_INVALID, "%d input token id(s) outside the vocabulary [0, %d)", hb, m->cfg.vocab);      // GgufLoraModel.cs:443-452
    if (loss_out) *loss_out = hl;
    if (valid_out) *valid_out = hv;
    return GT_OK;
}

}  // namespace

namespace gt {
void drop_step_graphs(gt_engine *e) {
    for (gt_model *m : e->models) drop_graph(m);
}
}  // namespace gt

extern "C" {

int gt_model_create(gt_engine *e, const gt_model_config *cfg, gt_model **out) {
    if (!e || !cfg || !out) return failf(GT_ERR_INVALID, "gt_model_create: null argument");
    *out = nullptr;
    const gt_model_config &c = *cfg;
    if (c.n_layers <= 0 || c.hidden <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.ffn <= 0 || c.vocab <= 0 ||
        c.max_tokens <= 0)
        return failf(GT_ERR_INVALID, "gt_model_create: every dimension must be positive");
    if (c.n_heads % c.n_kv_heads != 0) return failf(GT_ERR_INVALID, "gt_model_create: n_heads %d is not a multiple of n_kv_heads %d", c.n_heads, c.n_kv_heads);
    if (!gt_supports_attention(c.max_tokens, c.head_dim)) return failf(GT_ERR_UNSUPPORTED, "gt_model_create: head_dim %d is not supported", c.head_dim);
    if (c.hidden % 4 != 0 || c.ffn % 4 != 0) return failf(GT_ERR_INVALID, "gt_model_create: hidden and ffn must be multiples of 4");
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    gt_model *m = new (std::nothrow) gt_model();
    if (!m) return failf(GT_ERR_OOM, "out of host memory");
    m->eng = e;
    m->cfg = c;
    m->layers.resize(c.n_layers);
    const size_t T = c.max_tokens, H = c.hidden, F = c.ffn, QD = (size_t)c.n_heads * c.head_dim, KD = (size_t)c.n_kv_heads * c.head_dim;
    const int n_state = c.checkpoint ? 1 : c.n_layers;
    const size_t bh = a256(T * H * 4), bf = a256(T * F * 4), bq = a256(T * QD * 4), bk = a256(T * KD * 4), bl = a256((size_t)c.n_heads * T * 4);
    const size_t state_bytes = 3 * bh + 2 * bq + 2 * bk + bl + 3 * bf;       // n1, x1, n2 | q, attn | k, v | lse | gate, up, hidden
    size_t total = (size_t)(c.n_layers + 1) * bh + (size_t)n_state * state_bytes + 7 * bh /* tmp, fnorm, dfnorm, dx_a, dx_b, dn, dx1 */ +
                   2 * bq /* dattn, dq */ + 2 * bk + 2 * a256(T * 4) + 1024;
    cudaError_t ce = cudaMalloc((void **)&m->arena, total);
    if (ce != cudaSuccess) {
        delete m;
        return failf(GT_ERR_OOM, "gt_model_create: %zu bytes of activation buffers: %s", total, cudaGetErrorString(ce));
    }
    m->arena_bytes = total;
    char *p = (char *)m->arena;
    auto take = [&](size_t n) {
        float *r = (float *)p;
        p += n;
        return r;
    };
    m->x.resize(c.n_layers + 1);
    for (auto &xp : m->x) xp = take(bh);
    m->st.resize(n_state);
    for (BlockState &s : m->st) {
        s.n1 = take(bh); s.x1 = take(bh); s.n2 = take(bh);
        s.q = take(bq); s.attn = take(bq);
        s.k = take(bk); s.v = take(bk);
        s.lse = take(bl);
        s.gate = take(bf); s.up = take(bf); s.hidden = take(bf);
    }
    m->tmp_h = take(bh); m->fnorm = take(bh); m->dfnorm = take(bh); m->dx_a = take(bh); m->dx_b = take(bh); m->dn = take(bh); m->dx1 = take(bh);
    m->dattn = take(bq); m->dq = take(bq);
    m->dk = take(bk); m->dv = take(bk);
    m->tokens = (int *)take(a256(T * 4));
    m->labels = (int *)take(a256(T * 4));
    m->loss = take(256);
    m->valid = (int *)take(256);
    m->bad = (int *)take(256);
    m->graph_off = cfg->no_graph != 0;
    e->models.push_back(m);
    *out = m;
    return GT_OK;
}

int gt_model_destroy(gt_model *m) {
    if (!m) return GT_OK;
    gt_engine *e = m->eng;
    {
        std::lock_guard<std::mutex> lk(e->mu);
        cudaSetDevice(e->device);
        cudaStreamSynchronize(e->stream);
        if (e->s_comm) cudaStreamSynchronize(e->s_comm);
        drop_graph(m);
        for (size_t i = 0; i < e->models.size(); i++)
            if (e->models[i] == m) {
                e->models.erase(e->models.begin() + (long)i);
                break;
            }
        for (LayerDev &L : m->layers) {
            if (L.norm1) cudaFree(L.norm1);
            if (L.norm2) cudaFree(L.norm2);
        }
        if (m->out_norm) cudaFree(m->out_norm);
        if (m->arena) cudaFree(m->arena);
        if (m->grads) cudaFree(m->grads);      // the adapters must not be used for gradients after this
    }
    delete m;
    return GT_OK;
}

static int upload_vec(gt_engine *e, const float *host, int n, float **dev) {
    if (!*dev) GT_CUDA(cudaMalloc((void **)dev, (size_t)n * sizeof(float)));
    GT_CUDA(cudaMemcpyAsync(*dev, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    GT_CUDA(cudaStreamSynchronize(e->stream));
    return GT_OK;
}

int gt_model_set_block(gt_model *m, int32_t layer, const gt_weight *const *weights, gt_adapter *const *adapters, const float *attn_norm,
                       const float *ffn_norm) {
    if (!m || !weights || !attn_norm || !ffn_norm) return failf(GT_ERR_INVALID, "gt_model_set_block: null argument");
    if (layer < 0 || layer >= m->cfg.n_layers) return failf(GT_ERR_INVALID, "gt_model_set_block: layer %d outside [0, %d)", layer, m->cfg.n_layers);
    const gt_model_config &c = m->cfg;
    const int QD = c.n_heads * c.head_dim, KD = c.n_kv_heads * c.head_dim;
    const int want[kProj][2] = {{QD, c.hidden}, {KD, c.hidden}, {KD, c.hidden}, {c.hidden, QD}, {c.ffn, c.hidden}, {c.ffn, c.hidden}, {c.hidden, c.ffn}};
    static const char *names[kProj] = {"q", "k", "v", "o", "gate", "up", "down"};
    for (int j = 0; j < kProj; j++) {
        if (!weights[j]) return failf(GT_ERR_INVALID, "gt_model_set_block: weight %s is null", names[j]);
        if (weights[j]->eng != m->eng) return failf(GT_ERR_INVALID, "gt_model_set_block: weight %s belongs to another engine", names[j]);
        if (weights[j]->dev.N != want[j][0] || weights[j]->dev.K != want[j][1])
            return failf(GT_ERR_INVALID, "gt_model_set_block: %s is [%d, %d], expected [%d, %d]", names[j], weights[j]->dev.N, weights[j]->dev.K,
                         want[j][0], want[j][1]);
        gt_adapter *a = adapters ? adapters[j] : nullptr;
        if (a && (a->in != want[j][1] || a->out != want[j][0] || a->eng != m->eng))
            return failf(GT_ERR_INVALID, "gt_model_set_block: adapter of %s does not match its weight", names[j]);
    }
    if (m->grads) return failf(GT_ERR_INVALID, "gt_model_set_block: the gradient buffer is already bound; set every block first");
    gt_engine *e = m->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    drop_graph(m);      // a captured step points at what this call replaces
    GT_CUDA(cudaSetDevice(e->device));
    LayerDev &L = m->layers[layer];
    for (int j = 0; j < kProj; j++) {
        L.w[j] = weights[j];
        L.ad[j] = adapters ? adapters[j] : nullptr;
    }
    int rc = upload_vec(e, attn_norm, c.hidden, &L.norm1);
    if (rc == GT_OK) rc = upload_vec(e, ffn_norm, c.hidden, &L.norm2);
    return rc;
}

int gt_model_set_head(gt_model *m, const gt_weight *embedding, const float *out_norm, const gt_weight *lm_head) {
    if (!m || !embedding || !out_norm || !lm_head) return failf(GT_ERR_INVALID, "gt_model_set_head: null argument");
    const gt_model_config &c = m->cfg;
    if (embedding->dev.N != c.vocab || embedding->dev.K != c.hidden)
        return failf(GT_ERR_INVALID, "gt_model_set_head: embedding is [%d, %d], expected [%d, %d]", embedding->dev.N, embedding->dev.K, c.vocab, c.hidden);
    if (lm_head->dev.N != c.vocab || lm_head->dev.K != c.hidden)
        return failf(GT_ERR_INVALID, "gt_model_set_head: LM head is [%d, %d], expected [%d, %d]", lm_head->dev.N, lm_head->dev.K, c.vocab, c.hidden);
    if (lm_head->dev.qtype != kTypeF16 || !lm_head->dev.tma_ok)
        return failf(GT_ERR_UNSUPPORTED, "gt_model_set_head: the LM head must be an F16 tensor with hidden %% 128 == 0");
    gt_engine *e = m->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    drop_graph(m);      // a captured step points at what this call replaces
    GT_CUDA(cudaSetDevice(e->device));
    m->embedding = embedding;
    m->lm_head = lm_head;
    return upload_vec(e, out_norm, c.hidden, &m->out_norm);
}

int gt_model_bind_grads(gt_model *m, float **grads_dev, int64_t *count) {
    int rc = check_ready(m, "gt_model_bind_grads");
    if (rc != GT_OK) return rc;
    gt_engine *e = m->eng;
    if (!m->grads) {
        // parameter order of the reference: layer -> q, k, v, o, gate, up, down -> A, B (TransformerBlock.cs:167-174)
        int64_t n = 0;
        for (LayerDev &L : m->layers) {
            L.g0 = n;
            for (int j = 0; j < kProj; j++)
                if (L.ad[j]) n += (int64_t)L.ad[j]->rank * (L.ad[j]->in + L.ad[j]->out);
            L.g1 = n;
        }
        float *g = nullptr;
        {
            std::lock_guard<std::mutex> lk(e->mu);
            drop_graph(m);      // a captured step points at what this call replaces
            GT_CUDA(cudaSetDevice(e->device));
            GT_CUDA(cudaMalloc((void **)&g, (size_t)(n > 0 ? n : 1) * sizeof(float)));
            GT_CUDA(cudaMemsetAsync(g, 0, (size_t)(n > 0 ? n : 1) * sizeof(float), e->stream));
        }
        int64_t off = 0;
        for (LayerDev &L : m->layers)
            for (int j = 0; j < kProj; j++) {
                gt_adapter *a = L.ad[j];
                if (!a) continue;
                const int64_t na = (int64_t)a->in * a->rank, nb = (int64_t)a->rank * a->out;
                rc = gt_adapter_bind_grads(a, g + off, g + off + na);
                if (rc != GT_OK) return rc;
                off += na + nb;
                m->adapters.push_back(a);
            }
        m->grads = g;
        m->n_grads = n;
    }
    if (grads_dev) *grads_dev = m->grads;
    if (count) *count = m->n_grads;
    return GT_OK;
}

int gt_model_loss(gt_model *m, const int32_t *tokens, const int32_t *labels, int32_t T, float *loss_out, int32_t *valid_out, int32_t flags) {
    int rc = check_ready(m, "gt_model_loss");
    if (rc != GT_OK) return rc;
    if (!tokens || !labels || !loss_out) return failf(GT_ERR_INVALID, "gt_model_loss: null argument");
    if (T <= 0 || T > m->cfg.max_tokens) return failf(GT_ERR_INVALID, "gt_model_loss: T = %d outside (0, %d]", T, m->cfg.max_tokens);
    gt_engine *e = m->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    rc = stage_inputs(m, tokens, labels, T, flags);
    if (rc == GT_OK) rc = forward_all(m, T, false);
    if (rc == GT_OK) rc = lm_head_loss_on_device(e, m->lm_head, m->fnorm, m->labels, T, m->loss, m->valid, nullptr);
    if (rc != GT_OK) return rc;
    return finish_loss(m, loss_out, valid_out, flags);
}

namespace {
// Everything of a training step between the staged inputs and the read-back of the loss, queued on the engine stream
// (and its side streams); no host synchronisation, no allocation once the buffers have their size.
int step_body(gt_model *m, int T) {
    gt_engine *e = m->eng;
    const bool ckpt = m->cfg.checkpoint != 0;
    const int L = (int)m->layers.size(), H = m->cfg.hidden;
    int rc = forward_all(m, T, !ckpt);
    if (rc != GT_OK) return rc;
    // loss and its gradient with respect to the normed final hidden state, then through the final RMSNorm
    rc = lm_head_loss_on_device(e, m->lm_head, m->fnorm, m->labels, T, m->loss, m->valid, m->dfnorm);
    if (rc != GT_OK) return rc;
    GT_LAUNCH(e, launch_rmsnorm_bwd(m->dfnorm, m->x[L], m->out_norm, nullptr, m->dx_a, T, H, m->cfg.rms_eps, e->stream));
    float *d_cur = m->dx_a, *d_next = m->dx_b;
    const float inv_world = 1.0f / (float)e->dp_world;
    for (int l = L - 1; l >= 0; l--) {
        BlockState &s = m->st[ckpt ? 0 : l];
        // recompute this block's state into the one state set (not its output: that is x[l + 1], still there).  The last
        // block needs none: the forward pass ended with it, so the state set still holds its tensors (its attention norm
        // came with the residual add of the block before, its own last add wrote the output norm elsewhere)
        if (ckpt && l != L - 1) {
            rc = block_forward(m, l, m->x[l], nullptr, s, T, false, nullptr, nullptr);
            if (rc != GT_OK) return rc;
        }
        rc = block_backward(m, l, d_cur, m->x[l], s, d_next, T);
        if (rc != GT_OK) return rc;
        float *t = d_cur;
        d_cur = d_next;
        d_next = t;
        // this block's gradients are final: exchange them beside the backward of the blocks below
        if (e->comm && m->grads && m->layers[l].g1 > m->layers[l].g0) {
            rc = allreduce_begin_locked(e, m->grads + m->layers[l].g0, m->layers[l].g1 - m->layers[l].g0, inv_world);
            if (rc != GT_OK) return rc;
        }
    }
    return GT_OK;
}

bool step_graph_allowed(const gt_model *m) {
    static const bool env_on = !(getenv("GT_STEP_GRAPH") && atoi(getenv("GT_STEP_GRAPH")) == 0);
    const gt_engine *e = m->eng;
    if (!env_on || m->graph_off || e->profile || e->trace) return false;
    // the caller is capturing the engine stream itself: the kernels go into that graph one by one
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(e->stream, &cs) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return cs == cudaStreamCaptureStatusNone;
}

// Captures step_body into a graph.  On any failure the capture is closed, the error state cleared and the model keeps to
// eager launches from then on; nothing has run in that case (a capture only records).
bool capture_step(gt_model *m, int T) {
    gt_engine *e = m->eng;
    if (cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    const int64_t launches0 = e->kernel_launches;
    int rc = step_body(m, T);
    if (rc == GT_OK) rc = join_comm(e);      // the side stream of the gradient exchange rejoins inside the graph
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
    e->comm_pending = false;
    if (rc != GT_OK || ce != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        e->kernel_launches = launches0;
        return false;
    }
    m->step_launches = e->kernel_launches - launches0;
    e->kernel_launches = launches0;
    cudaGraphExec_t exec = nullptr;
    ce = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess || !exec) {
        cudaGetLastError();
        return false;
    }
    m->step_exec = exec;
    return true;
}
}  // namespace

int gt_model_forward_backward(gt_model *m, const int32_t *tokens, const int32_t *labels, int32_t T, float *loss_out, int32_t flags) {
    int rc = check_ready(m, "gt_model_forward_backward");
    if (rc != GT_OK) return rc;
    if (!tokens || !labels) return failf(GT_ERR_INVALID, "gt_model_forward_backward: null argument");
    if (T <= 0 || T > m->cfg.max_tokens) return failf(GT_ERR_INVALID, "gt_model_forward_backward: T = %d outside (0, %d]", T, m->cfg.max_tokens);
    gt_engine *e = m->eng;
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    // collectives of an earlier call that no optimizer step has waited for read the gradient buffer this call adds into
    rc = join_comm(e);
    if (rc != GT_OK) return rc;
    rc = stage_inputs(m, tokens, labels, T, flags);
    if (rc != GT_OK) return rc;
    bool queued = false;
    if (step_graph_allowed(m)) {
        gt_model::StepKey key;
        key.T = T;
        key.world = e->dp_world;
        key.math = e->math_mode;
        key.comm = e->comm;
        key.gen = gt::layout_generation().load();
        if (m->step_exec && !(m->step_key == key)) drop_graph(m);
        if (!m->step_exec && m->warm && m->warm_key == key) {
            if (capture_step(m, T)) {
                m->step_key = key;
            } else {
                m->graph_off = true;
                gt::logf(GT_LOG_INFO, "gt_model: the step could not be captured into a CUDA graph; launching eagerly");
            }
        }
        if (m->step_exec) {
            GT_CUDA(cudaGraphLaunch(m->step_exec, e->stream));
            e->kernel_launches += m->step_launches;
            m->step_replays += 1;
            queued = true;
        }
    }
    if (!queued) {
        rc = step_body(m, T);
        if (rc != GT_OK) return rc;
        // a later call with this shape may be captured, if this one moved no buffer
        m->warm_key.T = T;
        m->warm_key.world = e->dp_world;
        m->warm_key.math = e->math_mode;
        m->warm_key.comm = e->comm;
        m->warm_key.gen = gt::layout_generation().load();
        m->warm = true;
    }
    return finish_loss(m, loss_out, nullptr, flags);
}

int gt_model_step_info(gt_model *m, int32_t *graph_ready, int64_t *replays, int64_t *kernels_per_replay) {
    if (!m) return failf(GT_ERR_INVALID, "gt_model_step_info: model is null");
    std::lock_guard<std::mutex> lk(m->eng->mu);
    if (graph_ready) *graph_ready = m->step_exec ? 1 : 0;
    if (replays) *replays = m->step_replays;
    if (kernels_per_replay) *kernels_per_replay = m->step_exec ? m->step_launches : 0;
    return GT_OK;
}

int gt_model_optimizer_step(gt_model *m, float lr, float beta1, float beta2, float eps, float weight_decay, float grad_scale, double max_norm,
                            int32_t step, double *norm_out) {
    int rc = check_ready(m, "gt_model_optimizer_step");
    if (rc != GT_OK) return rc;
    if (!m->grads) return failf(GT_ERR_INVALID, "gt_model_optimizer_step: call gt_model_bind_grads first");
    if (step < 1) return failf(GT_ERR_INVALID, "gt_model_optimizer_step: step counts from 1");
    gt_engine *e = m->eng;
    {
        std::lock_guard<std::mutex> lk(e->mu);
        GT_CUDA(cudaSetDevice(e->device));
        rc = join_comm(e);      // every block's gradient exchange
        if (rc != GT_OK) return rc;
        // ScaleAccumulatedGradients(1 / accumulation steps) then ClipGradients(maxNorm) (LoraTrainer.cs:217-222)
        if (max_norm > 0.0 || norm_out) {
            GT_CUDA(launch_scale_clip(m->grads, m->n_grads, grad_scale, max_norm, e->clip, e->stream));
            if (norm_out) {
                double h[2] = {0, 0};
                GT_CUDA(cudaMemcpyAsync(h, e->clip, sizeof(h), cudaMemcpyDeviceToHost, e->stream));
                GT_CUDA(cudaStreamSynchronize(e->stream));
                *norm_out = max_norm > 0.0 ? h[1] : 0.0;
            }
        } else if (grad_scale != 1.0f) {
            GT_CUDA(launch_scale(m->grads, m->n_grads, grad_scale, e->stream));
        }
    }
    if (!m->adapters.empty()) {
        rc = gt_adapters_adamw_step(e, (int32_t)m->adapters.size(), m->adapters.data(), lr, beta1, beta2, eps, weight_decay, step);
        if (rc != GT_OK) return rc;
    }
    std::lock_guard<std::mutex> lk(e->mu);
    GT_CUDA(cudaSetDevice(e->device));
    GT_CUDA(cudaMemsetAsync(m->grads, 0, (size_t)m->n_grads * sizeof(float), e->stream));      // optimizer.ZeroGrad()
    return GT_OK;
}

}  // extern "C"
