// C++ host mirror of the reference's projection and training-step API over the C ABI of libglaciertune_b200.so.
//
// The reference host is C# (src/Glacier.Tune/Gpu/GpuLoraEngine*.cs, src/Glacier.Tune/Model/LoraAdapter.cs); this header
// keeps its member names, argument order and error behaviour (a failing call throws, as CuDriver.Check does) so a
// maintainer can read one against the other.  It contains no arithmetic: every call lands in the shared library.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/glaciertune_b200.h"

namespace Glacier::Tune {

enum class GgufType : int { F32 = GT_TYPE_F32, Q4_K = GT_TYPE_Q4_K, Q6_K = GT_TYPE_Q6_K };

// Minimal stand-in for Glacier.Tensor's Tensor<float>: caller-owned contiguous fp32 memory.
struct Tensor {
    float *DataPointer = nullptr;
    int Shape[2] = {0, 0};
    Tensor() = default;
    Tensor(float *p, int rows, int cols) : DataPointer(p), Shape{rows, cols} {}
    int64_t ElementCount() const { return (int64_t)Shape[0] * Shape[1]; }
};

inline void Check(int rc, const char *label) {
    if (rc != GT_OK) throw std::runtime_error(std::string(label) + ": " + gt_last_error());
}

// Replaces GpuLoraEngine (src/Glacier.Tune/Gpu/GpuLoraEngine.cs:114-218).  The constructor throws when no sm_100
// device is usable; the reference's caller logs and carries on on the CPU (src/Glacier.Tune/Model/GgufLoraModel.cs:76-80).
class GpuLoraEngine {
public:
    explicit GpuLoraEngine(int deviceOrdinal = 0, int mathMode = GT_MATH_BF16) {
        gt_config cfg{};
        cfg.device = deviceOrdinal;
        cfg.math_mode = mathMode;
        Check(gt_engine_create(&cfg, &eng_), "gt_engine_create");
    }
    ~GpuLoraEngine() { Dispose(); }
    GpuLoraEngine(const GpuLoraEngine &) = delete;
    GpuLoraEngine &operator=(const GpuLoraEngine &) = delete;

    void Dispose() {
        for (gt_weight *w : weights_) gt_weight_free(w);
        weights_.clear();
        if (eng_) gt_engine_destroy(eng_);
        eng_ = nullptr;
    }
    gt_engine *Handle() const { return eng_; }

    bool SupportsForwardGemm(GgufType t) const { return gt_supports((int)t, GT_DIR_FORWARD) != 0; }
    bool SupportsBackwardGemm(GgufType t) const { return gt_supports((int)t, GT_DIR_BACKWARD) != 0; }

    // One tensor of UploadBaseWeights (GpuLoraEngine.cs:240-321); the handle plays the role of GetQ/GetK/... (:323-333).
    gt_weight *UploadBaseWeight(GgufType type, const void *bytes, int64_t nbytes, int outFeatures, int inFeatures,
                                const float *bias = nullptr) {
        gt_weight *w = nullptr;
        Check(gt_weight_upload(eng_, (int)type, bytes, nbytes, outFeatures, inFeatures, bias, &w), "gt_weight_upload");
        weights_.push_back(w);
        return w;
    }

    // GpuLoraEngine.Forward.cs:16-48: host tensors in and out, complete on return.
    void ForwardProjection(GgufType, gt_weight *dW, const Tensor &x, Tensor &output, int /*inFeatures*/, int /*outFeatures*/,
                           int seqLen) {
        Check(gt_proj_forward(eng_, dW, nullptr, x.DataPointer, output.DataPointer, seqLen, 0), "ForwardProjection");
    }
    // GpuLoraEngine.Backward.cs:58-92: dXInput is accumulated into.
    void BackwardProjection(GgufType, gt_weight *dW, const Tensor &dY, Tensor &dXInput, int, int, int seqLen) {
        Check(gt_proj_backward(eng_, dW, nullptr, dY.DataPointer, nullptr, dXInput.DataPointer, seqLen, 0), "BackwardProjection");
    }
    // GpuLoraEngine.Forward.cs:83-129 / Backward.cs:15-56: device pointers, asynchronous.
    void LaunchGemmBatch(gt_weight *dW, float *dY, const float *dX, int batchSize, float *dResidual = nullptr) {
        Check(gt_launch_gemm_batch(eng_, dW, dY, dX, batchSize, dResidual), "LaunchGemmBatch");
    }
    void LaunchGemmBwd(gt_weight *dW, float *dDX, const float *dDY, int batchSize) {
        Check(gt_launch_gemm_bwd(eng_, dW, dDX, dDY, batchSize), "LaunchGemmBwd");
    }
    void Synchronize() { Check(gt_sync(eng_), "gt_sync"); }

private:
    gt_engine *eng_ = nullptr;
    std::vector<gt_weight *> weights_;
};

// Replaces LoraAdapter (src/Glacier.Tune/Model/LoraAdapter.cs).  A is [InFeatures, Rank], B is [Rank, OutFeatures].
class LoraAdapter {
public:
    LoraAdapter(GpuLoraEngine &engine, int inFeatures, int outFeatures, int rank = 16, float alpha = 32.f)
        : engine_(engine), in_(inFeatures), out_(outFeatures), rank_(rank), scaling_(rank > 0 ? alpha / rank : 0.f) {
        Check(gt_adapter_create(engine.Handle(), inFeatures, outFeatures, rank, alpha, &ad_), "gt_adapter_create");
    }
    ~LoraAdapter() { gt_adapter_free(ad_); }
    LoraAdapter(const LoraAdapter &) = delete;
    LoraAdapter &operator=(const LoraAdapter &) = delete;

    int InFeatures() const { return in_; }
    int OutFeatures() const { return out_; }
    int Rank() const { return rank_; }
    float Scaling() const { return scaling_; }

    void SetGpuBaseWeights(gt_weight *dBaseWeight) { w_ = dBaseWeight; }             // LoraAdapter.cs:79-84
    void UpdateAlpha(float alpha) {                                                    // LoraAdapter.cs:74-77
        scaling_ = rank_ > 0 ? alpha / rank_ : 0.f;
        Check(gt_adapter_set_alpha(ad_, alpha), "gt_adapter_set_alpha");
    }
    void SetParameters(const float *A, const float *B) { Check(gt_adapter_upload(ad_, A, B), "gt_adapter_upload"); }
    void GetParameters(float *A, float *B) { Check(gt_adapter_download(ad_, A, B), "gt_adapter_download"); }
    void GetGradients(float *dA, float *dB) { Check(gt_adapter_grads_download(ad_, dA, dB), "gt_adapter_grads_download"); }
    void ZeroGrad() { Check(gt_adapter_grads_zero(ad_), "gt_adapter_grads_zero"); }
    // The trainer's optimizer step on this adapter's A and B (AdamW.Step, LoraTrainer.cs:230), on the device;
    // step counts the optimizer steps taken so far, starting at 1.
    void OptimizerStep(float lr, float beta1, float beta2, float eps, float weightDecay, int step) {
        Check(gt_adapter_adamw_step(ad_, lr, beta1, beta2, eps, weightDecay, step), "gt_adapter_adamw_step");
    }

    // LoraAdapter.cs:128-184: output = x W^T + bias + scaling (x A) B (delta skipped while B == 0).
    void Forward(GgufType, const Tensor &x, Tensor &output, int seqLen) {
        Check(gt_proj_forward(engine_.Handle(), w_, ad_, x.DataPointer, output.DataPointer, seqLen, 0), "LoraAdapter.Forward");
    }
    // LoraAdapter.cs:190-219: dXInput (optional) += dY W + adapter term; dA, dB accumulate.
    void Backward(GgufType, const Tensor &dY, const Tensor &x, Tensor *dXInput = nullptr) {
        Check(gt_proj_backward(engine_.Handle(), w_, ad_, dY.DataPointer, x.DataPointer, dXInput ? dXInput->DataPointer : nullptr,
                               x.Shape[0], 0),
              "LoraAdapter.Backward");
    }

    gt_weight *Weight() const { return w_; }
    gt_adapter *Handle() const { return ad_; }

private:
    GpuLoraEngine &engine_;
    gt_weight *w_ = nullptr;
    gt_adapter *ad_ = nullptr;
    int in_, out_, rank_;
    float scaling_;
};

// GpuLoraEngine.ForwardQKV / the gate,up half of ForwardFfn (GpuLoraEngine.Forward.cs:205-364): n (1..3) adapted
// projections of the same input in one engine call.  outputs[j] receives projection j.
inline void ForwardGroup(GpuLoraEngine &engine, LoraAdapter *const *projections, int n, const Tensor &x, Tensor *const *outputs,
                         int seqLen) {
    gt_weight *w[3];
    gt_adapter *a[3];
    float *y[3];
    for (int j = 0; j < n && j < 3; j++) {
        w[j] = projections[j]->Weight();
        a[j] = projections[j]->Handle();
        y[j] = outputs[j]->DataPointer;
    }
    Check(gt_proj_forward_group(engine.Handle(), n, w, a, x.DataPointer, y, seqLen, 0), "ForwardGroup");
}
// The q|k|v (gate|up) Backward calls of a block and the sum of their input gradients (TransformerBlock.cs:660-663,
// 812-816): dXInput = sum_j (dY[j] W_j + adapter term j), written (not accumulated) by the call.
inline void BackwardGroup(GpuLoraEngine &engine, LoraAdapter *const *projections, int n, const Tensor *const *dY, const Tensor &x,
                          Tensor &dXInput) {
    gt_weight *w[3];
    gt_adapter *a[3];
    const float *g[3];
    for (int j = 0; j < n && j < 3; j++) {
        w[j] = projections[j]->Weight();
        a[j] = projections[j]->Handle();
        g[j] = dY[j]->DataPointer;
    }
    Check(gt_proj_backward_group(engine.Handle(), n, w, a, g, x.DataPointer, dXInput.DataPointer, x.Shape[0], GT_FLAG_DX_ASSIGN),
          "BackwardGroup");
}

// Replaces the training-step half of GgufLoraModel (src/Glacier.Tune/Model/GgufLoraModel.cs:370-557) and the step tail of
// LoraTrainer (src/Glacier.Tune/Trainer/LoraTrainer.cs:217-231) with the device-resident driver: the seven projections
// of every block are LoraAdapter objects of this header (their weights set with SetGpuBaseWeights), in the reference's
// order q, k, v, o, gate, up, down (TransformerBlock.cs:149-165).
class GgufLoraModel {
public:
    GgufLoraModel(GpuLoraEngine &engine, int layers, int hidden, int heads, int kvHeads, int headDim, int ffn, int vocab, int maxTokens,
                  float rmsEps = 1e-6f, float ropeTheta = 1e6f, bool checkpointActivations = true)
        : engine_(engine) {
        gt_model_config cfg{};
        cfg.n_layers = layers;
        cfg.hidden = hidden;
        cfg.n_heads = heads;
        cfg.n_kv_heads = kvHeads;
        cfg.head_dim = headDim;
        cfg.ffn = ffn;
        cfg.vocab = vocab;
        cfg.rms_eps = rmsEps;
        cfg.rope_theta = ropeTheta;
        cfg.max_tokens = maxTokens;
        cfg.checkpoint = checkpointActivations ? 1 : 0;
        Check(gt_model_create(engine.Handle(), &cfg, &model_), "gt_model_create");
    }
    ~GgufLoraModel() {
        if (model_) gt_model_destroy(model_);
    }
    GgufLoraModel(const GgufLoraModel &) = delete;
    GgufLoraModel &operator=(const GgufLoraModel &) = delete;

    // projections[7]: q, k, v, o, gate, up, down; attnNorm / ffnNorm: host arrays [hidden]
    void SetBlock(int layer, LoraAdapter *const *projections, const float *attnNorm, const float *ffnNorm) {
        const gt_weight *w[7];
        gt_adapter *a[7];
        for (int j = 0; j < 7; j++) {
            w[j] = projections[j]->Weight();
            a[j] = projections[j]->Handle();
        }
        Check(gt_model_set_block(model_, layer, w, a, attnNorm, ffnNorm), "gt_model_set_block");
    }
    void SetHead(gt_weight *embedding, const float *outNorm, gt_weight *lmHead) {
        Check(gt_model_set_head(model_, embedding, outNorm, lmHead), "gt_model_set_head");
    }
    // one flat gradient buffer in the reference's parameter order; returns its length
    int64_t BindGradients() {
        int64_t n = 0;
        Check(gt_model_bind_grads(model_, nullptr, &n), "gt_model_bind_grads");
        return n;
    }
    // GgufLoraModel.ComputeLoss (GgufLoraModel.cs:370-426)
    float ComputeLoss(const int32_t *inputTokens, const int32_t *targetTokens, int seqLen) {
        float loss = 0.f;
        Check(gt_model_loss(model_, inputTokens, targetTokens, seqLen, &loss, nullptr, 0), "gt_model_loss");
        return loss;
    }
    // GgufLoraModel.ForwardLossAndBackward (GgufLoraModel.cs:428-557): the adapters' gradients accumulate
    float ForwardLossAndBackward(const int32_t *inputTokens, const int32_t *targetTokens, int seqLen) {
        float loss = 0.f;
        Check(gt_model_forward_backward(model_, inputTokens, targetTokens, seqLen, &loss, 0), "gt_model_forward_backward");
        return loss;
    }
    // ScaleAccumulatedGradients -> ClipGradients -> AdamW -> ZeroGrad (LoraTrainer.cs:217-231); returns the pre-clip norm
    double OptimizerStep(float lr, float beta1, float beta2, float eps, float weightDecay, float gradScale, double maxNorm, int step) {
        double norm = 0.0;
        Check(gt_model_optimizer_step(model_, lr, beta1, beta2, eps, weightDecay, gradScale, maxNorm, step, &norm), "gt_model_optimizer_step");
        return norm;
    }
    gt_model *Handle() const { return model_; }

private:
    GpuLoraEngine &engine_;
    gt_model *model_ = nullptr;
};

}  // namespace Glacier::Tune
