// gt_launch_gemm_bwd_static: the input-gradient GEMM  dDX[batch, in] += dDY[batch, out] * W  for callers that must
// not allocate device memory at call time.
//
// Who needs it: a host that drives its training step from inside a CUDA stream capture, from a latency-critical
// loop that may not hit the implicit device synchronisation of cudaMalloc / cudaFree, or from a process whose
// memory is fully handed out to a pool after start-up.  The regular entry point gt_launch_gemm_bwd keeps the
// 16-bit copy of dDY that the tensor-core kernel reads in a grow-only buffer of the engine, so its first call, and
// any call with a larger batch than seen before, calls cudaMalloc.  This variant keeps that copy in a fixed array
// that is part of the library image instead, and calls no allocating routine at all.
//
// Limits and rules
//   * the array holds kStaticScratchBytes (4 MiB): batch * round_up(out, 8) must not exceed 2,097,152 elements
//     (for instance 512 tokens x 3584 outputs); larger calls are rejected with GT_ERR_UNSUPPORTED before any launch.
//     Every GPU that loads the library carries these 4 MiB until the process exits.
//   * only K-quant weights in whole 256-wide rows and the bf16 / fp16 math modes (the tensor-core path) are
//     served; the fp32 validation mode needs no scratch and should use gt_launch_gemm_bwd.
//   * the device address of the array is looked up once per device, on the first call made with that device's
//     engine (cudaGetSymbolAddress with that device current).  Make that first call before any stream capture.
//   * all calls share the one array.  It still holds the previous call's 16-bit dDY on entry; nothing in it has to
//     start at zero, because each call rewrites every element it later reads (rows x padded row length, the
//     padding columns included).  Two calls whose GPU work overlaps (different engines or streams on the same
//     device) would race on it: run them one after the other.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../../include/glaciertune_b200.h"
#include "gt_internal.h"
#include "gt_quant.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kMaxDevices = 64;

// Device-resident scratch.  In host code this name is only a handle for the symbol, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mu;
void *g_scratch_addr[kMaxDevices] = {};      // per device: address of g_static_scratch on that device

// Looks the array's device address up for `device`, which must be the current device.
cudaError_t scratch_for_device(int device, void **out) {
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!g_scratch_addr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int gt_launch_gemm_bwd_static(gt_engine *eng, const gt_weight *w, float *dDX_accum, const float *dDY, int32_t batch) {
    using namespace gt;
    if (!eng || !w || !dDX_accum || !dDY) return set_last_error(GT_ERR_INVALID, "gt_launch_gemm_bwd_static: null argument");
    if (batch <= 0) return set_last_error(GT_ERR_INVALID, "gt_launch_gemm_bwd_static: batch must be positive");
    // the engine's lock is taken before anything else of the engine is read (the math mode may be changed by another
    // thread through gt_engine_set_math_mode)
    std::lock_guard<std::mutex> lk(*static_cast<std::mutex *>(engine_view(eng).mutex));
    const EngineView ev = engine_view(eng);
    const WeightDev *wd = weight_view(w);
    if (ev.math_mode == GT_MATH_FP32 || !wd->tma_ok || (wd->qtype != kTypeQ4K && wd->qtype != kTypeQ6K))
        return set_last_error(GT_ERR_UNSUPPORTED,
                              "gt_launch_gemm_bwd_static serves K-quant weights with in_features % 256 == 0 in the bf16/fp16 "
                              "math modes only; use gt_launch_gemm_bwd");
    const int ld16 = (wd->N + 7) & ~7;
    const size_t need = (size_t)batch * (size_t)ld16 * 2;
    if (need > kStaticScratchBytes) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "gt_launch_gemm_bwd_static: batch %d x out_features %d needs %zu bytes of scratch, the fixed array holds %zu "
                 "(at most 2097152 elements); use gt_launch_gemm_bwd",
                 batch, wd->N, need, kStaticScratchBytes);
        return set_last_error(GT_ERR_UNSUPPORTED, msg);
    }
    cudaError_t ce = cudaSetDevice(ev.device);
    void *scratch = nullptr;
    if (ce == cudaSuccess) ce = scratch_for_device(ev.device, &scratch);
    if (ce != cudaSuccess) {
        char msg[200];
        snprintf(msg, sizeof(msg), "gt_launch_gemm_bwd_static: set-up failed: %s", cudaGetErrorString(ce));
        return set_last_error(GT_ERR_CUDA, msg);
    }
    const int fp16 = ev.math_mode == GT_MATH_FP16;
    // 16-bit copy of dDY into the fixed array (every element that the GEMM reads is rewritten here)
    ce = launch_cast16(dDY, scratch, batch, wd->N, ld16, fp16, ev.stream);
    if (ce != cudaSuccess) return set_last_error(GT_ERR_CUDA, cudaGetErrorString(ce));
    UmmaLaunch L;
    L.w = wd;
    L.backward = 1;
    L.fp16 = fp16;
    L.act16 = scratch;
    L.ld_act = ld16;
    L.T = batch;
    L.out = dDX_accum;
    L.ld_out = wd->K;
    L.splits = umma_pick_splits(wd, 1, batch, ev.sm_count);
    L.status = ev.status;
    const char *msg = nullptr;
    ce = launch_umma_gemm(L, ev.stream, &msg);
    if (ce != cudaSuccess) return set_last_error(GT_ERR_CUDA, msg ? msg : cudaGetErrorString(ce));
    return GT_OK;
}
