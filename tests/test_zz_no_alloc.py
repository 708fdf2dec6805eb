"""GPU test of gt_launch_gemm_bwd_static, the entry point that allocates nothing.

Some hosts cannot call cudaMalloc when they run a training step: they are inside a CUDA stream capture, or in a
loop that cannot take the device-wide synchronisation an allocation implies, or their memory already belongs to
a pool.  For them the library keeps the 16-bit operand copy of the input-gradient GEMM in a fixed 4 MiB array
instead of the engine's grow-only buffer.  This file checks, through the C ABI, that the variant returns what
gt_launch_gemm_bwd returns on two calls in a row (the second one smaller, so stale contents of the shared array
would show), that it accumulates into dDX like the regular call, that it agrees with the CPU path within the
bf16 gate, that the device's free memory is the same before and after a call at a batch no earlier call has seen,
and that it refuses sizes beyond its array.
It is collected last so that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest

from glacier.tune_b200 import synth as S

pytestmark = pytest.mark.gpu

TOL = 1e-5      # both paths run the same kernels; only the fp32 order of the split-K atomics differs


def _rel(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def test_static_scratch_backward_matches_regular_entry_point():
    import torch
    from glacier.tune_b200 import capi as G
    eng = G.Engine(0, G.MATH_BF16)
    try:
        # (qtype, out, in, batch): the second call is smaller than the first and uses a padded row length (out % 8 != 0)
        for qtype, N, K, T in ((S.TYPE_Q4_K, 3584, 512, 512), (S.TYPE_Q6_K, 100, 256, 37)):
            c = S.make_projection_case(qtype, N, K, T, seed=N + T)
            w = eng.upload_weight(qtype, c["w"], N, K)
            dY = torch.from_numpy(c["dy"]).cuda()
            base = torch.full((T, K), 0.25, device="cuda")
            want = base.clone()
            got = base.clone()
            eng.launch_gemm_bwd(w, want, dY, T)
            eng.launch_gemm_bwd_static(w, got, dY, T)      # first call on this device: looks the array's address up
            eng.sync()
            torch.cuda.synchronize()
            assert _rel(got.cpu().numpy(), want.cpu().numpy()) < TOL
            assert float((got - base).abs().max()) > 0.0          # it really accumulated something
            # and against the CPU restatement of the reference's input-gradient product (bf16 operands: 2e-2)
            from oracle import oracle as O
            O.build()
            ref = O.base_backward_f64(qtype, c["w"], c["dy"], K, N, T)
            assert _rel(got.cpu().numpy().astype(np.float64) - 0.25, ref) < 2e-2
            # the point of the entry point: a call takes no device memory (free memory is the same before and after)
            again = base.clone()
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            eng.launch_gemm_bwd_static(w, again, dY, T)
            eng.sync()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, (free_before, free_after)
            assert _rel(again.cpu().numpy(), want.cpu().numpy()) < TOL
            w.free()
        # a size beyond the fixed array is refused with a clear message and launches nothing
        N, K, T = 18944, 256, 512
        c = S.make_projection_case(S.TYPE_Q4_K, N, K, T, seed=3)
        w = eng.upload_weight(S.TYPE_Q4_K, c["w"], N, K)
        dY = torch.from_numpy(c["dy"]).cuda()
        dX = torch.zeros((T, K), device="cuda")
        with pytest.raises(G.GtError) as ei:
            eng.launch_gemm_bwd_static(w, dX, dY, T)
        assert ei.value.code == -2 and "fixed array" in str(ei.value)
        eng.sync()
        assert float(dX.abs().max()) == 0.0
        w.free()
    finally:
        eng.close()
