"""GPU parity of the causal grouped-query attention calls through the C ABI against the CPU restatement of
CausalAttentionKernel.Forward / Backward (src/Glacier.Tune/Kernels/CausalAttentionKernel.cs:17-213).

Gates: relative Frobenius error 2e-2 with bf16 MMA operands (the bf16 math mode), 2e-3 with fp16 operands (the
validation modes); the causal mask is checked the way the reference's test does (tests/Glacier.Tune.Tests/KernelTests.cs:99-131):
changing a later key / value must not change an earlier output row.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

D = 128
TOL = {0: 2e-2, 1: 2e-3, 2: 2e-3}


@pytest.fixture(scope="module")
def G():
    from glacier.tune_b200 import capi
    return capi


@pytest.fixture(scope="module")
def eng(G):
    e = G.Engine(0, G.MATH_BF16)
    yield e
    e.close()


def _run(eng, q, k, v, g, T, HQ, HK):
    import torch
    qd, kd, vd, gd = (torch.from_numpy(a).cuda() for a in (q, k, v, g))
    out = torch.empty_like(qd)
    lse = torch.empty((HQ, T), device="cuda")
    dq, dk, dv = torch.full_like(qd, 3.0), torch.full_like(kd, 3.0), torch.full_like(vd, 3.0)      # stale contents: overwritten
    eng.attention_forward(qd, kd, vd, out, lse, T, HQ, HK, D)
    eng.attention_backward(gd, qd, kd, vd, out, lse, dq, dk, dv, T, HQ, HK, D)
    eng.sync()
    return out.cpu().numpy(), dq.cpu().numpy(), dk.cpu().numpy(), dv.cpu().numpy(), lse.cpu().numpy()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("T,HQ,HK", [(64, 4, 2), (1, 2, 1), (37, 2, 2), (100, 6, 2), (200, 8, 1), (512, 28, 4)])
def test_attention_forward_backward_parity(G, eng, oracle, mode, T, HQ, HK):
    eng.set_math_mode(mode)
    rng = np.random.default_rng(T * 31 + HQ)
    q = rng.standard_normal((T, HQ * D), dtype=np.float32)
    k = rng.standard_normal((T, HK * D), dtype=np.float32)
    v = rng.standard_normal((T, HK * D), dtype=np.float32)
    g = rng.standard_normal((T, HQ * D), dtype=np.float32)
    out, dq, dk, dv, lse = _run(eng, q, k, v, g, T, HQ, HK)
    want, probs = oracle.attention_forward(q, k, v, HQ, HK, D)
    wdq, wdk, wdv = oracle.attention_backward(g, q, k, v, probs, HQ, HK, D)
    errs = dict(out=oracle.rel_fro(out, want), dq=oracle.rel_fro(dq, wdq), dk=oracle.rel_fro(dk, wdk), dv=oracle.rel_fro(dv, wdv))
    if T == 1:
        # one key: the softmax is the constant 1, so dq and dk are zero up to rounding on both sides - compare absolutely
        scale = float(np.abs(g).max() * np.abs(v).max())
        assert errs["out"] < TOL[mode] and errs["dv"] < TOL[mode], errs
        assert np.abs(dq).max() < TOL[mode] * scale and np.abs(dk).max() < TOL[mode] * scale
    else:
        assert all(e < TOL[mode] for e in errs.values()), errs
    eng.set_math_mode(0)


def test_attention_causal_mask_and_rerun_bitwise(G, eng, oracle):
    """Position i does not see j > i; and two runs on the same inputs give the same bits (no atomics anywhere)."""
    eng.set_math_mode(0)
    T, HQ, HK = 130, 4, 2
    rng = np.random.default_rng(3)
    q = rng.standard_normal((T, HQ * D), dtype=np.float32)
    k = rng.standard_normal((T, HK * D), dtype=np.float32)
    v = rng.standard_normal((T, HK * D), dtype=np.float32)
    g = rng.standard_normal((T, HQ * D), dtype=np.float32)
    a = _run(eng, q, k, v, g, T, HQ, HK)
    b = _run(eng, q, k, v, g, T, HQ, HK)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    k2, v2 = k.copy(), v.copy()
    k2[-1] += 3.0
    v2[-1] -= 2.0
    c = _run(eng, q, k2, v2, g, T, HQ, HK)
    assert np.array_equal(c[0][:-1], a[0][:-1]) and not np.array_equal(c[0][-1], a[0][-1])


def test_attention_argument_checks(G, eng):
    import torch
    t = torch.zeros((4, 64), device="cuda")
    with pytest.raises(G.GtError):
        eng.attention_forward(t, t, t, t, t, 4, 1, 1, 64)              # head_dim 64 is not served
    with pytest.raises(G.GtError):
        eng.attention_forward(t, t, t, t, t, 4, 3, 2, 128)             # heads_q not a multiple of heads_kv
    assert G.load_library().gt_supports_attention(512, 128) == 1 and G.load_library().gt_supports_attention(512, 64) == 0
