"""CPU tests: the oracle's layer operators against the Qwen2 definitions that ship with `transformers` and against torch
autograd - independent implementations of the architecture the workload names (Qwen2.5-7B: RMSNorm with eps 1e-6,
rotate-half RoPE with theta 1e6, SwiGLU, causal grouped-query attention with 1/sqrt(head_dim) scaling).

The reference's RMSNorm lives in a package that is not in its repository, so the oracle restates the textbook form;
these tests pin that form (forward and backward) to `Qwen2RMSNorm`, and pin the operators the oracle restates from the
reference's own files (RoPEKernel.cs, SwiGluKernel.cs, CausalAttentionKernel.cs) to a second, independent source.
Skipped when `transformers` / torch cannot be imported.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
qwen2 = pytest.importorskip("transformers.models.qwen2.modeling_qwen2")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).double().requires_grad_(True)


def test_rmsnorm_matches_qwen2_rmsnorm(oracle):
    rng = np.random.default_rng(1)
    T, H = 7, 96
    x = rng.standard_normal((T, H)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    dy = rng.standard_normal((T, H)).astype(np.float32)
    norm = qwen2.Qwen2RMSNorm(H, eps=1e-6).double()
    with torch.no_grad():
        norm.weight.copy_(torch.from_numpy(w).double())
    xt = _t(x)
    y = norm(xt)
    y.backward(torch.from_numpy(dy).double())
    assert np.allclose(oracle.rmsnorm_forward(x, w, 1e-6), y.detach().numpy(), rtol=2e-6, atol=2e-6)
    assert np.allclose(oracle.rmsnorm_backward(dy, x, w, 1e-6), xt.grad.numpy(), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("theta", [1e6, 1e4])
def test_rope_matches_qwen2_rotary_embedding(oracle, theta):
    rng = np.random.default_rng(2)
    T, hq, hk, d = 9, 4, 2, 32
    q = rng.standard_normal((T, hq * d)).astype(np.float32)
    k = rng.standard_normal((T, hk * d)).astype(np.float32)
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv_freq[None, :]
    emb = torch.cat([ang, ang], dim=-1)                       # rotate-half layout: element i pairs with i + d / 2
    cos, sin = emb.cos()[None], emb.sin()[None]               # [1, T, d]
    qt = torch.from_numpy(q).double().view(1, T, hq, d).transpose(1, 2)      # [batch, heads, T, d]
    kt = torch.from_numpy(k).double().view(1, T, hk, d).transpose(1, 2)
    q_rot, k_rot = qwen2.apply_rotary_pos_emb(qt, kt, cos, sin)
    want_q = q_rot.transpose(1, 2).reshape(T, hq * d).numpy()
    want_k = k_rot.transpose(1, 2).reshape(T, hk * d).numpy()
    got_q, got_k = oracle.rope(q, k, T, hq, hk, d, theta)
    # fp32 angles (as the reference computes them) against fp64: a few 1e-6 at these positions
    assert np.allclose(got_q, want_q, atol=2e-5) and np.allclose(got_k, want_k, atol=2e-5)
    # the inverse rotation undoes it
    back_q, back_k = oracle.rope(got_q, got_k, T, hq, hk, d, theta, inverse=True)
    assert np.allclose(back_q, q, atol=2e-6) and np.allclose(back_k, k, atol=2e-6)


def test_swiglu_matches_torch_silu(oracle):
    rng = np.random.default_rng(3)
    g = (3 * rng.standard_normal((5, 40))).astype(np.float32)
    u = rng.standard_normal((5, 40)).astype(np.float32)
    dh = rng.standard_normal((5, 40)).astype(np.float32)
    gt, ut = _t(g), _t(u)
    h = torch.nn.functional.silu(gt) * ut                     # Qwen2MLP: down(act(gate(x)) * up(x)), act = SiLU
    h.backward(torch.from_numpy(dh).double())
    assert np.allclose(oracle.swiglu_forward(g, u), h.detach().numpy(), rtol=1e-5, atol=1e-6)
    dg, du = oracle.swiglu_backward(dh, g, u)
    assert np.allclose(dg, gt.grad.numpy(), rtol=1e-5, atol=1e-6) and np.allclose(du, ut.grad.numpy(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("T,hq,hk,d", [(13, 4, 2, 16), (33, 6, 1, 32)])
def test_attention_matches_torch_causal_gqa(oracle, T, hq, hk, d):
    rng = np.random.default_rng(4)
    q = rng.standard_normal((T, hq * d)).astype(np.float32)
    k = rng.standard_normal((T, hk * d)).astype(np.float32)
    v = rng.standard_normal((T, hk * d)).astype(np.float32)
    d_out = rng.standard_normal((T, hq * d)).astype(np.float32)
    qt, kt, vt = _t(q), _t(k), _t(v)
    rep = hq // hk
    qh = qt.view(T, hq, d).transpose(0, 1)                                        # [heads, T, d]
    kh = kt.view(T, hk, d).transpose(0, 1).repeat_interleave(rep, dim=0)          # query head h reads KV head h / rep
    vh = vt.view(T, hk, d).transpose(0, 1).repeat_interleave(rep, dim=0)
    o = torch.nn.functional.scaled_dot_product_attention(qh[None], kh[None], vh[None], is_causal=True)[0]
    out = o.transpose(0, 1).reshape(T, hq * d)
    out.backward(torch.from_numpy(d_out).double())
    got, probs = oracle.attention_forward(q, k, v, hq, hk, d)
    assert np.allclose(got, out.detach().numpy(), rtol=1e-5, atol=2e-6)
    dq, dk, dv = oracle.attention_backward(d_out, q, k, v, probs, hq, hk, d)
    assert np.allclose(dq, qt.grad.numpy(), rtol=1e-4, atol=5e-6)
    assert np.allclose(dk, kt.grad.numpy(), rtol=1e-4, atol=5e-6)
    assert np.allclose(dv, vt.grad.numpy(), rtol=1e-4, atol=5e-6)
