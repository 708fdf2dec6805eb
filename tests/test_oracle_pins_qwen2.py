"""CPU tests: the oracle's layer operators, and its whole training-step chain, against the Qwen2 definitions that ship
with `transformers` and against torch autograd - independent implementations of the architecture the workload names (Qwen2.5-7B: RMSNorm with eps 1e-6,
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


def _qwen2_params(oracle, model, adapters):
    """State dict of a Qwen2ForCausalLM built from the oracle's model dict: every projection weight is the exactly
    dequantized base plus the adapter's delta s * (A B)^T, with A and B the torch leaves in `adapters`."""
    cfg = model["cfg"]
    H = cfg["hidden"]
    names = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj", "gate": "mlp.gate_proj",
             "up": "mlp.up_proj", "down": "mlp.down_proj"}
    sd = {}
    et, ew = model["embed"]
    lt, lw = model["lm_head"]
    sd["model.embed_tokens.weight"] = torch.from_numpy(oracle.dequant_rows(et, ew, H, 0, cfg["vocab"]).reshape(cfg["vocab"], H)).double()
    sd["lm_head.weight"] = torch.from_numpy(oracle.dequant_rows(lt, lw, H, 0, cfg["vocab"]).reshape(cfg["vocab"], H)).double()
    sd["model.norm.weight"] = torch.from_numpy(model["out_norm"]).double()
    for l, layer in enumerate(model["layers"]):
        pre = f"model.layers.{l}."
        sd[pre + "input_layernorm.weight"] = torch.from_numpy(layer["norm1"]).double()
        sd[pre + "post_attention_layernorm.weight"] = torch.from_numpy(layer["norm2"]).double()
        for name, mod in names.items():
            p = layer["proj"][name]
            W = torch.from_numpy(oracle.dequant_rows(p["qtype"], p["w"], p["K"], 0, p["N"]).reshape(p["N"], p["K"])).double()
            A, B = adapters[l][name]
            sd[pre + mod + ".weight"] = W + p["scaling"] * (A @ B).T
            if name in ("q", "k", "v"):
                bias = p["bias"] if p["bias"] is not None else np.zeros(p["N"], np.float32)
                sd[pre + mod + ".bias"] = torch.from_numpy(bias).double()
    return sd


@pytest.mark.parametrize("mix", [False, True])
def test_model_chain_matches_qwen2_for_causal_lm(oracle, mix):
    """The CPU chain of the training step (oracle.model_forward_backward: the order of TransformerBlock.Forward / Backward and
    GgufLoraModel.ForwardLossAndBackward) against `Qwen2ForCausalLM` of the transformers package in fp64, built from the same
    dequantized weights with the adapters merged as differentiable terms: the loss, and the gradient of every A and B."""
    transformers = pytest.importorskip("transformers")
    from test_gpu_model import _make_model, _tokens
    model = _make_model(oracle, n_layers=2, H=256, HQ=2, HK=1, F=512, V=300, mix=mix, bias=True, seed=31)
    cfg = model["cfg"]
    T = 24
    tokens, labels = _tokens(np.random.default_rng(7), cfg["vocab"], T)
    grads = oracle.new_grads(model)
    loss = oracle.model_forward_backward(model, tokens, labels, grads)
    got = oracle.flat_grads(model, grads)

    hf_cfg = transformers.Qwen2Config(vocab_size=cfg["vocab"], hidden_size=cfg["hidden"], intermediate_size=cfg["ffn"],
                                      num_hidden_layers=len(model["layers"]), num_attention_heads=cfg["n_heads"],
                                      num_key_value_heads=cfg["n_kv_heads"], rms_norm_eps=cfg["rms_eps"], max_position_embeddings=64,
                                      rope_parameters={"rope_type": "default", "rope_theta": cfg["rope_theta"]},
                                      tie_word_embeddings=False, use_sliding_window=False, attention_dropout=0.0)
    hf_cfg._attn_implementation = "eager"
    assert hf_cfg.hidden_size // hf_cfg.num_attention_heads == cfg["head_dim"]
    hf = transformers.Qwen2ForCausalLM(hf_cfg).double().eval()
    adapters = []
    for layer in model["layers"]:
        adapters.append({name: (torch.from_numpy(layer["proj"][name]["a"]).double().requires_grad_(True),
                                torch.from_numpy(layer["proj"][name]["b"]).double().requires_grad_(True)) for name in oracle.PROJ_NAMES})
    sd = _qwen2_params(oracle, model, adapters)
    ids = torch.from_numpy(tokens.astype(np.int64))[None]
    out = torch.func.functional_call(hf, sd, (ids,), {"use_cache": False})
    logits = out.logits[0]                                                    # [T, vocab]
    want_loss = torch.nn.functional.cross_entropy(logits, torch.from_numpy(labels.astype(np.int64)), ignore_index=-100)
    want_loss.backward()
    want = np.concatenate([t.grad.numpy().reshape(-1) for ad in adapters for name in oracle.PROJ_NAMES for t in ad[name]])
    ref_loss = float(want_loss.detach())
    assert abs(loss - ref_loss) < 2e-6 * abs(ref_loss), (loss, ref_loss)
    assert want.size == got.size
    cos = float(got.astype(np.float64) @ want / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos > 0.999999 and oracle.rel_fro(got, want) < 2e-4, (cos, oracle.rel_fro(got, want))


@pytest.mark.parametrize("qname", ["Q4_K", "Q6_K"])
def test_lora_projection_matches_torch_autograd(oracle, qname):
    """LoraAdapter.Forward / Backward on the CPU path (Y = X W^T + b + s (X A) B; dX, dA, dB) against torch autograd in fp64
    over the exactly dequantized weight."""
    from glacier.tune_b200 import synth as S
    qt = S.TYPE_Q4_K if qname == "Q4_K" else S.TYPE_Q6_K
    c = S.make_projection_case(qt, 96, 512, 11, seed=77)
    N, K, T, R, s = c["N"], c["K"], 11, 16, c["scaling"]
    bias = (0.1 * np.random.default_rng(5).standard_normal(N)).astype(np.float32)
    W = torch.from_numpy(oracle.dequant_rows(qt, c["w"], K, 0, N).reshape(N, K)).double()
    X, A, B = _t(c["x"]), _t(c["a"]), _t(c["b"])
    Y = X @ W.T + torch.from_numpy(bias).double() + s * (X @ A) @ B
    Y.backward(torch.from_numpy(c["dy"]).double())
    y = oracle.proj_forward(qt, c["w"], bias, c["x"], K, N, T, c["a"], c["b"], R, s)
    dx, da, db = oracle.proj_backward(qt, c["w"], c["dy"], c["x"], K, N, T, c["a"], c["b"], R, s)
    assert oracle.rel_fro(y, Y.detach().numpy()) < 1e-6
    assert oracle.rel_fro(dx, X.grad.numpy()) < 1e-6
    assert oracle.rel_fro(da, A.grad.numpy()) < 1e-6 and oracle.rel_fro(db, B.grad.numpy()) < 1e-6


def test_cross_entropy_matches_torch(oracle):
    """The streaming cross-entropy (vocabulary tiles, ignored labels) against torch.nn.functional.cross_entropy in fp64."""
    rng = np.random.default_rng(8)
    T, H, V = 9, 48, 1000
    hidden = rng.standard_normal((T, H)).astype(np.float32)
    W = (0.2 * rng.standard_normal((V, H))).astype(np.float32)
    labels = rng.integers(0, V, T).astype(np.int32)
    labels[3] = -100
    ht = _t(hidden)
    want = torch.nn.functional.cross_entropy(ht @ torch.from_numpy(W).double().T, torch.from_numpy(labels.astype(np.int64)), ignore_index=-100)
    want.backward()
    loss, valid, dh = oracle.cross_entropy(oracle.TYPE_F32, W, hidden, labels, V, tile=256)
    assert valid == T - 1 and abs(loss - float(want.detach())) < 1e-6 * float(want.detach())
    assert oracle.rel_fro(dh, ht.grad.numpy()) < 1e-5 and np.all(dh[3] == 0.0)


def test_clip_matches_torch_clip_grad_norm(oracle):
    """ClipGradients (global L2 norm over every gradient, scale by max / (norm + 1e-6) when above) against
    torch.nn.utils.clip_grad_norm_, which uses the same epsilon."""
    rng = np.random.default_rng(9)
    g = (3 * rng.standard_normal(5000)).astype(np.float32)
    p = torch.nn.Parameter(torch.zeros(5000, dtype=torch.float64))
    p.grad = torch.from_numpy(g).double()
    want_norm = float(torch.nn.utils.clip_grad_norm_([p], max_norm=1.0))
    got = g.copy()
    norm = oracle.clip_gradients(got, 1.0)
    assert abs(norm - want_norm) < 1e-6 * want_norm
    assert oracle.rel_fro(got, p.grad.numpy()) < 1e-6
