"""GPU parity of the device-resident training step (gt_model_*) against the CPU chain of the restated operators
(oracle.model_forward_backward: TransformerBlock.Forward / Backward and GgufLoraModel.ForwardLossAndBackward).

Small models of the workload's architecture (pre-norm blocks, GQA attention with head_dim 128, RoPE, SwiGLU, K-quant
base projections with LoRA on all seven, fp16 embedding and LM head).  Gates follow the reference's own CPU-vs-GPU
parity test (tests/Glacier.Tune.Tests/GradientAndGpuParityTests.cs:174-260: loss difference < 2e-4, gradient cosine
> 0.9998) in the fp16 and fp32 validation modes; in the bf16 mode the per-projection 2e-2 compounds over the chain of
two blocks (gradient cosine > 0.99 is asserted); and the workload's 10-step gate: per-step loss within 1e-3 relative
over 10 optimizer steps, in both the bf16 and the fp16 mode.  The test models use zero-mean weights and norm gains
below one so that attention does not saturate (see _centered_weight).
"""
import numpy as np
import pytest

from glacier.tune_b200 import synth as S

pytestmark = pytest.mark.gpu

HYPER = dict(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


@pytest.fixture(scope="module")
def G():
    from glacier.tune_b200 import capi
    return capi


def _centered_weight(oracle, qtype, N, K, seed):
    """Seeded K-quant bytes whose weights have zero mean.  The workload's Q4_K generator gives every weight a positive
    mean (d * sc * q - dmin * m with uniform fields: about +0.2); stacked blocks of such weights push every hidden
    state onto the all-ones direction, the attention scores reach the hundreds and each softmax row is exactly one-hot
    in fp32 - dq and dk are then zero up to rounding and nothing can be compared.  Here dmin = 7.5 d and m = sc, so
    w = d * sc * (q - 7.5).  Q6_K weights (d * scale * q, q in [-32, 31]) are centred as they are."""
    w = S.make_weight(qtype, N, K, seed)
    if qtype != S.TYPE_Q4_K:
        return w
    blocks = w.reshape(-1, 144).copy()
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)
    blocks[:, 2:4] = (np.float32(7.5) * d).astype(np.float16).view(np.uint8).reshape(-1, 2)
    sc, _ = oracle.np_unpack_scales_q4k(blocks[:, 4:16])
    blocks[:, 4:16] = S.pack_scales_q4k(sc, sc)
    return blocks.reshape(-1)


def _make_model(oracle, n_layers=2, H=256, HQ=2, HK=1, F=512, V=1000, R=16, mix=False, bias=False, zero_b=False, seed=0):
    """A seeded model in the oracle's dict form (see oracle/oracle.py)."""
    rng = np.random.default_rng(seed)
    D = 128
    cfg = dict(n_heads=HQ, n_kv_heads=HK, head_dim=D, rms_eps=1e-6, rope_theta=1e6, vocab=V, hidden=H, ffn=F)
    shapes = dict(q=(HQ * D, H), k=(HK * D, H), v=(HK * D, H), o=(H, HQ * D), gate=(F, H), up=(F, H), down=(H, F))
    layers = []
    for l in range(n_layers):
        P = {}
        for j, (name, (N, K)) in enumerate(shapes.items()):
            qt = S.TYPE_Q6_K if (mix and name in ("v", "down")) else S.TYPE_Q4_K
            a = (rng.standard_normal((K, R)) * (1.0 / np.sqrt(K))).astype(np.float32)
            b = np.zeros((R, N), np.float32) if zero_b else (rng.standard_normal((R, N)) * 0.02).astype(np.float32)
            P[name] = dict(qtype=qt, w=_centered_weight(oracle, qt, N, K, seed * 1000 + 10 * l + j), N=N, K=K,
                           bias=(rng.standard_normal(N) * 0.02).astype(np.float32) if (bias and name in ("q", "k", "v")) else None,
                           a=a, b=b, rank=R, scaling=32.0 / R)
        # norm gains below one keep q, k and the FFN activations of order one (the weights' standard deviation is ~0.16)
        layers.append(dict(norm1=(0.4 * (1.0 + 0.02 * rng.standard_normal(H))).astype(np.float32),
                           norm2=(0.4 * (1.0 + 0.02 * rng.standard_normal(H))).astype(np.float32), proj=P))
    embed = (rng.standard_normal((V, H)) * 0.02).astype(np.float16)
    head = (rng.standard_normal((V, H)) * 0.02).astype(np.float16)
    return dict(cfg=cfg, layers=layers, embed=(oracle.TYPE_F16, embed), out_norm=(1.0 + 0.02 * rng.standard_normal(H)).astype(np.float32),
                lm_head=(oracle.TYPE_F16, head))


def _to_device(G, eng, model, max_tokens, checkpoint=True, graph=True):
    cfg = model["cfg"]
    m = G.Model(eng, len(model["layers"]), cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                max_tokens, cfg["rms_eps"], cfg["rope_theta"], checkpoint=checkpoint, graph=graph)
    handles = []
    for l, layer in enumerate(model["layers"]):
        ws, ads = [], []
        for name in G.PROJ_NAMES:
            p = layer["proj"][name]
            w = eng.upload_weight(p["qtype"], p["w"], p["N"], p["K"], p["bias"])
            ad = eng.create_adapter(p["K"], p["N"], p["rank"], p["scaling"] * p["rank"])
            ad.upload(p["a"], p["b"])
            ws.append(w)
            ads.append(ad)
        m.set_block(l, ws, ads, layer["norm1"], layer["norm2"])
        handles.append((ws, ads))
    emb = eng.upload_weight(G.TYPE_F16, model["embed"][1], cfg["vocab"], cfg["hidden"])
    head = eng.upload_weight(G.TYPE_F16, model["lm_head"][1], cfg["vocab"], cfg["hidden"])
    m.set_head(emb, model["out_norm"], head)
    ptr, n = m.bind_grads()
    return m, handles, (emb, head), n


def _device_grads(handles):
    parts = []
    for ws, ads in handles:
        for ad in ads:
            da, db = ad.grads()
            parts += [da.reshape(-1), db.reshape(-1)]
    return np.concatenate(parts)


def _free(m, handles, heads):
    m.close()
    for ws, ads in handles:
        for h in ws + ads:
            h.free()
    for h in heads:
        h.free()


def _cos(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def _tokens(rng, V, T):
    tokens = rng.integers(0, V, T).astype(np.int32)
    labels = np.roll(tokens, -1).astype(np.int32)
    labels[-1] = -100
    return tokens, labels


@pytest.mark.parametrize("mode,checkpoint,mix,T", [(1, True, False, 48), (1, False, True, 100), (0, True, True, 300), (2, True, False, 33)])
def test_forward_backward_matches_cpu_chain(G, oracle, mode, checkpoint, mix, T):
    eng = G.Engine(0, mode)
    model = _make_model(oracle, mix=mix, bias=True, seed=3)
    m, handles, heads, n = _to_device(G, eng, model, max_tokens=T, checkpoint=checkpoint)
    tokens, labels = _tokens(np.random.default_rng(T), model["cfg"]["vocab"], T)
    loss = m.forward_backward(tokens, labels)
    got = _device_grads(handles)
    grads = oracle.new_grads(model)
    want_loss = oracle.model_forward_backward(model, tokens, labels, grads)
    want = oracle.flat_grads(model, grads)
    assert got.size == want.size == n
    loss_tol, cos_min, fro = {0: (5e-3, 0.99, 1.5e-1), 1: (2e-4, 0.9998, 1e-2), 2: (2e-4, 0.9998, 1e-2)}[mode]
    assert abs(loss - want_loss) < loss_tol * abs(want_loss), (loss, want_loss)
    assert _cos(got, want) > cos_min, _cos(got, want)
    assert oracle.rel_fro(got, want) < fro, oracle.rel_fro(got, want)
    # the evaluation entry point computes the same loss without touching the gradients
    eval_loss, valid = m.loss(tokens, labels)
    assert valid == T - 1 and abs(eval_loss - loss) < 1e-5 * abs(loss)
    assert np.array_equal(_device_grads(handles), got)
    # gradients accumulate over micro-batches (LoraTrainer gradient accumulation): a second pass doubles them
    m.forward_backward(tokens, labels)
    assert oracle.rel_fro(_device_grads(handles), 2 * got) < (5e-3 if mode == 0 else 1e-3)      # fp32 atomics: the order of the additions varies (and with it the 16-bit rounding of X*A)
    _free(m, handles, heads)
    eng.close()


@pytest.mark.parametrize("checkpoint,mix,T,zero_b,rank", [(True, True, 300, False, 16), (False, False, 200, True, 16), (True, False, 160, False, 24)])
def test_dual_ffn_forward_matches_cpu_chain(G, oracle, checkpoint, mix, T, zero_b, rank, monkeypatch):
    """gate | up in one launch with SiLU(gate) * up formed in its epilogue (the engine takes it where the 64-feature tiles
    fill the GPU; GT_FFN_DUAL_MIN_TILES lets this small model take it too): same loss and gradients as the CPU chain, one
    SwiGLU launch less per block forward.  Also with B == 0 (no rank-update stage at all) and with rank 24 (both adapters'
    ranks, padded to 32 each, fill the one 64-deep stage)."""
    model = _make_model(oracle, mix=mix, bias=True, seed=13, zero_b=zero_b, R=rank)
    tokens, labels = _tokens(np.random.default_rng(T), model["cfg"]["vocab"], T)
    grads = oracle.new_grads(model)
    want_loss = oracle.model_forward_backward(model, tokens, labels, grads)
    want = oracle.flat_grads(model, grads)
    launches, res = [], []
    for min_tiles in ("1", "1000000"):
        monkeypatch.setenv("GT_FFN_DUAL_MIN_TILES", min_tiles)
        eng = G.Engine(0, G.MATH_BF16)
        m, handles, heads, n = _to_device(G, eng, model, max_tokens=T, checkpoint=checkpoint, graph=False)
        eng.profile_read(reset=True)
        loss = m.forward_backward(tokens, labels)
        launches.append(eng.profile_read(reset=True)["kernel_launches"])
        got = _device_grads(handles)
        assert abs(loss - want_loss) < 5e-3 * abs(want_loss), (loss, want_loss)
        assert _cos(got, want) > 0.99 and oracle.rel_fro(got, want) < 1.5e-1
        res.append((loss, got))
        _free(m, handles, heads)
        eng.close()
    # the two routes do the same arithmetic (fp32 accumulators, fp32 SiLU, one rounding to bf16): they differ by the
    # run-to-run spread of the atomic sums only
    # (measured spread of two runs of ONE route in this mode: loss a few 1e-6 relative, first-block gradients up to 6e-3)
    assert abs(res[0][0] - res[1][0]) < 2e-4 * abs(res[1][0]) and oracle.rel_fro(res[0][1], res[1][1]) < 2e-2
    n_layers = len(model["layers"])
    # every block forward (and every recomputed one: all but the last block's) runs without its SwiGLU launch
    assert launches[1] - launches[0] == n_layers + (n_layers - 1 if checkpoint else 0), launches


def test_checkpointing_changes_nothing(G, oracle):
    eng = G.Engine(0, G.MATH_FP16)
    model = _make_model(oracle, seed=5)
    tokens, labels = _tokens(np.random.default_rng(1), model["cfg"]["vocab"], 64)
    out = []
    for ck in (True, False):
        m, handles, heads, _ = _to_device(G, eng, model, max_tokens=64, checkpoint=ck)
        loss = m.forward_backward(tokens, labels)
        out.append((loss, _device_grads(handles)))
        _free(m, handles, heads)
    assert abs(out[0][0] - out[1][0]) < 1e-6 * abs(out[0][0])
    # Not bitwise: split-K partial tiles and X*A are summed with fp32 atomics, and a last-bit difference of such a sum can
    # move the fp16 rounding of the next GEMM's operand by a whole fp16 step.  Two runs of the SAME configuration differ
    # by up to 5e-4 in the first block's q, k, v gradients at this size (measured over repeated runs); recomputing the
    # forward adds nothing to that.
    assert oracle.rel_fro(out[0][1], out[1][1]) < 2e-3
    eng.close()


@pytest.mark.parametrize("mix", [False, True])
def test_captured_step_matches_eager_launches(G, oracle, mix):
    """From the third call on gt_model_forward_backward replays a CUDA graph of the step.  Four accumulating passes and
    then three optimizer steps, once with the graph and once with one launch per kernel: same losses, same accumulated
    gradients (up to the run-to-run spread of the fp32 atomic sums), and the graph must in fact have been used."""
    eng = G.Engine(0, G.MATH_FP16)
    model = _make_model(oracle, mix=mix, seed=21)
    tokens, labels = _tokens(np.random.default_rng(3), model["cfg"]["vocab"], 64)
    out = []
    for graph in (True, False):
        m, handles, heads, _ = _to_device(G, eng, model, max_tokens=64, graph=graph)
        losses = [m.forward_backward(tokens, labels) for _ in range(4)]
        grads = _device_grads(handles)
        for step in range(1, 4):
            m.optimizer_step(step=step, max_norm=1.0, **HYPER)
            losses.append(m.forward_backward(tokens, labels))
        info = m.step_info()
        # (the call after the first eager one captures, unless a buffer still moved in between - then the one after)
        assert info["graph_ready"] == graph and (5 <= info["replays"] <= 6 if graph else info["replays"] == 0)
        assert (info["kernels_per_replay"] > 50) == graph
        out.append((np.array(losses), grads))
        _free(m, handles, heads)
    assert np.all(np.isfinite(out[0][0])) and out[0][0][-1] < out[0][0][0]
    assert np.max(np.abs(out[0][0][:4] - out[0][0][0])) < 1e-5 * out[0][0][0]      # the same pass four times
    # (after optimizer steps the two runs' parameters differ by the spread that Adam's normalisation amplifies)
    assert np.max(np.abs(out[0][0] - out[1][0]) / np.abs(out[1][0])) < 5e-4
    assert oracle.rel_fro(out[0][1], out[1][1]) < 2e-3
    eng.close()


def test_captured_step_follows_the_token_count(G, oracle):
    """Another token count drops the captured step and captures a new one; profiling switches replay off for the call.
    The loss of every call equals the loss of the same call on a model that never captures."""
    eng = G.Engine(0, G.MATH_FP16)
    model = _make_model(oracle, seed=22)
    rng = np.random.default_rng(4)
    seqs = {T: _tokens(rng, model["cfg"]["vocab"], T) for T in (64, 40)}
    plan = [64, 64, 64, 40, 40, 40, 40, 64, 64, 64]
    res = []
    for graph in (True, False):
        m, handles, heads, _ = _to_device(G, eng, model, max_tokens=64, graph=graph)
        losses, replays = [], []
        for i, T in enumerate(plan):
            if i == 8:
                eng.profile_enable(True)
            losses.append(m.forward_backward(*seqs[T]))
            if i == 8:
                eng.profile_enable(False)
            replays.append(m.step_info()["replays"])
        res.append((losses, replays))
        _free(m, handles, heads)
    # a new token count (calls 3 and 7) and profiling (call 8) launch eagerly; the call after an eager one captures the
    # step and launches the new graph, which counts as a replay
    r = res[0][1]
    assert r[0] == 0 and r[2] >= 1 and r[3] == r[2] and r[6] >= r[3] + 2 and r[7] == r[6] and r[8] == r[7] and r[9] == r[8] + 1
    assert res[1][1] == [0] * 10
    for a, b in zip(res[0][0], res[1][0]):
        assert abs(a - b) < 1e-5 * abs(b)
    eng.close()


@pytest.mark.parametrize("mode", [0, 1])
def test_ten_step_loss_gate(G, oracle, mode):
    """10 optimizer steps from the standard initial state (B = 0, so step 0 takes the zero-delta path and dA = 0):
    per-step loss within 1e-3 relative of the CPU chain (clip 1.0, AdamW), which trains its own copy of the adapters."""
    eng = G.Engine(0, mode)
    model = _make_model(oracle, zero_b=True, mix=True, seed=7)
    T = 64
    m, handles, heads, n = _to_device(G, eng, model, max_tokens=T)
    rng = np.random.default_rng(11)
    tokens, labels = _tokens(rng, model["cfg"]["vocab"], T)
    # CPU side: flat parameter views in the same order as the flat gradient buffer
    params = []
    for layer in model["layers"]:
        for name in G.PROJ_NAMES:
            params += [layer["proj"][name]["a"], layer["proj"][name]["b"]]
    mom = [(np.zeros_like(p), np.zeros_like(p)) for p in params]
    losses_gpu, losses_cpu = [], []
    for step in range(1, 11):
        losses_gpu.append(m.forward_backward(tokens, labels))
        if step == 1:
            g0 = _device_grads(handles)
            off = 0
            for pa, pb in zip(params[::2], params[1::2]):      # every dA is exactly zero while B == 0, every dB is not
                assert np.all(g0[off:off + pa.size] == 0.0)
                assert np.any(g0[off + pa.size:off + pa.size + pb.size] != 0.0)
                off += pa.size + pb.size
        norm = m.optimizer_step(step=step, max_norm=1.0, want_norm=True, **HYPER)
        grads = oracle.new_grads(model)
        losses_cpu.append(oracle.model_forward_backward(model, tokens, labels, grads))
        flat = oracle.flat_grads(model, grads)
        cpu_norm = oracle.clip_gradients(flat, 1.0)
        assert abs(norm - cpu_norm) < 2e-2 * max(cpu_norm, 1e-12), (step, norm, cpu_norm)
        off = 0
        for p, (mm, vv) in zip(params, mom):
            oracle.adamw_step(p.reshape(-1), flat[off:off + p.size], mm.reshape(-1), vv.reshape(-1), step=step, **HYPER)
            off += p.size
    rel = [abs(a - b) / abs(b) for a, b in zip(losses_gpu, losses_cpu)]
    assert max(rel) < 1e-3, (rel, losses_gpu, losses_cpu)
    assert losses_cpu[-1] < losses_cpu[0]              # the adapters learn: the loss on the repeated batch goes down
    # after the optimizer step the gradient buffer is zero again
    assert np.all(_device_grads(handles) == 0.0)
    _free(m, handles, heads)
    eng.close()


def test_model_argument_checks(G, oracle):
    eng = G.Engine(0, G.MATH_BF16)
    with pytest.raises(G.GtError):
        G.Model(eng, 1, 256, 3, 2, 128, 512, 1000, 64)              # heads not a multiple of KV heads
    with pytest.raises(G.GtError):
        G.Model(eng, 1, 256, 4, 2, 64, 512, 1000, 64)               # head_dim 64
    model = _make_model(oracle, n_layers=1, seed=9)
    m, handles, heads, _ = _to_device(G, eng, model, max_tokens=32)
    with pytest.raises(G.GtError):
        m.forward_backward(np.zeros(33, np.int32), np.zeros(33, np.int32))      # longer than max_tokens
    with pytest.raises(G.GtError):
        m.forward_backward(np.array([1, 5000], np.int32), np.array([2, 3], np.int32))   # token outside the vocabulary
    _free(m, handles, heads)
    eng.close()
