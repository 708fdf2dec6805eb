"""GPU parity of the LM-head calls through the C ABI: streaming cross-entropy with its input gradient, full logits and
the embedding lookup, against the CPU restatement of FusedCrossEntropyLoss.ComputeLossAndGradients
(src/Glacier.Tune/Kernels/FusedCrossEntropyLoss.cs:170-364) on an fp16 LM head.

The device GEMMs use fp16 operands with fp32 accumulation (hidden states and probabilities are rounded to fp16), so
the gates are the fp16 validation mode's: loss within 1e-3 relative, gradient within 1e-3 relative Frobenius error
(5e-3 at 4 tokens, where nothing averages the rounding).
"""
import numpy as np
import pytest

from glacier.tune_b200 import synth as S

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    from glacier.tune_b200 import capi
    return capi


@pytest.fixture(scope="module")
def eng(G):
    e = G.Engine(0, G.MATH_BF16)
    yield e
    e.close()


def _head(rng, V, H, std=0.02):
    w = np.empty((V, H), np.float16)
    for v0 in range(0, V, 16384):
        v1 = min(V, v0 + 16384)
        w[v0:v1] = (rng.standard_normal((v1 - v0, H), dtype=np.float32) * np.float32(std)).astype(np.float16)
    return w


@pytest.mark.parametrize("V,H,T", [(1024, 128, 4), (4096, 128, 4), (8192, 256, 4), (16384, 128, 4), (1000, 256, 37), (5000, 384, 300),
                                   (40000, 256, 600)])
def test_cross_entropy_matches_cpu_path(G, eng, oracle, V, H, T):
    """Vocabulary below, at and above one tile, not a multiple of 128, CTA-pair and two-chunk token counts; one ignored
    label (-100) and one out-of-range label, whose gradient rows must be exactly zero."""
    rng = np.random.default_rng(V + T)
    W = _head(rng, V, H, std=0.05)
    hidden = (rng.standard_normal((T, H), dtype=np.float32) * np.float32(2.0)).astype(np.float32)
    labels = rng.integers(0, V, T).astype(np.int32)
    labels[2] = -100
    if T > 8:
        labels[7] = V + 5
    w = eng.upload_weight(G.TYPE_F16, W, V, H)
    loss, valid, dh = eng.lm_head_loss(w, hidden, labels)
    want_loss, want_valid, want_dh = oracle.cross_entropy(oracle.TYPE_F16, W, hidden, labels, V)
    assert valid == want_valid
    assert abs(loss - want_loss) < 1e-3 * abs(want_loss), (loss, want_loss)
    assert np.all(dh[2] == 0.0)
    if T > 8:
        assert np.all(dh[7] == 0.0)
    tol = 5e-3 if T <= 8 else 1e-3
    assert oracle.rel_fro(dh, want_dh) < tol, oracle.rel_fro(dh, want_dh)
    # loss only (the evaluation path): same loss, no gradient
    loss2, valid2, none = eng.lm_head_loss(w, hidden, labels, want_grad=False)
    assert none is None and valid2 == valid and abs(loss2 - loss) < 1e-6 * abs(loss)
    w.free()


def test_cross_entropy_device_pointers_and_no_valid_label(G, eng, oracle):
    import torch
    rng = np.random.default_rng(5)
    V, H, T = 3000, 256, 64
    W = _head(rng, V, H, std=0.05)
    hidden = rng.standard_normal((T, H), dtype=np.float32)
    labels = rng.integers(0, V, T).astype(np.int32)
    w = eng.upload_weight(G.TYPE_F16, W, V, H)
    hd, ld = torch.from_numpy(hidden).cuda(), torch.from_numpy(labels).cuda()
    loss_d = torch.zeros(1, device="cuda")
    valid_d = torch.zeros(1, dtype=torch.int32, device="cuda")
    dh_d = torch.full((T, H), 9.0, device="cuda")
    eng.lm_head_loss(w, hd, ld, loss_dev=loss_d, valid_dev=valid_d, d_hidden=dh_d)
    eng.sync()
    want_loss, want_valid, want_dh = oracle.cross_entropy(oracle.TYPE_F16, W, hidden, labels, V)
    assert int(valid_d.item()) == want_valid == T
    assert abs(float(loss_d.item()) - want_loss) < 1e-3 * want_loss
    assert oracle.rel_fro(dh_d.cpu().numpy(), want_dh) < 1e-3
    # no valid label at all: loss 0, gradient all zero (FusedCrossEntropyLoss.cs:196)
    none = np.full(T, -100, np.int32)
    loss, valid, dh = eng.lm_head_loss(w, hidden, none)
    assert loss == 0.0 and valid == 0 and np.all(dh == 0.0)
    w.free()


def test_full_logits_and_embedding_rows(G, eng, oracle):
    import torch
    rng = np.random.default_rng(6)
    V, H, T = 2048, 256, 50
    W = _head(rng, V, H, std=0.05)
    hidden = rng.standard_normal((T, H), dtype=np.float32)
    w = eng.upload_weight(G.TYPE_F16, W, V, H)
    logits = torch.empty((T, V), device="cuda")
    eng.lm_head_logits(w, torch.from_numpy(hidden).cuda(), logits)
    eng.sync()
    want = oracle.matmul_batch(oracle.TYPE_F16, W, hidden, H, V, T, None, f64=True)
    assert oracle.rel_fro(logits.cpu().numpy(), want) < 1e-3
    # embedding rows: exact fp16 -> fp32
    tokens = np.array([0, 5, V - 1, 77, 5], np.int32)
    rows = eng.embedding(w, tokens)
    assert np.array_equal(rows, W[tokens].astype(np.float32))
    with pytest.raises(G.GtError):
        eng.embedding(w, np.array([1, V], np.int32))               # outside the vocabulary
    w.free()
    # a K-quant embedding: bit-exact rows, as the row decoder's
    c = S.make_projection_case(S.TYPE_Q4_K, 300, 512, 1, seed=12)
    wq = eng.upload_weight(S.TYPE_Q4_K, c["w"], 300, 512)
    tok = np.array([299, 0, 123], np.int32)
    got = eng.embedding(wq, tok)
    want_rows = np.concatenate([oracle.dequant_rows(S.TYPE_Q4_K, c["w"], 512, int(t), 1) for t in tok])
    assert np.array_equal(got.view(np.uint32), want_rows.view(np.uint32))
    wq.free()


def test_f16_projection_runs_on_the_exact_kernels(G, eng, oracle):
    """An F16 tensor as a LoRA projection base (not a workload case): served by the fp32 CUDA-core kernels."""
    rng = np.random.default_rng(9)
    N, K, T = 96, 256, 20
    W = _head(rng, N, K, std=0.05)
    x = rng.standard_normal((T, K), dtype=np.float32)
    dy = rng.standard_normal((T, N), dtype=np.float32)
    w = eng.upload_weight(G.TYPE_F16, W, N, K)
    y = eng.forward(w, None, x)
    dx = np.zeros((T, K), np.float32)
    eng.backward(w, None, dy, None, dx)
    Wf = W.astype(np.float64)
    assert oracle.rel_fro(y, x.astype(np.float64) @ Wf.T) < 1e-5
    assert oracle.rel_fro(dx, dy.astype(np.float64) @ Wf) < 1e-5
    w.free()


def test_full_size_head_152064_by_3584_at_512_tokens(G, eng, oracle):
    """The workload's LM head: vocabulary 152064, hidden 3584, fp16 ~ N(0, 0.02), 512 tokens, last label ignored."""
    rng = np.random.default_rng(2024)
    V, H, T = 152064, 3584, 512
    W = _head(rng, V, H)
    hidden = rng.standard_normal((T, H), dtype=np.float32)
    labels = rng.integers(0, V, T).astype(np.int32)
    labels[-1] = -100
    w = eng.upload_weight(G.TYPE_F16, W, V, H)
    loss, valid, dh = eng.lm_head_loss(w, hidden, labels)
    want_loss, want_valid, want_dh = oracle.cross_entropy(oracle.TYPE_F16, W, hidden, labels, V)
    assert valid == want_valid == T - 1
    assert abs(loss - want_loss) < 1e-3 * want_loss, (loss, want_loss)
    assert np.all(dh[-1] == 0.0)
    assert oracle.rel_fro(dh, want_dh) < 1e-3, oracle.rel_fro(dh, want_dh)
    w.free()
