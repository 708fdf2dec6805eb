"""CPU tests: the oracle's streaming cross-entropy and causal attention against closed forms in fp64.

The cross-entropy cases are the reference's own tests restated (tests/Glacier.Tune.Tests/KernelTests.cs:204-275:
vocabulary 32, hidden 32, gradient within 1e-5 of a dense softmax; AdversarialTuneTests.cs:80-209: vocabulary 1024 /
4096 / 8192 / 16384 at tile 4096, one ignored token, loss and gradient within 1e-5 of a double-precision dense softmax,
ignored rows exactly zero).  The attention cases mirror KernelTests.cs:99-131 (causal mask: position i must not see
j > i) and check forward / backward against dense fp64 softmax attention and finite differences.
"""
import numpy as np
import pytest


def _dense_ce(hidden, W, labels):
    """fp64 dense softmax cross-entropy: loss (mean over valid), dHidden."""
    V = W.shape[0]
    valid = [t for t, y in enumerate(labels) if 0 <= y < V]
    dh = np.zeros(hidden.shape, np.float64)
    total = 0.0
    for t in valid:
        logits = W.astype(np.float64) @ hidden[t].astype(np.float64)
        m = logits.max()
        lse = m + np.log(np.exp(logits - m).sum())
        total += lse - logits[labels[t]]
        p = np.exp(logits - lse)
        p[labels[t]] -= 1.0
        dh[t] = (p / len(valid)) @ W.astype(np.float64)
    return total / max(1, len(valid)), dh


def test_cross_entropy_small_dense_parity(oracle):
    rng = np.random.default_rng(1234)
    T, H, V = 4, 32, 32
    hidden = (rng.random((T, H)) * 0.5 - 0.25).astype(np.float32)
    W = (rng.random((V, H)) * 0.5 - 0.25).astype(np.float32)
    labels = np.array([5, 10, 15, 20], np.int32)
    loss, valid, dh = oracle.cross_entropy(oracle.TYPE_F32, W, hidden, labels, V)
    want_loss, want_dh = _dense_ce(hidden, W, labels)
    assert valid == 4 and loss > 0
    assert abs(loss - want_loss) < 1e-5
    assert np.max(np.abs(dh - want_dh)) < 1e-5


@pytest.mark.parametrize("V", [1024, 4096, 8192, 16384])
def test_cross_entropy_tiled_streaming_matches_double_precision(oracle, V):
    rng = np.random.default_rng(42 + V)
    T, H = 4, 64
    hidden = (rng.random((T, H)) * 0.4 - 0.2).astype(np.float32)
    labels = np.array([rng.integers(0, V), rng.integers(0, V), -100, rng.integers(0, V)], np.int32)
    W = (rng.random((V, H)) * 0.1 - 0.05).astype(np.float32)
    loss, valid, dh = oracle.cross_entropy(oracle.TYPE_F32, W, hidden, labels, V, tile=4096)
    want_loss, want_dh = _dense_ce(hidden, W, labels)
    assert valid == 3
    assert abs(loss - want_loss) < 1e-5
    assert np.all(dh[2] == 0.0)                       # ignored token: exactly zero
    assert np.max(np.abs(dh - want_dh)) < 1e-5
    # loss-only form and an fp16 LM head (the workload's head type): same numbers on the fp16-rounded weights
    loss2, _, none = oracle.cross_entropy(oracle.TYPE_F32, W, hidden, labels, V, want_grad=False)
    assert none is None and loss2 == loss
    W16 = W.astype(np.float16)
    l16, _, dh16 = oracle.cross_entropy(oracle.TYPE_F16, W16, hidden, labels, V, tile=1000)      # a tile that does not divide V
    w_loss, w_dh = _dense_ce(hidden, W16.astype(np.float32), labels)
    assert abs(l16 - w_loss) < 1e-5 and np.max(np.abs(dh16 - w_dh)) < 1e-5


def test_cross_entropy_no_valid_target(oracle):
    hidden = np.ones((3, 16), np.float32)
    W = np.ones((8, 16), np.float32)
    loss, valid, dh = oracle.cross_entropy(oracle.TYPE_F32, W, hidden, np.array([-100, 8, -1], np.int32), 8)
    assert loss == 0.0 and valid == 0 and np.all(dh == 0)


def _dense_attention(q, k, v, HQ, HK, D):
    T = q.shape[0]
    q3, k3, v3 = (a.astype(np.float64).reshape(T, -1, D) for a in (q, k, v))
    out = np.zeros((T, HQ, D))
    probs = np.zeros((HQ, T, T))
    for h in range(HQ):
        kh = h // (HQ // HK)
        s = q3[:, h] @ k3[:, kh].T / np.sqrt(D)
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        probs[h] = p
        out[:, h] = p @ v3[:, kh]
    return out.reshape(T, HQ * D), probs


def test_attention_forward_dense_parity_and_causal_mask(oracle):
    rng = np.random.default_rng(7)
    T, HQ, HK, D = 19, 4, 2, 16
    q = rng.standard_normal((T, HQ * D), dtype=np.float32)
    k = rng.standard_normal((T, HK * D), dtype=np.float32)
    v = rng.standard_normal((T, HK * D), dtype=np.float32)
    out, probs = oracle.attention_forward(q, k, v, HQ, HK, D)
    want, wprobs = _dense_attention(q, k, v, HQ, HK, D)
    assert np.max(np.abs(out - want)) < 1e-5 and np.max(np.abs(probs - wprobs)) < 1e-6
    assert np.all(np.triu(probs, 1) == 0.0)
    # position i must not depend on later positions: change the last key / value only
    k2, v2 = k.copy(), v.copy()
    k2[-1] += 3.0
    v2[-1] -= 2.0
    out2, _ = oracle.attention_forward(q, k2, v2, HQ, HK, D)
    assert np.array_equal(out2[:-1], out[:-1]) and not np.array_equal(out2[-1], out[-1])


def test_attention_backward_matches_finite_differences(oracle):
    rng = np.random.default_rng(8)
    T, HQ, HK, D = 7, 4, 2, 8
    q = rng.standard_normal((T, HQ * D)).astype(np.float32)
    k = rng.standard_normal((T, HK * D)).astype(np.float32)
    v = rng.standard_normal((T, HK * D)).astype(np.float32)
    g = rng.standard_normal((T, HQ * D)).astype(np.float32)
    _, probs = oracle.attention_forward(q, k, v, HQ, HK, D)
    dq, dk, dv = oracle.attention_backward(g, q, k, v, probs, HQ, HK, D)

    def f(qq, kk, vv):
        return float(np.sum(_dense_attention(qq, kk, vv, HQ, HK, D)[0] * g.astype(np.float64)))

    eps = 1e-3
    for arr, grad, which in ((q, dq, 0), (k, dk, 1), (v, dv, 2)):
        for idx in [(0, 0), (3, 5), (T - 1, arr.shape[1] - 1), (2, arr.shape[1] // 2)]:
            a1, a2 = arr.astype(np.float64).copy(), arr.astype(np.float64).copy()
            a1[idx] += eps
            a2[idx] -= eps
            args1 = [q, k, v]
            args2 = [q, k, v]
            args1[which], args2[which] = a1, a2
            fd = (f(*args1) - f(*args2)) / (2 * eps)
            assert abs(fd - grad[idx]) < 2e-3 * max(1.0, abs(fd)), (which, idx, fd, grad[idx])
