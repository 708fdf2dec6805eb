"""AdamW step on the adapter matrices: the CPU restatement against torch.optim.AdamW (the textbook rule; the
reference's own optimizer lives in a package that is not in its repository), and the CUDA kernel against the
restatement on a B200 - on flat buffers and through an adapter after a real forward/backward."""
import numpy as np
import pytest

from glacier.tune_b200 import synth as S

HYPER = [
    dict(lr=2e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01),      # the trainer's defaults
    dict(lr=1e-2, beta1=0.8, beta2=0.95, eps=1e-6, weight_decay=0.1),
    dict(lr=1e-3, beta1=0.0, beta2=0.5, eps=1e-8, weight_decay=0.0),
]


@pytest.mark.parametrize("h", HYPER)
def test_oracle_adamw_matches_torch(oracle, h):
    import torch
    rng = np.random.default_rng(3)
    n = 1000
    p0 = rng.standard_normal(n).astype(np.float32)
    p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    tp = torch.nn.Parameter(torch.from_numpy(p0.astype(np.float64)))           # fp64 torch: the more accurate side
    opt = torch.optim.AdamW([tp], lr=h["lr"], betas=(h["beta1"], h["beta2"]), eps=h["eps"], weight_decay=h["weight_decay"])
    for step in range(1, 21):
        g = (rng.standard_normal(n) * (0.1 if step % 3 else 10.0)).astype(np.float32)
        oracle.adamw_step(p, g, m, v, step=step, **h)
        tp.grad = torch.from_numpy(g.astype(np.float64))
        opt.step()
    want = tp.detach().numpy()
    assert np.max(np.abs(p - want)) < 2e-6 * max(1.0, float(np.max(np.abs(want))))
    st = opt.state[tp]
    # fp32 moments against fp64 ones: absolute error of a few ulp of the largest term that went into the sum
    assert np.max(np.abs(m - st["exp_avg"].numpy())) < 1e-5 and np.max(np.abs(v - st["exp_avg_sq"].numpy())) < 1e-4


def test_oracle_adamw_first_step_is_sign_of_gradient(oracle):
    """With zero moments the first bias-corrected update is lr * g / (|g| + eps): a known answer independent of beta."""
    g = np.array([0.5, -2.0, 1e-3, 0.0], np.float32)
    p, m, v = np.ones(4, np.float32), np.zeros(4, np.float32), np.zeros(4, np.float32)
    oracle.adamw_step(p, g, m, v, lr=0.1, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1)
    assert np.allclose(p, [0.9, 1.1, 0.9, 1.0], atol=1e-5)
    p2 = np.full(4, 2.0, np.float32)
    oracle.adamw_step(p2, np.zeros(4, np.float32), np.zeros(4, np.float32), np.zeros(4, np.float32), lr=0.1, beta1=0.9,
                      beta2=0.999, eps=1e-8, weight_decay=0.5, step=1)
    assert np.allclose(p2, 2.0 * (1 - 0.05))                                     # decay alone: p *= 1 - lr * wd


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def eng():
    from glacier.tune_b200 import capi as G
    e = G.Engine(0, G.MATH_BF16)
    yield e
    e.close()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 5, 4096, 1441792, 1000003])
@pytest.mark.parametrize("h", HYPER[:2])
def test_gpu_adamw_flat_buffers(eng, oracle, n, h):
    """Five steps on flat device buffers against the CPU restatement: same fp32 formula, so only the last bits of the
    division and square root may differ (relative error <= 1e-6 on p, m, v)."""
    import torch
    rng = np.random.default_rng(n)
    p = rng.standard_normal(n).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    P, M, V = (torch.from_numpy(a.copy()).cuda() for a in (p, m, v))
    off = 1 if n > 8 else 0                                                      # a misaligned view takes the scalar path
    P2, M2, V2 = (torch.cat([t.new_zeros(1), t])[1:] if off else t.clone() for t in (P, M, V))
    for step in range(1, 6):
        g = rng.standard_normal(n).astype(np.float32)
        Gd = torch.from_numpy(g).cuda()
        eng.adamw_step(P, Gd, M, V, step=step, **h)
        G2 = torch.cat([Gd.new_zeros(1), Gd])[1:] if off else Gd
        eng.adamw_step(P2, G2, M2, V2, step=step, **h)
        eng.sync()
        oracle.adamw_step(p, g, m, v, step=step, **h)
    for got, want in ((P, p), (M, m), (V, v), (P2, p), (M2, m), (V2, v)):
        assert oracle.rel_fro(got.cpu().numpy(), want) < 1e-6
    assert np.max(np.abs(P.cpu().numpy() - p)) < 1e-5


@pytest.mark.gpu
def test_gpu_adamw_argument_checks(eng):
    import torch
    from glacier.tune_b200 import capi as G
    t = torch.zeros(16, device="cuda")
    with pytest.raises(G.GtError):
        eng.adamw_step(t, t, t, t, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0)               # step counts from 1
    with pytest.raises(G.GtError):
        eng.adamw_step(t, t, t, t, 1e-3, 1.0, 0.999, 1e-8, 0.0, 1)               # beta1 = 1


@pytest.mark.gpu
def test_gpu_adapter_trains_on_device(eng, oracle):
    """Three optimizer steps of one projection entirely on the device: forward, backward, AdamW on A and B.  B starts
    at zero (the reference's initialisation), so step 1 moves only B and switches the adapter's delta on.  The CPU
    mirror takes the same steps with the restatement: its gradients are checked against the device's (2e-2, bf16
    tensor cores), and its AdamW step is fed the device's gradients so that both sides stay in lockstep and the
    updated A, B compare to rounding (an AdamW step is sign-like: a gradient that differs in its last bits near
    zero would otherwise move a parameter by 2 lr)."""
    N, K, T, R = 256, 512, 40, 16
    c = S.make_projection_case(S.TYPE_Q4_K, N, K, T, seed=11)
    h = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    w = eng.upload_weight(c["qtype"], c["w"], N, K)
    ad = eng.create_adapter(K, N, R, 32.0)
    A = c["a"].copy()
    B = np.zeros((R, N), np.float32)
    ad.upload(A, B)
    mA, vA, mB, vB = (np.zeros_like(a) for a in (A, A, B, B))
    for step in range(1, 4):
        y = eng.forward(w, ad, c["x"])
        y_ref = oracle.proj_forward(c["qtype"], c["w"], None, c["x"], K, N, T, A, B, R, c["scaling"])
        assert oracle.rel_fro(y, y_ref) < 2e-2
        ad.zero_grads()
        eng.backward(w, ad, c["dy"], c["x"], None)
        ga_dev, gb_dev = ad.grads()
        _, ga, gb = oracle.proj_backward(c["qtype"], c["w"], c["dy"], c["x"], K, N, T, A, B, R, c["scaling"], want_dx=False)
        assert oracle.rel_fro(gb_dev, gb) < 2e-2
        if step == 1:
            assert not ga.any() and not ga_dev.any()                               # B == 0: dA == 0
        else:
            assert oracle.rel_fro(ga_dev, ga) < 2e-2
        ad.adamw_step(step=step, **h)
        oracle.adamw_step(A, ga_dev, mA, vA, step=step, **h)
        oracle.adamw_step(B, gb_dev, mB, vB, step=step, **h)
        A_dev, B_dev = ad.download()
        assert oracle.rel_fro(A_dev, A) < 1e-6 and oracle.rel_fro(B_dev, B) < 1e-5
        assert np.max(np.abs(B_dev - B)) < 1e-6
        if step == 1:
            assert np.count_nonzero(B_dev) > 0.9 * B.size                          # the delta is switched on
    w.free()
    ad.free()


@pytest.mark.gpu
def test_gpu_many_adapters_in_one_call(eng, oracle):
    """gt_adapters_adamw_step over 19 adapters of mixed shapes (two launches: sixteen adapters each at most) leaves every A, B bit-identical
    to 19 single-adapter calls and equal to the CPU restatement to rounding."""
    import torch
    rng = np.random.default_rng(9)
    shapes = [(64 + 8 * i, 40 + 4 * i, (8, 16, 5)[i % 3]) for i in range(19)]           # (in, out, rank); rank 5: odd sizes
    h = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    sets, grads, cpu = [], [], []
    for which in range(2):
        ads, gs = [], []
        for K, N, R in shapes:
            ad = eng.create_adapter(K, N, R, 2.0 * R)
            A0 = np.random.default_rng(K).standard_normal((K, R)).astype(np.float32)
            ad.upload(A0, np.zeros((R, N), np.float32))
            g = (torch.zeros(K * R, device="cuda"), torch.zeros(R * N, device="cuda"))
            ad.bind_grads(*g)                                                          # gradients live in tensors of the test
            ads.append(ad)
            gs.append(g)
            if which == 0:
                cpu.append([A0.copy(), np.zeros((R, N), np.float32)] + [np.zeros((K, R), np.float32), np.zeros((K, R), np.float32),
                                                                          np.zeros((R, N), np.float32), np.zeros((R, N), np.float32)])
        sets.append(ads)
        grads.append(gs)
    for step in (1, 2, 3):
        for i, (K, N, R) in enumerate(shapes):
            ga, gb = rng.standard_normal((K, R)).astype(np.float32), rng.standard_normal((R, N)).astype(np.float32)
            for gs in grads:
                gs[i][0].copy_(torch.from_numpy(ga.reshape(-1)))
                gs[i][1].copy_(torch.from_numpy(gb.reshape(-1)))
            A, B, mA, vA, mB, vB = cpu[i]
            oracle.adamw_step(A, ga, mA, vA, step=step, **h)
            oracle.adamw_step(B, gb, mB, vB, step=step, **h)
        torch.cuda.synchronize()
        eng.adapters_adamw_step(sets[0], step=step, **h)
        for ad in sets[1]:
            ad.adamw_step(step=step, **h)
        eng.sync()
    for i, (a0, a1) in enumerate(zip(*sets)):
        A0, B0 = a0.download()
        A1, B1 = a1.download()
        assert np.array_equal(A0, A1) and np.array_equal(B0, B1)
        assert oracle.rel_fro(A0, cpu[i][0]) < 1e-6 and oracle.rel_fro(B0, cpu[i][1]) < 1e-5
    for ads in sets:
        for ad in ads:
            ad.free()
    with pytest.raises(Exception):
        eng.adapters_adamw_step([None], step=1, **h)
