"""Layer glue (SwiGLU, RoPE, RMSNorm, residual add): the oracle against closed forms and finite differences on the
CPU, and the CUDA kernels against the oracle on a B200 (through the C ABI, device tensors)."""
import numpy as np
import pytest


def _fd(f, x, dout, eps=1e-3):
    """<dout, f(x + eps e) - f(x - eps e)> / (2 eps) for a few random directions e: directional derivatives in fp64."""
    rng = np.random.default_rng(5)
    out = []
    for _ in range(4):
        e = rng.standard_normal(x.shape)
        e /= np.linalg.norm(e)
        out.append((e, float(np.sum(dout * (f(x + eps * e) - f(x - eps * e))) / (2 * eps))))
    return out


def test_oracle_swiglu_matches_closed_form_and_its_derivative(oracle):
    rng = np.random.default_rng(1)
    g = (3 * rng.standard_normal((7, 50))).astype(np.float32)
    u = rng.standard_normal((7, 50)).astype(np.float32)
    dh = rng.standard_normal((7, 50)).astype(np.float32)
    h = oracle.swiglu_forward(g, u)
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    assert np.allclose(h, g64 / (1 + np.exp(-g64)) * u64, rtol=1e-6, atol=1e-6)
    dg, du = oracle.swiglu_backward(dh, g, u)
    f = lambda gg: gg / (1 + np.exp(-gg)) * u64          # noqa: E731
    for e, want in _fd(f, g64, dh.astype(np.float64)):
        assert abs(np.sum(dg * e) - want) < 1e-4 * max(1.0, abs(want))
    assert np.allclose(du, dh * (g64 / (1 + np.exp(-g64))), rtol=1e-5, atol=1e-6)


def test_oracle_rope_is_a_rotation_with_exact_inverse(oracle):
    rng = np.random.default_rng(2)
    T, hq, hk, d = 33, 4, 2, 64
    q = rng.standard_normal((T, hq * d)).astype(np.float32)
    k = rng.standard_normal((T, hk * d)).astype(np.float32)
    q2, k2 = oracle.rope(q, k, T, hq, hk, d, 1e6)
    assert np.array_equal(q2[0], q[0]) and np.array_equal(k2[0], k[0])          # position 0: theta = 0
    # every (i, i + half) pair keeps its length
    pairs = lambda a, h: a.reshape(T, h, 2, d // 2)                              # noqa: E731
    assert np.allclose((pairs(q2, hq) ** 2).sum(2), (pairs(q, hq) ** 2).sum(2), rtol=1e-5)
    # closed form at one element: pos = 5, head 1, i = 3
    pos, i = 5, 3
    theta = np.float32(pos) * (np.float32(1.0) / np.float32(np.float32(1e6) ** np.float32(2 * i / d)))
    v0, v1 = q[pos, d + i], q[pos, d + i + d // 2]
    assert abs(q2[pos, d + i] - (v0 * np.cos(theta) - v1 * np.sin(theta))) < 1e-5
    q3, k3 = oracle.rope(q2, k2, T, hq, hk, d, 1e6, inverse=True)
    assert np.allclose(q3, q, atol=1e-5) and np.allclose(k3, k, atol=1e-5)
    # partial rotation (rope_dim < head_dim) leaves the tail of every head alone
    q4, _ = oracle.rope(q, None, T, hq, hk, d, 1e4, rope_dim=32)
    assert np.array_equal(q4.reshape(T, hq, d)[:, :, 32:], q.reshape(T, hq, d)[:, :, 32:])


def test_oracle_rmsnorm_forward_and_backward(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 96)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(96)).astype(np.float32)
    dy = rng.standard_normal((5, 96)).astype(np.float32)
    x64, w64 = x.astype(np.float64), w.astype(np.float64)
    f = lambda xx: xx / np.sqrt((xx ** 2).mean(1, keepdims=True) + 1e-6) * w64   # noqa: E731
    assert np.allclose(oracle.rmsnorm_forward(x, w), f(x64), rtol=1e-6, atol=1e-6)
    dx = oracle.rmsnorm_backward(dy, x, w)
    for e, want in _fd(f, x64, dy.astype(np.float64), eps=1e-4):
        assert abs(np.sum(dx * e) - want) < 1e-4 * max(1.0, abs(want))


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def eng():
    from glacier.tune_b200 import capi as G
    e = G.Engine(0, G.MATH_BF16)
    yield e
    e.close()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 7, 4096, 512 * 18944, 1000003])
def test_gpu_swiglu_and_add(eng, oracle, n):
    """fp32 element-wise kernels: relative error <= 2e-6 against the CPU restatement (expf differs in the last bits)."""
    import torch
    rng = np.random.default_rng(n)
    g = (2 * rng.standard_normal(n)).astype(np.float32)
    u = rng.standard_normal(n).astype(np.float32)
    dh = rng.standard_normal(n).astype(np.float32)
    G_, U_, D_ = (torch.from_numpy(a).cuda() for a in (g, u, dh))
    H_ = torch.empty_like(G_)
    eng.swiglu_forward(G_, U_, H_)
    dG_, dU_ = torch.empty_like(G_), torch.empty_like(G_)
    eng.swiglu_backward(D_, G_, U_, dG_, dU_)
    S_ = torch.empty_like(G_)
    eng.add(G_, U_, S_)
    eng.sync()
    assert oracle.rel_fro(H_.cpu().numpy(), oracle.swiglu_forward(g, u)) < 2e-6
    dg, du = oracle.swiglu_backward(dh, g, u)
    assert oracle.rel_fro(dG_.cpu().numpy(), dg) < 2e-6 and oracle.rel_fro(dU_.cpu().numpy(), du) < 2e-6
    assert np.array_equal(S_.cpu().numpy(), g + u)
    if n > 8:      # misaligned views take the scalar path
        H2 = torch.empty(n + 1, device="cuda")[1:]
        eng.swiglu_forward(G_[1:], U_[1:], H2[1:])
        eng.sync()
        assert oracle.rel_fro(H2[1:].cpu().numpy(), oracle.swiglu_forward(g[1:], u[1:])) < 2e-6


@pytest.mark.gpu
@pytest.mark.parametrize("T,hq,hk,d,base,rope_dim", [(512, 28, 4, 128, 1e6, -1), (33, 4, 2, 64, 1e4, -1), (17, 2, 1, 128, 1e6, 64), (1, 8, 8, 32, 5e5, -1)])
def test_gpu_rope(eng, oracle, T, hq, hk, d, base, rope_dim):
    """Rotation angles reach pos * 1 rad (hundreds of radians): powf / sincosf of the device and of the host differ by a
    few ulp in theta, i.e. up to ~1e-4 absolute in cos / sin: tolerance 3e-4 relative Frobenius, and an exact inverse."""
    import torch
    rng = np.random.default_rng(T + d)
    q = rng.standard_normal((T, hq * d)).astype(np.float32)
    k = rng.standard_normal((T, hk * d)).astype(np.float32)
    Q, K = torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda()
    eng.rope(Q, K, T, hq, hk, d, base, 1.0, rope_dim)
    eng.sync()
    qr, kr = oracle.rope(q, k, T, hq, hk, d, base, 1.0, rope_dim)
    assert oracle.rel_fro(Q.cpu().numpy(), qr) < 3e-4 and oracle.rel_fro(K.cpu().numpy(), kr) < 3e-4
    eng.rope(Q, K, T, hq, hk, d, base, 1.0, rope_dim, inverse=True)
    eng.sync()
    assert np.allclose(Q.cpu().numpy(), q, atol=2e-5) and np.allclose(K.cpu().numpy(), k, atol=2e-5)
    eng.rope(Q, None, T, hq, hk, d, base, 1.0, rope_dim)          # q alone
    eng.sync()
    assert oracle.rel_fro(Q.cpu().numpy(), qr) < 3e-4


@pytest.mark.gpu
@pytest.mark.parametrize("T,H", [(512, 3584), (3, 100), (17, 5000), (1, 128)])
def test_gpu_rmsnorm(eng, oracle, T, H):
    """fp32 sums on the device against fp64 sums in the oracle: <= 1e-5 relative."""
    import torch
    rng = np.random.default_rng(T + H)
    x = rng.standard_normal((T, H)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(H)).astype(np.float32)
    dy = rng.standard_normal((T, H)).astype(np.float32)
    X, W, DY = (torch.from_numpy(a).cuda() for a in (x, w, dy))
    Y, DX = torch.empty_like(X), torch.empty_like(X)
    eng.rmsnorm_forward(X, W, Y)
    eng.rmsnorm_backward(DY, X, W, DX)
    eng.sync()
    assert oracle.rel_fro(Y.cpu().numpy(), oracle.rmsnorm_forward(x, w)) < 1e-5
    assert oracle.rel_fro(DX.cpu().numpy(), oracle.rmsnorm_backward(dy, x, w)) < 1e-5


@pytest.mark.gpu
def test_gpu_glue_argument_checks(eng):
    import torch
    from glacier.tune_b200 import capi as G
    x = torch.zeros(8, device="cuda")
    with pytest.raises(G.GtError):
        eng.swiglu_forward(x, None, x)
    with pytest.raises(G.GtError):
        eng.rope(None, None, 4, 1, 1, 8)
    with pytest.raises(G.GtError):
        eng.rope(x, None, 1, 1, 1, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("T", [9, 100, 300])
def test_gpu_ffn_block_forward_and_backward(eng, oracle, T):
    """gt_ffn_forward / gt_ffn_backward against the oracle chained the way TransformerBlock does it: gate and up
    projections, SwiGLU, down projection, and back.  bf16 mode tolerances; T = 9 takes the few-token forward kernels,
    T = 100 keeps SiLU(gate) * up as bf16 only, T = 300 also dGate and dUp."""
    import torch
    from glacier.tune_b200 import capi as G, synth as S
    H, F = 256, 768
    eng.set_math_mode(0)
    cg = S.make_projection_case(S.TYPE_Q4_K, F, H, T, seed=11)
    cu = S.make_projection_case(S.TYPE_Q4_K, F, H, T, seed=12)
    cd = S.make_projection_case(S.TYPE_Q6_K, H, F, T, seed=13)
    x, dy = cg["x"], cd["dy"]
    ws = [eng.upload_weight(c["qtype"], c["w"], c["N"], c["K"]) for c in (cg, cu, cd)]
    ads = []
    for c in (cg, cu, cd):
        a = eng.create_adapter(c["K"], c["N"], 16, 32.0)
        a.upload(c["a"], c["b"])
        ads.append(a)
    # oracle chain (fp32 CPU path)
    proj = lambda c, xin: oracle.proj_forward(c["qtype"], c["w"], None, xin, c["K"], c["N"], T, c["a"], c["b"], 16, c["scaling"])   # noqa: E731
    g_ref, u_ref = proj(cg, x), proj(cu, x)
    h_ref = oracle.swiglu_forward(g_ref, u_ref)
    y_ref = proj(cd, h_ref)
    X = torch.from_numpy(x).cuda()
    Gt, Ut, Ht = (torch.empty((T, F), device="cuda") for _ in range(3))
    Y = torch.empty((T, H), device="cuda")
    eng.ffn_forward(ws[0], ws[1], ws[2], ads, X, Y, Gt, Ut, Ht)
    eng.sync()
    assert oracle.rel_fro(Gt.cpu().numpy(), g_ref) < 2e-2 and oracle.rel_fro(Ut.cpu().numpy(), u_ref) < 2e-2
    assert oracle.rel_fro(Ht.cpu().numpy(), h_ref) < 3e-2 and oracle.rel_fro(Y.cpu().numpy(), y_ref) < 3e-2
    # intermediate tensors left in engine scratch: same result
    Y2 = torch.empty_like(Y)
    eng.ffn_forward(ws[0], ws[1], ws[2], ads, X, Y2)
    eng.sync()
    assert oracle.rel_fro(Y2.cpu().numpy(), Y.cpu().numpy()) < 1e-3
    # host buffers, only the final output asked for
    yh = np.empty((T, H), np.float32)
    eng.ffn_forward(ws[0], ws[1], ws[2], ads, x, yh)
    assert oracle.rel_fro(yh, y_ref) < 3e-2
    # backward, on the device's own forward tensors so that only the backward arithmetic is compared
    g_d, u_d, h_d = Gt.cpu().numpy(), Ut.cpu().numpy(), Ht.cpu().numpy()
    back = lambda c, dyin, xin: oracle.proj_backward(c["qtype"], c["w"], dyin, xin, c["K"], c["N"], T, c["a"], c["b"], 16, c["scaling"])   # noqa: E731
    dh_ref, dad, dbd = back(cd, dy, h_d)
    dg_ref, du_ref = oracle.swiglu_backward(dh_ref, g_d, u_d)
    dx_g, dag, dbg = back(cg, dg_ref, x)
    dx_u, dau, dbu = back(cu, du_ref, x)
    for a in ads:
        a.zero_grads()
    dX = torch.full((T, H), 5.0, device="cuda")
    eng.ffn_backward(ws[0], ws[1], ws[2], ads, torch.from_numpy(dy).cuda(), X, Gt, Ut, Ht, dX, flags=G.FLAG_DX_ASSIGN)
    eng.sync()
    assert oracle.rel_fro(dX.cpu().numpy(), dx_g + dx_u) < 3e-2
    for a, (da_ref, db_ref) in zip(ads, ((dag, dbg), (dau, dbu), (dad, dbd))):
        da, db = a.grads()
        assert oracle.rel_fro(da, da_ref) < 3e-2 and oracle.rel_fro(db, db_ref) < 3e-2
    for h in ws + ads:
        h.free()
