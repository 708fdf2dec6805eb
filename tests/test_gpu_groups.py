"""GPU parity of the grouped projection calls (q,k,v and gate,up of a block): several projections of one input in
one launch, and their input gradients summed into one buffer, against the CPU oracle member by member."""
import numpy as np
import pytest

from glacier.tune_b200 import synth as S

pytestmark = pytest.mark.gpu

TOL = {0: 2e-2, 1: 1e-3, 2: 1e-3}
LTOL = {0: 5e-3, 1: 1e-3, 2: 1e-3}


@pytest.fixture(scope="module")
def G():
    from glacier.tune_b200 import capi
    return capi


@pytest.fixture(scope="module")
def eng(G):
    e = G.Engine(0, G.MATH_BF16)
    yield e
    e.close()


def _members(qtype, Ns, K, T, seed, adapted, biased):
    """Projection cases that share one input X; member j has an adapter / a bias where the masks say so."""
    cs = []
    for j, N in enumerate(Ns):
        c = S.make_projection_case(qtype, N, K, T, seed=seed + 17 * j, with_bias=True)
        c["x"] = cs[0]["x"] if cs else c["x"]
        c["lora"], c["has_bias"] = adapted[j], biased[j]
        cs.append(c)
    return cs


def _reference(oracle, cs):
    K, T = cs[0]["K"], cs[0]["T"]
    dx = np.zeros((T, K), np.float64)
    ys, das, dbs = [], [], []
    for c in cs:
        qt, N = c["qtype"], c["N"]
        y = oracle.matmul_batch(qt, c["w"], c["x"], K, N, T, c["bias"] if c["has_bias"] else None, f64=True)
        dx += oracle.base_backward_f64(qt, c["w"], c["dy"], K, N, T)
        da = db = None
        if c["lora"]:
            X, dY, A, B = (c[k].astype(np.float64) for k in ("x", "dy", "a", "b"))
            s = c["scaling"]
            dlow = dY @ B.T
            y = y + s * (X @ A) @ B
            dx += s * dlow @ A.T
            da, db = s * X.T @ dlow, s * (X @ A).T @ dY
        ys.append(y)
        das.append(da)
        dbs.append(db)
    return ys, dx, das, dbs


def _upload(eng, cs):
    ws, ads = [], []
    for c in cs:
        ws.append(eng.upload_weight(c["qtype"], c["w"], c["N"], c["K"], c["bias"] if c["has_bias"] else None))
        ad = None
        if c["lora"]:
            ad = eng.create_adapter(c["K"], c["N"], c["rank"], c["alpha"])
            ad.upload(c["a"], c["b"])
        ads.append(ad)
    return ws, ads


def _free(ws, ads):
    for w in ws:
        w.free()
    for a in ads:
        if a:
            a.free()


GROUPS = [
    # qtype, member out_features, K, T, adapters, biases
    (S.TYPE_Q4_K, (512, 128, 128), 512, 17, (1, 0, 1), (1, 1, 1)),        # q,k,v with grouped-query widths
    (S.TYPE_Q4_K, (512, 128, 128), 512, 300, (1, 1, 1), (1, 1, 0)),
    (S.TYPE_Q4_K, (384, 384), 768, 512, (1, 1), (0, 0)),                 # gate,up; odd tile count per member
    (S.TYPE_Q4_K, (640, 200), 256, 600, (0, 0), (0, 1)),                 # no adapters, ragged rows, two token chunks
    (S.TYPE_Q6_K, (256, 128, 128), 512, 96, (1, 0, 1), (1, 0, 1)),
    (S.TYPE_Q4_K, (256, 256), 3584, 512, (1, 1), (0, 0)),                # deep K (split across CTAs)
]


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("qtype,Ns,K,T,adapted,biased", GROUPS)
def test_group_forward_backward_parity(G, eng, oracle, mode, qtype, Ns, K, T, adapted, biased):
    import torch
    if mode == 2 and T * sum(Ns) * K > 2e8:
        pytest.skip("fp32 validation kernels are checked on the smaller shapes")
    cs = _members(qtype, Ns, K, T, seed=K + T, adapted=adapted, biased=biased)
    eng.set_math_mode(mode)
    ws, ads = _upload(eng, cs)
    X = torch.from_numpy(cs[0]["x"]).cuda()
    Ys = [torch.full((T, c["N"]), 7.0, device="cuda") for c in cs]          # stale contents must be overwritten
    dYs = [torch.from_numpy(c["dy"]).cuda() for c in cs]
    prior = torch.full((T, K), 0.5, device="cuda")
    dX = prior.clone()
    eng.forward_group(ws, ads, X, Ys)
    eng.backward_group(ws, ads, dYs, X, dX, flags=G.FLAG_REUSE_LOW)
    eng.sync()
    ys, dxr, das, dbs = _reference(oracle, cs)
    for j, c in enumerate(cs):
        assert oracle.rel_fro(Ys[j].cpu().numpy(), ys[j]) < TOL[mode], (j, "Y")
        if c["lora"]:
            da, db = ads[j].grads()
            assert oracle.rel_fro(da, das[j]) < LTOL[mode] and oracle.rel_fro(db, dbs[j]) < LTOL[mode], (j, "dA dB")
    assert oracle.rel_fro((dX - prior).cpu().numpy(), dxr) < TOL[mode]
    _free(ws, ads)


def test_group_equals_member_calls(G, eng, oracle):
    """The grouped launch and the per-projection calls run the same arithmetic per output tile; they differ only by
    the order of fp32 atomic sums (X*A partial sums, split-K partial tiles) and what a last-bit change of X*A does
    after its rounding to bf16."""
    import torch
    cs = _members(S.TYPE_Q4_K, (512, 128, 128), 512, 200, seed=5, adapted=(1, 1, 1), biased=(1, 1, 1))
    eng.set_math_mode(0)
    ws, ads = _upload(eng, cs)
    X = torch.from_numpy(cs[0]["x"]).cuda()
    dYs = [torch.from_numpy(c["dy"]).cuda() for c in cs]
    Yg = [torch.empty((200, c["N"]), device="cuda") for c in cs]
    Ym = [torch.empty((200, c["N"]), device="cuda") for c in cs]
    eng.forward_group(ws, ads, X, Yg)
    dXg = torch.zeros((200, 512), device="cuda")
    eng.backward_group(ws, ads, dYs, X, dXg)
    eng.sync()
    grads_g = [a.grads() for a in ads]
    for a in ads:
        a.zero_grads()
    dXm = torch.zeros((200, 512), device="cuda")
    for j in range(3):
        eng.forward(ws[j], ads[j], X, Ym[j])
        eng.backward(ws[j], ads[j], dYs[j], X, dXm)
    eng.sync()
    for j in range(3):
        assert oracle.rel_fro(Yg[j].cpu().numpy(), Ym[j].cpu().numpy()) < 1e-3
        da, db = ads[j].grads()
        assert oracle.rel_fro(grads_g[j][0], da) < 1e-4 and oracle.rel_fro(grads_g[j][1], db) < 1e-4
    assert oracle.rel_fro(dXg.cpu().numpy(), dXm.cpu().numpy()) < 1e-3
    _free(ws, ads)


@pytest.mark.parametrize("mode", [0, 1])
def test_q4km_mixed_group(G, eng, oracle, mode):
    """q, k in Q4_K and v in Q6_K (the Q4_K_M mix): one pass over X, one GEMM launch per quantization type, one dX."""
    import torch
    T, K = 200, 768
    cs = []
    for j, (qt, N) in enumerate(((S.TYPE_Q4_K, 384), (S.TYPE_Q4_K, 128), (S.TYPE_Q6_K, 128))):
        c = S.make_projection_case(qt, N, K, T, seed=300 + j, with_bias=True)
        if cs:
            c["x"] = cs[0]["x"]
        c["lora"], c["has_bias"] = True, j != 1
        cs.append(c)
    eng.set_math_mode(mode)
    ws, ads = _upload(eng, cs)
    X = torch.from_numpy(cs[0]["x"]).cuda()
    Ys = [torch.empty((T, c["N"]), device="cuda") for c in cs]
    dYs = [torch.from_numpy(c["dy"]).cuda() for c in cs]
    dX = torch.full((T, K), 2.0, device="cuda")
    eng.profile_read(True)
    eng.profile_enable(True)
    eng.forward_group(ws, ads, X, Ys)
    eng.backward_group(ws, ads, dYs, X, dX, flags=G.FLAG_REUSE_LOW | G.FLAG_DX_ASSIGN)
    eng.sync()
    pr = eng.profile_read(True)
    eng.profile_enable(False)
    assert pr["gemm_launches"] == 4          # (q,k) + (v), forward and backward
    ys, dxr, das, dbs = _reference(oracle, cs)
    for j in range(3):
        assert oracle.rel_fro(Ys[j].cpu().numpy(), ys[j]) < TOL[mode], j
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, das[j]) < LTOL[mode] and oracle.rel_fro(db, dbs[j]) < LTOL[mode], j
    assert oracle.rel_fro(dX.cpu().numpy(), dxr) < TOL[mode]
    _free(ws, ads)


def test_group_host_buffers_and_mixed_types(G, eng, oracle):
    """Host buffers and members of different quantization types give the same results as device tensors."""
    import torch
    a = S.make_projection_case(S.TYPE_Q4_K, 256, 512, 40, seed=3, with_bias=True)
    b = S.make_projection_case(S.TYPE_Q6_K, 128, 512, 40, seed=4, with_bias=True)
    b["x"] = a["x"]
    for c in (a, b):
        c["lora"], c["has_bias"] = True, True
    cs = [a, b]
    eng.set_math_mode(0)
    ws, ads = _upload(eng, cs)
    ys, dxr, das, dbs = _reference(oracle, cs)
    # host buffers
    Ys = [np.empty((40, c["N"]), np.float32) for c in cs]
    dX = np.zeros((40, 512), np.float32)
    eng.forward_group(ws, ads, a["x"], Ys)
    eng.backward_group(ws, ads, [c["dy"] for c in cs], a["x"], dX)
    for j in range(2):
        assert oracle.rel_fro(Ys[j], ys[j]) < 2e-2
    assert oracle.rel_fro(dX, dxr) < 2e-2
    # device buffers, mixed types
    for ad in ads:
        ad.zero_grads()
    X = torch.from_numpy(a["x"]).cuda()
    Yd = [torch.empty((40, c["N"]), device="cuda") for c in cs]
    dXd = torch.zeros((40, 512), device="cuda")
    eng.forward_group(ws, ads, X, Yd)
    eng.backward_group(ws, ads, [torch.from_numpy(c["dy"]).cuda() for c in cs], X, dXd)
    eng.sync()
    for j in range(2):
        assert oracle.rel_fro(Yd[j].cpu().numpy(), ys[j]) < 2e-2
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, das[j]) < 5e-3 and oracle.rel_fro(db, dbs[j]) < 5e-3
    assert oracle.rel_fro(dXd.cpu().numpy(), dxr) < 2e-2
    _free(ws, ads)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_dx_assign_overwrites_stale_contents(G, eng, oracle, mode):
    """GT_FLAG_DX_ASSIGN: dX = ... whatever the buffer held (single call with and without adapter, group, host buffers)."""
    import torch
    cs = _members(S.TYPE_Q4_K, (256, 128), 512, 150, seed=77, adapted=(1, 0), biased=(0, 0))
    eng.set_math_mode(mode)
    ws, ads = _upload(eng, cs)
    X = torch.from_numpy(cs[0]["x"]).cuda()
    dYs = [torch.from_numpy(c["dy"]).cuda() for c in cs]
    _, dx_group, _, _ = _reference(oracle, cs)
    singles = [_reference(oracle, [c])[1] for c in cs]
    dX = torch.full((150, 512), 3.0, device="cuda")
    eng.backward_group(ws, ads, dYs, X, dX, flags=G.FLAG_DX_ASSIGN)
    eng.sync()
    assert oracle.rel_fro(dX.cpu().numpy(), dx_group) < TOL[mode]
    for j in range(2):
        dX.fill_(-5.0)
        eng.backward(ws[j], ads[j], dYs[j], X, dX, flags=G.FLAG_DX_ASSIGN)
        eng.sync()
        assert oracle.rel_fro(dX.cpu().numpy(), singles[j]) < TOL[mode], j
    hdx = np.full((150, 512), 9.0, np.float32)
    eng.backward(ws[0], ads[0], cs[0]["dy"], cs[0]["x"], hdx, flags=G.FLAG_DX_ASSIGN)
    assert oracle.rel_fro(hdx, singles[0]) < TOL[mode]
    hdx.fill(9.0)
    eng.backward_group(ws, ads, [c["dy"] for c in cs], cs[0]["x"], hdx, flags=G.FLAG_DX_ASSIGN)
    assert oracle.rel_fro(hdx, dx_group) < TOL[mode]
    _free(ws, ads)


def test_repeated_backward_after_one_forward(G, eng, oracle):
    """Two backward calls that reuse X*A of one forward: the second must not see the first one's dY*B^T sums."""
    import torch
    c = S.make_projection_case(S.TYPE_Q4_K, 256, 512, 100, seed=9)
    eng.set_math_mode(0)
    w = eng.upload_weight(c["qtype"], c["w"], 256, 512)
    ad = eng.create_adapter(512, 256, 16, 32.0)
    ad.upload(c["a"], c["b"])
    X, dY = torch.from_numpy(c["x"]).cuda(), torch.from_numpy(c["dy"]).cuda()
    Y = torch.empty((100, 256), device="cuda")
    eng.forward(w, ad, X, Y)
    out = []
    for _ in range(2):
        ad.zero_grads()
        dX = torch.zeros((100, 512), device="cuda")
        eng.backward(w, ad, dY, X, dX, flags=G.FLAG_REUSE_LOW)
        eng.sync()
        out.append((dX.cpu().numpy(),) + tuple(ad.grads()))
    for a, b in zip(*out):
        assert oracle.rel_fro(a, b) < 1e-4
    w.free()
    ad.free()


def test_host_async_calls_complete_at_sync(G, eng, oracle):
    """GT_FLAG_HOST_ASYNC on page-locked buffers: more calls than staging slots queued back to back, results checked
    after one gt_sync(); they equal the synchronous calls' results."""
    import torch
    cs = _members(S.TYPE_Q4_K, (256, 128), 512, 130, seed=41, adapted=(1, 1), biased=(1, 0))
    eng.set_math_mode(0)
    ws, ads = _upload(eng, cs)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()      # noqa: E731
    hx = pin(cs[0]["x"])
    hdy = [pin(c["dy"]) for c in cs]
    rounds = 5
    hys = [[torch.zeros((130, c["N"])).pin_memory() for c in cs] for _ in range(rounds)]
    hdx = [torch.full((130, 512), 4.0).pin_memory() for _ in range(rounds)]
    fl = G.FLAG_HOST_ASYNC
    for r in range(rounds):
        eng.forward_group(ws, ads, hx.numpy(), [y.numpy() for y in hys[r]], flags=fl)
        eng.backward_group(ws, ads, [d.numpy() for d in hdy], hx.numpy(), hdx[r].numpy(), flags=fl | G.FLAG_DX_ASSIGN | G.FLAG_REUSE_LOW)
    eng.sync()
    ys, dxr, das, dbs = _reference(oracle, cs)
    for r in range(rounds):
        for j in range(2):
            assert oracle.rel_fro(hys[r][j].numpy(), ys[j]) < 2e-2, (r, j)
        assert oracle.rel_fro(hdx[r].numpy(), dxr) < 2e-2, r
    for j in range(2):
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, rounds * das[j]) < 5e-3 and oracle.rel_fro(db, rounds * dbs[j]) < 5e-3
    # a backward without GT_FLAG_REUSE_LOW uploads X again: same gradients as the one that reuses the kept copy
    for ad in ads:
        ad.zero_grads()
    hdx2 = torch.full((130, 512), 4.0).pin_memory()
    eng.forward_group(ws, ads, hx.numpy(), [y.numpy() for y in hys[0]], flags=fl)
    eng.backward_group(ws, ads, [d.numpy() for d in hdy], hx.numpy(), hdx2.numpy(), flags=fl | G.FLAG_DX_ASSIGN)
    eng.sync()
    assert oracle.rel_fro(hdx2.numpy(), hdx[0].numpy()) < 1e-3
    for j in range(2):
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, das[j]) < 5e-3 and oracle.rel_fro(db, dbs[j]) < 5e-3
    # synchronous host calls give the same numbers as the queued ones
    y_sync = [np.empty((130, c["N"]), np.float32) for c in cs]
    eng.forward_group(ws, ads, cs[0]["x"], y_sync)
    for j in range(2):
        assert oracle.rel_fro(y_sync[j], hys[0][j].numpy()) < 1e-3
    _free(ws, ads)


def test_group_with_different_ranks(G, eng, oracle):
    """Members with ranks 16, 32 and 8: the chunk lists of the shared passes span several launches."""
    import torch
    T, K = 150, 512
    cs = []
    for j, (N, r) in enumerate(((256, 16), (128, 32), (128, 8))):
        c = S.make_projection_case(S.TYPE_Q4_K, N, K, T, seed=700 + j, rank=r, alpha=2.0 * r)
        if cs:
            c["x"] = cs[0]["x"]
        c["lora"], c["has_bias"] = True, False
        cs.append(c)
    eng.set_math_mode(0)
    ws, ads = _upload(eng, cs)
    X = torch.from_numpy(cs[0]["x"]).cuda()
    Ys = [torch.empty((T, c["N"]), device="cuda") for c in cs]
    dYs = [torch.from_numpy(c["dy"]).cuda() for c in cs]
    dX = torch.zeros((T, K), device="cuda")
    eng.forward_group(ws, ads, X, Ys)
    eng.backward_group(ws, ads, dYs, X, dX, flags=G.FLAG_REUSE_LOW)
    eng.sync()
    ys, dxr, das, dbs = _reference(oracle, cs)
    for j in range(3):
        assert oracle.rel_fro(Ys[j].cpu().numpy(), ys[j]) < 2e-2, j
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, das[j]) < 5e-3 and oracle.rel_fro(db, dbs[j]) < 5e-3, j
    assert oracle.rel_fro(dX.cpu().numpy(), dxr) < 2e-2
    _free(ws, ads)


def test_calls_from_several_host_threads(G, eng, oracle):
    """The reference calls the engine from Parallel.Invoke (q | k | v, gate | up) and the engine serialises the calls
    with a lock (TransformerBlock.cs:381-385, GpuLoraEngine.Forward.cs:121): three threads, host buffers, one engine."""
    import threading
    cs = _members(S.TYPE_Q4_K, (256, 128, 128), 512, 70, seed=61, adapted=(1, 1, 1), biased=(1, 1, 1))
    eng.set_math_mode(0)
    ws, ads = _upload(eng, cs)
    ys, _, das, dbs = _reference(oracle, cs)
    out = [None] * 3
    errs = []

    def work(j):
        try:
            for _ in range(3):
                out[j] = eng.forward(ws[j], ads[j], cs[j]["x"])
            eng.backward(ws[j], ads[j], cs[j]["dy"], cs[j]["x"], np.zeros((70, 512), np.float32))
        except Exception as exc:      # noqa: BLE001
            errs.append(exc)

    threads = [threading.Thread(target=work, args=(j,)) for j in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errs, errs
    for j in range(3):
        assert oracle.rel_fro(out[j], ys[j]) < 2e-2
        da, db = ads[j].grads()
        assert oracle.rel_fro(da, das[j]) < 5e-3 and oracle.rel_fro(db, dbs[j]) < 5e-3
    _free(ws, ads)


def test_group_error_paths(G, eng):
    import torch
    a = S.make_projection_case(S.TYPE_Q4_K, 128, 512, 8, seed=1)
    b = S.make_projection_case(S.TYPE_Q4_K, 128, 256, 8, seed=2)
    wa = eng.upload_weight(a["qtype"], a["w"], 128, 512)
    wb = eng.upload_weight(b["qtype"], b["w"], 128, 256)
    X = torch.zeros((8, 512), device="cuda")
    Ys = [torch.zeros((8, 128), device="cuda") for _ in range(2)]
    with pytest.raises(G.GtError, match="share their input"):
        eng.forward_group([wa, wb], None, X, Ys)
    with pytest.raises(G.GtError, match="1 to 3"):
        eng.forward_group([wa] * 4, None, X, Ys * 2)
    wa.free()
    wb.free()
