"""CPU tests: the oracle against the reference's own known answers, its numpy mirror, and the golden fixtures.

Known answers come from the reference's tests (paths relative to the reference project root):
  tests/Glacier.Tune.Tests/AdversarialQuantizationTests.cs:15-60      Set/GetScaleMinK4 round trips
  tests/Glacier.Tune.Tests/SyntheticGgufFixture.cs:407-413            constant Q4_K block
  tests/Glacier.Tune.Tests/GgufMergerQuantizationTests.cs:118-191     quantize -> dequantize fidelity bounds
  tests/Glacier.Tune.Tests/AdversarialQuantizationTests.cs:62-166     adversarial quantizer inputs
  tests/Glacier.Tune.Tests/KernelTests.cs:133-202                     fast LoRA backward == naive, 1e-4
  tests/Glacier.Tune.Tests/GradientAndGpuParityTests.cs:37-64         B == 0: dA == 0 exactly, dB != 0
"""
import os

import numpy as np
import pytest

from glacier.tune_b200 import synth as S

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_scale_min_k4_exhaustive_roundtrip(oracle):
    scales = np.zeros(12, np.uint8)
    for j in range(8):
        for sc in range(64):
            for m in range(64):
                scales[:] = 0
                oracle.set_scale_min_k4(j, scales, sc, m)
                assert oracle.get_scale_min_k4(j, scales) == (sc, m)


def test_scale_min_k4_multiblock_no_interference(oracle):
    sc = [0, 15, 31, 45, 63, 7, 52, 1]
    m = [63, 44, 16, 2, 0, 59, 10, 33]
    scales = np.zeros(12, np.uint8)
    for j in range(8):
        oracle.set_scale_min_k4(j, scales, sc[j], m[j])
    assert [oracle.get_scale_min_k4(j, scales) for j in range(8)] == list(zip(sc, m))
    # the vectorised packer of the input generator and the numpy unpacker agree with the C functions
    packed = S.pack_scales_q4k(np.array([sc]), np.array([m]))
    assert np.array_equal(packed[0], scales)
    usc, um = oracle.np_unpack_scales_q4k(packed)
    assert usc[0].tolist() == sc and um[0].tolist() == m


def test_constant_block_fixture(oracle):
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([0.01], np.float16).view(np.uint8)
    blk[2:4] = 0
    blk[4:16] = 1
    blk[16:] = 0x11
    w = oracle.dequant_blocks(oracle.TYPE_Q4_K, blk)
    assert np.all(w == np.float32(np.float16(0.01)))


def _fidelity(oracle, src):
    q = oracle.quantize_row_q4k(src)
    deq = oracle.dequant_blocks(oracle.TYPE_Q4_K, q)
    assert np.all(np.isfinite(deq))
    return q, deq


def test_q4k_quantizer_fidelity_roundtrip(oracle):
    i = np.arange(512, dtype=np.float32)
    src = (np.sin(i * np.float32(0.05)) * np.cos(i * np.float32(0.013)) * np.float32(2.5)).astype(np.float32)
    _, deq = _fidelity(oracle, src)
    cos = float(src @ deq / (np.linalg.norm(src) * np.linalg.norm(deq)))
    assert cos > 0.995
    assert float(np.mean((deq - src) ** 2)) < 0.03
    assert float(np.max(np.abs(deq - src))) < 0.5


def test_q4k_quantizer_edge_cases(oracle):
    q, deq = _fidelity(oracle, np.zeros(256, np.float32))
    assert oracle.lib().gt_oracle_half_to_float(int(q[0:2].view(np.uint16)[0])) == 0.0
    assert np.all(deq == 0.0)
    _, deq = _fidelity(oracle, np.full(256, 4.0, np.float32))
    assert np.all(np.abs(deq - 4.0) < 0.1)
    src = np.zeros(512, np.float32)
    src[42], src[300] = 100.0, -50.0
    _, deq = _fidelity(oracle, src)
    assert deq[42] > 80.0 and deq[300] < -40.0
    _, deq = _fidelity(oracle, np.full(512, -1000.0, np.float32))
    assert np.all(np.abs(deq + 1000.0) < 50.0)
    den = np.where(np.arange(256) % 2 == 0, 1.401298e-45, -1.401298e-45).astype(np.float32)
    _fidelity(oracle, den)


def test_q4k_quantizer_gaussian_fidelity(oracle):
    rng = np.random.default_rng(42)
    src = (rng.standard_normal(2048) * 0.05).astype(np.float32)
    _, deq = _fidelity(oracle, src)
    cos = float(src @ deq / (np.linalg.norm(src) * np.linalg.norm(deq)))
    assert cos > 0.99


@pytest.mark.parametrize("qtype", [S.TYPE_Q4_K, S.TYPE_Q6_K])
def test_c_oracle_matches_numpy_mirror_bit_exact(oracle, qtype):
    rng = np.random.default_rng(3)
    blocks = S.make_q4k_blocks(513, rng) if qtype == S.TYPE_Q4_K else S.make_q6k_blocks(513, rng)
    got = oracle.dequant_blocks(qtype, blocks).reshape(-1, 256)
    want = oracle.np_dequant_q4k(blocks) if qtype == S.TYPE_Q4_K else oracle.np_dequant_q6k(blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q6k_generator_inverts_decode(oracle):
    # the generator places 6-bit quants by the inverse of the decode: every quant value must come back
    rng = np.random.default_rng(11)
    blocks = S.make_q6k_blocks(4, rng)
    blocks[:, 192:208] = np.int8(1).view(np.uint8)              # all sub-scales 1
    blocks[:, 208:210] = np.array([1.0], np.float16).view(np.uint8)   # d = 1
    w = oracle.np_dequant_q6k(blocks)
    assert w.min() >= -32 and w.max() <= 31 and np.all(w == np.round(w))
    assert len(np.unique(w)) == 64


def test_flat_stream_rows(oracle):
    # in_features = 896 is 3.5 super-blocks: odd rows start in the middle of a shared block
    c = S.make_projection_case(S.TYPE_Q4_K, 64, 896, 4, seed=3)
    rows = oracle.dequant_rows(S.TYPE_Q4_K, c["w"], 896, 0, 64)
    flat = oracle.dequant_blocks(S.TYPE_Q4_K, c["w"]).reshape(64, 896)
    assert np.array_equal(rows, flat)
    part = oracle.dequant_rows(S.TYPE_Q4_K, c["w"], 896, 5, 3)
    assert np.array_equal(part, flat[5:8])


def test_lora_backward_matches_naive(oracle):
    T, K, N, R = 8, 32, 24, 16
    scaling = 32.0 / R
    rng = np.random.default_rng(42)
    x = rng.uniform(-1, 1, (T, K)).astype(np.float32)
    dy = rng.uniform(-1, 1, (T, N)).astype(np.float32)
    a = (rng.standard_normal((K, R)) / np.sqrt(K)).astype(np.float32)
    b = rng.uniform(-0.05, 0.05, (R, N)).astype(np.float32)
    dx = np.zeros((T, K), np.float32)
    dx, ga, gb = oracle.lora_backward(x, dy, a, b, T, K, N, R, scaling, dx=dx)
    low = x @ a
    dlow = dy @ b.T
    assert np.max(np.abs(gb - scaling * low.T @ dy)) < 1e-4
    assert np.max(np.abs(ga - scaling * x.T @ dlow)) < 1e-4
    assert np.max(np.abs(dx - scaling * dlow @ a.T)) < 1e-4


@pytest.mark.parametrize("qtype,N,K,T", [(S.TYPE_Q4_K, 96, 512, 9), (S.TYPE_Q6_K, 64, 256, 5), (S.TYPE_Q4_K, 40, 896, 6)])
def test_projection_forward_backward_vs_fp64(oracle, qtype, N, K, T):
    c = S.make_projection_case(qtype, N, K, T, seed=5, with_bias=True)
    W = oracle.dequant_rows(qtype, c["w"], K, 0, N).astype(np.float64)
    X, dY, A, B = (c[k].astype(np.float64) for k in ("x", "dy", "a", "b"))
    s = c["scaling"]
    y = oracle.proj_forward(qtype, c["w"], c["bias"], c["x"], K, N, T, c["a"], c["b"], 16, s)
    assert oracle.rel_fro(y, X @ W.T + c["bias"] + s * (X @ A) @ B) < 1e-6
    y64 = oracle.matmul_batch(qtype, c["w"], c["x"], K, N, T, c["bias"], f64=True)
    assert oracle.rel_fro(y64, X @ W.T + c["bias"]) < 1e-12
    dx0 = np.ones((T, K), np.float32)                     # accumulate-into semantics
    dx, ga, gb = oracle.proj_backward(qtype, c["w"], c["dy"], c["x"], K, N, T, c["a"], c["b"], 16, s, dx=dx0.copy())
    dlow = dY @ B.T
    assert oracle.rel_fro(dx - 1.0, dY @ W + s * dlow @ A.T) < 1e-5
    assert oracle.rel_fro(ga, s * X.T @ dlow) < 1e-5
    assert oracle.rel_fro(gb, s * (X @ A).T @ dY) < 1e-5
    assert oracle.rel_fro(oracle.base_backward_f64(qtype, c["w"], c["dy"], K, N, T), dY @ W) < 1e-12


def test_zero_b_skips_delta_and_gives_zero_dA(oracle):
    c = S.make_projection_case(S.TYPE_Q4_K, 64, 256, 7, seed=9, zero_b=True)
    y = oracle.proj_forward(S.TYPE_Q4_K, c["w"], None, c["x"], 256, 64, 7, c["a"], c["b"], 16, 2.0)
    base = oracle.matmul_batch(S.TYPE_Q4_K, c["w"], c["x"], 256, 64, 7)
    assert np.array_equal(y, base)
    _, ga, gb = oracle.proj_backward(S.TYPE_Q4_K, c["w"], c["dy"], c["x"], 256, 64, 7, c["a"], c["b"], 16, 2.0)
    assert np.all(ga == 0.0) and np.any(gb != 0.0)


def test_clip_gradients(oracle):
    g = np.arange(1, 11, dtype=np.float32)
    norm = float(np.sqrt(np.sum(g.astype(np.float64) ** 2)))
    g1 = g.copy()
    assert abs(oracle.clip_gradients(g1, 1.0) - norm) < 1e-9
    assert abs(float(np.linalg.norm(g1)) - 1.0) < 1e-5
    g2 = g.copy()
    oracle.clip_gradients(g2, 1e9)
    assert np.array_equal(g2, g)
    g3 = g.copy()
    g3[3] = np.inf
    assert oracle.clip_gradients(g3, 1.0) == 0.0 and np.all(g3 == 0)


def test_golden_fixtures(oracle):
    """Committed vectors (tests/golden/make_golden.py): block bytes -> fp32 weights, and one small projection."""
    d = np.load(os.path.join(GOLDEN, "dequant_golden.npz"))
    for qtype, key in ((S.TYPE_Q4_K, "q4k"), (S.TYPE_Q6_K, "q6k")):
        got = oracle.dequant_blocks(qtype, d[f"{key}_blocks"]).reshape(-1, 256)
        assert np.array_equal(got.view(np.uint32), d[f"{key}_weights"].view(np.uint32))
    p = np.load(os.path.join(GOLDEN, "projection_golden.npz"))
    qtype, N, K, T, R = (int(p[k]) for k in ("qtype", "N", "K", "T", "rank"))
    s = float(p["scaling"])
    y = oracle.proj_forward(qtype, p["w"], p["bias"], p["x"], K, N, T, p["a"], p["b"], R, s)
    dx, ga, gb = oracle.proj_backward(qtype, p["w"], p["dy"], p["x"], K, N, T, p["a"], p["b"], R, s)
    for got, key in ((y, "y"), (dx, "dx"), (ga, "da"), (gb, "db")):
        assert oracle.rel_fro(got, p[key]) < 1e-6, key


def test_decoders_match_gguf_golden_fixture(oracle):
    """Q4_K and Q6_K decode pinned to the GGUF project's own decoder: the committed vectors were produced by
    gguf.quants.dequantize (tests/golden/make_gguf_golden.py).  C oracle and numpy mirror must match them bit for bit."""
    d = np.load(os.path.join(GOLDEN, "gguf_dequant_golden.npz"))
    for qtype, key, mirror in ((S.TYPE_Q4_K, "q4k", oracle.np_dequant_q4k), (S.TYPE_Q6_K, "q6k", oracle.np_dequant_q6k)):
        blocks, want = d[f"{key}_blocks"], d[f"{key}_weights"]
        got_c = oracle.dequant_blocks(qtype, blocks).reshape(want.shape)
        got_np = mirror(blocks).reshape(want.shape)
        assert np.array_equal(got_c.view(np.uint32), want.view(np.uint32)), key
        assert np.array_equal(got_np.view(np.uint32), want.view(np.uint32)), key


def test_q40_q80_decoders_match_gguf_golden_fixture(oracle):
    """Q4_0 and Q8_0 (the reference's other GEMM types, src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:18-26): the C oracle's row
    decoder against vectors produced by gguf.quants.dequantize, bit for bit; and against the generator when gguf is here."""
    d = np.load(os.path.join(GOLDEN, "gguf_dequant_golden_q40_q80.npz"))
    for qtype, key in ((S.TYPE_Q4_0, "q40"), (S.TYPE_Q8_0, "q80")):
        blocks, want = d[f"{key}_blocks"], d[f"{key}_weights"]
        nb = len(blocks)
        K = 256                                    # rows of 8 blocks
        got = oracle.dequant_rows(qtype, blocks.reshape(-1), K, 0, nb * 32 // K)
        assert np.array_equal(got.reshape(-1).view(np.uint32), want.reshape(-1).view(np.uint32)), key
    try:
        import gguf  # noqa: F401
    except ImportError:
        return
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("make_gguf_golden", os.path.join(root, "tests", "golden", "make_gguf_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    q40, q80 = gen.draw_small_blocks()
    w40, w80 = gen.gguf_decode_small(q40, q80)
    assert np.array_equal(q40, d["q40_blocks"]) and np.array_equal(q80, d["q80_blocks"])
    assert np.array_equal(w40.view(np.uint32), d["q40_weights"].view(np.uint32))
    assert np.array_equal(w80.view(np.uint32), d["q80_weights"].view(np.uint32))


def test_q40_q80_projection_oracle_matches_dense_numpy(oracle):
    """Forward and backward of the CPU path on Q4_0 / Q8_0 weights against a dense fp64 product of the decoded rows."""
    rng = np.random.default_rng(3)
    N, K, T = 48, 96, 7
    for qtype in (S.TYPE_Q4_0, S.TYPE_Q8_0):
        w = S.make_weight(qtype, N, K, seed=11)
        W = oracle.dequant_rows(qtype, w, K, 0, N).astype(np.float64)
        x = rng.standard_normal((T, K), dtype=np.float32)
        dy = rng.standard_normal((T, N), dtype=np.float32)
        y = oracle.matmul_batch(qtype, w, x, K, N, T, None, f64=True)
        assert np.allclose(y, x.astype(np.float64) @ W.T, rtol=1e-12, atol=1e-12)
        dx = oracle.base_backward_f64(qtype, w, dy, K, N, T)
        assert np.allclose(dx, dy.astype(np.float64) @ W, rtol=1e-12, atol=1e-12)


def test_decoders_match_gguf_package_live(oracle):
    """The same comparison against the installed gguf package on fresh seeded blocks (skipped where it is absent),
    and a check that the committed fixture is what the generator script writes today."""
    pytest.importorskip("gguf")
    sys_path_root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_gguf_golden", os.path.join(sys_path_root, "tests", "golden", "make_gguf_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    q4, q6 = gen.draw_blocks()
    w4, w6 = gen.gguf_decode(q4, q6)
    d = np.load(os.path.join(GOLDEN, "gguf_dequant_golden.npz"))
    assert np.array_equal(q4, d["q4k_blocks"]) and np.array_equal(q6, d["q6k_blocks"])
    assert np.array_equal(w4.view(np.uint32), d["q4k_weights"].view(np.uint32))
    assert np.array_equal(w6.view(np.uint32), d["q6k_weights"].view(np.uint32))
    rng = np.random.default_rng(77)
    q4, q6 = S.make_q4k_blocks(257, rng), S.make_q6k_blocks(257, rng)
    w4, w6 = gen.gguf_decode(q4, q6)
    assert np.array_equal(oracle.dequant_blocks(S.TYPE_Q4_K, q4).reshape(w4.shape).view(np.uint32), w4.view(np.uint32))
    assert np.array_equal(oracle.dequant_blocks(S.TYPE_Q6_K, q6).reshape(w6.shape).view(np.uint32), w6.view(np.uint32))
