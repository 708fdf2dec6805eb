"""ctypes front end of the CPU oracle (``oracle/gt_oracle.c``) plus numpy mirrors of its dequantizers.

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by ``__graft_entry__.smoke()`` (as the checker) and by
``bench.py``'s CPU-baseline leg.  The shipped package never imports this module.

The numpy functions restate the same reference lines as the C file, independently, so the two can be
checked against each other:
  Q4_K decode  src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:28-33,43-51,209-211,234-240
  Q6_K decode  src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:35-40,279-289,311-315   (the reference has no Q6_K test or
               CPU source; pinned instead to gguf.quants.dequantize, tests/golden/make_gguf_golden.py)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgt_oracle.so")

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 1, 2, 8, 12, 14
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q6_K: 210, TYPE_Q4_0: 18, TYPE_Q8_0: 34}

_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc, OpenMP)."""
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(
            os.path.join(HERE, "gt_oracle.c")):
        subprocess.check_call(["make", "-C", HERE, "-s"])
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = C.CDLL(LIB_PATH)
        _lib.gt_oracle_half_to_float.restype = C.c_float
        _lib.gt_oracle_half_to_float.argtypes = [C.c_uint16]
        _lib.gt_oracle_float_to_half.restype = C.c_uint16
        _lib.gt_oracle_float_to_half.argtypes = [C.c_float]
        _lib.gt_oracle_clip_gradients.restype = C.c_double
        _lib.gt_oracle_clip_gradients.argtypes = [C.c_void_p, C.c_int64, C.c_double]
        _lib.gt_oracle_block_bytes.restype = C.c_int64
        _lib.gt_oracle_cross_entropy.restype = C.c_float
        _lib.gt_oracle_cross_entropy.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                 C.c_void_p, C.c_void_p]
        _lib.gt_oracle_attention_forward.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4
        _lib.gt_oracle_attention_backward.argtypes = [C.c_void_p] * 8 + [C.c_int] * 4
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def num_threads() -> int:
    return int(lib().gt_oracle_num_threads())


def set_threads(n: int) -> None:
    lib().gt_oracle_set_threads(C.c_int(n))


def get_scale_min_k4(j: int, scales12) -> tuple[int, int]:
    q = _u8(scales12)
    sc, m = C.c_uint8(), C.c_uint8()
    lib().gt_oracle_get_scale_min_k4(C.c_int(j), _p(q), C.byref(sc), C.byref(m))
    return sc.value, m.value


def set_scale_min_k4(j: int, scales12: np.ndarray, sc: int, m: int) -> None:
    assert scales12.dtype == np.uint8 and scales12.flags.c_contiguous
    lib().gt_oracle_set_scale_min_k4(C.c_int(j), _p(scales12), C.c_uint8(sc), C.c_uint8(m))


def dequant_blocks(qtype: int, blocks) -> np.ndarray:
    b = _u8(blocks).reshape(-1)
    n = b.size // BLOCK_BYTES[qtype]
    out = np.empty(n * 256, np.float32)
    rc = lib().gt_oracle_dequant_blocks(C.c_int(qtype), _p(b), C.c_int64(n), _p(out))
    assert rc == 0
    return out


def dequant_rows(qtype: int, w, K: int, row0: int, nrows: int) -> np.ndarray:
    wb = _w(qtype, w)
    out = np.empty((nrows, K), np.float32)
    rc = lib().gt_oracle_dequant_rows(C.c_int(qtype), _p(wb), C.c_int(K), C.c_int64(row0), C.c_int64(nrows), _p(out))
    assert rc == 0
    return out


def quantize_row_q4k(src) -> np.ndarray:
    s = _f32(src).reshape(-1)
    assert s.size % 256 == 0
    out = np.zeros(s.size // 256 * 144, np.uint8)
    lib().gt_oracle_quantize_row_q4k(_p(s), _p(out), C.c_int(s.size))
    return out


def _w(qtype, w):
    if qtype == TYPE_F32:
        return _f32(w).reshape(-1)
    if qtype == TYPE_F16:
        return np.ascontiguousarray(w, dtype=np.float16).reshape(-1)
    return _u8(w).reshape(-1)


def matmul_batch(qtype, w, x, K, N, T, bias=None, f64=False) -> np.ndarray:
    wb, x = _w(qtype, w), _f32(x)
    bias = None if bias is None else _f32(bias)
    y = np.empty((T, N), np.float64 if f64 else np.float32)
    fn = lib().gt_oracle_matmul_batch_f64 if f64 else lib().gt_oracle_matmul_batch
    rc = fn(C.c_int(qtype), _p(wb), _p(x), _p(y), C.c_int(K), C.c_int(N), C.c_int(T), _p(bias))
    assert rc == 0
    return y


def proj_forward(qtype, w, bias, x, K, N, T, a=None, b=None, R=0, scaling=0.0) -> np.ndarray:
    """LoraAdapter.Forward on the CPU path (fp32)."""
    wb, x = _w(qtype, w), _f32(x)
    bias = None if bias is None else _f32(bias)
    a = None if a is None else _f32(a)
    b = None if b is None else _f32(b)
    y = np.empty((T, N), np.float32)
    rc = lib().gt_oracle_proj_forward(C.c_int(qtype), _p(wb), _p(bias), _p(x), _p(y), C.c_int(K), C.c_int(N),
                                      C.c_int(T), _p(a), _p(b), C.c_int(R), C.c_float(scaling))
    assert rc == 0
    return y


def proj_backward(qtype, w, dy, x, K, N, T, a=None, b=None, R=0, scaling=0.0, dx=None, ga=None, gb=None,
                  want_dx=True):
    """LoraAdapter.Backward on the CPU path: accumulates into dx / ga / gb (created as zeros when absent)."""
    wb, dy, x = _w(qtype, w), _f32(dy), _f32(x)
    if want_dx and dx is None:
        dx = np.zeros((T, K), np.float32)
    if a is not None:
        a, b = _f32(a), _f32(b)
        if ga is None:
            ga = np.zeros((K, R), np.float32)
        if gb is None:
            gb = np.zeros((R, N), np.float32)
    rc = lib().gt_oracle_proj_backward(C.c_int(qtype), _p(wb), _p(dy), _p(x), _p(dx), C.c_int(K), C.c_int(N),
                                       C.c_int(T), _p(a), _p(b), _p(ga), _p(gb), C.c_int(R), C.c_float(scaling))
    assert rc == 0
    return dx, ga, gb


def base_backward_f64(qtype, w, dy, K, N, T) -> np.ndarray:
    wb, dy = _w(qtype, w), _f32(dy)
    dx = np.empty((T, K), np.float64)
    rc = lib().gt_oracle_base_backward_f64(C.c_int(qtype), _p(wb), _p(dy), _p(dx), C.c_int(T), C.c_int(K), C.c_int(N))
    assert rc == 0
    return dx


def lora_backward(x, dy, a, b, T, K, N, R, scaling, dx=None, ga=None, gb=None):
    x, dy, a, b = _f32(x), _f32(dy), _f32(a), _f32(b)
    if ga is None:
        ga = np.zeros((K, R), np.float32)
    if gb is None:
        gb = np.zeros((R, N), np.float32)
    rc = lib().gt_oracle_lora_backward(_p(x), _p(dy), _p(a), _p(b), _p(ga), _p(gb), _p(dx), C.c_int(T), C.c_int(K),
                                       C.c_int(N), C.c_int(R), C.c_float(scaling))
    assert rc == 0
    return dx, ga, gb


def clip_gradients(g: np.ndarray, max_norm: float) -> float:
    assert g.dtype == np.float32 and g.flags.c_contiguous
    return float(lib().gt_oracle_clip_gradients(_p(g), C.c_int64(g.size), C.c_double(max_norm)))


# ------------------------------------------------------------------------------------------------
# numpy mirrors (independent restatement, vectorised)
# ------------------------------------------------------------------------------------------------
def np_unpack_scales_q4k(scales: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """scales [..., 12] uint8 -> (sc [..., 8], m [..., 8]) per tune_bwd.cu:43-51."""
    q = scales.astype(np.uint8)
    sc = np.empty(q.shape[:-1] + (8,), np.uint8)
    m = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = q[..., j] & 63
        m[..., j] = q[..., j + 4] & 63
    for j in range(4, 8):
        sc[..., j] = (q[..., j + 4] & 0x0F) | ((q[..., j - 4] >> 6) << 4)
        m[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, m


def np_dequant_q4k(blocks: np.ndarray) -> np.ndarray:
    """blocks [nb, 144] uint8 -> [nb, 256] float32, fp32 arithmetic in the reference's order."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)            # [nb,1]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, m = np_unpack_scales_q4k(b[:, 4:16])
    qs = b[:, 16:144].reshape(-1, 4, 32)
    nib = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)   # sub-block ib = 2g + hi
    d_sub = (d * sc.astype(np.float32))[:, :, None]
    m_sub = (dmin * m.astype(np.float32))[:, :, None]
    return (d_sub * nib - m_sub).astype(np.float32).reshape(-1, 256)


def np_dequant_q6k(blocks: np.ndarray) -> np.ndarray:
    """blocks [nb, 210] uint8 -> [nb, 256] float32 per tune_bwd.cu:279-289,311-315."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 210)
    ql, qh = b[:, 0:128], b[:, 128:192]
    scales = b[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
    c = np.arange(256)
    step, rem = c >> 7, c & 127
    quad, lane = rem >> 5, rem & 31
    ql_idx = step * 64 + (quad & 1) * 32 + lane
    ql_shift = np.where(quad >= 2, 4, 0).astype(np.uint8)
    qh_idx = step * 32 + lane
    qh_shift = (quad * 2).astype(np.uint8)
    sc_idx = step * 8 + (lane >> 4) + quad * 2
    q = (((ql[:, ql_idx] >> ql_shift) & 0x0F) | (((qh[:, qh_idx] >> qh_shift) & 0x03) << 4)).astype(np.int32) - 32
    return ((d * scales[:, sc_idx]).astype(np.float32) * q.astype(np.float32)).astype(np.float32)


def rel_fro(got, want) -> float:
    """Relative Frobenius error ||got - want|| / ||want|| in fp64."""
    g = np.asarray(got, np.float64)
    w = np.asarray(want, np.float64)
    den = np.linalg.norm(w)
    return float(np.linalg.norm(g - w) / (den if den > 0 else 1.0))


# ---- layer glue (SwiGLU, RoPE, RMSNorm): see the C file for the reference lines each one restates
def swiglu_forward(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().gt_oracle_swiglu_forward(_p(gate), _p(up), _p(out), C.c_int64(gate.size))
    return out


def swiglu_backward(dh, gate, up):
    dh, gate, up = _f32(dh), _f32(gate), _f32(up)
    dg, du = np.empty_like(gate), np.empty_like(gate)
    lib().gt_oracle_swiglu_backward(_p(dh), _p(gate), _p(up), _p(dg), _p(du), C.c_int64(gate.size))
    return dg, du


def rope(q, k, T, heads_q, heads_kv, head_dim, freq_base=1e6, freq_scale=1.0, rope_dim=-1, inverse=False):
    """Returns rotated copies of q [T, heads_q*head_dim] and k [T, heads_kv*head_dim] (either may be None)."""
    q = None if q is None else _f32(q).copy()
    k = None if k is None else _f32(k).copy()
    lib().gt_oracle_rope(_p(q) if q is not None else None, _p(k) if k is not None else None, T, heads_q, heads_kv, head_dim,
                         C.c_float(freq_base), C.c_float(freq_scale), rope_dim, 1 if inverse else 0)
    return q, k


def rmsnorm_forward(x, w, eps=1e-6) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    y = np.empty_like(x)
    lib().gt_oracle_rmsnorm_forward(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], C.c_float(eps))
    return y


def rmsnorm_backward(dy, x, w, eps=1e-6) -> np.ndarray:
    dy, x, w = _f32(dy), _f32(x), _f32(w)
    dx = np.empty_like(x)
    lib().gt_oracle_rmsnorm_backward(_p(dy), _p(x), _p(w), _p(dx), x.shape[0], x.shape[1], C.c_float(eps))
    return dx


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step):
    """One AdamW step in place on the fp32 arrays p, m, v (gradient g); step counts from 1."""
    for a in (p, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _f32(g)
    lib().gt_oracle_adamw_step(_p(p), _p(g), _p(m), _p(v), C.c_int64(p.size), C.c_float(lr), C.c_float(beta1),
                               C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay), C.c_int(step))



# ---- LM head and attention: see the C file for the reference lines each one restates
def cross_entropy(qtype, w, hidden, labels, V, tile=4096, want_grad=True):
    """FusedCrossEntropyLoss.ComputeLossAndGradients on the CPU path: (loss, valid count, dHidden or None).
    w is the [V, H] LM head (F32 / F16 / K-quant bytes), hidden [T, H], labels int32 [T] (ignored outside [0, V))."""
    wb, hidden = _w(qtype, w), _f32(hidden)
    labels = np.ascontiguousarray(labels, dtype=np.int32)
    T, H = hidden.shape
    dh = np.empty((T, H), np.float32) if want_grad else None
    valid = C.c_int32(0)
    loss = lib().gt_oracle_cross_entropy(C.c_int(qtype), _p(wb), _p(hidden), _p(labels), T, H, V, tile, _p(dh), C.byref(valid))
    return float(loss), int(valid.value), dh


def attention_forward(q, k, v, heads_q, heads_kv, head_dim):
    """CausalAttentionKernel.Forward: q [T, heads_q*head_dim], k / v [T, heads_kv*head_dim] -> (out, probs [heads_q, T, T])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    T = q.shape[0]
    out = np.empty_like(q)
    probs = np.empty((heads_q, T, T), np.float32)
    lib().gt_oracle_attention_forward(_p(q), _p(k), _p(v), _p(out), _p(probs), T, heads_q, heads_kv, head_dim)
    return out, probs


def attention_backward(d_out, q, k, v, probs, heads_q, heads_kv, head_dim):
    """CausalAttentionKernel.Backward -> (dq, dk, dv)."""
    d_out, q, k, v, probs = _f32(d_out), _f32(q), _f32(k), _f32(v), _f32(probs)
    T = q.shape[0]
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    lib().gt_oracle_attention_backward(_p(d_out), _p(q), _p(k), _p(v), _p(probs), _p(dq), _p(dk), _p(dv), T, heads_q, heads_kv, head_dim)
    return dq, dk, dv


# ---- the whole step on the CPU path: TransformerBlock.Forward / Backward and GgufLoraModel.ForwardLossAndBackward
# (src/Glacier.Tune/Model/TransformerBlock.cs:307-595,625-840, src/Glacier.Tune/Model/GgufLoraModel.cs:428-557) chained
# from the restated operators above.  A model is a dict:
#   cfg: n_heads, n_kv_heads, head_dim, rms_eps, rope_theta, vocab, hidden
#   layers: list of {"norm1", "norm2": fp32 [hidden], "proj": {name: {"qtype", "w", "N", "K", "bias" or None, "a", "b",
#           "rank", "scaling"}}} for name in q, k, v, o, gate, up, down
#   embed: (qtype, tensor), out_norm: fp32 [hidden], lm_head: (qtype, tensor)
PROJ_NAMES = ("q", "k", "v", "o", "gate", "up", "down")


def _pf(p, x):
    T = x.shape[0]
    return proj_forward(p["qtype"], p["w"], p.get("bias"), x, p["K"], p["N"], T, p.get("a"), p.get("b"), p.get("rank", 0), p.get("scaling", 0.0))


def _pb(p, dy, x, grads):
    """LoraAdapter.Backward into a zero-filled dX (AutogradScratchWorkspace.Wrap); dA / dB accumulate in grads[name]."""
    T = x.shape[0]
    ga, gb = grads if grads is not None else (None, None)
    dx, ga, gb = proj_backward(p["qtype"], p["w"], dy, x, p["K"], p["N"], T, p.get("a"), p.get("b"), p.get("rank", 0), p.get("scaling", 0.0),
                               ga=ga, gb=gb)
    return dx


def block_forward(cfg, layer, x):
    """Returns (out, state) - state holds what TransformerBlock.Backward reads (BlockActivationState)."""
    T = x.shape[0]
    P = layer["proj"]
    HQ, HK, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    n1 = rmsnorm_forward(x, layer["norm1"], cfg["rms_eps"])
    q, k, v = _pf(P["q"], n1), _pf(P["k"], n1), _pf(P["v"], n1)
    q, k = rope(q, k, T, HQ, HK, D, cfg["rope_theta"])
    attn, probs = attention_forward(q, k, v, HQ, HK, D)
    x1 = x + _pf(P["o"], attn)
    n2 = rmsnorm_forward(x1, layer["norm2"], cfg["rms_eps"])
    gate, up = _pf(P["gate"], n2), _pf(P["up"], n2)
    hidden = swiglu_forward(gate, up)
    out = x1 + _pf(P["down"], hidden)
    return out, dict(n1=n1, q=q, k=k, v=v, probs=probs, attn=attn, x1=x1, n2=n2, gate=gate, up=up, hidden=hidden)


def block_backward(cfg, layer, d_out, st, x_in, grads):
    """grads: {name: (dA, dB)} accumulated in place.  Returns dX of the block input."""
    P = layer["proj"]
    T = x_in.shape[0]
    HQ, HK, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    d_hidden = _pb(P["down"], d_out, st["hidden"], grads.get("down"))
    d_gate, d_up = swiglu_backward(d_hidden, st["gate"], st["up"])
    d_n2 = _pb(P["gate"], d_gate, st["n2"], grads.get("gate")) + _pb(P["up"], d_up, st["n2"], grads.get("up"))
    d_x1 = d_out + rmsnorm_backward(d_n2, st["x1"], layer["norm2"], cfg["rms_eps"])
    d_attn = _pb(P["o"], d_x1, st["attn"], grads.get("o"))
    dq, dk, dv = attention_backward(d_attn, st["q"], st["k"], st["v"], st["probs"], HQ, HK, D)
    dq, dk = rope(dq, dk, T, HQ, HK, D, cfg["rope_theta"], inverse=True)
    d_n1 = _pb(P["q"], dq, st["n1"], grads.get("q")) + _pb(P["k"], dk, st["n1"], grads.get("k"))
    d_n1 = d_n1 + _pb(P["v"], dv, st["n1"], grads.get("v"))
    return d_x1 + rmsnorm_backward(d_n1, x_in, layer["norm1"], cfg["rms_eps"])


def new_grads(model):
    """Zero dA / dB accumulators for every adapted projection, {layer: {name: (dA, dB)}}."""
    out = []
    for layer in model["layers"]:
        g = {}
        for name in PROJ_NAMES:
            p = layer["proj"][name]
            if p.get("a") is not None:
                g[name] = (np.zeros((p["K"], p["rank"]), np.float32), np.zeros((p["rank"], p["N"]), np.float32))
        out.append(g)
    return out


def flat_grads(model, grads) -> np.ndarray:
    """The reference's parameter order: layer -> q, k, v, o, gate, up, down -> A, B."""
    parts = []
    for g in grads:
        for name in PROJ_NAMES:
            if name in g:
                parts += [g[name][0].reshape(-1), g[name][1].reshape(-1)]
    return np.concatenate(parts) if parts else np.zeros(0, np.float32)


def model_forward(model, tokens):
    cfg = model["cfg"]
    et, ew = model["embed"]
    H = cfg["hidden"]
    x = np.concatenate([dequant_rows(et, ew, H, int(t), 1) for t in tokens]).astype(np.float32)
    xs, states = [], []
    for layer in model["layers"]:
        xs.append(x)
        x, st = block_forward(cfg, layer, x)
        states.append(st)
    return x, xs, states


def model_loss(model, tokens, labels):
    cfg = model["cfg"]
    x, _, _ = model_forward(model, tokens)
    fn = rmsnorm_forward(x, model["out_norm"], cfg["rms_eps"])
    lt, lw = model["lm_head"]
    loss, valid, _ = cross_entropy(lt, lw, fn, labels, cfg["vocab"], want_grad=False)
    return loss, valid


def model_forward_backward(model, tokens, labels, grads):
    """GgufLoraModel.ForwardLossAndBackward: returns the loss; grads (new_grads) accumulate."""
    cfg = model["cfg"]
    x, xs, states = model_forward(model, tokens)
    fn = rmsnorm_forward(x, model["out_norm"], cfg["rms_eps"])
    lt, lw = model["lm_head"]
    loss, _, d_fn = cross_entropy(lt, lw, fn, labels, cfg["vocab"])
    dx = rmsnorm_backward(d_fn, x, model["out_norm"], cfg["rms_eps"])
    for l in range(len(model["layers"]) - 1, -1, -1):
        dx = block_backward(cfg, model["layers"][l], dx, states[l], xs[l], grads[l])
    return loss
