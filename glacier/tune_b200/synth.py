"""Seeded synthetic inputs for the K-quant projection path (numpy only, no GPU, no oracle).

There is no public dataset on this path: the workloads are GGUF K-quant weight tensors plus dense
activations, so every benchmark and parity case is generated here from a seed with the block value
distributions the workload definitions state:

* Q4_K super-block (144 B, ``half d; half dmin; u8 scales[12]; u8 qs[128]``,
  src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:28-33): ``d ~ fp16(U(2e-4, 2e-3))``, ``dmin ~ fp16(U(0, 1e-3))``,
  eight 6-bit scales and mins uniform in 0..63 packed the way ``GgufMerger.SetScaleMinK4`` packs them
  (src/Glacier.Tune/Export/GgufMerger.cs:765-778), 256 quants uniform in 0..15 packed
  ``qs[g*32+l] = q[g*64+l] | q[g*64+l+32] << 4`` (GgufMerger.cs:746-754).
* Q6_K super-block (210 B, ``u8 ql[128]; u8 qh[64]; i8 scales[16]; half d``, tune_bwd.cu:35-40):
  256 six-bit quants uniform in 0..63 placed by the inverse of the decode at tune_bwd.cu:279-289,
  sixteen int8 sub-scales uniform in -32..31, ``d ~ fp16(U(1e-4, 1e-3))``.

Projection ordinals follow the reference's layer layout (src/Glacier.Tune/Model/TransformerBlock.cs:149-165).
"""
from __future__ import annotations

import numpy as np

TYPE_F32, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 2, 8, 12, 14
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q6_K: 210, TYPE_Q4_0: 18, TYPE_Q8_0: 34}
PROJ_ORDINAL = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6}

# (out_features N, in_features K) of the Qwen2.5-7B layer projections
QWEN7B_PROJ = {
    "q": (3584, 3584), "k": (512, 3584), "v": (512, 3584), "o": (3584, 3584),
    "gate": (18944, 3584), "up": (18944, 3584), "down": (3584, 18944),
}


def seed_for(config: int, layer: int, proj: str) -> int:
    return 20240 + 1000 * config + 10 * layer + PROJ_ORDINAL[proj]


def pack_scales_q4k(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """(sc, m) [nb, 8] in 0..63 -> scales [nb, 12] uint8 (vectorised SetScaleMinK4)."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), np.uint8)
    for j in range(4):
        out[:, j] = sc[:, j] & 0x3F
        out[:, j + 4] = m[:, j] & 0x3F
    for j in range(4, 8):
        out[:, j + 4] = (sc[:, j] & 0x0F) | ((m[:, j] & 0x0F) << 4)
        out[:, j - 4] |= (sc[:, j] >> 4) << 6
        out[:, j] |= (m[:, j] >> 4) << 6
    return out


def make_q4k_blocks(nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """[nblocks, 144] uint8."""
    d = rng.uniform(2e-4, 2e-3, nblocks).astype(np.float16)
    dmin = rng.uniform(0.0, 1e-3, nblocks).astype(np.float16)
    sc = rng.integers(0, 64, (nblocks, 8), dtype=np.uint8)
    m = rng.integers(0, 64, (nblocks, 8), dtype=np.uint8)
    q = rng.integers(0, 16, (nblocks, 4, 64), dtype=np.uint8)
    out = np.empty((nblocks, 144), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nblocks, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nblocks, 2)
    out[:, 4:16] = pack_scales_q4k(sc, m)
    out[:, 16:144] = (q[:, :, :32] | (q[:, :, 32:] << 4)).reshape(nblocks, 128)
    return out


def make_q6k_blocks(nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """[nblocks, 210] uint8."""
    q = rng.integers(0, 64, (nblocks, 256), dtype=np.uint8)
    scales = rng.integers(-32, 32, (nblocks, 16), dtype=np.int8)
    d = rng.uniform(1e-4, 1e-3, nblocks).astype(np.float16)
    c = np.arange(256)
    step, rem = c >> 7, c & 127
    quad, lane = rem >> 5, rem & 31
    ql_idx = step * 64 + (quad & 1) * 32 + lane
    ql_shift = np.where(quad >= 2, 4, 0).astype(np.uint8)
    qh_idx = step * 32 + lane
    qh_shift = (quad * 2).astype(np.uint8)
    ql = np.zeros((nblocks, 128), np.uint8)
    qh = np.zeros((nblocks, 64), np.uint8)
    for col in range(256):   # 256 vectorised scatters (indices collide across columns by design)
        ql[:, ql_idx[col]] |= (q[:, col] & 0x0F) << ql_shift[col]
        qh[:, qh_idx[col]] |= (q[:, col] >> 4) << qh_shift[col]
    out = np.empty((nblocks, 210), np.uint8)
    out[:, 0:128] = ql
    out[:, 128:192] = qh
    out[:, 192:208] = scales.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(nblocks, 2)
    return out


def make_q40_blocks(nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """[nblocks, 18] uint8: fp16 d, then 16 bytes of nibbles (weights 0-15 low, 16-31 high)."""
    out = np.empty((nblocks, 18), np.uint8)
    out[:, 0:2] = rng.uniform(2e-3, 2e-2, nblocks).astype(np.float16).view(np.uint8).reshape(nblocks, 2)
    out[:, 2:18] = rng.integers(0, 256, (nblocks, 16), dtype=np.uint8)
    return out


def make_q80_blocks(nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """[nblocks, 34] uint8: fp16 d, then 32 int8."""
    out = np.empty((nblocks, 34), np.uint8)
    out[:, 0:2] = rng.uniform(1e-4, 1e-3, nblocks).astype(np.float16).view(np.uint8).reshape(nblocks, 2)
    out[:, 2:34] = rng.integers(-127, 128, (nblocks, 32), dtype=np.int8).view(np.uint8)
    return out


def make_weight(qtype: int, N: int, K: int, seed: int) -> np.ndarray:
    """Quantized [N, K] weight as a flat uint8 byte stream of N*K/256 super-blocks (row-major); Q4_0 / Q8_0: N*K/32
    blocks, rows whole numbers of blocks."""
    rng = np.random.default_rng(seed)
    if qtype in (TYPE_Q4_0, TYPE_Q8_0):
        assert K % 32 == 0
        return (make_q40_blocks(N * K // 32, rng) if qtype == TYPE_Q4_0 else make_q80_blocks(N * K // 32, rng)).reshape(-1)
    assert (N * K) % 256 == 0, "weight element count must be a whole number of super-blocks"
    nb = N * K // 256
    blocks = make_q4k_blocks(nb, rng) if qtype == TYPE_Q4_K else make_q6k_blocks(nb, rng)
    return blocks.reshape(-1)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even), returned as fp32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def make_projection_case(qtype: int, N: int, K: int, T: int, seed: int, rank: int = 16, alpha: float = 32.0,
                         x_bf16: bool = False, zero_b: bool = False, with_bias: bool = False) -> dict:
    """One LoRA-adapted projection: weight bytes, X, dY, A [K, r], B [r, N] (reference-native layout)."""
    w = make_weight(qtype, N, K, seed)
    rng = np.random.default_rng(seed + 500_000)
    x = rng.standard_normal((T, K), dtype=np.float32)
    if x_bf16:
        x = bf16_round(x)
    dy = rng.standard_normal((T, N), dtype=np.float32)
    # drawn in the PEFT orientation (A r x K, B N x r), stored reference-native (A [K, r], B [r, N])
    a = np.ascontiguousarray((rng.standard_normal((rank, K), dtype=np.float32) * np.float32(0.02)).T)
    b = np.ascontiguousarray((rng.standard_normal((N, rank), dtype=np.float32) * np.float32(0.02)).T)
    if zero_b:
        b[:] = 0
    bias = (rng.standard_normal(N, dtype=np.float32) * np.float32(0.1)) if with_bias else None
    return dict(qtype=qtype, N=N, K=K, T=T, w=w, x=x, dy=dy, a=a, b=b, bias=bias, rank=rank, alpha=alpha,
                scaling=alpha / rank)
