"""Generates the committed golden fixtures.

The reference (C#/.NET with un-vendored NuGet packages) cannot be run to produce vectors, so these are
computed in fp64 numpy from the decode rules cited in oracle/oracle.py (tune_bwd.cu:43-51,209-211,234-240,
279-289,311-315) by the numpy mirror - NOT by the C oracle or the CUDA library, which are both checked
against them:
  dequant_golden.npz     64 seeded Q4_K blocks (+ the reference's constant-block fixture as block 0) and 64 seeded
                         Q6_K blocks with their fp32 weights
  projection_golden.npz  one small LoRA-adapted Q4_K projection (N=72, K=512, T=11, r=16, bias): inputs and
                         Y, dX, dA, dB evaluated in fp64 and stored as fp32

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from glacier.tune_b200 import synth as S  # noqa: E402
from oracle import oracle as O  # noqa: E402  (numpy mirror functions only)


def main():
    rng = np.random.default_rng(20240)
    q4 = S.make_q4k_blocks(64, rng)
    q4[0, 0:2] = np.array([0.01], np.float16).view(np.uint8)      # SyntheticGgufFixture.cs:407-413
    q4[0, 2:4] = 0
    q4[0, 4:16] = 1
    q4[0, 16:] = 0x11
    q6 = S.make_q6k_blocks(64, rng)
    np.savez_compressed(os.path.join(HERE, "dequant_golden.npz"), q4k_blocks=q4, q4k_weights=O.np_dequant_q4k(q4),
                        q6k_blocks=q6, q6k_weights=O.np_dequant_q6k(q6))

    N, K, T, R = 72, 512, 11, 16
    c = S.make_projection_case(S.TYPE_Q4_K, N, K, T, seed=20241, rank=R, alpha=32.0, with_bias=True)
    W = O.np_dequant_q4k(c["w"].reshape(-1, 144)).reshape(N, K).astype(np.float64)
    X, dY, A, B = (c[k].astype(np.float64) for k in ("x", "dy", "a", "b"))
    s = c["scaling"]
    dlow = dY @ B.T
    np.savez_compressed(os.path.join(HERE, "projection_golden.npz"), qtype=S.TYPE_Q4_K, N=N, K=K, T=T, rank=R, scaling=s,
                        w=c["w"], bias=c["bias"], x=c["x"], dy=c["dy"], a=c["a"], b=c["b"],
                        y=(X @ W.T + c["bias"] + s * (X @ A) @ B).astype(np.float32),
                        dx=(dY @ W + s * dlow @ A.T).astype(np.float32),
                        da=(s * X.T @ dlow).astype(np.float32), db=(s * (X @ A).T @ dY).astype(np.float32))


if __name__ == "__main__":
    main()
