"""Pins the Q4_K and Q6_K decoders to the GGUF project's own Python package.

The reference consumes GGUF tensors; its repository states the Q6_K layout only inside a CUDA kernel
(src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:263-332) and holds no Q6_K known answer.  The `gguf` package
(`gguf.quants.dequantize`, the format's reference decoder in numpy) is an independent implementation of the same
block formats.  This script draws seeded super-blocks with the workload generator, decodes them with `gguf`, and
stores blocks and fp32 weights in gguf_dequant_golden.npz.  The CPU tests compare the C oracle and its numpy mirror
with the stored weights bit for bit (and with `gguf` itself when it can be imported); the GPU test compares the
CUDA row decoder with the same file.

    python tests/golden/make_gguf_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from glacier.tune_b200 import synth as S  # noqa: E402

NBLOCKS = 96
SEED = 20246


def draw_blocks():
    """The seeded blocks of the fixture; block 0 of each type is replaced by an extreme-value block."""
    rng = np.random.default_rng(SEED)
    q4 = S.make_q4k_blocks(NBLOCKS, rng)
    q6 = S.make_q6k_blocks(NBLOCKS, rng)
    # extremes: largest scales / mins and all-ones quants (Q4_K); most negative sub-scales and quants 0 / 63 (Q6_K)
    q4[0, 4:16] = 0xFF
    q4[0, 16:] = 0xFF
    q6[0, 0:192] = 0xFF
    q6[0, 192:208] = np.array([-128] * 8 + [127] * 8, np.int8).view(np.uint8)
    q6[1, 0:192] = 0x00
    return q4, q6


def gguf_decode(q4, q6):
    from gguf import GGMLQuantizationType
    from gguf.quants import dequantize
    w4 = np.ascontiguousarray(dequantize(q4.reshape(-1), GGMLQuantizationType.Q4_K), np.float32).reshape(len(q4), 256)
    w6 = np.ascontiguousarray(dequantize(q6.reshape(-1), GGMLQuantizationType.Q6_K), np.float32).reshape(len(q6), 256)
    return w4, w6


def main():
    import gguf
    q4, q6 = draw_blocks()
    w4, w6 = gguf_decode(q4, q6)
    version = getattr(gguf, "__version__", None)
    if version is None:
        try:
            from importlib.metadata import version as _v
            version = _v("gguf")
        except Exception:  # noqa: BLE001
            version = "unknown"
    np.savez_compressed(os.path.join(HERE, "gguf_dequant_golden.npz"), q4k_blocks=q4, q4k_weights=w4, q6k_blocks=q6,
                        q6k_weights=w6, gguf_version=np.array(str(version)))
    print(f"wrote gguf_dequant_golden.npz from gguf {version}: {len(q4)} Q4_K + {len(q6)} Q6_K blocks")


if __name__ == "__main__":
    main()
