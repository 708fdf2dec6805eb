"""Pins the Q4_K, Q6_K, Q4_0 and Q8_0 decoders to the GGUF project's own Python package.

The reference consumes GGUF tensors; its repository states the Q6_K layout only inside a CUDA kernel
(src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:263-332) and holds no Q6_K known answer.  The `gguf` package
(`gguf.quants.dequantize`, the format's reference decoder in numpy) is an independent implementation of the same
block formats.  This script draws seeded super-blocks with the workload generator, decodes them with `gguf`, and
stores blocks and fp32 weights in gguf_dequant_golden.npz (K-quants) and gguf_dequant_golden_q40_q80.npz (the 32-weight
block types, which the reference states in tune_bwd.cu:18-26 and for which it holds no known answer either).  The CPU tests compare the C oracle and its numpy mirror
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


def draw_small_blocks():
    """Seeded Q4_0 and Q8_0 blocks; block 0 of each holds the extreme quants."""
    rng = np.random.default_rng(SEED + 1)
    q40 = S.make_q40_blocks(NBLOCKS * 8, rng)
    q80 = S.make_q80_blocks(NBLOCKS * 8, rng)
    q40[0, 2:] = 0xF0        # nibbles 0 (-> -8) and 15 (-> +7)
    q80[0, 2:] = np.array([-128, 127] * 16, np.int8).view(np.uint8)
    return q40, q80


def gguf_decode_small(q40, q80):
    from gguf import GGMLQuantizationType
    from gguf.quants import dequantize
    w40 = np.ascontiguousarray(dequantize(q40.reshape(-1), GGMLQuantizationType.Q4_0), np.float32).reshape(len(q40), 32)
    w80 = np.ascontiguousarray(dequantize(q80.reshape(-1), GGMLQuantizationType.Q8_0), np.float32).reshape(len(q80), 32)
    return w40, w80


def main():
    import gguf
    q4, q6 = draw_blocks()
    w4, w6 = gguf_decode(q4, q6)
    q40, q80 = draw_small_blocks()
    w40, w80 = gguf_decode_small(q40, q80)
    version = getattr(gguf, "__version__", None)
    if version is None:
        try:
            from importlib.metadata import version as _v
            version = _v("gguf")
        except Exception:  # noqa: BLE001
            version = "unknown"
    np.savez_compressed(os.path.join(HERE, "gguf_dequant_golden.npz"), q4k_blocks=q4, q4k_weights=w4, q6k_blocks=q6,
                        q6k_weights=w6, gguf_version=np.array(str(version)))
    np.savez_compressed(os.path.join(HERE, "gguf_dequant_golden_q40_q80.npz"), q40_blocks=q40, q40_weights=w40, q80_blocks=q80,
                        q80_weights=w80, gguf_version=np.array(str(version)))
    print(f"wrote gguf_dequant_golden.npz from gguf {version}: {len(q4)} Q4_K + {len(q6)} Q6_K blocks")
    print(f"wrote gguf_dequant_golden_q40_q80.npz: {len(q40)} Q4_0 + {len(q80)} Q8_0 blocks")


if __name__ == "__main__":
    main()
