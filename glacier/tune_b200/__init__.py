"""glacier.tune_b200 - B200 (sm_100a) backend for Glacier.Tune's frozen-base K-quant projection path.

The product is ``libglaciertune_b200.so`` (C ABI in ``include/glaciertune_b200.h``); this package holds its
sources (``csrc/``), the in-tree build, a ctypes binding used by the tests and the benchmark, the C++ host
mirror of the reference's ``GpuLoraEngine`` / ``LoraAdapter`` surface (``host/``) and the seeded synthetic
input generator.  There is no CPU implementation of the path in this package.
"""
from . import synth  # noqa: F401
from .capi import (Adapter, Engine, GtError, Weight, MATH_BF16, MATH_FP16, MATH_FP32, TYPE_F32, TYPE_Q4_K,  # noqa: F401
                   TYPE_Q6_K, load_library)
