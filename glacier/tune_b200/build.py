"""In-tree build of libglaciertune_b200.so (nvcc, sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libglaciertune_b200.so")
SOURCES = ["gt_engine.cu", "gt_fp32_kernels.cu", "gt_lora_tc.cu", "gt_umma_gemm.cu", "gt_umma_few.cu", "gt_noalloc.cu", "gt_stream_gemm.cu", "gt_glue.cu", "gt_lmhead.cu", "gt_attention.cu", "gt_model.cu"]
HEADERS = ["gt_internal.h", "gt_engine_priv.h", "gt_ptx.cuh", "gt_quant.cuh"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libglaciertune_b200.so cannot be built")
    return exe


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS if os.path.exists(os.path.join(CSRC, f))]
    deps.append(os.path.join(HERE, "..", "..", "include", "glaciertune_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of the package into one shared library next to this file."""
    if not force and not is_stale():
        return LIB_PATH
    srcs = [os.path.join(CSRC, f) for f in SOURCES if os.path.exists(os.path.join(CSRC, f))]
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *srcs, "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd, cwd=CSRC)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
