"""Builds the C++ host-mirror example against libglaciertune_b200.so (g++, no CUDA headers needed)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
EXE_PATH = os.path.join(HERE, "host_example")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "host_example.cpp")
    hdr = os.path.join(HERE, "glacier_tune_host.hpp")
    lib = os.path.join(PKG, "libglaciertune_b200.so")
    if not force and os.path.exists(EXE_PATH) and os.path.getmtime(EXE_PATH) >= max(os.path.getmtime(src), os.path.getmtime(hdr)):
        return EXE_PATH
    if not os.path.exists(lib):
        raise RuntimeError("build libglaciertune_b200.so first")
    subprocess.check_call(["/usr/bin/g++", "-O2", "-std=c++17", "-o", EXE_PATH, src, f"-L{PKG}", "-lglaciertune_b200",
                           "-Wl,-rpath,$ORIGIN/.."])
    return EXE_PATH
