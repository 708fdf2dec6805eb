"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol the header declares, and
refuses to run without a GPU (there is no CPU fallback).  No compute calls here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "glaciertune_b200.h")).read()
    return sorted(set(re.findall(r"GT_API\s+[\w\s\*]+?\b(gt_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = _header_symbols()
    for name in ("gt_engine_create", "gt_weight_upload", "gt_proj_forward", "gt_proj_backward", "gt_dequant_rows",
                 "gt_launch_gemm_batch", "gt_launch_gemm_bwd", "gt_dp_allreduce", "gt_last_error"):
        assert name in syms
    assert len(syms) >= 28


def test_library_exports_every_declared_symbol():
    from glacier.tune_b200 import capi
    lib = capi.load_library()
    for name in _header_symbols():
        assert hasattr(lib, name), f"{name} declared in include/glaciertune_b200.h but not exported"
    assert set(capi.EXPORTS) == set(_header_symbols())
    assert b"sm_100a" in lib.gt_version()


def test_supports_mirrors_reference_type_list():
    from glacier.tune_b200 import capi
    for t in (capi.TYPE_Q4_K, capi.TYPE_Q6_K, capi.TYPE_F32):
        assert capi.supports(t, capi.DIR_FORWARD) and capi.supports(t, capi.DIR_BACKWARD)
    assert not capi.supports(13, capi.DIR_FORWARD)      # Q5_K: not on this path
    assert not capi.supports(capi.TYPE_Q4_K, 7)


def test_engine_creation_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from glacier.tune_b200 import capi
    with pytest.raises(capi.GtError) as ei:
        capi.Engine(0)
    assert ei.value.code == -4 and "no CPU path" in str(ei.value)


def test_null_arguments_are_rejected_before_any_launch():
    from glacier.tune_b200 import capi
    lib = capi.load_library()
    assert lib.gt_engine_create(None, None) == -1
    assert lib.gt_proj_forward(None, None, None, None, None, 4, 0) == -1
    assert lib.gt_proj_backward(None, None, None, None, None, None, 4, 0) == -1
    assert lib.gt_sync(None) == -1
    assert b"null" in lib.gt_last_error()
    assert lib.gt_engine_destroy(None) == 0 and lib.gt_weight_free(None) == 0 and lib.gt_adapter_free(None) == 0


def test_package_does_not_import_the_oracle():
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); import glacier.tune_b200; "
            "assert not any(m == 'oracle' or m.startswith('oracle.') for m in sys.modules), 'oracle imported'") % ROOT
    subprocess.check_call([sys.executable, "-c", code])
    for dirpath, _, files in os.walk(os.path.join(ROOT, "glacier")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "gt_oracle" not in src and "from oracle" not in src and "import oracle" not in src, f


def test_logger_receives_the_error_texts():
    """gt_set_logger: every recorded error text reaches the callback (and nothing is printed without one)."""
    from glacier.tune_b200 import capi
    lib = capi.load_library()
    seen = []
    capi.set_logger(lambda level, msg: seen.append((level, msg)))
    try:
        assert lib.gt_sync(None) == -1
        assert seen and seen[-1][0] == 2 and "null" in seen[-1][1]
    finally:
        capi.set_logger(None)
    n = len(seen)
    assert lib.gt_sync(None) == -1
    assert len(seen) == n          # callback removed


def test_new_entry_points_reject_null_arguments():
    from glacier.tune_b200 import capi
    lib = capi.load_library()
    assert lib.gt_lm_head_loss(None, None, None, None, 4, None, None, None, 0) == -1
    assert lib.gt_attention_forward(None, None, None, None, None, None, 4, 2, 1, 128) == -1
    assert lib.gt_model_create(None, None, None) == -1
    assert lib.gt_model_forward_backward(None, None, None, 4, None, 0) == -1
    assert lib.gt_model_destroy(None) == 0
    assert lib.gt_supports_attention(512, 128) == 1 and lib.gt_supports_attention(512, 96) == 0
    assert capi.supports(capi.TYPE_F16, capi.DIR_FORWARD)


def test_ctypes_structs_match_the_header(tmp_path):
    """The ctypes mirrors of gt_config / gt_model_config have the header's size and field offsets (a C compiler is the
    judge): a field added on one side only would shift everything behind it silently."""
    import ctypes as C
    import shutil
    import subprocess
    from glacier.tune_b200 import capi as G
    HEADER = os.path.join(ROOT, "include", "glaciertune_b200.h")
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    fields_cfg = ["device", "math_mode", "stream", "max_tokens", "max_features"]
    fields_model = ["n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "rms_eps", "rope_theta", "max_tokens",
                    "checkpoint", "no_graph", "reserved"]
    src = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {",
           'printf("%zu\\n", sizeof(gt_config));']
    src += [f'printf("%zu\\n", offsetof(gt_config, {f}));' for f in fields_cfg]
    src += ['printf("%zu\\n", sizeof(gt_model_config));']
    src += [f'printf("%zu\\n", offsetof(gt_model_config, {f}));' for f in fields_model]
    src += ["return 0; }"]
    c_file, exe = tmp_path / "layout.c", tmp_path / "layout"
    c_file.write_text("\n".join(src))
    subprocess.check_call(["gcc", "-std=c11", "-o", str(exe), str(c_file)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(G.GtConfig)] + [getattr(G.GtConfig, f).offset for f in fields_cfg]
    want += [C.sizeof(G.GtModelConfig)] + [getattr(G.GtModelConfig, f).offset for f in fields_model]
    assert got == want
