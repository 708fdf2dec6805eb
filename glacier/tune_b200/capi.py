"""ctypes binding of libglaciertune_b200.so - the same C ABI a C# ``[LibraryImport]`` host binds.

Host arrays are numpy (C-contiguous fp32 / uint8); device arrays are anything with a ``data_ptr()`` (torch
tensors on the engine's device).  Every failure raises :class:`GtError` carrying ``gt_last_error()``;
nothing here falls back to a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 1, 2, 8, 12, 14
MATH_BF16, MATH_FP16, MATH_FP32 = 0, 1, 2
DIR_FORWARD, DIR_BACKWARD = 0, 1
FLAG_DEVICE_PTRS, FLAG_NO_LORA, FLAG_REUSE_LOW, FLAG_DX_ASSIGN, FLAG_HOST_ASYNC = 1, 2, 4, 8, 16

EXPORTS = [
    "gt_last_error", "gt_version", "gt_set_logger", "gt_engine_create", "gt_engine_destroy", "gt_engine_set_math_mode", "gt_sync",
    "gt_supports", "gt_weight_upload", "gt_weight_free", "gt_dequant_rows", "gt_adapter_create", "gt_adapter_free",
    "gt_adapter_upload", "gt_adapter_download", "gt_adapter_grads_download", "gt_adapter_grads_zero",
    "gt_adapter_set_alpha", "gt_adapter_device_ptrs", "gt_adapter_params_changed", "gt_adapter_bind_grads", "gt_proj_forward", "gt_proj_backward", "gt_proj_forward_group", "gt_proj_backward_group", "gt_stream_max_tokens", "gt_ffn_forward", "gt_ffn_backward", "gt_swiglu_forward", "gt_swiglu_backward", "gt_rope", "gt_rmsnorm_forward",
    "gt_rmsnorm_backward", "gt_add", "gt_lm_head_loss", "gt_lm_head_logits", "gt_embedding_forward", "gt_attention_forward", "gt_attention_backward", "gt_supports_attention", "gt_model_create", "gt_model_destroy", "gt_model_set_block", "gt_model_set_head", "gt_model_bind_grads", "gt_model_loss", "gt_model_forward_backward", "gt_model_step_info", "gt_model_optimizer_step",
    "gt_launch_gemm_batch", "gt_launch_gemm_bwd", "gt_launch_gemm_bwd_static", "gt_grads_scale_clip",
    "gt_adamw_step", "gt_adapter_adamw_step", "gt_adapters_adamw_step",
    "gt_profile_enable", "gt_profile_read", "gt_debug_set_trace", "gt_debug_wait_selftest", "gt_dp_init", "gt_dp_allreduce", "gt_dp_allreduce_begin", "gt_dp_allreduce_end", "gt_dp_finalize", "gt_dp_unique_id",
]


class GtError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"glaciertune_b200 error {code}: {msg}")
        self.code = code


class GtModelConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("max_tokens", C.c_int32), ("checkpoint", C.c_int32), ("no_graph", C.c_int32), ("reserved", C.c_int32 * 3)]


class GtConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("math_mode", C.c_int32), ("stream", C.c_void_p), ("max_tokens", C.c_int32),
                ("max_features", C.c_int32)]


_lib = None


def load_library(path: str | None = None) -> C.CDLL:
    """Load the shared library (building it in-tree when the sources are newer and nvcc is present)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or _build.LIB_PATH
    if path is None and _build.is_stale():
        try:
            _build.build()
        except Exception as exc:  # noqa: BLE001 - a stale/missing library is fatal, never a fallback
            if not os.path.exists(p):
                raise RuntimeError(f"libglaciertune_b200.so is missing and could not be built: {exc}") from exc
    lib = C.CDLL(p, mode=C.RTLD_GLOBAL)
    lib.gt_last_error.restype = C.c_char_p
    lib.gt_version.restype = C.c_char_p
    lib.gt_engine_create.argtypes = [C.POINTER(GtConfig), C.POINTER(C.c_void_p)]
    lib.gt_engine_destroy.argtypes = [C.c_void_p]
    lib.gt_engine_set_math_mode.argtypes = [C.c_void_p, C.c_int]
    lib.gt_sync.argtypes = [C.c_void_p]
    lib.gt_supports.argtypes = [C.c_int, C.c_int]
    lib.gt_weight_upload.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p,
                                     C.POINTER(C.c_void_p)]
    lib.gt_weight_free.argtypes = [C.c_void_p]
    lib.gt_dequant_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int32]
    lib.gt_adapter_create.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.POINTER(C.c_void_p)]
    lib.gt_adapter_free.argtypes = [C.c_void_p]
    for name in ("gt_adapter_upload", "gt_adapter_download", "gt_adapter_grads_download", "gt_adapter_bind_grads"):
        getattr(lib, name).argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.gt_adapter_grads_zero.argtypes = [C.c_void_p]
    lib.gt_adapter_params_changed.argtypes = [C.c_void_p]
    lib.gt_adapter_set_alpha.argtypes = [C.c_void_p, C.c_float]
    lib.gt_adapter_device_ptrs.argtypes = [C.c_void_p] + [C.POINTER(C.c_void_p)] * 4
    lib.gt_proj_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]
    lib.gt_proj_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                     C.c_int32]
    lib.gt_proj_forward_group.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]
    lib.gt_proj_backward_group.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                           C.c_int32]
    lib.gt_ffn_forward.argtypes = [C.c_void_p] * 10 + [C.c_int32, C.c_int32]
    lib.gt_ffn_backward.argtypes = [C.c_void_p] * 11 + [C.c_int32, C.c_int32]
    lib.gt_swiglu_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
    lib.gt_swiglu_backward.argtypes = [C.c_void_p] * 6 + [C.c_int64]
    lib.gt_add.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
    lib.gt_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_float,
                            C.c_int32, C.c_int32]
    lib.gt_rmsnorm_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float]
    lib.gt_rmsnorm_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float]
    lib.gt_lm_head_loss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]
    lib.gt_lm_head_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]
    lib.gt_embedding_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]
    lib.gt_attention_forward.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 4
    lib.gt_attention_backward.argtypes = [C.c_void_p] * 10 + [C.c_int32] * 4
    lib.gt_supports_attention.argtypes = [C.c_int32, C.c_int32]
    lib.gt_model_create.argtypes = [C.c_void_p, C.POINTER(GtModelConfig), C.POINTER(C.c_void_p)]
    lib.gt_model_destroy.argtypes = [C.c_void_p]
    lib.gt_model_set_block.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.gt_model_set_head.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.gt_model_bind_grads.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int64)]
    lib.gt_model_loss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32]
    lib.gt_model_forward_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]
    lib.gt_model_step_info.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    lib.gt_model_optimizer_step.argtypes = [C.c_void_p] + [C.c_float] * 6 + [C.c_double, C.c_int32, C.POINTER(C.c_double)]
    lib.gt_launch_gemm_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
    lib.gt_launch_gemm_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]
    lib.gt_launch_gemm_bwd_static.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]
    lib.gt_grads_scale_clip.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_double, C.POINTER(C.c_double)]
    lib.gt_adamw_step.argtypes = [C.c_void_p] + [C.c_void_p] * 4 + [C.c_int64] + [C.c_float] * 5 + [C.c_int32]
    lib.gt_adapter_adamw_step.argtypes = [C.c_void_p] + [C.c_float] * 5 + [C.c_int32]
    lib.gt_adapters_adamw_step.argtypes = [C.c_void_p, C.c_int32, C.c_void_p] + [C.c_float] * 5 + [C.c_int32]
    lib.gt_debug_set_trace.argtypes = [C.c_void_p, C.c_void_p]
    lib.gt_debug_wait_selftest.argtypes = [C.c_void_p, C.c_int64]
    lib.gt_profile_enable.argtypes = [C.c_void_p, C.c_int]
    lib.gt_profile_read.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_int64), C.POINTER(C.c_double),
                                    C.POINTER(C.c_int64), C.c_int]
    if hasattr(lib, "gt_dp_init"):
        lib.gt_dp_unique_id.argtypes = [C.c_void_p, C.c_int32]
        lib.gt_dp_init.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32]
        lib.gt_dp_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
        lib.gt_dp_allreduce_begin.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
        lib.gt_dp_allreduce_end.argtypes = [C.c_void_p]
        lib.gt_dp_finalize.argtypes = [C.c_void_p]
    if path is None:
        _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != 0:
        raise GtError(rc, load_library().gt_last_error().decode(errors="replace"))


def _ptr(a, dtype=None):
    """(address, is_device) of a numpy array or a device tensor."""
    if a is None:
        return None, False
    if hasattr(a, "data_ptr"):
        if not a.is_contiguous():
            raise ValueError("device tensors must be contiguous")
        return C.c_void_p(a.data_ptr()), bool(getattr(a, "is_cuda", False))
    if not isinstance(a, np.ndarray) or not a.flags.c_contiguous or (dtype is not None and a.dtype != dtype):
        raise ValueError(f"host arrays must be C-contiguous numpy {dtype}")
    return a.ctypes.data_as(C.c_void_p), False


LOG_FN = C.CFUNCTYPE(None, C.c_int, C.c_char_p, C.c_void_p)
_logger_keepalive = None


def set_logger(fn=None) -> None:
    """Install fn(level: int, message: str) as the library's log callback (None removes it)."""
    global _logger_keepalive
    lib = load_library()
    lib.gt_set_logger.argtypes = [C.c_void_p, C.c_void_p]
    if fn is None:
        lib.gt_set_logger(None, None)
        _logger_keepalive = None
        return
    cb = LOG_FN(lambda level, msg, user: fn(int(level), msg.decode(errors="replace")))
    lib.gt_set_logger(C.cast(cb, C.c_void_p), None)
    _logger_keepalive = cb


def stream_max_tokens() -> int:
    """Largest token count served by the few-token weight-streaming forward kernel (0: never)."""
    return int(load_library().gt_stream_max_tokens())


def supports(ggml_type: int, direction: int) -> bool:
    return bool(load_library().gt_supports(ggml_type, direction))


class Engine:
    """One CUDA context user: stream, scratch, math mode (replaces GpuLoraEngine's construction)."""

    def __init__(self, device: int = 0, math_mode: int = MATH_BF16, stream: int | None = None, max_tokens: int = 0, max_features: int = 0):
        self.lib = load_library()
        cfg = GtConfig(device=device, math_mode=math_mode, stream=C.c_void_p(stream) if stream else None, max_tokens=max_tokens,
                       max_features=max_features)
        h = C.c_void_p()
        _check(self.lib.gt_engine_create(C.byref(cfg), C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.gt_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def set_math_mode(self, mode: int):
        _check(self.lib.gt_engine_set_math_mode(self.h, mode))

    def sync(self):
        _check(self.lib.gt_sync(self.h))

    def upload_weight(self, ggml_type: int, data: np.ndarray, out_features: int, in_features: int, bias=None) -> "Weight":
        data = np.ascontiguousarray(data)
        bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
        h = C.c_void_p()
        _check(self.lib.gt_weight_upload(self.h, ggml_type, data.ctypes.data_as(C.c_void_p), data.nbytes, out_features,
                                         in_features, None if bias is None else bias.ctypes.data_as(C.c_void_p),
                                         C.byref(h)))
        return Weight(self, h, ggml_type, out_features, in_features)

    def create_adapter(self, in_features: int, out_features: int, rank: int = 16, alpha: float = 32.0) -> "Adapter":
        h = C.c_void_p()
        _check(self.lib.gt_adapter_create(self.h, in_features, out_features, rank, alpha, C.byref(h)))
        return Adapter(self, h, in_features, out_features, rank)

    # ---- projection calls -------------------------------------------------------------------------
    def forward(self, w: "Weight", adapter, X, Y=None, flags: int = 0):
        """Y[T, out] = X W^T + bias + scaling (X A) B.  Host numpy in -> numpy out; device tensors need Y."""
        xp, dev = _ptr(X, np.float32)
        T = X.shape[0]
        if dev:
            assert Y is not None
            flags |= FLAG_DEVICE_PTRS
        elif Y is None:
            Y = np.empty((T, w.N), np.float32)
        yp, _ = _ptr(Y, np.float32)
        _check(self.lib.gt_proj_forward(self.h, w.h, adapter.h if adapter else None, xp, yp, T, flags))
        return Y

    def backward(self, w: "Weight", adapter, dY, X, dX=None, flags: int = 0):
        """dX += dY W + adapter term; adapter grads accumulate.  dX None skips the input gradient."""
        gp, dev = _ptr(dY, np.float32)
        xp, _ = _ptr(X, np.float32)
        dp, _ = _ptr(dX, np.float32)
        if dev:
            flags |= FLAG_DEVICE_PTRS
        _check(self.lib.gt_proj_backward(self.h, w.h, adapter.h if adapter else None, gp, xp, dp, dY.shape[0], flags))
        return dX

    @staticmethod
    def _ptr_array(items):
        arr = (C.c_void_p * len(items))()
        for i, it in enumerate(items):
            arr[i] = None if it is None else (it.h if hasattr(it, "h") else _ptr(it)[0])
        return arr

    def forward_group(self, weights, adapters, X, Ys, flags: int = 0):
        """Projections of the same input (q,k,v or gate,up): Ys[j] = X W_j^T + ... in one launch (device tensors)."""
        xp, dev = _ptr(X, np.float32)
        if dev:
            flags |= FLAG_DEVICE_PTRS
        n = len(weights)
        ads = self._ptr_array(adapters if adapters is not None else [None] * n)
        _check(self.lib.gt_proj_forward_group(self.h, n, self._ptr_array(weights), ads, xp, self._ptr_array(Ys), X.shape[0], flags))
        return Ys

    def backward_group(self, weights, adapters, dYs, X, dX, flags: int = 0):
        """dX += sum_j dYs[j] W_j + adapter terms; adapter grads accumulate (device tensors for one launch)."""
        _, dev = _ptr(dYs[0], np.float32)
        if dev:
            flags |= FLAG_DEVICE_PTRS
        n = len(weights)
        ads = self._ptr_array(adapters if adapters is not None else [None] * n)
        _check(self.lib.gt_proj_backward_group(self.h, n, self._ptr_array(weights), ads, self._ptr_array(dYs), _ptr(X, np.float32)[0],
                                               _ptr(dX, np.float32)[0], dYs[0].shape[0], flags))
        return dX

    def ffn_forward(self, w_gate, w_up, w_down, adapters, X, out_down, out_gate=None, out_up=None, out_hidden=None, flags: int = 0):
        """ForwardFfn: down(SiLU(gate(X)) * up(X)) with the adapters' terms; optional outputs are skipped when None."""
        xp, dev = _ptr(X, np.float32)
        if dev:
            flags |= FLAG_DEVICE_PTRS
        ads = self._ptr_array(adapters) if adapters is not None else None
        _check(self.lib.gt_ffn_forward(self.h, w_gate.h, w_up.h, w_down.h, ads, xp, _ptr(out_gate)[0], _ptr(out_up)[0],
                                       _ptr(out_hidden)[0], _ptr(out_down)[0], X.shape[0], flags))
        return out_down

    def ffn_backward(self, w_gate, w_up, w_down, adapters, dY, X, gate, up, hidden, dX, flags: int = 0):
        ads = self._ptr_array(adapters) if adapters is not None else None
        _check(self.lib.gt_ffn_backward(self.h, w_gate.h, w_up.h, w_down.h, ads, _ptr(dY)[0], _ptr(X)[0], _ptr(gate)[0], _ptr(up)[0],
                                        _ptr(hidden)[0], _ptr(dX)[0], dY.shape[0], flags | FLAG_DEVICE_PTRS))
        return dX

    # ---- layer glue (device tensors, asynchronous on the engine stream)
    def swiglu_forward(self, gate, up, hidden):
        _check(self.lib.gt_swiglu_forward(self.h, _ptr(gate)[0], _ptr(up)[0], _ptr(hidden)[0], gate.numel()))
        return hidden

    def swiglu_backward(self, d_hidden, gate, up, d_gate, d_up):
        _check(self.lib.gt_swiglu_backward(self.h, _ptr(d_hidden)[0], _ptr(gate)[0], _ptr(up)[0], _ptr(d_gate)[0], _ptr(d_up)[0],
                                           gate.numel()))
        return d_gate, d_up

    def add(self, a, b, out):
        _check(self.lib.gt_add(self.h, _ptr(a)[0], _ptr(b)[0], _ptr(out)[0], a.numel()))
        return out

    def rope(self, q, k, T: int, heads_q: int, heads_kv: int, head_dim: int, freq_base: float = 1e6, freq_scale: float = 1.0,
             rope_dim: int = -1, inverse: bool = False):
        _check(self.lib.gt_rope(self.h, _ptr(q)[0], _ptr(k)[0], T, heads_q, heads_kv, head_dim, freq_base, freq_scale, rope_dim,
                                1 if inverse else 0))

    def rmsnorm_forward(self, x, w, y, eps: float = 1e-6):
        _check(self.lib.gt_rmsnorm_forward(self.h, _ptr(x)[0], _ptr(w)[0], _ptr(y)[0], x.shape[0], x.shape[1], eps))
        return y

    def rmsnorm_backward(self, dy, x, w, dx, eps: float = 1e-6):
        _check(self.lib.gt_rmsnorm_backward(self.h, _ptr(dy)[0], _ptr(x)[0], _ptr(w)[0], _ptr(dx)[0], x.shape[0], x.shape[1], eps))
        return dx

    # ---- attention (device tensors)
    def attention_forward(self, q, k, v, out, lse, T: int, heads_q: int, heads_kv: int, head_dim: int = 128):
        _check(self.lib.gt_attention_forward(self.h, _ptr(q)[0], _ptr(k)[0], _ptr(v)[0], _ptr(out)[0], _ptr(lse)[0], T, heads_q, heads_kv, head_dim))
        return out

    def attention_backward(self, d_out, q, k, v, out, lse, dq, dk, dv, T: int, heads_q: int, heads_kv: int, head_dim: int = 128):
        _check(self.lib.gt_attention_backward(self.h, _ptr(d_out)[0], _ptr(q)[0], _ptr(k)[0], _ptr(v)[0], _ptr(out)[0], _ptr(lse)[0],
                                              _ptr(dq)[0], _ptr(dk)[0], _ptr(dv)[0], T, heads_q, heads_kv, head_dim))
        return dq, dk, dv

    # ---- LM head
    def lm_head_loss(self, w: "Weight", hidden, labels, want_grad: bool = True, loss_dev=None, valid_dev=None, d_hidden=None):
        """Streaming cross-entropy over the LM head.  Host numpy in -> (loss, valid, dHidden or None); device tensors
        (hidden, labels int32, loss_dev [1] fp32, valid_dev [1] int32 or None, d_hidden or None) -> queued, returns None."""
        hp, dev = _ptr(hidden, np.float32)
        T = hidden.shape[0]
        if dev:
            _check(self.lib.gt_lm_head_loss(self.h, w.h, hp, _ptr(labels)[0], T, _ptr(loss_dev)[0], _ptr(valid_dev)[0],
                                            _ptr(d_hidden)[0], FLAG_DEVICE_PTRS))
            return None
        labels = np.ascontiguousarray(labels, np.int32)
        loss, valid = C.c_float(), C.c_int32()
        dh = np.empty((T, w.K), np.float32) if want_grad else None
        _check(self.lib.gt_lm_head_loss(self.h, w.h, hp, _ptr(labels)[0], T, C.cast(C.byref(loss), C.c_void_p), C.cast(C.byref(valid), C.c_void_p),
                                        _ptr(dh)[0], 0))
        return loss.value, valid.value, dh

    def lm_head_logits(self, w: "Weight", hidden, logits):
        _check(self.lib.gt_lm_head_logits(self.h, w.h, _ptr(hidden)[0], _ptr(logits)[0], hidden.shape[0], FLAG_DEVICE_PTRS))
        return logits

    def embedding(self, w: "Weight", tokens, out=None):
        """Rows tokens[t] of the embedding tensor as fp32 (host numpy or device tensors)."""
        tp, dev = _ptr(tokens)
        T = tokens.shape[0]
        if not dev:
            tokens = np.ascontiguousarray(tokens, np.int32)
            tp = _ptr(tokens)[0]
            if out is None:
                out = np.empty((T, w.K), np.float32)
        _check(self.lib.gt_embedding_forward(self.h, w.h, tp, T, _ptr(out)[0], FLAG_DEVICE_PTRS if dev else 0))
        return out

    def launch_gemm_batch(self, w: "Weight", Y, X, batch: int, residual=None):
        yp, _ = _ptr(Y)
        xp, _ = _ptr(X)
        rp, _ = _ptr(residual)
        _check(self.lib.gt_launch_gemm_batch(self.h, w.h, yp, xp, batch, rp))

    def launch_gemm_bwd(self, w: "Weight", dX, dY, batch: int):
        _check(self.lib.gt_launch_gemm_bwd(self.h, w.h, _ptr(dX)[0], _ptr(dY)[0], batch))

    def launch_gemm_bwd_static(self, w: "Weight", dX, dY, batch: int):
        """Allocation-free variant of launch_gemm_bwd (fixed 4 MiB scratch inside the library)."""
        _check(self.lib.gt_launch_gemm_bwd_static(self.h, w.h, _ptr(dX)[0], _ptr(dY)[0], batch))

    def dequant_rows(self, w: "Weight", row0: int, nrows: int, out=None):
        if out is None:
            out = np.empty((nrows, w.K), np.float32)
        op, dev = _ptr(out, np.float32)
        _check(self.lib.gt_dequant_rows(self.h, w.h, row0, nrows, op, FLAG_DEVICE_PTRS if dev else 0))
        return out

    def grads_scale_clip(self, g_dev, pre_scale: float, max_norm: float) -> float:
        norm = C.c_double()
        _check(self.lib.gt_grads_scale_clip(self.h, _ptr(g_dev)[0], g_dev.numel(), pre_scale, max_norm, C.byref(norm)))
        return norm.value

    def adamw_step(self, p_dev, g_dev, m_dev, v_dev, lr, beta1, beta2, eps, weight_decay, step: int):
        """One AdamW step in place on flat fp32 device tensors (queued on the engine stream)."""
        n = p_dev.numel()
        assert g_dev.numel() == n and m_dev.numel() == n and v_dev.numel() == n
        _check(self.lib.gt_adamw_step(self.h, _ptr(p_dev)[0], _ptr(g_dev)[0], _ptr(m_dev)[0], _ptr(v_dev)[0], n, lr, beta1, beta2, eps,
                                      weight_decay, step))

    def adapters_adamw_step(self, adapters, lr, beta1, beta2, eps, weight_decay, step: int):
        """AdamW on the A and B of every adapter in the list, sixteen adapters per launch."""
        _check(self.lib.gt_adapters_adamw_step(self.h, len(adapters), self._ptr_array(adapters), lr, beta1, beta2, eps, weight_decay, step))

    def wait_selftest(self, limit_cycles: int = 2_000_000):
        _check(self.lib.gt_debug_wait_selftest(self.h, limit_cycles))

    def set_trace(self, dev_buf=None):
        _check(self.lib.gt_debug_set_trace(self.h, None if dev_buf is None else C.c_void_p(dev_buf.data_ptr())))

    def profile_enable(self, on: bool = True):
        _check(self.lib.gt_profile_enable(self.h, 1 if on else 0))

    def profile_read(self, reset: bool = True) -> dict:
        ms, nl, fl, kl = C.c_double(), C.c_int64(), C.c_double(), C.c_int64()
        _check(self.lib.gt_profile_read(self.h, C.byref(ms), C.byref(nl), C.byref(fl), C.byref(kl), 1 if reset else 0))
        return dict(gemm_ms=ms.value, gemm_launches=nl.value, gemm_flops=fl.value, kernel_launches=kl.value)

    # ---- data parallel ----------------------------------------------------------------------------
    def dp_unique_id(self) -> bytes:
        buf = C.create_string_buffer(128)
        _check(self.lib.gt_dp_unique_id(buf, 128))
        return buf.raw

    def dp_init(self, world: int, rank: int, unique_id: bytes):
        _check(self.lib.gt_dp_init(self.h, world, rank, C.c_char_p(unique_id), len(unique_id)))

    def dp_allreduce(self, g_dev, scale: float = 1.0):
        _check(self.lib.gt_dp_allreduce(self.h, _ptr(g_dev)[0], g_dev.numel(), scale))

    def dp_allreduce_begin(self, g_dev, scale: float = 1.0):
        """All-reduce of one slice on the side stream, beside the engine-stream work queued after this call."""
        _check(self.lib.gt_dp_allreduce_begin(self.h, _ptr(g_dev)[0], g_dev.numel(), scale))

    def dp_allreduce_end(self):
        _check(self.lib.gt_dp_allreduce_end(self.h))

    def dp_finalize(self):
        _check(self.lib.gt_dp_finalize(self.h))


class Weight:
    def __init__(self, eng: Engine, h, qtype: int, N: int, K: int):
        self.eng, self.h, self.qtype, self.N, self.K = eng, h, qtype, N, K

    def free(self):
        if self.h:
            self.eng.lib.gt_weight_free(self.h)
            self.h = None


class Adapter:
    def __init__(self, eng: Engine, h, in_features: int, out_features: int, rank: int):
        self.eng, self.h, self.K, self.N, self.rank = eng, h, in_features, out_features, rank

    def upload(self, A=None, B=None):
        A = None if A is None else np.ascontiguousarray(A, np.float32)
        B = None if B is None else np.ascontiguousarray(B, np.float32)
        assert A is None or A.shape == (self.K, self.rank)
        assert B is None or B.shape == (self.rank, self.N)
        _check(self.eng.lib.gt_adapter_upload(self.h, _ptr(A)[0], _ptr(B)[0]))

    def download(self):
        A = np.empty((self.K, self.rank), np.float32)
        B = np.empty((self.rank, self.N), np.float32)
        _check(self.eng.lib.gt_adapter_download(self.h, _ptr(A)[0], _ptr(B)[0]))
        return A, B

    def grads(self):
        dA = np.empty((self.K, self.rank), np.float32)
        dB = np.empty((self.rank, self.N), np.float32)
        _check(self.eng.lib.gt_adapter_grads_download(self.h, _ptr(dA)[0], _ptr(dB)[0]))
        return dA, dB

    def zero_grads(self):
        _check(self.eng.lib.gt_adapter_grads_zero(self.h))

    def set_alpha(self, alpha: float):
        _check(self.eng.lib.gt_adapter_set_alpha(self.h, alpha))

    def adamw_step(self, lr, beta1, beta2, eps, weight_decay, step: int):
        """A, B <- AdamW(A, B; dA, dB) on the device; the moments live in the adapter."""
        _check(self.eng.lib.gt_adapter_adamw_step(self.h, lr, beta1, beta2, eps, weight_decay, step))

    def bind_grads(self, dA_dev, dB_dev):
        _check(self.eng.lib.gt_adapter_bind_grads(self.h, _ptr(dA_dev)[0], _ptr(dB_dev)[0]))

    def device_ptrs(self):
        ps = [C.c_void_p() for _ in range(4)]
        _check(self.eng.lib.gt_adapter_device_ptrs(self.h, *[C.byref(p) for p in ps]))
        return [p.value for p in ps]

    def params_changed(self):
        """A or B were written through the device pointers: refresh the B == 0 flag, drop the kept X*A."""
        _check(self.eng.lib.gt_adapter_params_changed(self.h))

    def free(self):
        if self.h:
            self.eng.lib.gt_adapter_free(self.h)
            self.h = None


PROJ_NAMES = ("q", "k", "v", "o", "gate", "up", "down")


class Model:
    """The device-resident training step (replaces GgufLoraModel.ForwardLossAndBackward + the trainer's step tail).

    ``blocks`` is a list of dicts per layer: {"w": [7 Weight], "ad": [7 Adapter or None], "norm1": fp32 [hidden],
    "norm2": fp32 [hidden]} in the order q, k, v, o, gate, up, down."""

    def __init__(self, eng: Engine, n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_tokens, rms_eps=1e-6,
                 rope_theta=1e6, checkpoint=True, graph=True):
        self.eng = eng
        cfg = GtModelConfig(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, ffn=ffn,
                            vocab=vocab, rms_eps=rms_eps, rope_theta=rope_theta, max_tokens=max_tokens, checkpoint=1 if checkpoint else 0,
                            no_graph=0 if graph else 1)
        h = C.c_void_p()
        _check(eng.lib.gt_model_create(eng.h, C.byref(cfg), C.byref(h)))
        self.h = h
        self.n_layers = n_layers
        self._keep = []

    def set_block(self, layer: int, weights, adapters, norm1, norm2):
        n1 = np.ascontiguousarray(norm1, np.float32)
        n2 = np.ascontiguousarray(norm2, np.float32)
        self._keep.append((weights, adapters))
        _check(self.eng.lib.gt_model_set_block(self.h, layer, Engine._ptr_array(weights),
                                               Engine._ptr_array(adapters) if adapters is not None else None, _ptr(n1)[0], _ptr(n2)[0]))

    def set_head(self, embedding: "Weight", out_norm, lm_head: "Weight"):
        on = np.ascontiguousarray(out_norm, np.float32)
        self._keep.append((embedding, lm_head))
        _check(self.eng.lib.gt_model_set_head(self.h, embedding.h, _ptr(on)[0], lm_head.h))

    def bind_grads(self):
        """Returns (device address, element count) of the flat gradient buffer."""
        p, n = C.c_void_p(), C.c_int64()
        _check(self.eng.lib.gt_model_bind_grads(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def loss(self, tokens, labels):
        tokens = np.ascontiguousarray(tokens, np.int32)
        labels = np.ascontiguousarray(labels, np.int32)
        loss, valid = C.c_float(), C.c_int32()
        _check(self.eng.lib.gt_model_loss(self.h, _ptr(tokens)[0], _ptr(labels)[0], tokens.shape[0], C.cast(C.byref(loss), C.c_void_p),
                                          C.cast(C.byref(valid), C.c_void_p), 0))
        return loss.value, valid.value

    def forward_backward(self, tokens, labels, loss_dev=None):
        """Host int32 arrays -> loss (synchronous); device tensors (+ optional loss_dev [1]) -> queued, returns None."""
        tp, dev = _ptr(tokens)
        if dev:
            _check(self.eng.lib.gt_model_forward_backward(self.h, tp, _ptr(labels)[0], tokens.shape[0], _ptr(loss_dev)[0], FLAG_DEVICE_PTRS))
            return None
        tokens = np.ascontiguousarray(tokens, np.int32)
        labels = np.ascontiguousarray(labels, np.int32)
        loss = C.c_float()
        _check(self.eng.lib.gt_model_forward_backward(self.h, _ptr(tokens)[0], _ptr(labels)[0], tokens.shape[0],
                                                      C.cast(C.byref(loss), C.c_void_p), 0))
        return loss.value

    def step_info(self) -> dict:
        """Whether a captured step stands ready, how many calls were replays, kernels per replay."""
        ready, n, k = C.c_int32(), C.c_int64(), C.c_int64()
        _check(self.eng.lib.gt_model_step_info(self.h, C.byref(ready), C.byref(n), C.byref(k)))
        return {"graph_ready": bool(ready.value), "replays": n.value, "kernels_per_replay": k.value}

    def optimizer_step(self, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, grad_scale=1.0, max_norm=1.0, step=1,
                       want_norm=False):
        norm = C.c_double()
        _check(self.eng.lib.gt_model_optimizer_step(self.h, lr, beta1, beta2, eps, weight_decay, grad_scale, max_norm, step,
                                                    C.byref(norm) if want_norm else None))
        return norm.value if want_norm else None

    def close(self):
        if getattr(self, "h", None):
            self.eng.lib.gt_model_destroy(self.h)
            self.h = None
