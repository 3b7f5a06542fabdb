"""ctypes binding of libmegabake_b200.so (the C ABI in include/megabake_b200.h).

There is no fallback: if the library is missing or a call fails, this raises.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libmegabake_b200.so"

MK_MAX_LAYERS = 96
MK_TOKEN_TILE = 16

MK_OK = 0
ERROR_NAMES = {
    0: "MK_OK", 1: "MK_ERR_INVALID", 2: "MK_ERR_UNSUPPORTED", 3: "MK_ERR_CUDA", 4: "MK_ERR_ALIGNMENT",
    5: "MK_ERR_WORKSPACE", 6: "MK_ERR_UNBOUND", 7: "MK_ERR_DEVICE_STATUS",
}
MK_ERR_INVALID, MK_ERR_UNSUPPORTED, MK_ERR_CUDA, MK_ERR_ALIGNMENT = 1, 2, 3, 4
MK_ERR_WORKSPACE, MK_ERR_UNBOUND, MK_ERR_DEVICE_STATUS = 5, 6, 7
STATUS_NAMES = {0: "OK", 1: "KV_OVERFLOW", 2: "BAD_INDEX", 3: "TIMEOUT"}
ROPE_STYLES = {"hf": 0, "half_swap": 1}
ENGINES = {"tcgen05": 0, "fma": 2, "auto": 3}

EXPORTS = (
    "mk_workspace_bytes", "mk_create", "mk_bind_weights", "mk_decode", "mk_prefill", "mk_linear",
    "mk_kv_attention", "mk_kv_attention_static", "mk_kv_attention_static_status", "mk_attention", "mk_status", "mk_set_trace",
    "mk_launch_info", "mk_last_error", "mk_destroy", "mk_decode_steps", "mk_decode_step_host", "mk_set_status_mirror", "mk_debug_skew_barrier",
    "mk_describe", "mk_decode_ragged", "mk_baseline_mma_gemm", "mk_tp_exchange_bytes", "mk_tp_bind", "mk_ipc_export", "mk_ipc_open", "mk_ipc_close",
)


class MkConfig(Structure):
    _fields_ = [
        ("hidden", c_int32), ("layers", c_int32), ("q_heads", c_int32), ("kv_heads", c_int32),
        ("head_dim", c_int32), ("intermediate", c_int32), ("vocab", c_int32), ("rms_eps", c_float),
        ("qkv_bias", c_int32), ("rope_style", c_int32), ("max_tokens", c_int32),
        ("max_positions", c_int32), ("engine", c_int32), ("sm_limit", c_int32),
        ("tp_size", c_int32), ("tp_rank", c_int32), ("embed_rows", c_int32),
    ]


class MkLayerWeights(Structure):
    _fields_ = [(name, c_void_p) for name in (
        "input_norm", "q", "k", "v", "q_bias", "k_bias", "v_bias", "o", "post_norm", "gate", "up", "down")]


class MkWeights(Structure):
    _fields_ = [
        ("embed", c_void_p), ("final_norm", c_void_p), ("lm_head", c_void_p),
        ("rope_cos", c_void_p), ("rope_sin", c_void_p), ("layers", POINTER(MkLayerWeights)),
    ]


class MkIpcHandle(Structure):
    _fields_ = [("bytes", ctypes.c_ubyte * 64), ("offset", ctypes.c_uint64)]


class MkStatusInfo(Structure):
    _fields_ = [("status", c_int32), ("where", c_int32), ("cta", c_int32), ("detail", c_int32)]


class NativeError(RuntimeError):
    def __init__(self, function: str, code: int, message: str):
        super().__init__(f"{function} failed: {ERROR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.function = function
        self.detail = message


_library = None


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise if it has not been built."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise RuntimeError(
            f"{LIBRARY_PATH} is missing: build it with `python -m megabake_b200.build` "
            "(there is no non-CUDA path)"
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    lib.mk_workspace_bytes.restype = c_size_t
    lib.mk_workspace_bytes.argtypes = [POINTER(MkConfig), c_int]
    lib.mk_create.restype = c_int
    lib.mk_create.argtypes = [POINTER(MkConfig), c_void_p, c_size_t, c_int, c_void_p, POINTER(c_void_p)]
    lib.mk_bind_weights.restype = c_int
    lib.mk_bind_weights.argtypes = [c_void_p, POINTER(MkWeights), c_void_p]
    lib.mk_decode.restype = c_int
    lib.mk_decode.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
        c_int, c_void_p, c_void_p,
    ]
    lib.mk_decode_ragged.restype = c_int
    lib.mk_decode_ragged.argtypes = lib.mk_decode.argtypes
    lib.mk_prefill.restype = c_int
    lib.mk_prefill.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.mk_linear.restype = c_int
    lib.mk_linear.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mk_kv_attention.restype = c_int
    lib.mk_kv_attention.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
    ]
    lib.mk_attention.restype = c_int
    lib.mk_attention.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
    ]
    lib.mk_kv_attention_static.restype = c_int
    lib.mk_kv_attention_static.argtypes = [
        c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
        c_int, c_void_p,
    ]
    lib.mk_kv_attention_static_status.restype = c_int
    lib.mk_kv_attention_static_status.argtypes = [c_int, c_void_p, POINTER(MkStatusInfo)]
    lib.mk_decode_steps.restype = c_int
    lib.mk_decode_steps.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
        c_int, c_int, c_void_p, c_void_p, c_void_p,
    ]
    lib.mk_decode_step_host.restype = c_int
    lib.mk_decode_step_host.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
        c_int, c_void_p, c_void_p, c_void_p,
    ]
    lib.mk_tp_exchange_bytes.restype = c_size_t
    lib.mk_tp_exchange_bytes.argtypes = [POINTER(MkConfig)]
    lib.mk_tp_bind.restype = c_int
    lib.mk_tp_bind.argtypes = [c_void_p, POINTER(c_void_p), c_size_t, c_void_p]
    lib.mk_ipc_export.restype = c_int
    lib.mk_ipc_export.argtypes = [c_void_p, POINTER(MkIpcHandle)]
    lib.mk_ipc_open.restype = c_int
    lib.mk_ipc_open.argtypes = [POINTER(MkIpcHandle), POINTER(c_void_p), POINTER(c_void_p)]
    lib.mk_ipc_close.restype = c_int
    lib.mk_ipc_close.argtypes = [c_void_p]
    lib.mk_baseline_mma_gemm.restype = c_int
    lib.mk_baseline_mma_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mk_describe.restype = c_int
    lib.mk_describe.argtypes = [c_void_p, ctypes.c_char_p, c_size_t]
    lib.mk_debug_skew_barrier.restype = c_int
    lib.mk_debug_skew_barrier.argtypes = [c_void_p, ctypes.c_uint32]
    lib.mk_set_status_mirror.restype = c_int
    lib.mk_set_status_mirror.argtypes = [c_void_p, c_void_p]
    lib.mk_status.restype = c_int
    lib.mk_status.argtypes = [c_void_p, c_void_p, POINTER(MkStatusInfo)]
    lib.mk_set_trace.restype = c_int
    lib.mk_set_trace.argtypes = [c_void_p, c_void_p, c_int]
    lib.mk_launch_info.restype = c_int
    lib.mk_launch_info.argtypes = [c_void_p, POINTER(c_int32), POINTER(c_int32), POINTER(c_int64)]
    lib.mk_last_error.restype = c_char_p
    lib.mk_last_error.argtypes = []
    lib.mk_destroy.restype = c_int
    lib.mk_destroy.argtypes = [c_void_p]
    _library = lib
    return lib


def check(function: str, code: int) -> None:
    if code != MK_OK:
        raise NativeError(function, code, load().mk_last_error().decode(errors="replace"))
