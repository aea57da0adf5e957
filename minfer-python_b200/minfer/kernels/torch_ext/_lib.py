"""ctypes binding of libminfer_attn.so (declarations: include/minfer_attn.h).

The library is the only compute path.  If it is missing, importing this
module raises: there is no CPU or PyTorch fallback behind the ops.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# MINFER_ATTN_LIBRARY points at another build of the same library (e.g. one compiled with tuning macros)
LIB_PATH = os.environ.get("MINFER_ATTN_LIBRARY") or os.path.join(_HERE, "libminfer_attn.so")

F16 = 0
BF16 = 1
KV_16BIT = 0
KV_Q8_0 = 1
ABI_VERSION = 5

EXPORTS = (
    "minfer_attn_prefill",
    "minfer_attn_prefill_workspace_bytes",
    "minfer_attn_decode",
    "minfer_attn_decode_static",
    "minfer_attn_rope_append",
    "minfer_attn_decode_workspace_bytes",
    "minfer_attn_decode_default_chunk",
    "minfer_attn_strerror",
    "minfer_attn_last_cuda_error",
    "minfer_attn_abi_version",
)


class PrefillParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("mask", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("kv_stride", ctypes.c_int64 * 3),
        ("out_stride", ctypes.c_int64 * 3),
        ("batch", ctypes.c_int32),
        ("n_heads", ctypes.c_int32),
        ("n_kv_heads", ctypes.c_int32),
        ("seq_q", ctypes.c_int32),
        ("seq_k", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("causal", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("flags", ctypes.c_int32),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("max_ctas", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("n_peer_out", ctypes.c_int32),
        ("reserved2", ctypes.c_int32),
        ("peer_out", ctypes.c_void_p * 7),
    ]


class DecodeParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p),
        ("v_cache", ctypes.c_void_p),
        ("lens", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("q_stride", ctypes.c_int64 * 2),
        ("kv_stride", ctypes.c_int64 * 3),
        ("out_stride", ctypes.c_int64 * 2),
        ("batch", ctypes.c_int32),
        ("n_heads", ctypes.c_int32),
        ("n_kv_heads", ctypes.c_int32),
        ("max_len", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("chunk", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("kv_format", ctypes.c_int32),
        ("block_table", ctypes.c_void_p),
        ("page_size", ctypes.c_int32),
        ("table_stride", ctypes.c_int32),
        ("n_pages", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("status", ctypes.c_void_p),
    ]


class RopeParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p),
        ("v_cache", ctypes.c_void_p),
        ("start", ctypes.c_void_p),
        ("q_stride", ctypes.c_int64 * 3),
        ("kv_stride", ctypes.c_int64 * 3),
        ("cache_stride", ctypes.c_int64 * 3),
        ("batch", ctypes.c_int32),
        ("seq", ctypes.c_int32),
        ("n_heads", ctypes.c_int32),
        ("n_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("rotary_dim", ctypes.c_int32),
        ("start_pos", ctypes.c_int32),
        ("max_len", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("style", ctypes.c_int32),
        ("freq_base", ctypes.c_float),
        ("cache_format", ctypes.c_int32),
        ("block_table", ctypes.c_void_p),
        ("page_size", ctypes.c_int32),
        ("table_stride", ctypes.c_int32),
        ("n_pages", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("status", ctypes.c_void_p),
    ]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python build.py` in the package root "
            "(nvcc, sm_100a). There is no fallback implementation."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.minfer_attn_prefill.argtypes = [ctypes.POINTER(PrefillParams), ctypes.c_void_p]
    lib.minfer_attn_prefill.restype = ctypes.c_int
    lib.minfer_attn_prefill_workspace_bytes.argtypes = [ctypes.c_int32] * 3
    lib.minfer_attn_prefill_workspace_bytes.restype = ctypes.c_size_t
    lib.minfer_attn_decode.argtypes = [ctypes.POINTER(DecodeParams), ctypes.c_void_p]
    lib.minfer_attn_decode.restype = ctypes.c_int
    lib.minfer_attn_decode_static.argtypes = [ctypes.POINTER(DecodeParams), ctypes.c_void_p]
    lib.minfer_attn_decode_static.restype = ctypes.c_int
    lib.minfer_attn_rope_append.argtypes = [ctypes.POINTER(RopeParams), ctypes.c_void_p]
    lib.minfer_attn_rope_append.restype = ctypes.c_int
    lib.minfer_attn_decode_workspace_bytes.argtypes = [ctypes.c_int32] * 5
    lib.minfer_attn_decode_workspace_bytes.restype = ctypes.c_size_t
    lib.minfer_attn_decode_default_chunk.argtypes = [ctypes.c_int32] * 3
    lib.minfer_attn_decode_default_chunk.restype = ctypes.c_int32
    lib.minfer_attn_strerror.argtypes = [ctypes.c_int]
    lib.minfer_attn_strerror.restype = ctypes.c_char_p
    lib.minfer_attn_last_cuda_error.argtypes = []
    lib.minfer_attn_last_cuda_error.restype = ctypes.c_char_p
    lib.minfer_attn_abi_version.argtypes = []
    lib.minfer_attn_abi_version.restype = ctypes.c_int
    if lib.minfer_attn_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.minfer_attn_abi_version()}, this binding needs "
                          f"{ABI_VERSION}: rebuild it with `python build.py --force`")
    return lib


lib = _load()


def strerror(code: int) -> str:
    return lib.minfer_attn_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        detail = f" [{lib.minfer_attn_last_cuda_error().decode()}]" if code == 3 else ""
        raise RuntimeError(f"{what}: {strerror(code)} (code {code}){detail}")
