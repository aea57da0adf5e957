"""Loads libminfer_attn.so and registers the torch.ops.minfer attention ops.

Importing this module is what registers the ops, as in the reference
(src/minfer/kernels/torch_ext/__init__.py:1-3, test/conftest.py:2): ops.py
loads the torch extension `_C` when it has been built and falls back to its
ctypes binding of the same library otherwise.  The shared library itself must
have been built (build.py); there is no fallback for that.
"""
from . import _lib  # noqa: F401  (dlopen first: ops need the entry points)
from .ops import flash_attn, flash_attn_causal, flash_attn_decode  # noqa: F401
from .ops import il_rope, neox_rope, rope_kv_append  # noqa: F401
from .ops import flash_attn_decode_q8, rope_kv_append_q8  # noqa: F401
from .ops import flash_attn_decode_paged, rope_kv_append_paged  # noqa: F401
